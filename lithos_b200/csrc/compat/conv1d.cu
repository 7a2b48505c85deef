// Drop-in for launch_conv1d (src/launcher.s:2641-2807): file conv1d.cubin, entry conv1d, parameters
//   (u64 input, u64 weight, u64 hist, u64 output, u32 num_heads, u32 channels), grid ceil(num_heads * channels / 256) x 256,
// called three times per DeltaNet layer (Q, K and V slices; in place: output == input).
// N = num_heads * channels.  The arithmetic of inference/recur.ls:12-40 (conv1d_infer):
//   y[c] = w[0][c] x[c] + w[1][c] h[0][c] + w[2][c] h[1][c] + w[3][c] h[2][c];  h[2] = h[1]; h[1] = h[0]; h[0] = x
// with weight [4][N] and hist [3][N] planar fp32, RELATIVE TO THE POINTERS GIVEN: the launcher hands every slice the
// layer's whole conv tensor (src/launcher.s:2711-2713), a maintainer passes the slice's own taps.  No activation: the
// launcher applies SiLU as a separate `activate` launch (src/launcher.s:838-840).
// `conv1d_bf16w`: the same with bf16 taps, the dtype of the checkpoint tensor.
#include <stdint.h>

template <typename W> __device__ __forceinline__ float ldw(const W* w, size_t i);
template <> __device__ __forceinline__ float ldw<float>(const float* w, size_t i) { return w[i]; }
template <> __device__ __forceinline__ float ldw<uint16_t>(const uint16_t* w, size_t i) { return __uint_as_float((uint32_t)w[i] << 16); }

template <typename W>
__device__ __forceinline__ void conv1d_core(const float* x, const W* w, float* hist, float* y, uint32_t N) {
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < N; c += gridDim.x * blockDim.x) {
        const float xi = x[c], s0 = hist[c], s1 = hist[(size_t)N + c], s2 = hist[(size_t)2 * N + c];
        float acc = ldw(w, c) * xi;
        acc = fmaf(ldw(w, (size_t)N + c), s0, acc);
        acc = fmaf(ldw(w, (size_t)2 * N + c), s1, acc);
        acc = fmaf(ldw(w, (size_t)3 * N + c), s2, acc);
        y[c] = acc;
        hist[(size_t)2 * N + c] = s1;
        hist[(size_t)N + c] = s0;
        hist[c] = xi;
    }
}
extern "C" __global__ void conv1d(const float* input, const float* weight, float* hist, float* output, uint32_t num_heads, uint32_t channels) {
    conv1d_core<float>(input, weight, hist, output, num_heads * channels);
}
extern "C" __global__ void conv1d_bf16w(const float* input, const uint16_t* weight, float* hist, float* output, uint32_t num_heads, uint32_t channels) {
    conv1d_core<uint16_t>(input, weight, hist, output, num_heads * channels);
}
