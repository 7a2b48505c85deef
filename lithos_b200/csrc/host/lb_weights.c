/* weight_index.bin: the reference launcher's own weight-table file, read and written.
 *
 * The reference's load_weights (src/launcher.s:3267-3683) opens <model_dir>/weight_index.bin, maps every shard file
 * it names, and resolves 64 x 26 per-layer slots + 3 globals to pointers `shard base + file offset`:
 *   [0] u32 magic 0x4C575449   [4] u32 version 1   [8] u32 num_shards   [12] u32 num_layers
 *   [16] u32 slots_per_layer   [20] u32 num_globals   [24] u32 reserved[2]
 *   [32] shard table: num_shards x 264 bytes (256-byte NUL-terminated file name, u64 file size)
 *   then the global table (num_globals x 24) and the layer table (num_layers x slots_per_layer x 24), every entry
 *   u32 shard index, u32 reserved, u64 file offset, u64 size; offset == size == 0 marks an unused slot (NULL).
 * The generator of that file (gen_weight_index.py) is not part of the reference tree; lb_save_weights writes the same
 * format (one raw shard file holding the tensors back to back, 64-byte aligned).
 *
 * Differences from the reference, all on the side of reporting: a wrong magic or version, a truncated index, a shard
 * index out of range, a shard file shorter than an entry needs, a size that does not match the model shape and a
 * missing required slot are errors here (LB_ERR_IO / LB_ERR_INVALID with the reason); the launcher prints a message
 * and carries on with NULL pointers (src/launcher.s:3660-3683).
 */
#define _GNU_SOURCE
#include "lb_internal.h"
#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#define WIDX_MAGIC 0x4C575449u
#define WIDX_VERSION 1u
#define WIDX_SHARD_ENTRY 264
#define WIDX_ENTRY 24
#define WIDX_MAX_SHARDS 64 /* the launcher's shard_bases table (src/launcher.s:313-319) */

struct lb_weight_index {
    unsigned char* idx; /* mapped weight_index.bin */
    size_t idx_bytes;
    uint32_t n_shards, n_layers, n_slots, n_globals;
    unsigned char* shard[WIDX_MAX_SHARDS];
    size_t shard_bytes[WIDX_MAX_SHARDS];
};

static int wfail(char* err, size_t errlen, int status, const char* fmt, ...) {
    if (err && errlen) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, errlen, fmt, ap);
        va_end(ap);
    }
    return status;
}

static uint32_t rd32(const unsigned char* p) { uint32_t v; memcpy(&v, p, 4); return v; }
static uint64_t rd64(const unsigned char* p) { uint64_t v; memcpy(&v, p, 8); return v; }

/* map a whole file read-only (private); *bytes receives its size */
static unsigned char* map_file(const char* path, size_t* bytes) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return NULL;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) { close(fd); return NULL; }
    void* p = mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return NULL;
    *bytes = (size_t)st.st_size;
    return (unsigned char*)p;
}

LB_API void lb_weight_index_close(lb_weight_index* w) {
    if (!w) return;
    for (uint32_t s = 0; s < w->n_shards && s < WIDX_MAX_SHARDS; s++)
        if (w->shard[s]) munmap(w->shard[s], w->shard_bytes[s]);
    if (w->idx) munmap(w->idx, w->idx_bytes);
    free(w);
}

LB_API int lb_weight_index_open(const char* model_dir, lb_weight_index** out, char* err, size_t errlen) {
    if (!model_dir || !out) return wfail(err, errlen, LB_ERR_INVALID, "weight index: NULL argument");
    *out = NULL;
    char path[1280];
    snprintf(path, sizeof path, "%s/weight_index.bin", model_dir);
    lb_weight_index* w = (lb_weight_index*)calloc(1, sizeof *w);
    if (!w) return wfail(err, errlen, LB_ERR_NOMEM, "weight index: out of memory");
    w->idx = map_file(path, &w->idx_bytes);
    if (!w->idx) { free(w); return wfail(err, errlen, LB_ERR_IO, "weight index: cannot open %s (%s)", path, strerror(errno)); }
    int st = LB_OK;
    if (w->idx_bytes < 32) st = wfail(err, errlen, LB_ERR_IO, "weight index: %s is %zu bytes, shorter than its header", path, w->idx_bytes);
    else if (rd32(w->idx) != WIDX_MAGIC) st = wfail(err, errlen, LB_ERR_IO, "weight index: bad magic 0x%08X (want 0x%08X)", rd32(w->idx), WIDX_MAGIC);
    else if (rd32(w->idx + 4) != WIDX_VERSION) st = wfail(err, errlen, LB_ERR_IO, "weight index: version %u (this library reads version %u)", rd32(w->idx + 4), WIDX_VERSION);
    if (st == LB_OK) {
        w->n_shards = rd32(w->idx + 8); w->n_layers = rd32(w->idx + 12); w->n_slots = rd32(w->idx + 16); w->n_globals = rd32(w->idx + 20);
        const uint64_t need = 32ull + (uint64_t)w->n_shards * WIDX_SHARD_ENTRY +
                              ((uint64_t)w->n_globals + (uint64_t)w->n_layers * w->n_slots) * WIDX_ENTRY;
        if (w->n_shards == 0 || w->n_shards > WIDX_MAX_SHARDS)
            st = wfail(err, errlen, LB_ERR_IO, "weight index: %u shards (1..%d)", w->n_shards, WIDX_MAX_SHARDS);
        else if (w->n_layers > 4096 || w->n_slots > 4096 || w->n_globals > 4096)
            st = wfail(err, errlen, LB_ERR_IO, "weight index: implausible table sizes (%u layers, %u slots, %u globals)", w->n_layers, w->n_slots, w->n_globals);
        else if (need > w->idx_bytes)
            st = wfail(err, errlen, LB_ERR_IO, "weight index: file is %zu bytes, its tables need %llu (truncated)", w->idx_bytes, (unsigned long long)need);
    }
    for (uint32_t s = 0; st == LB_OK && s < w->n_shards; s++) {
        const unsigned char* e = w->idx + 32 + (size_t)s * WIDX_SHARD_ENTRY;
        if (!memchr(e, 0, 256)) { st = wfail(err, errlen, LB_ERR_IO, "weight index: shard %u file name is not terminated", s); break; }
        snprintf(path, sizeof path, "%s/%s", model_dir, (const char*)e);
        w->shard[s] = map_file(path, &w->shard_bytes[s]);
        if (!w->shard[s]) { st = wfail(err, errlen, LB_ERR_IO, "weight index: cannot map shard %u '%s' (%s)", s, path, strerror(errno)); break; }
        const uint64_t want = rd64(e + 256);
        if (want != w->shard_bytes[s]) {
            st = wfail(err, errlen, LB_ERR_IO, "weight index: shard %u '%s' is %zu bytes, the index says %llu", s, path, w->shard_bytes[s], (unsigned long long)want);
            break;
        }
    }
    /* every entry must point inside its shard */
    const size_t n_entries = st == LB_OK ? (size_t)w->n_globals + (size_t)w->n_layers * w->n_slots : 0;
    const unsigned char* tab = w->idx + 32 + (size_t)w->n_shards * WIDX_SHARD_ENTRY;
    for (size_t i = 0; st == LB_OK && i < n_entries; i++) {
        const unsigned char* e = tab + i * WIDX_ENTRY;
        const uint32_t s = rd32(e);
        const uint64_t off = rd64(e + 8), size = rd64(e + 16);
        if (off == 0 && size == 0) continue;
        if (s >= w->n_shards) st = wfail(err, errlen, LB_ERR_IO, "weight index: entry %zu names shard %u of %u", i, s, w->n_shards);
        else if (off > w->shard_bytes[s] || size > w->shard_bytes[s] - off)
            st = wfail(err, errlen, LB_ERR_IO, "weight index: entry %zu (offset %llu, %llu bytes) runs past shard %u (%zu bytes)", i,
                       (unsigned long long)off, (unsigned long long)size, s, w->shard_bytes[s]);
    }
    if (st != LB_OK) { lb_weight_index_close(w); return st; }
    *out = w;
    return LB_OK;
}

LB_API int lb_weight_index_dims(const lb_weight_index* w, int* n_layers, int* n_slots, int* n_globals, int* n_shards) {
    if (!w) return LB_ERR_INVALID;
    if (n_layers) *n_layers = (int)w->n_layers;
    if (n_slots) *n_slots = (int)w->n_slots;
    if (n_globals) *n_globals = (int)w->n_globals;
    if (n_shards) *n_shards = (int)w->n_shards;
    return LB_OK;
}

/* layer < 0 addresses the global table (slot = global index) */
LB_API int lb_weight_index_entry(const lb_weight_index* w, int layer, int slot, const void** ptr, size_t* bytes) {
    if (!w || !ptr || !bytes || slot < 0) return LB_ERR_INVALID;
    const unsigned char* tab = w->idx + 32 + (size_t)w->n_shards * WIDX_SHARD_ENTRY;
    size_t i;
    if (layer < 0) {
        if ((uint32_t)slot >= w->n_globals) return LB_ERR_INVALID;
        i = (size_t)slot;
    } else {
        if ((uint32_t)layer >= w->n_layers || (uint32_t)slot >= w->n_slots) return LB_ERR_INVALID;
        i = (size_t)w->n_globals + (size_t)layer * w->n_slots + (size_t)slot;
    }
    const unsigned char* e = tab + i * WIDX_ENTRY;
    const uint64_t off = rd64(e + 8), size = rd64(e + 16);
    if (off == 0 && size == 0) { *ptr = NULL; *bytes = 0; return LB_OK; }
    *ptr = w->shard[rd32(e)] + off;
    *bytes = (size_t)size;
    return LB_OK;
}

/* ---- the shapes this build gives the slots (bytes; 0 = slot unused in that kind of layer) ---- */
static int layer_is_fa(const lb_model_cfg* c, int l) { return (l % c->fa_period) == c->fa_period - 1; }

static size_t q4_part(size_t K, size_t N, int part) {
    return part == 0 ? K / 8 * N * 4 : part == 1 ? K / 128 * N * 2 : K / 128 * (N / 8) * 4;
}

LB_API size_t lb_model_slot_bytes(const lb_model_cfg* c, int layer, int slot) {
    if (!c || slot < 0 || slot >= LB_WS_SLOTS || layer < 0 || layer >= c->n_layers) return 0;
    const size_t H = (size_t)c->hidden, I = (size_t)c->inter;
    if (slot >= 15 && slot <= 20) return q4_part(H, I, (slot - 15) % 3);    /* gate, up */
    if (slot >= 21 && slot <= 23) return q4_part(I, H, slot - 21);          /* down */
    if (slot == 24 || slot == 25) return H * 2;                             /* input / post-attention norm, bf16 */
    if (!layer_is_fa(c, layer)) {
        const size_t HV = (size_t)c->dn_v_heads, C = (size_t)(2 * c->dn_k_heads + c->dn_v_heads) * 128, V = HV * 128;
        if (slot <= 2) return q4_part(H, C, slot);
        if (slot <= 5) return q4_part(H, V, slot - 3);
        if (slot <= 8) return q4_part(V, H, slot - 6);
        if (slot == 9 || slot == 10) return HV * H * 2; /* in_proj_a / in_proj_b, bf16 */
        if (slot == 11) return HV * 4;                  /* A_log fp32 */
        if (slot == 12) return HV * 2;                  /* dt_bias bf16 */
        if (slot == 13) return 4 * C * 2;               /* conv taps bf16 [4,C] */
        return 128 * 4;                                 /* per-head norm weight fp32 */
    }
    const size_t Q = (size_t)c->fa_q_heads * 256, KV = (size_t)c->fa_kv_heads * 256;
    if (slot <= 2) return q4_part(H, 2 * Q, slot);
    if (slot <= 5) return q4_part(H, KV, slot - 3);
    if (slot <= 8) return q4_part(H, KV, slot - 6);
    if (slot <= 11) return q4_part(Q, H, slot - 9);
    if (slot == 12 || slot == 13) return 256 * 2; /* q / k norm weights bf16 */
    return 0;                                     /* slot 14 is unused in attention layers */
}

LB_API size_t lb_model_global_bytes(const lb_model_cfg* c, int which) {
    if (!c || which < 0 || which >= LB_WG_SLOTS) return 0;
    return which == 2 ? (size_t)c->hidden * 2 : (size_t)c->vocab * c->hidden * 2;
}

/* index tables against the model shape: every used slot present with the size the shape implies */
LB_API int lb_weight_index_check(const lb_weight_index* w, const lb_model_cfg* c, char* err, size_t errlen) {
    if (!w || !c) return wfail(err, errlen, LB_ERR_INVALID, "weight index: NULL argument");
    if ((int)w->n_layers != c->n_layers || w->n_slots != LB_WS_SLOTS || w->n_globals != LB_WG_SLOTS)
        return wfail(err, errlen, LB_ERR_IO, "weight index: %u layers x %u slots + %u globals, the model wants %d x %d + %d", w->n_layers,
                     w->n_slots, w->n_globals, c->n_layers, LB_WS_SLOTS, LB_WG_SLOTS);
    const void* p;
    size_t n;
    for (int g = 0; g < LB_WG_SLOTS; g++) {
        lb_weight_index_entry(w, -1, g, &p, &n);
        if (!p) return wfail(err, errlen, LB_ERR_INVALID, "weight index: global %d is NULL", g);
        if (n != lb_model_global_bytes(c, g))
            return wfail(err, errlen, LB_ERR_IO, "weight index: global %d holds %zu bytes, the shape needs %zu", g, n, lb_model_global_bytes(c, g));
    }
    for (int l = 0; l < c->n_layers; l++)
        for (int s = 0; s < LB_WS_SLOTS; s++) {
            const size_t want = lb_model_slot_bytes(c, l, s);
            lb_weight_index_entry(w, l, s, &p, &n);
            if (want == 0) continue;
            if (!p) return wfail(err, errlen, LB_ERR_INVALID, "weight index: layer %d slot %d is NULL", l, s);
            if (n != want) return wfail(err, errlen, LB_ERR_IO, "weight index: layer %d slot %d holds %zu bytes, the shape needs %zu", l, s, n, want);
        }
    return LB_OK;
}

/* ---- writer ---- */
static int put(FILE* f, const void* p, size_t n) { return fwrite(p, 1, n, f) == n ? 0 : -1; }

LB_API int lb_save_weights(const char* model_dir, const lb_model_cfg* c, const void* const* layer_slots, const void* const* globals,
                           char* err, size_t errlen) {
    if (!model_dir || !c || !layer_slots || !globals) return wfail(err, errlen, LB_ERR_INVALID, "lb_save_weights: NULL argument");
    static const char shard_name[] = "lithos-weights-00001-of-00001.bin";
    const size_t n_entries = (size_t)LB_WG_SLOTS + (size_t)c->n_layers * LB_WS_SLOTS;
    unsigned char* tab = (unsigned char*)calloc(n_entries, WIDX_ENTRY);
    if (!tab) return wfail(err, errlen, LB_ERR_NOMEM, "lb_save_weights: out of memory");
    char path[1280];
    snprintf(path, sizeof path, "%s/%s", model_dir, shard_name);
    FILE* f = fopen(path, "wb");
    if (!f) { free(tab); return wfail(err, errlen, LB_ERR_IO, "lb_save_weights: cannot create %s (%s)", path, strerror(errno)); }
    /* 64 bytes of header keep every tensor off offset 0 (offset 0 with size 0 means "unused" in the index) */
    static const unsigned char head[64] = "lithos_b200 raw weight shard";
    uint64_t off = 64;
    int bad = put(f, head, 64);
    static const unsigned char zeros[64];
    for (size_t i = 0; i < n_entries && !bad; i++) {
        const void* p;
        size_t n;
        if (i < LB_WG_SLOTS) { p = globals[i]; n = lb_model_global_bytes(c, (int)i); }
        else {
            const size_t j = i - LB_WG_SLOTS;
            p = layer_slots[j];
            n = lb_model_slot_bytes(c, (int)(j / LB_WS_SLOTS), (int)(j % LB_WS_SLOTS));
        }
        if (!p || !n) continue; /* unused slot: entry stays all zero */
        unsigned char* e = tab + i * WIDX_ENTRY;
        const uint32_t shard = 0;
        const uint64_t size = n;
        memcpy(e, &shard, 4); memcpy(e + 8, &off, 8); memcpy(e + 16, &size, 8);
        bad |= put(f, p, n);
        const size_t pad = (64 - n % 64) % 64;
        bad |= put(f, zeros, pad);
        off += n + pad;
    }
    bad |= fclose(f) != 0;
    if (bad) { free(tab); return wfail(err, errlen, LB_ERR_IO, "lb_save_weights: writing %s failed", path); }
    snprintf(path, sizeof path, "%s/weight_index.bin", model_dir);
    f = fopen(path, "wb");
    if (!f) { free(tab); return wfail(err, errlen, LB_ERR_IO, "lb_save_weights: cannot create %s (%s)", path, strerror(errno)); }
    uint32_t hdr[8] = {WIDX_MAGIC, WIDX_VERSION, 1, (uint32_t)c->n_layers, LB_WS_SLOTS, LB_WG_SLOTS, 0, 0};
    unsigned char se[WIDX_SHARD_ENTRY];
    memset(se, 0, sizeof se);
    memcpy(se, shard_name, sizeof shard_name);
    memcpy(se + 256, &off, 8);
    bad = put(f, hdr, 32) | put(f, se, sizeof se) | put(f, tab, n_entries * WIDX_ENTRY);
    bad |= fclose(f) != 0;
    free(tab);
    return bad ? wfail(err, errlen, LB_ERR_IO, "lb_save_weights: writing %s failed", path) : LB_OK;
}

/* ---- load into a model: replaces load_weights + the pointer table walk (src/launcher.s:3284-3683) ---- */
LB_API int lb_load_weights(lb_ctx* c, const char* model_dir, lb_model* m) {
    if (!c || !m) return LB_ERR_INVALID;
    lb_weight_index* w = NULL;
    int st = lb_weight_index_open(model_dir, &w, c->err, sizeof c->err);
    if (st != LB_OK) return st;
    const lb_model_cfg* cfg = lb_model_config(m);
    st = lb_weight_index_check(w, cfg, c->err, sizeof c->err);
    const void* slots[LB_WS_SLOTS];
    size_t n;
    for (int l = 0; st == LB_OK && l < cfg->n_layers; l++) {
        for (int s = 0; s < LB_WS_SLOTS; s++) lb_weight_index_entry(w, l, s, &slots[s], &n);
        st = lb_model_load_layer(m, l, slots);
    }
    if (st == LB_OK) {
        const void* g[LB_WG_SLOTS];
        for (int i = 0; i < LB_WG_SLOTS; i++) lb_weight_index_entry(w, -1, i, &g[i], &n);
        st = lb_model_load_globals(m, g);
    }
    lb_weight_index_close(w); /* every tensor has been re-laid and uploaded: the mappings are no longer needed */
    return st;
}

/* ---- safetensors -> weight_index.bin --------------------------------------------------------------------------------
 * The reference resolves its slots from a safetensors checkpoint by tensor name (compiler/megakernel-link.ls:220-269 for the
 * layers, :825-827 for the globals; slot names in src/launcher.s:92-141) and its launcher then reads weight_index.bin, whose
 * generator is not in the tree.  This is that generator: every *.safetensors file of the directory becomes a shard, every slot
 * the (shard, file offset, size) of the tensor `model.layers.<n>.<suffix>`.
 * A safetensors file is: u64 LE header length, a JSON object {"<name>": {"dtype": .., "shape": [..], "data_offsets": [b, e]},
 * ..., "__metadata__": {..}}, then the data; offsets are relative to the end of the header. */
static const char* const k_dn_suffix[LB_WS_SLOTS] = {
    "linear_attn.in_proj_qkv.qweight", "linear_attn.in_proj_qkv.scales", "linear_attn.in_proj_qkv.qzeros",
    "linear_attn.in_proj_z.qweight", "linear_attn.in_proj_z.scales", "linear_attn.in_proj_z.qzeros",
    "linear_attn.out_proj.qweight", "linear_attn.out_proj.scales", "linear_attn.out_proj.qzeros",
    "linear_attn.in_proj_a.weight", "linear_attn.in_proj_b.weight", "linear_attn.A_log", "linear_attn.dt_bias",
    "linear_attn.conv1d.weight", "linear_attn.norm.weight",
    "mlp.gate_proj.qweight", "mlp.gate_proj.scales", "mlp.gate_proj.qzeros", "mlp.up_proj.qweight", "mlp.up_proj.scales", "mlp.up_proj.qzeros",
    "mlp.down_proj.qweight", "mlp.down_proj.scales", "mlp.down_proj.qzeros", "input_layernorm.weight", "post_attention_layernorm.weight"};
static const char* const k_fa_suffix[15] = {
    "self_attn.q_proj.qweight", "self_attn.q_proj.scales", "self_attn.q_proj.qzeros", "self_attn.k_proj.qweight", "self_attn.k_proj.scales",
    "self_attn.k_proj.qzeros", "self_attn.v_proj.qweight", "self_attn.v_proj.scales", "self_attn.v_proj.qzeros", "self_attn.o_proj.qweight",
    "self_attn.o_proj.scales", "self_attn.o_proj.qzeros", "self_attn.q_norm.weight", "self_attn.k_norm.weight", NULL};
static const char* const k_global_name[LB_WG_SLOTS] = {"model.embed_tokens.weight", "lm_head.weight", "model.norm.weight"};

typedef struct { char* name; uint32_t shard; uint64_t off, size; } st_tensor;

/* p at an opening quote: returns the position after the closing quote, *s / *n the text between (escapes are skipped, not decoded) */
static const char* st_string(const char* p, const char* end, const char** s, size_t* n) {
    if (p >= end || *p != '"') return NULL;
    const char* q = ++p;
    while (q < end && *q != '"') q += (*q == '\\' && q + 1 < end) ? 2 : 1;
    if (q >= end) return NULL;
    *s = p; *n = (size_t)(q - p);
    return q + 1;
}
static const char* st_ws(const char* p, const char* end) { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; return p; }
/* p at the first character of a JSON value: returns the position after it (strings, nesting and escapes respected) */
static const char* st_skip_value(const char* p, const char* end) {
    int depth = 0;
    while (p < end) {
        if (*p == '"') { const char* s; size_t n; p = st_string(p, end, &s, &n); if (!p) return NULL; if (!depth) return p; continue; }
        if (*p == '{' || *p == '[') depth++;
        else if (*p == '}' || *p == ']') { if (--depth == 0) return p + 1; if (depth < 0) return NULL; }
        else if (!depth && (*p == ',')) return p;
        p++;
    }
    return depth ? NULL : p;
}

/* the tensors of one header; data_base = file offset of the data section */
static int st_parse_header(const char* js, size_t len, uint32_t shard, uint64_t data_base, uint64_t file_bytes, st_tensor** tab, size_t* n_tab,
                           size_t* cap, char* err, size_t errlen, const char* file) {
    const char *p = st_ws(js, js + len), *end = js + len;
    if (p >= end || *p != '{') return wfail(err, errlen, LB_ERR_IO, "%s: the header is not a JSON object", file);
    p = st_ws(p + 1, end);
    while (p < end && *p != '}') {
        const char* key; size_t klen;
        p = st_string(p, end, &key, &klen);
        if (!p) return wfail(err, errlen, LB_ERR_IO, "%s: malformed header (tensor name)", file);
        p = st_ws(p, end);
        if (p >= end || *p != ':') return wfail(err, errlen, LB_ERR_IO, "%s: malformed header (':' after a name)", file);
        p = st_ws(p + 1, end);
        const char* v0 = p;
        const char* v1 = st_skip_value(p, end);
        if (!v1) return wfail(err, errlen, LB_ERR_IO, "%s: malformed header (value of %.*s)", file, (int)klen, key);
        if (!(klen == 12 && !memcmp(key, "__metadata__", 12))) {
            /* "data_offsets": [begin, end] inside the value */
            const char* d = NULL;
            for (const char* q = v0; q + 14 <= v1; q++)
                if (!memcmp(q, "\"data_offsets\"", 14)) { d = q + 14; break; }
            unsigned long long b = 0, e = 0;
            char num[96]; /* a bounded, terminated copy: the header is a slice of a mapped file */
            size_t nn = d ? (size_t)(v1 - d) : 0;
            if (nn > sizeof num - 1) nn = sizeof num - 1;
            if (d) memcpy(num, d, nn);
            num[nn] = 0;
            if (!d || sscanf(num, " : [ %llu , %llu ]", &b, &e) != 2 || e < b || data_base + e > file_bytes)
                return wfail(err, errlen, LB_ERR_IO, "%s: tensor %.*s has no valid data_offsets", file, (int)klen, key);
            if (*n_tab == *cap) {
                *cap = *cap ? *cap * 2 : 1024;
                st_tensor* t = (st_tensor*)realloc(*tab, *cap * sizeof **tab);
                if (!t) return wfail(err, errlen, LB_ERR_NOMEM, "weight index: out of memory");
                *tab = t;
            }
            st_tensor* t = &(*tab)[(*n_tab)++];
            t->name = (char*)malloc(klen + 1);
            if (!t->name) return wfail(err, errlen, LB_ERR_NOMEM, "weight index: out of memory");
            memcpy(t->name, key, klen); t->name[klen] = 0;
            t->shard = shard; t->off = data_base + b; t->size = e - b;
        }
        p = st_ws(v1, end);
        if (p < end && *p == ',') p = st_ws(p + 1, end);
    }
    return LB_OK;
}

static int st_cmp_name(const void* a, const void* b) { return strcmp(((const st_tensor*)a)->name, ((const st_tensor*)b)->name); }
static int st_cmp_str(const void* a, const void* b) { return strcmp(*(const char* const*)a, *(const char* const*)b); }

#include <dirent.h>

LB_API int lb_weight_index_from_safetensors(const char* model_dir, const lb_model_cfg* c, char* err, size_t errlen) {
    if (!model_dir || !c) return wfail(err, errlen, LB_ERR_INVALID, "lb_weight_index_from_safetensors: NULL argument");
    /* the shard files, in name order */
    char* files[WIDX_MAX_SHARDS];
    int n_files = 0, st = LB_OK;
    DIR* d = opendir(model_dir);
    if (!d) return wfail(err, errlen, LB_ERR_IO, "cannot open %s (%s)", model_dir, strerror(errno));
    for (struct dirent* e; (e = readdir(d)) != NULL;) {
        const size_t n = strlen(e->d_name);
        if (n < 13 || n > 255 || strcmp(e->d_name + n - 12, ".safetensors")) continue;
        if (n_files == WIDX_MAX_SHARDS) { st = wfail(err, errlen, LB_ERR_IO, "%s holds more than %d safetensors files", model_dir, WIDX_MAX_SHARDS); break; }
        files[n_files++] = strdup(e->d_name);
    }
    closedir(d);
    if (st == LB_OK && !n_files) st = wfail(err, errlen, LB_ERR_IO, "%s holds no *.safetensors file", model_dir);
    qsort(files, (size_t)n_files, sizeof files[0], st_cmp_str);
    st_tensor* tab = NULL;
    size_t n_tab = 0, cap = 0;
    uint64_t shard_bytes[WIDX_MAX_SHARDS] = {0};
    for (int i = 0; i < n_files && st == LB_OK; i++) {
        char path[1536];
        snprintf(path, sizeof path, "%s/%s", model_dir, files[i]);
        size_t bytes = 0;
        unsigned char* m = map_file(path, &bytes);
        if (!m) { st = wfail(err, errlen, LB_ERR_IO, "cannot map %s (%s)", path, strerror(errno)); break; }
        shard_bytes[i] = bytes;
        uint64_t hlen = bytes >= 8 ? rd64(m) : 0;
        if (bytes < 8 || hlen > bytes - 8) st = wfail(err, errlen, LB_ERR_IO, "%s: header length %llu does not fit the file", path, (unsigned long long)hlen);
        else st = st_parse_header((const char*)m + 8, (size_t)hlen, (uint32_t)i, 8 + hlen, bytes, &tab, &n_tab, &cap, err, errlen, files[i]);
        munmap(m, bytes);
    }
    const size_t n_entries = (size_t)LB_WG_SLOTS + (size_t)c->n_layers * LB_WS_SLOTS;
    unsigned char* out = st == LB_OK ? (unsigned char*)calloc(n_entries, WIDX_ENTRY) : NULL;
    if (st == LB_OK && !out) st = wfail(err, errlen, LB_ERR_NOMEM, "weight index: out of memory");
    if (st == LB_OK) {
        qsort(tab, n_tab, sizeof *tab, st_cmp_name);
        for (size_t i = 0; i < n_entries && st == LB_OK; i++) {
            char name[320];
            size_t want;
            if (i < LB_WG_SLOTS) {
                snprintf(name, sizeof name, "%s", k_global_name[i]);
                want = lb_model_global_bytes(c, (int)i);
            } else {
                const int l = (int)((i - LB_WG_SLOTS) / LB_WS_SLOTS), s = (int)((i - LB_WG_SLOTS) % LB_WS_SLOTS);
                const char* suffix = (s < 15 && layer_is_fa(c, l)) ? k_fa_suffix[s] : k_dn_suffix[s];
                want = lb_model_slot_bytes(c, l, s);
                if (!suffix || !want) continue; /* slot unused in this kind of layer */
                snprintf(name, sizeof name, "model.layers.%d.%s", l, suffix);
            }
            st_tensor key;
            key.name = name;
            const st_tensor* t = (const st_tensor*)bsearch(&key, tab, n_tab, sizeof *tab, st_cmp_name);
            if (!t) { st = wfail(err, errlen, LB_ERR_INVALID, "tensor %s is not in the checkpoint", name); break; }
            if (t->size != want) { st = wfail(err, errlen, LB_ERR_IO, "tensor %s holds %llu bytes, the model shape needs %zu", name, (unsigned long long)t->size, want); break; }
            unsigned char* e = out + i * WIDX_ENTRY;
            memcpy(e, &t->shard, 4); memcpy(e + 8, &t->off, 8); memcpy(e + 16, &t->size, 8);
        }
    }
    if (st == LB_OK) {
        char path[1536];
        snprintf(path, sizeof path, "%s/weight_index.bin", model_dir);
        FILE* f = fopen(path, "wb");
        if (!f) st = wfail(err, errlen, LB_ERR_IO, "cannot create %s (%s)", path, strerror(errno));
        else {
            uint32_t hdr[8] = {WIDX_MAGIC, WIDX_VERSION, (uint32_t)n_files, (uint32_t)c->n_layers, LB_WS_SLOTS, LB_WG_SLOTS, 0, 0};
            int bad = put(f, hdr, 32);
            for (int i = 0; i < n_files; i++) {
                unsigned char se[WIDX_SHARD_ENTRY];
                memset(se, 0, sizeof se);
                memcpy(se, files[i], strlen(files[i]));
                memcpy(se + 256, &shard_bytes[i], 8);
                bad |= put(f, se, sizeof se);
            }
            bad |= put(f, out, n_entries * WIDX_ENTRY);
            bad |= fclose(f) != 0;
            if (bad) st = wfail(err, errlen, LB_ERR_IO, "writing %s failed", path);
        }
    }
    for (size_t i = 0; i < n_tab; i++) free(tab[i].name);
    free(tab);
    free(out);
    for (int i = 0; i < n_files; i++) free(files[i]);
    return st;
}
