"""CPU: the C-ABI library loads without a GPU driver and exports every symbol that
include/lithos_b200.h declares; the Python constants mirror the header's enums; and
calls that need a device fail loudly (no fallback)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "lithos_b200.h").read_text()


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(lb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lb):
    L = ctypes.CDLL(str(ROOT / "lithos_b200" / "liblithos_b200.so"))
    names = declared_functions()
    assert len(names) > 30
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_header_enums_match_python(lb):
    def enum_value(name):
        m = re.search(rf"\b{name}\s*=\s*([^,\n/]+)", HEADER)
        assert m, name
        return eval(m.group(1))

    for name in ("LB_OK", "LB_ERR_INVALID", "LB_ERR_NO_DRIVER", "LB_ERR_CUDA", "LB_ERR_NO_KERNEL", "LB_ERR_DEVICE_WAIT",
                 "LB_ERR_IO", "LB_ERR_NOMEM", "LB_ERR_STATE"):
        assert enum_value(name) == getattr(lb, name)
    assert enum_value("LB_GEMV_X_F32") == lb.GEMV_X_F32
    assert enum_value("LB_GEMV_Y_F32") == lb.GEMV_Y_F32
    assert enum_value("LB_GEMV_Y_ACCUM") == lb.GEMV_Y_ACCUM
    assert enum_value("LB_GEMV_Y_SWIGLU") == lb.GEMV_Y_SWIGLU


def test_kernel_images_are_built(lb):
    kdir = ROOT / "lithos_b200" / "kernels"
    for f in ("gemv.cubin", "chain.cubin", "batched.cubin", "batched_tc.cubin", "deltanet.cubin", "attention.cubin", "attention_mma.cubin", "small.cubin", "compat/gptq_gemv_safe.cubin", "compat/norm.cubin",
              "compat/activate.cubin", "compat/gate_sigmoid.cubin", "compat/reduce.cubin", "compat/embed_f16.cubin",
              "compat/lm_head.cubin", "compat/sample.cubin", "compat/attention_score.cubin", "compat/recur.cubin", "compat/conv1d.cubin",
              "compat/rotate.cubin"):
        assert (kdir / f).stat().st_size > 1000, f


def test_no_device_is_an_error_not_a_fallback(lb):
    """Without a CUDA driver/GPU the context cannot be created and says why."""
    import shutil
    if shutil.which("nvidia-smi"):
        pytest.skip("a GPU driver is present on this machine")
    with pytest.raises(lb.LithosError) as e:
        lb.Context(0)
    assert e.value.status == lb.LB_ERR_NO_DRIVER


def test_generator_is_counter_based(lb):
    import numpy as np
    a = lb.fill_u32(1000, 7, 3)
    b = lb.fill_u32(2000, 7, 3)
    assert np.array_equal(a, b[:1000])                       # element i depends on (seed, stream, i) only
    assert not np.array_equal(a, lb.fill_u32(1000, 8, 3))
    assert not np.array_equal(a, lb.fill_u32(1000, 7, 4))
    nib = np.stack([(a >> (4 * j)) & 0xF for j in range(8)])
    assert nib.min() == 0 and nib.max() == 15
    s = lb.fill_scales_f16(4096, 1, 2).astype(np.float64)
    assert s.min() >= 1e-3 - 1e-6 and abs(s.mean() - (0.01 * 0.7979 + 1e-3)) < 1e-3
    x = lb.fill_normal(100000, 1, 4).astype(np.float64)
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1) < 0.02
    bf = lb.fill_normal(1000, 1, 5, dtype="bf16")
    f = lb.fill_normal(1000, 1, 5, dtype="f32")
    assert np.array_equal(bf, lb.f32_to_bf16(f))
