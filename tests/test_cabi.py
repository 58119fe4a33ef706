"""CPU-side checks of the drop-in boundary: the shared library loads without a GPU driver,
exports every symbol include/deepgemm_b200.h declares, validates arguments like the reference
(deepgemm/src/api.rs:677-715, 868-879, 995-1022, 1489-1498) and refuses to compute without an
sm_100 device instead of falling back."""
import ctypes as C

import pytest
import torch

from deepgemm import _lib


@pytest.fixture(scope="module")
def L():
    return _lib.load()


def test_every_declared_symbol_is_exported(L):
    names = _lib.declared_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_version_and_sf_shape(L):
    assert b"sm_100a" in L.dg_version()
    r, c = C.c_uint32(), C.c_uint32()
    L.dg_sf_shape(101, 7168, 32, C.byref(r), C.byref(c))
    assert (r.value, c.value) == (56, 104)          # cpu_tests.rs:109-118
    L.dg_sf_shape(100, 7168, 128, C.byref(r), C.byref(c))
    assert (r.value, c.value) == (14, 100)


def _op(dtype, rows, k, sf=True, major=0, data=0x1000):
    s = _lib.SfTensorC((k + 127) // 128, (rows + 3) // 4 * 4, 32, 0x2000 if sf else None)
    return _lib.OperandC(dtype, major, rows, k, k, s, data)


def _out(rows, cols, dtype=2):
    return _lib.OutputC(dtype, rows, cols, cols, 0x3000)


def _err(L):
    return L.dg_last_error().decode()


@pytest.mark.parametrize("dtype,k,msg", [(0, 100, "FP8 K (100) must be a multiple of 128"),
                                         (1, 128, "FP4 K (128) must be a multiple of 256"),
                                         (2, 32, "BF16 K (32) must be a multiple of 64")])
def test_k_multiples(L, dtype, k, msg):
    a, b, o = _op(dtype, 128, k), _op(dtype, 128, k), _out(128, 128)
    assert L.dg_gemm_nt(C.byref(a), C.byref(b), C.byref(o), 0, None) == 3
    assert msg in _err(L)


def test_shape_and_dtype_checks(L):
    a, b = _op(0, 128, 256), _op(0, 64, 512)
    o = _out(128, 64)
    assert L.dg_gemm_nt(C.byref(a), C.byref(b), C.byref(o), 0, None) == 3 and "K mismatch" in _err(L)
    b = _op(0, 64, 256)
    o = _out(128, 65)
    assert L.dg_gemm_nt(C.byref(a), C.byref(b), C.byref(o), 0, None) == 3 and "output shape mismatch" in _err(L)
    o = _out(128, 64, dtype=0)
    assert L.dg_gemm_nt(C.byref(a), C.byref(b), C.byref(o), 0, None) == 3 and "BF16 or FP32" in _err(L)
    o = _out(128, 64)
    b = _op(0, 64, 256, sf=False)
    assert L.dg_gemm_nt(C.byref(a), C.byref(b), C.byref(o), 0, None) == 3 and "require scale factors" in _err(L)
    b = _op(0, 64, 256)
    assert L.dg_fp4_gemm_nt(C.byref(a), C.byref(b), C.byref(o), 0, None) == 3 and "must be FP4" in _err(L)
    a4, b4 = _op(1, 128, 256, major=1), _op(1, 64, 256)
    assert L.dg_gemm_nt(C.byref(a4), C.byref(b4), C.byref(o), 0, None) == 3 and "K-major" in _err(L)


def test_grouped_checks(L):
    a, b, o = _op(0, 192, 256), _op(0, 64, 256), _out(192, 64)
    assert L.dg_m_grouped_gemm_nt_contiguous(C.byref(a), C.byref(b), C.byref(o), 0x4000, 1, 2, None) == 3
    assert "multiple of 128" in _err(L)
    a, o = _op(0, 256, 256), _out(256, 64)
    assert L.dg_m_grouped_gemm_nt_contiguous(C.byref(a), C.byref(b), C.byref(o), 0x4000, 1, 2, None) == 3
    assert "one per 128-row block" in _err(L)
    am = _op(0, 256, 256, major=1)
    assert L.dg_m_grouped_gemm_nt_masked(C.byref(am), C.byref(b), C.byref(o), 0x4000, 2, 128, None) == 3
    assert "K-major" in _err(L)


def test_gathered_rows_checks(L):
    """The grouped GEMM that gathers the rows of A: row list, dtype and source row count are checked on any machine."""
    a, b, o = _op(0, 256, 256), _op(0, 64, 256), _out(256, 64)
    f = L.dg_m_grouped_gemm_nt_contiguous_gather
    assert f(C.byref(a), None, 300, C.byref(b), C.byref(o), 0x4000, 2, 2, None) == 3 and "row list" in _err(L)
    assert f(C.byref(a), 0x5000, 0, C.byref(b), C.byref(o), 0x4000, 2, 2, None) == 3 and "source row count" in _err(L)
    assert f(C.byref(a), 0x5004, 300, C.byref(b), C.byref(o), 0x4000, 2, 2, None) == 3 and "16-byte aligned" in _err(L)
    a4, b4 = _op(1, 256, 256), _op(1, 64, 256)
    assert f(C.byref(a4), 0x5000, 300, C.byref(b4), C.byref(o), 0x4000, 2, 2, None) == 3 and "K-major FP8" in _err(L)


def test_paged_mqa_checks(L):
    """dg_mqa_logits_paged reads the cache's scale words four tokens at a time: they must be 16-byte aligned."""
    q = _op(0, 2 * 64, 128)
    args = lambda kv_sf: (C.byref(q), 0x10000, kv_sf, 0x20000, 64, 8, 0x30000, 0x40000, 0x50000, 4, 2, 64, 128, 0x60000, 256, None)
    assert L.dg_mqa_logits_paged(*args(0x70004)) == 3 and "16-byte aligned" in _err(L)
    assert L.dg_mqa_logits_paged(*args(None)) == 3 and "null buffer" in _err(L)


def test_quant_checks(L):
    assert L.dg_quant_mx(0x1000, 16, 100, 0, 32, 0x2000, 0x3000, None) == 3      # K % gran
    assert L.dg_quant_mx(0x1000, 16, 256, 1, 128, 0x2000, 0x3000, None) == 3     # FP4 needs gran 32
    assert "FP4 requires granularity 32" in _err(L)
    assert L.dg_quant_mx(0x1000, 16, 256, 2, 32, 0x2000, 0x3000, None) == 3      # dtype
    assert L.dg_transform_sf(0x1000, 0, 4, 0x2000, None) == 3


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback(L):
    """Valid arguments, no sm_100 device: Unsupported, never a host computation."""
    a, b, o = _op(0, 128, 256), _op(0, 64, 256), _out(128, 64)
    assert L.dg_device_check() == 4
    assert L.dg_gemm_nt(C.byref(a), C.byref(b), C.byref(o), 0, None) == 4
    assert "SM100" in _err(L)
    assert L.dg_quant_mx(0x1000, 16, 256, 0, 32, 0x2000, 0x3000, None) == 4
    assert L.dg_transform_sf(0x1000, 4, 4, 0x2000, None) == 4


def test_peer_and_ffn_entry_checks(L):
    """The entries beyond the reference's API validate before they touch a device."""
    assert L.dg_swiglu_quant(0x1000, 512, 8, 192, 128, 0x2000, 0x3000, None) == 3      # width % granularity
    assert L.dg_swiglu_quant(0x1000, 512, 8, 512, 128, 0x2000, 0x3000, None) == 3      # pitch < 2 * inter
    assert L.dg_swiglu_quant(0x1000, 512, 8, 256, 64, 0x2000, 0x3000, None) == 3       # granularity
    assert L.dg_peer_barrier(0x1000, 0x2000, 2, 2, 1, None) == 3                       # rank outside the world
    assert L.dg_peer_barrier(0x1000, 0x2000, 0, 65, 1, None) == 3                      # more than 64 ranks
    assert L.dg_ep_route(0x1000, 3, 0, 8, 128, 1024, 1, None, 0x2000, 0x3000, 0x4000, None) == 3   # experts % ranks
    assert L.dg_ep_route(0x1000, 2, 0, 8, 128, 1000, 1, None, 0x2000, 0x3000, 0x4000, None) == 3   # capacity % alignment
    bounds = (C.c_uint32 * 3)(0, 3, 3)
    assert L.dg_ep_route(0x1000, 2, 0, 8, 128, 1024, 2, bounds, 0x2000, 0x3000, 0x4000, None) == 3          # bounds must ascend to e_local
    assert L.dg_moe_return_ptrs(0x1000, 4, 0x2000, 0x3000, 0x4000, 2, 100, 0x5000, None) == 3     # row bytes % 16
    assert L.dg_peer_copy(None, 0x1000, 16, None) == 3
    assert L.dg_peer_copy(0x1000, 0x2000, 0, None) == 0                                # empty copy is a no-op
    assert L.dg_m_grouped_gemm_nt_contiguous_rowptr(None, None, 0x1000, 1, 1, 0x2000, None, 0, 0, None) == 3


def test_layout_batch_and_output_quant_checks(L):
    a, b, o = _op(0, 128, 256), _op(0, 64, 256), _out(128, 64)
    for fn, who in ((L.dg_gemm_nn, "B"), (L.dg_gemm_tn, "A"), (L.dg_gemm_tt, "A")):
        assert fn(C.byref(a), C.byref(b), C.byref(o), 0, None) == 3 and f"{who} must be described as an MN-major view" in _err(L)
    amn = _lib.OperandC(0, 1, 128, 256, 64, a.sf, 0x1000)            # MN-major pitch below its rows
    assert L.dg_gemm_tn(C.byref(amn), C.byref(b), C.byref(o), 0, None) == 3 and "MN-major outer_stride" in _err(L)
    a2 = _op(2, 128, 256, sf=False)
    assert L.dg_gemm_nt(C.byref(a2), C.byref(b), C.byref(o), 0, None) == 3 and "cannot be multiplied" in _err(L)
    assert L.dg_fp8_bmm(C.byref(a2), C.byref(a2), C.byref(o), 2, 0, None) == 3 and "must be FP8" in _err(L)
    assert L.dg_bmm(C.byref(a), C.byref(b), C.byref(o), 0, 0, None) == 3 and "num_groups must be positive" in _err(L)
    assert L.dg_bmm(C.byref(a), C.byref(b), C.byref(o), 2, 0, None) == 3 and "scale-factor tensor" in _err(L)   # arenas hold one batch only
    assert L.dg_transform_sf_batched(0x1000, 0, 4, 4, 0x2000, None) == 3 and "batch must be nonzero" in _err(L)
    assert L.dg_quantize_output_fp8(0x1000, 16, 100, 100, 0, 0, 0x2000, 0x3000, None) == 3 and "n % 32 == 0" in _err(L)
    assert L.dg_quantize_output_fp8(0x1000, 16, 128, 64, 0, 0, 0x2000, 0x3000, None) == 3                          # pitch below n


def test_rust_binding_declares_every_entry():
    """deepgemm-rs_b200/rust/ffi_b200.rs (the binding a maintainer of the reference adds) lists exactly the
    functions of the public header."""
    import os
    import re
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(_lib.__file__))), "rust", "ffi_b200.rs")
    with open(path) as f:
        rust = set(re.findall(r"pub fn (dg_\w+)\s*\(", f.read()))
    assert rust == set(_lib.declared_symbols()), (sorted(set(_lib.declared_symbols()) - rust), sorted(rust - set(_lib.declared_symbols())))
