"""ctypes/numpy front-end of oracle/golden.c (the C restatement of the reference's CPU
golden model, deepgemm/src/golden.rs:56-510).  Test infrastructure only."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

FP8, FP4 = 0, 1


def build(force=False):
    """Compile golden.c into liboracle.so (gcc, OpenMP)."""
    src = os.path.join(_HERE, "golden.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        u8p, u32p, f32p = C.POINTER(C.c_uint8), C.POINTER(C.c_uint32), C.POINTER(C.c_float)
        u32 = C.c_uint32
        L.dgo_e4m3_decode.restype = C.c_float
        L.dgo_e4m3_decode.argtypes = [C.c_uint8]
        L.dgo_e2m1_decode.restype = C.c_float
        L.dgo_e2m1_decode.argtypes = [C.c_uint8]
        L.dgo_ue8m0_decode.restype = C.c_float
        L.dgo_ue8m0_decode.argtypes = [C.c_uint8]
        L.dgo_f32_to_ue8m0.restype = C.c_uint8
        L.dgo_f32_to_ue8m0.argtypes = [C.c_float]
        L.dgo_quant_e4m3.restype = C.c_uint8
        L.dgo_quant_e4m3.argtypes = [C.c_float]
        L.dgo_quant_e2m1.restype = C.c_uint8
        L.dgo_quant_e2m1.argtypes = [C.c_float]
        L.dgo_ue8m0_exp_fp8.restype = C.c_uint8
        L.dgo_ue8m0_exp_fp8.argtypes = [C.c_float]
        L.dgo_ue8m0_exp_fp4.restype = C.c_uint8
        L.dgo_ue8m0_exp_fp4.argtypes = [C.c_float]
        L.dgo_tma_aligned.restype = u32
        L.dgo_tma_aligned.argtypes = [u32, u32]
        L.dgo_f32_to_bf16_bits.restype = C.c_uint16
        L.dgo_f32_to_bf16_bits.argtypes = [C.c_float]
        L.dgo_quant_e4m3_vec.argtypes = [f32p, C.c_size_t, u8p]
        L.dgo_transform_sf_host.argtypes = [f32p, u32, u32, u32p]
        L.dgo_quant_mx_host.argtypes = [f32p, u32, u32, C.c_int, u32, u8p, u32p]
        L.dgo_quant_fp8_block128_host.argtypes = [f32p, u32, u32, u8p, u32p]
        L.dgo_dequant_mx_host.argtypes = [u8p, u32p, u32, u32, u32, C.c_int, u32, f32p]
        opnd = [u8p, u32p, u32, C.c_int, u32]
        L.dgo_gemm_ref_sub.argtypes = opnd + opnd + [u32, u32p, u32, u32p, u32, u32, f32p, u32]
        L.dgo_gemm_ref_naive.argtypes = opnd + opnd + [u32, u32, u32, f32p]
        L.dgo_gemm_f32_ref.argtypes = [f32p, f32p, u32, u32, u32, f32p]
        L.dgo_mqa_logits_ref.argtypes = [f32p, f32p, f32p, u32, u32, u32, u32p, u32p, u32p, u32, f32p]
        L.dgo_swiglu_f32.argtypes = [C.POINTER(C.c_uint16), u32, u32, u32, f32p]
        L.dgo_exp_taylor6.restype = C.c_float
        L.dgo_exp_taylor6.argtypes = [C.c_float]
        L.dgo_hash_u32.restype = u32
        L.dgo_hash_u32.argtypes = [C.c_uint64, u32]
        L.dgo_quantize_output_fp8.argtypes = [f32p, u32, u32, u32, C.c_int, u32, u8p, u32p]
        L.dgo_transform_sf_batched_host.argtypes = [f32p, u32, u32, u32, u32p]
        L.dgo_set_threads.argtypes = [C.c_int]
        L.dgo_get_threads.restype = C.c_int
        L.dgo_calc_diff.restype = C.c_double
        L.dgo_calc_diff.argtypes = [f32p, f32p, C.c_size_t]
        _lib = L
    return _lib


def _p(a, ty):
    return a.ctypes.data_as(C.POINTER(ty)) if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---- scalar codecs -------------------------------------------------------------------
def e4m3_decode(b): return float(lib().dgo_e4m3_decode(int(b)))
def e2m1_decode(n): return float(lib().dgo_e2m1_decode(int(n)))
def ue8m0_decode(c): return float(lib().dgo_ue8m0_decode(int(c)))
def f32_to_ue8m0(v): return int(lib().dgo_f32_to_ue8m0(float(v)))
def quant_e4m3(v): return int(lib().dgo_quant_e4m3(C.c_float(v)))
def quant_e2m1(v): return int(lib().dgo_quant_e2m1(C.c_float(v)))
def ue8m0_exp_fp8(a): return int(lib().dgo_ue8m0_exp_fp8(C.c_float(a)))
def ue8m0_exp_fp4(a): return int(lib().dgo_ue8m0_exp_fp4(C.c_float(a)))
def f32_to_bf16_bits(v): return int(lib().dgo_f32_to_bf16_bits(C.c_float(v)))
def tma_aligned(mn, elem_size=4): return int(lib().dgo_tma_aligned(mn, elem_size))
def ceil_div(a, b): return (a + b - 1) // b


def sf_shape(rows, k, gran):
    """(packed K rows, TMA-aligned MN) of the packed-UE8M0 tensor."""
    return ceil_div(k // gran, 4), tma_aligned(rows, 4)


# ---- array functions -----------------------------------------------------------------
def transform_sf_host(sf, mn):
    sf = _c(sf, np.float32).reshape(mn, -1)
    sf_k = sf.shape[1]
    out = np.zeros((ceil_div(sf_k, 4), tma_aligned(mn)), dtype=np.uint32)
    lib().dgo_transform_sf_host(_p(sf, C.c_float), mn, sf_k, _p(out, C.c_uint32))
    return out


def quant_mx_host(x, dtype, gran):
    """x f32 [m, k] -> (codes u8 [m, k] or [m, k/2], sf u32 [ceil(k/g/4), align4(m)])."""
    x = _c(x, np.float32)
    m, k = x.shape
    assert k % gran == 0
    data = np.zeros((m, k // 2 if dtype == FP4 else k), dtype=np.uint8)
    sf = np.zeros(sf_shape(m, k, gran), dtype=np.uint32)
    lib().dgo_quant_mx_host(_p(x, C.c_float), m, k, dtype, gran, _p(data, C.c_uint8), _p(sf, C.c_uint32))
    return data, sf


def quant_fp8_block128_host(x):
    """Input generator: E4M3 codes with one UE8M0 scale per 128x128 block, written as the
    per-row G128 packed layout (the block's byte replicated on its 128 rows)."""
    x = _c(x, np.float32)
    n, k = x.shape
    assert k % 128 == 0
    data = np.zeros((n, k), dtype=np.uint8)
    sf = np.zeros(sf_shape(n, k, 128), dtype=np.uint32)
    lib().dgo_quant_fp8_block128_host(_p(x, C.c_float), n, k, _p(data, C.c_uint8), _p(sf, C.c_uint32))
    return data, sf


def dequant_mx_host(data, sf, m, k, dtype, gran):
    data, sf = _c(data, np.uint8), _c(sf, np.uint32)
    out = np.zeros((m, k), dtype=np.float32)
    lib().dgo_dequant_mx_host(_p(data, C.c_uint8), _p(sf, C.c_uint32), sf.shape[-1], m, k, dtype, gran,
                              _p(out, C.c_float))
    return out


class GoldenOperand:
    """K-major codes + packed SF, as golden.rs:404-414."""

    def __init__(self, data, sf, dtype, gran, k):
        self.data, self.sf = _c(data, np.uint8), _c(sf, np.uint32)
        self.dtype, self.gran, self.k = dtype, gran, k

    def args(self):
        return [_p(self.data, C.c_uint8), _p(self.sf, C.c_uint32), self.sf.shape[-1], self.dtype, self.gran]


def gemm_ref(a, b, rows=None, cols=None, m=None, n=None, b_row0=0):
    """f32 [len(rows), len(cols)] of A.B^T in f64 (golden.rs:444-458) on a sub-rectangle."""
    assert a.k == b.k
    r = _c(rows, np.uint32) if rows is not None else None
    c = _c(cols, np.uint32) if cols is not None else None
    nr = len(r) if r is not None else m
    nc = len(c) if c is not None else n
    out = np.zeros((nr, nc), dtype=np.float32)
    lib().dgo_gemm_ref_sub(*a.args(), *b.args(), a.k, _p(r, C.c_uint32), nr, _p(c, C.c_uint32), nc,
                           b_row0, _p(out, C.c_float), nc)
    return out


def gemm_ref_naive(a, b, m, n):
    out = np.zeros((m, n), dtype=np.float32)
    lib().dgo_gemm_ref_naive(*a.args(), *b.args(), m, n, a.k, _p(out, C.c_float))
    return out


def gemm_f32_ref(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    m, k = a.shape
    n = b.shape[0]
    out = np.zeros((m, n), dtype=np.float32)
    lib().dgo_gemm_f32_ref(_p(a, C.c_float), _p(b, C.c_float), m, n, k, _p(out, C.c_float))
    return out


def mqa_logits_ref(q, kv, weights, k_start, k_end, tokens=None):
    """q f32 [T, H, D], kv f32 [S, D], weights f32 [T, H] -> f32 [len(tokens) or T, S]."""
    q, kv, weights = _c(q, np.float32), _c(kv, np.float32), _c(weights, np.float32)
    T, H, D = q.shape
    S = kv.shape[0]
    ks, ke = _c(k_start, np.uint32), _c(k_end, np.uint32)
    t = _c(tokens, np.uint32) if tokens is not None else None
    nt = len(t) if t is not None else T
    out = np.zeros((nt, S), dtype=np.float32)
    lib().dgo_mqa_logits_ref(_p(q, C.c_float), _p(kv, C.c_float), _p(weights, C.c_float), H, D, S,
                             _p(ks, C.c_uint32), _p(ke, C.c_uint32), _p(t, C.c_uint32), nt, _p(out, C.c_float))
    return out


def swiglu_f32(inter_bf16_bits, inter):
    """bf16 bits [m, 2 * inter] (gate half, up half) -> f32 [m, inter] = silu(gate) * up."""
    a = _c(inter_bf16_bits, np.uint16)
    m = a.shape[0]
    out = np.zeros((m, inter), dtype=np.float32)
    lib().dgo_swiglu_f32(_p(a, C.c_uint16), m, inter, a.shape[1], _p(out, C.c_float))
    return out


def quantize_output_fp8(x, n, stochastic=False, seed=0):
    """x f32 [m, in_stride >= n] -> (codes u8 [m, n], sf u32 [ceil(n/32/4), align4(m)]) (api.rs:1951-2011)."""
    x = _c(x, np.float32)
    m, in_stride = x.shape
    data = np.zeros((m, n), dtype=np.uint8)
    sf = np.zeros(sf_shape(m, n, 32), dtype=np.uint32)
    lib().dgo_quantize_output_fp8(_p(x, C.c_float), m, n, in_stride, 1 if stochastic else 0, seed, _p(data, C.c_uint8),
                                  _p(sf, C.c_uint32))
    return data, sf


def transform_sf_batched_host(sf, batch, mn):
    sf = _c(sf, np.float32).reshape(batch, mn, -1)
    sf_k = sf.shape[2]
    out = np.zeros((batch * ceil_div(sf_k, 4), tma_aligned(mn)), dtype=np.uint32)
    lib().dgo_transform_sf_batched_host(_p(sf, C.c_float), batch, mn, sf_k, _p(out, C.c_uint32))
    return out


def exp_taylor6(x): return float(lib().dgo_exp_taylor6(C.c_float(x)))
def hash_u32(idx, seed): return int(lib().dgo_hash_u32(int(idx), int(seed)))


def set_threads(n):
    """Thread count of the oracle's OpenMP loops (returns the count in effect)."""
    lib().dgo_set_threads(int(n))
    return int(lib().dgo_get_threads())


def calc_diff(x, y):
    x, y = _c(x, np.float32).ravel(), _c(y, np.float32).ravel()
    assert x.size == y.size
    return float(lib().dgo_calc_diff(_p(x, C.c_float), _p(y, C.c_float), x.size))


def bf16_bits_to_f32(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits_np(x):
    """Vector form of f32_to_bf16_bits (golden.rs:505-510)."""
    b = _c(x, np.float32).view(np.uint32).astype(np.uint64)
    r = 0x7FFF + ((b >> 16) & 1)
    return ((((b + r) >> 16) & 0x7FFF) | ((b >> 31) << 15)).astype(np.uint16)


def quant_e4m3_array(x):
    """Element-wise quant_e4m3 (golden.rs:180-189): f32 array -> E4M3 bytes of the same shape."""
    x = _c(x, np.float32)
    out = np.zeros(x.shape, dtype=np.uint8)
    lib().dgo_quant_e4m3_vec(_p(x, C.c_float), x.size, _p(out, C.c_uint8))
    return out


def e4m3_table():
    return np.array([e4m3_decode(i) for i in range(256)], dtype=np.float32)
