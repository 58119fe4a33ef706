"""Loads libdeepgemm_b200.so and declares its C ABI (include/deepgemm_b200.h) for ctypes."""
import ctypes as C
import os
import re

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libdeepgemm_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_PKG), "include", "deepgemm_b200.h")


class SfTensorC(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("cols", C.c_uint32), ("gran", C.c_uint32), ("data", C.c_void_p)]


class OperandC(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("major", C.c_int32), ("rows", C.c_uint32), ("k", C.c_uint32),
                ("outer_stride", C.c_uint32), ("sf", SfTensorC), ("data", C.c_void_p)]


class OutputC(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rows", C.c_uint32), ("cols", C.c_uint32), ("stride", C.c_uint32),
                ("data", C.c_void_p)]


class GemmConfigC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("block_m", "block_n", "block_k", "num_stages", "smem_bytes", "num_tiles", "grid", "cluster")]


def declared_symbols():
    """Every function name the public header declares."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return sorted(set(re.findall(r"DG_API\s+[\w\s\*]+?\b(dg_\w+)\s*\(", text)))


_lib = None


def launch_count():
    """Kernels launched by the library so far in this process."""
    return int(load().dg_launch_count())


def load(build_if_missing=True):
    """Returns the loaded library.  There is no fallback: if the shared object is missing and
    cannot be built, this raises."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise OSError(f"{LIB_PATH} is missing; run `python deepgemm-rs_b200/build.py`")
        import importlib.util
        spec = importlib.util.spec_from_file_location("_dg_build", os.path.join(_PKG, "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    L = C.CDLL(LIB_PATH)
    vp, u32, i32, u64 = C.c_void_p, C.c_uint32, C.c_int32, C.c_uint64
    opp, outp = C.POINTER(OperandC), C.POINTER(OutputC)
    L.dg_last_error.restype = C.c_char_p
    L.dg_version.restype = C.c_char_p
    L.dg_device_check.restype = i32
    L.dg_launch_count.restype = C.c_ulonglong
    L.dg_poll_device_status.argtypes = [vp]
    L.dg_sf_shape.argtypes = [u32, u32, u32, C.POINTER(u32), C.POINTER(u32)]
    L.dg_sf_shape.restype = None
    for n in ("dg_gemm_nt", "dg_fp8_gemm_nt", "dg_fp4_gemm_nt", "dg_bf16_gemm_nt"):
        getattr(L, n).argtypes = [opp, opp, outp, i32, vp]
    L.dg_gemm_nt_alpha.argtypes = [opp, opp, outp, i32, C.c_float, vp]
    for n in ("dg_gemm_nn", "dg_gemm_tn", "dg_gemm_tt"):
        getattr(L, n).argtypes = [opp, opp, outp, i32, vp]
    for n in ("dg_bmm", "dg_fp8_bmm"):
        getattr(L, n).argtypes = [opp, opp, outp, u32, i32, vp]
    L.dg_transform_sf_batched.argtypes = [vp, u32, u32, u32, vp, vp]
    L.dg_quantize_output_fp8.argtypes = [vp, u32, u32, u32, i32, u32, vp, vp, vp]
    for n in ("dg_m_grouped_gemm_nt_contiguous", "dg_m_grouped_fp8_gemm_nt_contiguous",
              "dg_m_grouped_fp4_gemm_nt_contiguous", "dg_m_grouped_bf16_gemm_nt_contiguous"):
        getattr(L, n).argtypes = [opp, opp, outp, vp, u32, u32, vp]
    L.dg_m_grouped_gemm_nt_contiguous_scatter.argtypes = [opp, opp, outp, vp, u32, u32, vp, u32, u32, vp]
    L.dg_m_grouped_gemm_nt_contiguous_gather.argtypes = [opp, vp, u32, opp, outp, vp, u32, u32, vp]
    for n in ("dg_m_grouped_gemm_nt_masked", "dg_m_grouped_fp8_gemm_nt_masked",
              "dg_m_grouped_fp4_gemm_nt_masked", "dg_m_grouped_bf16_gemm_nt_masked"):
        getattr(L, n).argtypes = [opp, opp, outp, vp, u32, u32, vp]
    L.dg_quant_mx.argtypes = [vp, u32, u32, i32, u32, vp, vp, vp]
    L.dg_quant_mx_host.argtypes = [vp, u32, u32, i32, u32, vp, vp, vp]
    L.dg_quant_mx_host_static.argtypes = [vp, u32, u32, i32, u32, vp, vp, vp]
    L.dg_swiglu_quant.argtypes = [vp, u64, u32, u32, u32, vp, vp, vp]
    L.dg_dequant_mx.argtypes = [vp, C.POINTER(SfTensorC), u32, u32, i32, vp, vp]
    L.dg_transform_sf.argtypes = [vp, u32, u32, vp, vp]
    L.dg_transform_sf_host.argtypes = [vp, u32, u32, vp, vp]
    if hasattr(L, "dg_mqa_logits_f32"):
        L.dg_mqa_logits_f32.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, vp, u32, vp]
    if hasattr(L, "dg_mqa_logits"):
        L.dg_mqa_logits.argtypes = [opp, opp, vp, vp, vp, u32, u32, u32, u32, vp, u32, vp]
    L.dg_mqa_logits_paged.argtypes = [opp, vp, vp, vp, u32, u32, vp, vp, vp, u32, u32, u32, u32, vp, u32, vp]
    L.dg_gather_rows.argtypes = [vp, u64, vp, vp, u64, u32, u32, vp]
    L.dg_gather_sf.argtypes = [vp, u64, u64, vp, vp, u64, u64, u32, u32, vp]
    L.dg_moe_plan.argtypes = [vp, u32, u32, u32, u32, u32, vp, vp, vp, vp, vp, vp, vp]
    L.dg_moe_combine.argtypes = [vp, u64, vp, vp, vp, u64, u32, u32, u32, vp]
    L.dg_peer_alloc.argtypes = [u64, C.POINTER(vp)]
    L.dg_peer_free.argtypes = [vp]
    L.dg_peer_export.argtypes = [vp, vp]
    L.dg_peer_open.argtypes = [vp, C.POINTER(vp)]
    L.dg_peer_close.argtypes = [vp]
    L.dg_peer_copy.argtypes = [vp, vp, u64, vp]
    L.dg_peer_barrier.argtypes = [vp, vp, u32, u32, u64, vp]
    L.dg_moe_return_ptrs.argtypes = [vp, u32, vp, vp, vp, u32, u64, vp, vp]
    L.dg_ep_route.argtypes = [vp, u32, u32, u32, u32, u32, u32, vp, vp, vp, vp, vp]
    L.dg_ep_push.argtypes = [vp, u64, u32, vp, u32, u64, vp, vp, vp, u32, u32, u32, u32, u32, u32, u64, vp, vp, vp, u32, vp]
    L.dg_ep_return_ptrs.argtypes = [vp, u32, vp, u32, u64, vp, u32, vp, vp]
    L.dg_m_grouped_gemm_nt_contiguous_rowptr.argtypes = [opp, opp, vp, u32, u32, vp, vp, u32, u32, vp]
    L.dg_get_gemm_config.argtypes = [i32, i32, u32, u32, u32, u32, C.POINTER(GemmConfigC)]
    _lib = L
    return L
