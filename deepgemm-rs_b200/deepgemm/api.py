"""Operator API with the names and argument meaning of the reference's `deepgemm::api`
(deepgemm/src/api.rs), bound to the C ABI of libdeepgemm_b200.so.

torch is used for device memory and streams only.  `dev` / `stream` of the reference
signatures collapse into an optional `stream` (a torch.cuda.Stream or None = current stream).
Errors surface as the DgError subclasses of .types.  There is no CPU path: without the
library or without an sm_100 GPU every operator raises.
"""
import ctypes as C

import torch

from . import _lib
from .types import Dtype, Major, Operand, Output, SfGran, SfTensor, error_for


def _stream_ptr(stream):
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream)


def _check(code):
    if code != 0:
        raise error_for(code, _lib.load().dg_last_error().decode())


def _sf_c(sf):
    if sf is None:
        return _lib.SfTensorC(0, 0, 0, None)
    return _lib.SfTensorC(sf.rows, sf.cols, int(sf.gran), sf.buf.data_ptr())


def _op_c(op):
    """C view of an Operand, cached on the object while its fields are unchanged (building the
    ctypes structures costs more host time than a small GEMM takes on the GPU)."""
    sf = op.sf
    key = (int(op.dtype), int(op.major), op.rows, op.k, op.outer_stride, op.data.data_ptr(),
           None if sf is None else (sf.rows, sf.cols, int(sf.gran), sf.buf.data_ptr()))
    cached = op.__dict__.get("_c")
    if cached is not None and cached[0] == key:
        return cached[1]
    c = _lib.OperandC(key[0], key[1], op.rows, op.k, op.outer_stride, _sf_c(sf), key[5])
    op.__dict__["_c"] = (key, c)
    return c


def _out_c(out):
    key = (int(out.dtype), out.rows, out.cols, out.stride, out.data.data_ptr())
    cached = out.__dict__.get("_c")
    if cached is not None and cached[0] == key:
        return cached[1]
    c = _lib.OutputC(*key)
    out.__dict__["_c"] = (key, c)
    return c


def device_check():
    _check(_lib.load().dg_device_check())


def poll_device_status(stream=None):
    """Synchronises the stream and raises DeviceTimeout if a kernel gave up on a wait."""
    _check(_lib.load().dg_poll_device_status(_stream_ptr(stream)))


def sf_shape(mn, k, gran):
    r, c = C.c_uint32(), C.c_uint32()
    _lib.load().dg_sf_shape(mn, k, int(gran), C.byref(r), C.byref(c))
    return r.value, c.value


# ---- dense GEMM (api.rs:648-657, 762-771, 829-850) -------------------------------------
def _gemm(fn, a, b, out, accumulate, stream):
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(fn(C.byref(ac), C.byref(bc), C.byref(oc), 1 if accumulate else 0, _stream_ptr(stream)))


def gemm_nt(a, b, out, accumulate=False, stream=None):
    _gemm(_lib.load().dg_gemm_nt, a, b, out, accumulate, stream)


def fp8_gemm_nt(a, b, out, accumulate=False, stream=None):
    _gemm(_lib.load().dg_fp8_gemm_nt, a, b, out, accumulate, stream)


def fp4_gemm_nt(a, b, out, accumulate=False, stream=None):
    _gemm(_lib.load().dg_fp4_gemm_nt, a, b, out, accumulate, stream)


def bf16_gemm_nt(a, b, out, accumulate=False, stream=None):
    _gemm(_lib.load().dg_bf16_gemm_nt, a, b, out, accumulate, stream)


def gemm_nt_alpha(a, b, out, accumulate=False, alpha=None, stream=None):
    """D = alpha * (A . B^T) (+ D) (api.rs:663-673); alpha None = 1."""
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(_lib.load().dg_gemm_nt_alpha(C.byref(ac), C.byref(bc), C.byref(oc), 1 if accumulate else 0,
                                        C.c_float(1.0 if alpha is None else alpha), _stream_ptr(stream)))


def gemm_nn(a, b, out, accumulate=False, stream=None):
    """A K-major [M, K], B an MN-major view of a [K, N] buffer (api.rs:720-732)."""
    _gemm(_lib.load().dg_gemm_nn, a, b, out, accumulate, stream)


def gemm_tn(a, b, out, accumulate=False, stream=None):
    """A an MN-major view of a [K, M] buffer, B K-major [N, K] (api.rs:734-746)."""
    _gemm(_lib.load().dg_gemm_tn, a, b, out, accumulate, stream)


def gemm_tt(a, b, out, accumulate=False, stream=None):
    """A and B MN-major views (api.rs:748-759)."""
    _gemm(_lib.load().dg_gemm_tt, a, b, out, accumulate, stream)


def fp8_bmm(a, b, out, batch, accumulate=False, stream=None):
    """Batched GEMM (api.rs:966-993): a / b / out describe one batch, the tensors hold `batch` of them stacked
    along the rows, the scale factors are transform_sf_batched arenas."""
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(_lib.load().dg_fp8_bmm(C.byref(ac), C.byref(bc), C.byref(oc), batch, 1 if accumulate else 0, _stream_ptr(stream)))


def bmm(a, b, out, batch, accumulate=False, stream=None):
    """fp8_bmm for any operand dtype."""
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(_lib.load().dg_bmm(C.byref(ac), C.byref(bc), C.byref(oc), batch, 1 if accumulate else 0, _stream_ptr(stream)))


# ---- grouped GEMM (api.rs:859-963) -----------------------------------------------------
def _contig(fn, a, b, out, m_indices, num_groups, stream):
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(fn(C.byref(ac), C.byref(bc), C.byref(oc), m_indices.data_ptr(), m_indices.numel(), num_groups,
              _stream_ptr(stream)))


def _masked(fn, a, b, out, masked_m, num_groups, expected_m, stream):
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(fn(C.byref(ac), C.byref(bc), C.byref(oc), masked_m.data_ptr(), num_groups, expected_m, _stream_ptr(stream)))


def m_grouped_gemm_nt_contiguous(a, b, out, m_indices, num_groups, stream=None):
    _contig(_lib.load().dg_m_grouped_gemm_nt_contiguous, a, b, out, m_indices, num_groups, stream)


def m_grouped_gemm_nt_contiguous_scatter(a, b, out, m_indices, num_groups, d_row_map, n_begin=0, n_count=0, stream=None):
    """Extension: row r of the result is stored at row d_row_map[r] of `out` (negative = dropped);
    only the output columns [n_begin, n_begin + n_count) of every expert are computed (0 = all)."""
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(_lib.load().dg_m_grouped_gemm_nt_contiguous_scatter(C.byref(ac), C.byref(bc), C.byref(oc), m_indices.data_ptr(),
                                                               m_indices.numel(), num_groups, d_row_map.data_ptr(),
                                                               n_begin, n_count, _stream_ptr(stream)))


def m_grouped_gemm_nt_contiguous_gather(a, a_row_src, a_src_rows, b, out, m_indices, num_groups, stream=None):
    """Extension: `a.data` holds `a_src_rows` un-permuted FP8 rows; row r of the grouped matrix (a.rows rows, never
    written out) is row a_row_src[r] of it (int32 device tensor, negative = padding).  a.sf is in the grouped order."""
    ac, bc, oc = _op_c(a), _op_c(b), _out_c(out)
    _check(_lib.load().dg_m_grouped_gemm_nt_contiguous_gather(C.byref(ac), a_row_src.data_ptr(), a_src_rows, C.byref(bc), C.byref(oc),
                                                              m_indices.data_ptr(), m_indices.numel(), num_groups,
                                                              _stream_ptr(stream)))


def m_grouped_gemm_nt_contiguous_rowptr(a, b, m_indices, num_groups, d_row_ptr, n_begin=0, n_count=0, stream=None,
                                        m_blocks_used=None):
    """Extension: BF16 result row r is stored at the address d_row_ptr[r] (int64 device tensor of
    a.rows addresses in this GPU's memory or a mapped peer's; 0 = dropped).  m_blocks_used: optional
    int32 device scalar, only that many leading entries of m_indices are visited."""
    ac, bc = _op_c(a), _op_c(b)
    _check(_lib.load().dg_m_grouped_gemm_nt_contiguous_rowptr(C.byref(ac), C.byref(bc), m_indices.data_ptr(), m_indices.numel(),
                                                              num_groups, d_row_ptr.data_ptr(),
                                                              None if m_blocks_used is None else m_blocks_used.data_ptr(),
                                                              n_begin, n_count, _stream_ptr(stream)))


def m_grouped_gemm_nt_masked(a, b, out, masked_m, num_groups, expected_m, stream=None):
    _masked(_lib.load().dg_m_grouped_gemm_nt_masked, a, b, out, masked_m, num_groups, expected_m, stream)


def m_grouped_fp8_gemm_nt_contiguous(a, b, out, m_indices, num_groups, stream=None):
    _contig(_lib.load().dg_m_grouped_fp8_gemm_nt_contiguous, a, b, out, m_indices, num_groups, stream)


def m_grouped_fp4_gemm_nt_contiguous(a, b, out, m_indices, num_groups, stream=None):
    _contig(_lib.load().dg_m_grouped_fp4_gemm_nt_contiguous, a, b, out, m_indices, num_groups, stream)


def m_grouped_bf16_gemm_nt_contiguous(a, b, out, m_indices, num_groups, stream=None):
    _contig(_lib.load().dg_m_grouped_bf16_gemm_nt_contiguous, a, b, out, m_indices, num_groups, stream)


def m_grouped_fp8_gemm_nt_masked(a, b, out, masked_m, num_groups, expected_m, stream=None):
    _masked(_lib.load().dg_m_grouped_fp8_gemm_nt_masked, a, b, out, masked_m, num_groups, expected_m, stream)


def m_grouped_fp4_gemm_nt_masked(a, b, out, masked_m, num_groups, expected_m, stream=None):
    _masked(_lib.load().dg_m_grouped_fp4_gemm_nt_masked, a, b, out, masked_m, num_groups, expected_m, stream)


def m_grouped_bf16_gemm_nt_masked(a, b, out, masked_m, num_groups, expected_m, stream=None):
    _masked(_lib.load().dg_m_grouped_bf16_gemm_nt_masked, a, b, out, masked_m, num_groups, expected_m, stream)


# ---- quantisation (api.rs:1480-1601) ---------------------------------------------------
def quant_mx(x, m, k, dtype, gran, stream=None):
    """x: f32 [m, k], a device tensor or a host tensor/ndarray (the reference takes a host
    slice, api.rs:1480-1488).  Returns (codes u8 device tensor, SfTensor)."""
    L = _lib.load()
    gran = SfGran(int(gran))
    host = not (isinstance(x, torch.Tensor) and x.is_cuda)
    if host:
        x = torch.as_tensor(x, dtype=torch.float32).contiguous()
    if x.numel() != m * k:
        raise error_for(3, "x must be [m, k] row-major")
    dev = torch.device("cuda", torch.cuda.current_device())
    rows, cols = sf_shape(m, k, gran)
    data = torch.empty((m, k // 2 if dtype == Dtype.Fp4 else k), dtype=torch.uint8, device=dev)
    sf = torch.empty((rows, cols), dtype=torch.int32, device=dev)
    fn = L.dg_quant_mx_host if host else L.dg_quant_mx
    _check(fn(x.data_ptr(), m, k, int(dtype), int(gran), data.data_ptr(), sf.data_ptr(), _stream_ptr(stream)))
    if host:
        torch.cuda.current_stream().synchronize() if stream is None else stream.synchronize()
    return data, SfTensor(rows, cols, gran, sf)


def swiglu_quant(gate_up, m, inter, gran, stream=None):
    """gate_up: bf16 device tensor [m, >= 2 * inter] (gate half, up half), the output of an MoE gate/up
    projection.  Returns (E4M3 codes u8 [m, inter] of silu(gate) * up, their packed SfTensor): the A
    operand of the down projection (the step deepgemm/src/api_serving.rs:371-375 leaves to the caller)."""
    gran = SfGran(int(gran))
    rows, cols = sf_shape(m, inter, gran)
    data = torch.empty((m, inter), dtype=torch.uint8, device=gate_up.device)
    sf = torch.empty((rows, cols), dtype=torch.int32, device=gate_up.device)
    _check(_lib.load().dg_swiglu_quant(gate_up.data_ptr(), gate_up.stride(0), m, inter, int(gran), data.data_ptr(), sf.data_ptr(),
                                       _stream_ptr(stream)))
    return data, SfTensor(rows, cols, gran, sf)


def dequant_mx(data, sf, m, k, dtype, stream=None):
    out = torch.empty((m, k), dtype=torch.float32, device=data.device)
    sc = _sf_c(sf)
    _check(_lib.load().dg_dequant_mx(data.data_ptr(), C.byref(sc), m, k, int(dtype), out.data_ptr(), _stream_ptr(stream)))
    return out


def transform_sf(sf, mn, gran, stream=None):
    """sf: f32 [mn, sf_k] powers of two, device tensor or host tensor/ndarray (api.rs:1031-1037).
    Returns the packed SfTensor."""
    L = _lib.load()
    host = not (isinstance(sf, torch.Tensor) and sf.is_cuda)
    if host:
        sf = torch.as_tensor(sf, dtype=torch.float32).contiguous()
    if mn == 0 or sf.numel() % mn != 0:
        raise error_for(3, "sf length must be mn * sf_k")
    sf_k = sf.numel() // mn
    dev = torch.device("cuda", torch.cuda.current_device())
    rows, cols = (sf_k + 3) // 4, (mn + 3) // 4 * 4
    out = torch.empty((rows, cols), dtype=torch.int32, device=dev)
    fn = L.dg_transform_sf_host if host else L.dg_transform_sf
    _check(fn(sf.data_ptr(), mn, sf_k, out.data_ptr(), _stream_ptr(stream)))
    if host:
        torch.cuda.current_stream().synchronize() if stream is None else stream.synchronize()
    return SfTensor(rows, cols, SfGran(int(gran)), out)


def transform_sf_batched(sf, batch, mn, gran, stream=None):
    """sf: f32 [batch, mn, sf_k] powers of two (device or host, api.rs:1263-1270).  Returns the arena SfTensor
    [batch * ceil(sf_k/4), align4(mn)]."""
    if not (isinstance(sf, torch.Tensor) and sf.is_cuda):
        sf = torch.as_tensor(sf, dtype=torch.float32).contiguous().cuda()
    if batch == 0:
        raise error_for(3, "batch must be nonzero")
    per_batch = sf.numel() // batch
    if per_batch == 0 or per_batch * batch != sf.numel() or per_batch % mn != 0:
        raise error_for(3, "batched SF must hold batch * mn * sf_k values")
    sf_k = per_batch // mn
    rows, cols = (sf_k + 3) // 4, (mn + 3) // 4 * 4
    out = torch.empty((batch * rows, cols), dtype=torch.int32, device=sf.device)
    _check(_lib.load().dg_transform_sf_batched(sf.data_ptr(), batch, mn, sf_k, out.data_ptr(), _stream_ptr(stream)))
    return SfTensor(batch * rows, cols, SfGran(int(gran)), out)


def quantize_output_fp8(src, m, n, in_stride, stochastic=False, seed=0, stream=None):
    """src: f32 device tensor [m, >= n] with row pitch in_stride (api.rs:1951-1959).  Returns (E4M3 codes
    u8 [m, n], packed UE8M0 words i32 [ceil(n/32/4), align4(m)])."""
    rows, cols = sf_shape(m, n, 32)
    data = torch.empty((m, n), dtype=torch.uint8, device=src.device)
    sf = torch.empty((rows, cols), dtype=torch.int32, device=src.device)
    _check(_lib.load().dg_quantize_output_fp8(src.data_ptr(), m, n, in_stride, 1 if stochastic else 0, seed, data.data_ptr(),
                                              sf.data_ptr(), _stream_ptr(stream)))
    return data, sf


# ---- MQA logits ------------------------------------------------------------------------
def mqa_logits_f32(q, kv, kv_scale, weights, cu_k_start, cu_k_end, num_tokens, num_kv_tokens, num_heads, head_dim,
                   logits, logits_stride, stream=None):
    _check(_lib.load().dg_mqa_logits_f32(q.data_ptr(), kv.data_ptr(), kv_scale.data_ptr(), weights.data_ptr(),
                                         cu_k_start.data_ptr(), cu_k_end.data_ptr(), num_tokens, num_kv_tokens,
                                         num_heads, head_dim, logits.data_ptr(), logits_stride, _stream_ptr(stream)))


def mqa_logits(q, kv, weights, cu_k_start, cu_k_end, num_tokens, num_kv_tokens, num_heads, head_dim, logits,
               logits_stride, stream=None):
    qc, kc = _op_c(q), _op_c(kv)
    _check(_lib.load().dg_mqa_logits(C.byref(qc), C.byref(kc), weights.data_ptr(), cu_k_start.data_ptr(),
                                     cu_k_end.data_ptr(), num_tokens, num_kv_tokens, num_heads, head_dim,
                                     logits.data_ptr(), logits_stride, _stream_ptr(stream)))


def mqa_logits_paged(q, kv_pages, kv_sf_pages, weights, page_kv, num_pages, context_lens, indices, block_table,
                     block_table_stride, num_tokens, num_heads, head_dim, logits, logits_stride, stream=None):
    """Paged-KV mqa_logits for decode (api.rs:1752-1775): q Operand with its scale factors, kv_pages
    [num_pages, page_kv, head_dim] codes, kv_sf_pages [num_pages, page_kv] int32, weights bf16 [T, H],
    context_lens / indices int32 [T], block_table int32 [T, block_table_stride], logits bf16."""
    qc = _op_c(q)
    _check(_lib.load().dg_mqa_logits_paged(C.byref(qc), kv_pages.data_ptr(), kv_sf_pages.data_ptr(), weights.data_ptr(), page_kv,
                                           num_pages, context_lens.data_ptr(), indices.data_ptr(), block_table.data_ptr(),
                                           block_table_stride, num_tokens, num_heads, head_dim, logits.data_ptr(), logits_stride,
                                           _stream_ptr(stream)))


def get_gemm_config(dtype, kind, m, n, k, num_groups=1):
    cfg = _lib.GemmConfigC()
    _check(_lib.load().dg_get_gemm_config(int(dtype), kind, m, n, k, num_groups, C.byref(cfg)))
    return {f: getattr(cfg, f) for f, _ in cfg._fields_}
