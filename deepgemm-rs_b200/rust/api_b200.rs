//! `deepgemm::api` for the block-scaled GEMM path, re-based on libdeepgemm_b200.so.
//!
//! Meant to replace the bodies of the hot-path functions of `deepgemm/src/api.rs` (same names, same
//! arguments, same `DgResult`): everything that used to plan tiles, build tensor maps, JIT-compile and
//! launch happens behind the C ABI now; what stays on the Rust side is the ownership model
//! (`DevBuffer` allocation for the operators that return buffers) and the error type.
//! `Device` / `DevStream` / `DevBuffer` (device.rs) are untouched and only lend their raw handles.
//! Written against the reference at the commit this build was derived from; it has not been compiled in
//! the build environment (no Rust toolchain there) -- the C ABI itself is exercised by the Python
//! binding, which marshals the same structs.
#![allow(clippy::too_many_arguments)]
use std::ffi::{c_void, CStr};

use crate::device::{DevBuffer, DevStream, Device};
use crate::error::{DgError, DgResult};
use crate::ffi_b200 as ffi;
use crate::types::{Dtype, Major, Operand, Output, SfGran, SfTensor};

fn status(code: i32) -> DgResult<()> {
    if code == ffi::DG_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(ffi::dg_last_error()) }.to_string_lossy().into_owned();
    Err(match code {
        ffi::DG_ERR_DRIVER => DgError::Driver(msg),
        ffi::DG_ERR_INVALID_ARG => DgError::InvalidArg(msg),
        ffi::DG_ERR_UNSUPPORTED => DgError::Unsupported(msg),
        ffi::DG_ERR_MISMATCH => DgError::Mismatch(msg),
        // DG_ERR_DEVICE_TIMEOUT (a bounded device-side wait gave up) has no variant of its own
        _ => DgError::Runtime(msg),
    })
}

fn dtype_code(d: Dtype) -> i32 {
    match d {
        Dtype::Fp8 => 0,
        Dtype::Fp4 => 1,
        Dtype::Bf16 => 2,
        Dtype::F32 => 3,
    }
}

fn sf(s: Option<&SfTensor>) -> ffi::DgSfTensor {
    match s {
        Some(s) => ffi::DgSfTensor { rows: s.rows, cols: s.cols, gran: s.gran.k(), data: s.buf.ptr as *const u32 },
        None => ffi::DgSfTensor { rows: 0, cols: 0, gran: 0, data: std::ptr::null() },
    }
}

fn op(o: &Operand) -> ffi::DgOperand {
    ffi::DgOperand {
        dtype: dtype_code(o.dtype),
        major: if o.major == Major::K { 0 } else { 1 },
        rows: o.rows,
        k: o.k,
        outer_stride: o.outer_stride,
        sf: sf(o.sf.as_ref()),
        data: o.data.ptr as *const c_void,
    }
}

fn out_c(o: &mut Output) -> ffi::DgOutput {
    ffi::DgOutput { dtype: dtype_code(o.dtype), rows: o.rows, cols: o.cols, stride: o.stride, data: o.data.ptr as *mut c_void }
}

fn raw(stream: &DevStream) -> *mut c_void {
    stream.raw() as *mut c_void
}

type GemmFn = unsafe extern "C" fn(*const ffi::DgOperand, *const ffi::DgOperand, *mut ffi::DgOutput, i32, *mut c_void) -> i32;

fn gemm_with(f: GemmFn, dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    dev.bind()?;
    let mut o = out_c(out);
    status(unsafe { f(&op(a), &op(b), &mut o, accumulate as i32, raw(stream)) })
}

// ---- dense GEMM ------------------------------------------------------------------------------
/// api.rs:648-657.  Operands may be K- or MN-major (api.rs:679-715), FP8 x FP4 pairs included.
pub fn gemm_nt(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    gemm_with(ffi::dg_gemm_nt, dev, stream, a, b, out, accumulate)
}
/// api.rs:762-771
pub fn fp8_gemm_nt(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    gemm_with(ffi::dg_fp8_gemm_nt, dev, stream, a, b, out, accumulate)
}
/// api.rs:829-838
pub fn fp4_gemm_nt(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    gemm_with(ffi::dg_fp4_gemm_nt, dev, stream, a, b, out, accumulate)
}
/// api.rs:841-850
pub fn bf16_gemm_nt(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    gemm_with(ffi::dg_bf16_gemm_nt, dev, stream, a, b, out, accumulate)
}
/// api.rs:663-673
pub fn gemm_nt_alpha(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool,
                     alpha: Option<f32>) -> DgResult<()> {
    dev.bind()?;
    let mut o = out_c(out);
    status(unsafe { ffi::dg_gemm_nt_alpha(&op(a), &op(b), &mut o, accumulate as i32, alpha.unwrap_or(1.0), raw(stream)) })
}
/// api.rs:679-715: the general entry is dg_gemm_nt itself.
pub fn gemm_nt_layout(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool,
                      alpha: Option<f32>) -> DgResult<()> {
    gemm_nt_alpha(dev, stream, a, b, out, accumulate, alpha)
}
/// api.rs:720-732
pub fn gemm_nn(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    gemm_with(ffi::dg_gemm_nn, dev, stream, a, b, out, accumulate)
}
/// api.rs:734-746
pub fn gemm_tn(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    gemm_with(ffi::dg_gemm_tn, dev, stream, a, b, out, accumulate)
}
/// api.rs:748-759
pub fn gemm_tt(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, accumulate: bool) -> DgResult<()> {
    gemm_with(ffi::dg_gemm_tt, dev, stream, a, b, out, accumulate)
}
/// api.rs:966-993
pub fn fp8_bmm(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, batch: u32, accumulate: bool) -> DgResult<()> {
    dev.bind()?;
    let mut o = out_c(out);
    status(unsafe { ffi::dg_fp8_bmm(&op(a), &op(b), &mut o, batch, accumulate as i32, raw(stream)) })
}

// ---- grouped GEMM ----------------------------------------------------------------------------
/// api.rs:859-903: `m_indices` holds one i32 per 128-row block.
pub fn m_grouped_gemm_nt_contiguous(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output,
                                    m_indices: &DevBuffer, num_groups: u32) -> DgResult<()> {
    dev.bind()?;
    let mut o = out_c(out);
    status(unsafe {
        ffi::dg_m_grouped_gemm_nt_contiguous(&op(a), &op(b), &mut o, m_indices.ptr as *const i32, (m_indices.len / 4) as u32, num_groups,
                                             raw(stream))
    })
}
/// api.rs:930-963
pub fn m_grouped_gemm_nt_masked(dev: &Device, stream: &DevStream, a: &Operand, b: &Operand, out: &mut Output, masked_m: &DevBuffer,
                                num_groups: u32, expected_m: u32) -> DgResult<()> {
    dev.bind()?;
    let mut o = out_c(out);
    status(unsafe {
        ffi::dg_m_grouped_gemm_nt_masked(&op(a), &op(b), &mut o, masked_m.ptr as *const i32, num_groups, expected_m, raw(stream))
    })
}

// ---- scale-factor layout and quantisation ------------------------------------------------------
/// api.rs:1031-1064: host slice in, owned packed tensor out.
pub fn transform_sf(dev: &Device, stream: &DevStream, sf: &[f32], mn: u32, gran: SfGran) -> DgResult<SfTensor> {
    if mn == 0 || sf.len() % mn as usize != 0 {
        return Err(DgError::InvalidArg("sf length must be mn * sf_k".into()));
    }
    dev.bind()?;
    let sf_k = (sf.len() / mn as usize) as u32;
    let (rows, cols) = (sf_k.div_ceil(4), mn.div_ceil(4) * 4);
    let buf = DevBuffer::alloc(dev, (rows * cols * 4) as usize)?; // every word is written: no zeroing
    status(unsafe { ffi::dg_transform_sf_host(sf.as_ptr(), mn, sf_k, buf.ptr as *mut u32, raw(stream)) })?;
    stream.sync()?; // the host slice may go away when the caller returns
    Ok(SfTensor { rows, cols, gran, buf })
}
/// api.rs:1263-1311
pub fn transform_sf_batched(dev: &Device, stream: &DevStream, sf: &[f32], batch: u32, mn: u32, gran: SfGran) -> DgResult<SfTensor> {
    if batch == 0 {
        return Err(DgError::InvalidArg("batch must be nonzero".into()));
    }
    let per_batch = (sf.len() / batch as usize) as u32;
    if per_batch == 0 || sf.len() as u32 != per_batch * batch || per_batch % mn != 0 {
        return Err(DgError::InvalidArg("batched SF must hold batch * mn * sf_k values".into()));
    }
    let sf_k = per_batch / mn;
    let (rows, cols) = (sf_k.div_ceil(4), mn.div_ceil(4) * 4);
    let staged = crate::device::alloc_and_upload(dev, sf, stream.raw())?;
    let arena = DevBuffer::alloc(dev, (rows * batch * cols * 4) as usize)?;
    status(unsafe { ffi::dg_transform_sf_batched(staged.ptr as *const f32, batch, mn, sf_k, arena.ptr as *mut u32, raw(stream)) })?;
    stream.sync()?; // `staged` is dropped on return
    Ok(SfTensor { rows: rows * batch, cols, gran, buf: arena })
}
/// api.rs:1480-1553
pub fn quant_mx(dev: &Device, stream: &DevStream, x: &[f32], m: u32, k: u32, dtype: Dtype, gran: SfGran) -> DgResult<(DevBuffer, SfTensor)> {
    if x.len() != (m as usize) * (k as usize) {
        return Err(DgError::InvalidArg("x must hold m * k values".into()));
    }
    dev.bind()?;
    let (rows, cols) = ((k / gran.k()).div_ceil(4), m.div_ceil(4) * 4);
    let bytes = if dtype == Dtype::Fp4 { (m as usize * k as usize) / 2 } else { m as usize * k as usize };
    let data = DevBuffer::alloc(dev, bytes)?;
    let sfb = DevBuffer::alloc(dev, (rows * cols * 4) as usize)?; // every word is written: no zeroing
    status(unsafe {
        ffi::dg_quant_mx_host(x.as_ptr(), m, k, dtype_code(dtype), gran.k(), data.ptr as *mut c_void, sfb.ptr as *mut u32, raw(stream))
    })?;
    stream.sync()?;
    Ok((data, SfTensor { rows, cols, gran, buf: sfb }))
}
/// api.rs:1556-1601
pub fn dequant_mx(dev: &Device, stream: &DevStream, data: &DevBuffer, sf_t: &SfTensor, m: u32, k: u32, dtype: Dtype) -> DgResult<DevBuffer> {
    dev.bind()?;
    let out = DevBuffer::alloc(dev, m as usize * k as usize * 4)?;
    let s = sf(Some(sf_t));
    status(unsafe { ffi::dg_dequant_mx(data.ptr as *const c_void, &s, m, k, dtype_code(dtype), out.ptr as *mut f32, raw(stream)) })?;
    Ok(out)
}
/// api.rs:1951-2011.  The stochastic mode draws from a hash of (element index, seed); the reference's
/// signature has no seed, 0 is passed.
pub fn quantize_output_fp8(dev: &Device, stream: &DevStream, src: &DevBuffer, m: u32, n: u32, in_stride: u32, stochastic: bool)
        -> DgResult<(DevBuffer, DevBuffer)> {
    if n % 32 != 0 {
        return Err(DgError::InvalidArg("quantize_output_fp8 needs n % 32 == 0".into()));
    }
    dev.bind()?;
    let out = DevBuffer::alloc(dev, m as usize * n as usize)?;
    let cols = m.div_ceil(4) * 4;
    let sfd = DevBuffer::alloc(dev, ((n / 32).div_ceil(4) * cols * 4) as usize)?;
    status(unsafe {
        ffi::dg_quantize_output_fp8(src.ptr as *const f32, m, n, in_stride, stochastic as i32, 0, out.ptr as *mut c_void,
                                    sfd.ptr as *mut u32, raw(stream))
    })?;
    Ok((out, sfd))
}

// ---- MQA logits --------------------------------------------------------------------------------
/// api.rs:1614-1745.  The scale factors travel inside the operands on the C side.
pub fn mqa_logits(dev: &Device, stream: &DevStream, q: &Operand, q_sf: &SfTensor, kv: &Operand, kv_sf: &SfTensor, weights: &DevBuffer,
                  cu_k_start: &DevBuffer, cu_k_end: &DevBuffer, num_tokens: u32, num_kv_tokens: u32, num_heads: u32, head_dim: u32,
                  logits: &mut DevBuffer, logits_stride: u32) -> DgResult<()> {
    dev.bind()?;
    let mut qc = op(q);
    qc.sf = sf(Some(q_sf));
    let mut kc = op(kv);
    kc.sf = sf(Some(kv_sf));
    status(unsafe {
        ffi::dg_mqa_logits(&qc, &kc, weights.ptr as *const c_void, cu_k_start.ptr as *const u32, cu_k_end.ptr as *const u32, num_tokens,
                           num_kv_tokens, num_heads, head_dim, logits.ptr as *mut c_void, logits_stride, raw(stream))
    })
}
/// api.rs:1752-1941
pub fn mqa_logits_paged(dev: &Device, stream: &DevStream, q: &Operand, q_sf: &SfTensor, kv_pages: &DevBuffer, kv_sf_pages: &DevBuffer,
                        weights: &DevBuffer, page_kv: u32, num_pages: u32, context_lens: &DevBuffer, indices: &DevBuffer,
                        block_table: &DevBuffer, block_table_stride: u32, num_tokens: u32, num_heads: u32, head_dim: u32,
                        logits: &mut DevBuffer, logits_stride: u32) -> DgResult<()> {
    dev.bind()?;
    let mut qc = op(q);
    qc.sf = sf(Some(q_sf));
    status(unsafe {
        ffi::dg_mqa_logits_paged(&qc, kv_pages.ptr as *const c_void, kv_sf_pages.ptr as *const u32, weights.ptr as *const c_void, page_kv,
                                 num_pages, context_lens.ptr as *const u32, indices.ptr as *const u32, block_table.ptr as *const u32,
                                 block_table_stride, num_tokens, num_heads, head_dim, logits.ptr as *mut c_void, logits_stride,
                                 raw(stream))
    })
}
/// The fp32-scale contract of api_sm90_mqa.rs:5-31 (raw E4M3 q, one f32 scale per kv token, f32 weights and logits).
pub fn mqa_logits_f32(dev: &Device, stream: &DevStream, q: &DevBuffer, kv: &DevBuffer, kv_scale: &DevBuffer, weights: &DevBuffer,
                      cu_k_start: &DevBuffer, cu_k_end: &DevBuffer, num_tokens: u32, num_kv_tokens: u32, num_heads: u32, head_dim: u32,
                      logits: &mut DevBuffer, logits_stride: u32) -> DgResult<()> {
    dev.bind()?;
    status(unsafe {
        ffi::dg_mqa_logits_f32(q.ptr as *const c_void, kv.ptr as *const c_void, kv_scale.ptr as *const f32, weights.ptr as *const f32,
                               cu_k_start.ptr as *const u32, cu_k_end.ptr as *const u32, num_tokens, num_kv_tokens, num_heads, head_dim,
                               logits.ptr as *mut f32, logits_stride, raw(stream))
    })
}

/// Synchronises the stream and reports a device-side wait that gave up (no counterpart: the reference's
/// device waits are unbounded).
pub fn poll_device_status(stream: &DevStream) -> DgResult<()> {
    status(unsafe { ffi::dg_poll_device_status(raw(stream)) })
}
