//! Raw bindings of libdeepgemm_b200.so (include/deepgemm_b200.h): the drop-in boundary of the
//! block-scaled GEMM path.  Meant to live in the reference crate as `deepgemm/src/ffi_b200.rs`
//! (`mod ffi_b200;` in lib.rs, `cargo:rustc-link-lib=deepgemm_b200` in build.rs); `api_b200.rs`
//! beside it keeps the signatures of `deepgemm::api` and calls through these.
//!
//! The structs are `#[repr(C)]` mirrors of dg_sf_tensor_t / dg_operand_t / dg_output_t /
//! dg_gemm_config_t.  Enum discriminants match the C enums: `Dtype::{Fp8, Fp4, Bf16, F32}` = 0..3
//! and `Major::{K, Mn}` = 0, 1 (deepgemm/src/types.rs:5-37).
#![allow(clippy::too_many_arguments)]
use std::ffi::c_void;
use std::os::raw::c_char;

#[repr(C)]
#[derive(Clone, Copy)]
pub struct DgSfTensor {
    pub rows: u32,
    pub cols: u32,
    pub gran: u32,
    pub data: *const u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct DgOperand {
    pub dtype: i32,
    pub major: i32,
    pub rows: u32,
    pub k: u32,
    pub outer_stride: u32,
    pub sf: DgSfTensor,
    pub data: *const c_void,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct DgOutput {
    pub dtype: i32,
    pub rows: u32,
    pub cols: u32,
    pub stride: u32,
    pub data: *mut c_void,
}

#[repr(C)]
#[derive(Clone, Copy, Default, Debug)]
pub struct DgGemmConfig {
    pub block_m: u32,
    pub block_n: u32,
    pub block_k: u32,
    pub num_stages: u32,
    pub smem_bytes: u32,
    pub num_tiles: u32,
    pub grid: u32,
    pub cluster: u32,
}

pub const DG_OK: i32 = 0;
pub const DG_ERR_DRIVER: i32 = 1;
pub const DG_ERR_INVALID_ARG: i32 = 3;
pub const DG_ERR_UNSUPPORTED: i32 = 4;
pub const DG_ERR_MISMATCH: i32 = 5;
pub const DG_ERR_RUNTIME: i32 = 6;
pub const DG_ERR_DEVICE_TIMEOUT: i32 = 8;

type Stream = *mut c_void;

#[link(name = "deepgemm_b200")]
extern "C" {
    // ---- library
    pub fn dg_last_error() -> *const c_char;
    pub fn dg_version() -> *const c_char;
    pub fn dg_device_check() -> i32;
    pub fn dg_poll_device_status(stream: Stream) -> i32;
    pub fn dg_launch_count() -> u64;
    pub fn dg_sf_shape(mn: u32, k: u32, gran: u32, rows: *mut u32, cols: *mut u32);

    // ---- dense GEMM (api.rs:648-850, 966-993)
    pub fn dg_gemm_nt(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_fp8_gemm_nt(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_fp4_gemm_nt(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_bf16_gemm_nt(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_gemm_nt_alpha(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, alpha: f32, stream: Stream) -> i32;
    pub fn dg_gemm_nn(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_gemm_tn(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_gemm_tt(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_bmm(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, batch: u32, accumulate: i32, stream: Stream) -> i32;
    pub fn dg_fp8_bmm(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, batch: u32, accumulate: i32, stream: Stream) -> i32;

    // ---- grouped GEMM (api.rs:859-963)
    pub fn dg_m_grouped_gemm_nt_contiguous(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, m_indices: *const i32,
                                           m_indices_len: u32, num_groups: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_gemm_nt_masked(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, masked_m: *const i32,
                                       num_groups: u32, expected_m: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_fp8_gemm_nt_contiguous(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, m_indices: *const i32,
                                               m_indices_len: u32, num_groups: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_fp4_gemm_nt_contiguous(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, m_indices: *const i32,
                                               m_indices_len: u32, num_groups: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_bf16_gemm_nt_contiguous(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, m_indices: *const i32,
                                                m_indices_len: u32, num_groups: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_fp8_gemm_nt_masked(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, masked_m: *const i32,
                                           num_groups: u32, expected_m: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_fp4_gemm_nt_masked(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, masked_m: *const i32,
                                           num_groups: u32, expected_m: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_bf16_gemm_nt_masked(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, masked_m: *const i32,
                                            num_groups: u32, expected_m: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_gemm_nt_contiguous_scatter(a: *const DgOperand, b: *const DgOperand, out: *mut DgOutput, m_indices: *const i32,
                                                   m_indices_len: u32, num_groups: u32, d_row_map: *const i32, n_begin: u32,
                                                   n_count: u32, stream: Stream) -> i32;
    pub fn dg_m_grouped_gemm_nt_contiguous_gather(a: *const DgOperand, a_row_src: *const i32, a_src_rows: u32, b: *const DgOperand,
                                                  out: *mut DgOutput, m_indices: *const i32, m_indices_len: u32, num_groups: u32,
                                                  stream: Stream) -> i32;
    pub fn dg_m_grouped_gemm_nt_contiguous_rowptr(a: *const DgOperand, b: *const DgOperand, m_indices: *const i32, m_indices_len: u32,
                                                  num_groups: u32, d_row_ptr: *const u64, m_blocks_used: *const i32, n_begin: u32,
                                                  n_count: u32, stream: Stream) -> i32;

    // ---- quantisation / scale-factor layout (api.rs:1031-1135, 1263-1311, 1480-1601, 1951-2011)
    pub fn dg_quant_mx(x: *const f32, m: u32, k: u32, dtype: i32, gran: u32, data_out: *mut c_void, sf_out: *mut u32, stream: Stream) -> i32;
    pub fn dg_quant_mx_host(x_host: *const f32, m: u32, k: u32, dtype: i32, gran: u32, data_out: *mut c_void, sf_out: *mut u32,
                            stream: Stream) -> i32;
    pub fn dg_quant_mx_host_static(x_host: *const f32, m: u32, k: u32, dtype: i32, gran: u32, data_out: *mut c_void, sf_out: *mut u32,
                                   stream: Stream) -> i32;
    pub fn dg_dequant_mx(data: *const c_void, sf: *const DgSfTensor, m: u32, k: u32, dtype: i32, out: *mut f32, stream: Stream) -> i32;
    pub fn dg_transform_sf(sf: *const f32, mn: u32, sf_k: u32, out: *mut u32, stream: Stream) -> i32;
    pub fn dg_transform_sf_host(sf_host: *const f32, mn: u32, sf_k: u32, out: *mut u32, stream: Stream) -> i32;
    pub fn dg_transform_sf_batched(sf: *const f32, batch: u32, mn: u32, sf_k: u32, out: *mut u32, stream: Stream) -> i32;
    pub fn dg_quantize_output_fp8(src: *const f32, m: u32, n: u32, in_stride: u32, stochastic: i32, seed: u32, data_out: *mut c_void,
                                  sf_out: *mut u32, stream: Stream) -> i32;
    pub fn dg_swiglu_quant(gate_up_bf16: *const c_void, pitch: u64, m: u32, inter: u32, gran: u32, data_out: *mut c_void,
                           sf_out: *mut u32, stream: Stream) -> i32;

    // ---- MQA logits (api.rs:1614-1941; fp32 contract api_sm90_mqa.rs:5-31)
    pub fn dg_mqa_logits_f32(q: *const c_void, kv: *const c_void, kv_scale: *const f32, weights: *const f32, cu_k_start: *const u32,
                             cu_k_end: *const u32, num_tokens: u32, num_kv_tokens: u32, num_heads: u32, head_dim: u32,
                             logits: *mut f32, logits_stride: u32, stream: Stream) -> i32;
    pub fn dg_mqa_logits(q: *const DgOperand, kv: *const DgOperand, weights_bf16: *const c_void, cu_k_start: *const u32,
                         cu_k_end: *const u32, num_tokens: u32, num_kv_tokens: u32, num_heads: u32, head_dim: u32,
                         logits_bf16: *mut c_void, logits_stride: u32, stream: Stream) -> i32;
    pub fn dg_mqa_logits_paged(q: *const DgOperand, kv_pages: *const c_void, kv_sf_pages: *const u32, weights_bf16: *const c_void,
                               page_kv: u32, num_pages: u32, context_lens: *const u32, indices: *const u32, block_table: *const u32,
                               block_table_stride: u32, num_tokens: u32, num_heads: u32, head_dim: u32, logits_bf16: *mut c_void,
                               logits_stride: u32, stream: Stream) -> i32;

    // ---- MoE row movement and expert parallelism (no counterpart in the reference)
    pub fn dg_gather_rows(src: *const c_void, src_pitch_bytes: u64, idx: *const i32, dst: *mut c_void, dst_pitch_bytes: u64,
                          n_rows: u32, row_bytes: u32, stream: Stream) -> i32;
    pub fn dg_gather_sf(src: *const u32, src_row_stride: u64, src_col_stride: u64, idx: *const i32, dst: *mut u32,
                        dst_row_stride: u64, dst_col_stride: u64, sf_rows: u32, n: u32, stream: Stream) -> i32;
    pub fn dg_moe_plan(expert_of_row: *const i32, n_rows: u32, num_experts: u32, align: u32, div: u32, capacity: u32,
                       counts: *mut i32, offsets: *mut i32, cursors: *mut i32, slot_src: *mut i32, slot_of_row: *mut i32,
                       block_expert: *mut i32, stream: Stream) -> i32;
    pub fn dg_moe_combine(src_bf16: *const c_void, src_pitch: u64, pos: *const i32, weights: *const f32, out_bf16: *mut c_void,
                          out_pitch: u64, tokens: u32, topk: u32, cols: u32, stream: Stream) -> i32;
    pub fn dg_peer_alloc(bytes: u64, ptr: *mut *mut c_void) -> i32;
    pub fn dg_peer_free(ptr: *mut c_void) -> i32;
    pub fn dg_peer_export(ptr: *const c_void, handle64: *mut c_void) -> i32;
    pub fn dg_peer_open(handle64: *const c_void, ptr: *mut *mut c_void) -> i32;
    pub fn dg_peer_close(ptr: *mut c_void) -> i32;
    pub fn dg_peer_copy(dst: *mut c_void, src: *const c_void, bytes: u64, stream: Stream) -> i32;
    pub fn dg_peer_barrier(peer_flags: *const u64, local_flags: *mut u64, me: u32, world: u32, seq: u64, stream: Stream) -> i32;
    pub fn dg_moe_return_ptrs(slot_src: *const i32, slots: u32, seg_start: *const i32, dst_base: *const u64, dst_row0: *const i32,
                              world: u32, row_bytes: u64, ptrs: *mut u64, stream: Stream) -> i32;
    pub fn dg_ep_route(counts: *const i32, world: u32, me: u32, num_experts: u32, align: u32, cap: u32, slices: u32,
                       slice_first: *const u32, dest_base: *mut i32, block_expert: *mut i32, blocks_used: *mut i32,
                       stream: Stream) -> i32;
    pub fn dg_ep_push(x: *const c_void, x_pitch_bytes: u64, row_bytes: u32, x_sf: *const u32, sf_rows: u32, sf_cols: u64,
                      slot_src: *const i32, my_offsets: *const i32, dest_base: *const i32, num_experts: u32, world: u32, me: u32,
                      e_lo: u32, e_hi: u32, n_copies: u32, cap: u64, a_bases: *const u64, sf_bases: *const u64,
                      ticket_bases: *const u64, max_blocks: u32, stream: Stream) -> i32;
    pub fn dg_ep_return_ptrs(tickets: *mut u64, slots: u32, ret_bases: *const u64, world: u32, row_bytes: u64,
                             block_expert: *const i32, align: u32, ptrs: *mut u64, stream: Stream) -> i32;

    // ---- introspection (heuristics.rs:559-608)
    pub fn dg_get_gemm_config(dtype: i32, kind: i32, m: u32, n: u32, k: u32, num_groups: u32, cfg: *mut DgGemmConfig) -> i32;
}
