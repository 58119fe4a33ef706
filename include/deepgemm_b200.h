/*
 * deepgemm_b200 -- C ABI of the B200 (sm_100a) block-scaled GEMM path.
 *
 * One entry point per operator of the reference crate's `deepgemm::api` hot path
 * (re-exported by deepgemm/src/lib.rs:55-61).  Every function
 *   - takes plain pointers and sizes (device pointers unless the name ends in `_host`),
 *   - enqueues on the caller's stream (`stream` is a cudaStream_t / CUstream; NULL = default
 *     stream) and returns without synchronising, like the reference
 *     (docs/PRODUCTION.md:84-86),
 *   - validates its arguments and returns a status instead of aborting
 *     (docs/PRODUCTION.md:103-107); the message is available from dg_last_error().
 * There is no CPU fallback: without an sm_100 device every compute entry returns
 * DG_ERR_UNSUPPORTED (deepgemm/src/api.rs:168-173).
 */
#ifndef DEEPGEMM_B200_H
#define DEEPGEMM_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define DG_API __attribute__((visibility("default")))
#else
#define DG_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; the names follow the reference's DgError variants (deepgemm/src/error.rs:6-15).
 * DG_ERR_DEVICE_TIMEOUT is new: a bounded device-side wait gave up (the reference's waits are
 * unbounded, deepgemm/kernels/prelude.h:252-262). */
typedef enum dg_status {
    DG_OK = 0,
    DG_ERR_DRIVER = 1,
    DG_ERR_NVRTC = 2,        /* never returned: kernels are compiled ahead of time */
    DG_ERR_INVALID_ARG = 3,
    DG_ERR_UNSUPPORTED = 4,
    DG_ERR_MISMATCH = 5,
    DG_ERR_RUNTIME = 6,
    DG_ERR_IO = 7,           /* never returned: nothing is read from or written to disk */
    DG_ERR_DEVICE_TIMEOUT = 8
} dg_status_t;

/* deepgemm/src/types.rs:5-11 (Dtype), :33-37 (Major), :55-68 (SfGran). */
typedef enum dg_dtype { DG_FP8 = 0, DG_FP4 = 1, DG_BF16 = 2, DG_F32 = 3 } dg_dtype_t;
typedef enum dg_major { DG_MAJOR_K = 0, DG_MAJOR_MN = 1 } dg_major_t;

/* Packed UE8M0 scale factors, deepgemm/src/types.rs:87-96: u32 [rows = ceil(K/(gran*4)),
 * cols = align4(MN)], MN contiguous; byte j of word [r][m] scales k-group 4r+j of row m. */
typedef struct dg_sf_tensor {
    uint32_t rows;
    uint32_t cols;
    uint32_t gran;            /* 32 or 128 */
    const uint32_t* data;     /* device */
} dg_sf_tensor_t;

/* deepgemm/src/types.rs:98-111 (Operand).  K-major [rows, k]: element (r, k) at
 * r * outer_stride + k; FP4 counts logical elements (the buffer holds k/2 bytes per row,
 * even k in the low nibble). `sf.data == NULL` means "no scale factors" (Option::None). */
typedef struct dg_operand {
    int32_t dtype;            /* dg_dtype_t */
    int32_t major;            /* dg_major_t */
    uint32_t rows;
    uint32_t k;
    uint32_t outer_stride;    /* elements */
    dg_sf_tensor_t sf;
    const void* data;         /* device */
} dg_operand_t;

/* deepgemm/src/types.rs:113-121 (Output): row-major [rows, cols], BF16 or F32. */
typedef struct dg_output {
    int32_t dtype;            /* DG_BF16 or DG_F32 */
    uint32_t rows;
    uint32_t cols;
    uint32_t stride;          /* elements */
    void* data;               /* device */
} dg_output_t;

/* ---- library ------------------------------------------------------------------------ */
DG_API const char* dg_last_error(void);          /* thread-local message of the last failing call */
DG_API const char* dg_version(void);
/* Returns DG_OK when the current device is sm_100 and the kernels can be launched there
 * (replaces the arch gate of deepgemm/src/api.rs:168-173). */
DG_API int32_t dg_device_check(void);
/* Synchronises `stream`, then reports DG_ERR_DEVICE_TIMEOUT if any kernel launched by this
 * library on the current device gave up on a wait since the last call, and clears the flag. */
DG_API int32_t dg_poll_device_status(void* stream);

/* Number of kernels this library has launched in this process (all devices, all threads). */
DG_API unsigned long long dg_launch_count(void);

/* Shape of the packed SF tensor of an [mn, k] operand: rows = ceil(k/(gran*4)),
 * cols = align4(mn) (deepgemm/src/heuristics.rs:617-624, deepgemm/src/golden.rs:71-73). */
DG_API void dg_sf_shape(uint32_t mn, uint32_t k, uint32_t gran, uint32_t* rows, uint32_t* cols);

/* ---- dense GEMM: D[M,N] (+)= A[M,K] . B[N,K]^T ---------------------------------------
 * replaces api::gemm_nt / fp8_gemm_nt / fp4_gemm_nt / bf16_gemm_nt
 * (deepgemm/src/api.rs:648-657, 762-771, 829-838, 841-850). */
DG_API int32_t dg_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream);
DG_API int32_t dg_fp8_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream);
DG_API int32_t dg_fp4_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream);
DG_API int32_t dg_bf16_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream);
/* Operands may individually be K-major or MN-major (dg_operand_t.major; the general entry
 * api::gemm_nt_layout, deepgemm/src/api.rs:679-715, which dg_gemm_nt implements).  An MN-major operand
 * is a [K, rows] buffer: element (r, k) at r + k * outer_stride (deepgemm/src/types.rs:128-137); FP8 and
 * BF16 only -- FP4 operands must be K-major (api.rs:176-180).  The scale-factor layout does not depend
 * on the major.  FP8 x FP4 and FP4 x FP8 operand pairs are accepted (the FP4 side is unpacked to one
 * code per byte on its way into shared memory, api.rs:264-265).
 * replaces api::gemm_nt_alpha (api.rs:663-673): D = alpha * (A . B^T) (+ D); alpha scales the f32
 * accumulator before the output cast, the accumulated D is not scaled. */
DG_API int32_t dg_gemm_nt_alpha(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate,
                                float alpha, void* stream);
/* replace api::gemm_nn / gemm_tn / gemm_tt (api.rs:720-759): the BLAS layouts over zero-copy MN-major
 * views.  nn: B is MN-major ([K, N] buffer); tn: A is MN-major ([K, M] buffer); tt: both.  They check
 * the orientation of the views and run dg_gemm_nt. */
DG_API int32_t dg_gemm_nn(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream);
DG_API int32_t dg_gemm_tn(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream);
DG_API int32_t dg_gemm_tt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream);
/* replaces api::fp8_bmm (api.rs:966-993): `batch` independent GEMMs.  a, b and out describe ONE batch
 * (rows = M / N, out.rows = M); the buffers hold the batches stacked along the rows ([batch * M, K],
 * [batch * N, K], [batch * M, N]; MN-major operands: [batch * K, rows]) and the scale-factor tensors are
 * the arenas of dg_transform_sf_batched: [batch * ceil(K/(4 gran)), align4(rows)], batch b's word rows
 * starting at b * ceil(K/(4 gran)).  dg_bmm takes any operand dtype, dg_fp8_bmm insists on FP8. */
DG_API int32_t dg_bmm(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, uint32_t batch, int32_t accumulate, void* stream);
DG_API int32_t dg_fp8_bmm(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, uint32_t batch, int32_t accumulate, void* stream);

/* ---- grouped GEMM (MoE) ----------------------------------------------------------------
 * replaces api::m_grouped_gemm_nt_contiguous (deepgemm/src/api.rs:859-903).  a.rows must be
 * a multiple of 128; m_indices (device, int32, a.rows/128 entries) holds the expert of each
 * 128-row block, negative = skip the block; b is the stacked [num_groups * b.rows, K] weight
 * whose SF tensor is that of the stacked matrix (deepgemm/tests/e2e_gpu.rs:421). */
DG_API int32_t dg_m_grouped_gemm_nt_contiguous(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                        const int32_t* m_indices, uint32_t m_indices_len,
                                        uint32_t num_groups, void* stream);
/* Extension (no counterpart in the reference): the contiguous grouped GEMM whose epilogue stores
 * row r of the result at row d_row_map[r] of `out` (device, int32, a.rows entries; negative = the
 * row is not stored) and which computes only the output columns [n_begin, n_begin + n_count) of every
 * expert (n_count = 0: all; out.cols = the number of computed columns, n_begin a multiple of 4).
 * out.rows is the number of destination rows and every valid map entry must be below it.  Lets an
 * expert-parallel layer write expert outputs straight into its return buffer, one column slice at a
 * time so that the slices' return transfers overlap the remaining GEMM. */
DG_API int32_t dg_m_grouped_gemm_nt_contiguous_scatter(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                                       const int32_t* m_indices, uint32_t m_indices_len,
                                                       uint32_t num_groups, const int32_t* d_row_map,
                                                       uint32_t n_begin, uint32_t n_count, void* stream);
/* Extension (no counterpart in the reference): the contiguous grouped GEMM that gathers the rows of A itself.
 * a.data holds a_src_rows un-permuted rows (K-major FP8, pitch a.outer_stride); a.rows is the row count M of the
 * grouped matrix (a multiple of 128) that is never written out: its row r is row a_row_src[r] of a.data (device,
 * int32, M entries, 16-byte aligned; negative = padding row, whose result is unspecified).  a.sf holds the scale
 * factors in the grouped order, as for dg_m_grouped_gemm_nt_contiguous.  The producer warp fetches four rows per
 * TMA instruction (tile::gather4), so a MoE layer needs no permuted copy of its tokens (the caller of
 * Serving::moe_grouped_layer, deepgemm/src/api_serving.rs:308-370, builds one).  It trades time for that memory:
 * a k-block needs 32 such instructions, which the producer warp issues more slowly than the tensor core consumes
 * the tile (about a third of the throughput of dg_m_grouped_gemm_nt_contiguous on 16384 tokens x top-8). */
DG_API int32_t dg_m_grouped_gemm_nt_contiguous_gather(const dg_operand_t* a, const int32_t* a_row_src, uint32_t a_src_rows,
                                                      const dg_operand_t* b, dg_output_t* out, const int32_t* m_indices,
                                                      uint32_t m_indices_len, uint32_t num_groups, void* stream);
/* replaces api::m_grouped_gemm_nt_masked (deepgemm/src/api.rs:930-963).  a, b and out are
 * stacked per group ([num_groups * rows, ...]); masked_m (device, int32, num_groups entries)
 * holds the valid rows of each group; rows beyond it are neither computed nor written.
 * expected_m only steers the tile choice. */
DG_API int32_t dg_m_grouped_gemm_nt_masked(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                    const int32_t* masked_m, uint32_t num_groups, uint32_t expected_m,
                                    void* stream);
/* dtype-named spellings of the two grouped entries (deepgemm/src/api.rs:907, README.md:26-27);
 * they additionally check the operand dtype. */
DG_API int32_t dg_m_grouped_fp8_gemm_nt_contiguous(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                            const int32_t* m_indices, uint32_t m_indices_len,
                                            uint32_t num_groups, void* stream);
DG_API int32_t dg_m_grouped_fp4_gemm_nt_contiguous(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                            const int32_t* m_indices, uint32_t m_indices_len,
                                            uint32_t num_groups, void* stream);
DG_API int32_t dg_m_grouped_bf16_gemm_nt_contiguous(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                             const int32_t* m_indices, uint32_t m_indices_len,
                                             uint32_t num_groups, void* stream);
DG_API int32_t dg_m_grouped_fp8_gemm_nt_masked(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                        const int32_t* masked_m, uint32_t num_groups, uint32_t expected_m,
                                        void* stream);
DG_API int32_t dg_m_grouped_fp4_gemm_nt_masked(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                        const int32_t* masked_m, uint32_t num_groups, uint32_t expected_m,
                                        void* stream);
DG_API int32_t dg_m_grouped_bf16_gemm_nt_masked(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                         const int32_t* masked_m, uint32_t num_groups, uint32_t expected_m,
                                         void* stream);

/* ---- quantisation / scale-factor layout ------------------------------------------------
 * replaces api::quant_mx (deepgemm/src/api.rs:1480-1553): x f32 [m,k] -> codes (E4M3 [m,k]
 * bytes, or packed E2M1 [m,k/2] bytes) + packed UE8M0 SF words [ceil(k/gran/4), align4(m)].
 * Every output word is written (padding columns and missing k bytes are zero), so the
 * outputs need not be cleared.  FP4 requires gran 32.  The reference takes a host slice and
 * returns owned device buffers; here the caller owns the buffers.  `_host` takes x in host
 * memory and copies it to the device on `stream` first. */
DG_API int32_t dg_quant_mx(const float* x, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran,
                    void* data_out, uint32_t* sf_out, void* stream);
DG_API int32_t dg_quant_mx_host(const float* x_host, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran,
                         void* data_out, uint32_t* sf_out, void* stream);
/* No counterpart in the reference.  Same result as dg_quant_mx_host, for callers that must not
 * allocate device memory while they run: code inside a region where cudaMalloc / cudaMallocAsync is
 * forbidden or would stall (a latency-critical serving loop, a process whose memory is entirely
 * handed to another allocator, a plugin host that audits allocations).  The host tensor is staged
 * in a 16 MiB array built into the library image (held by every GPU that loads the library, until
 * exit), so m * k * 4 bytes must not exceed 16 MiB; larger inputs are rejected with
 * DG_ERR_INVALID_ARG.  The call makes no cudaMalloc / cudaFree / pool allocation.  Its first call
 * on a device looks up the array's device address once: make that first call outside any stream
 * capture.  All calls share the one staging array and it keeps the previous call's contents (each
 * call overwrites exactly the bytes it then reads, nothing needs clearing): calls whose work can
 * overlap on the GPU -- different streams, or several host threads -- race on it and must be
 * serialised by the caller. */
DG_API int32_t dg_quant_mx_host_static(const float* x_host, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran,
                                       void* data_out, uint32_t* sf_out, void* stream);
/* replaces api::dequant_mx (deepgemm/src/api.rs:1556-1601): codes + SF -> f32 [m,k]. */
DG_API int32_t dg_dequant_mx(const void* data, const dg_sf_tensor_t* sf, uint32_t m, uint32_t k, int32_t dtype,
                      float* out, void* stream);
/* replaces api::transform_sf (deepgemm/src/api.rs:1031-1064): f32 power-of-two scales
 * [mn, sf_k] row-major -> packed words [ceil(sf_k/4), align4(mn)]. */
DG_API int32_t dg_transform_sf(const float* sf, uint32_t mn, uint32_t sf_k, uint32_t* out, void* stream);
DG_API int32_t dg_transform_sf_host(const float* sf_host, uint32_t mn, uint32_t sf_k, uint32_t* out, void* stream);
/* replaces api::transform_sf_batched (deepgemm/src/api.rs:1263-1311): sf f32 [batch, mn, sf_k] (device) ->
 * one arena [batch * ceil(sf_k/4), align4(mn)], batch b's rows starting at b * ceil(sf_k/4): the SF
 * operand layout of dg_bmm. */
DG_API int32_t dg_transform_sf_batched(const float* sf, uint32_t batch, uint32_t mn, uint32_t sf_k, uint32_t* out, void* stream);
/* replaces api::quantize_output_fp8 (deepgemm/src/api.rs:1951-2011; device side
 * deepgemm/kernels/layout_quant.cu:318-361): src f32 [m, n] (device) with row pitch in_stride elements ->
 * E4M3 codes [m, n] and packed UE8M0 words [ceil(n/32/4), align4(m)], one scale per (row, 32 columns),
 * so that a GEMM's f32 output can feed the next FP8 GEMM.  n % 32 == 0.  stochastic == 0: round to
 * nearest, bit-identical to dg_quant_mx at granularity 32 (exponent rule of deepgemm/src/golden.rs:211-224).
 * stochastic != 0: a value between two neighbouring E4M3 values goes up with probability equal to its
 * relative position between them, the draw being a hash of (element index, seed): unbiased, and
 * reproducible for a given seed. */
DG_API int32_t dg_quantize_output_fp8(const float* src, uint32_t m, uint32_t n, uint32_t in_stride, int32_t stochastic,
                                      uint32_t seed, void* data_out, uint32_t* sf_out, void* stream);

/* ---- MQA logits (lightning indexer) ----------------------------------------------------
 * logits[i, j] = sum_h w[i,h] * relu(<q[i,h,:], kv[j,:]>) for j in [ks[i], min(ke[i], S)).
 * fp32 contract (deepgemm/src/api_sm90_mqa.rs:5-31): q raw E4M3 [T,H,D]; kv E4M3 [S,D]
 * with one f32 scale per kv token applied after the head sum; weights f32 [T,H]; logits f32
 * with row pitch `logits_stride` elements, stored compressed: the value for kv token j of query i
 * goes to column j - ks[i] of row i (absolute columns when ks = 0); columns outside the range are not
 * written.  q and kv are dense ([T*H, D] and [S, D] bytes, row pitch D). */
DG_API int32_t dg_mqa_logits_f32(const void* q, const void* kv, const float* kv_scale, const float* weights,
                          const uint32_t* cu_k_start, const uint32_t* cu_k_end,
                          uint32_t num_tokens, uint32_t num_kv_tokens, uint32_t num_heads, uint32_t head_dim,
                          float* logits, uint32_t logits_stride, void* stream);
/* reference SM100 contract, api::mqa_logits (deepgemm/src/api.rs:1614-1745): q and kv carry
 * packed UE8M0 per-32 scales (the reference passes them as separate SfTensors, here they ride in
 * q.sf / kv.sf), FP8 or packed FP4 codes (head_dim 64 / 128), weights are bf16 [T,H], logits are bf16 and
 * stored compressed at column j - ks[i] (deepgemm/kernels/mqa_logits_sm100.cu:1014-1020).  num_heads: any
 * multiple of 4 whose query block fits 192 score columns (up to 192 heads). */
DG_API int32_t dg_mqa_logits(const dg_operand_t* q, const dg_operand_t* kv, const void* weights_bf16,
                      const uint32_t* cu_k_start, const uint32_t* cu_k_end,
                      uint32_t num_tokens, uint32_t num_kv_tokens, uint32_t num_heads, uint32_t head_dim,
                      void* logits_bf16, uint32_t logits_stride, void* stream);

/* replaces api::mqa_logits_paged (deepgemm/src/api.rs:1752-1941) and its metadata kernel
 * (deepgemm/kernels/mqa_logits_sm100.cu:359-492): the ue8m0 contract over a paged KV cache, for decode.
 * q as in dg_mqa_logits ([num_tokens * num_heads, head_dim], FP8 or FP4, per-32 scales); kv_pages
 * [num_pages, page_kv, head_dim] codes and kv_sf_pages [num_pages, page_kv] one scale word per token (16-byte aligned);
 * weights bf16 [num_tokens, num_heads].  indices[t] = request of query token t (sorted: tokens of a request
 * are neighbours), context_lens[t] = kv tokens visible to token t (growing inside a request),
 * block_table[first token of the request][i] = page holding the request's kv tokens [i * page_kv, (i+1) *
 * page_kv).  logits[t, j] (bf16, row pitch logits_stride) for j in [0, context_lens[t]); other columns are
 * not written.  page_kv divides 256 and is a multiple of 4.  The call takes a few words of stream-ordered
 * scratch per query token for its work list (cudaMallocAsync on `stream`). */
DG_API int32_t dg_mqa_logits_paged(const dg_operand_t* q, const void* kv_pages, const uint32_t* kv_sf_pages,
                                   const void* weights_bf16, uint32_t page_kv, uint32_t num_pages,
                                   const uint32_t* context_lens, const uint32_t* indices, const uint32_t* block_table,
                                   uint32_t block_table_stride, uint32_t num_tokens, uint32_t num_heads, uint32_t head_dim,
                                   void* logits_bf16, uint32_t logits_stride, void* stream);

/* ---- MoE row movement around the grouped GEMM -----------------------------------------------
 * The steps the reference leaves to the caller of Serving::moe_grouped_layer
 * (deepgemm/src/api_serving.rs:293-377): gather token rows (and the MN columns of their packed
 * scale factors) into the 128-row-padded contiguous layout, and combine expert outputs per token.
 * dg_gather_rows: dst[i,:] = src[idx[i],:], zeros when idx[i] < 0; rows and pitches in bytes,
 * multiples of 16. */
DG_API int32_t dg_gather_rows(const void* src, uint64_t src_pitch_bytes, const int32_t* idx, void* dst,
                              uint64_t dst_pitch_bytes, uint32_t n_rows, uint32_t row_bytes, void* stream);
/* dst[r*dst_row_stride + i*dst_col_stride] = src[r*src_row_stride + idx[i]*src_col_stride] for r < sf_rows,
 * i < n (strides in words; 0 when idx[i] < 0): permutes the MN columns of a packed SF tensor, or converts
 * it to / from a row-per-token wire format. */
DG_API int32_t dg_gather_sf(const uint32_t* src, uint64_t src_row_stride, uint64_t src_col_stride, const int32_t* idx,
                            uint32_t* dst, uint64_t dst_row_stride, uint64_t dst_col_stride, uint32_t sf_rows, uint32_t n,
                            void* stream);
/* Grouping plan on the device (no host synchronisation): rows with expert ids expert_of_row[r]
 * (negative = drop) are assigned slots so that each expert's rows are contiguous and every group
 * is padded to `align` rows (128 for the grouped GEMM, 1 for a plain sort by expert).
 *   counts[E]        rows per expert            offsets[E+1]   first slot of each group, total
 *   slot_src[cap]    r / div of the row in each slot, -1 = padding (div = top-k maps a copy to its token)
 *   slot_of_row[n]   slot of every row          block_expert[cap/align]  expert of each block, -1 = none
 *                    (may be NULL); with align = 128 this is `m_indices` (deepgemm/src/api.rs:852-853)
 * cursors[E] is caller-provided scratch.  capacity >= n_rows + E*(align-1), a multiple of align. */
DG_API int32_t dg_moe_plan(const int32_t* expert_of_row, uint32_t n_rows, uint32_t num_experts, uint32_t align,
                           uint32_t div, uint32_t capacity, int32_t* counts, int32_t* offsets, int32_t* cursors,
                           int32_t* slot_src, int32_t* slot_of_row, int32_t* block_expert, void* stream);
/* out[t,:] = sum_j weights[t,j] * src[pos[t,j],:] over the topk copies of token t (bf16 rows, f32 sum in
 * the order j = 0..topk-1); pos < 0 skips a copy; weights == NULL means 1; pitches in elements. */
DG_API int32_t dg_moe_combine(const void* src_bf16, uint64_t src_pitch, const int32_t* pos, const float* weights,
                              void* out_bf16, uint64_t out_pitch, uint32_t tokens, uint32_t topk, uint32_t cols,
                              void* stream);

/* SwiGLU + re-quantisation between the two grouped GEMMs of an MoE layer, the step the reference's
 * Serving::moe_grouped_layer leaves to its caller (deepgemm/src/api_serving.rs:371-375): gate_up is the
 * BF16 output [m, 2 * inter] of the gate/up projection (pitch in elements; gate = columns [0, inter), up =
 * columns [inter, 2 * inter)); writes E4M3 codes [m, inter] of silu(gate) * up and their packed UE8M0 scale
 * factors [ceil(inter / (4 * gran)), align4(m)], ready to be the A operand of the down projection.
 * Arithmetic as in the golden model's fused path (golden.rs:569-577): f32 on the bf16 values, no clamp. */
DG_API int32_t dg_swiglu_quant(const void* gate_up_bf16, uint64_t pitch, uint32_t m, uint32_t inter, uint32_t gran,
                               void* data_out, uint32_t* sf_out, void* stream);

/* ---- expert parallelism over peer memory (extensions; the reference runs on one GPU and has no
 * counterpart for any entry of this block) ---------------------------------------------------
 * One process per GPU inside one NVLink/NVSwitch domain.  A rank allocates buffers that the other
 * ranks map through a 64-byte handle; token rows travel to the expert owners by copy engine
 * (dg_peer_copy, no SM involved), the grouped GEMM stores its result rows straight into the token
 * owner's buffer (dg_m_grouped_gemm_nt_contiguous_rowptr), and dg_peer_barrier tells every rank that
 * the others' writes have landed. */
/* Device memory (cleared) whose handle other processes can open; free with dg_peer_free. */
DG_API int32_t dg_peer_alloc(uint64_t bytes, void** ptr);
DG_API int32_t dg_peer_free(void* ptr);
/* handle64: 64 bytes to hand to the other ranks (any host channel). */
DG_API int32_t dg_peer_export(const void* ptr, void* handle64);
/* Maps another process's buffer into this one (not valid for a handle this process exported). */
DG_API int32_t dg_peer_open(const void* handle64, void** ptr);
DG_API int32_t dg_peer_close(void* ptr);
/* Asynchronous copy between any two device addresses visible here, local or mapped. */
DG_API int32_t dg_peer_copy(void* dst, const void* src, uint64_t bytes, void* stream);
/* Barrier between the `world` ranks on `stream`: peer_flags (device array of `world` addresses) points
 * at every rank's flag array (`world` 64-bit words, cleared at allocation, one array per barrier
 * channel), local_flags is this rank's own.  `seq` must grow by one per call on a channel, alike on
 * all ranks.  Work queued on `stream` before the call is visible to every rank once its own barrier
 * call has completed.  The wait gives up after 10 s (DG_PEER_WAIT_MS in the environment changes the
 * bound); dg_poll_device_status then reports DG_ERR_DEVICE_TIMEOUT and names the missing rank. */
DG_API int32_t dg_peer_barrier(const uint64_t* peer_flags, uint64_t* local_flags, uint32_t me, uint32_t world,
                               uint64_t seq, void* stream);
/* Row address table for the return path of an expert-parallel step: ptrs[s] (device, uint64) = where
 * slot s of the padded expert layout must store its result row, 0 for padding.  slot_src[s] = position
 * of the slot's row in the received order (source rank 0's rows first); seg_start[world+1] = first
 * position of every source; dst_base[r] = rank r's return buffer as mapped here; dst_row0[r] = row of
 * that buffer where this rank's results begin; row_bytes = pitch of the return buffers. */
DG_API int32_t dg_moe_return_ptrs(const int32_t* slot_src, uint32_t slots, const int32_t* seg_start,
                                  const uint64_t* dst_base, const int32_t* dst_row0, uint32_t world,
                                  uint64_t row_bytes, uint64_t* ptrs, void* stream);
/* Dispatch by direct stores, without any host synchronisation.  counts[src * num_experts + g] (device)
 * = copies that rank src routes to global expert g, alike on every rank (one all-gather).  Experts of
 * one owner rank follow each other in its layout, each padded to `align` rows; inside an expert of
 * owner d the source ranks follow each other in the order d+1, d+2, ..., d.  dg_ep_route writes
 * dest_base[g] = first slot of this rank's copies of expert g in the owner's layout (-1 and a recorded
 * status if the owner's `cap` rows would overflow).  The local experts are cut into `slices` ranges
 * [slice_first[s], slice_first[s + 1]) (host array of slices + 1 entries from 0 to e_local; NULL =
 * equal ranges; at most 16) that can be dispatched and computed one after the other:
 * block_expert[s * (cap / align) + b] = `m_indices` entry of block b of this rank's own layout for
 * slice s (-1 for blocks of other slices), blocks_used[s] = number of leading blocks that hold
 * slices 0..s. */
DG_API int32_t dg_ep_route(const int32_t* counts, uint32_t world, uint32_t me, uint32_t num_experts, uint32_t align,
                           uint32_t cap, uint32_t slices, const uint32_t* slice_first, int32_t* dest_base,
                           int32_t* block_expert, int32_t* blocks_used, void* stream);
/* Stores the copies of this rank whose local expert index at the owner lies in [e_lo, e_hi) into the
 * owner's memory: for copy p of the copies sorted by global expert (slot_src[p] = token row,
 * my_offsets[num_experts + 1] = first p of every expert, both from dg_moe_plan with align 1), the
 * token's row of x goes to row `slot` of the owner's A buffer (a_bases[owner], rows of row_bytes), its
 * scale-factor words to column `slot` of the owner's packed SF tensor [sf_rows, cap] (sf_bases[owner])
 * and a return ticket (this rank, p) to ticket_bases[owner][slot] (64-bit words, zero = empty).  The
 * three address tables are device arrays of `world` addresses, this GPU's own or mapped peers'.
 * max_blocks > 0 bounds the grid (to share the GPU with a running GEMM). */
DG_API int32_t dg_ep_push(const void* x, uint64_t x_pitch_bytes, uint32_t row_bytes, const uint32_t* x_sf, uint32_t sf_rows,
                          uint64_t sf_cols, const int32_t* slot_src, const int32_t* my_offsets, const int32_t* dest_base,
                          uint32_t num_experts, uint32_t world, uint32_t me, uint32_t e_lo, uint32_t e_hi,
                          uint32_t n_copies, uint64_t cap, const uint64_t* a_bases, const uint64_t* sf_bases,
                          const uint64_t* ticket_bases, uint32_t max_blocks, void* stream);
/* Turns the tickets of this rank's layout into the row address table of
 * dg_m_grouped_gemm_nt_contiguous_rowptr (ptrs[s] = ret_bases[ticket rank] + position * row_bytes,
 * 0 for slots without a ticket) and clears the tickets for the next step.  With block_expert given
 * (entries per `align` slots), only slots of blocks with a non-negative entry are touched. */
DG_API int32_t dg_ep_return_ptrs(uint64_t* tickets, uint32_t slots, const uint64_t* ret_bases, uint32_t world,
                                 uint64_t row_bytes, const int32_t* block_expert, uint32_t align, uint64_t* ptrs,
                                 void* stream);
/* m_grouped_gemm_nt_contiguous whose BF16 result rows are stored at d_row_ptr[r] + column * 2 for
 * every row r of A (device table of a.rows addresses, 16-byte aligned, in this GPU's memory or a
 * mapped peer's; 0 = drop the row).  Columns [n_begin, n_begin + n_count) of every expert are computed
 * (n_count = 0: all); column n_begin lands at the row address itself.  m_blocks_used (device int32,
 * may be NULL): only the first *m_blocks_used entries of m_indices are visited, so a layout sized for
 * the worst case costs nothing for its unused tail. */
DG_API int32_t dg_m_grouped_gemm_nt_contiguous_rowptr(const dg_operand_t* a, const dg_operand_t* b,
                                                      const int32_t* m_indices, uint32_t m_indices_len,
                                                      uint32_t num_groups, const uint64_t* d_row_ptr,
                                                      const int32_t* m_blocks_used, uint32_t n_begin,
                                                      uint32_t n_count, void* stream);

/* ---- tuning / introspection -------------------------------------------------------------
 * Describes the tile configuration the library would use for a dense / grouped GEMM
 * (counterpart of heuristics::get_best_config, deepgemm/src/heuristics.rs:559-608, and of
 * DG_PRINT_CONFIGS, :23-27).  kind: 0 normal, 1 contiguous, 2 masked. */
typedef struct dg_gemm_config {
    uint32_t block_m, block_n, block_k;
    uint32_t num_stages;
    uint32_t smem_bytes;
    uint32_t num_tiles;
    uint32_t grid;
    uint32_t cluster;
} dg_gemm_config_t;
DG_API int32_t dg_get_gemm_config(int32_t dtype, int32_t kind, uint32_t m, uint32_t n, uint32_t k,
                           uint32_t num_groups, dg_gemm_config_t* cfg);

#ifdef __cplusplus
}
#endif
#endif /* DEEPGEMM_B200_H */
