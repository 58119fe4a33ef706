// Row movement around the grouped GEMM for MoE layers: building the 128-row-padded contiguous
// layout (token rows and their packed scale factors) and combining expert outputs back per
// token.  These are the steps the reference leaves to the caller of
// Serving::moe_grouped_layer (deepgemm/src/api_serving.rs:293-377); they are pure HBM streaming.
#include "host.h"

#include <cuda_bf16.h>

namespace dg {

// dst[i, :] = src[idx[i], :], or zeros when idx[i] < 0.  One warp per row, 16-byte vectors.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ idx,
                                                         uint4* __restrict__ dst, uint32_t n_rows, uint32_t vec_per_row,
                                                         uint64_t src_pitch_vec, uint64_t dst_pitch_vec) {
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (row >= n_rows) return;
    const int32_t s = __ldg(idx + row);
    uint4* d = dst + (size_t)row * dst_pitch_vec;
    if (s < 0) {
        for (uint32_t v = lane; v < vec_per_row; v += 32u) d[v] = make_uint4(0, 0, 0, 0);
    } else {
        // source rows are read once per top-k copy: keep them cached, stream the copies out
        const uint4* p = src + (size_t)s * src_pitch_vec;
        uint32_t v = lane;
        for (; v + 96u < vec_per_row; v += 128u) {     // four loads in flight per lane before the stores
            const uint4 r0 = __ldg(p + v), r1 = __ldg(p + v + 32u), r2 = __ldg(p + v + 64u), r3 = __ldg(p + v + 96u);
            __stcs(d + v, r0); __stcs(d + v + 32u, r1); __stcs(d + v + 64u, r2); __stcs(d + v + 96u, r3);
        }
        for (; v < vec_per_row; v += 32u) __stcs(d + v, __ldg(p + v));
    }
}

// dst[r * dst_sr + i * dst_si] = src[r * src_sr + idx[i] * src_si] (0 when idx[i] < 0), words.
// With (sr, si) = (cols, 1) on both sides this permutes the MN columns of a packed SF tensor;
// with one side (1, sf_rows) it converts to / from a row-per-token wire format.
__global__ void __launch_bounds__(256) gather_sf_kernel(const uint32_t* __restrict__ src, uint64_t src_sr, uint64_t src_si,
                                                       const int32_t* __restrict__ idx, uint32_t* __restrict__ dst,
                                                       uint64_t dst_sr, uint64_t dst_si, uint32_t sf_rows, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int32_t s = __ldg(idx + i);
    for (uint32_t r = 0; r < sf_rows; ++r)
        dst[r * dst_sr + (size_t)i * dst_si] = s < 0 ? 0u : __ldg(src + r * src_sr + (size_t)s * src_si);
}

// out[t, :] = sum_j w[t, j] * src[pos[t, j], :] over the top-k copies of token t (f32 sum in the
// order j = 0..topk-1, one bf16 rounding at the end); pos < 0 skips a copy; w == NULL means 1.
__global__ void __launch_bounds__(256) combine_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ pos,
                                                     const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                     uint32_t tokens, uint32_t topk, uint32_t cols, uint64_t src_pitch,
                                                     uint64_t out_pitch) {
    const uint32_t t = blockIdx.x;
    if (t >= tokens) return;
    for (uint32_t c = threadIdx.x * 8u; c < cols; c += blockDim.x * 8u) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (uint32_t j = 0; j < topk; ++j) {
            const int32_t p = __ldg(pos + (size_t)t * topk + j);
            if (p < 0) continue;
            const float g = w ? __ldg(w + (size_t)t * topk + j) : 1.f;
            const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src + (size_t)p * src_pitch + c));
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[2 * q] += g * __uint_as_float(u[q] << 16);
                acc[2 * q + 1] += g * __uint_as_float(u[q] & 0xffff0000u);
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
            o[q] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * out_pitch + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- grouping plan: rows -> expert-contiguous slots ---------------------------------------------
// plan_count: counts[e] = number of rows routed to expert e (counts zeroed by the caller's stream).
__global__ void __launch_bounds__(256) plan_count_kernel(const int32_t* __restrict__ expert_of_row, uint32_t n_rows,
                                                        uint32_t num_experts, int32_t* __restrict__ counts) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const int32_t e = __ldg(expert_of_row + r);
    if (e >= 0 && (uint32_t)e < num_experts) atomicAdd(counts + e, 1);
}

// plan_scan (one block): offsets[e] = first slot of expert e with every group padded to `align`
// rows, offsets[E] = total; block_expert[b] = expert owning the b-th `align`-row block or -1;
// cursors reset to 0.
__global__ void __launch_bounds__(1024) plan_scan_kernel(const int32_t* __restrict__ counts, uint32_t num_experts,
                                                        uint32_t align, uint32_t capacity, int32_t* __restrict__ offsets,
                                                        int32_t* __restrict__ cursors, int32_t* __restrict__ block_expert) {
    extern __shared__ int32_t sh_off[];  // [num_experts + 1]
    if (threadIdx.x == 0) {
        int32_t acc = 0;
        for (uint32_t e = 0; e < num_experts; ++e) {
            sh_off[e] = acc;
            acc += (int32_t)(((uint32_t)counts[e] + align - 1) / align * align);
        }
        sh_off[num_experts] = acc;
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e <= num_experts; e += blockDim.x) {
        offsets[e] = sh_off[e];
        if (e < num_experts) cursors[e] = 0;
    }
    if (block_expert) {
        const uint32_t total = (uint32_t)sh_off[num_experts];
        for (uint32_t b = threadIdx.x; b < capacity / align; b += blockDim.x) {
            const uint32_t row = b * align;
            int32_t owner = -1;
            if (row < total) {
                uint32_t lo = 0, hi = num_experts;      // last e with sh_off[e] <= row
                while (hi - lo > 1) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if ((uint32_t)sh_off[mid] <= row) lo = mid; else hi = mid;
                }
                owner = (int32_t)lo;
            }
            block_expert[b] = owner;
        }
    }
}

// plan_place: every row takes the next free slot of its expert.  slot_src[slot] = r / div (the
// token of copy r when div = top-k), slot_of_row[r] = slot.  The order of rows inside a group is
// not fixed from run to run; no result depends on it (a GEMM row does not see its neighbours).
__global__ void __launch_bounds__(256) plan_place_kernel(const int32_t* __restrict__ expert_of_row, uint32_t n_rows,
                                                        uint32_t num_experts, uint32_t div, const int32_t* __restrict__ offsets,
                                                        int32_t* __restrict__ cursors, int32_t* __restrict__ slot_src,
                                                        int32_t* __restrict__ slot_of_row) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const int32_t e = __ldg(expert_of_row + r);
    if (e < 0 || (uint32_t)e >= num_experts) { slot_of_row[r] = -1; return; }
    const int32_t slot = offsets[e] + atomicAdd(cursors + e, 1);
    slot_src[slot] = (int32_t)(r / div);
    slot_of_row[r] = slot;
}

}  // namespace dg

extern "C" {

int32_t dg_moe_plan(const int32_t* expert_of_row, uint32_t n_rows, uint32_t num_experts, uint32_t align, uint32_t div,
                    uint32_t capacity, int32_t* counts, int32_t* offsets, int32_t* cursors, int32_t* slot_src,
                    int32_t* slot_of_row, int32_t* block_expert, void* stream) {
    if (!expert_of_row || !counts || !offsets || !cursors || !slot_src || !slot_of_row)
        return dg::fail(DG_ERR_INVALID_ARG, "moe_plan: null buffer");
    if (num_experts == 0 || num_experts > 8192 || align == 0 || div == 0 || capacity % align != 0)
        return dg::fail(DG_ERR_INVALID_ARG, "moe_plan: need 1..8192 experts, align > 0, div > 0 and capacity %% align == 0");
    if ((uint64_t)capacity < (uint64_t)n_rows + (uint64_t)num_experts * (align - 1))
        return dg::fail(DG_ERR_INVALID_ARG, "moe_plan: capacity %u cannot hold %u rows in %u groups padded to %u", capacity,
                        n_rows, num_experts, align);
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DG_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int32_t) * num_experts, s));
    DG_CUDA_CHECK(cudaMemsetAsync(slot_src, 0xff, sizeof(int32_t) * (size_t)capacity, s));
    if (n_rows) {
        dg::plan_count_kernel<<<dg::ceil_div(n_rows, 256), 256, 0, s>>>(expert_of_row, n_rows, num_experts, counts);
        dg::note_launch();
    }
    dg::plan_scan_kernel<<<1, 1024, sizeof(int32_t) * (num_experts + 1), s>>>(counts, num_experts, align, capacity, offsets,
                                                                              cursors, block_expert);
    dg::note_launch();
    if (n_rows) {
        dg::plan_place_kernel<<<dg::ceil_div(n_rows, 256), 256, 0, s>>>(expert_of_row, n_rows, num_experts, div, offsets,
                                                                        cursors, slot_src, slot_of_row);
        dg::note_launch();
    }
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_gather_rows(const void* src, uint64_t src_pitch_bytes, const int32_t* idx, void* dst, uint64_t dst_pitch_bytes,
                       uint32_t n_rows, uint32_t row_bytes, void* stream) {
    if (!src || !idx || !dst) return dg::fail(DG_ERR_INVALID_ARG, "gather_rows: null buffer");
    if (row_bytes % 16 || src_pitch_bytes % 16 || dst_pitch_bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15u) ||
        (reinterpret_cast<uintptr_t>(dst) & 15u))
        return dg::fail(DG_ERR_INVALID_ARG, "gather_rows: rows, pitches and bases must be 16-byte multiples");
    if (n_rows == 0) return DG_OK;
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    dg::gather_rows_kernel<<<dg::ceil_div(n_rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), idx, static_cast<uint4*>(dst), n_rows, row_bytes / 16, src_pitch_bytes / 16,
        dst_pitch_bytes / 16);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_gather_sf(const uint32_t* src, uint64_t src_row_stride, uint64_t src_col_stride, const int32_t* idx, uint32_t* dst,
                     uint64_t dst_row_stride, uint64_t dst_col_stride, uint32_t sf_rows, uint32_t n, void* stream) {
    if (!src || !idx || !dst) return dg::fail(DG_ERR_INVALID_ARG, "gather_sf: null buffer");
    if (n == 0 || sf_rows == 0) return DG_OK;
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    dg::gather_sf_kernel<<<dg::ceil_div(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, src_row_stride, src_col_stride, idx, dst, dst_row_stride, dst_col_stride, sf_rows, n);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_moe_combine(const void* src_bf16, uint64_t src_pitch, const int32_t* pos, const float* weights, void* out_bf16,
                       uint64_t out_pitch, uint32_t tokens, uint32_t topk, uint32_t cols, void* stream) {
    if (!src_bf16 || !pos || !out_bf16) return dg::fail(DG_ERR_INVALID_ARG, "moe_combine: null buffer");
    if (cols % 8 || src_pitch % 8 || out_pitch % 8 || (reinterpret_cast<uintptr_t>(src_bf16) & 15u) ||
        (reinterpret_cast<uintptr_t>(out_bf16) & 15u))
        return dg::fail(DG_ERR_INVALID_ARG, "moe_combine: columns and pitches must be multiples of 8 elements, bases 16-byte aligned");
    if (tokens == 0) return DG_OK;
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    dg::combine_kernel<<<tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(src_bf16), pos, weights, static_cast<__nv_bfloat16*>(out_bf16), tokens, topk, cols,
        src_pitch, out_pitch);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

}  // extern "C"
