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
        const uint4* p = src + (size_t)s * src_pitch_vec;
        for (uint32_t v = lane; v < vec_per_row; v += 32u) d[v] = __ldcs(p + v);
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

}  // namespace dg

extern "C" {

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
