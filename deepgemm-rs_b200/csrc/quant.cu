// quant_mx, dequant_mx and transform_sf for sm_100a: HBM-streaming kernels (128-bit loads,
// warp-shuffle amax, whole-word scale-factor stores, no atomics, no pre-cleared outputs).
//
// Contract (bit-exact): the reference's CPU golden model, deepgemm/src/golden.rs:211-396;
// the kernels they replace are quant_mx_impl / dequant_mx_impl / transform_sf_impl in
// deepgemm/kernels/layout_quant.cu:43-252 behind api::quant_mx / dequant_mx / transform_sf
// (deepgemm/src/api.rs:1031-1135, 1480-1601).
#include <cuda_fp16.h>

#include <atomic>

#include "host.h"
#include "mx_codec.cuh"

namespace dg {


// ------------------------------------------------------------------------- quant_mx
// One warp owns 32 consecutive rows x one "span" of 4 scale groups (4*G floats), so that it
// produces whole SF words: lane r keeps the word of row r and the warp stores 128 contiguous
// bytes of the SF row.  G = 32: one float4 per lane covers the span (8 lanes per group);
// G = 128: four float4 per lane, load j is group j.
// SWIGLU: the values to quantise are not read as f32 but formed on the fly from the BF16 output
// [m, 2k] of an MoE gate/up projection (row pitch src_pitch elements): silu(gate) * up with gate =
// columns [0, k), up = columns [k, 2k), f32 arithmetic on the bf16 values (the golden model's
// convention, deepgemm/src/golden.rs:569-577, without clamp).
// STOCH (FP8, G = 32; api::quantize_output_fp8 with `stochastic`): instead of rounding to nearest, a
// scaled value between two neighbouring E4M3 values lo < hi becomes hi with probability
// (v - lo) / (hi - lo), so that the expectation is v.  The 24 random bits of element (row, col) come from
// a counter-based hash of its index and `seed`; all the arithmetic is exact in f32, so the result is
// a pure function of (x, seed) and is checked bit for bit against the same definition on the CPU.
template <uint32_t G, bool FP4, bool SWIGLU = false, bool STOCH = false, bool PITCHED = false>
__global__ void __launch_bounds__(256) quant_mx_kernel(const float* __restrict__ x, uint32_t m, uint32_t k,
                                                      uint8_t* __restrict__ data, uint32_t* __restrict__ sf,
                                                      uint32_t sf_cols, uint32_t num_spans, uint32_t num_row_blocks,
                                                      uint64_t src_pitch = 0, uint32_t seed = 0) {
    constexpr uint32_t kLoads = G / 32;                   // float4 loads per lane per row
    // Row pitch of a plain f32 input: K itself unless PITCHED (quantize_output_fp8), as a 32-bit value so that the
    // row offset is one widening multiply.  A run-time 64-bit select in its place made the per-128 kernel 35 %
    // slower (146 against 108 us on 16384 x 7168), a 32-bit one still 7 %.
    const uint32_t x_pitch = PITCHED ? (uint32_t)src_pitch : k;
    constexpr uint32_t kRowsPerIter = G == 32 ? 8 : 2;    // rows in flight per warp
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (warp_global >= num_spans * num_row_blocks) return;
    // Consecutive warps walk the spans of one row block, so a block of 8 warps reads
    // 8 * 4G contiguous floats of each row.
    const uint32_t span = warp_global % num_spans;
    const uint32_t row0 = (warp_global / num_spans) * 32u;
    const uint32_t num_groups = k / G;
    const uint32_t groups_here = min(4u, num_groups - span * 4u);
    const uint32_t col0 = span * 4u * G;
    uint32_t my_word = 0;

    for (uint32_t rb = 0; rb < 32u; rb += kRowsPerIter) {
        float4 v[kRowsPerIter][kLoads];
        // SWIGLU: the raw BF16 gate and up values of all rows in flight; every load is issued before the first
        // value is formed (formed inside a branch beside its loads, each pair of loads was waited for in turn
        // and the kernel ran at the memory latency)
        uint2 graw[SWIGLU ? kRowsPerIter : 1][SWIGLU ? kLoads : 1], uraw[SWIGLU ? kRowsPerIter : 1][SWIGLU ? kLoads : 1];
#pragma unroll
        for (uint32_t i = 0; i < kRowsPerIter; ++i) {
            const uint32_t row = row0 + rb + i;
#pragma unroll
            for (uint32_t j = 0; j < kLoads; ++j) {
                const uint32_t grp = G == 32 ? (lane >> 3) : j;
                const bool ok = row < m && grp < groups_here;
                if (SWIGLU) {
                    const uint16_t* src = reinterpret_cast<const uint16_t*>(x) + (size_t)row * src_pitch + col0 + j * 128u + lane * 4u;
                    graw[i][j] = ok ? __ldcs(reinterpret_cast<const uint2*>(src)) : make_uint2(0u, 0u);
                    uraw[i][j] = ok ? __ldcs(reinterpret_cast<const uint2*>(src + k)) : make_uint2(0u, 0u);
                } else {
                    v[i][j] = ok ? __ldcs(reinterpret_cast<const float4*>(x + (size_t)row * x_pitch + col0 + j * 128u + lane * 4u))
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
#pragma unroll
        for (uint32_t i = 0; i < kRowsPerIter; ++i) {
            const uint32_t row = row0 + rb + i;
            uint32_t word = 0;
#pragma unroll
            for (uint32_t j = 0; j < kLoads; ++j) {
                if (SWIGLU) {
                    // rows and groups outside the tensor were loaded as zeros and give zeros
                    const uint2 gb = graw[i][j], ub = uraw[i][j];
                    float4 sv;
                    swiglu_value2(__uint_as_float(gb.x << 16), __uint_as_float(gb.x & 0xffff0000u),
                                  __uint_as_float(ub.x << 16), __uint_as_float(ub.x & 0xffff0000u), sv.x, sv.y);
                    swiglu_value2(__uint_as_float(gb.y << 16), __uint_as_float(gb.y & 0xffff0000u),
                                  __uint_as_float(ub.y << 16), __uint_as_float(ub.y & 0xffff0000u), sv.z, sv.w);
                    v[i][j] = sv;
                }
                float a = amax4(v[i][j]);
                if (G == 32) {
#pragma unroll
                    for (uint32_t s = 1; s < 8; s <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, s));
                } else {
#pragma unroll
                    for (uint32_t s = 1; s < 32; s <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, s));
                }
                a = fmaxf(a, 1e-30f);
                const uint32_t e = ue8m0_exp<FP4>(a);
                const float inv = __uint_as_float((254u - e) << 23);
                const uint32_t grp = G == 32 ? (lane >> 3) : j;
                const bool ok = row < m && grp < groups_here;
                float4 q = make_float4(v[i][j].x * inv, v[i][j].y * inv, v[i][j].z * inv, v[i][j].w * inv);
                const size_t col = col0 + j * 128u + lane * 4u;
                if (STOCH) {
                    const uint64_t idx = (uint64_t)row * k + col;
                    q.x = stochastic_e4m3_value(q.x, hash_u32(idx, seed));
                    q.y = stochastic_e4m3_value(q.y, hash_u32(idx + 1, seed));
                    q.z = stochastic_e4m3_value(q.z, hash_u32(idx + 2, seed));
                    q.w = stochastic_e4m3_value(q.w, hash_u32(idx + 3, seed));
                }
                if (FP4) {
                    const uint32_t b = cvt_e2m1x2(q.x, q.y, v[i][j].x, v[i][j].y) | (cvt_e2m1x2(q.z, q.w, v[i][j].z, v[i][j].w) << 8);
                    if (ok) *reinterpret_cast<uint16_t*>(data + ((size_t)row * k + col) / 2) = (uint16_t)b;
                } else {
                    const uint32_t b = cvt_e4m3x4(q.x, q.y, q.z, q.w, v[i][j]);
                    if (ok) *reinterpret_cast<uint32_t*>(data + (size_t)row * k + col) = b;
                }
                if (G == 32) {
                    // every lane of group g holds the group's exponent: place it in byte g and OR the
                    // four 8-lane groups together (two butterfly steps)
                    uint32_t part = grp < groups_here ? e << (8u * grp) : 0u;
                    part |= __shfl_xor_sync(0xffffffffu, part, 8);
                    part |= __shfl_xor_sync(0xffffffffu, part, 16);
                    word = part;
                } else {
                    if (j < groups_here) word |= e << (8u * j);
                }
            }
            if (lane == rb + i) my_word = row < m ? word : 0u;
        }
    }
    // One SF word per (span, row); columns m .. sf_cols-1 are padding and get zeros.
    const uint32_t row = row0 + lane;
    if (row < sf_cols) sf[(size_t)span * sf_cols + row] = my_word;
}

// ------------------------------------------------------------------------- dequant_mx
// One thread decodes 8 consecutive elements (8 or 4 code bytes) and stores two float4.
template <bool FP4>
__global__ void __launch_bounds__(256) dequant_mx_kernel(const uint8_t* __restrict__ data, const uint32_t* __restrict__ sf,
                                                        uint32_t sf_cols, uint32_t m, uint32_t k, uint32_t gran,
                                                        float* __restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t per_row = k / 8u;
    if (idx >= (size_t)m * per_row) return;
    const uint32_t row = (uint32_t)(idx / per_row);
    const uint32_t col = (uint32_t)(idx % per_row) * 8u;
    const uint32_t slot = col / gran;  // 8 | gran, so all 8 elements share one scale
    const uint32_t word = __ldg(sf + (size_t)(slot >> 2) * sf_cols + row);
    const uint32_t e = (word >> (8u * (slot & 3u))) & 0xffu;
    const float scale = __uint_as_float(e == 0u ? 0x00400000u : e << 23);  // 2^(e-127); e = 0 is subnormal
    float r[8];
    if (FP4) {
        const uint32_t c = *reinterpret_cast<const uint32_t*>(data + ((size_t)row * k + col) / 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t h2;
            const uint16_t b = (uint16_t)((c >> (8 * i)) & 0xffu);
            asm("{ .reg .b8 t, z;\n mov.b16 {t, z}, %1;\n cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "h"(b));
            const float2 f = __half22float2(*reinterpret_cast<__half2*>(&h2));
            r[2 * i] = f.x * scale;
            r[2 * i + 1] = f.y * scale;
        }
    } else {
        const uint2 c = *reinterpret_cast<const uint2*>(data + (size_t)row * k + col);
        const uint32_t w[2] = {c.x, c.y};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t h2;
            const uint16_t b = (uint16_t)((w[i >> 1] >> (16 * (i & 1))) & 0xffffu);
            asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(b));
            const float2 f = __half22float2(*reinterpret_cast<__half2*>(&h2));
            r[2 * i] = f.x * scale;
            r[2 * i + 1] = f.y * scale;
        }
    }
    float4* o = reinterpret_cast<float4*>(out + (size_t)row * k + col);
    __stcs(o, make_float4(r[0], r[1], r[2], r[3]));
    __stcs(o + 1, make_float4(r[4], r[5], r[6], r[7]));
}

// ------------------------------------------------------------------------- transform_sf
// f32 [mn, sf_k] -> u32 [ceil(sf_k/4), align4(mn)].  A block stages 64 rows x 64 scales in
// shared memory with row-contiguous loads, then writes words with mn-contiguous stores.
__global__ void __launch_bounds__(256) transform_sf_kernel(const float* __restrict__ sf, uint32_t mn, uint32_t sf_k,
                                                          uint32_t* __restrict__ out, uint32_t out_cols) {
    __shared__ uint32_t tile[64][65];
    // blockIdx.z = batch (transform_sf_batched): inputs [batch, mn, sf_k], outputs stacked along the word rows
    sf += (size_t)blockIdx.z * mn * sf_k;
    out += (size_t)blockIdx.z * ((sf_k + 3u) / 4u) * out_cols;
    const uint32_t m0 = blockIdx.x * 64u, k0 = blockIdx.y * 64u;
    for (uint32_t i = threadIdx.x; i < 64u * 64u; i += 256u) {
        const uint32_t r = i >> 6, c = i & 63u;
        const uint32_t m = m0 + r, kk = k0 + c;
        // exponent byte of the f32 (golden.rs:115-117); rows / scales outside the tensor give 0
        tile[r][c] = (m < mn && kk < sf_k) ? ((__float_as_uint(__ldg(sf + (size_t)m * sf_k + kk)) >> 23) & 0xffu) : 0u;
    }
    __syncthreads();
    // 16 word rows x 64 columns per block
    for (uint32_t i = threadIdx.x; i < 16u * 64u; i += 256u) {
        const uint32_t wr = i >> 6, c = i & 63u;
        const uint32_t m = m0 + c, word_row = (k0 >> 2) + wr;
        if (m < out_cols && word_row * 4u < sf_k) {
            const uint32_t w = tile[c][4 * wr] | (tile[c][4 * wr + 1] << 8) | (tile[c][4 * wr + 2] << 16) |
                               (tile[c][4 * wr + 3] << 24);
            out[(size_t)word_row * out_cols + m] = w;
        }
    }
}

// ------------------------------------------------------------------------- host side
static int32_t check_quant_args(const void* x, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran,
                                const void* data_out, const void* sf_out, bool x_on_host = false) {
    if (!x || !data_out || !sf_out) return fail(DG_ERR_INVALID_ARG, "quant_mx: null buffer");
    if (m == 0 || k == 0) return fail(DG_ERR_INVALID_ARG, "quant_mx: empty shape %u x %u", m, k);
    if (dtype != DG_FP8 && dtype != DG_FP4) return fail(DG_ERR_INVALID_ARG, "quant_mx: dtype must be FP8 or FP4");
    if (gran != 32 && gran != 128) return fail(DG_ERR_INVALID_ARG, "quant_mx: granularity must be 32 or 128");
    // deepgemm/src/api.rs:1489-1498
    if (dtype == DG_FP4 && (gran != 32 || k % 32 != 0))
        return fail(DG_ERR_INVALID_ARG, "quant_mx: FP4 requires granularity 32 and K (%u) %% 32 == 0", k);
    if (k % gran != 0) return fail(DG_ERR_INVALID_ARG, "quant_mx: K (%u) must be a multiple of the SF granularity %u", k, gran);
    // the kernel reads x in 16-byte vectors; a host tensor is only the source of a copy into an aligned staging area
    if (!x_on_host && (reinterpret_cast<uintptr_t>(x) & 15u)) return fail(DG_ERR_INVALID_ARG, "quant_mx: x must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(data_out) & 3u) return fail(DG_ERR_INVALID_ARG, "quant_mx: the code buffer must be 4-byte aligned");
    return DG_OK;
}

static int32_t launch_quant(const float* x, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran, void* data_out,
                            uint32_t* sf_out, cudaStream_t s) {
    const uint32_t sf_cols = align_up(m, 4);
    const uint32_t num_spans = ceil_div(k / gran, 4);
    const uint32_t num_row_blocks = ceil_div(sf_cols, 32);
    const uint64_t warps = (uint64_t)num_spans * num_row_blocks;
    const uint32_t blocks = (uint32_t)((warps + 7) / 8);
    uint8_t* d = static_cast<uint8_t*>(data_out);
    if (dtype == DG_FP4)
        quant_mx_kernel<32, true><<<blocks, 256, 0, s>>>(x, m, k, d, sf_out, sf_cols, num_spans, num_row_blocks);
    else if (gran == 32)
        quant_mx_kernel<32, false><<<blocks, 256, 0, s>>>(x, m, k, d, sf_out, sf_cols, num_spans, num_row_blocks);
    else
        quant_mx_kernel<128, false><<<blocks, 256, 0, s>>>(x, m, k, d, sf_out, sf_cols, num_spans, num_row_blocks);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

}  // namespace dg

extern "C" {

int32_t dg_swiglu_quant(const void* gate_up_bf16, uint64_t pitch, uint32_t m, uint32_t inter, uint32_t gran, void* data_out,
                        uint32_t* sf_out, void* stream) {
    if (!gate_up_bf16 || !data_out || !sf_out) return dg::fail(DG_ERR_INVALID_ARG, "swiglu_quant: null buffer");
    if (gran != 32 && gran != 128) return dg::fail(DG_ERR_INVALID_ARG, "swiglu_quant: SF granularity must be 32 or 128");
    if (m == 0 || inter == 0 || inter % gran != 0 || inter % 4 != 0)
        return dg::fail(DG_ERR_INVALID_ARG, "swiglu_quant: the intermediate width (%u) must be a positive multiple of the granularity", inter);
    if (pitch < 2ull * inter || pitch % 4 != 0 || (reinterpret_cast<uintptr_t>(gate_up_bf16) & 7u))
        return dg::fail(DG_ERR_INVALID_ARG, "swiglu_quant: the row pitch must cover 2 x %u columns and keep rows 8-byte aligned", inter);
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    const uint32_t sf_cols = dg::align_up(m, 4);
    const uint32_t num_spans = dg::ceil_div(inter / gran, 4);
    const uint32_t num_row_blocks = dg::ceil_div(sf_cols, 32);
    const uint32_t blocks = (uint32_t)(((uint64_t)num_spans * num_row_blocks + 7) / 8);
    const float* src = static_cast<const float*>(gate_up_bf16);
    uint8_t* d = static_cast<uint8_t*>(data_out);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gran == 32)
        dg::quant_mx_kernel<32, false, true><<<blocks, 256, 0, s>>>(src, m, inter, d, sf_out, sf_cols, num_spans, num_row_blocks, pitch);
    else
        dg::quant_mx_kernel<128, false, true><<<blocks, 256, 0, s>>>(src, m, inter, d, sf_out, sf_cols, num_spans, num_row_blocks, pitch);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_quant_mx(const float* x, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran, void* data_out,
                    uint32_t* sf_out, void* stream) {
    int32_t st = dg::check_quant_args(x, m, k, dtype, gran, data_out, sf_out);
    if (st != DG_OK) return st;
    const dg::DeviceInfo* dev;
    if ((st = dg::current_device(&dev)) != DG_OK) return st;
    return dg::launch_quant(x, m, k, dtype, gran, data_out, sf_out, static_cast<cudaStream_t>(stream));
}

int32_t dg_quant_mx_host(const float* x_host, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran, void* data_out,
                         uint32_t* sf_out, void* stream) {
    int32_t st = dg::check_quant_args(x_host, m, k, dtype, gran, data_out, sf_out, true);
    if (st != DG_OK) return st;
    const dg::DeviceInfo* dev;
    if ((st = dg::current_device(&dev)) != DG_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* staging = nullptr;
    const size_t bytes = (size_t)m * k * sizeof(float);
    DG_CUDA_CHECK(cudaMallocAsync(&staging, bytes, s));
    cudaError_t e = cudaMemcpyAsync(staging, x_host, bytes, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) st = dg::launch_quant(staging, m, k, dtype, gran, data_out, sf_out, s);
    cudaFreeAsync(staging, s);
    if (e != cudaSuccess) return dg::fail(DG_ERR_DRIVER, "quant_mx: host to device copy failed: %s", cudaGetErrorString(e));
    return st;
}

// ---- quant_mx from host memory without any allocation --------------------------------------
// Staging area for the host tensor, owned by the library image: every GPU that loads the
// library holds these bytes until the process exits.
constexpr size_t kStaticStagingBytes = 16u << 20;   // 16 MiB = 4 Mi f32 elements
static __device__ __align__(256) unsigned char g_quant_staging[kStaticStagingBytes];
// g_quant_staging names a host-side handle in host code, not a device address: the address the
// kernel and the copy engine need comes from cudaGetSymbolAddress, once per device.
// (Several host threads may make the first call on a device at once: they all look up the same address,
// and the atomic slot keeps the publication well defined.)
static std::atomic<float*> g_quant_staging_addr[64];

int32_t dg_quant_mx_host_static(const float* x_host, uint32_t m, uint32_t k, int32_t dtype, uint32_t gran,
                                void* data_out, uint32_t* sf_out, void* stream) {
    int32_t st = dg::check_quant_args(x_host, m, k, dtype, gran, data_out, sf_out, true);
    if (st != DG_OK) return st;
    const size_t bytes = (size_t)m * k * sizeof(float);
    if (bytes > kStaticStagingBytes)
        return dg::fail(DG_ERR_INVALID_ARG,
                        "quant_mx (static staging): %u x %u f32 = %zu bytes exceeds the %zu-byte built-in staging area; "
                        "use dg_quant_mx_host or split the rows",
                        m, k, bytes, (size_t)kStaticStagingBytes);
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return dg::fail(DG_ERR_UNSUPPORTED, "no usable CUDA device; the kernels require SM100 (Blackwell)");
    }
    if (!g_quant_staging_addr[dev].load(std::memory_order_acquire)) {
        // one-time set-up on this device (it is the current one)
        int major = 0;
        DG_CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return dg::fail(DG_ERR_UNSUPPORTED, "the kernels require SM100 (Blackwell); this device is sm_%d*", major);
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_quant_staging);
        if (e != cudaSuccess || !p)
            return dg::fail(DG_ERR_DRIVER, "cudaGetSymbolAddress(static staging area) failed: %s", cudaGetErrorString(e));
        g_quant_staging_addr[dev].store(static_cast<float*>(p), std::memory_order_release);
    }
    float* staging = g_quant_staging_addr[dev].load(std::memory_order_acquire);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DG_CUDA_CHECK(cudaMemcpyAsync(staging, x_host, bytes, cudaMemcpyHostToDevice, s));
    return dg::launch_quant(staging, m, k, dtype, gran, data_out, sf_out, s);
}

int32_t dg_dequant_mx(const void* data, const dg_sf_tensor_t* sf, uint32_t m, uint32_t k, int32_t dtype, float* out,
                      void* stream) {
    int32_t st;
    if (!data || !sf || !sf->data || !out) return dg::fail(DG_ERR_INVALID_ARG, "dequant_mx: null buffer");
    if (dtype != DG_FP8 && dtype != DG_FP4) return dg::fail(DG_ERR_INVALID_ARG, "dequant_mx: dtype must be FP8 or FP4");
    if (sf->gran != 32 && sf->gran != 128) return dg::fail(DG_ERR_INVALID_ARG, "dequant_mx: granularity must be 32 or 128");
    if (m == 0 || k == 0 || k % sf->gran != 0)
        return dg::fail(DG_ERR_INVALID_ARG, "dequant_mx: K (%u) must be a positive multiple of the SF granularity %u", k, sf->gran);
    if (sf->cols < m || sf->rows < dg::ceil_div(k, sf->gran * 4))
        return dg::fail(DG_ERR_INVALID_ARG, "dequant_mx: SF tensor %u x %u too small for %u x %u", sf->rows, sf->cols, m, k);
    if ((reinterpret_cast<uintptr_t>(data) & 7u) || (reinterpret_cast<uintptr_t>(out) & 15u))
        return dg::fail(DG_ERR_INVALID_ARG, "dequant_mx: buffers must be 8/16-byte aligned");
    const dg::DeviceInfo* dev;
    if ((st = dg::current_device(&dev)) != DG_OK) return st;
    const uint64_t threads = (uint64_t)m * (k / 8);
    const uint32_t blocks = (uint32_t)((threads + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == DG_FP4)
        dg::dequant_mx_kernel<true><<<blocks, 256, 0, s>>>(static_cast<const uint8_t*>(data), sf->data, sf->cols, m, k, sf->gran, out);
    else
        dg::dequant_mx_kernel<false><<<blocks, 256, 0, s>>>(static_cast<const uint8_t*>(data), sf->data, sf->cols, m, k, sf->gran, out);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

static int32_t transform_sf_impl(const float* sf, uint32_t mn, uint32_t sf_k, uint32_t* out, cudaStream_t s, uint32_t batch = 1) {
    const uint32_t cols = dg::align_up(mn, 4);
    dim3 grid(dg::ceil_div(cols, 64), dg::ceil_div(sf_k, 64), batch);
    dg::transform_sf_kernel<<<grid, 256, 0, s>>>(sf, mn, sf_k, out, cols);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_transform_sf(const float* sf, uint32_t mn, uint32_t sf_k, uint32_t* out, void* stream) {
    if (!sf || !out) return dg::fail(DG_ERR_INVALID_ARG, "transform_sf: null buffer");
    if (mn == 0 || sf_k == 0) return dg::fail(DG_ERR_INVALID_ARG, "sf length must be mn * sf_k");
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    return transform_sf_impl(sf, mn, sf_k, out, static_cast<cudaStream_t>(stream));
}

int32_t dg_transform_sf_batched(const float* sf, uint32_t batch, uint32_t mn, uint32_t sf_k, uint32_t* out, void* stream) {
    if (!sf || !out) return dg::fail(DG_ERR_INVALID_ARG, "transform_sf_batched: null buffer");
    if (batch == 0) return dg::fail(DG_ERR_INVALID_ARG, "batch must be nonzero");
    if (batch > 65535) return dg::fail(DG_ERR_INVALID_ARG, "transform_sf_batched: at most 65535 batches");
    if (mn == 0 || sf_k == 0) return dg::fail(DG_ERR_INVALID_ARG, "batched SF must hold batch * mn * sf_k values");
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    return transform_sf_impl(sf, mn, sf_k, out, static_cast<cudaStream_t>(stream), batch);
}

int32_t dg_quantize_output_fp8(const float* src, uint32_t m, uint32_t n, uint32_t in_stride, int32_t stochastic, uint32_t seed,
                               void* data_out, uint32_t* sf_out, void* stream) {
    if (!src || !data_out || !sf_out) return dg::fail(DG_ERR_INVALID_ARG, "quantize_output_fp8: null buffer");
    if (m == 0 || n == 0 || n % 32 != 0) return dg::fail(DG_ERR_INVALID_ARG, "quantize_output_fp8 needs n %% 32 == 0 (n = %u, m = %u)", n, m);
    if (in_stride < n || in_stride % 4 != 0 || (reinterpret_cast<uintptr_t>(src) & 15u) || (reinterpret_cast<uintptr_t>(data_out) & 3u))
        return dg::fail(DG_ERR_INVALID_ARG, "quantize_output_fp8: in_stride (%u) must cover n, rows must stay 16-byte aligned", in_stride);
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    const uint32_t sf_cols = dg::align_up(m, 4);
    const uint32_t num_spans = dg::ceil_div(n / 32, 4);
    const uint32_t num_row_blocks = dg::ceil_div(sf_cols, 32);
    const uint32_t blocks = (uint32_t)(((uint64_t)num_spans * num_row_blocks + 7) / 8);
    uint8_t* d = static_cast<uint8_t*>(data_out);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (stochastic)
        dg::quant_mx_kernel<32, false, false, true, true><<<blocks, 256, 0, s>>>(src, m, n, d, sf_out, sf_cols, num_spans, num_row_blocks, in_stride, seed);
    else
        dg::quant_mx_kernel<32, false, false, false, true><<<blocks, 256, 0, s>>>(src, m, n, d, sf_out, sf_cols, num_spans, num_row_blocks, in_stride);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_transform_sf_host(const float* sf_host, uint32_t mn, uint32_t sf_k, uint32_t* out, void* stream) {
    if (!sf_host || !out) return dg::fail(DG_ERR_INVALID_ARG, "transform_sf: null buffer");
    if (mn == 0 || sf_k == 0) return dg::fail(DG_ERR_INVALID_ARG, "sf length must be mn * sf_k");
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* staging = nullptr;
    const size_t bytes = (size_t)mn * sf_k * sizeof(float);
    DG_CUDA_CHECK(cudaMallocAsync(&staging, bytes, s));
    cudaError_t e = cudaMemcpyAsync(staging, sf_host, bytes, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) st = transform_sf_impl(staging, mn, sf_k, out, s);
    cudaFreeAsync(staging, s);
    if (e != cudaSuccess) return dg::fail(DG_ERR_DRIVER, "transform_sf: host to device copy failed: %s", cudaGetErrorString(e));
    return st;
}

}  // extern "C"
