// MQA logits (MLA lightning indexer) for sm_100a:
//   logits[i, j] = s_kv[j] * sum_h w[i,h] * relu(<q[i,h,:], kv[j,:]>),  j in [ks[i], min(ke[i], S))
// stored compressed at column j - ks[i] of row i.
//
// Two contracts of the reference share this kernel:
//   fp32  (deepgemm/src/api_sm90_mqa.rs:5-31): raw E4M3 q, E4M3 kv with one f32 scale per kv
//         token, f32 weights, f32 logits           -> tcgen05.mma kind::f8f6f4
//   ue8m0 (api::mqa_logits, deepgemm/src/api.rs:1614-1745; device side
//         deepgemm/kernels/mqa_logits_sm100.cu:514-1084): UE8M0 scales per 32 along head_dim on
//         q and kv, bf16 weights, bf16 logits      -> tcgen05.mma kind::mxf8f6f4.block_scale
// Numerical contract: mqa_logits_ref of the golden model (deepgemm/src/golden.rs:469-501).
//
// The contraction runs with the 128 kv tokens of a block on the UMMA M side (TMEM lanes) and
// the (query, head) pairs of a query block on the N side, so one epilogue thread owns one kv
// token, reduces over heads with weights broadcast from shared memory and the warp stores 32
// consecutive columns of a logits row.
//   warp 0      TMA producer (Q tile per query block, KV tiles streamed through a ring)
//   warp 1      MMA issuer (head_dim/32 MMAs per kv block, two accumulator stages in TMEM)
//   warp 2      TMEM owner; ue8m0 contract: scale-factor transposer
//   warps 4-..  two or four epilogue warpgroups, each reducing its share of the query block's
//               columns with the next TMEM load in flight while a chunk is consumed
#include "host.h"
#include "ptx.cuh"

#include <cstdlib>

namespace dg {

constexpr uint32_t kMqaBlockKv = 128;
constexpr uint32_t kMqaMaxKvStages = 10;
constexpr uint32_t kMqaMaxThreads = 640;   // 4 role warps + up to 4 epilogue warpgroups
constexpr uint32_t kMqaSfaCol = 448;   // ue8m0 contract only: accumulators are <= 192 wide
constexpr uint32_t kMqaSfbCol = 452;

struct MqaParams {
    uint32_t num_tokens, num_kv, num_heads, head_dim;
    uint32_t block_q, n;          // n = block_q * num_heads (UMMA N)
    uint32_t ep_groups;           // epilogue warpgroups (2 or 4); each reduces block_q / ep_groups queries
    uint32_t num_q_blocks;
    uint32_t kv_stages, kv_stage_bytes, q_stage_bytes;
    uint32_t off_w, off_q, off_kv;  // offsets from the 1024-aligned base
    uint32_t kv_sf_off, q_sf_off;   // SF words inside a kv / q stage (ue8m0 contract)
    uint32_t sbo;                   // 8-row group pitch of the swizzled tiles
    uint32_t layout;                // UMMA layout type of the tiles
    uint32_t logits_stride;
    const uint32_t* ks;
    const uint32_t* ke;
    const float* kv_scale;          // fp32 contract
    const void* weights;            // f32 (fp32 contract) or bf16 (ue8m0 contract)
    void* logits;
    uint32_t* status;
};

struct __align__(8) MqaBarriers {
    uint64_t kv_full[kMqaMaxKvStages];
    uint64_t kv_ready[kMqaMaxKvStages];   // ue8m0: SF transposed
    uint64_t kv_empty[kMqaMaxKvStages];
    uint64_t q_full[2], q_ready[2], q_empty[2];
    uint64_t tmem_full[2], tmem_empty[2];
    uint64_t w_full[2];                   // weights of a query block staged by the 8 epilogue warps
    uint32_t tmem_base;
    uint32_t abort;
};

// kv-block range [b0, b1) that a query block touches; identical in every role.
struct QRange { uint32_t b0, b1; };
__device__ __forceinline__ QRange q_block_range(const MqaParams& p, uint32_t qb) {
    uint32_t lo = 0xffffffffu, hi = 0;
    for (uint32_t i = 0; i < p.block_q; ++i) {
        const uint32_t q = qb * p.block_q + i;
        if (q < p.num_tokens) {
            const uint32_t s = __ldg(p.ks + q), e = min(__ldg(p.ke + q), p.num_kv);
            if (s < e) { lo = min(lo, s); hi = max(hi, e); }
        }
    }
    QRange r;
    r.b0 = hi > lo ? lo / kMqaBlockKv : 0;
    r.b1 = hi > lo ? (hi + kMqaBlockKv - 1) / kMqaBlockKv : 0;
    return r;
}

__device__ __forceinline__ void tc_mma_f8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc_f8(uint32_t m, uint32_t n) {
    return (1u << 4) /*D=f32*/ | ((n >> 3) << 17) | ((m >> 4) << 24);  // A, B = E4M3 (format 0), K-major
}

template <bool SCALED>
__global__ void __launch_bounds__(kMqaMaxThreads, 1)
mqa_logits_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                  const __grid_constant__ CUtensorMap tm_qsf, const __grid_constant__ CUtensorMap tm_kvsf,
                  const MqaParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base = (raw_u32 + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_u32);
    MqaBarriers* bars = reinterpret_cast<MqaBarriers*>(base_ptr);
    float* w_smem = reinterpret_cast<float*>(base_ptr + p.off_w);   // [2][n]
    uint32_t* win_smem = reinterpret_cast<uint32_t*>(base_ptr + 512);  // [2][2][16]: ks / ke of the queries of a block
    static_assert(sizeof(MqaBarriers) <= 512, "barrier block overlaps the window table");
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const WaitCtx wc{p.status, &bars->abort};

    if (threadIdx.x == 0) {
        bars->abort = 0;
        for (uint32_t s = 0; s < p.kv_stages; ++s) {
            mbar_init(smem_u32(&bars->kv_full[s]), 1);
            mbar_init(smem_u32(&bars->kv_ready[s]), 1);
            mbar_init(smem_u32(&bars->kv_empty[s]), 1);
        }
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bars->q_full[s]), 1);
            mbar_init(smem_u32(&bars->q_ready[s]), 1);
            mbar_init(smem_u32(&bars->q_empty[s]), 1);
            mbar_init(smem_u32(&bars->tmem_full[s]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[s]), 4 * p.ep_groups);
            mbar_init(smem_u32(&bars->w_full[s]), 4 * p.ep_groups);
        }
        fence_barrier_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_kv);
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(&bars->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_wait();                 // the kernel before this one in the stream produced q / kv / weights
    griddep_launch_dependents();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
    const uint32_t acc_stride = SCALED ? 192u : 256u;
    const uint32_t num_mma = p.head_dim / 32u;

    if (warp == 0) {
        // ===================================================== producer (warp-converged, one lane issues)
        uint32_t stage = 0, phase = 0, qcount = 0;
        bool ok = true;
        for (uint32_t qb = blockIdx.x; ok && qb < p.num_q_blocks; qb += gridDim.x) {
            const QRange r = q_block_range(p, qb);
            if (r.b1 <= r.b0) continue;
            const uint32_t qs = qcount & 1u, qphase = (qcount >> 1) & 1u;
            ++qcount;
            if (!(ok = DG_WARP_WAIT(smem_u32(&bars->q_empty[qs]), qphase ^ 1u, wc, kWaitEmpty))) break;
            const uint32_t qbar = smem_u32(&bars->q_full[qs]);
            const uint32_t qdst = base + p.off_q + qs * p.q_stage_bytes;
            if (elect_one()) {
                mbar_arrive_expect_tx(qbar, p.n * p.head_dim + (SCALED ? p.n * 4u : 0u));
                tma_load_2d(&tm_q, qbar, qdst, 0, (int32_t)(qb * p.n));
                if (SCALED) tma_load_2d(&tm_qsf, qbar, qdst + p.q_sf_off, (int32_t)(qb * p.n), 0);
            }
            __syncwarp();
            for (uint32_t kb = r.b0; kb < r.b1; ++kb) {
                if (!(ok = DG_WARP_WAIT(smem_u32(&bars->kv_empty[stage]), phase ^ 1u, wc, kWaitEmpty))) break;
                const uint32_t bar = smem_u32(&bars->kv_full[stage]);
                const uint32_t dst = base + p.off_kv + stage * p.kv_stage_bytes;
                if (elect_one()) {
                    mbar_arrive_expect_tx(bar, kMqaBlockKv * p.head_dim + (SCALED ? kMqaBlockKv * 4u : 0u));
                    tma_load_2d(&tm_kv, bar, dst, 0, (int32_t)(kb * kMqaBlockKv));
                    if (SCALED) tma_load_2d(&tm_kvsf, bar, dst + p.kv_sf_off, (int32_t)(kb * kMqaBlockKv), 0);
                }
                __syncwarp();
                if (++stage == p.kv_stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ===================================================== MMA issuer (warp-converged, one lane issues)
        uint32_t stage = 0, phase = 0, qcount = 0, acount = 0;
        const uint32_t idesc = SCALED ? make_idesc_bs(0u, 0u, kMqaBlockKv, p.n) : make_idesc_f8(kMqaBlockKv, p.n);
        bool ok = true;
        for (uint32_t qb = blockIdx.x; ok && qb < p.num_q_blocks; qb += gridDim.x) {
            const QRange r = q_block_range(p, qb);
            if (r.b1 <= r.b0) continue;
            const uint32_t qs = qcount & 1u, qphase = (qcount >> 1) & 1u;
            ++qcount;
            if (!(ok = DG_WARP_WAIT(smem_u32(&bars->q_full[qs]), qphase, wc, kWaitFull))) break;
            if (SCALED && !(ok = DG_WARP_WAIT(smem_u32(&bars->q_ready[qs]), qphase, wc, kWaitSfReady))) break;
            tc_fence_after();
            const uint32_t qaddr = base + p.off_q + qs * p.q_stage_bytes;
            const uint64_t q_desc = make_smem_desc(qaddr, p.sbo, 0, p.layout);
            if (SCALED) {
                if (elect_one()) {
                    for (uint32_t c = 0; c < (p.n + 127u) / 128u; ++c)
                        tc_cp_32x128b_warpx4(tmem + kMqaSfbCol + c * 4u, make_sf_desc(qaddr + p.q_sf_off + c * 512u));
                }
                __syncwarp();
            }
            for (uint32_t kb = r.b0; kb < r.b1; ++kb) {
                const uint32_t as = acount & 1u, aphase = (acount >> 1) & 1u;
                ++acount;
                if (!(ok = DG_WARP_WAIT(smem_u32(&bars->kv_full[stage]), phase, wc, kWaitFull))) break;
                if (SCALED && !(ok = DG_WARP_WAIT(smem_u32(&bars->kv_ready[stage]), phase, wc, kWaitSfReady))) break;
                if (!(ok = DG_WARP_WAIT(smem_u32(&bars->tmem_empty[as]), aphase ^ 1u, wc, kWaitTmemEmpty))) break;
                tc_fence_after();
                const uint32_t kaddr = base + p.off_kv + stage * p.kv_stage_bytes;
                const uint64_t kv_desc = make_smem_desc(kaddr, p.sbo, 0, p.layout);
                const uint32_t d_tmem = tmem + as * acc_stride;
                if (elect_one()) {
                if (SCALED) tc_cp_32x128b_warpx4(tmem + kMqaSfaCol, make_sf_desc(kaddr + p.kv_sf_off));
                for (uint32_t k = 0; k < num_mma; ++k) {
                    if (SCALED)
                        tc_mma_mxf8(d_tmem, kv_desc + 2u * k, q_desc + 2u * k, idesc_with_sf_ids(idesc, k, k), k != 0u,
                                    tmem + kMqaSfaCol, tmem + kMqaSfbCol);
                    else
                        tc_mma_f8(d_tmem, kv_desc + 2u * k, q_desc + 2u * k, idesc, k != 0u);
                }
                tc_commit(smem_u32(&bars->kv_empty[stage]));
                tc_commit(smem_u32(&bars->tmem_full[as]));
                if (kb + 1 == r.b1) tc_commit(smem_u32(&bars->q_empty[qs]));
                }
                __syncwarp();
                if (++stage == p.kv_stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 2 && SCALED) {
        // ===================================================== SF transposer (ue8m0 contract)
        uint32_t stage = 0, phase = 0, qcount = 0;
        bool ok = true;
        auto transpose128 = [&](uint32_t* q) {
            const uint32_t v0 = q[lane], v1 = q[32 + lane], v2 = q[64 + lane], v3 = q[96 + lane];
            __syncwarp();
            *reinterpret_cast<uint4*>(q + lane * 4u) = make_uint4(v0, v1, v2, v3);
        };
        for (uint32_t qb = blockIdx.x; ok && qb < p.num_q_blocks; qb += gridDim.x) {
            const QRange r = q_block_range(p, qb);
            if (r.b1 <= r.b0) continue;
            const uint32_t qs = qcount & 1u, qphase = (qcount >> 1) & 1u;
            ++qcount;
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->q_full[qs]), qphase, wc, kWaitFull));
            if (!ok) break;
            uint32_t* qsf = reinterpret_cast<uint32_t*>(base_ptr + p.off_q + qs * p.q_stage_bytes + p.q_sf_off);
            for (uint32_t c = 0; c < (p.n + 127u) / 128u; ++c) transpose128(qsf + c * 128u);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->q_ready[qs]));
            for (uint32_t kb = r.b0; kb < r.b1; ++kb) {
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->kv_full[stage]), phase, wc, kWaitFull));
                if (!ok) break;
                transpose128(reinterpret_cast<uint32_t*>(base_ptr + p.off_kv + stage * p.kv_stage_bytes + p.kv_sf_off));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->kv_ready[stage]));
                if (++stage == p.kv_stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp >= 4) {
        // ===================================================== epilogue (2 or 4 warpgroups)
        const uint32_t et = threadIdx.x - 128u;
        const uint32_t wg = et >> 7;                  // which share of the query block
        const uint32_t quarter = warp & 3u;           // TMEM lane quarter of this warp
        const uint32_t q_per_wg = p.block_q / p.ep_groups;
        const uint32_t units_per_q = p.num_heads / 16u;
        const uint32_t nunits = q_per_wg * units_per_q;        // 16-column TMEM loads per kv block
        const uint32_t q_first = wg * q_per_wg;
        const uint32_t col_base = q_first * p.num_heads;
        uint32_t qcount = 0, acount = 0;
        bool ok = true;
        for (uint32_t qb = blockIdx.x; ok && qb < p.num_q_blocks; qb += gridDim.x) {
            const QRange r = q_block_range(p, qb);
            if (r.b1 <= r.b0) continue;
            const uint32_t wb = qcount & 1u, wphase = (qcount >> 1) & 1u;
            float* w = w_smem + wb * p.n;
            ++qcount;
            if (et < p.n) {
                const uint32_t q = qb * p.block_q + et / p.num_heads;
                float v = 0.f;
                if (q < p.num_tokens) {
                    const size_t idx = (size_t)q * p.num_heads + et % p.num_heads;
                    v = SCALED ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.weights)[idx])
                               : reinterpret_cast<const float*>(p.weights)[idx];
                }
                w[et] = 0.5f * v;      // see the epilogue loop: relu(x) * w = (x + |x|) * (w / 2)
            }
            // the kv windows of the block's queries travel with the weights: the reduction loop reads
            // them from shared memory instead of waiting on two global loads per query and kv block
            uint32_t* win = win_smem + wb * 32u;
            if (et < p.block_q) {
                const uint32_t q = qb * p.block_q + et;
                win[et] = q < p.num_tokens ? __ldg(p.ks + q) : 0u;
                win[16u + et] = q < p.num_tokens ? min(__ldg(p.ke + q), p.num_kv) : 0u;
            }
            // The two buffers alternate, and no warp can run more than one query block ahead of
            // the slowest one (it waits here), so a buffer is never rewritten while still read.
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->w_full[wb]));
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->w_full[wb]), wphase, wc, kWaitWeights));
            if (!ok) break;
            for (uint32_t kb = r.b0; kb < r.b1; ++kb) {
                const uint32_t as = acount & 1u, aphase = (acount >> 1) & 1u;
                ++acount;
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->tmem_full[as]), aphase, wc, kWaitTmemFull));
                if (!ok) break;
                tc_fence_after();
                const uint32_t j = kb * kMqaBlockKv + quarter * 32u + lane;
                float scale = 1.f;
                if (!SCALED) scale = j < p.num_kv ? __ldg(p.kv_scale + j) : 0.f;
                const uint32_t taddr = tmem + ((quarter * 32u) << 16) + as * acc_stride + col_base;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;    // four partial sums of the current query
                uint32_t unit_in_q = 0, q_done = 0;              // position inside this warp's share of the query block

                // The reduction runs in units of 16 columns.  relu(x) * w is computed as
                // (x + |x|) * (w / 2): the addition takes |x| as a source modifier and runs on the FMA
                // pipe at full rate, where a max would go through the half-rate ALU pipe; both
                // scalings are by powers of two, so the result is the same bit for bit (the weights in
                // shared memory are already halved).  The TMEM load and the four weight vectors of
                // unit u + 1 are requested before the arithmetic of unit u starts, so that neither the
                // tensor-memory latency nor the shared-memory latency sits between dependent
                // instructions; 16-column units keep both register sets inside the 102 registers a
                // 640-thread block leaves per thread.
                auto load_w = [&](float4 (&dst)[4], uint32_t u) {
                    const float4* w4 = reinterpret_cast<const float4*>(w + col_base + u * 16u);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) dst[i] = w4[i];
                };
                auto consume = [&](const uint32_t (&v)[16], const float4 (&ww)[4]) {
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const float x0 = __uint_as_float(v[4 * i]), x1 = __uint_as_float(v[4 * i + 1]);
                        const float x2 = __uint_as_float(v[4 * i + 2]), x3 = __uint_as_float(v[4 * i + 3]);
                        a0 = fmaf(x0 + fabsf(x0), ww[i].x, a0);
                        a1 = fmaf(x1 + fabsf(x1), ww[i].y, a1);
                        a2 = fmaf(x2 + fabsf(x2), ww[i].z, a2);
                        a3 = fmaf(x3 + fabsf(x3), ww[i].w, a3);
                    }
                    if (++unit_in_q == units_per_q) {
                        const uint32_t qi = q_first + q_done;        // index inside the query block
                        const uint32_t s = win[qi], e = win[16u + qi];   // e = 0 for queries past the end
                        if (j >= s && j < e) {
                            const float val = ((a0 + a1) + (a2 + a3)) * scale;
                            const size_t o = (size_t)(qb * p.block_q + qi) * p.logits_stride + (j - s);
                            if (SCALED) reinterpret_cast<__nv_bfloat16*>(p.logits)[o] = __float2bfloat16_rn(val);
                            else reinterpret_cast<float*>(p.logits)[o] = val;
                        }
                        a0 = a1 = a2 = a3 = 0.f;
                        unit_in_q = 0;
                        ++q_done;
                    }
                };
                auto release = [&]() {
                    // every column of this stage is in registers: hand the TMEM stage back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[as]));
                };
                uint32_t va[16], vb[16];
                float4 wa[4], wb4[4];
                __syncwarp();
                tmem_ld_x16(taddr, va);
                load_w(wa, 0);
                tmem_ld_wait();
                for (uint32_t u = 0; u < nunits; u += 2) {
                    if (u + 1 < nunits) { tmem_ld_x16(taddr + (u + 1) * 16u, vb); load_w(wb4, u + 1); } else release();
                    consume(va, wa);
                    if (u + 1 < nunits) {
                        tmem_ld_wait();
                        if (u + 2 < nunits) { tmem_ld_x16(taddr + (u + 2) * 16u, va); load_w(wa, u + 2); } else release();
                        consume(vb, wb4);
                        if (u + 2 < nunits) tmem_ld_wait();
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ============================================================================ host side
static int32_t check_mqa_common(uint32_t num_tokens, uint32_t num_kv, uint32_t num_heads, uint32_t head_dim,
                                uint32_t logits_stride, const void* ks, const void* ke, const void* w, const void* logits) {
    if (!ks || !ke || !w || !logits) return fail(DG_ERR_INVALID_ARG, "mqa_logits: null buffer");
    if (num_tokens == 0 || num_kv == 0) return fail(DG_ERR_INVALID_ARG, "mqa_logits: empty problem");
    // deepgemm/src/api.rs:1639-1650
    if (head_dim % 32 != 0 || head_dim > 128 || head_dim == 96 || head_dim == 0)
        return fail(DG_ERR_INVALID_ARG, "head_dim must be 32/64/128");
    if (num_heads % 4 != 0 || num_heads > 256 || num_heads == 0)
        return fail(DG_ERR_INVALID_ARG, "num_heads must be a multiple of 4 (<= 256)");
    if (logits_stride == 0) return fail(DG_ERR_INVALID_ARG, "mqa_logits: logits_stride must be positive");
    return DG_OK;
}

template <bool SCALED>
static int32_t run_mqa(const void* q, const void* kv, const uint32_t* q_sf, uint32_t q_sf_cols, const uint32_t* kv_sf,
                       uint32_t kv_sf_cols, const float* kv_scale, const void* weights, const uint32_t* ks,
                       const uint32_t* ke, uint32_t num_tokens, uint32_t num_kv, uint32_t num_heads, uint32_t head_dim,
                       void* logits, uint32_t logits_stride, void* stream) {
    // Tiling: the query block holds an even number of queries so that the two epilogue
    // warpgroups split it; heads must come in whole 32-column TMEM loads.
    const uint32_t max_n = SCALED ? 192u : 256u;
    if (num_heads % 32 != 0 || 2 * num_heads > max_n)
        return fail(DG_ERR_UNSUPPORTED, "mqa_logits: this build handles num_heads in {32, 64%s}, got %u",
                    SCALED ? ", 96" : ", 96, 128", num_heads);
    const DeviceInfo* dev;
    int32_t st = current_device(&dev);
    if (st != DG_OK) return st;
    MqaParams p{};
    p.num_tokens = num_tokens; p.num_kv = num_kv; p.num_heads = num_heads; p.head_dim = head_dim;
    p.block_q = 2 * (max_n / 2 / num_heads);
    p.n = p.block_q * num_heads;
    p.ep_groups = p.block_q % 4 == 0 ? 4u : 2u;
    p.num_q_blocks = ceil_div(num_tokens, p.block_q);
    p.sbo = 8 * head_dim;
    p.layout = head_dim == 128 ? 2u : head_dim == 64 ? 4u : 6u;
    const CUtensorMapSwizzle sw = head_dim == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : head_dim == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    p.off_w = 1024;
    p.off_q = 1024 + 2048;
    p.q_sf_off = align_up(p.n * head_dim, 1024);
    p.q_stage_bytes = p.q_sf_off + (SCALED ? 1024u : 0u);
    p.off_kv = p.off_q + 2 * p.q_stage_bytes;
    p.kv_sf_off = kMqaBlockKv * head_dim;
    p.kv_stage_bytes = align_up(p.kv_sf_off + (SCALED ? 512u : 0u), 1024);
    const uint32_t budget = (uint32_t)dev->smem_optin - 1024u;
    uint32_t stages = (budget - p.off_kv) / p.kv_stage_bytes;
    if (stages > kMqaMaxKvStages) stages = kMqaMaxKvStages;
    if (stages < 2) return fail(DG_ERR_RUNTIME, "mqa_logits: shared memory budget too small");
    p.kv_stages = stages;
    const uint32_t smem_bytes = 1024u + p.off_kv + stages * p.kv_stage_bytes;
    p.logits_stride = logits_stride;
    p.ks = ks; p.ke = ke; p.kv_scale = kv_scale; p.weights = weights; p.logits = logits;
    p.status = dev->status;

    CUtensorMap tq, tkv, tqsf, tkvsf;
    if ((st = make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, head_dim, (uint64_t)num_tokens * num_heads, head_dim,
                           head_dim, p.n, sw, "q")) != DG_OK) return st;
    if ((st = make_tmap_2d(&tkv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, kv, head_dim, num_kv, head_dim, head_dim, kMqaBlockKv,
                           sw, "kv")) != DG_OK) return st;
    if (SCALED) {
        if ((st = make_tmap_2d(&tqsf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, q_sf, q_sf_cols, 1, (uint64_t)q_sf_cols * 4, p.n, 1,
                               CU_TENSOR_MAP_SWIZZLE_NONE, "q_sf")) != DG_OK) return st;
        if ((st = make_tmap_2d(&tkvsf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, kv_sf, kv_sf_cols, 1, (uint64_t)kv_sf_cols * 4,
                               kMqaBlockKv, 1, CU_TENSOR_MAP_SWIZZLE_NONE, "kv_sf")) != DG_OK) return st;
    } else {
        tqsf = tq; tkvsf = tkv;
    }
    auto* fn = mqa_logits_kernel<SCALED>;
    DG_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    uint32_t grid = (uint32_t)dev->sm_count;
    if (p.num_q_blocks < grid) grid = p.num_q_blocks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(128u + 128u * p.ep_groups);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // set-up overlaps the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DG_CUDA_CHECK(cudaLaunchKernelEx(&cfg, fn, tq, tkv, tqsf, tkvsf, p));
    dg::note_launch();
    return DG_OK;
}

}  // namespace dg

extern "C" {

int32_t dg_mqa_logits_f32(const void* q, const void* kv, const float* kv_scale, const float* weights,
                          const uint32_t* cu_k_start, const uint32_t* cu_k_end, uint32_t num_tokens,
                          uint32_t num_kv_tokens, uint32_t num_heads, uint32_t head_dim, float* logits,
                          uint32_t logits_stride, void* stream) {
    if (!q || !kv || !kv_scale) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: null buffer");
    int32_t st = dg::check_mqa_common(num_tokens, num_kv_tokens, num_heads, head_dim, logits_stride, cu_k_start, cu_k_end,
                                      weights, logits);
    if (st != DG_OK) return st;
    return dg::run_mqa<false>(q, kv, nullptr, 0, nullptr, 0, kv_scale, weights, cu_k_start, cu_k_end, num_tokens,
                              num_kv_tokens, num_heads, head_dim, logits, logits_stride, stream);
}

int32_t dg_mqa_logits(const dg_operand_t* q, const dg_operand_t* kv, const void* weights_bf16, const uint32_t* cu_k_start,
                      const uint32_t* cu_k_end, uint32_t num_tokens, uint32_t num_kv_tokens, uint32_t num_heads,
                      uint32_t head_dim, void* logits_bf16, uint32_t logits_stride, void* stream) {
    if (!q || !kv || !q->data || !kv->data) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: null operand");
    if (q->dtype != kv->dtype) return dg::fail(DG_ERR_INVALID_ARG, "Q/KV dtype mismatch");
    int32_t st = dg::check_mqa_common(num_tokens, num_kv_tokens, num_heads, head_dim, logits_stride, cu_k_start, cu_k_end,
                                      weights_bf16, logits_bf16);
    if (st != DG_OK) return st;
    if (q->dtype == DG_FP4) {
        if (head_dim != 64 && head_dim != 128) return dg::fail(DG_ERR_INVALID_ARG, "MXFP4 requires head_dim 64/128");
        return dg::fail(DG_ERR_UNSUPPORTED, "mqa_logits: the MXFP4 flavour is not built");
    }
    if (q->dtype != DG_FP8) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: q/kv must be FP8 or FP4");
    if (!q->sf.data || !kv->sf.data) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: q and kv require scale factors");
    if (q->sf.gran != 32 || kv->sf.gran != 32) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: scale granularity must be 32");
    if (q->rows != num_tokens * num_heads || q->k != head_dim || kv->rows != num_kv_tokens || kv->k != head_dim)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: q must be [num_tokens*num_heads, head_dim] and kv [num_kv_tokens, head_dim]");
    if (q->major != DG_MAJOR_K || kv->major != DG_MAJOR_K || q->outer_stride != head_dim || kv->outer_stride != head_dim)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: q and kv must be dense K-major rows (outer_stride == head_dim)");
    if (q->sf.cols < dg::align_up(q->rows, 4) || kv->sf.cols < dg::align_up(kv->rows, 4) || q->sf.rows < 1 || kv->sf.rows < 1)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: scale-factor tensors too small");
    return dg::run_mqa<true>(q->data, kv->data, q->sf.data, q->sf.cols, kv->sf.data, kv->sf.cols, nullptr, weights_bf16,
                             cu_k_start, cu_k_end, num_tokens, num_kv_tokens, num_heads, head_dim, logits_bf16,
                             logits_stride, stream);
}

}  // extern "C"
