// MQA logits (MLA lightning indexer) for sm_100a:
//   logits[i, j] = s_kv[j] * sum_h w[i,h] * relu(<q[i,h,:], kv[j,:]>),  j in [ks[i], min(ke[i], S))
// stored compressed at column j - ks[i] of row i.
//
// Contracts of the reference that share this kernel:
//   fp32  (deepgemm/src/api_sm90_mqa.rs:5-31): raw E4M3 q, E4M3 kv with one f32 scale per kv
//         token, f32 weights, f32 logits           -> tcgen05.mma kind::f8f6f4
//   ue8m0 (api::mqa_logits, deepgemm/src/api.rs:1614-1745; device side
//         deepgemm/kernels/mqa_logits_sm100.cu:514-1084): UE8M0 scales per 32 along head_dim on
//         q and kv, bf16 weights, bf16 logits; FP8 codes (kind::mxf8f6f4.block_scale) or packed FP4
//         codes (kind::mxf4.block_scale.block32)
//   paged (api::mqa_logits_paged, api.rs:1752-1941; scheduler and metadata kernel
//         mqa_logits_sm100.cu:110-492): the ue8m0 contract over a paged KV cache for decode --
//         query tokens carry a request id and a context length, the kv tokens of a request are
//         found through its row of the block table
// Numerical contract: mqa_logits_ref of the golden model (deepgemm/src/golden.rs:469-501), within
// calc_diff <= 1e-3.
//
// The contraction runs with the 128 kv tokens of a block on the UMMA M side (TMEM lanes) and
// the (query, head) pairs of a query block on the N side, so one epilogue thread owns one kv
// token and a warp stores 32 consecutive columns of a logits row.
//   warp 0      TMA producer (Q tile per task, KV blocks streamed through a ring; paged: page by page)
//   warp 1      MMA issuer (scores into one of two accumulator stages in TMEM)
//   warp 2      TMEM owner; ue8m0 contracts: scale factors into the layout tcgen05.cp needs
//   warps 4-..  epilogue warpgroups: relu(x) * w accumulated in f32 per thread, every warpgroup reducing its
//               share of the query block's columns.  With one query of 64 or 128 heads per warpgroup the query's
//               weights stay in registers for all kv blocks of a task (the role warps hand registers over for
//               that): as broadcast loads from shared memory inside the kv loop they took as much of the shared
//               memory bandwidth as the tensor core needs for its operands, and that bandwidth, not the
//               instruction stream, bounded the kernel
// (A head reduction on the tensor cores -- ReLU'd scores written back to tensor memory as bf16 and multiplied
// with a block-diagonal weight tile by a second MMA whose A operand is read from tensor memory -- was built
// and measured on this kernel: correct, but twice as slow, because the 16 narrow MMAs it adds per kv block cost
// more tensor-pipe time than the reduction costs the CUDA cores.)
// The epilogue warpgroups of this file's kernels run under a register limit raised inside the kernel; code under
// such a limit cannot call functions, so the slow path of the bounded waits is inlined here.
#define DG_WAIT_SLOW_ATTR __forceinline__
#include "host.h"
#include "ptx.cuh"

#include <cstdlib>

namespace dg {

constexpr uint32_t kMqaBlockKv = 128;
constexpr uint32_t kMqaMaxKvStages = 10;
constexpr uint32_t kMqaMaxThreads = 640;   // 4 role warps + up to 4 epilogue warpgroups
// One query of 16 * NUN heads per warpgroup (NUN = 4: 4 queries, 640 threads; NUN = 8: 2 queries, 384 threads):
// registers per thread at launch (what the block size leaves, in steps of 8), what the role warps keep, and
// what an epilogue thread then gets (8 * NUN packed weight pairs, 16 scores, about 30 of state).
__host__ __device__ constexpr uint32_t mqa_threads(uint32_t nun) { return nun == 8u ? 384u : kMqaMaxThreads; }
__host__ __device__ constexpr uint32_t mqa_launch_regs(uint32_t nun) { return (65536u / mqa_threads(nun)) & ~7u; }
constexpr uint32_t kMqaRoleRegs = 40;
__host__ __device__ constexpr uint32_t mqa_epilogue_regs(uint32_t nun) {
    return ((mqa_launch_regs(nun) * mqa_threads(nun) - 128u * kMqaRoleRegs) / (mqa_threads(nun) - 128u)) & ~7u;
}
static_assert(mqa_launch_regs(4) == 96 && mqa_epilogue_regs(4) == 104, "register budget of the 64-head variant");
static_assert(mqa_launch_regs(8) == 168 && mqa_epilogue_regs(8) == 232, "register budget of the 128-head variant");
constexpr uint32_t kMqaSfaCol = 448;       // ue8m0 contracts only: the accumulators are <= 192 wide
constexpr uint32_t kMqaSfbCol = 452;

struct MqaParams {
    uint32_t num_tokens, num_kv, num_heads, head_dim;
    uint32_t block_q, n, n_mma;   // n = block_q * num_heads score columns, n_mma = n rounded up to the MMA's granule
    uint32_t ep_groups;           // epilogue warpgroups; each reduces block_q / ep_groups queries
    uint32_t unit;                // columns per TMEM load (16, or 4 for head counts not divisible by 16)
    uint32_t num_q_blocks;
    uint32_t kv_splits;           // contiguous kv: pieces a query block's kv range is cut into (few query blocks, many SMs)
    uint32_t kv_stages, kv_stage_bytes, q_stage_bytes;
    uint32_t off_w, off_q, off_kv;  // offsets from the 1024-aligned base
    uint32_t kv_sf_off, q_sf_off;   // SF words inside a kv / q stage (ue8m0 contracts)
    uint32_t row_bytes;             // bytes of one q / kv row (head_dim, or head_dim / 2 for FP4)
    uint32_t sbo;                   // 8-row group pitch of the swizzled tiles
    uint32_t layout;                // UMMA layout type of the tiles
    uint32_t num_mma;               // MMAs per kv block
    uint32_t idesc;                 // instruction descriptor of the score MMA
    uint32_t acc_stride;            // TMEM columns between the two accumulator stages
    uint32_t logits_stride;
    const uint32_t* ks;
    const uint32_t* ke;
    const float* kv_scale;          // fp32 contract
    const void* weights;            // f32 (fp32 contract) or bf16 (ue8m0 contracts)
    void* logits;
    uint32_t* status;
    // paged KV
    uint32_t page_kv, boxes_per_block, box_rows;   // kv rows per page; TMA boxes per 128-token block and their height
    const uint32_t* kv_sf;          // scale words of the cache, one per token in page order
    const uint32_t* context_lens;
    const uint32_t* block_table;
    uint32_t block_table_stride;
    const uint32_t* cum;            // [num_tokens + 1] kv blocks of the query blocks that start before a token
    const uint32_t* qb_tokens;      // [num_tokens] tokens of the query block that starts here, 0 elsewhere
    const uint32_t* req_first;      // [num_tokens] first token of the token's request
};

struct __align__(8) MqaBarriers {
    uint64_t kv_full[kMqaMaxKvStages];
    uint64_t kv_ready[kMqaMaxKvStages];   // ue8m0: scale factors in place
    uint64_t kv_empty[kMqaMaxKvStages];
    uint64_t q_full[2], q_ready[2], q_empty[2];
    uint64_t tmem_full[2], tmem_empty[2];
    uint64_t w_full[2];                   // weights of a task staged by the epilogue warps
    uint32_t tmem_base;
    uint32_t abort;
};

// One unit of work, identical in every role: `nq` queries starting at token q0 against the kv blocks
// [kb0, kb1) (128 tokens each; paged: blocks of the request's own token order).
struct MqaTask { uint32_t q0, nq, kb0, kb1, table_row; };

// Contiguous KV: query block qb = blockIdx.x, + gridDim.x, ...; its kv range follows from the windows.
// Paged KV: every CTA takes an equal share of all (query block, kv block) pairs, cut out of the list
// the metadata kernel prepared; a share may begin and end in the middle of a query block's kv range.
template <bool PAGED>
struct MqaTasks {
    uint32_t qb;                // contiguous
    uint32_t t, u, u_end;       // paged: next query block's first token, next unit, end of this CTA's share
    __device__ explicit MqaTasks(const MqaParams& p) : qb(blockIdx.x), t(0), u(0), u_end(0) {
        if (PAGED) {
            const uint64_t total = __ldg(p.cum + p.num_tokens);
            u = (uint32_t)(total * blockIdx.x / gridDim.x);
            u_end = (uint32_t)(total * (blockIdx.x + 1) / gridDim.x);
            // the query block that holds unit u: the first token i with cum[i + 1] > u
            uint32_t lo = 0, hi = p.num_tokens;
            while (lo < hi) {
                const uint32_t mid = (lo + hi) >> 1;
                if (__ldg(p.cum + mid + 1) > u) hi = mid; else lo = mid + 1;
            }
            t = lo;
        }
    }
    __device__ bool next(const MqaParams& p, MqaTask& k) {
        if (PAGED) {
            while (u < u_end && t < p.num_tokens) {
                const uint32_t c0 = __ldg(p.cum + t), c1 = __ldg(p.cum + t + 1);
                const uint32_t nq = __ldg(p.qb_tokens + t);
                if (c1 <= u || nq == 0) { t += nq ? nq : 1u; continue; }   // a query block without kv tokens, or not a start
                k.q0 = t; k.nq = nq;
                k.kb0 = u - c0;
                k.kb1 = min(c1, u_end) - c0;
                k.table_row = __ldg(p.req_first + t);
                u = min(c1, u_end);
                if (u == c1) t += nq;
                return true;
            }
            return false;
        }
        while (qb < p.num_q_blocks * p.kv_splits) {
            const uint32_t b = qb / p.kv_splits, piece = qb - b * p.kv_splits;
            qb += gridDim.x;
            uint32_t lo = 0xffffffffu, hi = 0;
            for (uint32_t i = 0; i < p.block_q; ++i) {
                const uint32_t q = b * p.block_q + i;
                if (q < p.num_tokens) {
                    const uint32_t s = __ldg(p.ks + q), e = min(__ldg(p.ke + q), p.num_kv);
                    if (s < e) { lo = min(lo, s); hi = max(hi, e); }
                }
            }
            if (hi <= lo) continue;
            k.q0 = b * p.block_q; k.nq = min(p.block_q, p.num_tokens - k.q0);
            k.kb0 = lo / kMqaBlockKv; k.kb1 = (hi + kMqaBlockKv - 1) / kMqaBlockKv;
            k.table_row = 0;
            if (p.kv_splits > 1u) {
                // the pieces of a query block write disjoint columns of its logits rows: no reduction between them
                const uint32_t len = (k.kb1 - k.kb0 + p.kv_splits - 1u) / p.kv_splits;
                k.kb0 += piece * len;
                k.kb1 = min(k.kb1, k.kb0 + len);
                if (k.kb0 >= k.kb1) continue;
            }
            return true;
        }
        return false;
    }
};

// Row of the paged cache that holds token `tok` (request order) of the request whose table row is given;
// tokens past the table's width or pages outside the cache read row 0 (they lie beyond every context
// length and are masked by the epilogue).
__device__ __forceinline__ uint32_t paged_row(const MqaParams& p, uint32_t table_row, uint32_t tok, uint32_t span) {
    const uint32_t pg = tok / p.page_kv;
    const uint32_t page = pg < p.block_table_stride ? __ldg(p.block_table + (size_t)table_row * p.block_table_stride + pg) : 0u;
    const uint32_t row = page * p.page_kv + tok % p.page_kv;
    return row + span <= p.num_kv ? row : 0u;
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
__device__ __forceinline__ void tmem_ld_x4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
// Packed pairs of f32 (sm_100: one instruction, two FMAs).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ float lo_f32(uint64_t v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi_f32(uint64_t v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// max(x, 0) that keeps a NaN (as x + |x| would)
__device__ __forceinline__ float relu_nan(float x) {
    float r;
    asm("max.NaN.f32 %0, %1, 0f00000000;" : "=f"(r) : "f"(x));
    return r;
}
// SCALED: ue8m0 contracts (scale factors on q and kv, bf16 weights and logits); FP4: packed E2M1 codes;
// PAGED: kv through a block table, work from the metadata kernel.
// U4: head counts that are not a multiple of 16 (their 4-column reduction loop is a variant of its own: as a
// run-time branch beside the 16-column loop it cost the common case 4 %).
// QPW: queries per warpgroup of the NUN variants (their NUN units are QPW queries of 16 * NUN / QPW heads).
// NUN: 16-column units a warpgroup reduces per kv block when that is known at compile time (4 / 8 = one query of
// 64 / 128 heads per warpgroup: the unit loop is then straight-line code without counters), 0 = any.
template <bool SCALED, bool FP4, bool PAGED, bool U4 = false, uint32_t NUN = 0, uint32_t QPW = 1>
__global__ void __launch_bounds__(mqa_threads(NUN), 1)
mqa_logits_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                  const __grid_constant__ CUtensorMap tm_qsf, const __grid_constant__ CUtensorMap tm_kvsf,
                  const MqaParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base = (raw_u32 + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_u32);
    MqaBarriers* bars = reinterpret_cast<MqaBarriers*>(base_ptr);
    float* w_smem = reinterpret_cast<float*>(base_ptr + p.off_w);      // [2][n] halved weights
    uint32_t* win_smem = reinterpret_cast<uint32_t*>(base_ptr + 512);  // [2][2][16]: ks / ke of the queries of a task
    static_assert(sizeof(MqaBarriers) <= 512, "barrier block overlaps the window table");
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const WaitCtx wc{p.status, &bars->abort};
    const uint32_t ep_warps = 4u * p.ep_groups;

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
            mbar_init(smem_u32(&bars->w_full[s]), ep_warps);
            mbar_init(smem_u32(&bars->tmem_full[s]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[s]), ep_warps);
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
    griddep_wait();                 // the kernel before this one in the stream produced q / kv / weights / the task list
    griddep_launch_dependents();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
    const uint32_t acc_stride = p.acc_stride;
    const uint32_t kv_tx = kMqaBlockKv * p.row_bytes + ((SCALED && !PAGED) ? kMqaBlockKv * 4u : 0u);

    if (warp < 4) {
    if (NUN) reg_release<kMqaRoleRegs>();
    if (warp == 0) {
        // ===================================================== producer (warp-converged, one lane issues)
        uint32_t stage = 0, phase = 0, qcount = 0;
        bool ok = true;
        MqaTasks<PAGED> tasks(p);
        MqaTask k;
        while (ok && tasks.next(p, k)) {
            const uint32_t qs = qcount & 1u, qphase = (qcount >> 1) & 1u;
            ++qcount;
            if (!(ok = DG_WARP_WAIT(smem_u32(&bars->q_empty[qs]), qphase ^ 1u, wc, kWaitEmpty))) break;
            const uint32_t qbar = smem_u32(&bars->q_full[qs]);
            const uint32_t qdst = base + p.off_q + qs * p.q_stage_bytes;
            if (elect_one()) {
                // the box always holds block_q queries; rows of queries beyond the task's own are never stored
                mbar_arrive_expect_tx(qbar, p.n * p.row_bytes + (SCALED ? p.n * 4u : 0u));
                tma_load_2d(&tm_q, qbar, qdst, 0, (int32_t)(k.q0 * p.num_heads));
                if (SCALED) tma_load_2d(&tm_qsf, qbar, qdst + p.q_sf_off, (int32_t)(k.q0 * p.num_heads), 0);
            }
            __syncwarp();
            if (PAGED) {
                // A block of 128 tokens is a run of whole pages (or half / a quarter of a large page): lane i looks up
                // the page of box i in the block table.  The look-ups run four blocks ahead of the loads, and the
                // loop is unrolled by four so that an entry stays in its register, untouched, until its block comes
                // up: looked up inside the loop, each block cost the producer a trip to memory, and decode ran at
                // that latency instead of the cache's bandwidth.
                const uint32_t* trow = p.block_table + (size_t)k.table_row * p.block_table_stride;
                const uint32_t page_shift = (uint32_t)__ffs((int)p.page_kv) - 1u;      // the page size is a power of two
                auto tok_of = [&](uint32_t kbx) { return kbx * kMqaBlockKv + lane * p.box_rows; };
                auto page_of = [&](uint32_t kbx) -> uint32_t {
                    const uint32_t pg = tok_of(kbx) >> page_shift;
                    return (kbx < k.kb1 && lane < p.boxes_per_block && pg < p.block_table_stride) ? __ldg(trow + pg) : 0u;
                };
                uint32_t pq[4];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) pq[j] = page_of(k.kb0 + j);
                for (uint32_t kb4 = k.kb0; ok && kb4 < k.kb1; kb4 += 4u) {
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        const uint32_t kb = kb4 + j;
                        if (kb >= k.kb1) break;
                        if (!(ok = DG_WARP_WAIT(smem_u32(&bars->kv_empty[stage]), phase ^ 1u, wc, kWaitEmpty))) break;
                        const uint32_t bar = smem_u32(&bars->kv_full[stage]);
                        const uint32_t dst = base + p.off_kv + stage * p.kv_stage_bytes;
                        // rows past the table's width or pages outside the cache read row 0 (paged_row)
                        uint32_t row = pq[j] * p.page_kv + (tok_of(kb) & (p.page_kv - 1u));
                        if (row + p.box_rows > p.num_kv) row = 0u;
                        pq[j] = page_of(kb + 4u);
                        if (lane == 0) mbar_arrive_expect_tx(bar, kv_tx);
                        __syncwarp();
                        if (lane < p.boxes_per_block) tma_load_2d(&tm_kv, bar, dst + lane * p.box_rows * p.row_bytes, 0, (int32_t)row);
                        __syncwarp();
                        if (++stage == p.kv_stages) { stage = 0; phase ^= 1u; }
                    }
                }
                continue;
            }
            for (uint32_t kb = k.kb0; kb < k.kb1; ++kb) {
                if (!(ok = DG_WARP_WAIT(smem_u32(&bars->kv_empty[stage]), phase ^ 1u, wc, kWaitEmpty))) break;
                const uint32_t bar = smem_u32(&bars->kv_full[stage]);
                const uint32_t dst = base + p.off_kv + stage * p.kv_stage_bytes;
                if (elect_one()) {
                    mbar_arrive_expect_tx(bar, kv_tx);
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
        bool ok = true;
        MqaTasks<PAGED> tasks(p);
        MqaTask k;
        while (ok && tasks.next(p, k)) {
            const uint32_t qs = qcount & 1u, qphase = (qcount >> 1) & 1u;
            ++qcount;
            if (!(ok = DG_WARP_WAIT(smem_u32(&bars->q_full[qs]), qphase, wc, kWaitFull))) break;
            if (SCALED && !(ok = DG_WARP_WAIT(smem_u32(&bars->q_ready[qs]), qphase, wc, kWaitSfReady))) break;
            tc_fence_after();
            const uint32_t qaddr = base + p.off_q + qs * p.q_stage_bytes;
            const uint64_t q_desc = make_smem_desc(qaddr, p.sbo, 0, p.layout);
            bool q_sf_copied = false;
            // ue8m0 contracts: the kv loop of a task is run by one elected lane alone.  Warp-wide waits (a vote and a
            // re-convergence per barrier, three barriers per kv block, then the scale-factor copy) cost the issuer
            // more than the MMAs of a block take: 1380 -> 1690 TFLOPS on 4096 x 64 heads x 32768.  The fp32 contract
            // (two barriers, no copy) is 1.5 % faster with the warp-wide loop and keeps it.
            constexpr bool kLaneLoop = SCALED;
            const bool issuer = elect_one();
            const uint32_t issuer_lane = (uint32_t)__ffs(__ballot_sync(0xffffffffu, issuer)) - 1u;
            auto wait_on = [&](uint32_t bar, uint32_t parity, uint32_t site) -> bool {
                return kLaneLoop ? mbar_wait(bar, parity, wc, site) : (bool)DG_WARP_WAIT(bar, parity, wc, site);
            };
            if (!kLaneLoop || issuer) {
            for (uint32_t kb = k.kb0; ok && kb < k.kb1; ++kb) {
                if (!(ok = wait_on(smem_u32(&bars->kv_full[stage]), phase, kWaitFull))) break;
                if (SCALED && !(ok = wait_on(smem_u32(&bars->kv_ready[stage]), phase, kWaitSfReady))) break;
                const uint32_t kaddr = base + p.off_kv + stage * p.kv_stage_bytes;
                const uint64_t kv_desc = make_smem_desc(kaddr, p.sbo, 0, p.layout);
                const uint32_t as = acount & 1u, aphase = (acount >> 1) & 1u;
                ++acount;
                if (!(ok = wait_on(smem_u32(&bars->tmem_empty[as]), aphase ^ 1u, kWaitTmemEmpty))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem + as * acc_stride;
                if (kLaneLoop || elect_one()) {
                    if (SCALED) {
                        if (!q_sf_copied)    // the q scales of this task: in order behind every MMA that used the previous task's
                            for (uint32_t c = 0; c < (p.n + 127u) / 128u; ++c)
                                tc_cp_32x128b_warpx4(tmem + kMqaSfbCol + c * 4u, make_sf_desc(qaddr + p.q_sf_off + c * 512u));
                        tc_cp_32x128b_warpx4(tmem + kMqaSfaCol, make_sf_desc(kaddr + p.kv_sf_off));
                    }
                    for (uint32_t m = 0; m < p.num_mma; ++m) {
                        if (SCALED && FP4)      // 64 elements per MMA: half-word (m & 1) of the row's scale word
                            tc_mma_mxf4(d_tmem, kv_desc + 2u * m, q_desc + 2u * m, idesc_with_sf_ids(p.idesc, (m & 1u) * 2u, (m & 1u) * 2u),
                                        m != 0u, tmem + kMqaSfaCol, tmem + kMqaSfbCol);
                        else if (SCALED)
                            tc_mma_mxf8(d_tmem, kv_desc + 2u * m, q_desc + 2u * m, idesc_with_sf_ids(p.idesc, m, m), m != 0u,
                                        tmem + kMqaSfaCol, tmem + kMqaSfbCol);
                        else
                            tc_mma_f8(d_tmem, kv_desc + 2u * m, q_desc + 2u * m, p.idesc, m != 0u);
                    }
                    tc_commit(smem_u32(&bars->kv_empty[stage]));
                    tc_commit(smem_u32(&bars->tmem_full[as]));
                    if (kb + 1 == k.kb1) tc_commit(smem_u32(&bars->q_empty[qs]));
                }
                if (!kLaneLoop) __syncwarp();
                q_sf_copied = true;
                if (++stage == p.kv_stages) { stage = 0; phase ^= 1u; }
            }
            }
            if (kLaneLoop) {
                // the other lanes take over the issuer's position in the rings
                __syncwarp();
                stage = __shfl_sync(0xffffffffu, stage, issuer_lane);
                phase = __shfl_sync(0xffffffffu, phase, issuer_lane);
                acount = __shfl_sync(0xffffffffu, acount, issuer_lane);
                ok = __shfl_sync(0xffffffffu, (uint32_t)ok, issuer_lane) != 0u;
            }
        }
    } else if (warp == 2 && SCALED) {
        // ===================================================== scale factors (ue8m0 contracts)
        // tcgen05.cp wants the word of row 32 i + l at position 4 l + i.  Contiguous kv: the TMA load
        // brought the 128 words in row order, rewrite them in place.  Paged kv: the words are fetched
        // here, page by page with plain loads (a page's words may be fewer than a TMA box can address),
        // as soon as the stage is free, and stored in the final order directly.
        uint32_t stage = 0, phase = 0, qcount = 0;
        bool ok = true;
        auto transpose128 = [&](uint32_t* q) {
            const uint32_t v0 = q[lane], v1 = q[32 + lane], v2 = q[64 + lane], v3 = q[96 + lane];
            __syncwarp();
            *reinterpret_cast<uint4*>(q + lane * 4u) = make_uint4(v0, v1, v2, v3);
        };
        MqaTasks<PAGED> tasks(p);
        MqaTask k;
        while (ok && tasks.next(p, k)) {
            const uint32_t qs = qcount & 1u, qphase = (qcount >> 1) & 1u;
            ++qcount;
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->q_full[qs]), qphase, wc, kWaitFull));
            if (!ok) break;
            uint32_t* qsf = reinterpret_cast<uint32_t*>(base_ptr + p.off_q + qs * p.q_stage_bytes + p.q_sf_off);
            for (uint32_t c = 0; c < (p.n + 127u) / 128u; ++c) transpose128(qsf + c * 128u);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->q_ready[qs]));
            if (PAGED) {
                // Lane l fetches the words of tokens 4 l .. 4 l + 3 of a block: they lie in one page (pages hold a
                // multiple of four tokens), so it is one block-table entry and one 16-byte load.  Both run ahead
                // of the block that is written -- entries four blocks, words two -- in registers that are not touched
                // before their block comes up (the loop is unrolled by four for that): fetched inside the loop, one
                // after the other, they cost two trips to memory per block, and decode ran at that latency.
                const uint32_t* trow = p.block_table + (size_t)k.table_row * p.block_table_stride;
                const uint32_t page_shift = (uint32_t)__ffs((int)p.page_kv) - 1u;
                auto page_of = [&](uint32_t kbx) -> uint32_t {
                    const uint32_t pg = (kbx * kMqaBlockKv + 4u * lane) >> page_shift;
                    return (kbx < k.kb1 && pg < p.block_table_stride) ? __ldg(trow + pg) : 0u;
                };
                auto words_of = [&](uint32_t kbx, uint32_t page) -> uint4 {
                    uint32_t row = page * p.page_kv + ((kbx * kMqaBlockKv + 4u * lane) & (p.page_kv - 1u));
                    if (row + 4u > p.num_kv) row = 0u;       // tokens past the table or the cache: masked by the epilogue
                    return __ldg(reinterpret_cast<const uint4*>(p.kv_sf + row));
                };
                uint32_t pq[4];
                uint4 wq2[2];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) pq[j] = page_of(k.kb0 + j);
                wq2[0] = words_of(k.kb0, pq[0]);
                wq2[1] = words_of(k.kb0 + 1u, pq[1]);
                for (uint32_t kb4 = k.kb0; ok && kb4 < k.kb1; kb4 += 4u) {
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        const uint32_t kb = kb4 + j;
                        if (kb >= k.kb1) break;
                        const uint4 cur = wq2[j & 1u];
                        wq2[j & 1u] = words_of(kb + 2u, pq[(j + 2u) & 3u]);
                        pq[j] = page_of(kb + 4u);
                        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->kv_empty[stage]), phase ^ 1u, wc, kWaitEmpty));
                        if (!ok) break;
                        uint32_t* sf = reinterpret_cast<uint32_t*>(base_ptr + p.off_kv + stage * p.kv_stage_bytes + p.kv_sf_off);
                        // row r = 4 l + i of the block goes to position 4 (r % 32) + r / 32
                        const uint32_t hi = lane >> 3;
                        sf[4u * ((4u * lane + 0u) & 31u) + hi] = cur.x;
                        sf[4u * ((4u * lane + 1u) & 31u) + hi] = cur.y;
                        sf[4u * ((4u * lane + 2u) & 31u) + hi] = cur.z;
                        sf[4u * ((4u * lane + 3u) & 31u) + hi] = cur.w;
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars->kv_ready[stage]));
                        if (++stage == p.kv_stages) { stage = 0; phase ^= 1u; }
                    }
                }
                continue;
            }
            for (uint32_t kb = k.kb0; kb < k.kb1; ++kb) {
                uint32_t* sf = reinterpret_cast<uint32_t*>(base_ptr + p.off_kv + stage * p.kv_stage_bytes + p.kv_sf_off);
                {
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->kv_full[stage]), phase, wc, kWaitFull));
                    if (!ok) break;
                    transpose128(sf);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->kv_ready[stage]));
                if (++stage == p.kv_stages) { stage = 0; phase ^= 1u; }
            }
        }
    }
    } else {
        // ===================================================== epilogue warpgroups
        if (NUN) reg_acquire<mqa_epilogue_regs(NUN)>();
        const uint32_t et = threadIdx.x - 128u;
        const uint32_t wg = et >> 7;                  // warpgroup index
        const uint32_t quarter = warp & 3u;           // TMEM lane quarter of this warp
        uint32_t qcount = 0, acount = 0;
        bool ok = true;
        MqaTasks<PAGED> tasks(p);
        MqaTask k;

        // windows of a task's queries into shared memory (the first block_q epilogue threads)
        auto stage_windows = [&](uint32_t wb) {
            uint32_t* win = win_smem + wb * 32u;
            if (et < p.block_q) {
                const uint32_t q = k.q0 + et;
                const bool live = et < k.nq && q < p.num_tokens;
                uint32_t s = 0, e = 0;
                if (live) {
                    if (PAGED) e = min(__ldg(p.context_lens + q), p.block_table_stride * p.page_kv);
                    else { s = __ldg(p.ks + q); e = min(__ldg(p.ke + q), p.num_kv); }
                }
                win[et] = s;
                win[16u + et] = e;       // e = 0: nothing of this query is stored
            }
        };
        auto load_weight = [&](uint32_t q, uint32_t h) -> float {
            const size_t idx = (size_t)q * p.num_heads + h;
            return SCALED ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.weights)[idx])
                          : reinterpret_cast<const float*>(p.weights)[idx];
        };

        {
            const uint32_t q_per_wg = NUN ? QPW : p.block_q / p.ep_groups;
            const uint32_t units_per_q = NUN ? NUN / QPW : p.num_heads / (U4 ? 4u : 16u);
            const uint32_t nunits = NUN ? NUN : q_per_wg * units_per_q;        // TMEM loads per kv block
            const uint32_t q_first = wg * q_per_wg;
            const uint32_t col_base = q_first * p.num_heads;
            while (ok && tasks.next(p, k)) {
                const uint32_t wb = qcount & 1u, wphase = (qcount >> 1) & 1u;
                float* w = w_smem + wb * p.n;
                ++qcount;
                for (uint32_t c = et; c < p.n; c += 128u * p.ep_groups) {
                    const uint32_t qi = c / p.num_heads, q = k.q0 + qi;
                    float v = 0.f;
                    if (qi < k.nq && q < p.num_tokens) v = load_weight(q, c % p.num_heads);
                    w[c] = v;
                }
                // the kv windows of the task's queries travel with the weights: the reduction loop reads
                // them from shared memory instead of waiting on two global loads per query and kv block
                stage_windows(wb);
                const uint32_t* win = win_smem + wb * 32u;
                // The two buffers alternate, and no warp can run more than one task ahead of
                // the slowest one (it waits here), so a buffer is never rewritten while still read.
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->w_full[wb]));
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->w_full[wb]), wphase, wc, kWaitWeights));
                if (!ok) break;
                if (NUN) {
                    // QPW queries of 16 * NUN / QPW heads per warpgroup, NUN 16-column units per kv block.  The
                    // weights do not change over the kv blocks of the task: they are read from shared memory once,
                    // as the packed pairs the FMAs take, and stay in registers; with one query per warpgroup so do
                    // its window and the address of its logits row.  The kernel is bound by what the kv loop asks
                    // of the SM, so relu(x) * w costs 1.5 instructions per element there: a max on the ALU pipe and
                    // half of a packed FMA (fma.rn.f32x2, two accumulators per instruction; the sums are the same
                    // bit for bit as with scalar FMAs).  One 16-column TMEM load at a time: the other warps of the
                    // scheduler cover its latency, a second set of 16 registers would not fit.
                    constexpr uint32_t UPQ = NUN / QPW;       // units per query
                    const uint32_t s_fix = win[q_first], e_fix = win[16u + q_first];
                    const uint32_t span_fix = e_fix > s_fix ? e_fix - s_fix : 0u;       // length of the query's window
                    const size_t row = (size_t)(k.q0 + q_first) * p.logits_stride;
                    __nv_bfloat16* const out_bf16 = reinterpret_cast<__nv_bfloat16*>(p.logits) + row;
                    float* const out_f32 = reinterpret_cast<float*>(p.logits) + row;
                    const uint32_t lane_base = tmem + ((quarter * 32u) << 16) + col_base;
                    const uint32_t full0 = smem_u32(&bars->tmem_full[0]), empty0 = smem_u32(&bars->tmem_empty[0]);
                    uint64_t wp[NUN ? 8u * NUN : 1u];
#pragma unroll
                    for (uint32_t i = 0; i < 4u * NUN; ++i) {
                        const float4 w4 = reinterpret_cast<const float4*>(w + col_base)[i];
                        wp[2 * i] = pack_f32x2(w4.x, w4.y);
                        wp[2 * i + 1] = pack_f32x2(w4.z, w4.w);
                    }
                    uint32_t j = k.kb0 * kMqaBlockKv + quarter * 32u + lane;
                    // A warpgroup none of whose queries the task has (decode: one or two tokens of a request in a block
                    // of three or four) only hands the accumulator stages back; its issue slots go to the others.
                    // (A loop of its own: as a branch inside the reduction loop below it cost that loop 17 %.)
                    if (PAGED && q_first >= k.nq) {
                        for (uint32_t kb = k.kb0; kb < k.kb1; ++kb) {
                            const uint32_t as = acount & 1u, aphase = (acount >> 1) & 1u;
                            ++acount;
                            ok = __all_sync(0xffffffffu, mbar_wait(full0 + as * 8u, aphase, wc, kWaitTmemFull));
                            if (!ok) break;
                            tc_fence_after();
                            tc_fence_before();
                            if (lane == 0) mbar_arrive(empty0 + as * 8u);
                        }
                        continue;
                    }
                    for (uint32_t kb = k.kb0; kb < k.kb1; ++kb, j += kMqaBlockKv) {
                        const uint32_t as = acount & 1u, aphase = (acount >> 1) & 1u;
                        ++acount;
                        ok = __all_sync(0xffffffffu, mbar_wait(full0 + as * 8u, aphase, wc, kWaitTmemFull));
                        if (!ok) break;
                        tc_fence_after();
                        float scale = 1.f;
                        if (!SCALED) scale = j < p.num_kv ? __ldg(p.kv_scale + j) : 0.f;
                        const uint32_t taddr = lane_base + as * acc_stride;
                        uint64_t a01 = 0ull, a23 = 0ull;          // four f32 partial sums as two packed pairs
                        uint32_t v[16];
#pragma unroll
                        for (uint32_t u = 0; u < NUN; ++u) {
                            tmem_ld_x16(taddr + u * 16u, v);
                            tmem_ld_wait();
                            if (u + 1 == NUN) {
                                // every column of this stage is in registers: hand the TMEM stage back
                                tc_fence_before();
                                if (lane == 0) mbar_arrive(empty0 + as * 8u);
                            }
#pragma unroll
                            for (uint32_t i = 0; i < 4; ++i) {
                                const float x0 = __uint_as_float(v[4 * i]), x1 = __uint_as_float(v[4 * i + 1]);
                                const float x2 = __uint_as_float(v[4 * i + 2]), x3 = __uint_as_float(v[4 * i + 3]);
                                a01 = fma_f32x2(pack_f32x2(relu_nan(x0), relu_nan(x1)), wp[8 * u + 2 * i], a01);
                                a23 = fma_f32x2(pack_f32x2(relu_nan(x2), relu_nan(x3)), wp[8 * u + 2 * i + 1], a23);
                            }
                            if ((u + 1) % UPQ == 0) {
                                // a query is complete
                                const uint32_t qq = u / UPQ;
                                const uint32_t s = QPW == 1 ? s_fix : win[q_first + qq];
                                const uint32_t span = QPW == 1 ? span_fix : (win[16u + q_first + qq] > s ? win[16u + q_first + qq] - s : 0u);
                                const uint32_t off = j - s;       // a token in front of the window wraps around and fails the test
                                if (off < span) {
                                    const float val = ((lo_f32(a01) + hi_f32(a01)) + (lo_f32(a23) + hi_f32(a23))) * scale;
                                    if (SCALED) out_bf16[(size_t)qq * p.logits_stride + off] = __float2bfloat16_rn(val);
                                    else out_f32[(size_t)qq * p.logits_stride + off] = val;
                                }
                                a01 = a23 = 0ull;
                            }
                        }
                    }
                    continue;
                }
                for (uint32_t kb = k.kb0; kb < k.kb1; ++kb) {
                    const uint32_t as = acount & 1u, aphase = (acount >> 1) & 1u;
                    ++acount;
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->tmem_full[as]), aphase, wc, kWaitTmemFull));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t j = kb * kMqaBlockKv + quarter * 32u + lane;
                    float scale = 1.f;
                    if (!SCALED) scale = j < p.num_kv ? __ldg(p.kv_scale + j) : 0.f;
                    const uint32_t taddr = tmem + ((quarter * 32u) << 16) + as * acc_stride + col_base;
                    uint64_t a01 = 0ull, a23 = 0ull;                 // four f32 partial sums of the current query, as two packed pairs
                    uint32_t unit_in_q = 0, q_done = 0;              // position inside this warp's share of the query block
                    auto store_query = [&]() {
                        const uint32_t qi = q_first + q_done;        // index inside the query block
                        const uint32_t s = win[qi], e = win[16u + qi];   // e = 0 for queries past the end
                        if (j >= s && j < e) {
                            const float val = ((lo_f32(a01) + hi_f32(a01)) + (lo_f32(a23) + hi_f32(a23))) * scale;
                            const size_t o = (size_t)(k.q0 + qi) * p.logits_stride + (j - s);
                            if (SCALED) reinterpret_cast<__nv_bfloat16*>(p.logits)[o] = __float2bfloat16_rn(val);
                            else reinterpret_cast<float*>(p.logits)[o] = val;
                        }
                        a01 = a23 = 0ull;
                        unit_in_q = 0;
                        ++q_done;
                    };
                    auto release = [&]() {
                        // every column of this stage is in registers: hand the TMEM stage back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[as]));
                    };
                    if (U4) {
                        // head counts that are not a multiple of 16: four columns at a time, no software pipeline
                        for (uint32_t u = 0; u < nunits; ++u) {
                            uint32_t v[4];
                            __syncwarp();
                            tmem_ld_x4(taddr + u * 4u, v);
                            tmem_ld_wait();
                            if (u + 1 == nunits) release();
                            const float4 ww = *reinterpret_cast<const float4*>(w + col_base + u * 4u);
                            const float x0 = __uint_as_float(v[0]), x1 = __uint_as_float(v[1]);
                            const float x2 = __uint_as_float(v[2]), x3 = __uint_as_float(v[3]);
                            a01 = fma_f32x2(pack_f32x2(relu_nan(x0), relu_nan(x1)), pack_f32x2(ww.x, ww.y), a01);
                            a23 = fma_f32x2(pack_f32x2(relu_nan(x2), relu_nan(x3)), pack_f32x2(ww.z, ww.w), a23);
                            if (++unit_in_q == units_per_q) store_query();
                        }
                        continue;
                    }
                    // Any other head count that is a multiple of 16: units of 16 columns, the TMEM load and the four
                    // weight vectors of unit u + 1 requested before the arithmetic of unit u starts, so that neither
                    // the tensor-memory latency nor the shared-memory latency sits between dependent instructions.
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
                            a01 = fma_f32x2(pack_f32x2(relu_nan(x0), relu_nan(x1)), pack_f32x2(ww[i].x, ww[i].y), a01);
                            a23 = fma_f32x2(pack_f32x2(relu_nan(x2), relu_nan(x3)), pack_f32x2(ww[i].z, ww[i].w), a23);
                        }
                        if (++unit_in_q == units_per_q) store_query();
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
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ---------------------------------------------------------------------------- paged metadata
// Counterpart of mqa_paged_metadata_impl (deepgemm/kernels/mqa_logits_sm100.cu:359-492): one block turns the
// sorted request ids and the context lengths into the list the main kernel cuts its shares from.
//   req_first[t]  first token of t's request (runs of equal ids)
//   qb_tokens[t]  a query block starts at every block_q-th token of a request: its token count, else 0
//   cum[t]        kv blocks (128 tokens) of all query blocks that start before t; cum[T] = all work
// A query block needs the kv tokens [0, context length of its last token): context lengths grow inside a
// request (deepgemm/kernels/mqa_logits_sm100.cu:207-216), so that is the longest of its own.
constexpr uint32_t kMetaThreads = 1024;
__device__ __forceinline__ uint32_t block_scan_excl(uint32_t v, uint32_t* sh, bool use_max) {
    // exclusive scan (sum or max) of one value per thread over the block; identity 0
    const uint32_t tid = threadIdx.x;
    sh[tid] = v;
    __syncthreads();
    for (uint32_t d = 1; d < kMetaThreads; d <<= 1) {
        const uint32_t other = tid >= d ? sh[tid - d] : 0u;
        __syncthreads();
        sh[tid] = use_max ? max(sh[tid], other) : sh[tid] + other;
        __syncthreads();
    }
    const uint32_t r = tid ? sh[tid - 1] : 0u;
    __syncthreads();
    return r;
}
__global__ void __launch_bounds__(kMetaThreads) mqa_paged_metadata_kernel(const uint32_t* __restrict__ context_lens,
                                                                         const uint32_t* __restrict__ indices, uint32_t num_tokens,
                                                                         uint32_t block_q, uint32_t max_ctx, uint32_t* cum,
                                                                         uint32_t* qb_tokens, uint32_t* req_first) {
    __shared__ uint32_t sh[kMetaThreads];
    const uint32_t per = (num_tokens + kMetaThreads - 1) / kMetaThreads;
    const uint32_t t0 = min(threadIdx.x * per, num_tokens), t1 = min(t0 + per, num_tokens);
    // request starts: running maximum of (start position + 1)
    uint32_t run = 0;
    for (uint32_t t = t0; t < t1; ++t)
        if (t == 0 || indices[t] != indices[t - 1]) run = t + 1;
    uint32_t carry = block_scan_excl(run, sh, true);
    for (uint32_t t = t0; t < t1; ++t) {
        if (t == 0 || indices[t] != indices[t - 1]) carry = t + 1;
        req_first[t] = carry - 1u;
    }
    // query blocks and their kv blocks
    uint32_t local = 0;
    for (uint32_t t = t0; t < t1; ++t) {
        const uint32_t first = req_first[t];
        uint32_t nq = 0;
        if ((t - first) % block_q == 0) {
            nq = 1;
            while (nq < block_q && t + nq < num_tokens && indices[t + nq] == indices[t]) ++nq;
        }
        qb_tokens[t] = nq;
        if (nq) local += (min(context_lens[t + nq - 1], max_ctx) + kMqaBlockKv - 1) / kMqaBlockKv;
    }
    uint32_t acc = block_scan_excl(local, sh, false);
    for (uint32_t t = t0; t < t1; ++t) {
        cum[t] = acc;
        const uint32_t nq = qb_tokens[t];
        if (nq) acc += (min(context_lens[t + nq - 1], max_ctx) + kMqaBlockKv - 1) / kMqaBlockKv;
    }
    if (threadIdx.x == kMetaThreads - 1) cum[num_tokens] = acc;
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

struct MqaPaged {
    uint32_t page_kv = 0, num_pages = 0, block_table_stride = 0;
    const uint32_t* context_lens = nullptr;
    const uint32_t* indices = nullptr;
    const uint32_t* block_table = nullptr;
};

template <bool SCALED, bool FP4, bool PAGED>
static int32_t run_mqa(const void* q, const void* kv, const uint32_t* q_sf, uint32_t q_sf_cols, const uint32_t* kv_sf,
                       uint32_t kv_sf_cols, const float* kv_scale, const void* weights, const uint32_t* ks,
                       const uint32_t* ke, uint32_t num_tokens, uint32_t num_kv, uint32_t num_heads, uint32_t head_dim,
                       void* logits, uint32_t logits_stride, const MqaPaged& pg, void* stream) {
    const DeviceInfo* dev;
    int32_t st = current_device(&dev);
    if (st != DG_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MqaParams p{};
    p.num_tokens = num_tokens; p.num_kv = num_kv; p.num_heads = num_heads; p.head_dim = head_dim;
    // Tiling: n = block_q * num_heads score columns per kv block, at most 256 (192 beside the scale-factor
    // columns of the ue8m0 contracts); the MMA wants a multiple of 16 columns and computes a few unused ones
    // when n is not.
    const uint32_t max_n = SCALED ? 192u : 256u;
    uint32_t block_q = max_n / num_heads;
    if (block_q > 16) block_q = 16;
    // The epilogue warpgroups split the query block evenly: 1, 2, 3 or 4 of them.  64 and 32 heads under the 192
    // columns of the ue8m0 contracts keep all three (six) queries that fit, on three warpgroups (one query of 64
    // heads or two of 32 each): with two queries the MMAs are 128 columns wide and only eight warps reduce.
    const bool three_groups = SCALED && ((num_heads == 64 && block_q == 3) || (num_heads == 32 && block_q == 6));
    if (three_groups) { /* keep */ }
    else if (block_q >= 4) block_q &= ~3u;
    else if (block_q == 3) block_q = 2;
    if (block_q == 0) return fail(DG_ERR_UNSUPPORTED, "mqa_logits: %u heads do not fit the %u score columns of this contract", num_heads, max_n);
    p.acc_stride = SCALED ? 192u : 256u;
    p.block_q = block_q;
    p.n = block_q * num_heads;
    p.n_mma = align_up(p.n, 16);
    p.ep_groups = three_groups ? 3u : block_q % 4 == 0 ? 4u : block_q % 2 == 0 ? 2u : 1u;
    p.unit = num_heads % 16 == 0 ? 16u : 4u;
    p.num_q_blocks = ceil_div(num_tokens, block_q);
    // Contiguous kv: the work items are query blocks, each over its whole kv range.  With fewer query blocks than
    // twice the SMs (a short prefill chunk, a handful of queries) the range is cut into pieces of at least eight
    // kv blocks, so that every SM gets work.
    p.kv_splits = 1;
    if (!PAGED && p.num_q_blocks < 2u * (uint32_t)dev->sm_count) {
        const uint32_t kv_blocks = ceil_div(num_kv, kMqaBlockKv);
        const uint32_t want = ceil_div(2u * (uint32_t)dev->sm_count, p.num_q_blocks);
        const uint32_t most = kv_blocks / 8u > 1u ? kv_blocks / 8u : 1u;
        p.kv_splits = want < most ? want : most;
    }
    p.row_bytes = FP4 ? head_dim / 2 : head_dim;
    p.sbo = 8 * p.row_bytes;
    p.layout = p.row_bytes == 128 ? 2u : p.row_bytes == 64 ? 4u : p.row_bytes == 32 ? 6u : 0u;
    if (p.layout == 0) return fail(DG_ERR_INVALID_ARG, "MXFP4 requires head_dim 64/128");
    const CUtensorMapSwizzle sw = p.row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : p.row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    p.num_mma = p.row_bytes / 32u;
    p.idesc = SCALED ? make_idesc_bs(FP4 ? 1u : 0u, FP4 ? 1u : 0u, kMqaBlockKv, p.n_mma) : make_idesc_f8(kMqaBlockKv, p.n_mma);
    p.off_w = 1024;
    p.off_q = 1024 + 2048u;
    p.q_sf_off = align_up(p.n_mma * p.row_bytes, 1024);   // the MMA of the last rows may read a few rows past the box
    p.q_stage_bytes = p.q_sf_off + (SCALED ? 1024u : 0u);
    p.off_kv = p.off_q + 2 * p.q_stage_bytes;
    p.kv_sf_off = kMqaBlockKv * p.row_bytes;
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

    uint32_t* meta = nullptr;
    bool meta_owned = false;        // allocated for this call alone (graph capture): freed behind the launch
    if (PAGED) {
        p.page_kv = pg.page_kv;
        p.box_rows = pg.page_kv < kMqaBlockKv ? pg.page_kv : kMqaBlockKv;
        p.boxes_per_block = kMqaBlockKv / p.box_rows;
        p.kv_sf = kv_sf;
        p.context_lens = pg.context_lens;
        p.block_table = pg.block_table;
        p.block_table_stride = pg.block_table_stride;
        // Scratch of the metadata kernel: three arrays of one word per token.  One buffer per (thread, device,
        // stream), grown on demand with stream-ordered allocation and kept for the next call: work on one stream is
        // ordered, so consecutive calls may share it, and an allocation per call costs a decode step more than its
        // kernels (after a synchronisation the pool has given its memory back and the next call waits for the
        // driver).  Inside a graph capture the buffer must belong to the graph: allocated and freed per call.
        const size_t words = 3 * (size_t)num_tokens + 4;
        struct MetaWs { cudaStream_t stream; int device; uint32_t* ptr; size_t bytes; };
        static thread_local MetaWs cache[8] = {};
        static thread_local int cache_next = 0;
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        DG_CUDA_CHECK(cudaStreamIsCapturing(s, &capturing));
        if (capturing != cudaStreamCaptureStatusNone) {
            DG_CUDA_CHECK(cudaMallocAsync(&meta, words * sizeof(uint32_t), s));
            meta_owned = true;
        } else {
            MetaWs* slot = nullptr;
            for (auto& c : cache)
                if (c.ptr && c.stream == s && c.device == dev->device) { slot = &c; break; }
            if (!slot) {
                slot = &cache[cache_next];
                cache_next = (cache_next + 1) % 8;
                if (slot->ptr) { cudaFreeAsync(slot->ptr, slot->stream); *slot = MetaWs{}; }
            }
            if (slot->bytes < words * sizeof(uint32_t)) {
                if (slot->ptr) cudaFreeAsync(slot->ptr, s);
                *slot = MetaWs{};
                uint32_t* fresh = nullptr;
                const size_t bytes = align_up((uint32_t)(words * sizeof(uint32_t)), 65536u);
                DG_CUDA_CHECK(cudaMallocAsync(&fresh, bytes, s));
                *slot = MetaWs{s, dev->device, fresh, bytes};
            }
            meta = slot->ptr;
        }
        uint32_t* cum = meta;
        uint32_t* qb_tokens = meta + num_tokens + 1;
        uint32_t* req_first = qb_tokens + num_tokens;
        p.cum = cum; p.qb_tokens = qb_tokens; p.req_first = req_first;
        const uint64_t max_ctx64 = (uint64_t)pg.block_table_stride * pg.page_kv;
        mqa_paged_metadata_kernel<<<1, kMetaThreads, 0, s>>>(pg.context_lens, pg.indices, num_tokens, block_q,
                                                             (uint32_t)(max_ctx64 > 0xffffff00ull ? 0xffffff00ull : max_ctx64), cum,
                                                             qb_tokens, req_first);
        note_launch();
    }

    CUtensorMap tq, tkv, tqsf, tkvsf;
    auto fail_free = [&](int32_t code) { if (meta_owned) cudaFreeAsync(meta, s); return code; };
    if ((st = make_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, p.row_bytes, (uint64_t)num_tokens * num_heads, p.row_bytes,
                           p.row_bytes, p.n, sw, "q")) != DG_OK) return fail_free(st);
    if ((st = make_tmap_2d(&tkv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, kv, p.row_bytes, num_kv, p.row_bytes, p.row_bytes,
                           PAGED ? p.box_rows : kMqaBlockKv, sw, "kv")) != DG_OK) return fail_free(st);
    tqsf = tq; tkvsf = tkv;
    if (SCALED) {
        if ((st = make_tmap_2d(&tqsf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, q_sf, q_sf_cols, 1, (uint64_t)q_sf_cols * 4, p.n, 1,
                               CU_TENSOR_MAP_SWIZZLE_NONE, "q_sf")) != DG_OK) return fail_free(st);
        if (!PAGED && (st = make_tmap_2d(&tkvsf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, kv_sf, kv_sf_cols, 1, (uint64_t)kv_sf_cols * 4,
                                         kMqaBlockKv, 1, CU_TENSOR_MAP_SWIZZLE_NONE, "kv_sf")) != DG_OK) return fail_free(st);
    }
    uint32_t grid = (uint32_t)dev->sm_count;
    if (!PAGED && p.num_q_blocks * p.kv_splits < grid) grid = p.num_q_blocks * p.kv_splits;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(128u + 128u * p.ep_groups);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // set-up overlaps the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
    // The variants that move registers from the role warps to the epilogue warpgroups block inside the kernel if the
    // registers the block got at launch do not cover what its warpgroups ask for: refuse the launch instead.
    // the dynamic shared memory limit of a kernel is raised once per thread and device, not on every call
    auto set_smem = [&](const void* fn) -> cudaError_t {
        static thread_local const void* done_fn[8] = {};
        static thread_local uint32_t done_bytes[8] = {};
        static thread_local int done_dev[8] = {};
        for (int i = 0; i < 8; ++i)
            if (done_fn[i] == fn && done_dev[i] == dev->device && done_bytes[i] >= smem_bytes) return cudaSuccess;
        const cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (err == cudaSuccess) {
            static thread_local int next = 0;
            done_fn[next] = fn; done_bytes[next] = smem_bytes; done_dev[next] = dev->device;
            next = (next + 1) % 8;
        }
        return err;
    };
    auto budget_ok = [&](const void* fn, uint32_t nun) {
        // registers per thread of the (at most four) kernels this instantiation launches, looked up once per thread
        static thread_local const void* seen_fn[4] = {nullptr, nullptr, nullptr, nullptr};
        static thread_local uint32_t seen_regs[4] = {0, 0, 0, 0};
        uint32_t regs = 0;
        for (int i = 0; i < 4 && !regs; ++i)
            if (seen_fn[i] == fn) regs = seen_regs[i];
        if (!regs) {
            cudaFuncAttributes fa;
            if (cudaFuncGetAttributes(&fa, fn) != cudaSuccess) return false;
            regs = (uint32_t)fa.numRegs;
            for (int i = 0; i < 4; ++i)
                if (!seen_fn[i]) { seen_fn[i] = fn; seen_regs[i] = regs; break; }
        }
        const uint32_t threads = cfg.blockDim.x;
        return threads <= mqa_threads(nun) && regs * threads >= 128u * kMqaRoleRegs + (threads - 128u) * mqa_epilogue_regs(nun);
    };
    if (p.unit == 4u) {
        auto* fn = mqa_logits_kernel<SCALED, FP4, PAGED, true>;
        e = set_smem((const void*)fn);
        if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, fn, tq, tkv, tqsf, tkvsf, p);
    } else if (num_heads == 32 && p.block_q == 2u * p.ep_groups && p.ep_groups >= 3u) {
        auto* fn = mqa_logits_kernel<SCALED, FP4, PAGED, false, 4, 2>;   // two queries of 32 heads per warpgroup
        if (!budget_ok((const void*)fn, 4)) return fail_free(fail(DG_ERR_RUNTIME, "mqa_logits: register budget of the 32-head kernel does not add up"));
        e = set_smem((const void*)fn);
        if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, fn, tq, tkv, tqsf, tkvsf, p);
    } else if (num_heads == 64 && p.block_q == p.ep_groups) {
        auto* fn = mqa_logits_kernel<SCALED, FP4, PAGED, false, 4>;   // one query of 64 heads per warpgroup
        if (!budget_ok((const void*)fn, 4)) return fail_free(fail(DG_ERR_RUNTIME, "mqa_logits: register budget of the 64-head kernel does not add up"));
        e = set_smem((const void*)fn);
        if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, fn, tq, tkv, tqsf, tkvsf, p);
    } else if (num_heads == 128 && p.block_q == p.ep_groups) {
        auto* fn = mqa_logits_kernel<SCALED, FP4, PAGED, false, 8>;   // one query of 128 heads per warpgroup
        if (!budget_ok((const void*)fn, 8)) return fail_free(fail(DG_ERR_RUNTIME, "mqa_logits: register budget of the 128-head kernel does not add up"));
        e = set_smem((const void*)fn);
        if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, fn, tq, tkv, tqsf, tkvsf, p);
    } else {
        auto* fn = mqa_logits_kernel<SCALED, FP4, PAGED, false>;
        e = set_smem((const void*)fn);
        if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, fn, tq, tkv, tqsf, tkvsf, p);
    }
    if (meta_owned) cudaFreeAsync(meta, s);
    if (e != cudaSuccess) return fail(DG_ERR_DRIVER, "mqa_logits launch failed: %s", cudaGetErrorString(e));
    dg::note_launch();
    return DG_OK;
}

// q operand checks shared by the contiguous and the paged ue8m0 entries
static int32_t check_mqa_q(const dg_operand_t* q, uint32_t num_tokens, uint32_t num_heads, uint32_t head_dim) {
    if (!q || !q->data) return fail(DG_ERR_INVALID_ARG, "mqa_logits: null operand");
    if (q->dtype != DG_FP8 && q->dtype != DG_FP4) return fail(DG_ERR_INVALID_ARG, "mqa_logits: q/kv must be FP8 or FP4");
    if (q->dtype == DG_FP4 && head_dim != 64 && head_dim != 128) return fail(DG_ERR_INVALID_ARG, "MXFP4 requires head_dim 64/128");
    if (!q->sf.data) return fail(DG_ERR_INVALID_ARG, "mqa_logits: q and kv require scale factors");
    if (q->sf.gran != 32) return fail(DG_ERR_INVALID_ARG, "mqa_logits: scale granularity must be 32");
    if (q->rows != num_tokens * num_heads || q->k != head_dim)
        return fail(DG_ERR_INVALID_ARG, "mqa_logits: q must be [num_tokens*num_heads, head_dim] and kv [num_kv_tokens, head_dim]");
    if (q->major != DG_MAJOR_K || q->outer_stride != head_dim)
        return fail(DG_ERR_INVALID_ARG, "mqa_logits: q and kv must be dense K-major rows (outer_stride == head_dim)");
    if (q->sf.cols < align_up(q->rows, 4) || q->sf.rows < 1) return fail(DG_ERR_INVALID_ARG, "mqa_logits: scale-factor tensors too small");
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
    return dg::run_mqa<false, false, false>(q, kv, nullptr, 0, nullptr, 0, kv_scale, weights, cu_k_start, cu_k_end, num_tokens,
                                            num_kv_tokens, num_heads, head_dim, logits, logits_stride, dg::MqaPaged{}, stream);
}

int32_t dg_mqa_logits(const dg_operand_t* q, const dg_operand_t* kv, const void* weights_bf16, const uint32_t* cu_k_start,
                      const uint32_t* cu_k_end, uint32_t num_tokens, uint32_t num_kv_tokens, uint32_t num_heads,
                      uint32_t head_dim, void* logits_bf16, uint32_t logits_stride, void* stream) {
    if (!q || !kv || !q->data || !kv->data) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: null operand");
    if (q->dtype != kv->dtype) return dg::fail(DG_ERR_INVALID_ARG, "Q/KV dtype mismatch");
    int32_t st = dg::check_mqa_common(num_tokens, num_kv_tokens, num_heads, head_dim, logits_stride, cu_k_start, cu_k_end,
                                      weights_bf16, logits_bf16);
    if (st != DG_OK) return st;
    if ((st = dg::check_mqa_q(q, num_tokens, num_heads, head_dim)) != DG_OK) return st;
    if (!kv->sf.data || kv->sf.gran != 32) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: q and kv require scale factors of granularity 32");
    if (kv->rows != num_kv_tokens || kv->k != head_dim)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: q must be [num_tokens*num_heads, head_dim] and kv [num_kv_tokens, head_dim]");
    if (kv->major != DG_MAJOR_K || kv->outer_stride != head_dim)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: q and kv must be dense K-major rows (outer_stride == head_dim)");
    if (kv->sf.cols < dg::align_up(kv->rows, 4) || kv->sf.rows < 1)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits: scale-factor tensors too small");
    if (q->dtype == DG_FP4)
        return dg::run_mqa<true, true, false>(q->data, kv->data, q->sf.data, q->sf.cols, kv->sf.data, kv->sf.cols, nullptr, weights_bf16,
                                              cu_k_start, cu_k_end, num_tokens, num_kv_tokens, num_heads, head_dim, logits_bf16,
                                              logits_stride, dg::MqaPaged{}, stream);
    return dg::run_mqa<true, false, false>(q->data, kv->data, q->sf.data, q->sf.cols, kv->sf.data, kv->sf.cols, nullptr, weights_bf16,
                                           cu_k_start, cu_k_end, num_tokens, num_kv_tokens, num_heads, head_dim, logits_bf16,
                                           logits_stride, dg::MqaPaged{}, stream);
}

int32_t dg_mqa_logits_paged(const dg_operand_t* q, const void* kv_pages, const uint32_t* kv_sf_pages, const void* weights_bf16,
                            uint32_t page_kv, uint32_t num_pages, const uint32_t* context_lens, const uint32_t* indices,
                            const uint32_t* block_table, uint32_t block_table_stride, uint32_t num_tokens, uint32_t num_heads,
                            uint32_t head_dim, void* logits_bf16, uint32_t logits_stride, void* stream) {
    if (!kv_pages || !kv_sf_pages || !context_lens || !indices || !block_table)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits_paged: null buffer");
    if (reinterpret_cast<uintptr_t>(kv_sf_pages) & 15u)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits_paged: the scale words of the cache must be 16-byte aligned (they are read four tokens at a time)");
    // deepgemm/src/api.rs:1778-1795
    if (head_dim % 32 != 0 || head_dim > 128 || head_dim == 96 || head_dim == 0)
        return dg::fail(DG_ERR_INVALID_ARG, "head_dim must be 32/64/128");
    if (num_heads % 4 != 0 || num_heads > 256 || num_heads == 0)
        return dg::fail(DG_ERR_INVALID_ARG, "num_heads must be a multiple of 4 (<= 256)");
    if (page_kv == 0 || page_kv % 4 != 0 || 256 % page_kv != 0)
        return dg::fail(DG_ERR_INVALID_ARG, "page_kv must divide 256 (multiple of 4)");
    if (!q || (q->dtype != DG_FP8 && q->dtype != DG_FP4)) return dg::fail(DG_ERR_INVALID_ARG, "paged MQA needs FP8 or FP4 Q");
    if (num_tokens == 0 || num_pages == 0 || block_table_stride == 0 || logits_stride == 0 || !weights_bf16 || !logits_bf16)
        return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits_paged: empty problem");
    if ((uint64_t)num_pages * page_kv >= (1ull << 31)) return dg::fail(DG_ERR_INVALID_ARG, "mqa_logits_paged: the cache exceeds 2^31 tokens");
    int32_t st = dg::check_mqa_q(q, num_tokens, num_heads, head_dim);
    if (st != DG_OK) return st;
    dg::MqaPaged pg;
    pg.page_kv = page_kv; pg.num_pages = num_pages; pg.block_table_stride = block_table_stride;
    pg.context_lens = context_lens; pg.indices = indices; pg.block_table = block_table;
    const uint32_t num_kv = num_pages * page_kv;
    if (q->dtype == DG_FP4)
        return dg::run_mqa<true, true, true>(q->data, kv_pages, q->sf.data, q->sf.cols, kv_sf_pages, num_kv, nullptr, weights_bf16, nullptr,
                                             nullptr, num_tokens, num_kv, num_heads, head_dim, logits_bf16, logits_stride, pg, stream);
    return dg::run_mqa<true, false, true>(q->data, kv_pages, q->sf.data, q->sf.cols, kv_sf_pages, num_kv, nullptr, weights_bf16, nullptr,
                                          nullptr, num_tokens, num_kv, num_heads, head_dim, logits_bf16, logits_stride, pg, stream);
}

}  // extern "C"
