// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM
// alloc/ld/cp/commit) and the shared-memory / instruction descriptor encodings.
//
// Every wait in this file is bounded: a wait that does not complete within
// kWaitTimeoutNs records a status word in global memory, raises a CTA-wide abort flag and
// returns false, so the kernel tears down (TMEM freed) and the context stays usable.
// The reference's device waits are unbounded spins (deepgemm/kernels/prelude.h:252-262).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dg {

constexpr unsigned long long kWaitTimeoutNs = 2000000000ull;  // 2 s
#ifndef DG_PARK_NS
#define DG_PARK_NS 20000u
#endif

// Status word layout: low byte = which wait gave up, bits 8.. = blockIdx.x.
enum WaitSite : uint32_t {
    kWaitEmpty = 1, kWaitFull = 2, kWaitSfReady = 3, kWaitTmemFull = 4, kWaitTmemEmpty = 5,
    kWaitStore = 6, kWaitPeer = 7, kWaitSched = 8, kWaitWeights = 9, kWaitSfFree = 10,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }
// One lane of a fully converged warp.  The single-thread roles (TMA producer, MMA issuer) run
// their loops warp-converged and predicate only the issuing instructions with this, so that
// descriptors, coordinates and barrier addresses stay warp-uniform values.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// Bounded wait by every lane of a converged warp; the result is warp-uniform.
#define DG_WARP_WAIT(bar, parity, wc, site) __all_sync(0xffffffffu, ::dg::mbar_wait((bar), (parity), (wc), (site)))

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while the
// kernel before it in the stream is still running; griddep_wait() blocks until that kernel has
// completed and its writes are visible, so everything before the call (barrier set-up, TMEM
// allocation, descriptor prefetch) overlaps the predecessor's tail.  griddep_launch_dependents()
// lets the successor start as soon as every CTA of this grid has got this far.  Both are no-ops
// for a normally launched kernel.  (The reference launches with the same attribute,
// deepgemm/src/sys.rs:287-294, and waits at deepgemm/kernels/gemm_sm100.cu:566.)
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- register reallocation between warpgroups
// All four warps of a warpgroup (warps 4 g .. 4 g + 3) execute the same call.  A warpgroup that gives registers
// back lets the others raise their limit above what the launch gave every thread; the sum over the block must
// stay within the block's allocation at launch (reg_acquire waits until the registers are there, so a budget
// that does not add up would block for ever: the host checks it before the launch).  N: 24 .. 256, a multiple
// of 8.  Code that runs under a changed limit cannot call functions: everything in it is inlined.
template <uint32_t N> __device__ __forceinline__ void reg_release() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <uint32_t N> __device__ __forceinline__ void reg_acquire() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ---------------------------------------------------------------- clusters (CTA pairs)
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Shared by all roles of a CTA: where to report, and the CTA-wide abort flag.
struct WaitCtx {
    uint32_t* status;            // global; 0 = healthy
    volatile uint32_t* abort;    // shared; non-zero = some role gave up
};

// try_wait that lets the hardware park the thread for up to `ns` nanoseconds (it still wakes as
// soon as the phase completes), so that a waiting role does not take issue slots from working warps.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}

// (a translation unit whose kernels move registers between warpgroups defines DG_WAIT_SLOW_ATTR as
// __forceinline__ before it includes this file)
#ifndef DG_WAIT_SLOW_ATTR
#define DG_WAIT_SLOW_ATTR __noinline__
#endif
static __device__ DG_WAIT_SLOW_ATTR bool mbar_wait_slow(uint32_t bar, uint32_t parity, const WaitCtx& w, uint32_t site) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait_parked(bar, parity, DG_PARK_NS)) {
        if ((++spins & 63u) == 0) {
            if (*w.abort) return false;
            if (globaltimer_ns() - t0 > kWaitTimeoutNs) {
                atomicCAS(w.status, 0u, site | (blockIdx.x << 8));
                *w.abort = 1u;
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, uint32_t site) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, w, site);
}

// ---------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> this CTA's shared memory, completion on `bar` (bytes).
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* m, uint32_t bar, uint32_t dst, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Four rows of a 2-D tensor, picked by their row coordinates y0..y3, at inner coordinate x: the four boxes (the
// map's box is one row high) land one after the other at `dst`, swizzled by their shared-memory address like
// the rows of an ordinary tile, so a tile can be assembled from arbitrary rows, four per instruction.
__device__ __forceinline__ void tma_gather4_2d(const CUtensorMap* m, uint32_t bar, uint32_t dst, int32_t x, int32_t y0, int32_t y1,
                                               int32_t y2, int32_t y3) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::1 "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3) : "memory");
}
// The same load issued by either CTA of a pair: `bar` is a shared::cluster address (the leader
// CTA's barrier), the destination is this CTA's own shared memory.  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* m, uint32_t bar, uint32_t dst, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y) : "memory");
}
// ---------------------------------------------------------------- TMEM management (whole warp)
// CL = 1: one CTA; CL = 2: a CTA pair (the same warp index of both CTAs executes the call).
template <int CL = 1>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    if (CL == 1) asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    else asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
template <int CL = 1>
__device__ __forceinline__ void tmem_relinquish() {
    if (CL == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CL = 1>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if (CL == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor (64 bit): start>>4 [0,14), LBO>>4 [16,30), SBO>>4 [32,46),
// version=1 [46,48), base offset [49,52), layout type [61,64).
constexpr uint64_t kLayoutNone = 0, kLayoutSw128 = 2;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t lbo_bytes, uint64_t layout) {
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4)
         | (static_cast<uint64_t>(lbo_bytes >> 4) << 16)
         | (static_cast<uint64_t>(sbo_bytes >> 4) << 32)
         | (1ull << 46)
         | (layout << 61);
}
// K-major operand tile, 128-byte rows, 128B swizzle: 8-row groups are 1024 B apart.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t saddr) {
    return make_smem_desc(saddr, 1024, 0, kLayoutSw128);
}
// 32 rows x 16 B, no swizzle: the source of tcgen05.cp.32x128b (8-row groups 128 B apart).
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
    return make_smem_desc(saddr, 128, 0, kLayoutNone);
}

// Instruction descriptor, kind::f16 (bf16 x bf16 -> f32), K-major A and B.
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t m, uint32_t n) {
    return (1u << 4) /*D=f32*/ | (1u << 7) /*A=bf16*/ | (1u << 10) /*B=bf16*/ | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Block-scaled kinds (mxf8f6f4: format 0 = E4M3, 5 = E2M1 in byte containers; mxf4: 1 = E2M1),
// UE8M0 scales, K-major.
__host__ __device__ constexpr uint32_t make_idesc_bs(uint32_t fmt_a, uint32_t fmt_b, uint32_t m, uint32_t n) {
    return (fmt_a << 7) | (fmt_b << 10) | ((n >> 3) << 17) | (1u << 23) /*UE8M0*/ | ((m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_sf_id, uint32_t b_sf_id) {
    return idesc | (b_sf_id << 4) | (a_sf_id << 29);
}

// ---------------------------------------------------------------- tcgen05 ops (single thread)
// `bar` is a shared::cluster address: this CTA's own barrier, or the peer's through mapa().
template <int CL = 1>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    if (CL == 1) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    else asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// One commit whose completion signal arrives on the barrier at the same shared-memory offset in both CTAs
// of a pair (the multicast here is of the signal only; no data moves).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_local) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar_local), "h"(mask) : "memory");
}
// 32 rows x 128 bit from shared memory, broadcast to the four 32-lane quarters of TMEM
// (CL = 2: each CTA of the pair copies from its own shared memory into its own TMEM).
template <int CL = 1>
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    if (CL == 1) asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
    else asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
template <int CL = 1>
__device__ __forceinline__ void tc_mma_bf16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    if (CL == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
template <int CL = 1>
__device__ __forceinline__ void tc_mma_mxf8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc,
                                            uint32_t sfa, uint32_t sfb) {
    if (CL == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
template <int CL = 1>
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc,
                                            uint32_t sfa, uint32_t sfb) {
    if (CL == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}

// ---------------------------------------------------------------- TMEM loads (whole warp)
// Lane i of the warp reads 32-bit columns [col, col+N) of TMEM lane (quarter*32 + i).
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

}  // namespace dg
