// Peer-memory plumbing for expert-parallel MoE steps on the GPUs of one NVSwitch domain: buffers
// that other ranks can map (CUDA IPC), copy-engine pushes into a peer's buffer, a flag barrier
// between ranks, and the table of per-row destination addresses that lets the grouped GEMM's
// epilogue store every result row straight into the memory of the rank that owns the token.
//
// One process per GPU.  Data travels either by copy engine (dg_peer_copy: no SM is used, so the
// copy overlaps a GEMM that occupies every SM) or by plain stores from the GEMM epilogue.  The
// barrier is a one-block kernel that co-resides with anything; its wait is bounded
// (kPeerWaitNs), after which the device status word reports the give-up and the kernel returns.
// No load with cluster multicast touches peer memory anywhere in this library.
//
// The reference runs on one GPU (its MoE layer, deepgemm/src/api_serving.rs:293-377, is a local
// call); none of these entries has a counterpart there.
#include "host.h"
#include "ptx.cuh"

#include <cstdlib>
#include <cstring>

namespace dg {

constexpr unsigned long long kPeerWaitNs = 10000000000ull;  // 10 s: ranks may be far apart at a step boundary

// Thread r tells rank r "I have reached `seq`" by writing my slot of its flag array, then waits
// until rank r has written `seq` (or more) into its slot of mine.  Everything this rank put on
// the stream before the barrier (copies, GEMM epilogue stores to peers) is complete when the
// kernel starts; the system-scope fence orders it before the flag for observers on other GPUs.
__global__ void __launch_bounds__(64) peer_barrier_kernel(unsigned long long* const* __restrict__ peer_flags,
                                                         volatile unsigned long long* local_flags, uint32_t me, uint32_t world,
                                                         unsigned long long seq, unsigned long long wait_ns, uint32_t* status) {
    const uint32_t r = threadIdx.x;
    if (r >= world) return;
    __threadfence_system();
    unsigned long long* remote = peer_flags[r] + me;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(remote), "l"(seq) : "memory");
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(local_flags + r) : "memory");
        if (v >= seq) break;
        if ((++spins & 63u) == 0) {
            if (globaltimer_ns() - t0 > wait_ns) {
                atomicCAS(status, 0u, (uint32_t)kWaitPeer | (r << 8));
                break;
            }
            __nanosleep(200);
        }
    }
}

// ptrs[s] = address of the row of the owning rank's return buffer that slot s of the padded
// expert layout produces, or 0 for padding.  slot_src[s] is the position of the slot's row in the
// received order (rows of source rank 0 first, then rank 1, ...); seg_start[r] the first position
// of source r (world + 1 entries); dst_base[r] the return buffer of rank r as mapped here;
// dst_row0[r] the row of that buffer where this rank's results for r begin.
__global__ void __launch_bounds__(256) return_ptrs_kernel(const int32_t* __restrict__ slot_src, uint32_t slots,
                                                         const int32_t* __restrict__ seg_start,
                                                         const unsigned long long* __restrict__ dst_base,
                                                         const int32_t* __restrict__ dst_row0, uint32_t world,
                                                         uint64_t row_bytes, unsigned long long* __restrict__ ptrs) {
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= slots) return;
    const int32_t i = __ldg(slot_src + s);
    unsigned long long out = 0;
    if (i >= 0 && i < __ldg(seg_start + world)) {
        uint32_t r = 0;
        while (r + 1 < world && i >= __ldg(seg_start + r + 1)) ++r;
        out = __ldg(dst_base + r) + (uint64_t)(uint32_t)(__ldg(dst_row0 + r) + i - __ldg(seg_start + r)) * row_bytes;
    }
    ptrs[s] = out;
}


// ---- expert-parallel dispatch by direct stores ("push") -------------------------------------
// Every rank knows counts[src][g] = copies that rank src routes to global expert g (one all-gather).
// From that table alone each rank derives, without talking to anyone, where in the owner's padded
// expert layout its own copies of expert g begin: experts of one owner follow each other, each padded
// to `align` rows, and inside an expert of owner d the source ranks follow each other in the order
// d+1, d+2, ..., d.

// One block.  dest_base[g] = first slot, in the owner's layout, of this rank's copies for expert g
// (-1 if the owner's layout would overflow `cap` rows; the status word records it).
// The local experts are cut into `slices` ranges [first[s], first[s + 1]) that are dispatched and
// computed one after the other: block_expert[s][b] = local expert of the b-th `align`-row block of
// this rank's own layout if it belongs to slice s, else -1; blocks_used[s] = blocks up to the end
// of slice s.
constexpr uint32_t kMaxSlices = 16;
struct SliceBounds { uint32_t first[kMaxSlices + 1]; };
__global__ void __launch_bounds__(1024) ep_route_kernel(const int32_t* __restrict__ counts, uint32_t world, uint32_t me,
                                                       uint32_t num_experts, uint32_t e_local, uint32_t align, uint32_t cap,
                                                       uint32_t slices, const SliceBounds bounds, int32_t* __restrict__ dest_base,
                                                       int32_t* __restrict__ block_expert, int32_t* __restrict__ blocks_used,
                                                       uint32_t* status) {
    __shared__ int32_t s_padded[1024];
    __shared__ int32_t s_base[1024];
    const uint32_t g = threadIdx.x;
    int32_t before = 0;
    if (g < num_experts) {
        // Inside an expert of owner d the sources follow each other in the order d+1, d+2, ..., d:
        // ranks that walk their layouts in step then store their result rows to different peers.
        const uint32_t owner = g / e_local, my_pos = (me + world - owner - 1u) % world;
        int32_t total = 0;
        for (uint32_t src = 0; src < world; ++src) {
            const int32_t v = __ldg(counts + (size_t)src * num_experts + g);
            if ((src + world - owner - 1u) % world < my_pos) before += v;
            total += v;
        }
        s_padded[g] = (int32_t)((((uint32_t)total + align - 1u) / align) * align);
    }
    __syncthreads();
    if (g < num_experts) {
        const uint32_t first = g / e_local * e_local;
        int32_t base = 0;
        for (uint32_t e = first; e < g; ++e) base += s_padded[e];
        s_base[g] = base;
        const bool fits = (uint32_t)(base + s_padded[g]) <= cap;
        dest_base[g] = fits ? base + before : -1;
        if (!fits) atomicCAS(status, 0u, (uint32_t)kWaitPeer | 0x8000u | (g << 16));
    }
    __syncthreads();
    const uint32_t n_blocks = cap / align;
    for (uint32_t b = threadIdx.x; b < n_blocks; b += blockDim.x) {
        const int32_t row = (int32_t)(b * align);
        int32_t found = -1;
        for (uint32_t e = 0; e < e_local; ++e) {
            const uint32_t gg = me * e_local + e;
            if (row >= s_base[gg] && row < s_base[gg] + s_padded[gg]) { found = (int32_t)e; break; }
        }
        for (uint32_t sl = 0; sl < slices; ++sl)
            block_expert[(size_t)sl * n_blocks + b] =
                (found >= 0 && (uint32_t)found >= bounds.first[sl] && (uint32_t)found < bounds.first[sl + 1]) ? found : -1;
    }
    if (threadIdx.x < slices) {
        const uint32_t last = bounds.first[threadIdx.x + 1u] - 1u, gg = me * e_local + last;
        blocks_used[threadIdx.x] = (int32_t)min((uint32_t)(s_base[gg] + s_padded[gg]) / align, n_blocks);
    }
}

// One warp per copy of this rank's copies (sorted by global expert, so the copies for one owner
// rank are one run; only local experts [e_lo, e_hi) of every owner are handled): stores the token's
// row, its scale-factor words (straight into the owner's packed SF tensor [sf_rows, cap]) and the
// return ticket (source rank + 1, position p) at the copy's slot in the owner's memory, local or
// peer.  Consecutive warps serve different owners, starting with this rank's successor, so that at
// any moment the ranks spread their stores over all peers instead of converging on one.
__global__ void __launch_bounds__(256) ep_push_kernel(const uint4* __restrict__ x, uint64_t x_pitch_vec, uint32_t vec_per_row,
                                                     const uint32_t* __restrict__ x_sf, uint32_t sf_rows, uint64_t sf_cols,
                                                     const int32_t* __restrict__ slot_src, const int32_t* __restrict__ my_offsets,
                                                     const int32_t* __restrict__ dest_base, uint32_t num_experts,
                                                     uint32_t e_local, uint32_t e_lo, uint32_t e_hi, uint32_t world, uint32_t me,
                                                     uint64_t cap, const unsigned long long* __restrict__ a_bases,
                                                     const unsigned long long* __restrict__ sf_bases,
                                                     const unsigned long long* __restrict__ ticket_bases) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps = gridDim.x * (blockDim.x >> 5);
    uint32_t longest = 0;
    for (uint32_t d = 0; d < world; ++d)
        longest = max(longest, (uint32_t)(__ldg(my_offsets + d * e_local + e_hi) - __ldg(my_offsets + d * e_local + e_lo)));
    const uint32_t total = longest * world;
    for (uint32_t v = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); v < total; v += warps) {
        const uint32_t owner = (me + 1u + v % world) % world, i = v / world;
        const uint32_t first = (uint32_t)__ldg(my_offsets + owner * e_local + e_lo);
        const uint32_t p = first + i;
        if (p >= (uint32_t)__ldg(my_offsets + owner * e_local + e_hi)) continue;
        const int32_t token = __ldg(slot_src + p);
        if (token < 0) continue;
        uint32_t lo = owner * e_local + e_lo, hi = owner * e_local + e_hi;   // largest g in the range with my_offsets[g] <= p
        while (hi - lo > 1u) {
            const uint32_t mid = (lo + hi) >> 1;
            if ((uint32_t)__ldg(my_offsets + mid) <= p) lo = mid; else hi = mid;
        }
        const int32_t base = __ldg(dest_base + lo);
        if (base < 0) continue;
        const uint64_t slot = (uint64_t)(uint32_t)base + (p - (uint32_t)__ldg(my_offsets + lo));
        uint4* dst = reinterpret_cast<uint4*>(a_bases[owner]) + slot * vec_per_row;
        const uint4* src = x + (uint64_t)token * x_pitch_vec;
        uint32_t c = lane;
        for (; c + 96u < vec_per_row; c += 128u) {     // four loads in flight per lane before the stores
            const uint4 r0 = __ldg(src + c), r1 = __ldg(src + c + 32u), r2 = __ldg(src + c + 64u), r3 = __ldg(src + c + 96u);
            dst[c] = r0; dst[c + 32u] = r1; dst[c + 64u] = r2; dst[c + 96u] = r3;
        }
        for (; c < vec_per_row; c += 32u) dst[c] = __ldg(src + c);
        uint32_t* sf_dst = reinterpret_cast<uint32_t*>(sf_bases[owner]);
        for (uint32_t r = lane; r < sf_rows; r += 32u) sf_dst[r * cap + slot] = __ldg(x_sf + r * sf_cols + (uint32_t)token);
        if (lane == 0)
            reinterpret_cast<unsigned long long*>(ticket_bases[owner])[slot] = ((unsigned long long)(me + 1u) << 32) | p;
    }
}

// ptrs[s] = where slot s's result row goes: row `position` of the ticket's source rank's return
// buffer; 0 for slots nobody wrote this step.  Tickets are cleared for the next step.
// With block_expert given, only slots of blocks with a non-negative entry are touched (the slice
// whose rows have arrived; other slices' tickets may still be in flight).
__global__ void __launch_bounds__(256) ep_return_ptrs_kernel(unsigned long long* __restrict__ tickets, uint32_t slots,
                                                            const unsigned long long* __restrict__ ret_bases, uint32_t world,
                                                            uint64_t row_bytes, const int32_t* __restrict__ block_expert,
                                                            uint32_t align, unsigned long long* __restrict__ ptrs) {
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= slots) return;
    if (block_expert && __ldg(block_expert + s / align) < 0) return;
    const unsigned long long w = tickets[s];
    const uint32_t src = (uint32_t)(w >> 32);
    ptrs[s] = (src == 0 || src > world) ? 0ull : ret_bases[src - 1u] + (w & 0xffffffffull) * row_bytes;
    if (w) tickets[s] = 0ull;
}

}  // namespace dg

extern "C" {

int32_t dg_peer_alloc(uint64_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return dg::fail(DG_ERR_INVALID_ARG, "peer_alloc: null result or zero size");
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    void* p = nullptr;
    DG_CUDA_CHECK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) {
        cudaFree(p);
        return dg::fail(DG_ERR_DRIVER, "peer_alloc: clearing %llu bytes failed: %s", (unsigned long long)bytes, cudaGetErrorString(e));
    }
    DG_CUDA_CHECK(cudaDeviceSynchronize());
    *ptr = p;
    return DG_OK;
}

int32_t dg_peer_free(void* ptr) {
    if (!ptr) return DG_OK;
    DG_CUDA_CHECK(cudaFree(ptr));
    return DG_OK;
}

int32_t dg_peer_export(const void* ptr, void* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!ptr || !handle64) return dg::fail(DG_ERR_INVALID_ARG, "peer_export: null argument");
    cudaIpcMemHandle_t h;
    DG_CUDA_CHECK(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
    memcpy(handle64, &h, 64);
    return DG_OK;
}

int32_t dg_peer_open(const void* handle64, void** ptr) {
    if (!ptr || !handle64) return dg::fail(DG_ERR_INVALID_ARG, "peer_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    DG_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return DG_OK;
}

int32_t dg_peer_close(void* ptr) {
    if (!ptr) return DG_OK;
    DG_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
    return DG_OK;
}

int32_t dg_peer_copy(void* dst, const void* src, uint64_t bytes, void* stream) {
    if (bytes == 0) return DG_OK;
    if (!dst || !src) return dg::fail(DG_ERR_INVALID_ARG, "peer_copy: null buffer");
    DG_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
    return DG_OK;
}

int32_t dg_peer_barrier(const uint64_t* peer_flags, uint64_t* local_flags, uint32_t me, uint32_t world, uint64_t seq,
                        void* stream) {
    if (!peer_flags || !local_flags) return dg::fail(DG_ERR_INVALID_ARG, "peer_barrier: null flag table");
    if (world == 0 || world > 64 || me >= world) return dg::fail(DG_ERR_INVALID_ARG, "peer_barrier: rank %u of %u (at most 64 ranks)", me, world);
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    // DG_PEER_WAIT_MS shortens (or extends) the bound of the wait, e.g. for failure-detection tests
    unsigned long long wait_ns = dg::kPeerWaitNs;
    if (const char* v = getenv("DG_PEER_WAIT_MS")) {
        const unsigned long long ms = strtoull(v, nullptr, 10);
        if (ms > 0) wait_ns = ms * 1000000ull;
    }
    dg::peer_barrier_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<unsigned long long* const*>(peer_flags), reinterpret_cast<volatile unsigned long long*>(local_flags), me,
        world, seq, wait_ns, dev->status);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_moe_return_ptrs(const int32_t* slot_src, uint32_t slots, const int32_t* seg_start, const uint64_t* dst_base,
                           const int32_t* dst_row0, uint32_t world, uint64_t row_bytes, uint64_t* ptrs, void* stream) {
    if (!slot_src || !seg_start || !dst_base || !dst_row0 || !ptrs) return dg::fail(DG_ERR_INVALID_ARG, "moe_return_ptrs: null buffer");
    if (world == 0 || row_bytes % 16 != 0) return dg::fail(DG_ERR_INVALID_ARG, "moe_return_ptrs: rows must be multiples of 16 bytes");
    if (slots == 0) return DG_OK;
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    dg::return_ptrs_kernel<<<dg::ceil_div(slots, 256u), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        slot_src, slots, seg_start, reinterpret_cast<const unsigned long long*>(dst_base), dst_row0, world, row_bytes,
        reinterpret_cast<unsigned long long*>(ptrs));
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_ep_route(const int32_t* counts, uint32_t world, uint32_t me, uint32_t num_experts, uint32_t align, uint32_t cap,
                    uint32_t slices, const uint32_t* slice_first, int32_t* dest_base, int32_t* block_expert, int32_t* blocks_used,
                    void* stream) {
    if (!counts || !dest_base || !block_expert || !blocks_used) return dg::fail(DG_ERR_INVALID_ARG, "ep_route: null buffer");
    if (world == 0 || me >= world || num_experts == 0 || num_experts > 1024 || num_experts % world != 0)
        return dg::fail(DG_ERR_INVALID_ARG, "ep_route: %u experts over %u ranks (at most 1024 experts, divisible by the ranks)", num_experts, world);
    if (align == 0 || cap % align != 0) return dg::fail(DG_ERR_INVALID_ARG, "ep_route: capacity must be a multiple of the alignment");
    const uint32_t e_local = num_experts / world;
    if (slices == 0 || slices > e_local || slices > dg::kMaxSlices)
        return dg::fail(DG_ERR_INVALID_ARG, "ep_route: %u slices for %u local experts (at most %u)", slices, e_local, dg::kMaxSlices);
    dg::SliceBounds bounds = {};
    for (uint32_t i = 0; i <= slices; ++i) {
        // slice_first (host, slices + 1 entries, ascending from 0 to e_local); NULL = equal slices
        bounds.first[i] = slice_first ? slice_first[i] : (uint32_t)((uint64_t)e_local * i / slices);
        if (bounds.first[i] > e_local || (i > 0 && bounds.first[i] <= bounds.first[i - 1]))
            return dg::fail(DG_ERR_INVALID_ARG, "ep_route: slice bounds must ascend from 0 to %u", e_local);
    }
    if (bounds.first[0] != 0 || bounds.first[slices] != e_local)
        return dg::fail(DG_ERR_INVALID_ARG, "ep_route: slice bounds must start at 0 and end at %u", e_local);
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    dg::ep_route_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(counts, world, me, num_experts, e_local, align, cap,
                                                                           slices, bounds, dest_base, block_expert, blocks_used,
                                                                           dev->status);
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_ep_push(const void* x, uint64_t x_pitch_bytes, uint32_t row_bytes, const uint32_t* x_sf, uint32_t sf_rows,
                   uint64_t sf_cols, const int32_t* slot_src, const int32_t* my_offsets, const int32_t* dest_base,
                   uint32_t num_experts, uint32_t world, uint32_t me, uint32_t e_lo, uint32_t e_hi, uint32_t n_copies, uint64_t cap,
                   const uint64_t* a_bases, const uint64_t* sf_bases, const uint64_t* ticket_bases, uint32_t max_blocks,
                   void* stream) {
    if (!x || !x_sf || !slot_src || !my_offsets || !dest_base || !a_bases || !sf_bases || !ticket_bases)
        return dg::fail(DG_ERR_INVALID_ARG, "ep_push: null buffer");
    if (row_bytes % 16 || x_pitch_bytes % 16 || (reinterpret_cast<uintptr_t>(x) & 15u))
        return dg::fail(DG_ERR_INVALID_ARG, "ep_push: rows must be 16-byte aligned multiples of 16 bytes");
    if (world == 0 || me >= world || num_experts % world != 0) return dg::fail(DG_ERR_INVALID_ARG, "ep_push: bad rank layout");
    if (e_lo >= e_hi || e_hi > num_experts / world) return dg::fail(DG_ERR_INVALID_ARG, "ep_push: expert range [%u, %u) outside the %u local experts", e_lo, e_hi, num_experts / world);
    if (n_copies == 0) return DG_OK;
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    uint32_t blocks = dg::ceil_div(n_copies, 8u);
    if (max_blocks && blocks > max_blocks) blocks = max_blocks;
    dg::ep_push_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x), x_pitch_bytes / 16, row_bytes / 16, x_sf, sf_rows, sf_cols, slot_src, my_offsets, dest_base,
        num_experts, num_experts / world, e_lo, e_hi, world, me, cap, reinterpret_cast<const unsigned long long*>(a_bases),
        reinterpret_cast<const unsigned long long*>(sf_bases), reinterpret_cast<const unsigned long long*>(ticket_bases));
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

int32_t dg_ep_return_ptrs(uint64_t* tickets, uint32_t slots, const uint64_t* ret_bases, uint32_t world, uint64_t row_bytes,
                          const int32_t* block_expert, uint32_t align, uint64_t* ptrs, void* stream) {
    if (!tickets || !ret_bases || !ptrs) return dg::fail(DG_ERR_INVALID_ARG, "ep_return_ptrs: null buffer");
    if (row_bytes % 16 != 0) return dg::fail(DG_ERR_INVALID_ARG, "ep_return_ptrs: rows must be multiples of 16 bytes");
    if (block_expert && align == 0) return dg::fail(DG_ERR_INVALID_ARG, "ep_return_ptrs: zero alignment");
    if (slots == 0) return DG_OK;
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    dg::ep_return_ptrs_kernel<<<dg::ceil_div(slots, 256u), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<unsigned long long*>(tickets), slots, reinterpret_cast<const unsigned long long*>(ret_bases), world,
        row_bytes, block_expert, align, reinterpret_cast<unsigned long long*>(ptrs));
    dg::note_launch();
    DG_CUDA_CHECK(cudaGetLastError());
    return DG_OK;
}

}  // extern "C"
