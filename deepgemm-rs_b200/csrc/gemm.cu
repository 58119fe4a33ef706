// Block-scaled GEMM for sm_100a: D[M,N] (+)= A[M,K] . B[N,K]^T on tcgen05 tensor cores.
//
// One persistent kernel covers the reference's dense, M-grouped contiguous and M-grouped
// masked GEMMs (api::gemm_nt / m_grouped_gemm_nt_contiguous / m_grouped_gemm_nt_masked,
// deepgemm/src/api.rs:648-963, whose device side is gemm_sm100_impl in
// deepgemm/kernels/gemm_sm100.cu:442-891), for three operand kinds:
//   FP8  E4M3 x E4M3, UE8M0 scales per 32 or 128 K  -> tcgen05.mma kind::mxf8f6f4.block_scale
//   FP4  E2M1 x E2M1 (packed), UE8M0 scales per 32 K -> tcgen05.mma kind::mxf4.block_scale.block32
//   BF16                                              -> tcgen05.mma kind::f16
// Numerical contract: gemm_ref of the reference's golden model (deepgemm/src/golden.rs:444-458)
// within calc_diff <= 1e-3 (FP8) / 2e-3 (FP4).
//
// Structure of a CTA (256 threads, one CTA per SM, 128 x BLOCK_N output tiles):
//   warp 0   TMA producer: A / B tiles (128B-swizzled, K-major) and packed-SF rows into a
//            multi-stage shared-memory ring, one mbarrier per stage
//   warp 1   MMA issuer: scale factors shared memory -> TMEM (tcgen05.cp), then 4 MMAs per
//            k-block; tcgen05.commit frees the stage / publishes the accumulator
//   warp 2   scale-factor transposer: rewrites each 128-word SF row from [4][32] to [32][4]
//            order, the layout tcgen05.cp.32x128b.warpx4 needs; also owns TMEM alloc/free
//   warps 4-7 epilogue: TMEM -> registers -> bf16/f32 -> global, double-buffered against the
//            next tile's main loop (two accumulator stages in TMEM)
// BLOCK_N, the stage count and the scale granularities are run-time parameters: the TMA boxes
// come from the tensor maps and the MMA shape from a run-time instruction descriptor.
#include "host.h"

#include <mutex>
#include "ptx.cuh"

#include <cstdio>
#include <cstdlib>

namespace dg {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kMaxStages = 10;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccStageCols = 256;   // accumulator stage s starts at column s * 256
// Scale factors live above the <=224-wide accumulators, in two sets that take turns: set 0 in columns
// 224..255, set 1 in 480..511; inside a set A's rows start at +0 (<= 8 columns), B's at +8 (<= 24).
__host__ __device__ constexpr uint32_t sf_set_col(uint32_t set) { return set ? 480u : 224u; }
constexpr uint32_t kSfaOff = 0;
constexpr uint32_t kSfbOff = 8;
constexpr uint32_t kSmemBarrierBytes = 1024;
constexpr uint32_t kMaxPairedBlocks = 4096;   // contiguous layout on CTA pairs: m_indices entries the in-kernel tile list holds
constexpr uint32_t kPairedListBytes = 17 * 1024;  // tile list + run list (u16 each), 1024-aligned

enum Kind : int { kFp8 = 0, kFp4 = 1, kBf16 = 2 };
enum GType : int { kNormal = 0, kContiguous = 1, kMasked = 2, kBatched = 3 };

struct GemmParams {
    uint32_t m;            // rows of A/D (normal, contiguous); rows per group (masked)
    uint32_t n;            // columns of D = rows of B per group
    uint32_t num_groups;
    uint32_t num_k_blocks;
    uint32_t block_n;
    uint32_t num_m_blocks; // normal / contiguous
    uint32_t num_n_blocks;
    uint32_t band;         // m-blocks per L2 band
    uint32_t num_stages;
    uint32_t stage_bytes;  // A + B + SFA + SFB, 1024-aligned
    uint32_t off_b, off_sfa, off_sfb;
    uint32_t sf_cp_by_mma;            // host-side choice of the instantiation: 1 = the MMA issuer copies the SF rows into tensor memory itself, 0 = the SF warp does (single CTAs)
    uint32_t sf_load_mask;            // SF rows of both operands are loaded on k-blocks with (kb & mask) == 0: every k-block, or every fourth when both operands carry per-128 scales
    uint32_t sfa_shift, sfb_shift;    // log2 of the k-blocks per packed SF row: 0 (gran 32) or 2 (gran 128); shifts and masks, no run-time division in the k-loops
    uint32_t sfb_chunks;   // 128-row chunks of the B scale factors per tile
    uint32_t sf_sub;       // SF rows per k-block: 1 (FP8) or 2 (FP4)
    uint32_t tx_ab, tx_sfa, tx_sfb;
    uint32_t out_f32, accumulate;
    uint64_t ldd;          // D row pitch in elements
    void* d;
    const int32_t* layout; // m_indices (contiguous) or masked_m (masked)
    const int32_t* d_row_map;  // optional: D row of every A row (negative = drop the row); NULL = identity
    const uint64_t* d_row_ptr; // optional (contiguous, bf16): address of every A row's D row, this or a peer GPU's (0 = drop)
    const int32_t* a_row_src;  // GA kernels: row of the A buffer that holds row r of the (never materialised) grouped matrix
    const int32_t* m_blocks_dev;  // optional (contiguous, single CTA): device-side count of leading 128-row blocks to visit
    uint32_t* tile_counter;       // dynamic schedule: [0] next tile id, [1] CTAs that have finished; both zero at launch
    uint32_t sched_runs;          // dynamic schedule: bands restart at every run of equal m_indices entries (0 = plain bands)
    uint32_t* status;
    uint32_t k_splits;          // dense GEMM with few tiles: K is cut into this many ranges (1 = off)
    uint32_t kb_per_split;      // k-blocks per range (a multiple of 4)
    float* split_ws;            // f32 partial tiles [k_splits][m][n] when k_splits > 1
    float alpha;                // factor on the product before the output cast (1 = none)
    uint32_t idesc;             // tcgen05 instruction descriptor
    uint32_t tail_n;            // width of the last column tile when it is narrower than block_n (rounded up to 16; 0 = none): that tile loads and multiplies only its own columns
    uint32_t idesc_tail;        // instruction descriptor of that tile
    uint32_t tx_ab_tail;        // bytes of its A and B tiles per k-block and CTA
    uint32_t b_group_rows;      // rows of B per group (grouped GEMMs); >= n when only a column range is computed
    uint32_t b_row_offset;      // first B row inside every group
    uint32_t sf_rows_a, sf_rows_b;  // batched: packed SF rows per batch
    // MN-major operand views ([K, MN] buffers; the MNM instantiation only)
    uint32_t a_mn, b_mn;        // 1 = the operand is MN-major
    uint32_t a_boxes, b_boxes;  // TMA boxes (one 128-byte swizzle atom wide, BLOCK_K rows deep) per stage
    uint32_t box_elems;         // MN elements per box (128 for FP8, 64 for BF16)
    uint32_t box_bytes;         // bytes per box = distance between neighbouring atoms along MN (LBO)
    uint32_t mn_kstep;          // descriptor advance (16-byte units) per MMA along K for an MN-major operand
    uint32_t k_elems;           // K per batch in elements (first K row of batch b = b * k_elems)
};

struct Tile {
    uint32_t a_row;     // first row in A / SFA-column / D coordinates
    uint32_t row_end;   // rows >= row_end are not stored
    uint32_t n0;        // first column of D
    uint32_t b_row;     // first row in (stacked) B / SFB-column coordinates
    uint32_t kb0, kb1;  // k-block range of this work item
    uint32_t split;     // index of the K range (0 without split-K)
    uint32_t mn_a;      // batched: first row of the tile inside its batch (SFA column, MN coordinate of an MN-major A)
    uint32_t batch;     // batched: index of the batch
    bool skip;
    bool tail;          // the narrow last column tile
};

// Static persistent schedule: cluster c (one CTA, or a CTA pair) takes tiles c, c + C, c + 2C, ...
// A tile is (128 * CL) x BLOCK_N; CTA `rank` of a pair owns rows [rank*128, rank*128 + 128) of it.
// Tile ids walk bands of `band` m-tiles, m fastest inside a band, so that the tiles in flight
// share a few A row-blocks and B column-blocks in L2.
// DYN (contiguous layout, single CTA): tile ids are not strided but claimed one by one from a global
// counter by the CTA's scheduler warp and handed to the roles through a small ring in shared memory,
// so that a CTA that is slowed down (an SM shared with another kernel, a slow tile) simply takes
// fewer tiles instead of holding up the whole grid.
constexpr uint32_t kSchedRing = 4;
constexpr uint32_t kSchedRunBytes = 4096; // dynamic schedule: room for the run list behind the barrier block
constexpr uint32_t kSchedMaxRuns = kSchedRunBytes / 2 - 1;   // runs of equal m_indices entries the scheduler warp keeps (u16 first blocks + end)
struct SchedRing {
    uint64_t full[kSchedRing];     // scheduler warp -> roles: tile published
    uint64_t empty[kSchedRing];    // roles -> scheduler warp: every role has read the tile
    uint64_t tile[kSchedRing];     // (m block << 32) | n block; m block 0xffffffff = no more tiles
};

template <int GTYPE, int CL, bool SPLIT = false, bool DYN = false>
struct Scheduler {
    uint32_t next_id, stride, rank;
    SchedRing* ring = nullptr;         // DYN
    const WaitCtx* wc = nullptr;
    uint32_t slot = 0, ring_phase = 0;
    uint32_t g = 0, g_first_tile = 0;  // masked: current group and its first tile id
    const uint16_t* mtiles = nullptr;  // contiguous on CTA pairs: first block of every m-tile, bit 15 = both blocks share the expert
    const uint16_t* run_first = nullptr;  // first m-tile of every run of equal experts, [n_runs + 1]
    uint32_t n_mtiles = 0, n_runs = 0;
    __device__ explicit Scheduler(uint32_t rank_) : next_id(blockIdx.x / CL), stride(gridDim.x / CL), rank(rank_) {}
    __device__ Scheduler(uint32_t rank_, const uint16_t* mt, uint32_t n, const uint16_t* rf, uint32_t nr)
        : next_id(blockIdx.x / CL), stride(gridDim.x / CL), rank(rank_), mtiles(mt), run_first(rf), n_mtiles(n), n_runs(nr) {}
    __device__ bool first_tile_pending() const { return next_id == blockIdx.x / CL + stride; }
    __device__ void attach(SchedRing* r, const WaitCtx* w) { ring = r; wc = w; }

    // Called by all lanes of a converged warp; the result is warp-uniform.
    __device__ bool next(const GemmParams& p, Tile& t) {
        constexpr uint32_t kTileM = kBlockM * CL;
        uint32_t id = next_id;
        next_id += stride;
        if (DYN) {
            // the scheduler warp has already turned the claimed id into a tile (contiguous layout, one CTA)
            if (!DG_WARP_WAIT(smem_u32(&ring->full[slot]), ring_phase, *wc, kWaitSched)) return false;
            const uint64_t entry = *reinterpret_cast<volatile uint64_t*>(&ring->tile[slot]);
            __syncwarp();
            if ((threadIdx.x & 31u) == 0) mbar_arrive(smem_u32(&ring->empty[slot]));
            if (++slot == kSchedRing) { slot = 0; ring_phase ^= 1u; }
            const uint32_t mb = (uint32_t)(entry >> 32), nb = (uint32_t)entry;
            if (mb == 0xffffffffu) return false;
            t.kb0 = 0; t.kb1 = p.num_k_blocks; t.split = 0;
            t.a_row = mb * kBlockM;
            t.row_end = p.m;
            t.n0 = nb * p.block_n; t.tail = p.tail_n != 0u && nb + 1u == p.num_n_blocks;
            const int32_t e = __ldg(p.layout + mb);
            t.skip = e < 0 || (uint32_t)e >= p.num_groups;
            t.b_row = (t.skip ? 0u : (uint32_t)e * p.b_group_rows + p.b_row_offset) + t.n0;
            return true;
        }
        t.skip = false;
        t.kb0 = 0; t.kb1 = p.num_k_blocks; t.split = 0;
        if (GTYPE == kContiguous && CL == 2) {
            // m-tiles come from the list built at kernel start: a pair of 128-row blocks of one
            // expert, or a single block whose partner rows (the next block, another expert's) are
            // computed by the second CTA and dropped.
            // Tile order: one expert after the other; inside an expert its m-tiles are fastest, so
            // the tiles that share a weight tile run next to each other and the expert's few A
            // blocks are reused across all its n-blocks.
            if (id >= n_mtiles * p.num_n_blocks) return false;
            uint32_t lo = 0, hi = n_runs;   // last run with run_first[run] * num_n_blocks <= id
            while (hi - lo > 1) {
                const uint32_t mid = (lo + hi) >> 1;
                if ((uint32_t)run_first[mid] * p.num_n_blocks <= id) lo = mid; else hi = mid;
            }
            const uint32_t mt0 = run_first[lo], rows = run_first[lo + 1] - mt0;
            const uint32_t rem = id - mt0 * p.num_n_blocks;
            const uint32_t nb = rem / rows, mt = mt0 + (rem - nb * rows);
            const uint32_t entry = mtiles[mt], blk = entry & 0x7fffu;
            const bool paired = (entry & 0x8000u) != 0;
            t.a_row = (blk + rank) * kBlockM;
            t.row_end = (rank == 0 || paired) ? p.m : 0u;
            t.n0 = nb * p.block_n; t.tail = p.tail_n != 0u && nb + 1u == p.num_n_blocks;
            t.b_row = (uint32_t)__ldg(p.layout + blk) * p.b_group_rows + p.b_row_offset + t.n0;
            return true;
        } else if (GTYPE != kMasked && GTYPE != kBatched) {
            uint32_t tile = id;
            // a layout sized for the worst case is mostly unused blocks: the device-side count ends the walk early
            const uint32_t m_blocks = (GTYPE == kContiguous && CL == 1 && p.m_blocks_dev)
                                          ? min(p.num_m_blocks, (uint32_t)__ldg(p.m_blocks_dev)) : p.num_m_blocks;
            if (SPLIT) {
                // work item = (tile, K range); ranges of one tile are neighbours in the order
                if (id >= p.num_m_blocks * p.num_n_blocks * p.k_splits) return false;
                tile = id / p.k_splits;
                t.split = id - tile * p.k_splits;
                t.kb0 = t.split * p.kb_per_split;
                t.kb1 = min(p.num_k_blocks, t.kb0 + p.kb_per_split);
            } else if (id >= m_blocks * p.num_n_blocks) {
                return false;
            }
            const uint32_t per_band = p.band * p.num_n_blocks;
            const uint32_t b = tile / per_band, rem = tile - b * per_band;
            const uint32_t mb0 = b * p.band;
            const uint32_t rows = min(p.band, m_blocks - mb0);
            const uint32_t nb = rem / rows, mb = mb0 + (rem - nb * rows);
            t.a_row = mb * kTileM + rank * kBlockM;
            t.row_end = p.m;
            t.n0 = nb * p.block_n; t.tail = p.tail_n != 0u && nb + 1u == p.num_n_blocks;
            t.b_row = p.b_row_offset + t.n0;
            if (GTYPE == kContiguous) {
                const int32_t e = __ldg(p.layout + mb);
                t.skip = e < 0 || (uint32_t)e >= p.num_groups;
                t.b_row = (t.skip ? 0u : (uint32_t)e * p.b_group_rows + p.b_row_offset) + t.n0;
            }
            return true;
        } else if (GTYPE == kBatched) {
            // every batch is a dense [m, n] problem of its own: A, B and D stacked along the rows, the
            // packed scale factors stacked along their K rows (transform_sf_batched's arena)
            const uint32_t mbs = (p.m + kTileM - 1) / kTileM;
            const uint32_t per_batch = mbs * p.num_n_blocks;
            if (id >= per_batch * p.num_groups) return false;
            const uint32_t b = id / per_batch, rem = id - b * per_batch;
            const uint32_t nb = rem / mbs, mb = rem - nb * mbs;
            t.batch = b;
            t.mn_a = mb * kTileM + rank * kBlockM;
            t.a_row = b * p.m + t.mn_a;
            t.row_end = b * p.m + p.m;
            t.n0 = nb * p.block_n; t.tail = p.tail_n != 0u && nb + 1u == p.num_n_blocks;
            t.b_row = b * p.b_group_rows + p.b_row_offset + t.n0;
            return true;
        } else {
            while (g < p.num_groups) {
                const int32_t mm = __ldg(p.layout + g);
                const uint32_t rows = mm <= 0 ? 0u : min((uint32_t)mm, p.m);
                const uint32_t mbs = (rows + kTileM - 1) / kTileM;
                const uint32_t cnt = mbs * p.num_n_blocks;
                if (id < g_first_tile + cnt) {
                    const uint32_t rem = id - g_first_tile;
                    const uint32_t nb = rem / mbs, mb = rem - nb * mbs;
                    t.a_row = g * p.m + mb * kTileM + rank * kBlockM;
                    t.row_end = g * p.m + rows;
                    t.n0 = nb * p.block_n; t.tail = p.tail_n != 0u && nb + 1u == p.num_n_blocks;
                    t.b_row = g * p.b_group_rows + p.b_row_offset + t.n0;
                    return true;
                }
                g_first_tile += cnt;
                ++g;
            }
            return false;
        }
    }
};

struct __align__(8) Barriers {
    uint64_t full[kMaxStages];      // A and B tiles landed (pair: both CTAs' tiles, on the leader's barrier)
    uint64_t sf_full[kMaxStages];   // this CTA's SF rows landed (only on k-blocks that load SF)
    uint64_t sf_ready[kMaxStages];  // SF rows copied into tensor memory (commit of the copies; pair: on the leader)
    uint64_t sf_free[2];            // the MMAs that read SF set s have completed (commit of the MMA issuer)
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];         // pair: the leader's barrier collects both CTAs' epilogue warps
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t n_mtiles, n_runs;
    SchedRing sched;                // dynamic schedule only
};
static_assert(sizeof(Barriers) <= kSmemBarrierBytes, "barrier block too large");

// CL = 1: one CTA per tile.  CL = 2: a CTA pair per 256-row tile (tcgen05 cta_group::2): each CTA
// loads its own 128 rows of A and its own half of the B tile, the leader CTA issues MMAs that read
// both CTAs' shared memory and write both CTAs' TMEM, each CTA drains its own accumulator.
// SPLIT (dense, single CTA only): a work item is a K range of a tile and the epilogue stores f32
// partial tiles.  It is a separate instantiation because a k-loop that starts at a run-time
// block measurably slows the common case (the k-block index feeds every role's bookkeeping).
// GA (contiguous layout, single CTA, K-major FP8): the rows of A are gathered inside the kernel -- row r of the
// grouped matrix is row p.a_row_src[r] of the buffer behind tm_a (a map whose box is one row), fetched four rows
// per TMA instruction (tile::gather4) -- so the caller need not write a permuted copy of its rows first.  A
// k-block needs 32 such instructions and a warp issues them one lane after the other (22 ns each), so extra
// warps (8 ..) share them; warp 0 still announces the bytes and loads B and the scale factors.  Measured on the
// grouped GEMM of the MoE step (2018 TFLOPS from a permuted copy): issued by warp 0 alone 695 TFLOPS, by 4 / 8 /
// 16 extra warps 1598 / 1713 / 1811.
constexpr uint32_t kGatherWarps = 16;
template <int KIND, int GTYPE, int CL, bool SPLIT, bool DYN, bool MNM = false, bool SFW = false, bool GA = false>
__global__ void __launch_bounds__(GA ? 256 + 32 * kGatherWarps : 256, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_bt,
            const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb, const GemmParams p) {
    constexpr bool kHasSf = KIND != kBf16;
    static_assert(!(SFW && CL == 2), "the SF warp copies scale factors only on single CTAs");
    static_assert(!GA || (GTYPE == kContiguous && CL == 1 && !SPLIT && !MNM && KIND == kFp8), "gathered A rows: contiguous FP8, single CTAs");
    // Whether one elected lane runs the MMA issuer's k-loop alone (no warp-wide vote and re-convergence per
    // k-block).  Measured on one B200, warp-wide -> single lane: FP4 3470 -> 4200 TFLOPS, masked FP8 1009 -> 1052,
    // split-K FP8 at M = 128 2 to 7 % faster, the contiguous grouped GEMM on 208-wide tiles (five stages) 1842 ->
    // 1994 (on 224-wide tiles, four stages, where the pipeline depth bounds it, 1849 -> 1809); dense FP8 on CTA
    // pairs 1950 -> 1925, so pairs keep the warp-wide loop.
    constexpr bool kConsLane = KIND == kFp4 || SPLIT || GTYPE == kMasked || ((GTYPE == kNormal || GTYPE == kContiguous) && CL == 1);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // Dynamic shared memory: [barriers (512 B, padded to 1024)] [stage 0] [stage 1] ...
    // (identical offsets in both CTAs of a pair: the launch gives every CTA the same window offset)
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    Barriers* bars = reinterpret_cast<Barriers*>(smem_raw + (smem_base - smem_u32(smem_raw)));
    constexpr bool kPairedContig = GTYPE == kContiguous && CL == 2;
    // [tile list, 16 KB] only for the contiguous layout on CTA pairs
    uint16_t* mtiles = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(bars) + 1024);
    uint16_t* run_first = mtiles + kMaxPairedBlocks;    // [kMaxPairedBlocks + 1], padded to 17 KB
    // [run list, 4 KB] only for the dynamic schedule
    const uint32_t stages_base = smem_base + 1024u + (kPairedContig ? kPairedListBytes : 0u) + (DYN ? kSchedRunBytes : 0u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = CL == 2 ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;
    const WaitCtx wc{p.status, &bars->abort};

    if (threadIdx.x == 0) {
        bars->abort = 0;
        for (uint32_t s = 0; s < p.num_stages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->sf_full[s]), 1);
            mbar_init(smem_u32(&bars->sf_ready[s]), SFW ? 1 : CL);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bars->sf_free[s]), 1);
            mbar_init(smem_u32(&bars->tmem_full[s]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[s]), 4 * CL);
        }
        if (DYN) {
            // readers of a tile id: producer, MMA issuer, (SF transposer,) four epilogue warps
            for (uint32_t s = 0; s < kSchedRing; ++s) {
                mbar_init(smem_u32(&bars->sched.full[s]), 1);
                mbar_init(smem_u32(&bars->sched.empty[s]), (kHasSf ? 7 : 6) + (GA ? kGatherWarps : 0u));
            }
        }
        fence_barrier_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (kHasSf) {
            tma_prefetch_desc(&tm_sfa);
            tma_prefetch_desc(&tm_sfb);
        }
    }
    if (warp == 2) {
        tmem_alloc<CL>(smem_u32(&bars->tmem_base), kTmemCols);
        tmem_relinquish<CL>();
    }
    // Everything above touches no global data; from here on the kernel before this one in the
    // stream must have finished (its outputs are this kernel's operands, layout and row tables).
    griddep_wait();
    griddep_launch_dependents();
    if (kPairedContig && warp == 3) {
        // Tile list of the contiguous layout: walk m_indices 32 blocks at a time.  Inside a run of
        // equal experts every second block starts a tile; it is a pair when the next block has
        // the same expert.  Both CTAs of a pair build the same list.
        const uint32_t nblk = p.m / kBlockM;
        uint32_t ntiles = 0, nruns = 0, carry_start = 0;
        int32_t carry_e = -2;
        for (uint32_t base = 0; base < nblk; base += 32u) {
            const uint32_t b = base + lane;
            int32_t e = -3;
            if (b < nblk) {
                e = __ldg(p.layout + b);
                if (e < 0 || (uint32_t)e >= p.num_groups) e = -1;
            }
            int32_t e_prev = __shfl_up_sync(0xffffffffu, e, 1);
            if (lane == 0) e_prev = carry_e;
            const uint32_t bnd = __ballot_sync(0xffffffffu, e != e_prev);
            const uint32_t upto = bnd & (0xffffffffu >> (31u - lane));
            const uint32_t run_start = upto ? base + (31u - (uint32_t)__clz((int)upto)) : carry_start;
            int32_t e_next = __shfl_down_sync(0xffffffffu, e, 1);
            if (lane == 31) {
                e_next = -3;
                if (b + 1 < nblk) {
                    e_next = __ldg(p.layout + b + 1);
                    if (e_next < 0 || (uint32_t)e_next >= p.num_groups) e_next = -1;
                }
            }
            const bool is_start = b < nblk && e >= 0 && ((b - run_start) & 1u) == 0;
            const uint32_t starts = __ballot_sync(0xffffffffu, is_start);
            const uint32_t my_tile = ntiles + __popc(starts & ((1u << lane) - 1u));
            if (is_start) mtiles[my_tile] = (uint16_t)(b | (e_next == e ? 0x8000u : 0u));
            // a run of a valid expert begins where the expert changes
            const bool run_begin = b < nblk && e >= 0 && e != e_prev;
            const uint32_t begins = __ballot_sync(0xffffffffu, run_begin);
            if (run_begin) run_first[nruns + __popc(begins & ((1u << lane) - 1u))] = (uint16_t)my_tile;
            nruns += __popc(begins);
            ntiles += __popc(starts);
            carry_start = __shfl_sync(0xffffffffu, run_start, 31);
            carry_e = __shfl_sync(0xffffffffu, e, 31);
        }
        if (lane == 0) {
            run_first[nruns] = (uint16_t)ntiles;
            bars->n_mtiles = ntiles;
            bars->n_runs = nruns;
        }
    }
    tc_fence_before();
    if (CL == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
    const uint32_t n_mtiles = kPairedContig ? *reinterpret_cast<volatile uint32_t*>(&bars->n_mtiles) : 0u;
    const uint32_t n_runs = kPairedContig ? *reinterpret_cast<volatile uint32_t*>(&bars->n_runs) : 0u;

    auto stage_addr = [&](uint32_t s) { return stages_base + s * p.stage_bytes; };

    if (warp == 0) {
        // ===================================================== TMA producer (warp-converged, one lane issues)
        Scheduler<GTYPE, CL, SPLIT, DYN> sched(rank, mtiles, n_mtiles, run_first, n_runs);
        sched.attach(&bars->sched, &wc);
        Tile t;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        while (ok && sched.next(p, t)) {
            if (t.skip) continue;
            const uint32_t kb_first = SPLIT ? t.kb0 : 0u, kb_count = SPLIT ? t.kb1 - t.kb0 : p.num_k_blocks;
            // the narrow last column tile has a tensor map of its own (a box of just its rows) and fewer bytes per stage
            const CUtensorMap* bmap = t.tail ? &tm_bt : &tm_b;
            const uint32_t tx_ab = t.tail ? p.tx_ab_tail : p.tx_ab;
            const uint32_t b_rows_per_cta = (t.tail ? p.tail_n : p.block_n) / CL;
            for (uint32_t ki = 0; ki < kb_count; ++ki) {
                const uint32_t kb = kb_first + ki;
                if (!(ok = DG_WARP_WAIT(smem_u32(&bars->empty[stage]), phase ^ 1u, wc, kWaitEmpty))) break;
                const uint32_t sa = stage_addr(stage);
                const bool ld_sfa = kHasSf && (kb & p.sf_load_mask) == 0, ld_sfb = ld_sfa;
                // Inner coordinate kx in elements: 128 bytes per k-block (128 FP8, 256 FP4 = 128 B, 64 BF16).
                const int32_t kx = (int32_t)(kb * (KIND == kBf16 ? 64u : 128u));
                if (elect_one()) {
                    // Scale factors go first and complete on this CTA's own barrier, so that their
                    // transposition overlaps the (much larger) A/B transfer.
                    if (ld_sfa || ld_sfb) {
                        const uint32_t sbar = smem_u32(&bars->sf_full[stage]);
                        mbar_arrive_expect_tx(sbar, (ld_sfa ? p.tx_sfa : 0u) + (ld_sfb ? p.tx_sfb : 0u));
                        // batched: the SF rows of batch b start at b * (packed rows per batch), columns count inside the batch
                        const uint32_t sfa_x = GTYPE == kBatched ? t.mn_a : t.a_row, sfb_x = GTYPE == kBatched ? t.n0 : t.b_row;
                        const uint32_t sfa_y = (GTYPE == kBatched ? t.batch * p.sf_rows_a : 0u) + (kb >> p.sfa_shift) * p.sf_sub;
                        const uint32_t sfb_y = (GTYPE == kBatched ? t.batch * p.sf_rows_b : 0u) + (kb >> p.sfb_shift) * p.sf_sub;
                        if (ld_sfa) tma_load_2d(&tm_sfa, sbar, sa + p.off_sfa, (int32_t)sfa_x, (int32_t)sfa_y);
                        if (ld_sfb) tma_load_2d(&tm_sfb, sbar, sa + p.off_sfb, (int32_t)sfb_x, (int32_t)sfb_y);
                    }
                    if (MNM) {
                        // An MN-major operand is a [K, MN] buffer: a box is one swizzle atom (128 bytes of MN)
                        // wide and BLOCK_K rows deep, neighbouring atoms along MN lie box_bytes apart.
                        const uint32_t bar = smem_u32(&bars->full[stage]);
                        mbar_arrive_expect_tx(bar, p.tx_ab);
                        const int32_t ky = (int32_t)((GTYPE == kBatched ? t.batch * p.k_elems : 0u) + (uint32_t)kx);
                        if (p.a_mn) {
                            const uint32_t mn0 = GTYPE == kBatched ? t.mn_a : t.a_row;
                            for (uint32_t i = 0; i < p.a_boxes; ++i)
                                tma_load_2d(&tm_a, bar, sa + i * p.box_bytes, (int32_t)(mn0 + i * p.box_elems), ky);
                        } else {
                            tma_load_2d(&tm_a, bar, sa, kx, (int32_t)t.a_row);
                        }
                        if (p.b_mn) {
                            const uint32_t mn0 = GTYPE == kBatched ? t.n0 + p.b_row_offset : t.b_row;
                            for (uint32_t i = 0; i < p.b_boxes; ++i)
                                tma_load_2d(&tm_b, bar, sa + p.off_b + i * p.box_bytes, (int32_t)(mn0 + i * p.box_elems), ky);
                        } else {
                            tma_load_2d(&tm_b, bar, sa + p.off_b, kx, (int32_t)t.b_row);
                        }
                    } else if (CL == 1) {
                        const uint32_t bar = smem_u32(&bars->full[stage]);
                        mbar_arrive_expect_tx(bar, tx_ab);
                        if (!GA) tma_load_2d(&tm_a, bar, sa, kx, (int32_t)t.a_row);
                        tma_load_2d(bmap, bar, sa + p.off_b, kx, (int32_t)t.b_row);
                    } else {
                        // both CTAs' tiles complete on the leader's barrier; the leader announces the bytes of both
                        if (leader) mbar_arrive_expect_tx(smem_u32(&bars->full[stage]), 2u * tx_ab);
                        const uint32_t bar = mapa(smem_u32(&bars->full[stage]), 0);
                        tma_load_2d_pair(&tm_a, bar, sa, kx, (int32_t)t.a_row);
                        tma_load_2d_pair(bmap, bar, sa + p.off_b, kx, (int32_t)(t.b_row + rank * b_rows_per_cta));
                    }
                }
                __syncwarp();
                if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1 && leader) {
        // ===================================================== MMA issuer (the warp walks the tiles, one lane issues)
        Scheduler<GTYPE, CL, SPLIT, DYN> sched(rank, mtiles, n_mtiles, run_first, n_runs);
        sched.attach(&bars->sched, &wc);
        Tile t;
        uint32_t stage = 0, phase = 0, tile_count = 0;
        uint32_t sf_bits = 0;  // per-stage parity of sf_ready (it completes only on SF k-blocks)
        uint32_t sf_set = 1;   // SF set the MMAs read; it changes at every SF k-block (the first one takes set 0)
        // The tile walk is done by the whole warp, the k-loop of a tile by one elected lane alone: warp-wide votes
        // and re-convergence on every k-block cost the issuer more than the MMAs of a k-block take to execute.
        const bool issuer = elect_one();
        const uint32_t issuer_lane = (uint32_t)__ffs(__ballot_sync(0xffffffffu, issuer)) - 1u;
        uint32_t ok = 1;
        while (ok && sched.next(p, t)) {
            if (t.skip) continue;
            const uint32_t as = tile_count & 1u, aphase = (tile_count >> 1) & 1u;
            ++tile_count;
            if (!(ok = DG_WARP_WAIT(smem_u32(&bars->tmem_empty[as]), aphase ^ 1u, wc, kWaitTmemEmpty))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem + as * kAccStageCols;
            const uint32_t idesc = t.tail ? p.idesc_tail : p.idesc;   // operand formats, tile shape and majors, built by the host
            const uint32_t kb_first = SPLIT ? t.kb0 : 0u, kb_count = SPLIT ? t.kb1 - t.kb0 : p.num_k_blocks;
            if (!kConsLane || issuer) {
            for (uint32_t ki = 0; ki < kb_count; ++ki) {
                const uint32_t kb = kb_first + ki;
                if (!(ok = kConsLane ? (uint32_t)mbar_wait(smem_u32(&bars->full[stage]), phase, wc, kWaitFull)
                                     : (uint32_t)DG_WARP_WAIT(smem_u32(&bars->full[stage]), phase, wc, kWaitFull))) break;
                if (kHasSf && (kb & p.sf_load_mask) == 0) {
                    // the SF warp has copied this k-block's scale factors into the other set (its commit arrives here)
                    if (!(ok = kConsLane ? (uint32_t)mbar_wait(smem_u32(&bars->sf_ready[stage]), (sf_bits >> stage) & 1u, wc, kWaitSfReady)
                                         : (uint32_t)DG_WARP_WAIT(smem_u32(&bars->sf_ready[stage]), (sf_bits >> stage) & 1u, wc, kWaitSfReady))) break;
                    sf_bits ^= 1u << stage;
                    if (SFW) sf_set ^= 1u;
                }
                tc_fence_after();
                const uint32_t sa = stage_addr(stage);
                const uint32_t sfa_col = tmem + sf_set_col(sf_set) + kSfaOff, sfb_col = tmem + sf_set_col(sf_set) + kSfbOff;
                if (kConsLane || elect_one()) {
                    if (kHasSf && !SFW && (kb & p.sf_load_mask) == 0) {
                        // in order with the MMAs in the tensor pipe: the copy may overwrite the set the MMAs before it read
                        const uint32_t na = p.sf_sub, nb = p.sf_sub * p.sfb_chunks;
                        for (uint32_t c = 0; c < na; ++c) tc_cp_32x128b_warpx4<CL>(sfa_col + c * 4u, make_sf_desc(sa + p.off_sfa + c * 512u));
                        for (uint32_t c = 0; c < nb; ++c) tc_cp_32x128b_warpx4<CL>(sfb_col + c * 4u, make_sf_desc(sa + p.off_sfb + c * 512u));
                    }
                    // K-major tile: 8-row groups 1024 B apart.  MN-major tile: 8 K rows of an atom are 1024 B
                    // apart (SBO), atoms along MN box_bytes apart (LBO).
                    const uint64_t a_desc = (MNM && p.a_mn) ? make_smem_desc(sa, 1024, p.box_bytes, kLayoutSw128) : make_kmajor_sw128_desc(sa);
                    const uint64_t b_desc = (MNM && p.b_mn) ? make_smem_desc(sa + p.off_b, 1024, p.box_bytes, kLayoutSw128)
                                                            : make_kmajor_sw128_desc(sa + p.off_b);
                    const uint32_t a_step = (MNM && p.a_mn) ? p.mn_kstep : 2u, b_step = (MNM && p.b_mn) ? p.mn_kstep : 2u;
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k) {
                        // 32 bytes of K per MMA (32 FP8, 64 FP4, 16 BF16): +2 in the >>4 address field of a
                        // K-major tile, that many whole K rows of 128 bytes in an MN-major one.
                        const uint64_t ad = a_desc + a_step * k, bd = b_desc + b_step * k;
                        const uint32_t acc = (ki | k) != 0u ? 1u : 0u;
                        if (KIND == kBf16) {
                            tc_mma_bf16<CL>(d_tmem, ad, bd, idesc, acc);
                        } else if (KIND == kFp8) {
                            // one SF byte per row per MMA: byte k of the word (gran 32), or the
                            // byte of this k-block within its 512-wide SF row (gran 128)
                            const uint32_t ida = p.sfa_shift == 0 ? k : (kb & 3u);
                            const uint32_t idb = p.sfb_shift == 0 ? k : (kb & 3u);
                            tc_mma_mxf8<CL>(d_tmem, ad, bd, idesc_with_sf_ids(idesc, ida, idb), acc, sfa_col, sfb_col);
                        } else {
                            // two SF bytes per row per MMA (64 elements): half-word (k & 1) of SF row (k >> 1)
                            const uint32_t sub = k >> 1, id = (k & 1u) * 2u;
                            tc_mma_mxf4<CL>(d_tmem, ad, bd, idesc_with_sf_ids(idesc, id, id), acc,
                                            sfa_col + sub * 4u, sfb_col + sub * p.sfb_chunks * 4u);
                        }
                    }
                    // free the stage in both CTAs / publish the accumulator to both epilogues (a pair: one commit
                    // whose completion signal goes to the same barrier of both CTAs; 2 to 6 % faster than two commits)
                    if (CL == 2) {
                        tc_commit_pair(smem_u32(&bars->empty[stage]));
                        if (ki + 1 == kb_count) tc_commit_pair(smem_u32(&bars->tmem_full[as]));
                    } else {
                        tc_commit<CL>(smem_u32(&bars->empty[stage]));
                        if (ki + 1 == kb_count) tc_commit<CL>(smem_u32(&bars->tmem_full[as]));
                    }
                    // last k-block that reads this SF set: once its MMAs are through, the SF warp may overwrite the set
                    if (kHasSf && SFW && (ki + 1 == kb_count || ((kb + 1u) & p.sf_load_mask) == 0)) tc_commit<CL>(smem_u32(&bars->sf_free[sf_set]));
                }
                if (!kConsLane) __syncwarp();
                if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
            }
            }
            __syncwarp();
            if (kConsLane) {
                ok = __shfl_sync(0xffffffffu, ok, issuer_lane);
                stage = __shfl_sync(0xffffffffu, stage, issuer_lane);
                phase = __shfl_sync(0xffffffffu, phase, issuer_lane);
                sf_bits = __shfl_sync(0xffffffffu, sf_bits, issuer_lane);
                sf_set = __shfl_sync(0xffffffffu, sf_set, issuer_lane);
            }
        }
    } else if (warp == 2 && kHasSf) {
        // ===================================================== SF warp: transposes the SF rows in shared memory and copies them into tensor memory
        // With SFW the copies (tcgen05.cp) are issued here, not by the MMA issuer: each costs the issuing thread
        // some 200 cycles, and the MMA issuer's loop, not the tensor pipe, bounded the single-CTA kernel.  Two sets of SF columns
        // take turns; the set written for SF k-block n was last read by the MMAs of SF k-block n - 2, whose
        // completion the MMA issuer reports on sf_free.  (Single CTAs only: on a pair the copy reads both CTAs'
        // shared memory, the leader's warp would have to wait for its partner, and that measured slower.)
        Scheduler<GTYPE, CL, SPLIT, DYN> sched(rank, mtiles, n_mtiles, run_first, n_runs);
        sched.attach(&bars->sched, &wc);
        Tile t;
        uint32_t stage = 0, sf_bits = 0, n_sf = 0;
        bool ok = true;
        while (ok && sched.next(p, t)) {
            if (t.skip) continue;
            const uint32_t kb_first = SPLIT ? t.kb0 : 0u, kb_count = SPLIT ? t.kb1 - t.kb0 : p.num_k_blocks;
            for (uint32_t ki = 0; ki < kb_count; ++ki) {
                const uint32_t kb = kb_first + ki;
                if ((kb & p.sf_load_mask) == 0) {
                    const uint32_t parity = (sf_bits >> stage) & 1u;
                    sf_bits ^= 1u << stage;
                    ok = DG_WARP_WAIT(smem_u32(&bars->sf_full[stage]), parity, wc, kWaitFull);
                    if (!ok) break;
                    const uint32_t sa = stage_addr(stage);
                    uint32_t* sfa = reinterpret_cast<uint32_t*>(smem_raw + (sa + p.off_sfa - smem_u32(smem_raw)));
                    uint32_t* sfb = reinterpret_cast<uint32_t*>(smem_raw + (sa + p.off_sfb - smem_u32(smem_raw)));
                    const uint32_t na = p.sf_sub, nb = p.sf_sub * p.sfb_chunks;
                    // Up to 6 chunks of 128 words: word of row 32*i + lane -> position lane*4 + i.
                    // All loads are issued before the first store.
                    uint4 v[6];
#pragma unroll
                    for (uint32_t c = 0; c < 6; ++c) {
                        if (c < na + nb) {
                            const uint32_t* q = c < na ? sfa + c * 128u : sfb + (c - na) * 128u;
                            v[c] = make_uint4(q[lane], q[32 + lane], q[64 + lane], q[96 + lane]);
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (uint32_t c = 0; c < 6; ++c) {
                        if (c < na + nb) {
                            uint32_t* q = c < na ? sfa + c * 128u : sfb + (c - na) * 128u;
                            *reinterpret_cast<uint4*>(q + lane * 4u) = v[c];
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (!SFW) {
                        if (lane == 0) {
                            if (CL == 1 || leader) mbar_arrive(smem_u32(&bars->sf_ready[stage]));
                            else mbar_arrive_cluster(mapa(smem_u32(&bars->sf_ready[stage]), 0));
                        }
                    } else {
                        const uint32_t set = n_sf & 1u;
                        if (n_sf >= 2u && !(ok = DG_WARP_WAIT(smem_u32(&bars->sf_free[set]), ((n_sf >> 1) - 1u) & 1u, wc, kWaitSfFree))) break;
                        tc_fence_after();
                        if (elect_one()) {
                            const uint32_t sfa_col = tmem + sf_set_col(set) + kSfaOff, sfb_col = tmem + sf_set_col(set) + kSfbOff;
                            for (uint32_t c = 0; c < na; ++c) tc_cp_32x128b_warpx4<CL>(sfa_col + c * 4u, make_sf_desc(sa + p.off_sfa + c * 512u));
                            for (uint32_t c = 0; c < nb; ++c) tc_cp_32x128b_warpx4<CL>(sfb_col + c * 4u, make_sf_desc(sa + p.off_sfb + c * 512u));
                            tc_commit<CL>(smem_u32(&bars->sf_ready[stage]));
                        }
                        __syncwarp();
                    }
                    ++n_sf;
                }
                if (++stage == p.num_stages) stage = 0;
            }
        }
    } else if (DYN && warp == 3) {
        // ===================================================== tile scheduler (dynamic schedule)
        const uint32_t m_blocks = p.m_blocks_dev ? min(p.num_m_blocks, (uint32_t)__ldg(p.m_blocks_dev)) : p.num_m_blocks;
        const uint32_t nn = p.num_n_blocks;
        const uint32_t total = m_blocks * nn;
        // Runs of equal m_indices entries (an expert's blocks; also runs of unused blocks, whose tiles
        // the roles skip).  Bands of `band` row blocks, m fastest, never straddle a run: the tiles in
        // flight then share the weight tiles of one or two experts, and an expert's weights are read
        // from DRAM once instead of once per band they fall into.  More than kSchedMaxRuns runs (or
        // more blocks than a u16 holds): plain bands over the whole layout.
        uint16_t* run_block0 = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(bars) + 1024);
        uint32_t n_runs = 0;
        if (p.sched_runs && m_blocks <= 0xffffu) {
            int32_t carry = -0x7fffffff;
            bool fits = true;
            for (uint32_t base = 0; base < m_blocks && fits; base += 32u) {
                const uint32_t b = base + lane;
                int32_t e = -0x7ffffffe;
                if (b < m_blocks) {
                    e = __ldg(p.layout + b);
                    if (e < 0 || (uint32_t)e >= p.num_groups) e = -1;
                }
                int32_t e_prev = __shfl_up_sync(0xffffffffu, e, 1);
                if (lane == 0) e_prev = carry;
                const bool begins = b < m_blocks && e != e_prev;
                const uint32_t mask = __ballot_sync(0xffffffffu, begins);
                const uint32_t pos = n_runs + __popc(mask & ((1u << lane) - 1u));
                fits = n_runs + __popc(mask) <= kSchedMaxRuns;
                if (begins && fits) run_block0[pos] = (uint16_t)b;
                n_runs += __popc(mask);
                carry = __shfl_sync(0xffffffffu, e, 31);
            }
            if (!fits) n_runs = 0;
            else if (lane == 0) run_block0[n_runs] = (uint16_t)m_blocks;
            __syncwarp();
        }
        uint32_t slot = 0, phase = 0;
        for (;;) {
            if (!DG_WARP_WAIT(smem_u32(&bars->sched.empty[slot]), phase ^ 1u, wc, kWaitSched)) break;
            uint32_t id = 0;
            if (lane == 0) id = atomicAdd(p.tile_counter, 1u);
            id = __shfl_sync(0xffffffffu, id, 0);
            uint32_t mb = 0xffffffffu, nb = 0;
            if (id < total) {
                uint32_t b0 = 0, b1 = m_blocks;                   // the run (or the whole layout) the tile lies in
                if (n_runs) {
                    uint32_t lo = 0, hi = n_runs;                 // last run with run_block0[run] * nn <= id
                    while (hi - lo > 1u) {
                        const uint32_t mid = (lo + hi) >> 1;
                        if ((uint32_t)run_block0[mid] * nn <= id) lo = mid; else hi = mid;
                    }
                    b0 = run_block0[lo];
                    b1 = run_block0[lo + 1];
                }
                const uint32_t rem = id - b0 * nn, per_band = p.band * nn;
                const uint32_t bi = rem / per_band, rem2 = rem - bi * per_band;
                const uint32_t mb0 = b0 + bi * p.band, rows = min(p.band, b1 - mb0);
                nb = rem2 / rows;
                mb = mb0 + (rem2 - nb * rows);
            }
            if (lane == 0) {
                *reinterpret_cast<volatile uint64_t*>(&bars->sched.tile[slot]) = ((uint64_t)mb << 32) | nb;
                mbar_arrive(smem_u32(&bars->sched.full[slot]));   // release: the tile is visible to the waiters
            }
            if (id >= total) break;                               // the roles read the end marker and stop as well
            if (++slot == kSchedRing) { slot = 0; phase ^= 1u; }
        }
    } else if (GA && warp >= 8) {
        // ===================================================== A rows gathered through the row list
        // Gather warp g assembles rows 32 g .. 32 g + 31 of every A tile: lanes 0 .. 7 hold four source rows each
        // (read once per tile; padding rows, negative entries, read row 0: their scale factors are zero and their
        // outputs belong to nobody) and issue one four-row load per k-block into the stage the producer announced.
        Scheduler<GTYPE, CL, SPLIT, DYN> sched(rank, mtiles, n_mtiles, run_first, n_runs);
        sched.attach(&bars->sched, &wc);
        Tile t;
        constexpr uint32_t kLanes = 32u / kGatherWarps;      // lanes of a gather warp that issue loads
        const uint32_t row0 = (warp - 8u) * (128u / kGatherWarps) + lane * 4u;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        while (ok && sched.next(p, t)) {
            if (t.skip) continue;
            int4 src = make_int4(0, 0, 0, 0);
            if (lane < kLanes) {
                src = __ldg(reinterpret_cast<const int4*>(p.a_row_src + t.a_row + row0));
                src.x = max(src.x, 0); src.y = max(src.y, 0); src.z = max(src.z, 0); src.w = max(src.w, 0);
            }
            for (uint32_t kb = 0; kb < p.num_k_blocks; ++kb) {
                if (!(ok = DG_WARP_WAIT(smem_u32(&bars->empty[stage]), phase ^ 1u, wc, kWaitEmpty))) break;
                if (lane < kLanes)
                    tma_gather4_2d(&tm_a, smem_u32(&bars->full[stage]), stage_addr(stage) + row0 * 128u, (int32_t)(kb * 128u),
                                   src.x, src.y, src.z, src.w);
                __syncwarp();
                if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ===================================================== epilogue
        Scheduler<GTYPE, CL, SPLIT, DYN> sched(rank, mtiles, n_mtiles, run_first, n_runs);
        sched.attach(&bars->sched, &wc);
        Tile t;
        const uint32_t q = warp - 4u;  // TMEM lane quarter == warp index % 4
        uint32_t tile_count = 0;
        bool ok = true;
        const bool vec_ok = (p.ldd * (p.out_f32 ? 4u : 2u)) % 16u == 0 && (reinterpret_cast<uintptr_t>(p.d) & 15u) == 0;
        while (ok && sched.next(p, t)) {
            if (t.skip) continue;
            const uint32_t as = tile_count & 1u, aphase = (tile_count >> 1) & 1u;
            ++tile_count;
            ok = DG_WARP_WAIT(smem_u32(&bars->tmem_full[as]), aphase, wc, kWaitTmemFull);
            if (!ok) break;
            tc_fence_after();
            uint32_t row = t.a_row + q * 32u + lane;
            bool row_ok = row < t.row_end;
            // rows of D addressed one by one (they may live in a peer GPU's memory)
            const bool by_ptr = GTYPE == kContiguous && !SPLIT && p.d_row_ptr != nullptr;
            uint64_t row_addr = 0;
            if (by_ptr) {
                if (row_ok) row_addr = __ldg(reinterpret_cast<const unsigned long long*>(p.d_row_ptr) + row);
                row_ok = row_ok && row_addr != 0;
            } else if (p.d_row_map && row_ok) {
                const int32_t mapped = __ldg(p.d_row_map + row);
                row_ok = mapped >= 0;
                row = (uint32_t)mapped;
            }
            const uint32_t taddr = tmem + ((q * 32u) << 16) + as * kAccStageCols;
            const uint32_t chunks = ((t.tail ? p.tail_n : p.block_n) + 31u) / 32u;   // the last chunk of a 16-column-granular tile is half used
            const uint32_t n_end = min(p.n, t.n0 + p.block_n);   // columns from here on belong to the next tile (or to nobody)
            if (!SPLIT && !p.out_f32 && !p.accumulate && (vec_ok || by_ptr) && p.n % 8u == 0) {
                // BF16 rows leave the SM in runs of 128 contiguous bytes.  A lane holds 32 columns of
                // its own row after the TMEM load; the lanes of a group of 8 exchange 16-byte pieces
                // of two neighbouring column chunks (an 8x8 transpose by shuffles) so that one store
                // instruction writes 128 bytes of one row per group: full lines for the memory
                // system and full-size packets when the row lives in a peer GPU's memory.
                const unsigned long long my_row = !row_ok ? 0ull
                    : by_ptr ? row_addr : reinterpret_cast<unsigned long long>(p.d) + (unsigned long long)row * p.ldd * 2ull;
                uint32_t c = 0;
                while (c < chunks) {
                    const uint32_t col0 = t.n0 + c * 32u;
                    const bool two = (col0 % 64u) == 0 && c + 1u < chunks;   // pairs start on 128-byte boundaries of the row
                    uint32_t r0[32], r1[32];
                    __syncwarp();
                    tmem_ld_x32(taddr + c * 32u, r0);
                    if (two) tmem_ld_x32(taddr + (c + 1u) * 32u, r1);
                    tmem_ld_wait();
                    c += two ? 2u : 1u;
                    if (c >= chunks) {
                        // accumulator drained into registers: hand the TMEM stage back to the MMA issuer
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (CL == 1 || leader) mbar_arrive(smem_u32(&bars->tmem_empty[as]));
                            else mbar_arrive_cluster(mapa(smem_u32(&bars->tmem_empty[as]), 0));
                        }
                    }
                    if (col0 >= n_end) continue;
                    uint4 a[8];
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const float al = p.alpha;
                        a[i] = make_uint4(pack_bf16x2(__uint_as_float(r0[8 * i]) * al, __uint_as_float(r0[8 * i + 1]) * al),
                                          pack_bf16x2(__uint_as_float(r0[8 * i + 2]) * al, __uint_as_float(r0[8 * i + 3]) * al),
                                          pack_bf16x2(__uint_as_float(r0[8 * i + 4]) * al, __uint_as_float(r0[8 * i + 5]) * al),
                                          pack_bf16x2(__uint_as_float(r0[8 * i + 6]) * al, __uint_as_float(r0[8 * i + 7]) * al));
                        a[4 + i] = make_uint4(pack_bf16x2(__uint_as_float(r1[8 * i]) * al, __uint_as_float(r1[8 * i + 1]) * al),
                                              pack_bf16x2(__uint_as_float(r1[8 * i + 2]) * al, __uint_as_float(r1[8 * i + 3]) * al),
                                              pack_bf16x2(__uint_as_float(r1[8 * i + 4]) * al, __uint_as_float(r1[8 * i + 5]) * al),
                                              pack_bf16x2(__uint_as_float(r1[8 * i + 6]) * al, __uint_as_float(r1[8 * i + 7]) * al));
                    }
                    if (two && col0 + 64u <= n_end) {
#pragma unroll
                        for (uint32_t sft = 4; sft >= 1; sft >>= 1) {
                            const bool up = (lane & sft) != 0;
#pragma unroll
                            for (uint32_t k = 0; k < 8; ++k) {
                                if ((k & sft) != 0) continue;
                                const uint4 send = up ? a[k] : a[k | sft];
                                uint4 recv;
                                recv.x = __shfl_xor_sync(0xffffffffu, send.x, sft);
                                recv.y = __shfl_xor_sync(0xffffffffu, send.y, sft);
                                recv.z = __shfl_xor_sync(0xffffffffu, send.z, sft);
                                recv.w = __shfl_xor_sync(0xffffffffu, send.w, sft);
                                if (up) a[k] = recv; else a[k | sft] = recv;
                            }
                        }
                        // a[i] = piece (lane % 8) of the row held by lane (lane & 24) + i
#pragma unroll
                        for (uint32_t i = 0; i < 8; ++i) {
                            const unsigned long long dst = __shfl_sync(0xffffffffu, my_row, (lane & 24u) + i);
                            if (dst) *reinterpret_cast<uint4*>(dst + col0 * 2ull + (lane & 7u) * 16ull) = a[i];
                        }
                    } else {
                        // a single chunk (64-byte runs by a 4x4 transpose inside groups of 4 lanes), or
                        // the ragged end of the row, stored piece by piece by the lane that owns the row
#pragma unroll
                        for (uint32_t h = 0; h < 2; ++h) {
                            const uint32_t cc = col0 + 32u * h;
                            if ((h == 1 && !two) || cc >= n_end) break;
                            if (cc + 32u <= n_end) {
#pragma unroll
                                for (uint32_t sft = 2; sft >= 1; sft >>= 1) {
                                    const bool up = (lane & sft) != 0;
#pragma unroll
                                    for (uint32_t k = 0; k < 4; ++k) {
                                        if ((k & sft) != 0) continue;
                                        const uint4 send = up ? a[4 * h + k] : a[4 * h + (k | sft)];
                                        uint4 recv;
                                        recv.x = __shfl_xor_sync(0xffffffffu, send.x, sft);
                                        recv.y = __shfl_xor_sync(0xffffffffu, send.y, sft);
                                        recv.z = __shfl_xor_sync(0xffffffffu, send.z, sft);
                                        recv.w = __shfl_xor_sync(0xffffffffu, send.w, sft);
                                        if (up) a[4 * h + k] = recv; else a[4 * h + (k | sft)] = recv;
                                    }
                                }
#pragma unroll
                                for (uint32_t i = 0; i < 4; ++i) {
                                    const unsigned long long dst = __shfl_sync(0xffffffffu, my_row, (lane & 28u) + i);
                                    if (dst) *reinterpret_cast<uint4*>(dst + cc * 2ull + (lane & 3u) * 16ull) = a[4 * h + i];
                                }
                            } else if (my_row) {
#pragma unroll
                                for (uint32_t i = 0; i < 4; ++i)
                                    if (cc + 8u * i + 8u <= n_end) *reinterpret_cast<uint4*>(my_row + (cc + 8u * i) * 2ull) = a[4 * h + i];
                            }
                        }
                    }
                }
                continue;
            }
            // One row's 32 columns starting at col0, as f32 bit patterns, to the output: scaled by
            // alpha, rounded to the output type, optionally added to what D holds.
            auto store_chunk = [&](const uint32_t (&r)[32], uint32_t col0) {
                if (p.out_f32) {
                    float* dst = reinterpret_cast<float*>(p.d) + (size_t)row * p.ldd + col0;
                    if (vec_ok && col0 + 32u <= n_end) {
#pragma unroll
                        for (uint32_t i = 0; i < 8; ++i) {
                            float4 v = make_float4(__uint_as_float(r[4 * i]) * p.alpha, __uint_as_float(r[4 * i + 1]) * p.alpha,
                                                   __uint_as_float(r[4 * i + 2]) * p.alpha, __uint_as_float(r[4 * i + 3]) * p.alpha);
                            if (p.accumulate) {
                                const float4 o = *reinterpret_cast<const float4*>(dst + 4 * i);
                                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                            }
                            *reinterpret_cast<float4*>(dst + 4 * i) = v;
                        }
                    } else {
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i)
                            if (col0 + i < n_end) dst[i] = __uint_as_float(r[i]) * p.alpha + (p.accumulate ? dst[i] : 0.f);
                    }
                } else {
                    __nv_bfloat16* dst = by_ptr ? reinterpret_cast<__nv_bfloat16*>(row_addr) + col0
                                                : reinterpret_cast<__nv_bfloat16*>(p.d) + (size_t)row * p.ldd + col0;
                    if ((vec_ok || by_ptr) && col0 + 32u <= n_end) {
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) {
                            uint32_t w[4];
#pragma unroll
                            for (uint32_t j = 0; j < 4; ++j)
                                w[j] = pack_bf16x2(__uint_as_float(r[8 * i + 2 * j]) * p.alpha, __uint_as_float(r[8 * i + 2 * j + 1]) * p.alpha);
                            if (p.accumulate) {
                                // D += bf16(acc), the add itself rounded to bf16 (the reference
                                // accumulates with a bf16 reduce-add, gemm_sm100.cu:309-315)
                                const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * i);
                                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                for (uint32_t j = 0; j < 4; ++j) {
                                    const float lo = __uint_as_float(ow[j] << 16) + __uint_as_float(w[j] << 16);
                                    const float hi = __uint_as_float(ow[j] & 0xffff0000u) + __uint_as_float(w[j] & 0xffff0000u);
                                    w[j] = pack_bf16x2(lo, hi);
                                }
                            }
                            *reinterpret_cast<uint4*>(dst + 8 * i) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i) {
                            if (col0 + i < n_end) {
                                __nv_bfloat16 v = __float2bfloat16_rn(__uint_as_float(r[i]) * p.alpha);
                                if (p.accumulate) v = __float2bfloat16_rn(__bfloat162float(dst[i]) + __bfloat162float(v));
                                dst[i] = v;
                            }
                        }
                    }
                }
            };
            for (uint32_t c = 0; c < chunks; ++c) {
                uint32_t r[32];
                __syncwarp();
                tmem_ld_x32(taddr + c * 32u, r);
                tmem_ld_wait();
                if (c + 1 == chunks) {
                    // accumulator drained into registers: hand the TMEM stage back to the MMA issuer
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (CL == 1 || leader) mbar_arrive(smem_u32(&bars->tmem_empty[as]));
                        else mbar_arrive_cluster(mapa(smem_u32(&bars->tmem_empty[as]), 0));
                    }
                }
                const uint32_t col0 = t.n0 + c * 32u;
                if (!row_ok || col0 >= n_end) continue;
                if (SPLIT) {
                    // partial sum of this K range
                    float* dst = p.split_ws + ((size_t)t.split * p.m + row) * p.n + col0;
                    if (p.n % 4 == 0 && col0 + 32u <= n_end) {
#pragma unroll
                        for (uint32_t i = 0; i < 8; ++i)
                            *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                                                  __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                    } else {
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i)
                            if (col0 + i < n_end) dst[i] = __uint_as_float(r[i]);
                    }
                    continue;
                }
                store_chunk(r, col0);
            }
        }
    }

    // The peer's shared memory and barriers are in use until the leader's last MMA and commit have
    // completed, which every epilogue has observed by now: both CTAs leave together.
    tc_fence_before();
    if (CL == 2) cluster_sync_all(); else __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<CL>(tmem, kTmemCols);
    }
    if (DYN && threadIdx.x == 0) {
        // the last CTA to leave puts the counters back to zero for the next launch that uses them
        __threadfence();
        if (atomicAdd(p.tile_counter + 1, 1u) == gridDim.x - 1u) {
            p.tile_counter[0] = 0;
            p.tile_counter[1] = 0;
            __threadfence();
        }
    }
}

// Second pass of a split-K GEMM: D[r][c] (+)= alpha * sum over the K ranges, added in range order (fixed, so
// results repeat bit for bit), rounded once to the output type.  Four columns per thread; launched with
// the programmatic-serialization attribute, so its blocks are resident when the GEMM's last CTA leaves.
__global__ void __launch_bounds__(256) split_reduce_kernel(const float* __restrict__ ws, uint32_t splits, uint32_t m, uint32_t n,
                                                          void* __restrict__ d, uint64_t ldd, uint32_t out_f32, uint32_t accumulate,
                                                          float alpha) {
    // lets the next kernel of the stream become resident (its set-up runs) as soon as this one is
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t n4 = (n + 3u) / 4u;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)m * n4) return;
    const uint32_t r = (uint32_t)(idx / n4), c = (uint32_t)(idx % n4) * 4u;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool vec = n % 4u == 0;
    for (uint32_t s = 0; s < splits; ++s) {
        const float* src = ws + ((size_t)s * m + r) * n + c;
        if (vec) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src));
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        } else {
            for (uint32_t i = 0; i < 4u; ++i) if (c + i < n) acc[i] += __ldcg(src + i);
        }
    }
    for (uint32_t i = 0; i < 4u; ++i) {
        if (c + i >= n) break;
        const float v = acc[i] * alpha;
        if (out_f32) {
            float* o = reinterpret_cast<float*>(d) + (size_t)r * ldd + c + i;
            *o = accumulate ? *o + v : v;
        } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(d) + (size_t)r * ldd + c + i;
            __nv_bfloat16 b = __float2bfloat16_rn(v);
            if (accumulate) b = __float2bfloat16_rn(__bfloat162float(*o) + __bfloat162float(b));
            *o = b;
        }
    }
}

// ============================================================================ host side
struct Plan {
    GemmParams p;
    CUtensorMap tb_tail;   // B with a box of the narrow last column tile's rows (a copy of B's map when there is none)
    uint32_t smem_bytes;
    uint32_t grid;
    uint32_t num_tiles;
    uint32_t cluster;   // CTAs per tile: 1, or 2 (CTA pair)
    bool dynamic;       // tiles claimed from a global counter instead of strided (contiguous layout, single CTA)
};

// A pair of zeroed counters for one launch of the dynamic schedule.  Launches take the pairs of the
// device's pool (allocated and cleared with the device entry, outside any stream) in turn; a kernel
// leaves its pair zeroed, so a pair is reusable as soon as the launch that used it has finished, and
// 256 pairs outlast any realistic number of GEMMs in flight.  A launch recorded into a CUDA graph
// would keep its pair for the life of the graph and collide with later eager launches, so captured
// launches use the static schedule instead (see run_gemm).
static uint32_t* tile_counters(const DeviceInfo* dev) {
    static std::mutex mu;
    static uint32_t next[64] = {0};
    std::lock_guard<std::mutex> lock(mu);
    return dev->tile_pool + 2u * (next[dev->device & 63]++ % kTilePoolPairs);
}

static uint32_t env_u32(const char* name, uint32_t dflt) {
    const char* v = getenv(name);
    return v && *v ? (uint32_t)strtoul(v, nullptr, 10) : dflt;
}

// Tile choice.  A tile is (128 * cluster) x BLOCK_N with BLOCK_N in {32..224 step 32} (256 for
// BF16, which needs no SF columns in TMEM), chosen to minimise waves x per-tile cost, where a
// tile's cost is its MMA time (~BLOCK_N) plus a share of its operand traffic and a fixed part.
// DG_BLOCK_N / DG_NUM_STAGES / DG_CLUSTER override (the reference's DG_* overrides: heuristics.rs:41-58).
static uint32_t pick_block_n(int kind, uint32_t m_tiles_total, uint32_t n, uint32_t units, uint32_t step = 32) {
    const uint32_t max_bn = kind == kBf16 ? 256u : 224u;
    const uint32_t forced = env_u32("DG_BLOCK_N", 0);
    if (forced >= step && forced <= max_bn && forced % (step == 32 ? 16u : step) == 0) return forced;   // K-major B: any multiple of 16
    uint32_t best = step;
    double best_cost = 1e30;
    for (uint32_t bn = step; bn <= max_bn; bn += step) {
        const uint64_t tiles = (uint64_t)m_tiles_total * ceil_div(n, bn);
        const uint64_t waves = (tiles + units - 1) / units;
        const double per_tile = (double)bn + 0.25 * (128.0 + bn) + 24.0;
        const double cost = (double)waves * per_tile;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
    }
    return best;
}

// Dense FP8 with per-128 scales: tile shape from measured tile times.  A tile of kb k-blocks takes about
// fixed + kb * per_kb nanoseconds (B200, 4096 x 7168 x {2048, 16384}, both modes; widths are multiples of 16, the 224-wide
// single-CTA tile has four pipeline stages where 192 has five, hence its jump; a CTA pair takes the same
// time per k-block at every width), and a launch takes waves x tile time.
static void pick_dense_fp8_tile(uint32_t m, uint32_t groups, uint32_t n, uint32_t kb, uint32_t sms, uint32_t* cl_out, uint32_t* bn_out,
                                bool pairs_allowed = true) {
    static const uint32_t widths[8] = {64, 96, 128, 160, 176, 192, 208, 224};
    static const double single_kb[8] = {214, 233, 273, 331, 355, 361, 394, 537};
    static const double pair_kb[8] = {423, 417, 414, 392, 0, 442, 0, 447};   // 0: not measured, not offered
    double best = 1e30;
    for (uint32_t cl = 1; cl <= ((m > kBlockM && pairs_allowed) ? 2u : 1u); ++cl) {
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t bn = widths[i];
            if (cl == 2 && pair_kb[i] == 0) continue;
            const uint64_t tiles = (uint64_t)groups * ceil_div(m, kBlockM * cl) * ceil_div(n, bn);
            const uint64_t waves = (tiles + sms / cl - 1) / (sms / cl);
            const double cost = (double)waves * (cl == 1 ? 1300.0 + kb * single_kb[i] : 400.0 + kb * pair_kb[i]);
            if (cost < best) { best = cost; *cl_out = cl; *bn_out = bn; }
        }
    }
}

static int32_t make_plan(int kind, int gtype, uint32_t m, uint32_t n, uint32_t k, uint32_t num_groups,
                         uint32_t expected_m, uint32_t gran_a, uint32_t gran_b, const DeviceInfo* dev, Plan* plan,
                         bool allow_dynamic = true, bool a_mn = false, bool b_mn = false) {
    GemmParams& p = plan->p;
    p = GemmParams{};
    const uint32_t sms = (uint32_t)dev->sm_count;
    const uint32_t block_k = kind == kFp4 ? 256u : (kind == kFp8 ? 128u : 64u);
    p.m = m; p.n = n; p.num_groups = num_groups;
    p.num_k_blocks = k / block_k;
    // CTA pairs (256-row tiles) halve the B traffic per SM; they need at least two row blocks
    // that share B.  In the contiguous grouped layout the kernel pairs neighbouring blocks of one
    // expert and runs an odd last block with an idle partner.
    const uint32_t rows_per_group = gtype == kMasked ? (expected_m ? expected_m : m) : m;
    // Measured on B200: pairs win for FP8 / BF16 dense and masked GEMMs; FP4 (scale factors on
    // every k-block, twice the UTCCP traffic) and the contiguous layout (an expert's weights are
    // shared by only a few row blocks) run faster on single CTAs.
    // With FP8 scale factors per 32 (copies into TMEM on every k-block, issued for both CTAs) pairs lose: 960 against
    // 1570 TFLOPS on 4096 x 7168 x 16384.
    const bool sf_every_block = kind == kFp8 && (gran_a == 32 || gran_b == 32);
    uint32_t cl = (rows_per_group > kBlockM && kind != kFp4 && gtype != kContiguous && !sf_every_block) ? 2u : 1u;
    const uint32_t forced_cl = env_u32("DG_CLUSTER", 0);
    if (forced_cl == 1 || forced_cl == 2) cl = forced_cl;
    if (gtype == kContiguous && m / kBlockM > kMaxPairedBlocks) cl = 1;   // the in-kernel tile list is bounded
    if (a_mn || b_mn) cl = 1;   // MN-major tiles are loaded atom by atom by one CTA
    uint32_t dense_bn = 0;
    if (kind == kFp8 && (gtype == kNormal || gtype == kMasked) && gran_a == 128 && gran_b == 128 && !a_mn && !b_mn &&
        (gtype == kMasked || m > kBlockM) && forced_cl == 0 && env_u32("DG_BLOCK_N", 0) == 0)
        pick_dense_fp8_tile(rows_per_group, gtype == kMasked ? num_groups : 1u, n, p.num_k_blocks, sms, &cl, &dense_bn);   // masked: expected rows per group
    // the contiguous grouped layout on single CTAs: the same table (208 columns and five stages for N = 4096: 1994
    // against 1849 TFLOPS on 224 columns and four)
    if (kind == kFp8 && gtype == kContiguous && cl == 1 && gran_a == 128 && gran_b == 128 && !a_mn && !b_mn && env_u32("DG_BLOCK_N", 0) == 0)
        pick_dense_fp8_tile(m, 1u, n, p.num_k_blocks, sms, &cl, &dense_bn, false);
    plan->cluster = cl;
    const uint32_t tile_m = kBlockM * cl;
    const uint32_t units = sms / cl;
    uint32_t m_tiles_total;
    if (gtype == kMasked) m_tiles_total = num_groups * ceil_div(rows_per_group, tile_m);
    else if (gtype == kBatched) m_tiles_total = num_groups * ceil_div(m, tile_m);
    else m_tiles_total = ceil_div(m, tile_m);
    // an MN-major B is loaded in whole swizzle atoms of 128 bytes along N: 128 columns of FP8, 64 of BF16
    p.block_n = dense_bn ? dense_bn : pick_block_n(kind, m_tiles_total, n, units, b_mn ? (kind == kBf16 ? 64u : 128u) : 32u);
    p.num_m_blocks = ceil_div(m, tile_m);
    p.num_n_blocks = ceil_div(n, p.block_n);
    // Split-K for weight-streaming shapes (a single row block, long K): with one tile per SM at
    // best, the k-loop latency of a tile bounds the run, so K is cut into ranges that run on
    // otherwise idle SMs; partial tiles are summed in range order by a second kernel.
    p.k_splits = 1;
    p.kb_per_split = p.num_k_blocks;
    if (gtype == kNormal && cl == 1 && !a_mn && !b_mn && m <= kBlockM && p.num_k_blocks >= 16 && env_u32("DG_SPLIT_K", 1)) {
        // Cost of a (tile width, K ranges) choice in nanoseconds, fitted to a sweep on B200 (M = 128, rotating
        // weights): the longer of the busiest CTA's k-loop (its k-blocks x the measured time per k-block of that
        // width) and the weight stream from DRAM, a fixed part per wave, and the second kernel: a fixed part plus
        // one pass over the f32 partial tiles per range.  Few ranges on narrow tiles beat many on wide ones.
        const uint32_t forced_bn = env_u32("DG_BLOCK_N", 0);
        uint32_t best_bn = p.block_n, best_splits = 1;
        double best_cost = 1e30;
        static const uint32_t widths[6] = {96, 128, 160, 192, 208, 224};
        static const double kb_ns[6] = {233, 273, 331, 361, 394, 537};
        const double stream_ns = (double)n * k * (kind == kBf16 ? 2.0 : (kind == kFp4 ? 0.5 : 1.0)) / 5.5e3;
        for (uint32_t i = 0; i < 6; ++i) {
            const uint32_t bn = widths[i];
            if (forced_bn && bn != forced_bn) continue;
            const uint32_t tiles = ceil_div(n, bn);
            for (uint32_t sp = 1; sp <= 16; ++sp) {
                const uint32_t per = align_up(ceil_div(p.num_k_blocks, sp), 4);
                if (ceil_div(p.num_k_blocks, per) != sp) continue;
                const uint32_t waves = ceil_div(tiles * sp, sms);
                const double cost = std::max((double)waves * per * kb_ns[i], stream_ns) + waves * 1000.0 +
                                    (sp > 1 ? 2500.0 + sp * ((double)m * n * 4.0 / 3.5e3) : 0.0);
                if (cost < best_cost) { best_cost = cost; best_bn = bn; best_splits = sp; }
            }
        }
        const uint32_t forced_sp = env_u32("DG_SPLIT_K", 1);
        if (forced_sp > 1) best_splits = forced_sp;
        p.block_n = best_bn;
        p.num_n_blocks = ceil_div(n, p.block_n);
        p.kb_per_split = align_up(ceil_div(p.num_k_blocks, best_splits), 4);
        p.k_splits = ceil_div(p.num_k_blocks, p.kb_per_split);
    }
    p.band = env_u32("DG_BAND", 8 / cl);
    if (p.band == 0) p.band = 8 / cl;
    const bool has_sf = kind != kBf16;
    p.sf_sub = kind == kFp4 ? 2u : 1u;
    p.sfb_chunks = ceil_div(p.block_n, 128u);
    p.sfa_shift = gran_a == 128 ? 2u : 0u;
    p.sfb_shift = gran_b == 128 ? 2u : 0u;
    p.sf_load_mask = (gran_a == 128 && gran_b == 128) ? 3u : 0u;
    // Who copies the SF rows into tensor memory (tcgen05.cp, some 200 cycles of issue time each).  FP8 with per-128
    // scales on single CTAs: the SF warp, which takes the copies off the MMA issuer's loop (grouped GEMM 1710 ->
    // 1776 TFLOPS, M = 128 shapes 2 to 4 % faster).  SF on every k-block (FP4, per-32 FP8): the SF warp's own loop
    // (transposition + up to six copies) then becomes the limit, the MMA issuer keeps the copies.  CTA pairs: the
    // MMA issuer as well (dense FP8 2411 against 2317 TFLOPS).  The choice is a template parameter: as a run-time
    // branch in the k-loop it cost the pair kernel 13 %.
    p.sf_cp_by_mma = env_u32("DG_SF_CP_BY_MMA", p.sf_load_mask == 0 ? 1u : 0u);
    // per CTA; a K-major tile holds its rows x 128 bytes of K, an MN-major one whole atoms of 128 bytes x BLOCK_K rows
    const uint32_t block_k_rows = kind == kBf16 ? 64u : 128u;
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.box_elems = kind == kBf16 ? 64u : 128u;
    p.box_bytes = 128u * block_k_rows;
    p.a_boxes = kBlockM / p.box_elems;
    p.b_boxes = ceil_div(p.block_n, p.box_elems);
    p.mn_kstep = (kind == kBf16 ? 16u : 32u) * 128u / 16u;
    p.k_elems = k;
    const uint32_t a_bytes = kBlockM * 128u, b_bytes = b_mn ? p.b_boxes * p.box_bytes : p.block_n / cl * 128u;
    const uint32_t sfa_bytes = has_sf ? p.sf_sub * 512u : 0u;
    const uint32_t sfb_bytes = has_sf ? p.sf_sub * p.sfb_chunks * 512u : 0u;
    p.off_b = a_bytes;
    p.off_sfa = align_up(a_bytes + b_bytes, 1024u);
    p.off_sfb = p.off_sfa + sfa_bytes;
    p.stage_bytes = align_up(p.off_sfb + sfb_bytes, 1024u);
    p.tx_ab = a_bytes + b_bytes;
    p.tx_sfa = sfa_bytes;
    p.tx_sfb = sfb_bytes;
    const uint32_t budget = (uint32_t)dev->smem_optin;
    plan->dynamic = allow_dynamic && gtype == kContiguous && cl == 1 && p.k_splits == 1 && env_u32("DG_DYNAMIC", 1) != 0;
    const uint32_t fixed = 1024u /*alignment slack*/ + 1024u /*barriers*/ +
                           ((gtype == kContiguous && cl == 2) ? kPairedListBytes : 0u) /*tile and run lists*/ +
                           (plan->dynamic ? kSchedRunBytes : 0u) /*run list of the scheduler warp*/;
    uint32_t stages = (budget - fixed) / p.stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    const uint32_t forced = env_u32("DG_NUM_STAGES", 0);
    if (forced >= 2 && forced <= stages) stages = forced;
    if (stages < 2) return fail(DG_ERR_RUNTIME, "shared memory budget %u B too small for a %u-wide tile", budget, p.block_n);
    p.num_stages = stages;
    plan->smem_bytes = fixed + stages * p.stage_bytes;
    plan->num_tiles = (gtype == kMasked || gtype == kBatched) ? m_tiles_total * p.num_n_blocks : p.num_m_blocks * p.num_n_blocks * p.k_splits;
    uint32_t clusters = units;
    uint32_t worst = gtype == kMasked ? num_groups * ceil_div(m, tile_m) * p.num_n_blocks : plan->num_tiles;
    if (gtype == kContiguous && cl == 2) worst = (m / kBlockM) * p.num_n_blocks;   // every block may be a tile of its own
    if (worst < clusters) clusters = worst;
    if (clusters == 0) clusters = 1;
    plan->grid = clusters * cl;
    p.status = dev->status;
    p.tile_counter = nullptr;
    p.sched_runs = env_u32("DG_SCHED_RUNS", 1);
    if (env_u32("DG_PRINT_CONFIGS", 0))
        fprintf(stderr, "[deepgemm_b200] kind=%d gtype=%d m=%u n=%u k=%u groups=%u -> tile %ux%ux%u cluster=%u stages=%u smem=%u grid=%u tiles=%u\n",
                kind, gtype, m, n, k, num_groups, tile_m, p.block_n, block_k, cl, stages, plan->smem_bytes, plan->grid, plan->num_tiles);
    return DG_OK;
}

static bool pdl_enabled() {
    static const bool on = env_u32("DG_PDL", 1) != 0;
    return on;
}

template <int KIND, int GTYPE, int CL, bool SPLIT = false, bool DYN = false, bool MNM = false, bool SFW = false, bool GA = false>
static int32_t launch(const Plan& plan, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa,
                      const CUtensorMap& tsb, cudaStream_t s) {
    auto* fn = gemm_kernel<KIND, GTYPE, CL, SPLIT, DYN, MNM, SFW, GA>;
    static thread_local uint32_t configured[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured[dev & 63] < plan.smem_bytes) {
        DG_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem_bytes));
        configured[dev & 63] = plan.smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(GA ? 256 + 32 * kGatherWarps : 256);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: the set-up of this kernel overlaps the tail of the one before it
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    if (env_u32("DG_PRINT_CONFIGS", 0)) {
        int clusters = -1;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg);
        fprintf(stderr, "[deepgemm_b200] launch: grid %u, cluster %d, smem %u: %d clusters can be resident (%s)\n", plan.grid, CL,
                plan.smem_bytes, clusters, cudaGetErrorString(e));
    }
    DG_CUDA_CHECK(cudaLaunchKernelEx(&cfg, fn, ta, tb, plan.tb_tail, tsa, tsb, plan.p));
    note_launch();
    return DG_OK;
}

static const char* dtype_name(int32_t d) {
    switch (d) { case DG_FP8: return "FP8"; case DG_FP4: return "FP4"; case DG_BF16: return "BF16"; case DG_F32: return "F32"; }
    return "?";
}

// Checks of deepgemm/src/api.rs:995-1022 (K multiples) and :175-185 (SF presence, majors).
static int32_t validate_operand(const dg_operand_t* op, const char* name) {
    if (!op || !op->data) return fail(DG_ERR_INVALID_ARG, "%s: null operand", name);
    const uint32_t k = op->k;
    switch (op->dtype) {
        case DG_FP4: if (k % 256 != 0) return fail(DG_ERR_INVALID_ARG, "%s: FP4 K (%u) must be a multiple of 256", name, k); break;
        case DG_FP8: if (k % 128 != 0) return fail(DG_ERR_INVALID_ARG, "%s: FP8 K (%u) must be a multiple of 128", name, k); break;
        case DG_BF16: if (k % 64 != 0) return fail(DG_ERR_INVALID_ARG, "%s: BF16 K (%u) must be a multiple of 64", name, k); break;
        default: return fail(DG_ERR_INVALID_ARG, "%s: operand dtype must be FP8, FP4 or BF16", name);
    }
    if (k == 0 || op->rows == 0) return fail(DG_ERR_INVALID_ARG, "%s: empty operand (%u x %u)", name, op->rows, k);
    if (op->major != DG_MAJOR_K && op->major != DG_MAJOR_MN) return fail(DG_ERR_INVALID_ARG, "%s: major must be K or MN", name);
    if (op->major == DG_MAJOR_K && op->outer_stride < k)
        return fail(DG_ERR_INVALID_ARG, "%s: outer_stride (%u) smaller than K (%u)", name, op->outer_stride, k);
    if (op->major == DG_MAJOR_MN && op->outer_stride < op->rows)
        return fail(DG_ERR_INVALID_ARG, "%s: MN-major outer_stride (%u) smaller than its rows (%u)", name, op->outer_stride, op->rows);
    return DG_OK;
}

static int32_t run_gemm(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int gtype, const int32_t* layout,
                        uint32_t layout_len, uint32_t num_groups, uint32_t expected_m, int32_t accumulate, void* stream,
                        const int32_t* d_row_map = nullptr, uint32_t n_begin = 0, uint32_t n_count = 0,
                        const uint64_t* d_row_ptr = nullptr, const int32_t* m_blocks_dev = nullptr, float alpha = 1.f,
                        const int32_t* a_row_src = nullptr, uint32_t a_src_rows = 0) {
    int32_t st;
    if ((st = validate_operand(a, "A")) != DG_OK) return st;
    if ((st = validate_operand(b, "B")) != DG_OK) return st;
    if (!out || (!out->data && !d_row_ptr)) return fail(DG_ERR_INVALID_ARG, "null output");
    if (d_row_ptr && (out->dtype != DG_BF16 || out->cols % 8 != 0))
        return fail(DG_ERR_INVALID_ARG, "row-pointer output must be BF16 with a multiple of 8 columns");
    if (a->k != b->k) return fail(DG_ERR_INVALID_ARG, "A/B K mismatch");
    if (n_count == 0) { n_begin = 0; n_count = b ? b->rows : 0; }
    if (n_begin + n_count > b->rows || n_begin % 4 != 0)
        return fail(DG_ERR_INVALID_ARG, "column range [%u, %u) must lie inside N = %u and start on a multiple of 4", n_begin,
                    n_begin + n_count, b->rows);
    if (out->cols != n_count || (!d_row_map && !d_row_ptr && out->rows != a->rows)) return fail(DG_ERR_INVALID_ARG, "output shape mismatch");
    if (out->dtype != DG_BF16 && out->dtype != DG_F32) return fail(DG_ERR_INVALID_ARG, "output must be BF16 or FP32");
    if (out->stride < out->cols) return fail(DG_ERR_INVALID_ARG, "output stride (%u) smaller than its columns (%u)", out->stride, out->cols);
    const bool a_mn = a->major == DG_MAJOR_MN, b_mn = b->major == DG_MAJOR_MN;
    // FP8 x FP4 (either way round) runs as kind::mxf8f6f4 with the FP4 operand unpacked to one code per
    // byte on its way into shared memory (deepgemm/src/api.rs:264-265); everything else needs equal dtypes.
    const bool mixed = (a->dtype == DG_FP8 && b->dtype == DG_FP4) || (a->dtype == DG_FP4 && b->dtype == DG_FP8);
    if (a->dtype != b->dtype && !mixed)
        return fail(DG_ERR_INVALID_ARG, "operand dtypes %s x %s cannot be multiplied", dtype_name(a->dtype), dtype_name(b->dtype));
    if ((a_mn && a->dtype == DG_FP4) || (b_mn && b->dtype == DG_FP4)) return fail(DG_ERR_INVALID_ARG, "FP4 operands must be K-major");
    if ((a_mn || b_mn) && gtype != kNormal && gtype != kBatched)
        return fail(DG_ERR_INVALID_ARG, "m-grouped GEMMs require K-major operands");
    const int kind = mixed ? kFp8 : a->dtype == DG_FP8 ? kFp8 : (a->dtype == DG_FP4 ? kFp4 : kBf16);
    const bool has_sf = kind != kBf16;
    if (has_sf && (!a->sf.data || !b->sf.data)) return fail(DG_ERR_INVALID_ARG, "FP8/FP4 operands require scale factors");
    const uint32_t groups_a = (gtype == kMasked || gtype == kBatched) ? num_groups : 1u;
    const uint32_t groups_b = gtype == kNormal ? 1u : num_groups;
    if (gtype != kNormal) {
        if (num_groups == 0) return fail(DG_ERR_INVALID_ARG, "num_groups must be positive");
        if (!layout && gtype != kBatched) return fail(DG_ERR_INVALID_ARG, "grouped GEMM requires a layout buffer");
        if (accumulate && gtype != kBatched) return fail(DG_ERR_INVALID_ARG, "grouped GEMM does not accumulate");
    }
    if (gtype == kContiguous) {
        if (a->rows % 128 != 0)
            return fail(DG_ERR_INVALID_ARG, "contiguous layout requires M (%u) to be a multiple of 128", a->rows);
        if (layout_len != a->rows / 128)
            return fail(DG_ERR_INVALID_ARG, "m_indices must hold M/128 = %u entries (one per 128-row block), got %u", a->rows / 128, layout_len);
    }
    if (a_row_src) {
        if (gtype != kContiguous || mixed || a->dtype != DG_FP8 || a_mn || b_mn)
            return fail(DG_ERR_INVALID_ARG, "gathered A rows need the contiguous layout and K-major FP8 operands");
        if (a_src_rows == 0 || a_src_rows >= (1u << 31)) return fail(DG_ERR_INVALID_ARG, "gathered A rows: the source row count must be positive");
        if (reinterpret_cast<uintptr_t>(a_row_src) & 15u) return fail(DG_ERR_INVALID_ARG, "gathered A rows: the row list must be 16-byte aligned");
    }
    const uint32_t m = a->rows, n = n_count, n_full = b->rows, k = a->k;
    if ((uint64_t)groups_a * m >= (1ull << 31) || (uint64_t)groups_b * n_full >= (1ull << 31))
        return fail(DG_ERR_INVALID_ARG, "stacked row count exceeds 2^31");
    uint32_t gran_a = 32, gran_b = 32;
    if (has_sf) {
        gran_a = a->sf.gran; gran_b = b->sf.gran;
        if ((gran_a != 32 && gran_a != 128) || (gran_b != 32 && gran_b != 128))
            return fail(DG_ERR_INVALID_ARG, "SF granularity must be 32 or 128");
        if (kind == kFp4 && (gran_a != 32 || gran_b != 32)) return fail(DG_ERR_INVALID_ARG, "FP4 requires SF granularity 32");
        if (mixed && (a->dtype == DG_FP4 ? gran_a : gran_b) != 32) return fail(DG_ERR_INVALID_ARG, "FP4 requires SF granularity 32");
        // grouped layouts stack the groups along the SF columns; batches stack along the packed K rows
        const uint32_t sfr_a = (gtype == kBatched ? num_groups : 1u) * ceil_div(k, gran_a * 4);
        const uint32_t sfr_b = (gtype == kBatched ? num_groups : 1u) * ceil_div(k, gran_b * 4);
        const uint32_t sfc_a = align_up((gtype == kBatched ? 1u : groups_a) * m, 4);
        const uint32_t sfc_b = align_up((gtype == kBatched ? 1u : groups_b) * n_full, 4);
        if (a->sf.rows < sfr_a || a->sf.cols < sfc_a)
            return fail(DG_ERR_INVALID_ARG, "A scale-factor tensor is %u x %u, need at least %u x %u", a->sf.rows, a->sf.cols, sfr_a, sfc_a);
        if (b->sf.rows < sfr_b || b->sf.cols < sfc_b)
            return fail(DG_ERR_INVALID_ARG, "B scale-factor tensor is %u x %u, need at least %u x %u", b->sf.rows, b->sf.cols, sfr_b, sfc_b);
        // TMA starts SF boxes at column group*rows + tile offset: keep that 16-byte aligned.
        if (gtype != kNormal && gtype != kBatched && n_full % 4 != 0) return fail(DG_ERR_INVALID_ARG, "grouped GEMM requires N (%u) %% 4 == 0", n_full);
        if (gtype == kMasked && m % 4 != 0) return fail(DG_ERR_INVALID_ARG, "masked GEMM requires per-group M (%u) %% 4 == 0", m);
    }

    // Arguments are checked first so that a bad call reports InvalidArg on any machine; the
    // device gate follows (deepgemm/src/api.rs:168-173).
    const DeviceInfo* dev;
    if ((st = current_device(&dev)) != DG_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    DG_CUDA_CHECK(cudaStreamIsCapturing(s, &capturing));
    Plan plan;
    if ((st = make_plan(kind, gtype, m, n, k, num_groups, expected_m, gran_a, gran_b, dev, &plan,
                        capturing == cudaStreamCaptureStatusNone, a_mn, b_mn)) != DG_OK) return st;
    GemmParams& p = plan.p;
    p.out_f32 = out->dtype == DG_F32;
    p.accumulate = accumulate ? 1u : 0u;
    p.ldd = out->stride;
    p.d = out->data;
    p.layout = layout;
    p.d_row_map = d_row_map;
    p.d_row_ptr = d_row_ptr;
    p.m_blocks_dev = m_blocks_dev;
    p.a_row_src = a_row_src;
    p.b_group_rows = n_full;
    p.b_row_offset = n_begin;
    p.alpha = alpha;
    if (mixed) {
        // The copy that unpacks FP4 codes into byte containers reports the bytes it read (two codes per
        // byte), not the bytes it wrote, to the stage's barrier (measured: with the shared-memory size the
        // barrier never completes).
        const uint32_t a_b = kBlockM * 128u, b_b = p.block_n / plan.cluster * 128u;
        p.tx_ab = (a->dtype == DG_FP4 ? a_b / 2 : a_b) + (b->dtype == DG_FP4 ? b_b / 2 : b_b);
    }
    p.sf_rows_a = has_sf ? ceil_div(k, gran_a * 4) : 0u;
    p.sf_rows_b = has_sf ? ceil_div(k, gran_b * 4) : 0u;
    // instruction descriptor: operand formats (mxf8f6f4: E4M3 = 0, E2M1 = 5; mxf4: E2M1 = 1), tile shape, majors
    if (kind == kBf16) p.idesc = make_idesc_bf16(kBlockM * plan.cluster, p.block_n);
    else if (kind == kFp4) p.idesc = make_idesc_bs(1u, 1u, kBlockM * plan.cluster, p.block_n);
    else p.idesc = make_idesc_bs(a->dtype == DG_FP4 ? 5u : 0u, b->dtype == DG_FP4 ? 5u : 0u, kBlockM * plan.cluster, p.block_n);
    p.idesc |= ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16);   // bits 15 / 16: A / B is MN-major
    // The last column tile, when narrower than the others, gets its own width (a multiple of 16), instruction
    // descriptor and B box: it then costs its share of a tile (N = 4096 in tiles of 224: 64 columns) instead of
    // loading and multiplying 224 rows of B of which most belong to the next expert or to nobody.
    p.tail_n = 0; p.idesc_tail = p.idesc; p.tx_ab_tail = p.tx_ab;
    {
        const uint32_t last = n_count - (p.num_n_blocks - 1u) * p.block_n, tail = align_up(last, 16u);
        if (!a_mn && !b_mn && tail < p.block_n && env_u32("DG_TAIL_TILE", 1)) {
            p.tail_n = tail;
            if (kind == kBf16) p.idesc_tail = make_idesc_bf16(kBlockM * plan.cluster, tail);
            else if (kind == kFp4) p.idesc_tail = make_idesc_bs(1u, 1u, kBlockM * plan.cluster, tail);
            else p.idesc_tail = make_idesc_bs(a->dtype == DG_FP4 ? 5u : 0u, b->dtype == DG_FP4 ? 5u : 0u, kBlockM * plan.cluster, tail);
            const uint32_t a_b = kBlockM * 128u, b_b = tail / plan.cluster * 128u;
            p.tx_ab_tail = mixed ? (a->dtype == DG_FP4 ? a_b / 2 : a_b) + (b->dtype == DG_FP4 ? b_b / 2 : b_b) : a_b + b_b;
        }
    }

    CUtensorMap ta, tb, tsa, tsb;
    const uint32_t ebytes = kind == kBf16 ? 2u : 1u;
    const uint32_t box_k = kind == kBf16 ? 64u : 128u;      // K elements (FP4 x FP4: bytes) per k-block
    auto operand_map = [&](CUtensorMap* tm, const dg_operand_t* op, bool mn, uint32_t groups, uint32_t box_rows, const char* what) -> int32_t {
        if (mn)   // [groups * K, MN] buffer: boxes of one swizzle atom along MN x BLOCK_K rows
            return make_tmap_2d(tm, kind == kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, ebytes, op->data,
                                op->rows, (uint64_t)groups * k, (uint64_t)op->outer_stride * ebytes, p.box_elems, box_k,
                                CU_TENSOR_MAP_SWIZZLE_128B, what);
        if (kind == kFp4)   // FP4 x FP4: rows of k/2 bytes moved as bytes (two codes per byte stay packed in shared memory)
            return make_tmap_2d(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, op->data, k / 2, (uint64_t)groups * op->rows, op->outer_stride / 2,
                                128u, box_rows, CU_TENSOR_MAP_SWIZZLE_128B, what);
        if (op->dtype == DG_FP4)   // FP4 against FP8: 16 codes are unpacked into 16 bytes of shared memory by the copy itself
            return make_tmap_2d(tm, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 1, op->data, k, (uint64_t)groups * op->rows, op->outer_stride / 2,
                                128u, box_rows, CU_TENSOR_MAP_SWIZZLE_128B, what);
        return make_tmap_2d(tm, kind == kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, ebytes, op->data, k,
                            (uint64_t)groups * op->rows, (uint64_t)op->outer_stride * ebytes, box_k, box_rows, CU_TENSOR_MAP_SWIZZLE_128B, what);
    };
    if (a_row_src) {
        // the un-permuted rows, one per box: tile::gather4 takes four of them per instruction
        if (plan.cluster != 1 || p.k_splits > 1) return fail(DG_ERR_UNSUPPORTED, "gathered A rows run on single CTAs without split-K");
        if ((st = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->data, k, a_src_rows, (uint64_t)a->outer_stride, box_k, 1u,
                               CU_TENSOR_MAP_SWIZZLE_128B, "A (gathered rows)")) != DG_OK) return st;
    } else if ((st = operand_map(&ta, a, a_mn, groups_a, kBlockM, "A")) != DG_OK) return st;
    if ((st = operand_map(&tb, b, b_mn, groups_b, p.block_n / plan.cluster, "B")) != DG_OK) return st;
    plan.tb_tail = tb;
    if (p.tail_n && (st = operand_map(&plan.tb_tail, b, false, groups_b, p.tail_n / plan.cluster, "B (last column tile)")) != DG_OK) return st;
    if (has_sf) {
        if ((st = make_tmap_2d(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a->sf.data, a->sf.cols, a->sf.rows,
                               (uint64_t)a->sf.cols * 4, 128u, p.sf_sub, CU_TENSOR_MAP_SWIZZLE_NONE, "SFA")) != DG_OK) return st;
        if ((st = make_tmap_2d(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, b->sf.data, b->sf.cols, b->sf.rows,
                               (uint64_t)b->sf.cols * 4, p.sfb_chunks * 128u, p.sf_sub, CU_TENSOR_MAP_SWIZZLE_NONE, "SFB")) != DG_OK) return st;
    } else {
        tsa = ta; tsb = tb;
    }
    // FP8 with per-128 scales on both operands: the instantiation whose SF warp copies the scale factors into tensor memory
    const bool sfw = kind == kFp8 && plan.cluster == 1 && !a_mn && !b_mn && gtype != kBatched && p.sf_cp_by_mma == 0;
    if (p.k_splits > 1) {
        // Scratch for the partial tiles: one buffer per (thread, device, stream), grown on demand with
        // stream-ordered allocation and kept for the next call (work on one stream is ordered, so
        // consecutive calls may share it; allocating per call costs more host time than the GEMM).
        struct SplitWs { cudaStream_t stream; int device; float* ptr; size_t bytes; };
        static thread_local SplitWs cache[8] = {};
        static thread_local int cache_next = 0;
        const size_t need = sizeof(float) * (size_t)p.k_splits * m * n;
        float* graph_ws = nullptr;
        if (capturing != cudaStreamCaptureStatusNone) {
            // inside a graph capture the buffer must belong to the graph: allocate and free per call
            DG_CUDA_CHECK(cudaMallocAsync(&graph_ws, need, s));
            p.split_ws = graph_ws;
        } else {
            SplitWs* slot = nullptr;
            for (auto& c : cache)
                if (c.ptr && c.stream == s && c.device == dev->device) { slot = &c; break; }
            if (!slot) {
                slot = &cache[cache_next];
                cache_next = (cache_next + 1) % 8;
                if (slot->ptr) { cudaFreeAsync(slot->ptr, slot->stream); *slot = SplitWs{}; }
            }
            if (slot->bytes < need) {
                if (slot->ptr) cudaFreeAsync(slot->ptr, s);
                *slot = SplitWs{};
                float* fresh = nullptr;
                DG_CUDA_CHECK(cudaMallocAsync(&fresh, need, s));
                *slot = SplitWs{s, dev->device, fresh, need};
            }
            p.split_ws = slot->ptr;
        }
        int32_t lst = DG_OK;
        if (kind == kFp8 && sfw) lst = launch<kFp8, kNormal, 1, true, false, false, true>(plan, ta, tb, tsa, tsb, s);
        else if (kind == kFp8) lst = launch<kFp8, kNormal, 1, true>(plan, ta, tb, tsa, tsb, s);
        else if (kind == kFp4) lst = launch<kFp4, kNormal, 1, true>(plan, ta, tb, tsa, tsb, s);
        else lst = launch<kBf16, kNormal, 1, true>(plan, ta, tb, tsa, tsb, s);
        if (lst == DG_OK) {
            const size_t threads = (size_t)m * ((n + 3) / 4);
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((uint32_t)((threads + 255) / 256));
            cfg.blockDim = dim3(256);
            cfg.stream = s;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = pdl_enabled() ? 1 : 0;
            cudaError_t e = cudaLaunchKernelEx(&cfg, split_reduce_kernel, (const float*)p.split_ws, p.k_splits, m, n, out->data,
                                               (uint64_t)out->stride, p.out_f32, p.accumulate, alpha);
            if (e != cudaSuccess) lst = fail(DG_ERR_DRIVER, "split-K reduction launch failed: %s", cudaGetErrorString(e));
            else note_launch();
        }
        if (graph_ws) cudaFreeAsync(graph_ws, s);
        return lst;
    }
    if (a_row_src) {
        if (plan.dynamic) p.tile_counter = tile_counters(dev);
        if (plan.dynamic && sfw) return launch<kFp8, kContiguous, 1, false, true, false, true, true>(plan, ta, tb, tsa, tsb, s);
        if (plan.dynamic) return launch<kFp8, kContiguous, 1, false, true, false, false, true>(plan, ta, tb, tsa, tsb, s);
        if (sfw) return launch<kFp8, kContiguous, 1, false, false, false, true, true>(plan, ta, tb, tsa, tsb, s);
        return launch<kFp8, kContiguous, 1, false, false, false, false, true>(plan, ta, tb, tsa, tsb, s);
    }
    if (plan.dynamic) {
        p.tile_counter = tile_counters(dev);
        if (kind == kFp8 && sfw) return launch<kFp8, kContiguous, 1, false, true, false, true>(plan, ta, tb, tsa, tsb, s);
        if (kind == kFp8) return launch<kFp8, kContiguous, 1, false, true>(plan, ta, tb, tsa, tsb, s);
        if (kind == kFp4) return launch<kFp4, kContiguous, 1, false, true>(plan, ta, tb, tsa, tsb, s);
        return launch<kBf16, kContiguous, 1, false, true>(plan, ta, tb, tsa, tsb, s);
    }
    if (a_mn || b_mn) {
        if (kind == kFp8 && gtype == kNormal) return launch<kFp8, kNormal, 1, false, false, true>(plan, ta, tb, tsa, tsb, s);
        if (kind == kFp8 && gtype == kBatched) return launch<kFp8, kBatched, 1, false, false, true>(plan, ta, tb, tsa, tsb, s);
        if (kind == kBf16 && gtype == kNormal) return launch<kBf16, kNormal, 1, false, false, true>(plan, ta, tb, tsa, tsb, s);
        if (kind == kBf16 && gtype == kBatched) return launch<kBf16, kBatched, 1, false, false, true>(plan, ta, tb, tsa, tsb, s);
    }
#define DG_DISPATCH_SFW(G)                                                                               \
    if (kind == kFp8 && gtype == G && sfw) {                                                             \
        return launch<kFp8, G, 1, false, false, false, true>(plan, ta, tb, tsa, tsb, s);                 \
    }
    DG_DISPATCH_SFW(kNormal) DG_DISPATCH_SFW(kContiguous) DG_DISPATCH_SFW(kMasked)
#undef DG_DISPATCH_SFW
#define DG_DISPATCH(K, G)                                                            \
    if (kind == K && gtype == G) {                                                   \
        if (plan.cluster == 2) return launch<K, G, 2>(plan, ta, tb, tsa, tsb, s);    \
        return launch<K, G, 1>(plan, ta, tb, tsa, tsb, s);                           \
    }
    DG_DISPATCH(kFp8, kNormal) DG_DISPATCH(kFp8, kContiguous) DG_DISPATCH(kFp8, kMasked) DG_DISPATCH(kFp8, kBatched)
    DG_DISPATCH(kFp4, kNormal) DG_DISPATCH(kFp4, kContiguous) DG_DISPATCH(kFp4, kMasked) DG_DISPATCH(kFp4, kBatched)
    DG_DISPATCH(kBf16, kNormal) DG_DISPATCH(kBf16, kContiguous) DG_DISPATCH(kBf16, kMasked) DG_DISPATCH(kBf16, kBatched)
#undef DG_DISPATCH
    return fail(DG_ERR_RUNTIME, "no kernel for kind %d / type %d", kind, gtype);
}

}  // namespace dg

extern "C" {

int32_t dg_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream) {
    return dg::run_gemm(a, b, out, dg::kNormal, nullptr, 0, 1, a ? a->rows : 0, accumulate, stream);
}
// api::gemm_nt_alpha (deepgemm/src/api.rs:663-673): D = alpha * (A . B^T) (+ D); alpha multiplies the f32
// accumulator before the output cast, the accumulated D is not scaled.
int32_t dg_gemm_nt_alpha(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, float alpha, void* stream) {
    return dg::run_gemm(a, b, out, dg::kNormal, nullptr, 0, 1, a ? a->rows : 0, accumulate, stream, nullptr, 0, 0, nullptr, nullptr, alpha);
}
// api::gemm_nn / gemm_tn / gemm_tt (deepgemm/src/api.rs:717-759): the BLAS layouts are the NT GEMM over
// operands described as MN-major views; the entries only check that the view has the orientation the
// layout needs, so that a mis-described operand fails here instead of computing wrong numbers.
static int32_t want_major(const dg_operand_t* op, int32_t major, const char* fn, const char* name) {
    if (!op) return dg::fail(DG_ERR_INVALID_ARG, "%s: null operand", fn);
    if (op->major != major)
        return dg::fail(DG_ERR_INVALID_ARG, "%s: %s must be described as %s", fn, name,
                        major == DG_MAJOR_MN ? "an MN-major view ([K, MN] buffer, outer_stride = pitch of the K slices)" : "a K-major operand");
    return DG_OK;
}
int32_t dg_gemm_nn(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream) {
    int32_t st = want_major(b, DG_MAJOR_MN, "gemm_nn", "B");
    return st != DG_OK ? st : dg_gemm_nt(a, b, out, accumulate, stream);
}
int32_t dg_gemm_tn(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream) {
    int32_t st = want_major(a, DG_MAJOR_MN, "gemm_tn", "A");
    return st != DG_OK ? st : dg_gemm_nt(a, b, out, accumulate, stream);
}
int32_t dg_gemm_tt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream) {
    int32_t st = want_major(a, DG_MAJOR_MN, "gemm_tt", "A");
    if (st == DG_OK) st = want_major(b, DG_MAJOR_MN, "gemm_tt", "B");
    return st != DG_OK ? st : dg_gemm_nt(a, b, out, accumulate, stream);
}
// api::fp8_bmm (deepgemm/src/api.rs:966-993): `batch` independent GEMMs, A [batch * M, K], B [batch * N, K]
// and D [batch * M, N] stacked along the rows, scale factors in transform_sf_batched's arena.
int32_t dg_bmm(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, uint32_t batch, int32_t accumulate, void* stream) {
    return dg::run_gemm(a, b, out, dg::kBatched, nullptr, 0, batch, a ? a->rows : 0, accumulate, stream);
}
static int32_t typed(const dg_operand_t* a, const dg_operand_t* b, int32_t want, const char* fn);
int32_t dg_fp8_bmm(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, uint32_t batch, int32_t accumulate, void* stream) {
    int32_t st = typed(a, b, DG_FP8, "fp8_bmm");
    return st != DG_OK ? st : dg_bmm(a, b, out, batch, accumulate, stream);
}
static int32_t typed(const dg_operand_t* a, const dg_operand_t* b, int32_t want, const char* fn) {
    if (!a || !b) return dg::fail(DG_ERR_INVALID_ARG, "%s: null operand", fn);
    if (a->dtype != want || b->dtype != want)
        return dg::fail(DG_ERR_INVALID_ARG, "%s: operands must be %s", fn, dg::dtype_name(want));
    return DG_OK;
}
int32_t dg_fp8_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream) {
    int32_t st = typed(a, b, DG_FP8, "fp8_gemm_nt");
    return st != DG_OK ? st : dg_gemm_nt(a, b, out, accumulate, stream);
}
int32_t dg_fp4_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream) {
    int32_t st = typed(a, b, DG_FP4, "fp4_gemm_nt");
    return st != DG_OK ? st : dg_gemm_nt(a, b, out, accumulate, stream);
}
int32_t dg_bf16_gemm_nt(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, int32_t accumulate, void* stream) {
    int32_t st = typed(a, b, DG_BF16, "bf16_gemm_nt");
    return st != DG_OK ? st : dg_gemm_nt(a, b, out, accumulate, stream);
}

int32_t dg_m_grouped_gemm_nt_contiguous(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                        const int32_t* m_indices, uint32_t m_indices_len, uint32_t num_groups, void* stream) {
    if (a && a->major != DG_MAJOR_K) return dg::fail(DG_ERR_INVALID_ARG, "m-grouped contiguous requires K-major A");
    return dg::run_gemm(a, b, out, dg::kContiguous, m_indices, m_indices_len, num_groups, a ? a->rows : 0, 0, stream);
}
int32_t dg_m_grouped_gemm_nt_contiguous_scatter(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,
                                                const int32_t* m_indices, uint32_t m_indices_len, uint32_t num_groups,
                                                const int32_t* d_row_map, uint32_t n_begin, uint32_t n_count, void* stream) {
    if (!d_row_map) return dg::fail(DG_ERR_INVALID_ARG, "m-grouped contiguous scatter requires a row map");
    if (!a || !b) return dg::fail(DG_ERR_INVALID_ARG, "null operand");
    if (a->major != DG_MAJOR_K) return dg::fail(DG_ERR_INVALID_ARG, "m-grouped contiguous requires K-major A");
    return dg::run_gemm(a, b, out, dg::kContiguous, m_indices, m_indices_len, num_groups, a->rows, 0, stream, d_row_map,
                        n_begin, n_count);
}
int32_t dg_m_grouped_gemm_nt_contiguous_gather(const dg_operand_t* a, const int32_t* a_row_src, uint32_t a_src_rows,
                                               const dg_operand_t* b, dg_output_t* out, const int32_t* m_indices,
                                               uint32_t m_indices_len, uint32_t num_groups, void* stream) {
    if (!a_row_src) return dg::fail(DG_ERR_INVALID_ARG, "m-grouped contiguous gather requires the row list");
    return dg::run_gemm(a, b, out, dg::kContiguous, m_indices, m_indices_len, num_groups, 0, 0, stream, nullptr, 0, 0, nullptr,
                        nullptr, 1.f, a_row_src, a_src_rows);
}

int32_t dg_m_grouped_gemm_nt_contiguous_rowptr(const dg_operand_t* a, const dg_operand_t* b, const int32_t* m_indices,
                                               uint32_t m_indices_len, uint32_t num_groups, const uint64_t* d_row_ptr,
                                               const int32_t* m_blocks_used, uint32_t n_begin, uint32_t n_count, void* stream) {
    if (!d_row_ptr) return dg::fail(DG_ERR_INVALID_ARG, "m-grouped contiguous rowptr requires the row address table");
    if (!a || !b) return dg::fail(DG_ERR_INVALID_ARG, "null operand");
    if (a->major != DG_MAJOR_K) return dg::fail(DG_ERR_INVALID_ARG, "m-grouped contiguous requires K-major A");
    if (n_count == 0) { n_begin = 0; n_count = b->rows; }
    dg_output_t out = {DG_BF16, 0, n_count, n_count, nullptr};
    return dg::run_gemm(a, b, &out, dg::kContiguous, m_indices, m_indices_len, num_groups, a->rows, 0, stream, nullptr,
                        n_begin, n_count, d_row_ptr, m_blocks_used);
}
int32_t dg_m_grouped_gemm_nt_masked(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out, const int32_t* masked_m,
                                    uint32_t num_groups, uint32_t expected_m, void* stream) {
    if (a && b && (a->major != DG_MAJOR_K || b->major != DG_MAJOR_K))
        return dg::fail(DG_ERR_INVALID_ARG, "m-grouped masked requires K-major A/B");
    return dg::run_gemm(a, b, out, dg::kMasked, masked_m, num_groups, num_groups, expected_m, 0, stream);
}

#define DG_TYPED_GROUPED(NAME, DT)                                                                                         \
    int32_t dg_m_grouped_##NAME##_gemm_nt_contiguous(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,        \
                                                     const int32_t* mi, uint32_t len, uint32_t g, void* stream) {          \
        int32_t st = typed(a, b, DT, "m_grouped_" #NAME "_gemm_nt_contiguous");                                            \
        return st != DG_OK ? st : dg_m_grouped_gemm_nt_contiguous(a, b, out, mi, len, g, stream);                          \
    }                                                                                                                      \
    int32_t dg_m_grouped_##NAME##_gemm_nt_masked(const dg_operand_t* a, const dg_operand_t* b, dg_output_t* out,            \
                                                 const int32_t* mm, uint32_t g, uint32_t em, void* stream) {               \
        int32_t st = typed(a, b, DT, "m_grouped_" #NAME "_gemm_nt_masked");                                                \
        return st != DG_OK ? st : dg_m_grouped_gemm_nt_masked(a, b, out, mm, g, em, stream);                               \
    }
DG_TYPED_GROUPED(fp8, DG_FP8)
DG_TYPED_GROUPED(fp4, DG_FP4)
DG_TYPED_GROUPED(bf16, DG_BF16)
#undef DG_TYPED_GROUPED

int32_t dg_get_gemm_config(int32_t dtype, int32_t kind, uint32_t m, uint32_t n, uint32_t k, uint32_t num_groups,
                           dg_gemm_config_t* cfg) {
    const dg::DeviceInfo* dev;
    int32_t st = dg::current_device(&dev);
    if (st != DG_OK) return st;
    if (!cfg || kind < 0 || kind > 2 || dtype < 0 || dtype > 2) return dg::fail(DG_ERR_INVALID_ARG, "get_gemm_config: bad argument");
    dg::Plan plan;
    st = dg::make_plan(dtype == DG_FP8 ? dg::kFp8 : dtype == DG_FP4 ? dg::kFp4 : dg::kBf16, kind, m, n, k,
                       num_groups ? num_groups : 1, m, dtype == DG_FP8 ? 128 : 32, dtype == DG_FP8 ? 128 : 32, dev, &plan);   // FP8: per-128 scales assumed
    if (st != DG_OK) return st;
    cfg->block_m = dg::kBlockM;
    cfg->block_n = plan.p.block_n;
    cfg->block_k = dtype == DG_FP4 ? 256 : dtype == DG_FP8 ? 128 : 64;
    cfg->num_stages = plan.p.num_stages;
    cfg->smem_bytes = plan.smem_bytes;
    cfg->num_tiles = plan.num_tiles;
    cfg->grid = plan.grid;
    cfg->cluster = plan.cluster;
    cfg->block_m = dg::kBlockM * plan.cluster;
    return DG_OK;
}

}  // extern "C"
