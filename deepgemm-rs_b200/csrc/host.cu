// Error reporting, device gate, status word, tensor-map encoding.
#include "host.h"

#include <cstdarg>
#include <cstdio>
#include <atomic>
#include <mutex>

namespace dg {

static thread_local char g_err[512] = "";

int32_t fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

static std::mutex g_mu;
static DeviceInfo g_dev[64];

int32_t current_device(const DeviceInfo** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return fail(DG_ERR_UNSUPPORTED, "no usable CUDA device (%s); the tcgen05 kernels require SM100 (Blackwell)",
                    cudaGetErrorString(e));
    }
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceInfo& d = g_dev[dev];
    if (d.device != dev) {
        cudaDeviceProp p;
        DG_CUDA_CHECK(cudaGetDeviceProperties(&p, dev));
        if (p.major != 10)
            return fail(DG_ERR_UNSUPPORTED, "the tcgen05 kernels require SM100 (Blackwell); this device is sm_%d%d",
                        p.major, p.minor);
        d.sm_count = p.multiProcessorCount;
        d.cc_major = p.major;
        d.cc_minor = p.minor;
        d.smem_optin = (int)p.sharedMemPerBlockOptin;
        // status word (first 256 bytes) and the tile-counter pool behind it, cleared before any stream uses them
        const size_t bytes = 256 + kTilePoolPairs * 2 * sizeof(uint32_t);
        DG_CUDA_CHECK(cudaMalloc(&d.status, bytes));
        DG_CUDA_CHECK(cudaMemset(d.status, 0, bytes));
        DG_CUDA_CHECK(cudaDeviceSynchronize());
        d.tile_pool = d.status + 64;
        d.device = dev;
    }
    *out = &d;
    return DG_OK;
}

static int32_t encode_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base,
                              uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                              uint32_t box_outer, CUtensorMapSwizzle swizzle, const char* what);

int32_t get_encode_tiled(EncodeTiledFn* fn) {
    static EncodeTiledFn cached = nullptr;
    if (!cached) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
            return fail(DG_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
        cached = reinterpret_cast<EncodeTiledFn>(p);
    }
    *fn = cached;
    return DG_OK;
}

// Encoding a tensor map costs about a microsecond of host time and a GEMM needs four or five; calls
// in a serving loop repeat the same operands, so the last few encodings are kept per thread.
struct TmapKey {
    const void* base;
    uint64_t inner, outer, pitch;
    uint32_t dt, box_inner, box_outer, swizzle;
    bool operator==(const TmapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && pitch == o.pitch && dt == o.dt &&
               box_inner == o.box_inner && box_outer == o.box_outer && swizzle == o.swizzle;
    }
};
struct TmapCache {
    static constexpr int kSlots = 32;
    TmapKey key[kSlots];
    CUtensorMap map[kSlots];
    int device[kSlots];
    int used = 0, next = 0;
};
static thread_local TmapCache g_tmaps;

int32_t make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base,
                     uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                     uint32_t box_outer, CUtensorMapSwizzle swizzle, const char* what) {
    const TmapKey key{base, inner, outer, row_pitch_bytes, (uint32_t)dt, box_inner, box_outer, (uint32_t)swizzle};
    int dev = 0;
    cudaGetDevice(&dev);
    for (int i = 0; i < g_tmaps.used; ++i)
        if (g_tmaps.device[i] == dev && g_tmaps.key[i] == key) { *map = g_tmaps.map[i]; return DG_OK; }
    int32_t st = encode_tmap_2d(map, dt, elem_bytes, base, inner, outer, row_pitch_bytes, box_inner, box_outer, swizzle, what);
    if (st != DG_OK) return st;
    const int slot = g_tmaps.next;
    g_tmaps.next = (g_tmaps.next + 1) % TmapCache::kSlots;
    if (g_tmaps.used < TmapCache::kSlots) ++g_tmaps.used;
    g_tmaps.key[slot] = key;
    g_tmaps.map[slot] = *map;
    g_tmaps.device[slot] = dev;
    return DG_OK;
}

static int32_t encode_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base,
                       uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                       uint32_t box_outer, CUtensorMapSwizzle swizzle, const char* what) {
    EncodeTiledFn enc;
    int32_t st = get_encode_tiled(&enc);
    if (st != DG_OK) return st;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
        return fail(DG_ERR_INVALID_ARG, "%s: base address must be 16-byte aligned", what);
    if (row_pitch_bytes % 16 != 0)
        return fail(DG_ERR_INVALID_ARG, "%s: row pitch (%llu bytes) must be a multiple of 16", what,
                    (unsigned long long)row_pitch_bytes);
    if (box_inner > 256 || box_outer > 256 || (uint64_t)box_inner * elem_bytes % 16 != 0)
        return fail(DG_ERR_RUNTIME, "%s: bad TMA box %u x %u", what, box_inner, box_outer);
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DG_ERR_DRIVER, "%s: cuTensorMapEncodeTiled failed with %d (dims %llu x %llu, pitch %llu, box %u x %u)",
                    what, (int)r, (unsigned long long)inner, (unsigned long long)outer,
                    (unsigned long long)row_pitch_bytes, box_inner, box_outer);
    return DG_OK;
}

}  // namespace dg

extern "C" {

const char* dg_last_error(void) { return dg::g_err; }
const char* dg_version(void) { return "deepgemm_b200 0.1 (sm_100a)"; }

int32_t dg_device_check(void) {
    const dg::DeviceInfo* d;
    return dg::current_device(&d);
}

int32_t dg_poll_device_status(void* stream) {
    const dg::DeviceInfo* d;
    int32_t st = dg::current_device(&d);
    if (st != DG_OK) return st;
    uint32_t word = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DG_CUDA_CHECK(cudaMemcpyAsync(&word, d->status, 4, cudaMemcpyDeviceToHost, s));
    DG_CUDA_CHECK(cudaStreamSynchronize(s));
    if (word != 0) {
        DG_CUDA_CHECK(cudaMemsetAsync(d->status, 0, 4, s));
        DG_CUDA_CHECK(cudaStreamSynchronize(s));
        // site 7 comes from the peer-memory kernels: bit 15 set = a layout overflow found by
        // dg_ep_route (expert in bits 16..), else the barrier gave up waiting for the rank in bits 8..
        if ((word & 0xffu) == 7u && (word & 0x8000u))
            return dg::fail(DG_ERR_RUNTIME, "expert-parallel dispatch: the rows routed to the owner of expert %u exceed its layout capacity; they were dropped",
                            word >> 16);
        if ((word & 0xffu) == 7u)
            return dg::fail(DG_ERR_DEVICE_TIMEOUT, "a barrier between ranks gave up waiting for rank %u", word >> 8);
        return dg::fail(DG_ERR_DEVICE_TIMEOUT, "a device-side wait gave up: site %u in block %u", word & 0xffu, word >> 8);
    }
    return DG_OK;
}

unsigned long long dg_launch_count(void) { return dg::g_launches.load(); }

void dg_sf_shape(uint32_t mn, uint32_t k, uint32_t gran, uint32_t* rows, uint32_t* cols) {
    if (rows) *rows = gran ? dg::ceil_div(k, gran * 4) : 0;
    if (cols) *cols = dg::align_up(mn, 4);
}

}  // extern "C"
