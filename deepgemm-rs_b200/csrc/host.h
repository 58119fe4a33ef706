// Host-side helpers shared by the C-ABI translation units: error reporting, the device gate,
// the per-device status word and the driver entry point for tensor-map encoding.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/deepgemm_b200.h"

namespace dg {

// Records a printf-formatted message for dg_last_error() and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define DG_CUDA_CHECK(expr)                                                                   \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            return ::dg::fail(DG_ERR_DRIVER, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    int smem_optin = 0;
    uint32_t* status = nullptr;  // one zero-initialised word in global memory
    uint32_t* tile_pool = nullptr;  // kTilePoolPairs zeroed counter pairs for dynamically scheduled GEMMs
};
constexpr uint32_t kTilePoolPairs = 256;

// Information about the current device (cached per device).  Returns a status; on success
// `*out` points at the cached entry.  Fails with DG_ERR_UNSUPPORTED when there is no CUDA
// device or it is not sm_100.
int32_t current_device(const DeviceInfo** out);

// cuTensorMapEncodeTiled resolved through the runtime (the library does not link libcuda, so
// it loads on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int32_t get_encode_tiled(EncodeTiledFn* fn);

// 2-D tiled tensor map over row-major [outer, inner] with `row_pitch_bytes` between rows.
int32_t make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, uint32_t elem_bytes, const void* base,
                     uint64_t inner, uint64_t outer, uint64_t row_pitch_bytes, uint32_t box_inner,
                     uint32_t box_outer, CUtensorMapSwizzle swizzle, const char* what);

// Counts kernel launches made by this library (dg_launch_count reports it).
void note_launch();

inline uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
inline uint32_t align_up(uint32_t a, uint32_t b) { return ceil_div(a, b) * b; }

}  // namespace dg
