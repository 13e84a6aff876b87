// opscvUpsampleBilinear2dNoAlloc: bilinear up/down-sampling in one call that allocates no device memory and
// takes no workspace.
//
// Who it is for. The two-phase aclnn entry points need a caller-owned workspace for their per-axis tap tables.
// Some callers cannot provide one at the point of the call: a plugin inside a host framework that owns every byte
// of device memory and has no workspace hook, a real-time loop in which allocator calls are forbidden, code that
// runs after a memory pool has been frozen. For them the tap tables live in a fixed array in device global memory
// that is part of this library's image, so the call needs nothing but its input and output.
//
// How it works. The kernels are the ones behind aclnnUpsampleBilinear2d (table builder + the direct forward
// kernel); only the home of the tables differs. The array below holds, per axis, lo[kMaxExtent], hi[kMaxExtent]
// (int32) and delta[kMaxExtent] (fp32): 2 * 3 * kMaxExtent * 4 bytes = 192 KiB per device. Output extents beyond
// kMaxExtent are rejected with ACLNN_ERR_PARAM_INVALID. The device address of the array is looked up once per
// device, on the first call made with that device current, and cached; that first call should therefore come
// before any stream capture on that device. (If the application destroys the device's context with
// cudaDeviceReset, the next call notices that the cached address is no longer device memory and looks it up
// again; that call, too, should come before any capture.) Nothing in the array has to start at zero: every call rewrites the
// entries it reads, on the caller's stream, before the sampling kernel runs.
//
// Sharing. Every call on a device uses the same array. Calls on one stream are ordered and safe. Calls that may
// overlap on different streams of one device (or from different threads without ordering) race on the tables and
// can corrupt each other's results: serialise them, or use the two-phase API with separate workspaces.
#include <mutex>

#include "host_common.h"

namespace opscv {
namespace {

constexpr int32_t kMaxExtent = 8192;                 // largest output height / width accepted
constexpr int32_t kScratchWords = 2 * 3 * kMaxExtent; // H and W axis: lo, hi, delta
constexpr int kMaxDevices = 64;

static __device__ __align__(256) uint32_t g_tapScratch[kScratchWords];

std::mutex g_setupMutex;
uint32_t* g_scratchAddr[kMaxDevices] = {};

// Device address of g_tapScratch on the current device (looked up once per device; `refresh` drops the cached
// address first, for a device whose context was destroyed and re-created since the look-up).
cudaError_t ScratchForCurrentDevice(uint32_t** out, bool refresh)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        return cudaErrorInvalidDevice;
    }
    std::lock_guard<std::mutex> lock(g_setupMutex);
    if (refresh) {
        g_scratchAddr[dev] = nullptr;
    }
    if (g_scratchAddr[dev] == nullptr) {
        uint32_t* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_tapScratch);
        if (e != cudaSuccess) {
            return e;
        }
        g_scratchAddr[dev] = ptr;
    }
    *out = g_scratchAddr[dev];
    return cudaSuccess;
}

} // namespace
} // namespace opscv

using namespace opscv;

extern "C" ACLNN_API aclnnStatus opscvUpsampleBilinear2dNoAlloc(const void* self, void* out, aclDataType dtype,
                                                                aclFormat format, int64_t n, int64_t c, int64_t inH,
                                                                int64_t inW, int64_t outH, int64_t outW,
                                                                bool alignCorners, double scalesH, double scalesW,
                                                                aclrtStream stream)
{
    const char* api = "opscvUpsampleBilinear2dNoAlloc";
    if (self == nullptr || out == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null tensor pointer", api);
    }
    if (!DtypeSupported(dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: dtype %s is not supported (float, float16, bfloat16)", api,
                    DtypeName(dtype));
    }
    if (format != ACL_FORMAT_NCHW && format != ACL_FORMAT_NHWC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format must be NCHW or NHWC", api);
    }
    if (n < 0 || c < 0 || inH <= 0 || inW <= 0 || outH < 0 || outW < 0 || scalesH < 0 || scalesW < 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: bad extents or scales", api);
    }
    if (outH > kMaxExtent || outW > kMaxExtent) {
        return Fail(ACLNN_ERR_PARAM_INVALID,
                    "%s: output %lld x %lld exceeds the built-in table capacity of %d per axis; use "
                    "aclnnUpsampleBilinear2d with a workspace",
                    api, static_cast<long long>(outH), static_cast<long long>(outW), kMaxExtent);
    }
    if (inH > INT32_MAX || inW > INT32_MAX || n * c > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: extents exceed the supported range", api);
    }
    if (n == 0 || c == 0 || outH == 0 || outW == 0) {
        return ACLNN_SUCCESS;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (inH == outH && inW == outW) {
        // Same extents: a plain copy whatever the scales say, as in the two-phase entry point and the reference
        // (all-copy schedule, resize_bilinear_v2_tiling_arch35.cpp:245-252). No tables, so no shared state.
        const size_t bytes = static_cast<size_t>(n) * c * inH * inW * ElemSize(dtype);
        const cudaError_t ce = cudaMemcpyAsync(out, self, bytes, cudaMemcpyDeviceToDevice, s);
        if (ce != cudaSuccess) {
            return Fail(ACLNN_ERR_RUNTIME_ERROR, "%s: %s", api, cudaGetErrorString(ce));
        }
        return ACLNN_SUCCESS;
    }
    uint32_t* scratch = nullptr;
    cudaError_t e = ScratchForCurrentDevice(&scratch, false);
    if (e == cudaSuccess) {
        // A cached address outlives its context if the application called cudaDeviceReset: ask the runtime
        // whether the pointer is still device memory of the current context, and look it up again if not.
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, scratch) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
            (void)cudaGetLastError();
            e = ScratchForCurrentDevice(&scratch, true);
        }
    }
    if (e != cudaSuccess) {
        return Fail(ACLNN_ERR_RUNTIME_ERROR, "%s: cannot locate the table array: %s", api, cudaGetErrorString(e));
    }
    const LerpAxis th{reinterpret_cast<int32_t*>(scratch), reinterpret_cast<int32_t*>(scratch + kMaxExtent),
                      reinterpret_cast<float*>(scratch + 2 * kMaxExtent)};
    const LerpAxis tw{reinterpret_cast<int32_t*>(scratch + 3 * kMaxExtent),
                      reinterpret_cast<int32_t*>(scratch + 4 * kMaxExtent),
                      reinterpret_cast<float*>(scratch + 5 * kMaxExtent)};
    Shape4 sh{};
    sh.n = n;
    sh.c = c;
    sh.hin = static_cast<int32_t>(inH);
    sh.win = static_cast<int32_t>(inW);
    sh.hout = static_cast<int32_t>(outH);
    sh.wout = static_cast<int32_t>(outW);
    const AxisGeom ah{sh.hin, sh.hout, BilinearScale(inH, outH, alignCorners, static_cast<float>(scalesH))};
    const AxisGeom aw{sh.win, sh.wout, BilinearScale(inW, outW, alignCorners, static_cast<float>(scalesW))};
    const bool halfPixel = !alignCorners;
    e = BuildLerpTables(ah, aw, halfPixel, 0, th, tw, s);
    if (e == cudaSuccess) {
        BilinearPlan plan{};
        plan.schedule = BilinearPlan::kDirect; // the schedule that needs nothing but the two tables
        e = BilinearFwd(ToDt(dtype), format == ACL_FORMAT_NHWC ? kNHWC : kNCHW, self, out, sh, th, tw, plan, s);
    }
    if (e != cudaSuccess) {
        return Fail(ACLNN_ERR_RUNTIME_ERROR, "%s: %s", api, cudaGetErrorString(e));
    }
    return ACLNN_SUCCESS;
}
