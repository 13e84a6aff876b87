// UpsampleNearest2d forward and backward.
//
// Both directions are output-major: one thread produces one 16-byte (or narrower, when alignment or the row
// length does not allow it) group of consecutive output elements, so every store is a full-width coalesced
// vector store; the gathered loads of neighbouring threads fall in the same or adjacent 32-byte sectors and are
// merged by L1. The per-row / per-column source indices come from the tables built by tables.cu.
//
// Reference arithmetic: image/resize_nearest_neighbor_v2/op_kernel/arch35/resize_nearest_neighbor_v2_simt.h:127-155
// (forward copy) and image/resize_nearest_neighbor_v2_grad/op_kernel/arch35/
// resize_nearest_neighbor_v2_grad_simt_determine.h:90-118 (backward: fp32 sum over the window, rows outer,
// columns inner, then one cast).
#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

// ---- forward ----------------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdNCHWKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, const int32_t* __restrict__ sh, const int32_t* __restrict__ sw,
                         int64_t totalGroups)
{
    const int32_t groups = wout / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t row = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - row * groups);
        const int64_t p = row / hout;
        const int32_t h = static_cast<int32_t>(row - p * hout);
        const T* xr = x + (p * hin + __ldg(sh + h)) * static_cast<int64_t>(win);
        Pack<T, V> out;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            out.v[k] = __ldg(xr + __ldg(sw + g * V + k));
        }
        *reinterpret_cast<Pack<T, V>*>(y + row * wout + static_cast<int64_t>(g) * V) = out;
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdNHWCKernel(const T* __restrict__ x, T* __restrict__ y, int32_t c, int32_t hin, int32_t win,
                         int32_t hout, int32_t wout, const int32_t* __restrict__ sh,
                         const int32_t* __restrict__ sw, int64_t totalGroups)
{
    const int32_t groups = c / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t pix = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - pix * groups);
        const int64_t nh = pix / wout;
        const int32_t w = static_cast<int32_t>(pix - nh * wout);
        const int64_t n = nh / hout;
        const int32_t h = static_cast<int32_t>(nh - n * hout);
        const T* src = x + ((n * hin + __ldg(sh + h)) * win + __ldg(sw + w)) * static_cast<int64_t>(c) + g * V;
        *reinterpret_cast<Pack<T, V>*>(y + pix * c + static_cast<int64_t>(g) * V) =
            *reinterpret_cast<const Pack<T, V>*>(src);
    }
}

// ---- backward ---------------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestBwdNCHWKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, RangeAxis th, RangeAxis tw, int64_t totalGroups)
{
    const int32_t groups = win / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t row = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - row * groups);
        const int64_t p = row / hin;
        const int32_t h = static_cast<int32_t>(row - p * hin);
        const int32_t hs = __ldg(th.start + h), he = __ldg(th.end + h);
        int32_t ws[V], we[V];
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            ws[k] = __ldg(tw.start + g * V + k);
            we[k] = __ldg(tw.end + g * V + k);
            acc[k] = 0.0f;
        }
        const T* gp = go + p * hout * static_cast<int64_t>(wout);
        for (int32_t i = hs; i < he; ++i) {
            const T* gr = gp + static_cast<int64_t>(i) * wout;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                for (int32_t j = ws[k]; j < we[k]; ++j) {
                    acc[k] = Add(acc[k], DType<T>::Load(gr + j));
                }
            }
        }
        StorePack<T, V>(gi + row * win + static_cast<int64_t>(g) * V, acc);
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestBwdNHWCKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t c, int32_t hin, int32_t win,
                         int32_t hout, int32_t wout, RangeAxis th, RangeAxis tw, int64_t totalGroups)
{
    const int32_t groups = c / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t pix = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - pix * groups);
        const int64_t nh = pix / win;
        const int32_t w = static_cast<int32_t>(pix - nh * win);
        const int64_t n = nh / hin;
        const int32_t h = static_cast<int32_t>(nh - n * hin);
        const int32_t hs = __ldg(th.start + h), he = __ldg(th.end + h);
        const int32_t ws = __ldg(tw.start + w), we = __ldg(tw.end + w);
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            acc[k] = 0.0f;
        }
        for (int32_t i = hs; i < he; ++i) {
            for (int32_t j = ws; j < we; ++j) {
                float v[V];
                LoadPackLdg<T, V>(go + ((n * hout + i) * wout + j) * static_cast<int64_t>(c) + g * V, v);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    acc[k] = Add(acc[k], v[k]);
                }
            }
        }
        StorePack<T, V>(gi + pix * c + static_cast<int64_t>(g) * V, acc);
    }
}

} // namespace

cudaError_t NearestFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, NearestAxis th, NearestAxis tw,
                       cudaStream_t s)
{
    const int64_t planes = sh.n * sh.c;
    OPSCV_DISPATCH_DT(dt, T, {
        if (lay == kNCHW) {
            const int v = PickVec(sizeof(T), sh.wout, {y});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    const int64_t total = planes * sh.hout * (sh.wout / V);
                    NearestFwdNCHWKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th.src,
                        tw.src, total);
                }
            });
        } else {
            const int v = PickVec(sizeof(T), sh.c, {x, y});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    const int64_t total = sh.n * sh.hout * sh.wout * (sh.c / V);
                    NearestFwdNHWCKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(x), static_cast<T*>(y), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                        sh.hout, sh.wout, th.src, tw.src, total);
                }
            });
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t NearestBwd(Dt dt, Layout lay, const void* go, void* gi, Shape4 sh, RangeAxis th, RangeAxis tw,
                       cudaStream_t s)
{
    const int64_t planes = sh.n * sh.c;
    OPSCV_DISPATCH_DT(dt, T, {
        if (lay == kNCHW) {
            const int v = PickVec(sizeof(T), sh.win, {gi});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    const int64_t total = planes * sh.hin * (sh.win / V);
                    NearestBwdNCHWKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(go), static_cast<T*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th, tw,
                        total);
                }
            });
        } else {
            const int v = PickVec(sizeof(T), sh.c, {go, gi});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    const int64_t total = sh.n * sh.hin * sh.win * (sh.c / V);
                    NearestBwdNHWCKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(go), static_cast<T*>(gi), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                        sh.hout, sh.wout, th, tw, total);
                }
            });
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
