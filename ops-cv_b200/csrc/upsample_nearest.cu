// UpsampleNearest2d forward and backward.
//
// Both directions are output-major: one thread produces one 16-byte (or narrower, when alignment or the row
// length does not allow it) group of consecutive output elements, so every store is a full-width coalesced
// vector store. NCHW: a block owns a band of output rows of one plane, copies the input rows that band reads into
// shared memory with coalesced 16-byte loads (tile_stage.cuh) and gathers from there; a thread keeps the source
// columns of its output group in registers and walks down the rows of the band. NHWC: a gathered pixel is a
// contiguous run of channels, so the taps are 16-byte global loads. The per-row / per-column source indices come
// from the tables built by tables.cu.
//
// Reference arithmetic: image/resize_nearest_neighbor_v2/op_kernel/arch35/resize_nearest_neighbor_v2_simt.h:127-155
// (forward copy) and image/resize_nearest_neighbor_v2_grad/op_kernel/arch35/
// resize_nearest_neighbor_v2_grad_simt_determine.h:90-118 (backward: fp32 sum over the window, rows outer,
// columns inner, then one cast).
#include <algorithm>

#include "launch_util.cuh"
#include "tile_stage.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;
constexpr int64_t kStageBudget = 32 * 1024; // staged bytes per block: keeps >= 6 blocks resident per SM

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

// NCHW, shared-memory staged. grid.x = planes * tilesPerPlane; a tile is `tileRows` output rows of one plane.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdTileKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, const int32_t* __restrict__ sh, const int32_t* __restrict__ sw,
                         int32_t tileRows, int32_t tilesPerPlane, int64_t capElems)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    const int64_t p = blockIdx.x / tilesPerPlane;
    const int32_t tile = blockIdx.x - p * tilesPerPlane;
    const int32_t h0 = tile * tileRows, h1 = min(hout, h0 + tileRows);
    const int32_t r0 = __ldg(sh + h0), r1 = __ldg(sh + h1 - 1) + 1;
    const T* plane = x + p * hin * static_cast<int64_t>(win);
    const int64_t count = static_cast<int64_t>(r1 - r0) * win;
    const T* src = plane; // fallback: gather from global memory if the band does not fit (never with host tiling)
    int32_t rbase = 0;
    if (count <= capElems) {
        src = StageSpan<T>(plane + static_cast<int64_t>(r0) * win, count, smemRaw);
        rbase = r0;
    }
    __syncthreads();
    // Lanes of a warp take adjacent column groups (whole warps per row), so that their shared-memory reads fall in
    // adjacent words (no bank conflicts) and each warp stores one contiguous run per row.
    const int32_t groups = wout / V;
    const int32_t colThreads = min((groups + 31) & ~31, static_cast<int32_t>(blockDim.x));
    const int32_t rowThreads = static_cast<int32_t>(blockDim.x) / colThreads;
    const int32_t cg0 = threadIdx.x % colThreads, rc = threadIdx.x / colThreads;
    if (rc >= rowThreads) {
        return;
    }
    T* yp = y + p * hout * static_cast<int64_t>(wout);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        int32_t col[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            col[k] = __ldg(sw + g * V + k);
        }
        for (int32_t h = h0 + rc; h < h1; h += rowThreads) {
            const T* row = src + static_cast<int64_t>(__ldg(sh + h) - rbase) * win;
            Pack<T, V> out;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                out.v[k] = row[col[k]];
            }
            *reinterpret_cast<Pack<T, V>*>(yp + static_cast<int64_t>(h) * wout + g * V) = out;
        }
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

// NCHW, shared-memory staged: a tile is `tileRows` grad_input rows of one plane; the grads rows of their windows
// are staged. Summation order per element is the reference's (window rows outer, columns inner), in fp32.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestBwdTileKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, RangeAxis th, RangeAxis tw, int32_t tileRows, int32_t tilesPerPlane,
                         int64_t capElems)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    const int64_t p = blockIdx.x / tilesPerPlane;
    const int32_t tile = blockIdx.x - p * tilesPerPlane;
    const int32_t y0 = tile * tileRows, y1 = min(hin, y0 + tileRows);
    const int32_t r0 = __ldg(th.start + y0);
    const int32_t r1 = max(r0, __ldg(th.end + y1 - 1));
    const T* plane = go + p * hout * static_cast<int64_t>(wout);
    const int64_t count = static_cast<int64_t>(r1 - r0) * wout;
    const T* src = plane;
    int32_t rbase = 0;
    if (count <= capElems) {
        src = StageSpan<T>(plane + static_cast<int64_t>(r0) * wout, count, smemRaw);
        rbase = r0;
    }
    __syncthreads();
    // Lanes of a warp take adjacent column groups (whole warps per row), so that their shared-memory reads fall in
    // adjacent words (no bank conflicts) and each warp stores one contiguous run per row.
    const int32_t groups = win / V;
    const int32_t colThreads = min((groups + 31) & ~31, static_cast<int32_t>(blockDim.x));
    const int32_t rowThreads = static_cast<int32_t>(blockDim.x) / colThreads;
    const int32_t cg0 = threadIdx.x % colThreads, rc = threadIdx.x / colThreads;
    if (rc >= rowThreads) {
        return;
    }
    T* gp = gi + p * hin * static_cast<int64_t>(win);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        int32_t ws[V], we[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            ws[k] = __ldg(tw.start + g * V + k);
            we[k] = __ldg(tw.end + g * V + k);
        }
        for (int32_t yy = y0 + rc; yy < y1; yy += rowThreads) {
            const int32_t hs = __ldg(th.start + yy), he = __ldg(th.end + yy);
            float acc[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                acc[k] = 0.0f;
            }
            for (int32_t i = hs; i < he; ++i) {
                const T* row = src + static_cast<int64_t>(i - rbase) * wout;
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    for (int32_t j = ws[k]; j < we[k]; ++j) {
                        acc[k] = Add(acc[k], DType<T>::ToF(row[j]));
                    }
                }
            }
            StorePack<T, V>(gp + static_cast<int64_t>(yy) * win + g * V, acc);
        }
    }
}

} // namespace

cudaError_t NearestFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, NearestAxis th, NearestAxis tw,
                       cudaStream_t s)
{
    const int64_t planes = sh.n * sh.c;
    OPSCV_DISPATCH_DT(dt, T, {
        if (lay == kNCHW) {
            int v = PickVec(sizeof(T), sh.wout, {y});
            // rows of input needed by t consecutive output rows: src = floor(dst * scale), so at most
            // floor((t-1)*scale) + 2; the ratio in/out bounds the scale the tables were built with from above
            // unless user scales were given, hence the generous +3 and the in-kernel fallback.
            const double ratio = static_cast<double>(sh.hin) / sh.hout;
            auto need = [&](int32_t t) {
                const int64_t r = static_cast<int64_t>((t - 1) * ratio) + 3;
                return static_cast<int32_t>(r < sh.hin ? r : sh.hin);
            };
            const int64_t rowBytes = static_cast<int64_t>(sh.win) * sizeof(T);
            const int32_t tileRows = PickTileRows(sh.hout, rowBytes, kStageBudget, need);
            const bool tiled = tileRows > 0 && planes * CeilDiv(sh.hout, tileRows) < (1LL << 31);
            if (tiled) {
                v = std::min<int>(v, 4 / static_cast<int>(sizeof(T))); // 4 bytes per lane: see the kernel's mapping
            }
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    if (tiled) {
                        const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hout, tileRows));
                        const int64_t cap = static_cast<int64_t>(need(tileRows)) * sh.win;
                        NearestFwdTileKernel<T, V>
                            <<<static_cast<unsigned>(planes * tiles), kThreads, StageBytes(cap, sizeof(T)), s>>>(
                                static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th.src,
                                tw.src, tileRows, tiles, cap);
                    } else {
                        const int64_t total = planes * sh.hout * (sh.wout / V);
                        NearestFwdNCHWKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                            static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th.src,
                            tw.src, total);
                    }
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
            int v = PickVec(sizeof(T), sh.win, {gi});
            // grads rows needed by t consecutive grad_input rows: [ceil(y*inv), ceil((y+t)*inv)) -> t*inv + 2
            const double inv = static_cast<double>(sh.hout) / sh.hin;
            auto need = [&](int32_t t) {
                const int64_t r = static_cast<int64_t>(t * inv) + 3;
                return static_cast<int32_t>(r < sh.hout ? r : sh.hout);
            };
            const int64_t rowBytes = static_cast<int64_t>(sh.wout) * sizeof(T);
            const int32_t tileRows = PickTileRows(sh.hin, rowBytes, kStageBudget, need);
            const bool tiled = tileRows > 0 && planes * CeilDiv(sh.hin, tileRows) < (1LL << 31);
            if (tiled) {
                v = std::min<int>(v, 4 / static_cast<int>(sizeof(T)));
            }
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    if (tiled) {
                        const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hin, tileRows));
                        const int64_t cap = static_cast<int64_t>(need(tileRows)) * sh.wout;
                        NearestBwdTileKernel<T, V>
                            <<<static_cast<unsigned>(planes * tiles), kThreads, StageBytes(cap, sizeof(T)), s>>>(
                                static_cast<const T*>(go), static_cast<T*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th, tw,
                                tileRows, tiles, cap);
                    } else {
                        const int64_t total = planes * sh.hin * (sh.win / V);
                        NearestBwdNCHWKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                            static_cast<const T*>(go), static_cast<T*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th, tw,
                            total);
                    }
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
