// UpsampleBilinear2d forward and backward.
//
// Forward, NCHW: a block copies the input rows its band of output rows reads into shared memory (coalesced
// 16-byte loads, tile_stage.cuh). A thread owns one 16-byte group of output columns and walks down a chunk of output rows. The
// reference formula  (1-dy)*((1-dx)*TL + dx*TR) + dy*((1-dx)*BL + dx*BR)  is a vertical blend of two horizontally
// interpolated input rows, so the thread keeps the horizontal interpolation of the current top and bottom input
// rows in registers and only touches memory when the walk reaches a new input row: for 2x up-sampling that is
// one gathered load per output element instead of four, with bit-identical results.
// Forward, NHWC: a thread owns 16 bytes of channels of one output pixel; the four taps are 16-byte loads.
//
// Backward, gather (default and deterministic mode). NCHW: the grads rows feeding a band of grad_input rows are
// staged in shared memory; a thread owns a group of grad_input columns, holds their horizontal tap weights in
// registers and walks down the grads rows: each grads row is reduced horizontally once and added, with its two
// vertical weights, to the (at most two) grad_input rows it touches. Fixed summation order: reproducible.
// NHWC (and NCHW shapes the walk does not cover): a thread owns a 16-byte group of grad_input elements and sums, in
// grads row-major order, the products the reference's scatter kernel would add to them; equal to that kernel run
// serially.
// Backward, atomic: the scatter itself with fp32 atomics (kept selectable; slower than the gather here).
//
// Reference arithmetic: image/resize_bilinear_v2/op_kernel/arch35/resize_bilinear_v2_simt_nchw.h:84-146,
// _simt_nhwc.h:88-151; image/resize_bilinear_v2_grad/op_kernel/arch35/resize_bilinear_v2_grad_simt.h:107-152.
#include <algorithm>

#include "launch_util.cuh"
#include "tile_stage.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;
constexpr int kWalkThreads = 256;
constexpr int64_t kStageBudget = 32 * 1024; // staged bytes per block: keeps >= 6 blocks resident per SM

// ---- forward, NCHW ----------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdNCHWKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                          int32_t wout, LerpAxis th, LerpAxis tw, int32_t rowsPerThread, int32_t rowChunks,
                          int64_t totalThreads)
{
    const int32_t groups = wout / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; tid < totalThreads; tid += stride) {
        const int64_t pc = tid / groups;
        const int32_t g = static_cast<int32_t>(tid - pc * groups);
        const int64_t p = pc / rowChunks;
        const int32_t chunk = static_cast<int32_t>(pc - p * rowChunks);
        int32_t wl[V], wh[V];
        float dx[V], dx1[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            wl[k] = __ldg(tw.lo + g * V + k);
            wh[k] = __ldg(tw.hi + g * V + k);
            dx[k] = __ldg(tw.delta + g * V + k);
            dx1[k] = Sub(1.0f, dx[k]);
        }
        const T* xp = x + p * hin * static_cast<int64_t>(win);
        T* yp = y + p * hout * static_cast<int64_t>(wout) + static_cast<int64_t>(g) * V;
        float top[V], bot[V];
        int32_t curTop = -1, curBot = -1;
        const int32_t h0 = chunk * rowsPerThread;
        const int32_t h1 = min(hout, h0 + rowsPerThread);
        for (int32_t h = h0; h < h1; ++h) {
            const int32_t lo = __ldg(th.lo + h), hi = __ldg(th.hi + h);
            const float dy = __ldg(th.delta + h);
            if (lo != curTop) {
                if (lo == curBot) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = bot[k];
                    }
                } else {
                    const T* xr = xp + static_cast<int64_t>(lo) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = Add(Mul(dx1[k], DType<T>::Load(xr + wl[k])), Mul(dx[k], DType<T>::Load(xr + wh[k])));
                    }
                }
                curTop = lo;
            }
            if (hi != curBot) {
                if (hi == curTop) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = top[k];
                    }
                } else {
                    const T* xr = xp + static_cast<int64_t>(hi) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = Add(Mul(dx1[k], DType<T>::Load(xr + wl[k])), Mul(dx[k], DType<T>::Load(xr + wh[k])));
                    }
                }
                curBot = hi;
            }
            const float dy1 = Sub(1.0f, dy);
            float out[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                out[k] = Add(Mul(dy1, top[k]), Mul(dy, bot[k]));
            }
            StorePack<T, V>(yp + static_cast<int64_t>(h) * wout, out);
        }
    }
}

// ---- forward, NCHW, shared-memory staged ---------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdTileKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                          int32_t wout, LerpAxis th, LerpAxis tw, int32_t tileRows, int32_t tilesPerPlane,
                          int64_t capElems)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    const int64_t p = blockIdx.x / tilesPerPlane;
    const int32_t tile = blockIdx.x - p * tilesPerPlane;
    const int32_t h0 = tile * tileRows, h1 = min(hout, h0 + tileRows);
    const int32_t r0 = __ldg(th.lo + h0), r1 = __ldg(th.hi + h1 - 1) + 1;
    const T* plane = x + p * hin * static_cast<int64_t>(win);
    const int64_t count = static_cast<int64_t>(r1 - r0) * win;
    const T* src = plane;
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
    const int32_t chunk = (h1 - h0 + rowThreads - 1) / rowThreads;
    const int32_t ha = h0 + rc * chunk, hb = min(h1, ha + chunk);
    T* yp = y + p * hout * static_cast<int64_t>(wout);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        int32_t wl[V], wh[V];
        float dx[V], dx1[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            wl[k] = __ldg(tw.lo + g * V + k);
            wh[k] = __ldg(tw.hi + g * V + k);
            dx[k] = __ldg(tw.delta + g * V + k);
            dx1[k] = Sub(1.0f, dx[k]);
        }
        float top[V], bot[V];
        int32_t curTop = -1, curBot = -1;
        for (int32_t h = ha; h < hb; ++h) {
            const int32_t lo = __ldg(th.lo + h), hi = __ldg(th.hi + h);
            const float dy = __ldg(th.delta + h);
            if (lo != curTop) {
                if (lo == curBot) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = bot[k];
                    }
                } else {
                    const T* xr = src + static_cast<int64_t>(lo - rbase) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        top[k] = Add(Mul(dx1[k], DType<T>::ToF(xr[wl[k]])), Mul(dx[k], DType<T>::ToF(xr[wh[k]])));
                    }
                }
                curTop = lo;
            }
            if (hi != curBot) {
                if (hi == curTop) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = top[k];
                    }
                } else {
                    const T* xr = src + static_cast<int64_t>(hi - rbase) * win;
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        bot[k] = Add(Mul(dx1[k], DType<T>::ToF(xr[wl[k]])), Mul(dx[k], DType<T>::ToF(xr[wh[k]])));
                    }
                }
                curBot = hi;
            }
            const float dy1 = Sub(1.0f, dy);
            float out[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                out[k] = Add(Mul(dy1, top[k]), Mul(dy, bot[k]));
            }
            StorePack<T, V>(yp + static_cast<int64_t>(h) * wout + g * V, out);
        }
    }
}

// ---- forward, NHWC ----------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdNHWCKernel(const T* __restrict__ x, T* __restrict__ y, int32_t c, int32_t hin, int32_t win,
                          int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, int64_t totalGroups)
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
        const int32_t hl = __ldg(th.lo + h), hh = __ldg(th.hi + h);
        const int32_t wl = __ldg(tw.lo + w), wh = __ldg(tw.hi + w);
        const float dy = __ldg(th.delta + h), dx = __ldg(tw.delta + w);
        const float dy1 = Sub(1.0f, dy), dx1 = Sub(1.0f, dx);
        const T* xn = x + n * hin * static_cast<int64_t>(win) * c + g * V;
        float lt[V], rt[V], lb[V], rb[V], out[V];
        LoadPackLdg<T, V>(xn + (static_cast<int64_t>(hl) * win + wl) * c, lt);
        LoadPackLdg<T, V>(xn + (static_cast<int64_t>(hl) * win + wh) * c, rt);
        LoadPackLdg<T, V>(xn + (static_cast<int64_t>(hh) * win + wl) * c, lb);
        LoadPackLdg<T, V>(xn + (static_cast<int64_t>(hh) * win + wh) * c, rb);
#pragma unroll
        for (int k = 0; k < V; ++k) {
            out[k] = Add(Mul(dy1, Add(Mul(dx1, lt[k]), Mul(dx, rt[k]))), Mul(dy, Add(Mul(dx1, lb[k]), Mul(dx, rb[k]))));
        }
        StorePack<T, V>(y + pix * c + static_cast<int64_t>(g) * V, out);
    }
}

// ---- backward, gather ---------------------------------------------------------------------------------------
// Adds to acc what the serial scatter would add to destination (y, x) from source (i, j), in its order
// TL, TR, BL, BR (resize_bilinear_v2_grad_simt.h:147-150): weights (dx1*dy1), (dx*dy1), (dx1*dy), (dx*dy) times g.
__device__ __forceinline__ float GatherTap(float acc, float g, int32_t y, int32_t x, int32_t loY, int32_t hiY,
                                           float dY, int32_t loX, int32_t hiX, float dX)
{
    const float dY1 = Sub(1.0f, dY), dX1 = Sub(1.0f, dX);
    if (loY == y) {
        if (loX == x) {
            acc = Add(acc, Mul(Mul(dX1, dY1), g));
        }
        if (hiX == x) {
            acc = Add(acc, Mul(Mul(dX, dY1), g));
        }
    }
    if (hiY == y) {
        if (loX == x) {
            acc = Add(acc, Mul(Mul(dX1, dY), g));
        }
        if (hiX == x) {
            acc = Add(acc, Mul(Mul(dX, dY), g));
        }
    }
    return acc;
}

template <typename TIn, typename TOut, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdGatherNCHWKernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int32_t hin, int32_t win,
                                int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, RangeAxis rh, RangeAxis rw,
                                int64_t totalGroups)
{
    const int32_t groups = win / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t row = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - row * groups);
        const int64_t p = row / hin;
        const int32_t y = static_cast<int32_t>(row - p * hin);
        const int32_t is = __ldg(rh.start + y), ie = __ldg(rh.end + y);
        int32_t js[V], je[V];
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            js[k] = __ldg(rw.start + g * V + k);
            je[k] = __ldg(rw.end + g * V + k);
            acc[k] = 0.0f;
        }
        const TIn* gp = go + p * hout * static_cast<int64_t>(wout);
        for (int32_t i = is; i < ie; ++i) {
            const int32_t loY = __ldg(th.lo + i), hiY = __ldg(th.hi + i);
            const float dY = __ldg(th.delta + i);
            const TIn* gr = gp + static_cast<int64_t>(i) * wout;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int32_t x = g * V + k;
                for (int32_t j = js[k]; j < je[k]; ++j) {
                    acc[k] = GatherTap(acc[k], DType<TIn>::Load(gr + j), y, x, loY, hiY, dY, __ldg(tw.lo + j),
                                       __ldg(tw.hi + j), __ldg(tw.delta + j));
                }
            }
        }
        StorePack<TOut, V>(gi + row * win + static_cast<int64_t>(g) * V, acc);
    }
}

template <typename TIn, typename TOut, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdGatherNHWCKernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int32_t c, int32_t hin,
                                int32_t win, int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, RangeAxis rh,
                                RangeAxis rw, int64_t totalGroups)
{
    const int32_t groups = c / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t pix = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - pix * groups);
        const int64_t nh = pix / win;
        const int32_t x = static_cast<int32_t>(pix - nh * win);
        const int64_t n = nh / hin;
        const int32_t y = static_cast<int32_t>(nh - n * hin);
        const int32_t is = __ldg(rh.start + y), ie = __ldg(rh.end + y);
        const int32_t js = __ldg(rw.start + x), je = __ldg(rw.end + x);
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            acc[k] = 0.0f;
        }
        for (int32_t i = is; i < ie; ++i) {
            const int32_t loY = __ldg(th.lo + i), hiY = __ldg(th.hi + i);
            const float dY = __ldg(th.delta + i);
            for (int32_t j = js; j < je; ++j) {
                const int32_t loX = __ldg(tw.lo + j), hiX = __ldg(tw.hi + j);
                const float dX = __ldg(tw.delta + j);
                float v[V];
                LoadPackLdg<TIn, V>(go + ((n * hout + i) * wout + j) * static_cast<int64_t>(c) + g * V, v);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    acc[k] = GatherTap(acc[k], v[k], y, x, loY, hiY, dY, loX, hiX, dX);
                }
            }
        }
        StorePack<TOut, V>(gi + pix * c + static_cast<int64_t>(g) * V, acc);
    }
}

// ---- backward, gather, NCHW, shared-memory staged row walk -----------------------------------------------------
// KW = compile-time bound on the number of grads columns feeding one grad_input column.
template <typename TIn, typename TOut, int V, int KW>
__global__ void __launch_bounds__(kWalkThreads)
    BilinearBwdWalkKernel(const TIn* __restrict__ go, TOut* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                          int32_t wout, LerpAxis th, LerpAxis tw, RangeAxis rh, RangeAxis rw, int32_t tileRows,
                          int32_t tilesPerPlane, int64_t capElems)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    const int64_t p = blockIdx.x / tilesPerPlane;
    const int32_t tile = blockIdx.x - p * tilesPerPlane;
    const int32_t y0 = tile * tileRows, y1 = min(hin, y0 + tileRows);
    const int32_t r0 = __ldg(rh.start + y0);
    const int32_t r1 = max(r0, __ldg(rh.end + y1 - 1));
    const TIn* plane = go + p * hout * static_cast<int64_t>(wout);
    const int64_t count = static_cast<int64_t>(r1 - r0) * wout;
    const TIn* src = plane;
    int32_t rbase = 0;
    if (count <= capElems) {
        src = StageSpan<TIn>(plane + static_cast<int64_t>(r0) * wout, count, smemRaw);
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
    const int32_t chunk = (y1 - y0 + rowThreads - 1) / rowThreads;
    const int32_t ya = y0 + rc * chunk, yb = min(y1, ya + chunk);
    if (ya >= yb) {
        return;
    }
    TOut* gp = gi + p * hin * static_cast<int64_t>(win);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        // horizontal taps of my columns: grads columns [js, js + cnt), cnt <= KW, with their combined weights
        int32_t js[V], cnt[V];
        float wx[V][KW];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const int32_t xcol = g * V + k;
            js[k] = __ldg(rw.start + xcol);
            cnt[k] = __ldg(rw.end + xcol) - js[k]; // normally <= KW; longer runs take the slow tail loop below
#pragma unroll
            for (int t = 0; t < KW; ++t) {
                float w = 0.0f;
                if (t < cnt[k]) {
                    const int32_t j = js[k] + t;
                    const float d = __ldg(tw.delta + j);
                    if (__ldg(tw.lo + j) == xcol) {
                        w = Sub(1.0f, d);
                    }
                    if (__ldg(tw.hi + j) == xcol) {
                        w = Add(w, d);
                    }
                }
                wx[k][t] = w;
            }
        }
        float accA[V], accB[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            accA[k] = 0.0f;
            accB[k] = 0.0f;
        }
        int32_t cur = ya;
        const int32_t is = __ldg(rh.start + ya), ie = max(is, __ldg(rh.end + yb - 1));
        for (int32_t i = is; i < ie; ++i) {
            const int32_t loY = __ldg(th.lo + i), hiY = __ldg(th.hi + i);
            const float dY = __ldg(th.delta + i);
            while (cur < loY && cur < yb) { // rows below loY are complete
                StorePack<TOut, V>(gp + static_cast<int64_t>(cur) * win + g * V, accA);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    accA[k] = accB[k];
                    accB[k] = 0.0f;
                }
                ++cur;
            }
            if (cur >= yb) {
                break;
            }
            const TIn* row = src + static_cast<int64_t>(i - rbase) * wout;
            float hp[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                float a = 0.0f;
#pragma unroll
                for (int t = 0; t < KW; ++t) {
                    // taps past the run are not read (they may lie outside the row, or hold Inf / NaN)
                    const float v = (t < cnt[k]) ? DType<TIn>::ToF(row[js[k] + t]) : 0.0f;
                    a = fmaf(wx[k][t], v, a);
                }
                for (int32_t t = KW; t < cnt[k]; ++t) { // run longer than the register-held taps (not expected)
                    const int32_t j = js[k] + t, xcol = g * V + k;
                    const float d = __ldg(tw.delta + j);
                    float w = 0.0f;
                    if (__ldg(tw.lo + j) == xcol) {
                        w = Sub(1.0f, d);
                    }
                    if (__ldg(tw.hi + j) == xcol) {
                        w = Add(w, d);
                    }
                    a = fmaf(w, DType<TIn>::ToF(row[j]), a);
                }
                hp[k] = a;
            }
            const float wLo = Sub(1.0f, dY), wHi = dY;
            if (loY == cur) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    accA[k] = fmaf(wLo, hp[k], accA[k]);
                }
            } else if (loY == cur + 1) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    accB[k] = fmaf(wLo, hp[k], accB[k]);
                }
            }
            if (hiY == cur) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    accA[k] = fmaf(wHi, hp[k], accA[k]);
                }
            } else if (hiY == cur + 1 && cur + 1 < yb) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    accB[k] = fmaf(wHi, hp[k], accB[k]);
                }
            }
        }
        while (cur < yb) {
            StorePack<TOut, V>(gp + static_cast<int64_t>(cur) * win + g * V, accA);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                accA[k] = accB[k];
                accB[k] = 0.0f;
            }
            ++cur;
        }
    }
}

// ---- backward, atomic ---------------------------------------------------------------------------------------
template <typename TIn, int V, int LAY>
__global__ void __launch_bounds__(kThreads)
    BilinearBwdAtomicKernel(const TIn* __restrict__ go, float* __restrict__ acc, int32_t c, int32_t hin, int32_t win,
                            int32_t hout, int32_t wout, LerpAxis th, LerpAxis tw, int64_t totalGroups)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        float v[V];
        LoadPackLdg<TIn, V>(go + gid * V, v);
        if constexpr (LAY == kNCHW) {
            const int32_t groups = wout / V;
            const int64_t row = gid / groups;
            const int32_t g = static_cast<int32_t>(gid - row * groups);
            const int64_t p = row / hout;
            const int32_t h = static_cast<int32_t>(row - p * hout);
            const int32_t loY = __ldg(th.lo + h), hiY = __ldg(th.hi + h);
            const float dY = __ldg(th.delta + h), dY1 = Sub(1.0f, dY);
            float* ap = acc + p * hin * static_cast<int64_t>(win);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int32_t w = g * V + k;
                const int32_t loX = __ldg(tw.lo + w), hiX = __ldg(tw.hi + w);
                const float dX = __ldg(tw.delta + w), dX1 = Sub(1.0f, dX);
                atomicAdd(ap + static_cast<int64_t>(loY) * win + loX, Mul(Mul(dX1, dY1), v[k]));
                atomicAdd(ap + static_cast<int64_t>(loY) * win + hiX, Mul(Mul(dX, dY1), v[k]));
                atomicAdd(ap + static_cast<int64_t>(hiY) * win + loX, Mul(Mul(dX1, dY), v[k]));
                atomicAdd(ap + static_cast<int64_t>(hiY) * win + hiX, Mul(Mul(dX, dY), v[k]));
            }
        } else {
            const int32_t groups = c / V;
            const int64_t pix = gid / groups;
            const int32_t g = static_cast<int32_t>(gid - pix * groups);
            const int64_t nh = pix / wout;
            const int32_t w = static_cast<int32_t>(pix - nh * wout);
            const int64_t n = nh / hout;
            const int32_t h = static_cast<int32_t>(nh - n * hout);
            const int32_t loY = __ldg(th.lo + h), hiY = __ldg(th.hi + h);
            const int32_t loX = __ldg(tw.lo + w), hiX = __ldg(tw.hi + w);
            const float dY = __ldg(th.delta + h), dY1 = Sub(1.0f, dY);
            const float dX = __ldg(tw.delta + w), dX1 = Sub(1.0f, dX);
            float* an = acc + n * hin * static_cast<int64_t>(win) * c + g * V;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                atomicAdd(an + (static_cast<int64_t>(loY) * win + loX) * c + k, Mul(Mul(dX1, dY1), v[k]));
                atomicAdd(an + (static_cast<int64_t>(loY) * win + hiX) * c + k, Mul(Mul(dX, dY1), v[k]));
                atomicAdd(an + (static_cast<int64_t>(hiY) * win + loX) * c + k, Mul(Mul(dX1, dY), v[k]));
                atomicAdd(an + (static_cast<int64_t>(hiY) * win + hiX) * c + k, Mul(Mul(dX, dY), v[k]));
            }
        }
    }
}

template <typename TIn, typename TOut>
cudaError_t LaunchGather(Layout lay, const void* go, void* gi, Shape4 sh, LerpAxis th, LerpAxis tw, RangeAxis rh,
                         RangeAxis rw, bool exactScale, float scaleH, float scaleW, cudaStream_t s)
{
    if (lay == kNCHW) {
        int v = PickVec(sizeof(TOut), sh.win, {gi});
        // grads rows / columns feeding one grad_input row / column: those with source coordinate in (y-1, y+1),
        // i.e. at most 2/scale + 2. That bound needs the source coordinates to stay inside the input (true for
        // scale = in/out and for align_corners); user scales that overshoot pile many grads columns onto the last
        // input column, so they go to the direct kernel (exactScale = false).
        const double invH = scaleH > 0.0f ? 1.0 / scaleH : 1e9, invW = scaleW > 0.0f ? 1.0 / scaleW : 1e9;
        const int64_t tapsW = invW > 100.0 ? 1000 : static_cast<int64_t>(2.0 * invW) + 2;
        auto need = [&](int32_t t) {
            const double r = (t + 1) * invH + 4.0;
            return r < sh.hout ? static_cast<int32_t>(r) : sh.hout;
        };
        const int64_t rowBytes = static_cast<int64_t>(sh.wout) * sizeof(TIn);
        const int32_t tileRows = PickTileRows(sh.hin, rowBytes, kStageBudget, need);
        const int64_t planes = sh.n * sh.c;
        const bool walk = exactScale && tapsW <= 8 && tileRows > 0 && planes * CeilDiv(sh.hin, tileRows) < (1LL << 31);
        if (walk) {
            v = std::min<int>(v, std::max<int>(1, 4 / static_cast<int>(sizeof(TOut)))); // 4 bytes per lane
            const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hin, tileRows));
            const int64_t cap = static_cast<int64_t>(need(tileRows)) * sh.wout;
            const size_t smem = StageBytes(cap, sizeof(TIn));
            const unsigned blocks = static_cast<unsigned>(planes * tiles);
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V <= 2) {
                    if (tapsW <= 4) {
                        BilinearBwdWalkKernel<TIn, TOut, V, 4><<<blocks, kWalkThreads, smem, s>>>(
                            static_cast<const TIn*>(go), static_cast<TOut*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th,
                            tw, rh, rw, tileRows, tiles, cap);
                    } else {
                        BilinearBwdWalkKernel<TIn, TOut, V, 8><<<blocks, kWalkThreads, smem, s>>>(
                            static_cast<const TIn*>(go), static_cast<TOut*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th,
                            tw, rh, rw, tileRows, tiles, cap);
                    }
                }
            });
        } else {
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(TOut) <= 16) {
                    const int64_t total = sh.n * sh.c * sh.hin * (sh.win / V);
                    BilinearBwdGatherNCHWKernel<TIn, TOut, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const TIn*>(go), static_cast<TOut*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th, tw,
                        rh, rw, total);
                }
            });
        }
    } else {
        const int elem = sizeof(TIn) > sizeof(TOut) ? sizeof(TIn) : sizeof(TOut);
        const int v = PickVec(elem, sh.c, {go, gi});
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(TIn) <= 16 && V * sizeof(TOut) <= 16) {
                const int64_t total = sh.n * sh.hin * sh.win * (sh.c / V);
                BilinearBwdGatherNHWCKernel<TIn, TOut, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                    static_cast<const TIn*>(go), static_cast<TOut*>(gi), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                    sh.hout, sh.wout, th, tw, rh, rw, total);
            }
        });
    }
    CountLaunch();
    return cudaGetLastError();
}

} // namespace

cudaError_t BilinearFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, LerpAxis th, LerpAxis tw,
                        cudaStream_t s)
{
    OPSCV_DISPATCH_DT(dt, T, {
        if (lay == kNCHW) {
            int v = PickVec(sizeof(T), sh.wout, {y});
            // input rows read by t consecutive output rows: hi(h0+t-1) - lo(h0) + 1 <= (t-1)*scale + 3
            const double ratio = static_cast<double>(sh.hin) / sh.hout;
            auto need = [&](int32_t t) {
                const int64_t r = static_cast<int64_t>((t - 1) * ratio) + 4;
                return static_cast<int32_t>(r < sh.hin ? r : sh.hin);
            };
            const int64_t rowBytes = static_cast<int64_t>(sh.win) * sizeof(T);
            const int32_t tileRows = PickTileRows(sh.hout, rowBytes, kStageBudget, need);
            const int64_t planes = sh.n * sh.c;
            const bool tiled = tileRows > 0 && planes * CeilDiv(sh.hout, tileRows) < (1LL << 31);
            if (tiled) {
                v = std::min<int>(v, 4 / static_cast<int>(sizeof(T))); // 4 bytes per lane: see the kernel's mapping
            }
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    if (tiled) {
                        const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hout, tileRows));
                        const int64_t cap = static_cast<int64_t>(need(tileRows)) * sh.win;
                        BilinearFwdTileKernel<T, V>
                            <<<static_cast<unsigned>(planes * tiles), kThreads, StageBytes(cap, sizeof(T)), s>>>(
                                static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th, tw,
                                tileRows, tiles, cap);
                    } else {
                        // Rows too long to stage: gather from global memory. Split the rows of a plane into
                        // chunks only as far as needed to fill the machine (longer walks reuse more rows).
                        const int64_t columns = planes * (sh.wout / V);
                        const int64_t wanted = static_cast<int64_t>(NumSMs()) * 2048 * 2;
                        int64_t chunks = CeilDiv(wanted, columns > 0 ? columns : 1);
                        chunks = chunks < 1 ? 1 : (chunks > sh.hout ? sh.hout : chunks);
                        const int32_t rows = static_cast<int32_t>(CeilDiv(sh.hout, chunks));
                        const int32_t rowChunks = static_cast<int32_t>(CeilDiv(sh.hout, rows));
                        const int64_t total = columns * rowChunks;
                        BilinearFwdNCHWKernel<T, V><<<GridFor(total, kThreads, 16), kThreads, 0, s>>>(
                            static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th, tw,
                            rows, rowChunks, total);
                    }
                }
            });
        } else {
            const int v = PickVec(sizeof(T), sh.c, {x, y});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    const int64_t total = sh.n * sh.hout * sh.wout * (sh.c / V);
                    BilinearFwdNHWCKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(x), static_cast<T*>(y), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                        sh.hout, sh.wout, th, tw, total);
                }
            });
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BilinearBwdGather(Dt dtIn, Dt dtOut, Layout lay, const void* go, void* gi, Shape4 sh, LerpAxis th,
                              LerpAxis tw, RangeAxis rh, RangeAxis rw, bool exactScale, float scaleH, float scaleW, cudaStream_t s)
{
    if (dtIn == dtOut) {
        OPSCV_DISPATCH_DT(dtIn, T, { return (LaunchGather<T, T>(lay, go, gi, sh, th, tw, rh, rw, exactScale, scaleH, scaleW, s)); });
    }
    if (dtIn == Dt::F32 && dtOut == Dt::F16) {
        return LaunchGather<float, __half>(lay, go, gi, sh, th, tw, rh, rw, exactScale, scaleH, scaleW, s);
    }
    if (dtIn == Dt::F32 && dtOut == Dt::BF16) {
        return LaunchGather<float, __nv_bfloat16>(lay, go, gi, sh, th, tw, rh, rw, exactScale, scaleH, scaleW, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t BilinearBwdAtomic(Dt dtIn, Dt dtOut, Layout lay, const void* go, void* gi, float* acc, Shape4 sh,
                              LerpAxis th, LerpAxis tw, cudaStream_t s)
{
    const int64_t outElems = sh.n * sh.c * sh.hin * sh.win;
    cudaError_t e = cudaMemsetAsync(acc, 0, static_cast<size_t>(outElems) * sizeof(float), s);
    if (e != cudaSuccess) {
        return e;
    }
    OPSCV_DISPATCH_DT(dtIn, T, {
        const int64_t inner = lay == kNCHW ? sh.wout : sh.c;
        const int v = PickVec(sizeof(T), inner, {go});
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                const int64_t total = sh.n * sh.c * sh.hout * static_cast<int64_t>(sh.wout) / V;
                if (lay == kNCHW) {
                    BilinearBwdAtomicKernel<T, V, kNCHW><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(go), acc, static_cast<int32_t>(sh.c), sh.hin, sh.win, sh.hout, sh.wout,
                        th, tw, total);
                } else {
                    BilinearBwdAtomicKernel<T, V, kNHWC><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(go), acc, static_cast<int32_t>(sh.c), sh.hin, sh.win, sh.hout, sh.wout,
                        th, tw, total);
                }
            }
        });
    });
    CountLaunch(2);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        return e;
    }
    if (dtOut != Dt::F32 || static_cast<void*>(acc) != gi) {
        return CastFromF32(dtOut, gi, acc, outElems, s);
    }
    return cudaSuccess;
}

} // namespace opscv
