// UpsampleBilinear2d forward and backward.
//
// Forward, NCHW: a thread owns one 16-byte group of output columns and walks down a chunk of output rows. The
// reference formula  (1-dy)*((1-dx)*TL + dx*TR) + dy*((1-dx)*BL + dx*BR)  is a vertical blend of two horizontally
// interpolated input rows, so the thread keeps the horizontal interpolation of the current top and bottom input
// rows in registers and only touches memory when the walk reaches a new input row: for 2x up-sampling that is
// one gathered load per output element instead of four, with bit-identical results.
// Forward, NHWC: a thread owns 16 bytes of channels of one output pixel; the four taps are 16-byte loads.
//
// Backward, gather (default and deterministic mode): a thread owns a 16-byte group of grad_input elements and
// sums, in grads row-major order, the contributions the reference's scatter kernel would add to them. The order
// and the products are those of the scatter kernel run serially, so the result is reproducible and equal to it.
// Backward, atomic: the scatter itself with fp32 atomics (kept selectable; slower than the gather here).
//
// Reference arithmetic: image/resize_bilinear_v2/op_kernel/arch35/resize_bilinear_v2_simt_nchw.h:84-146,
// _simt_nhwc.h:88-151; image/resize_bilinear_v2_grad/op_kernel/arch35/resize_bilinear_v2_grad_simt.h:107-152.
#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

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
                         RangeAxis rw, cudaStream_t s)
{
    if (lay == kNCHW) {
        const int v = PickVec(sizeof(TOut), sh.win, {gi});
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(TOut) <= 16) {
                const int64_t total = sh.n * sh.c * sh.hin * (sh.win / V);
                BilinearBwdGatherNCHWKernel<TIn, TOut, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                    static_cast<const TIn*>(go), static_cast<TOut*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th, tw, rh,
                    rw, total);
            }
        });
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
            const int v = PickVec(sizeof(T), sh.wout, {y});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    // Split the rows of a plane into chunks only as far as needed to fill the machine: longer
                    // walks reuse more input rows from registers.
                    const int64_t columns = sh.n * sh.c * (sh.wout / V);
                    const int64_t wanted = static_cast<int64_t>(NumSMs()) * 2048 * 2;
                    int64_t chunks = CeilDiv(wanted, columns > 0 ? columns : 1);
                    chunks = chunks < 1 ? 1 : (chunks > sh.hout ? sh.hout : chunks);
                    const int32_t rows = static_cast<int32_t>(CeilDiv(sh.hout, chunks));
                    const int32_t rowChunks = static_cast<int32_t>(CeilDiv(sh.hout, rows));
                    const int64_t total = columns * rowChunks;
                    BilinearFwdNCHWKernel<T, V><<<GridFor(total, kThreads, 16), kThreads, 0, s>>>(
                        static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th, tw, rows,
                        rowChunks, total);
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
                              LerpAxis tw, RangeAxis rh, RangeAxis rw, cudaStream_t s)
{
    if (dtIn == dtOut) {
        OPSCV_DISPATCH_DT(dtIn, T, { return (LaunchGather<T, T>(lay, go, gi, sh, th, tw, rh, rw, s)); });
    }
    if (dtIn == Dt::F32 && dtOut == Dt::F16) {
        return LaunchGather<float, __half>(lay, go, gi, sh, th, tw, rh, rw, s);
    }
    if (dtIn == Dt::F32 && dtOut == Dt::BF16) {
        return LaunchGather<float, __nv_bfloat16>(lay, go, gi, sh, th, tw, rh, rw, s);
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
