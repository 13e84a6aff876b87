// Nearest and bilinear forward on an NCHW input VIEW (any non-negative element strides: crops, steps, broadcast
// batches) with a dense NCHW output: the kernels read the taps through the view's strides, so the gather copy that
// would first make the input contiguous (a read and a write of the whole input, and a launch) is not needed. The
// index tables and the arithmetic are those of the dense kernels: nearest is a copy; bilinear blends
// (1 - dx) * v_lo + dx * v_hi per source row and then (1 - dy) * top + dy * bottom, every operation rounded on its
// own (image/resize_bilinear_v2/op_kernel/arch35/resize_bilinear_v2_simt_nchw.h:84-146).
#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdStridedKernel(const T* __restrict__ x, InStrides st, T* __restrict__ y, int32_t hout, int32_t wout,
                            const int32_t* __restrict__ sh, const int32_t* __restrict__ sw, int64_t rows)
{
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (t0 >= wout) {
        return;
    }
    int64_t off[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
        off[k] = __ldg(sw + t0 + k) * st.w;
    }
    const bool small = rows <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rows; row += rowStep) {
        int64_t n; // row = (n, c, h)
        int32_t c, h;
        SplitRow(row, hout, st.chan, small, n, c, h);
        const T* xr = x + n * st.n + c * st.c + __ldg(sh + h) * st.h;
        Pack<T, V> out;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            out.v[k] = __ldg(xr + off[k]);
        }
        *reinterpret_cast<Pack<T, V>*>(y + row * wout + t0) = out;
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdStridedKernel(const T* __restrict__ x, InStrides st, T* __restrict__ y, int32_t hout, int32_t wout,
                             LerpAxis th, LerpAxis tw, int64_t rows)
{
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (t0 >= wout) {
        return;
    }
    int64_t ol[V], oh[V];
    float dx[V], dx1[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
        ol[k] = __ldg(tw.lo + t0 + k) * st.w;
        oh[k] = __ldg(tw.hi + t0 + k) * st.w;
        dx[k] = __ldg(tw.delta + t0 + k);
        dx1[k] = Sub(1.0f, dx[k]);
    }
    const bool small = rows <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rows; row += rowStep) {
        int64_t n;
        int32_t c, h;
        SplitRow(row, hout, st.chan, small, n, c, h);
        const T* xp = x + n * st.n + c * st.c;
        const T* r0 = xp + __ldg(th.lo + h) * st.h;
        const T* r1 = xp + __ldg(th.hi + h) * st.h;
        const float dy = __ldg(th.delta + h);
        const float dy1 = Sub(1.0f, dy);
        float out[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const float top = Add(Mul(dx1[k], DType<T>::Load(r0 + ol[k])), Mul(dx[k], DType<T>::Load(r0 + oh[k])));
            const float bot = Add(Mul(dx1[k], DType<T>::Load(r1 + ol[k])), Mul(dx[k], DType<T>::Load(r1 + oh[k])));
            out[k] = Add(Mul(dy1, top), Mul(dy, bot));
        }
        StorePack<T, V>(y + row * wout + t0, out);
    }
}

} // namespace

cudaError_t NearestFwdStrided(Dt dt, const void* x, InStrides st, void* y, Shape4 sh, NearestAxis th, NearestAxis tw,
                              cudaStream_t s)
{
    const int64_t rows = sh.n * sh.c * sh.hout;
    const int v = PickVec(DtSize(dt), sh.wout, {y});
    const RowLaunch rl = RowTiling(rows, CeilDiv(static_cast<int64_t>(sh.wout), v), kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                NearestFwdStridedKernel<T, V><<<rl.grid, rl.block, 0, s>>>(static_cast<const T*>(x), st, static_cast<T*>(y),
                                                                           sh.hout, sh.wout, th.src, tw.src, rows);
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BilinearFwdStrided(Dt dt, const void* x, InStrides st, void* y, Shape4 sh, LerpAxis th, LerpAxis tw,
                               cudaStream_t s)
{
    const int64_t rows = sh.n * sh.c * sh.hout;
    const int v = PickVec(DtSize(dt), sh.wout, {y});
    const RowLaunch rl = RowTiling(rows, CeilDiv(static_cast<int64_t>(sh.wout), v), kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                BilinearFwdStridedKernel<T, V><<<rl.grid, rl.block, 0, s>>>(static_cast<const T*>(x), st, static_cast<T*>(y),
                                                                            sh.hout, sh.wout, th, tw, rows);
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
