// Nearest and bilinear forward on NCHW VIEWS (any non-negative element strides: crops, steps, channel slices of a
// larger buffer, broadcast batches on the input side): the kernels read the taps and write the results through the
// views' strides, so neither the gather copy that would first make the input contiguous nor the scatter copy that
// would move a staged result into the output view (each a read and a write of a whole tensor, and a launch) is
// needed. Packs of adjacent outputs are stored as one vector when the output's W stride is 1 and its other strides
// and base keep the alignment; otherwise element by element. The
// index tables and the arithmetic are those of the dense kernels: nearest is a copy; bilinear blends
// (1 - dx) * v_lo + dx * v_hi per source row and then (1 - dy) * top + dy * bottom, every operation rounded on its
// own (image/resize_bilinear_v2/op_kernel/arch35/resize_bilinear_v2_simt_nchw.h:84-146).
#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdStridedKernel(const T* __restrict__ x, InStrides st, T* __restrict__ y, InStrides so, int32_t hout,
                            int32_t wout, const int32_t* __restrict__ sh, const int32_t* __restrict__ sw, int64_t rows)
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
        T* yr = y + n * so.n + c * so.c + h * so.h + t0 * so.w;
        if (V > 1) { // chosen only for a unit W stride
            *reinterpret_cast<Pack<T, V>*>(yr) = out;
        } else {
            *yr = out.v[0];
        }
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    BilinearFwdStridedKernel(const T* __restrict__ x, InStrides st, T* __restrict__ y, InStrides so, int32_t hout,
                             int32_t wout, LerpAxis th, LerpAxis tw, int64_t rows)
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
        T* yr = y + n * so.n + c * so.c + h * so.h + t0 * so.w;
        if (V > 1) {
            StorePack<T, V>(yr, out);
        } else {
            *yr = DType<T>::FromF(out[0]);
        }
    }
}

// Widest pack the output view allows: unit W stride, every other stride and the base aligned to the pack.
int OutVec(int es, int32_t wout, const void* y, const InStrides& so)
{
    if (so.w != 1) {
        return 1;
    }
    for (int v = 16 / es; v > 1; v >>= 1) {
        if (wout % v == 0 && so.n % v == 0 && so.c % v == 0 && so.h % v == 0 && Aligned(y, static_cast<size_t>(v) * es)) {
            return v;
        }
    }
    return 1;
}

} // namespace

cudaError_t NearestFwdStrided(Dt dt, const void* x, InStrides st, void* y, InStrides so, Shape4 sh, NearestAxis th,
                              NearestAxis tw, cudaStream_t s)
{
    const int64_t rows = sh.n * sh.c * sh.hout;
    const int v = OutVec(DtSize(dt), sh.wout, y, so);
    const RowLaunch rl = RowTiling(rows, CeilDiv(static_cast<int64_t>(sh.wout), v), kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                NearestFwdStridedKernel<T, V><<<rl.grid, rl.block, 0, s>>>(static_cast<const T*>(x), st, static_cast<T*>(y),
                                                                           so, sh.hout, sh.wout, th.src, tw.src, rows);
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BilinearFwdStrided(Dt dt, const void* x, InStrides st, void* y, InStrides so, Shape4 sh, LerpAxis th,
                               LerpAxis tw, cudaStream_t s)
{
    const int64_t rows = sh.n * sh.c * sh.hout;
    const int v = OutVec(DtSize(dt), sh.wout, y, so);
    const RowLaunch rl = RowTiling(rows, CeilDiv(static_cast<int64_t>(sh.wout), v), kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                BilinearFwdStridedKernel<T, V><<<rl.grid, rl.block, 0, s>>>(static_cast<const T*>(x), st, static_cast<T*>(y),
                                                                            so, sh.hout, sh.wout, th, tw, rows);
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
