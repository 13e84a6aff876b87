// UpsampleBicubic2dAA forward and backward (NCHW).
//
// The anti-aliased bicubic filter is separable: out[i][j] = sum_m wH[i][m] * sum_n wW[j][n] * x[hmin_i+m][wmin_j+n]
// with per-axis windows and normalised weights that depend only on the output index. tables.cu builds those
// windows / weights once per call; the kernels here never evaluate the cubic.
//
// Forward
//   * streaming kernel (down-scaling, the common case): a block owns a band of output rows of one plane and
//     streams the input rows that band needs exactly once, 16 bytes per thread, fully coalesced. Each thread
//     owns four input columns and carries a small ring of partial sums, one per output row whose vertical window
//     is currently open (an input row touches only ~support/scale output rows). When an output row's window
//     closes, its vertically filtered row (still at input width) goes to shared memory and the block applies the
//     horizontal filter, each thread producing output columns with its weights held in registers.
//     Input is read once from HBM, nothing but the output is written.
//   * direct kernel (any shape): one thread per output element, double loop over the window in the reference's
//     accumulation order (rows outer, columns inner).
// Backward
//   * gather kernel: one thread per grad_input element sums the outputs whose windows cover it, rows outer,
//     columns inner; deterministic. A block-tiled variant serves the down-scaling case, where each output row
//     fans out to many input rows.
//   * atomic kernel: the reference's scatter with fp32 atomics (selectable).
//
// Reference arithmetic: image/upsample_bicubic2d_aa/op_kernel/arch35/upsample_bicubic2d_aa_simt_base.h:52-127,
// image/upsample_bicubic2d_aa_grad/op_kernel/arch35/upsample_bicubic2d_aa_grad_simt_base.h:32-102 and
// upsample_bicubic2d_aa_grad_simt_base_deter.h:30-122.
#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

// ---- forward, direct ----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    AAFwdDirectKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                      int32_t wout, AAAxis th, AAAxis tw, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / wout;
        const int32_t w = static_cast<int32_t>(idx - row * wout);
        const int64_t p = row / hout;
        const int32_t h = static_cast<int32_t>(row - p * hout);
        const int32_t hmin = __ldg(th.xmin + h), hsz = __ldg(th.xsize + h);
        const int32_t wmin = __ldg(tw.xmin + w), wsz = __ldg(tw.xsize + w);
        const float* wh = th.w + static_cast<int64_t>(h) * th.taps;
        const float* ww = tw.w + static_cast<int64_t>(w) * tw.taps;
        const T* xp = x + p * hin * static_cast<int64_t>(win);
        float value = 0.0f;
        for (int32_t m = 0; m < hsz; ++m) {
            const float weightH = __ldg(wh + m);
            const T* xr = xp + static_cast<int64_t>(hmin + m) * win + wmin;
            for (int32_t n = 0; n < wsz; ++n) {
                // value += x * weightsH * weightsW  (simt_base.h:121)
                value = Add(value, Mul(Mul(DType<T>::Load(xr + n), weightH), __ldg(ww + n)));
            }
        }
        y[idx] = DType<T>::FromF(value);
    }
}

// ---- backward, gather (direct) --------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    AABwdGatherKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                      int32_t wout, AAAxis th, AAAxis tw, RangeAxis rh, RangeAxis rw, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / win;
        const int32_t x = static_cast<int32_t>(idx - row * win);
        const int64_t p = row / hin;
        const int32_t y = static_cast<int32_t>(row - p * hin);
        const int32_t is = __ldg(rh.start + y), ie = __ldg(rh.end + y);
        const int32_t js = __ldg(rw.start + x), je = __ldg(rw.end + x);
        const T* gp = go + p * hout * static_cast<int64_t>(wout);
        float value = 0.0f;
        for (int32_t i = is; i < ie; ++i) {
            const int32_t ty = y - __ldg(th.xmin + i);
            if (ty < 0 || ty >= __ldg(th.xsize + i)) {
                continue;
            }
            const float weightH = __ldg(th.w + static_cast<int64_t>(i) * th.taps + ty);
            if (weightH == 0.0f) {
                continue;
            }
            const T* gr = gp + static_cast<int64_t>(i) * wout;
            for (int32_t j = js; j < je; ++j) {
                const int32_t tx = x - __ldg(tw.xmin + j);
                if (tx < 0 || tx >= __ldg(tw.xsize + j)) {
                    continue;
                }
                const float weightW = __ldg(tw.w + static_cast<int64_t>(j) * tw.taps + tx);
                if (weightW == 0.0f) {
                    continue;
                }
                value = Add(value, Mul(Mul(DType<T>::Load(gr + j), weightH), weightW));
            }
        }
        gi[idx] = DType<T>::FromF(value);
    }
}

// ---- backward, atomic -------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    AABwdAtomicKernel(const T* __restrict__ go, float* __restrict__ acc, int32_t hin, int32_t win, int32_t hout,
                      int32_t wout, AAAxis th, AAAxis tw, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / wout;
        const int32_t w = static_cast<int32_t>(idx - row * wout);
        const int64_t p = row / hout;
        const int32_t h = static_cast<int32_t>(row - p * hout);
        const int32_t hmin = __ldg(th.xmin + h), hsz = __ldg(th.xsize + h);
        const int32_t wmin = __ldg(tw.xmin + w), wsz = __ldg(tw.xsize + w);
        const float* wh = th.w + static_cast<int64_t>(h) * th.taps;
        const float* ww = tw.w + static_cast<int64_t>(w) * tw.taps;
        const float v = DType<T>::Load(go + idx);
        float* ap = acc + p * hin * static_cast<int64_t>(win);
        for (int32_t m = 0; m < hsz; ++m) {
            const float weightH = __ldg(wh + m);
            if (weightH == 0.0f) {
                continue;
            }
            float* ar = ap + static_cast<int64_t>(hmin + m) * win + wmin;
            for (int32_t n = 0; n < wsz; ++n) {
                const float weightW = __ldg(ww + n);
                if (weightW == 0.0f) {
                    continue;
                }
                atomicAdd(ar + n, Mul(Mul(v, weightH), weightW));
            }
        }
    }
}

} // namespace

cudaError_t BicubicAAFwd(Dt dt, const void* x, void* y, Shape4 sh, AAAxis th, AAAxis tw, cudaStream_t s)
{
    const int64_t total = sh.n * sh.c * sh.hout * static_cast<int64_t>(sh.wout);
    OPSCV_DISPATCH_DT(dt, T, {
        AAFwdDirectKernel<T><<<GridFor(total, kThreads), kThreads, 0, s>>>(
            static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th, tw, total);
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BicubicAABwdGather(Dt dt, const void* go, void* gi, Shape4 sh, AAAxis th, AAAxis tw, RangeAxis rh,
                               RangeAxis rw, cudaStream_t s)
{
    const int64_t total = sh.n * sh.c * sh.hin * static_cast<int64_t>(sh.win);
    OPSCV_DISPATCH_DT(dt, T, {
        AABwdGatherKernel<T><<<GridFor(total, kThreads), kThreads, 0, s>>>(
            static_cast<const T*>(go), static_cast<T*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th, tw, rh, rw, total);
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BicubicAABwdAtomic(Dt dt, const void* go, void* gi, float* acc, Shape4 sh, AAAxis th, AAAxis tw,
                               cudaStream_t s)
{
    const int64_t outElems = sh.n * sh.c * sh.hin * static_cast<int64_t>(sh.win);
    const int64_t total = sh.n * sh.c * sh.hout * static_cast<int64_t>(sh.wout);
    cudaError_t e = cudaMemsetAsync(acc, 0, static_cast<size_t>(outElems) * sizeof(float), s);
    if (e != cudaSuccess) {
        return e;
    }
    OPSCV_DISPATCH_DT(dt, T, {
        AABwdAtomicKernel<T><<<GridFor(total, kThreads), kThreads, 0, s>>>(static_cast<const T*>(go), acc, sh.hin,
                                                                           sh.win, sh.hout, sh.wout, th, tw, total);
    });
    CountLaunch(2);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        return e;
    }
    if (dt != Dt::F32 || static_cast<void*>(acc) != gi) {
        return CastFromF32(dt, gi, acc, outElems, s);
    }
    return cudaSuccess;
}

} // namespace opscv
