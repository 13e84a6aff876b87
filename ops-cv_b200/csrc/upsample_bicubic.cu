// UpsampleBicubic2d forward and backward (cubic convolution with A = -0.75, no antialiasing), NCHW and NHWC.
//
// Forward: one thread per output element; the sixteen clamped taps are read through the read-only path and
// combined in the reference's order (four row sums left to right, then the column sum), every operation rounded
// on its own, so fp32 results carry the bits of a serial CPU statement of
// image/resize_bicubic_v2/op_kernel/arch35/resize_bicubic_v2_simt_base.h:23-120. The four special schedules of
// resize_bicubic_v2_simt_nchw.h:50-90 (copy, one input pixel, one output pixel, integer positions) are selected on
// the host with the reference's rule and are plain copies here too.
//
// Backward: one thread per grad_input element gathers the grads that reach it, walking them in ascending
// (row, column) order. The walk, its start, its end and the coefficient expressions are those of the reference's
// gather kernel (image/resize_bicubic_v2_grad/op_kernel/arch35/resize_bicubic_v2_grad_simt_determine.h:95-350):
// an axis on which the element is interior is walked by distance to the source position, a first or last index
// tap by tap with clamped destinations. The sum has a fixed order, so results are reproducible from run to run
// and fp32 results carry the bits of that kernel run serially.
#include <algorithm>

#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;
constexpr float kA = -0.75f;

// ((a + 2) x - (a + 3)) x x + 1
__device__ __forceinline__ float Conv1(float x)
{
    return Add(Mul(Mul(Sub(Mul(kA + 2.0f, x), kA + 3.0f), x), x), 1.0f);
}
// ((a x - 5 a) x + 8 a) x - 4 a
__device__ __forceinline__ float Conv2(float x)
{
    return Sub(Mul(Add(Mul(Sub(Mul(kA, x), 5.0f * kA), x), 8.0f * kA), x), 4.0f * kA);
}
__device__ __forceinline__ void TapCoeff(float t, float (&c)[4])
{
    c[0] = Conv2(Add(t, 1.0f));
    c[1] = Conv1(t);
    const float u = Sub(1.0f, t);
    c[2] = Conv1(u);
    c[3] = Conv2(Add(u, 1.0f)); // the forward kernel writes 2 - t; see FwdCoeff
}
// resize_bicubic_v2_simt_base.h:33-41: the last argument is 2 - t (the backward kernels use (1 - t) + 1)
__device__ __forceinline__ void FwdCoeff(float t, float (&c)[4])
{
    c[0] = Conv2(Add(t, 1.0f));
    c[1] = Conv1(t);
    c[2] = Conv1(Sub(1.0f, t));
    c[3] = Conv2(Sub(2.0f, t));
}
// resize_bicubic_v2_grad_base.h:44-56
__device__ __forceinline__ float PointCoeff(float d)
{
    if (d <= 1.0f) {
        return Conv1(d);
    }
    if (d < 2.0f) {
        return Conv2(d);
    }
    return 0.0f;
}
__device__ __forceinline__ int32_t ClampIdx(long long v, int32_t last)
{
    return static_cast<int32_t>(v < 0 ? 0 : (v > last ? last : v));
}

struct BicubicGeom {
    int64_t rows;  // forward: planes * hout; backward: planes * hin
    int32_t hin, win, hout, wout;
    int32_t chan;  // NHWC: channels; NCHW: 1
    float scaleH, scaleW, invH, invW;
    int32_t align; // backward: align_corners; forward: !halfPixel
    int32_t schedule;
};

template <typename T, bool NHWC>
__global__ void __launch_bounds__(kThreads) Bicubic2dFwdKernel(const T* __restrict__ x, T* __restrict__ y, BicubicGeom g)
{
    const int32_t inner = g.wout * g.chan;
    const int64_t planeIn = static_cast<int64_t>(g.hin) * g.win * g.chan;
    const int64_t rowIn = static_cast<int64_t>(g.win) * g.chan;
    for (int64_t row = blockIdx.y; row < g.rows; row += gridDim.y) {
        const int64_t plane = row / g.hout;
        const int32_t H = static_cast<int32_t>(row - plane * g.hout);
        const float oh = g.align ? Mul(static_cast<float>(H), g.scaleH)
                                 : Sub(Mul(Add(static_cast<float>(H), 0.5f), g.scaleH), 0.5f);
        const float fh = floorf(oh);
        const long long top = static_cast<long long>(fh);
        float ch[4];
        FwdCoeff(Sub(oh, fh), ch);
        const T* px = x + plane * planeIn;
        const T* r0 = px + ClampIdx(top - 1, g.hin - 1) * rowIn;
        const T* r1 = px + ClampIdx(top, g.hin - 1) * rowIn;
        const T* r2 = px + ClampIdx(top + 1, g.hin - 1) * rowIn;
        const T* r3 = px + ClampIdx(top + 2, g.hin - 1) * rowIn;
        T* py = y + row * inner;
        for (int32_t t = blockIdx.x * kThreads + threadIdx.x; t < inner; t += gridDim.x * kThreads) {
            const int32_t W = NHWC ? t / g.chan : t;
            const int32_t c = NHWC ? t - W * g.chan : 0;
            if (g.schedule == 2 || g.schedule == 3) { // one input pixel / one output pixel: x[plane][0][0]
                py[t] = px[c];
                continue;
            }
            const float ow = g.align ? Mul(static_cast<float>(W), g.scaleW)
                                     : Sub(Mul(Add(static_cast<float>(W), 0.5f), g.scaleW), 0.5f);
            const float fw = floorf(ow);
            const long long left = static_cast<long long>(fw);
            if (g.schedule == 4) { // integer source positions: the pixel itself
                py[t] = r1[static_cast<int64_t>(ClampIdx(left, g.win - 1)) * g.chan + c];
                continue;
            }
            float cw[4];
            FwdCoeff(Sub(ow, fw), cw);
            const int64_t w0 = static_cast<int64_t>(ClampIdx(left - 1, g.win - 1)) * g.chan + c;
            const int64_t w1 = static_cast<int64_t>(ClampIdx(left, g.win - 1)) * g.chan + c;
            const int64_t w2 = static_cast<int64_t>(ClampIdx(left + 1, g.win - 1)) * g.chan + c;
            const int64_t w3 = static_cast<int64_t>(ClampIdx(left + 2, g.win - 1)) * g.chan + c;
            auto rowSum = [&](const T* r) {
                const float v0 = DType<T>::Load(r + w0), v1 = DType<T>::Load(r + w1), v2 = DType<T>::Load(r + w2),
                            v3 = DType<T>::Load(r + w3);
                return Add(Add(Add(Mul(v0, cw[0]), Mul(v1, cw[1])), Mul(v2, cw[2])), Mul(v3, cw[3]));
            };
            const float s0 = rowSum(r0), s1 = rowSum(r1), s2 = rowSum(r2), s3 = rowSum(r3);
            const float out = Add(Add(Add(Mul(s0, ch[0]), Mul(s1, ch[1])), Mul(s2, ch[2])), Mul(s3, ch[3]));
            py[t] = DType<T>::FromF(out);
        }
    }
}

__device__ __forceinline__ float BwdSrc(float scale, int32_t idx, int32_t align)
{
    return align ? Mul(scale, static_cast<float>(idx)) : Sub(Mul(scale, Add(static_cast<float>(idx), 0.5f)), 0.5f);
}

// First grads index of the walk for grad_input index yIdx (resize_bicubic_v2_grad_simt_determine.h:95-113)
__device__ __forceinline__ int32_t WalkStart(int32_t yIdx, float inverse, float offset)
{
    const float v = ceilf(Sub(Mul(Add(Sub(static_cast<float>(yIdx), 2.0f), offset), inverse), offset));
    const long long s = static_cast<long long>(v);
    return static_cast<int32_t>(s < 0 ? 0 : (s > INT32_MAX ? INT32_MAX : s));
}

template <typename T, bool NHWC>
__global__ void __launch_bounds__(kThreads) Bicubic2dBwdKernel(const T* __restrict__ go, T* __restrict__ gi, BicubicGeom g)
{
    const int32_t inner = g.win * g.chan;
    const int64_t planeGo = static_cast<int64_t>(g.hout) * g.wout * g.chan;
    const int64_t rowGo = static_cast<int64_t>(g.wout) * g.chan;
    const float offset = g.align ? 0.0f : 0.5f;
    for (int64_t row = blockIdx.y; row < g.rows; row += gridDim.y) {
        const int64_t plane = row / g.hin;
        const int32_t yh = static_cast<int32_t>(row - plane * g.hin);
        const int32_t hStart = WalkStart(yh, g.invH, offset);
        const float rhStart = Sub(Mul(Add(static_cast<float>(hStart), offset), g.scaleH), offset);
        const bool borderH = yh == 0 || yh == g.hin - 1;
        const T* pg = go + plane * planeGo;
        T* po = gi + row * inner;
        for (int32_t t = blockIdx.x * kThreads + threadIdx.x; t < inner; t += gridDim.x * kThreads) {
            const int32_t yw = NHWC ? t / g.chan : t;
            const int32_t c = NHWC ? t - yw * g.chan : 0;
            const int32_t wStart = WalkStart(yw, g.invW, offset);
            const float rwStart = Sub(Mul(Add(static_cast<float>(wStart), offset), g.scaleW), offset);
            const bool borderW = yw == 0 || yw == g.win - 1;
            float add = 0.0f;
            float rh = rhStart;
            for (int32_t h = hStart; h < g.hout; ++h, rh = BwdSrc(g.scaleH, h, g.align)) {
                float chTap[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                float chPoint = 0.0f;
                long long fh = 0;
                if (borderH) {
                    const float fl = floorf(rh);
                    fh = static_cast<long long>(fl);
                    if (yh == 0 && fh > 1 && g.hin > 1) {
                        break;
                    }
                    TapCoeff(Sub(rh, static_cast<float>(fh)), chTap);
                } else {
                    if (!(rh < Add(static_cast<float>(yh), 2.0f))) {
                        break;
                    }
                    chPoint = PointCoeff(fabsf(Sub(rh, static_cast<float>(yh))));
                }
                const T* prow = pg + h * rowGo + c;
                float rw = rwStart;
                for (int32_t w = wStart; w < g.wout; ++w, rw = BwdSrc(g.scaleW, w, g.align)) {
                    float cwTap[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    float cwPoint = 0.0f;
                    long long fw = 0;
                    if (borderW) {
                        fw = static_cast<long long>(floorf(rw));
                        if (yw == 0 && fw > 1 && g.win > 1) {
                            break;
                        }
                        TapCoeff(Sub(rw, static_cast<float>(fw)), cwTap);
                    } else {
                        if (!(rw < Add(static_cast<float>(yw), 2.0f))) {
                            break;
                        }
                        cwPoint = PointCoeff(fabsf(Sub(rw, static_cast<float>(yw))));
                    }
                    const float gv = DType<T>::Load(prow + static_cast<int64_t>(w) * g.chan);
                    if (!borderH && !borderW) {
                        add = Add(add, Mul(Mul(gv, chPoint), cwPoint));
                    } else if (!borderH) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (ClampIdx(fw - 1 + j, g.win - 1) == yw) {
                                add = Add(add, Mul(Mul(gv, chPoint), cwTap[j]));
                            }
                        }
                    } else if (!borderW) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (ClampIdx(fh - 1 + i, g.hin - 1) == yh) {
                                add = Add(add, Mul(Mul(gv, chTap[i]), cwPoint));
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (ClampIdx(fh - 1 + i, g.hin - 1) == yh && ClampIdx(fw - 1 + j, g.win - 1) == yw) {
                                    add = Add(add, Mul(Mul(gv, chTap[i]), cwTap[j]));
                                }
                            }
                        }
                    }
                }
            }
            po[t] = DType<T>::FromF(add);
        }
    }
}

dim3 RowGrid(int64_t rows, int64_t inner)
{
    const int64_t gx = std::min<int64_t>(std::max<int64_t>(CeilDiv(inner, kThreads), 1), 64);
    const int64_t cap = std::max<int64_t>(static_cast<int64_t>(NumSMs()) * 16 / gx, 1);
    const int64_t gy = std::min<int64_t>(std::max<int64_t>(rows, 1), std::min<int64_t>(cap, 65535));
    return dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy), 1);
}

} // namespace

cudaError_t Bicubic2dFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, float scaleH, float scaleW,
                         bool halfPixel, int32_t schedule, cudaStream_t s)
{
    const bool nhwc = lay == kNHWC;
    BicubicGeom g;
    g.rows = (nhwc ? sh.n : sh.n * sh.c) * sh.hout;
    g.hin = sh.hin;
    g.win = sh.win;
    g.hout = sh.hout;
    g.wout = sh.wout;
    g.chan = nhwc ? static_cast<int32_t>(sh.c) : 1;
    g.scaleH = scaleH;
    g.scaleW = scaleW;
    g.invH = g.invW = 0.0f;
    g.align = halfPixel ? 0 : 1;
    g.schedule = schedule;
    const dim3 grid = RowGrid(g.rows, static_cast<int64_t>(g.wout) * g.chan);
    OPSCV_DISPATCH_DT(dt, T, {
        if (nhwc) {
            Bicubic2dFwdKernel<T, true><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(y), g);
        } else {
            Bicubic2dFwdKernel<T, false><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(y), g);
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t Bicubic2dBwd(Dt dt, Layout lay, const void* go, void* gi, Shape4 sh, float scaleH, float scaleW,
                         float invH, float invW, bool align, cudaStream_t s)
{
    const bool nhwc = lay == kNHWC;
    BicubicGeom g;
    g.rows = (nhwc ? sh.n : sh.n * sh.c) * sh.hin;
    g.hin = sh.hin;
    g.win = sh.win;
    g.hout = sh.hout;
    g.wout = sh.wout;
    g.chan = nhwc ? static_cast<int32_t>(sh.c) : 1;
    g.scaleH = scaleH;
    g.scaleW = scaleW;
    g.invH = invH;
    g.invW = invW;
    g.align = align ? 1 : 0;
    g.schedule = 0;
    const dim3 grid = RowGrid(g.rows, static_cast<int64_t>(g.win) * g.chan);
    OPSCV_DISPATCH_DT(dt, T, {
        if (nhwc) {
            Bicubic2dBwdKernel<T, true><<<grid, kThreads, 0, s>>>(static_cast<const T*>(go), static_cast<T*>(gi), g);
        } else {
            Bicubic2dBwdKernel<T, false><<<grid, kThreads, 0, s>>>(static_cast<const T*>(go), static_cast<T*>(gi), g);
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
