// UpsampleTrilinear3d forward and UpsampleTrilinear3dBackward on NCDHW and NDHWC tensors.
//
// Forward: the arithmetic of the reference's SIMT kernel
// (image/resize_upsample_trilinear/op_kernel/arch35/resize_upsample_trilinear_simt_base_common.h:47-188). Per axis
// the source coordinate is fmaf(dst + 0.5, scale, -0.5) clamped at 0 (fmaf(dst, scale, 0) with align_corners), the
// taps are i0 = min(int(real), in - 1), i1 = min(i0 + 1, in - 1) with weights w1 = clamp(real - i0, 0, 1),
// w0 = 1 - w1, and the value is wD0 * (wH0 * (wW0 * v000 + wW1 * v001) + wH1 * (...)) + wD1 * (...) in separate
// multiplies and adds. A tap that holds Inf or NaN under a zero weight makes the output NaN. When only one axis is
// resampled (the other two scales are exactly 1.0f) the reference runs a two-tap loop, fmaf(w0, v0, w1 * v1), in
// which any Inf / NaN tap gives NaN (resize_upsample_trilinear_simt_base.h:30-60); equal extents are a copy.
// A thread row of a block walks output rows (plane, d, h) and finds the D and H taps of each once; each thread keeps
// the W taps of its pack of adjacent outputs for all the rows it visits.
//
// Backward: the reference runs three separable fp32 stages, W then H then D, each a product with a matrix of the
// per-axis weights (image/upsample_trilinear3d_backward/op_kernel/upsample_trilinear3d_backward.h:141-163,
// :205-263; 16-bit tensors are cast to fp32 around it). Here one gather kernel evaluates the same nesting for
// every grad_input element: sum over a of wD * (sum over b of wH * (sum over e of wW * g[a, b, e])), ascending
// grad_output index in each sum, fp32 throughout, rounded once. The weights of each grad_input index (one list per
// axis, zero padded to the longest) are built on the device by BuildTrilinearBwdTables.
#include <algorithm>

#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

struct Tap {
    int32_t i0, i1;
    float w0, w1;
};

__device__ __forceinline__ Tap FwdTap(float scale, int32_t dst, int32_t align, int32_t in)
{
    float real;
    if (align) {
        real = __fmaf_rn(static_cast<float>(dst), scale, 0.0f);
    } else {
        real = __fmaf_rn(Add(static_cast<float>(dst), 0.5f), scale, -0.5f);
        real = real < 0.0f ? 0.0f : real;
    }
    Tap t;
    const long long i = static_cast<long long>(real);
    const long long last = in - 1;
    t.i0 = static_cast<int32_t>(i < last ? i : last);
    t.i1 = t.i0 + 1 < in ? t.i0 + 1 : in - 1;
    t.w1 = fminf(fmaxf(Sub(real, static_cast<float>(t.i0)), 0.0f), 1.0f);
    t.w0 = Sub(1.0f, t.w1);
    return t;
}

// Inf or NaN: all exponent bits set.
__device__ __forceinline__ bool Special(float v) { return (__float_as_uint(v) & 0x7f800000u) == 0x7f800000u; }

__device__ __forceinline__ bool ZeroSpecial(float v, float wd, float wh, float ww)
{
    return (wd == 0.0f || wh == 0.0f || ww == 0.0f) && Special(v);
}

__device__ __forceinline__ float Plane(float wh0, float wh1, float ww0, float ww1, float v00, float v01, float v10,
                                       float v11)
{
    return Add(Mul(wh0, Add(Mul(ww0, v00), Mul(ww1, v01))), Mul(wh1, Add(Mul(ww0, v10), Mul(ww1, v11))));
}

// MODE: 0 full, 1 D only, 2 H only, 3 W only, 4 copy.
template <typename T, int V, bool CHANNELS_LAST, int MODE>
__global__ void __launch_bounds__(kThreads) Trilinear3dFwdKernel(const T* __restrict__ x, T* __restrict__ y,
                                                                 Trilinear3dGeom g)
{
    const int64_t inner = static_cast<int64_t>(g.wo) * g.chan; // elements of an output row
    const int64_t rowIn = static_cast<int64_t>(g.wi) * g.chan;
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (t0 >= inner) {
        return;
    }
    const bool small = g.rows <= 0x7fffffffLL;
    // W taps of this thread's pack (the same for every row). Channels-last packs are V channels of one pixel.
    constexpr int NW = CHANNELS_LAST ? 1 : V;
    int32_t o0[NW], o1[NW];
    float ww0[NW], ww1[NW];
    bool colZero = false; // some W weight of the pack is zero: the zero-weight test below has to look at the taps
    {
        const int32_t wFirst = CHANNELS_LAST ? static_cast<int32_t>(t0 / g.chan) : static_cast<int32_t>(t0);
        const int32_t cOff = CHANNELS_LAST ? static_cast<int32_t>(t0 - static_cast<int64_t>(wFirst) * g.chan) : 0;
#pragma unroll
        for (int v = 0; v < NW; ++v) {
            Tap t;
            if (MODE == 0 || MODE == 3) {
                t = FwdTap(g.sw, wFirst + v, g.align, g.wi);
            } else {
                t.i0 = t.i1 = wFirst + v;
                t.w0 = 1.0f;
                t.w1 = 0.0f;
            }
            o0[v] = t.i0 * g.chan + cOff;
            o1[v] = t.i1 * g.chan + cOff;
            ww0[v] = t.w0;
            ww1[v] = t.w1;
            colZero = colZero || t.w0 == 0.0f || t.w1 == 0.0f;
        }
    }
    const float nan = __int_as_float(0x7fc00000);
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < g.rows; row += rowStep) {
        int64_t plane; // row = (plane, d, h)
        int32_t d, h;
        SplitRow(row, g.ho, g.dout, small, plane, d, h);
        Tap td, th;
        if (MODE == 0 || MODE == 1) {
            td = FwdTap(g.sd, d, g.align, g.di);
        } else {
            td.i0 = td.i1 = d;
            td.w0 = 1.0f;
            td.w1 = 0.0f;
        }
        if (MODE == 0 || MODE == 2) {
            th = FwdTap(g.sh, h, g.align, g.hi);
        } else {
            th.i0 = th.i1 = h;
            th.w0 = 1.0f;
            th.w1 = 0.0f;
        }
        const bool anyZero = colZero || td.w0 == 0.0f || td.w1 == 0.0f || th.w0 == 0.0f || th.w1 == 0.0f;
        const T* p00 = x + ((plane * g.di + td.i0) * g.hi + th.i0) * rowIn;
        const T* p01 = x + ((plane * g.di + td.i0) * g.hi + th.i1) * rowIn;
        const T* p10 = x + ((plane * g.di + td.i1) * g.hi + th.i0) * rowIn;
        const T* p11 = x + ((plane * g.di + td.i1) * g.hi + th.i1) * rowIn;
        float out[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int k = CHANNELS_LAST ? 0 : v;
            const int e = CHANNELS_LAST ? v : 0; // channel offset inside a channels-last pack
            if (MODE == 4) {
                out[v] = DType<T>::Load(p00 + o0[k] + e);
            } else if (MODE == 1) {
                const float v0 = DType<T>::Load(p00 + o0[k] + e), v1 = DType<T>::Load(p10 + o0[k] + e);
                out[v] = (Special(v0) || Special(v1)) ? nan : __fmaf_rn(td.w0, v0, Mul(td.w1, v1));
            } else if (MODE == 2) {
                const float v0 = DType<T>::Load(p00 + o0[k] + e), v1 = DType<T>::Load(p01 + o0[k] + e);
                out[v] = (Special(v0) || Special(v1)) ? nan : __fmaf_rn(th.w0, v0, Mul(th.w1, v1));
            } else if (MODE == 3) {
                const float v0 = DType<T>::Load(p00 + o0[k] + e), v1 = DType<T>::Load(p00 + o1[k] + e);
                out[v] = (Special(v0) || Special(v1)) ? nan : __fmaf_rn(ww0[k], v0, Mul(ww1[k], v1));
            } else {
                const float v000 = DType<T>::Load(p00 + o0[k] + e), v001 = DType<T>::Load(p00 + o1[k] + e);
                const float v010 = DType<T>::Load(p01 + o0[k] + e), v011 = DType<T>::Load(p01 + o1[k] + e);
                const float v100 = DType<T>::Load(p10 + o0[k] + e), v101 = DType<T>::Load(p10 + o1[k] + e);
                const float v110 = DType<T>::Load(p11 + o0[k] + e), v111 = DType<T>::Load(p11 + o1[k] + e);
                bool bad = false;
                if (anyZero) { // no weight is zero for most rows and packs: nothing to test then
                    bad = ZeroSpecial(v000, td.w0, th.w0, ww0[k]) || ZeroSpecial(v001, td.w0, th.w0, ww1[k]) ||
                          ZeroSpecial(v010, td.w0, th.w1, ww0[k]) || ZeroSpecial(v011, td.w0, th.w1, ww1[k]) ||
                          ZeroSpecial(v100, td.w1, th.w0, ww0[k]) || ZeroSpecial(v101, td.w1, th.w0, ww1[k]) ||
                          ZeroSpecial(v110, td.w1, th.w1, ww0[k]) || ZeroSpecial(v111, td.w1, th.w1, ww1[k]);
                }
                const float lo = Plane(th.w0, th.w1, ww0[k], ww1[k], v000, v001, v010, v011);
                const float hi = Plane(th.w0, th.w1, ww0[k], ww1[k], v100, v101, v110, v111);
                out[v] = bad ? nan : Add(Mul(td.w0, lo), Mul(td.w1, hi));
            }
        }
        StorePack<T, V>(y + row * inner + t0, out);
    }
}

// ---- backward ----------------------------------------------------------------------------------------------
__device__ __forceinline__ Tap BwdTap(float scale, int32_t dst, int32_t align, int32_t in)
{
    float real;
    if (align) {
        real = Mul(scale, static_cast<float>(dst));
    } else {
        real = fmaxf(Sub(Mul(scale, Add(static_cast<float>(dst), 0.5f)), 0.5f), 0.0f);
    }
    Tap t;
    const long long i = static_cast<long long>(real);
    const long long last = in - 1;
    t.i0 = static_cast<int32_t>(i < last ? i : last);
    t.w1 = fminf(fmaxf(Sub(real, static_cast<float>(t.i0)), 0.0f), 1.0f);
    t.i1 = t.i0 + 1 < in ? t.i0 + 1 : in - 1;
    t.w0 = t.i0 == t.i1 ? 1.0f : Sub(1.0f, t.w1);
    return t;
}

// First grad_output index whose lower tap is at least `key` (the lower tap never decreases along the axis).
__device__ __forceinline__ int32_t FirstWithLowerTap(float scale, int32_t align, int32_t in, int32_t out, int32_t key)
{
    int32_t lo = 0, hi = out;
    while (lo < hi) {
        const int32_t mid = lo + (hi - lo) / 2;
        if (BwdTap(scale, mid, align, in).i0 >= key) {
            hi = mid;
        } else {
            lo = mid + 1;
        }
    }
    return lo;
}

// blockIdx.y = axis (0 D, 1 H, 2 W); one thread per grad_input index of that axis.
__global__ void TrilinearBwdTableKernel(TrilinearBwdTables t, Trilinear3dGeom g)
{
    const int axis = blockIdx.y;
    const int32_t in = axis == 0 ? g.di : (axis == 1 ? g.hi : g.wi);
    const int32_t out = axis == 0 ? g.dout : (axis == 1 ? g.ho : g.wo);
    const float scale = axis == 0 ? g.sd : (axis == 1 ? g.sh : g.sw);
    const int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= in) {
        return;
    }
    const int32_t taps = t.taps[axis];
    const int32_t first = FirstWithLowerTap(scale, g.align, in, out, i - 1);
    const int32_t end = FirstWithLowerTap(scale, g.align, in, out, i + 1);
    int32_t count = end - first;
    count = count < taps ? count : taps;
    t.start[axis][i] = first;
    t.count[axis][i] = count;
    float* w = t.w[axis] + static_cast<int64_t>(i) * taps;
    for (int32_t k = 0; k < taps; ++k) {
        float v = 0.0f;
        if (k < count) {
            const Tap tp = BwdTap(scale, first + k, g.align, in);
            v = tp.i0 == i ? tp.w0 : tp.w1;
        }
        w[k] = v;
    }
}

// KW > 0: the W weight list of every grad_input column has at most KW entries and is kept in registers (zero padded,
// so the padding adds nothing and is never read from grad_output); KW == 0: read through the table. KH > 0: the H
// list has at most KH entries and the loop over it is unrolled, so that the loads of a whole (depth) slab of taps
// are in flight together.
template <typename T, int KW, int KH>
__global__ void __launch_bounds__(kThreads) Trilinear3dBwdKernel(const T* __restrict__ go, T* __restrict__ gi,
                                                                 Trilinear3dGeom g, TrilinearBwdTables t)
{
    const int64_t inner = static_cast<int64_t>(g.wi) * g.chan; // elements of a grad_input row
    const int64_t rowGo = static_cast<int64_t>(g.wo) * g.chan;
    const int64_t e0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e0 >= inner) {
        return;
    }
    const bool small = g.rows <= 0x7fffffffLL;
    const int32_t w = static_cast<int32_t>(e0 / g.chan);
    const int32_t c = static_cast<int32_t>(e0 - static_cast<int64_t>(w) * g.chan);
    const int32_t ws = __ldg(t.start[2] + w), wc = __ldg(t.count[2] + w);
    const float* __restrict__ ww = t.w[2] + static_cast<int64_t>(w) * t.taps[2];
    float wr[KW > 0 ? KW : 1];
#pragma unroll
    for (int e = 0; e < KW; ++e) {
        wr[e] = e < t.taps[2] ? __ldg(ww + e) : 0.0f;
    }
    const int64_t colOff = static_cast<int64_t>(ws) * g.chan + c;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < g.rows; row += rowStep) {
        int64_t plane; // row = (plane, d, h) of grad_input
        int32_t d, h;
        SplitRow(row, g.hi, g.di, small, plane, d, h);
        const int32_t ds = __ldg(t.start[0] + d), dc = __ldg(t.count[0] + d);
        const int32_t hs = __ldg(t.start[1] + h), hc = __ldg(t.count[1] + h);
        const float* __restrict__ wd = t.w[0] + static_cast<int64_t>(d) * t.taps[0];
        const float* __restrict__ wh = t.w[1] + static_cast<int64_t>(h) * t.taps[1];
        float accD = 0.0f;
        for (int32_t a = 0; a < dc; ++a) {
            float accH = 0.0f;
            const T* pa = go + ((plane * g.dout + ds + a) * g.ho + hs) * rowGo + colOff;
            if constexpr (KW > 0 && KH > 0) {
                float gv[KH][KW];
#pragma unroll
                for (int b = 0; b < KH; ++b) {
#pragma unroll
                    for (int e = 0; e < KW; ++e) {
                        gv[b][e] = (b < hc && e < wc) ? DType<T>::Load(pa + b * rowGo + static_cast<int64_t>(e) * g.chan) : 0.0f;
                    }
                }
#pragma unroll
                for (int b = 0; b < KH; ++b) {
                    if (b < hc) {
                        float accW = 0.0f;
#pragma unroll
                        for (int e = 0; e < KW; ++e) {
                            if (e < wc) {
                                accW = Add(accW, Mul(wr[e], gv[b][e]));
                            }
                        }
                        accH = Add(accH, Mul(__ldg(wh + b), accW));
                    }
                }
            } else {
                for (int32_t b = 0; b < hc; ++b) {
                    const T* pr = pa + b * rowGo;
                    float accW = 0.0f;
                    if (KW > 0) {
#pragma unroll
                        for (int e = 0; e < KW; ++e) {
                            if (e < wc) {
                                accW = Add(accW, Mul(wr[e], DType<T>::Load(pr + static_cast<int64_t>(e) * g.chan)));
                            }
                        }
                    } else {
                        for (int32_t e = 0; e < wc; ++e) {
                            accW = Add(accW, Mul(__ldg(ww + e), DType<T>::Load(pr + static_cast<int64_t>(e) * g.chan)));
                        }
                    }
                    accH = Add(accH, Mul(__ldg(wh + b), accW));
                }
            }
            accD = Add(accD, Mul(__ldg(wd + a), accH));
        }
        gi[row * inner + e0] = DType<T>::FromF(accD);
    }
}

template <typename T, int V, bool CL>
void LaunchFwd(const T* x, T* y, const Trilinear3dGeom& g, const RowLaunch& rl, cudaStream_t s)
{
    switch (g.loop) {
        case 1: Trilinear3dFwdKernel<T, V, CL, 1><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
        case 2: Trilinear3dFwdKernel<T, V, CL, 2><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
        case 3: Trilinear3dFwdKernel<T, V, CL, 3><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
        case 4: Trilinear3dFwdKernel<T, V, CL, 4><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
        default: Trilinear3dFwdKernel<T, V, CL, 0><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
    }
}

} // namespace

cudaError_t Trilinear3dFwd(Dt dt, const void* x, void* y, Trilinear3dGeom g, cudaStream_t s)
{
    const int64_t inner = static_cast<int64_t>(g.wo) * g.chan;
    const int es = DtSize(dt);
    const bool cl = g.chan > 1;
    // pack width: at most 16 bytes of outputs; channels-last packs stay inside one pixel. The taps are read one
    // element at a time, so only the output needs the alignment.
    int v = 16 / es;
    while (v > 1 && (inner % v != 0 || (cl && g.chan % v != 0) || !Aligned(y, static_cast<size_t>(v) * es))) {
        v >>= 1;
    }
    const RowLaunch rl = RowTiling(g.rows, CeilDiv(inner, v), kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        const T* px = static_cast<const T*>(x);
        T* py = static_cast<T*>(y);
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                if (cl) {
                    LaunchFwd<T, V, true>(px, py, g, rl, s);
                } else {
                    LaunchFwd<T, V, false>(px, py, g, rl, s);
                }
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BuildTrilinearBwdTables(TrilinearBwdTables t, Trilinear3dGeom g, cudaStream_t s)
{
    const int32_t longest = std::max(g.di, std::max(g.hi, g.wi));
    const dim3 grid(static_cast<unsigned>(CeilDiv(static_cast<int64_t>(longest), 128)), 3, 1);
    TrilinearBwdTableKernel<<<grid, 128, 0, s>>>(t, g);
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t Trilinear3dBwd(Dt dt, const void* go, void* gi, Trilinear3dGeom g, TrilinearBwdTables t, cudaStream_t s)
{
    const int64_t inner = static_cast<int64_t>(g.wi) * g.chan;
    const RowLaunch rl = RowTiling(g.rows, inner, kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        const T* pg = static_cast<const T*>(go);
        T* pi = static_cast<T*>(gi);
        if (t.taps[2] <= 4 && t.taps[1] <= 4) {
            Trilinear3dBwdKernel<T, 4, 4><<<rl.grid, rl.block, 0, s>>>(pg, pi, g, t);
        } else if (t.taps[2] <= 4) {
            Trilinear3dBwdKernel<T, 4, 0><<<rl.grid, rl.block, 0, s>>>(pg, pi, g, t);
        } else if (t.taps[2] <= 8) {
            Trilinear3dBwdKernel<T, 8, 0><<<rl.grid, rl.block, 0, s>>>(pg, pi, g, t);
        } else {
            Trilinear3dBwdKernel<T, 0, 0><<<rl.grid, rl.block, 0, s>>>(pg, pi, g, t);
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
