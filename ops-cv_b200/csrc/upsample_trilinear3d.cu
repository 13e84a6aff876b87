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
// The three axes are resampled one after the other, which is the nesting of the reference's expression: a W stage
// writes a(plane, d_in, h_in, w_out) = wW0 * v0 + wW1 * v1 in fp32 to the workspace, and an H + D stage blends
// four rows of it, wD0 * (wH0 * a00 + wH1 * a01) + wD1 * (wH0 * a10 + wH1 * a11), with 16-byte loads. The same
// multiplies and adds in the same order as the reference's single expression, so the bits are the same; a zero
// weight on an Inf or NaN tap gives NaN through the IEEE product itself, which is what the reference's explicit test
// returns. The one-axis loops and the copy run in one kernel (two taps, explicit Inf / NaN test).
//
// Backward: the reference runs three separable fp32 stages, W then H then D, each a product with a matrix of the
// per-axis weights (image/upsample_trilinear3d_backward/op_kernel/upsample_trilinear3d_backward.h:141-163,
// :205-263; 16-bit tensors are cast to fp32 around it). Here each stage is one launch of a gather kernel,
// out(o, i, j) = sum over k of w[i][k] * in(o, start[i] + k, j), in ascending grad_output order, with fp32
// intermediates in the workspace and one rounding at the end. The weights of each grad_input index (one list per
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
    const int32_t i = __float2int_rz(real); // real >= 0; saturates at INT32_MAX, above every valid index
    t.i0 = i < in - 1 ? i : in - 1;
    t.i1 = t.i0 + 1 < in ? t.i0 + 1 : in - 1;
    t.w1 = fminf(fmaxf(Sub(real, static_cast<float>(t.i0)), 0.0f), 1.0f);
    t.w0 = Sub(1.0f, t.w1);
    return t;
}

// Inf or NaN: all exponent bits set.
__device__ __forceinline__ bool Special(float v) { return (__float_as_uint(v) & 0x7f800000u) == 0x7f800000u; }

// One-axis loops and the copy. MODE: 1 D only, 2 H only, 3 W only, 4 copy.
template <typename T, int V, bool CHANNELS_LAST, int MODE>
__global__ void __launch_bounds__(kThreads) Trilinear3dAxisKernel(const T* __restrict__ x, T* __restrict__ y,
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
    {
        const int32_t wFirst = CHANNELS_LAST ? static_cast<int32_t>(t0 / g.chan) : static_cast<int32_t>(t0);
        const int32_t cOff = CHANNELS_LAST ? static_cast<int32_t>(t0 - static_cast<int64_t>(wFirst) * g.chan) : 0;
#pragma unroll
        for (int v = 0; v < NW; ++v) {
            Tap t;
            if (MODE == 3) {
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
        }
    }
    const float nan = __int_as_float(0x7fc00000);
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < g.rows; row += rowStep) {
        int64_t plane; // row = (plane, d, h)
        int32_t d, h;
        SplitRow(row, g.ho, g.dout, small, plane, d, h);
        Tap td, th;
        if (MODE == 1) {
            td = FwdTap(g.sd, d, g.align, g.di);
        } else {
            td.i0 = td.i1 = d;
            td.w0 = 1.0f;
            td.w1 = 0.0f;
        }
        if (MODE == 2) {
            th = FwdTap(g.sh, h, g.align, g.hi);
        } else {
            th.i0 = th.i1 = h;
            th.w0 = 1.0f;
            th.w1 = 0.0f;
        }
        const T* p00 = x + ((plane * g.di + td.i0) * g.hi + th.i0) * rowIn;
        const T* p01 = x + ((plane * g.di + td.i0) * g.hi + th.i1) * rowIn;
        const T* p10 = x + ((plane * g.di + td.i1) * g.hi + th.i0) * rowIn;
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
            }
        }
        StorePack<T, V>(y + row * inner + t0, out);
    }
}

// ---- the full (three-axis) forward in two launches -----------------------------------------------------------
// W stage: a[row][w_out] = wW0 * x[row][i0] + wW1 * x[row][i1] for every input row (plane, d_in, h_in), fp32.
template <typename T, int V, bool CHANNELS_LAST>
__global__ void __launch_bounds__(kThreads) TrilinearWStageKernel(const T* __restrict__ x, float* __restrict__ a,
                                                                  Trilinear3dGeom g, int64_t rowsIn)
{
    const int64_t inner = static_cast<int64_t>(g.wo) * g.chan;
    const int64_t rowIn = static_cast<int64_t>(g.wi) * g.chan;
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (t0 >= inner) {
        return;
    }
    constexpr int NW = CHANNELS_LAST ? 1 : V;
    int32_t o0[NW], o1[NW];
    float ww0[NW], ww1[NW];
    {
        const int32_t wFirst = CHANNELS_LAST ? static_cast<int32_t>(t0 / g.chan) : static_cast<int32_t>(t0);
        const int32_t cOff = CHANNELS_LAST ? static_cast<int32_t>(t0 - static_cast<int64_t>(wFirst) * g.chan) : 0;
#pragma unroll
        for (int v = 0; v < NW; ++v) {
            const Tap t = FwdTap(g.sw, wFirst + v, g.align, g.wi);
            o0[v] = t.i0 * g.chan + cOff;
            o1[v] = t.i1 * g.chan + cOff;
            ww0[v] = t.w0;
            ww1[v] = t.w1;
        }
    }
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rowsIn; row += rowStep) {
        const T* px = x + row * rowIn;
        float out[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int k = CHANNELS_LAST ? 0 : v;
            const int e = CHANNELS_LAST ? v : 0;
            out[v] = Add(Mul(ww0[k], DType<T>::Load(px + o0[k] + e)), Mul(ww1[k], DType<T>::Load(px + o1[k] + e)));
        }
        StorePack<float, V>(a + row * inner + t0, out);
    }
}

// H + D stage: y[plane, d, h, :] = wD0 * (wH0 * a[d0, h0, :] + wH1 * a[d0, h1, :]) + wD1 * (wH0 * a[d1, h0, :] + ...).
// A thread owns V adjacent elements of one output row position (h, w) of one plane and walks down a range of output
// depths. Its H taps never change, and the two H-blended rows (input depths d0 and d1) stay in registers: when the
// next output depth keeps its input depths they are reused, when it moves on by one the second becomes the first
// and one new row is blended. The sums are the same expressions as in the one-pass form, so the bits are the same.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads) TrilinearHDStageKernel(const float* __restrict__ a, T* __restrict__ y,
                                                                   Trilinear3dGeom g, int32_t packs, int32_t depthChunks,
                                                                   int64_t planeChunks)
{
    const int64_t inner = static_cast<int64_t>(g.wo) * g.chan;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; // (h, pack)
    if (item >= static_cast<int64_t>(g.ho) * packs) {
        return;
    }
    const int32_t h = static_cast<int32_t>(item / packs);
    const int64_t t0 = (item - static_cast<int64_t>(h) * packs) * V;
    const Tap th = FwdTap(g.sh, h, g.align, g.hi);
    const int32_t perChunk = (g.dout + depthChunks - 1) / depthChunks;
    for (int64_t pc = blockIdx.y; pc < planeChunks; pc += gridDim.y) {
        const int64_t plane = pc / depthChunks;
        const int32_t chunk = static_cast<int32_t>(pc - plane * depthChunks);
        const int32_t dBegin = chunk * perChunk;
        const int32_t dEnd = dBegin + perChunk < g.dout ? dBegin + perChunk : g.dout;
        constexpr int C = V / 4 > 0 ? V / 4 : 1; // 16-byte chunks per row
        constexpr int L = V < 4 ? V : 4;
        const float* pa = a + plane * g.di * g.hi * inner + t0;
        const int64_t off0 = th.i0 * inner, off1 = th.i1 * inner, depthStride = g.hi * inner;
        auto blend = [&](int32_t j, float (&row)[V]) {
            const float* p = pa + j * depthStride;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                float v0[L], v1[L];
                LoadPack<float, L>(p + off0 + c * L, v0);
                LoadPack<float, L>(p + off1 + c * L, v1);
#pragma unroll
                for (int v = 0; v < L; ++v) {
                    row[c * L + v] = Add(Mul(th.w0, v0[v]), Mul(th.w1, v1[v]));
                }
            }
        };
        float lo[V], hi[V];
        int32_t cur0 = -1, cur1 = -1;
        T* py = y + ((plane * g.dout + dBegin) * g.ho + h) * inner + t0;
        for (int32_t d = dBegin; d < dEnd; ++d, py += g.ho * inner) {
            const Tap td = FwdTap(g.sd, d, g.align, g.di);
            if (td.i0 != cur0) {
                if (td.i0 == cur1) {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        lo[v] = hi[v];
                    }
                } else {
                    blend(td.i0, lo);
                }
                cur0 = td.i0;
            }
            if (td.i1 != cur1) {
                if (td.i1 == cur0) {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        hi[v] = lo[v];
                    }
                } else {
                    blend(td.i1, hi);
                }
                cur1 = td.i1;
            }
            float out[V];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                out[v] = Add(Mul(td.w0, lo[v]), Mul(td.w1, hi[v]));
            }
            StorePack<T, V>(py, out);
        }
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

// One separable stage of the backward: the axis of extent nIn shrinks to nOut,
// out(o, i, j) = sum over k < count[i] of w[i * taps + k] * in(o, start[i] + k, j), j < inner, ascending k. A thread
// owns V adjacent j of one (o, i).
template <typename TI, typename TO, int V>
__global__ void __launch_bounds__(kThreads) TrilinearBwdStageKernel(const TI* __restrict__ in, TO* __restrict__ out,
                                                                    int64_t rows, int32_t nIn, int32_t nOut,
                                                                    int64_t inner, const int32_t* __restrict__ start,
                                                                    const int32_t* __restrict__ count,
                                                                    const float* __restrict__ w, int32_t taps)
{
    const int64_t j0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (j0 >= inner) {
        return;
    }
    const bool small = rows <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rows; row += rowStep) {
        int64_t o; // row = (o, i)
        int32_t i;
        if (small) {
            const uint32_t r = static_cast<uint32_t>(row), q = r / static_cast<uint32_t>(nOut);
            o = q;
            i = static_cast<int32_t>(r - q * static_cast<uint32_t>(nOut));
        } else {
            o = row / nOut;
            i = static_cast<int32_t>(row - o * nOut);
        }
        const int32_t first = __ldg(start + i), n = __ldg(count + i);
        const float* __restrict__ wi = w + static_cast<int64_t>(i) * taps;
        const TI* p = in + (o * nIn + first) * inner + j0;
        float acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            acc[v] = 0.0f;
        }
        for (int32_t k = 0; k < n; ++k) {
            float gv[V];
            LoadPack<TI, V>(p + k * inner, gv);
            const float wk = __ldg(wi + k);
#pragma unroll
            for (int v = 0; v < V; ++v) {
                acc[v] = Add(acc[v], Mul(wk, gv[v]));
            }
        }
        StorePack<TO, V>(out + row * inner + j0, acc);
    }
}

// The W stage of the backward for narrow inner extents (NCDHW: one element per column): a thread owns one
// (column, channel) of the shrunken row for all the rows it visits and keeps that column's weights in registers
// (KW > 0: at most KW of them, zero padded; KW == 0: read through the table). UNIT: chan == 1, so the taps of a
// column sit at constant offsets from its first one.
template <typename T, int KW, bool UNIT>
__global__ void __launch_bounds__(kThreads) TrilinearBwdWStageKernel(const T* __restrict__ go, float* __restrict__ out,
                                                                     int64_t rows, int32_t wo, int32_t wi, int32_t chanArg,
                                                                     const int32_t* __restrict__ start,
                                                                     const int32_t* __restrict__ count,
                                                                     const float* __restrict__ w, int32_t taps)
{
    const int32_t chan = UNIT ? 1 : chanArg;
    const int64_t inner = static_cast<int64_t>(wi) * chan;
    const int64_t rowGo = static_cast<int64_t>(wo) * chan;
    const int64_t e0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e0 >= inner) {
        return;
    }
    const int32_t col = static_cast<int32_t>(e0 / chan);
    const int32_t c = static_cast<int32_t>(e0 - static_cast<int64_t>(col) * chan);
    const int32_t first = __ldg(start + col), n = __ldg(count + col);
    const float* __restrict__ wc = w + static_cast<int64_t>(col) * taps;
    float wr[KW > 0 ? KW : 1];
#pragma unroll
    for (int e = 0; e < KW; ++e) {
        wr[e] = e < taps ? __ldg(wc + e) : 0.0f;
    }
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    const int64_t row0 = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y;
    const T* pr = go + row0 * rowGo + static_cast<int64_t>(first) * chan + c;
    float* po = out + row0 * inner + e0;
    const int64_t stepIn = rowStep * rowGo, stepOut = rowStep * inner;
    for (int64_t row = row0; row < rows; row += rowStep, pr += stepIn, po += stepOut) {
        float acc = 0.0f;
        if (KW > 0) {
#pragma unroll
            for (int e = 0; e < KW; ++e) {
                if (e < n) {
                    acc = Add(acc, Mul(wr[e], DType<T>::Load(pr + (UNIT ? e : e * chan))));
                }
            }
        } else {
            for (int32_t e = 0; e < n; ++e) {
                acc = Add(acc, Mul(__ldg(wc + e), DType<T>::Load(pr + static_cast<int64_t>(e) * chan)));
            }
        }
        *po = acc;
    }
}

template <typename T, int KW>
void LaunchBwdWStage(const T* go, float* out, int64_t rows, const Trilinear3dGeom& g, const TrilinearBwdTables& t,
                     const RowLaunch& rl, cudaStream_t s)
{
    if (g.chan == 1) {
        TrilinearBwdWStageKernel<T, KW, true><<<rl.grid, rl.block, 0, s>>>(go, out, rows, g.wo, g.wi, 1, t.start[2],
                                                                          t.count[2], t.w[2], t.taps[2]);
    } else {
        TrilinearBwdWStageKernel<T, KW, false><<<rl.grid, rl.block, 0, s>>>(go, out, rows, g.wo, g.wi, g.chan, t.start[2],
                                                                           t.count[2], t.w[2], t.taps[2]);
    }
}

template <typename TI, typename TO>
void LaunchBwdStage(const TI* in, TO* out, int64_t outer, int32_t nIn, int32_t nOut, int64_t inner, const int32_t* start,
                    const int32_t* count, const float* w, int32_t taps, cudaStream_t s)
{
    // 16 bytes of the wider type per thread where the rows keep that alignment
    int v = 16 / static_cast<int>(sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO));
    while (v > 1 && (inner % v != 0 || !Aligned(in, v * sizeof(TI)) || !Aligned(out, v * sizeof(TO)))) {
        v >>= 1;
    }
    const int64_t rows = outer * nOut;
    const RowLaunch rl = RowTiling(rows, CeilDiv(inner, v), kThreads);
    OPSCV_DISPATCH_VEC(v, V, {
        if constexpr (V <= 4) {
            TrilinearBwdStageKernel<TI, TO, V><<<rl.grid, rl.block, 0, s>>>(in, out, rows, nIn, nOut, inner, start, count,
                                                                          w, taps);
        }
    });
    CountLaunch();
}

template <typename T, int V, bool CL>
void LaunchAxis(const T* x, T* y, const Trilinear3dGeom& g, const RowLaunch& rl, cudaStream_t s)
{
    switch (g.loop) {
        case 1: Trilinear3dAxisKernel<T, V, CL, 1><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
        case 2: Trilinear3dAxisKernel<T, V, CL, 2><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
        case 3: Trilinear3dAxisKernel<T, V, CL, 3><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
        default: Trilinear3dAxisKernel<T, V, CL, 4><<<rl.grid, rl.block, 0, s>>>(x, y, g); break;
    }
}

} // namespace

uint64_t Trilinear3dFwdWorkspace(const Trilinear3dGeom& g, int64_t planes)
{
    if (g.loop != 0) {
        return 0;
    }
    return static_cast<uint64_t>(planes) * g.di * g.hi * g.wo * g.chan * sizeof(float);
}

cudaError_t Trilinear3dFwd(Dt dt, const void* x, void* y, float* stage, Trilinear3dGeom g, cudaStream_t s)
{
    const int64_t inner = static_cast<int64_t>(g.wo) * g.chan;
    const int es = DtSize(dt);
    const bool cl = g.chan > 1;
    if (g.loop == 0) {
        const int64_t rowsIn = g.rows / (static_cast<int64_t>(g.dout) * g.ho) * g.di * g.hi; // planes * di * hi
        int v = 4; // W stage: 16 bytes of the fp32 stage buffer per thread
        while (v > 1 && (inner % v != 0 || (cl && g.chan % v != 0) ||
                         !Aligned(stage, static_cast<size_t>(v) * sizeof(float)))) {
            v >>= 1;
        }
        int vh = 16 / es; // H + D stage: 16 bytes of outputs per thread, read as 16-byte chunks of the stage buffer
        while (vh > 1 && (inner % vh != 0 || !Aligned(y, static_cast<size_t>(vh) * es) ||
                          !Aligned(stage, static_cast<size_t>(vh < 4 ? vh : 4) * sizeof(float)))) {
            vh >>= 1;
        }
        const RowLaunch rw = RowTiling(rowsIn, CeilDiv(inner, v), kThreads);
        const int64_t planes = g.rows / (static_cast<int64_t>(g.dout) * g.ho);
        const int32_t packs = static_cast<int32_t>(inner / vh);
        const int64_t items = static_cast<int64_t>(g.ho) * packs;
        // enough depth chunks to fill the machine about twice over, each at least eight output depths long
        int64_t chunks = CeilDiv(static_cast<int64_t>(NumSMs()) * 4096, std::max<int64_t>(planes * items, 1));
        chunks = std::max<int64_t>(1, std::min<int64_t>(chunks, std::max<int32_t>(g.dout / 8, 1)));
        const dim3 gridH(static_cast<unsigned>(CeilDiv(items, kThreads)), static_cast<unsigned>(std::min<int64_t>(planes * chunks, 65535)), 1);
        OPSCV_DISPATCH_DT(dt, T, {
            const T* px = static_cast<const T*>(x);
            T* py = static_cast<T*>(y);
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V <= 4) {
                    if (cl) {
                        TrilinearWStageKernel<T, V, true><<<rw.grid, rw.block, 0, s>>>(px, stage, g, rowsIn);
                    } else {
                        TrilinearWStageKernel<T, V, false><<<rw.grid, rw.block, 0, s>>>(px, stage, g, rowsIn);
                    }
                }
            });
            OPSCV_DISPATCH_VEC(vh, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    TrilinearHDStageKernel<T, V><<<gridH, kThreads, 0, s>>>(stage, py, g, packs, static_cast<int32_t>(chunks),
                                                                             planes * chunks);
                }
            });
        });
        CountLaunch(2);
        return cudaGetLastError();
    }
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
                    LaunchAxis<T, V, true>(px, py, g, rl, s);
                } else {
                    LaunchAxis<T, V, false>(px, py, g, rl, s);
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

uint64_t Trilinear3dBwdWorkspace(const Trilinear3dGeom& g, int64_t planes)
{
    // after the W stage: planes * dout * ho * wi; after the H stage: planes * dout * hi * wi
    const uint64_t t1 = static_cast<uint64_t>(planes) * g.dout * g.ho * g.wi * g.chan * sizeof(float);
    const uint64_t t2 = static_cast<uint64_t>(planes) * g.dout * g.hi * g.wi * g.chan * sizeof(float);
    return ((t1 + 255) & ~static_cast<uint64_t>(255)) + t2;
}

cudaError_t Trilinear3dBwd(Dt dt, const void* go, void* gi, float* stage, Trilinear3dGeom g, TrilinearBwdTables t,
                           cudaStream_t s)
{
    const int64_t planes = g.rows / (static_cast<int64_t>(g.di) * g.hi);
    const uint64_t t1Bytes = static_cast<uint64_t>(planes) * g.dout * g.ho * g.wi * g.chan * sizeof(float);
    float* t1 = stage;
    float* t2 = reinterpret_cast<float*>(reinterpret_cast<char*>(stage) + ((t1Bytes + 255) & ~static_cast<uint64_t>(255)));
    OPSCV_DISPATCH_DT(dt, T, {
        // W: (planes * dout * ho) x wo x chan -> wi;  H: (planes * dout) x ho x (wi * chan) -> hi;  D: planes x dout x
        // (hi * wi * chan) -> di
        if (g.chan <= 4) {
            const int64_t rowsW = planes * g.dout * g.ho;
            const RowLaunch rl = RowTiling(rowsW, static_cast<int64_t>(g.wi) * g.chan, kThreads);
            const T* pg = static_cast<const T*>(go);
            if (t.taps[2] <= 4) {
                LaunchBwdWStage<T, 4>(pg, t1, rowsW, g, t, rl, s);
            } else if (t.taps[2] <= 6) {
                LaunchBwdWStage<T, 6>(pg, t1, rowsW, g, t, rl, s);
            } else if (t.taps[2] <= 10) {
                LaunchBwdWStage<T, 10>(pg, t1, rowsW, g, t, rl, s);
            } else {
                LaunchBwdWStage<T, 0>(pg, t1, rowsW, g, t, rl, s);
            }
            CountLaunch();
        } else {
            LaunchBwdStage<T, float>(static_cast<const T*>(go), t1, planes * g.dout * g.ho, g.wo, g.wi, g.chan,
                                     t.start[2], t.count[2], t.w[2], t.taps[2], s);
        }
        LaunchBwdStage<float, float>(t1, t2, planes * g.dout, g.ho, g.hi, static_cast<int64_t>(g.wi) * g.chan,
                                     t.start[1], t.count[1], t.w[1], t.taps[1], s);
        LaunchBwdStage<float, T>(t2, static_cast<T*>(gi), planes, g.dout, g.di,
                                 static_cast<int64_t>(g.hi) * g.wi * g.chan, t.start[0], t.count[0], t.w[0], t.taps[0], s);
    });
    return cudaGetLastError();
}

} // namespace opscv
