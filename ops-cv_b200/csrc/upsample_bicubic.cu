// UpsampleBicubic2d forward and backward (cubic convolution with A = -0.75, no antialiasing), NCHW and NHWC.
//
// Forward: a thread owns one or two adjacent elements of an output row and walks down a band of rows, keeping the
// four horizontal sums of the current source rows in registers; the sixteen clamped taps are combined in the
// reference's order (four row sums left to right, then the column sum), every operation rounded on its own, so
// fp32 results carry the bits of a serial CPU statement of
// image/resize_bicubic_v2/op_kernel/arch35/resize_bicubic_v2_simt_base.h:23-120. The four special schedules of
// resize_bicubic_v2_simt_nchw.h:50-90 (copy, one input pixel, one output pixel, integer positions) are selected on
// the host with the reference's rule and are plain copies here too.
//
// Backward: one thread per grad_input element gathers the grads that reach it, walking them in ascending
// (row, column) order. The walk, its start, its end and the coefficient expressions are those of the reference's
// gather kernel (image/resize_bicubic_v2_grad/op_kernel/arch35/resize_bicubic_v2_grad_simt_determine.h:95-350):
// an axis on which the element is interior is walked by distance to the source position, a first or last index
// tap by tap with clamped destinations. The sum has a fixed order, so results are reproducible from run to run
// and fp32 results carry the bits of that kernel run serially. The column side of the walk is the same for every
// row, so each thread evaluates it once into a shared-memory list.
//
// Calls at exactly 2x on NCHW tensors (scales 0.5 with half-pixel coordinates: every source coordinate is exact and
// the coefficients are a handful of constants, evaluated on the host) have kernels of their own in both directions:
// Bicubic2dFwdX2Kernel and Bicubic2dBwdX2Kernel stage a band of rows in shared memory as fp32 once and work from
// register windows; their terms, order and rounding are those of the general kernels.
#include <algorithm>
#include <vector>

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
__device__ __forceinline__ int32_t ClampIdx32(int32_t v, int32_t last) { return min(max(v, 0), last); }

struct BicubicGeom {
    int64_t rows;  // forward: planes * hout; backward: planes * hin
    int32_t hin, win, hout, wout;
    int32_t chan;  // NHWC: channels; NCHW: 1
    float scaleH, scaleW, invH, invW;
    int32_t align; // backward: align_corners; forward: !halfPixel
    int32_t schedule;
};

// Copy schedules (one input pixel, one output pixel, integer source positions): no arithmetic.
template <typename T, bool NHWC>
__global__ void __launch_bounds__(kThreads) Bicubic2dFwdCopyKernel(const T* __restrict__ x, T* __restrict__ y, BicubicGeom g)
{
    const int32_t inner = g.wout * g.chan;
    const int64_t planeIn = static_cast<int64_t>(g.hin) * g.win * g.chan;
    const int64_t rowIn = static_cast<int64_t>(g.win) * g.chan;
    for (int64_t row = blockIdx.y; row < g.rows; row += gridDim.y) {
        const int64_t plane = row / g.hout;
        const int32_t H = static_cast<int32_t>(row - plane * g.hout);
        const float oh = g.align ? Mul(static_cast<float>(H), g.scaleH)
                                 : Sub(Mul(Add(static_cast<float>(H), 0.5f), g.scaleH), 0.5f);
        const T* px = x + plane * planeIn;
        const T* r1 = px + ClampIdx(static_cast<long long>(floorf(oh)), g.hin - 1) * rowIn;
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
            const long long left = static_cast<long long>(floorf(ow));
            py[t] = r1[static_cast<int64_t>(ClampIdx(left, g.win - 1)) * g.chan + c]; // integer positions
        }
    }
}

// General schedule. A thread owns V adjacent elements of an output row (one column for NHWC: its channel of one
// pixel) and walks down a band of output rows. The four horizontal sums that an output row needs are kept in
// registers and shifted as the source row advances: an input row's horizontal sum is computed once per band and
// column instead of once per output row that uses it, and the vertical combination stays the reference's
// left-to-right sum of four products, so the bits do not change.
template <typename T, bool NHWC, int V>
__global__ void __launch_bounds__(kThreads) Bicubic2dFwdKernel(const T* __restrict__ x, T* __restrict__ y, BicubicGeom g,
                                                                int32_t bandRows, int32_t bands)
{
    // per output row of the band: the source row above the four taps and the four vertical coefficients, evaluated
    // once per band by the block instead of once per row by every thread
    extern __shared__ float sRow[];
    float* sCh = sRow;                                                   // [bandRows][4]
    int32_t* sTop = reinterpret_cast<int32_t*>(sRow + 4 * bandRows);     // [bandRows]
    const int32_t inner = g.wout * g.chan;
    const int32_t t0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const bool active = t0 < inner;
    const int64_t planeIn = static_cast<int64_t>(g.hin) * g.win * g.chan;
    const int64_t rowIn = static_cast<int64_t>(g.win) * g.chan;
    // per-column taps and weights (V columns)
    int32_t off[V][4];
    float cw[V][4];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int32_t t = active ? t0 + v : 0;
        const int32_t W = NHWC ? t / g.chan : t;
        const int32_t c = NHWC ? t - W * g.chan : 0;
        const float ow = g.align ? Mul(static_cast<float>(W), g.scaleW)
                                 : Sub(Mul(Add(static_cast<float>(W), 0.5f), g.scaleW), 0.5f);
        const float fw = floorf(ow);
        const long long left = static_cast<long long>(fw);
        FwdCoeff(Sub(ow, fw), cw[v]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            off[v][j] = ClampIdx(left - 1 + j, g.win - 1) * g.chan + c;
        }
    }
    int32_t tableBand = -1;
    for (int64_t item = blockIdx.y; item < g.rows; item += gridDim.y) { // g.rows = planes * bands here
        const int64_t plane = item / bands;
        const int32_t band = static_cast<int32_t>(item - plane * bands);
        const int32_t h0 = band * bandRows;
        const int32_t h1 = min(h0 + bandRows, g.hout);
        if (band != tableBand) { // uniform over the block
            __syncthreads();
            for (int32_t r = threadIdx.x; r < h1 - h0; r += blockDim.x) {
                const int32_t H = h0 + r;
                const float oh = g.align ? Mul(static_cast<float>(H), g.scaleH)
                                         : Sub(Mul(Add(static_cast<float>(H), 0.5f), g.scaleH), 0.5f);
                const float fh = floorf(oh);
                float ch[4];
                FwdCoeff(Sub(oh, fh), ch);
                // tops outside [-2, hin + 1] clamp every tap to the same row as the bound does
                const float lim = fminf(fmaxf(fh, -2.0f), static_cast<float>(g.hin) + 1.0f);
                sTop[r] = static_cast<int32_t>(lim);
                sCh[4 * r + 0] = ch[0];
                sCh[4 * r + 1] = ch[1];
                sCh[4 * r + 2] = ch[2];
                sCh[4 * r + 3] = ch[3];
            }
            __syncthreads();
            tableBand = band;
        }
        if (!active) {
            continue;
        }
        const T* px = x + plane * planeIn;
        T* py = y + (plane * g.hout + h0) * static_cast<int64_t>(inner) + t0;
        float rs[V][4];
        int32_t curTop = 0;
        bool have = false;
        auto rowSums = [&](int32_t srcRow, int slot) {
            const T* r = px + ClampIdx32(srcRow, g.hin - 1) * rowIn;
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float v0 = DType<T>::Load(r + off[v][0]), v1 = DType<T>::Load(r + off[v][1]),
                            v2 = DType<T>::Load(r + off[v][2]), v3 = DType<T>::Load(r + off[v][3]);
                rs[v][slot] = Add(Add(Add(Mul(v0, cw[v][0]), Mul(v1, cw[v][1])), Mul(v2, cw[v][2])), Mul(v3, cw[v][3]));
            }
        };
        for (int32_t r = 0; r < h1 - h0; ++r, py += inner) {
            const int32_t top = sTop[r];
            const float4 ch = *reinterpret_cast<const float4*>(sCh + 4 * r);
            const int32_t shift = top - curTop;
            if (!have || shift < 0 || shift >= 4) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    rowSums(top - 1 + k, k);
                }
                have = true;
            } else {
                for (int32_t sft = 0; sft < shift; ++sft) {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        rs[v][0] = rs[v][1];
                        rs[v][1] = rs[v][2];
                        rs[v][2] = rs[v][3];
                    }
                    rowSums(curTop + sft + 3, 3);
                }
            }
            curTop = top;
            float out[V];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                out[v] = Add(Add(Add(Mul(rs[v][0], ch.x), Mul(rs[v][1], ch.y)), Mul(rs[v][2], ch.z)), Mul(rs[v][3], ch.w));
            }
            StorePack<T, V>(py, out);
        }
    }
}

// General schedule, NCHW, tiled through shared memory. A block takes a (plane, band of output rows) item: it loads
// the source rows the band touches once (converted to fp32), forms every horizontal sum of those rows once,
// a[source row][output column], and then combines four rows of `a` per output row with 16-byte shared-memory loads.
// The sums are the expressions of the kernel above in the same order, so the bits are the same; what changes is
// that a tap is loaded and converted once per block instead of once per output column that uses it, and that the
// column coefficients live in registers for all the rows of the tile.
struct BicubicTile {
    int32_t bandRows; // output rows per item
    int32_t bands;
    int32_t maxSrc;   // most source rows any band touches
    int32_t tw;       // threads along a row in the horizontal pass (power of two)
    int32_t pw;       // threads along a row in the vertical pass (power of two)
};

__host__ __device__ __forceinline__ int32_t FwdTop(int32_t H, float scaleH, int32_t align, int32_t hin, float (*ch)[4])
{
#ifdef __CUDA_ARCH__
    const float oh = align ? Mul(static_cast<float>(H), scaleH) : Sub(Mul(Add(static_cast<float>(H), 0.5f), scaleH), 0.5f);
    const float fh = floorf(oh);
    if (ch != nullptr) {
        FwdCoeff(Sub(oh, fh), *ch);
    }
#else
    (void)ch;
    float oh;
    if (align) {
        oh = static_cast<float>(H) * scaleH;
    } else {
        const float t = (static_cast<float>(H) + 0.5f) * scaleH;
        oh = t - 0.5f;
    }
    const float fh = floorf(oh);
#endif
    // tops outside [-2, hin + 1] clamp every tap to the same row as the bound does
    return static_cast<int32_t>(fminf(fmaxf(fh, -2.0f), static_cast<float>(hin) + 1.0f));
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads) Bicubic2dFwdTileKernel(const T* __restrict__ x, T* __restrict__ y, BicubicGeom g,
                                                                   BicubicTile tile, int64_t items)
{
    extern __shared__ __align__(16) float sTile[];
    float* sCh = sTile;                                           // [bandRows][4], read as float4
    float* sA = sCh + 4 * tile.bandRows;                          // [maxSrc][wout], 16-byte aligned rows when V >= 4
    float* sX = sA + static_cast<size_t>(tile.maxSrc) * g.wout;   // [maxSrc][win]
    int32_t* sTop = reinterpret_cast<int32_t*>(sX + static_cast<size_t>(tile.maxSrc) * g.win); // [bandRows]
    const int32_t tid = threadIdx.x;
    const int32_t tx = tid & (tile.tw - 1), ty = tid / tile.tw, tyN = kThreads / tile.tw;
    const int32_t px_ = tid & (tile.pw - 1), py_ = tid / tile.pw, pyN = kThreads / tile.pw;
    const int32_t packs = g.wout / V;
    const bool pairAligned = (g.wout & 1) == 0; // rows of sums start on 8-byte boundaries
    const int64_t planeIn = static_cast<int64_t>(g.hin) * g.win;
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t plane = item / tile.bands;
        const int32_t band = static_cast<int32_t>(item - plane * tile.bands);
        const int32_t h0 = band * tile.bandRows;
        const int32_t nOut = min(tile.bandRows, g.hout - h0);
        __syncthreads(); // the previous item's tiles are no longer read
        for (int32_t r = tid; r < nOut; r += kThreads) {
            float ch[4];
            sTop[r] = FwdTop(h0 + r, g.scaleH, g.align, g.hin, &ch);
            *reinterpret_cast<float4*>(sCh + 4 * r) = make_float4(ch[0], ch[1], ch[2], ch[3]);
        }
        __syncthreads();
        const int32_t srcLo = ClampIdx32(sTop[0] - 1, g.hin - 1);
        const int32_t srcHi = ClampIdx32(sTop[nOut - 1] + 2, g.hin - 1);
        const int32_t nSrc = min(srcHi - srcLo + 1, tile.maxSrc);
        const T* px = x + plane * planeIn + static_cast<int64_t>(srcLo) * g.win;
        for (int32_t i = tid; i < nSrc * g.win; i += kThreads) {
            sX[i] = DType<T>::Load(px + i);
        }
        __syncthreads();
        // horizontal sums: a thread keeps the taps and coefficients of two adjacent columns for all the rows of the
        // tile. When the second column's window is the first one's moved on by zero or one source pixel (any
        // up-scale) the two sums share their tap reads: five shared-memory loads instead of eight.
        for (int32_t w = 2 * tx; w < g.wout; w += 2 * tile.tw) {
            float cw0[4], cw1[4];
            long long left0, left1;
            {
                const float ow = g.align ? Mul(static_cast<float>(w), g.scaleW)
                                         : Sub(Mul(Add(static_cast<float>(w), 0.5f), g.scaleW), 0.5f);
                const float fw = floorf(ow);
                left0 = static_cast<long long>(fw);
                FwdCoeff(Sub(ow, fw), cw0);
            }
            const bool two = w + 1 < g.wout;
            {
                const float ow = g.align ? Mul(static_cast<float>(w + 1), g.scaleW)
                                         : Sub(Mul(Add(static_cast<float>(w + 1), 0.5f), g.scaleW), 0.5f);
                const float fw = floorf(ow);
                left1 = static_cast<long long>(fw);
                FwdCoeff(Sub(ow, fw), cw1);
            }
            const int32_t o0 = ClampIdx(left0 - 1, g.win - 1), o1 = ClampIdx(left0, g.win - 1),
                          o2 = ClampIdx(left0 + 1, g.win - 1), o3 = ClampIdx(left0 + 2, g.win - 1),
                          o4 = ClampIdx(left0 + 3, g.win - 1);
            const long long step = left1 - left0;
            if (two && (step == 0 || step == 1)) {
                for (int32_t r = ty; r < nSrc; r += tyN) {
                    const float* row = sX + r * g.win;
                    const float v0 = row[o0], v1 = row[o1], v2 = row[o2], v3 = row[o3];
                    const float v4 = step == 1 ? row[o4] : 0.0f;
                    const float u0 = step == 1 ? v1 : v0, u1 = step == 1 ? v2 : v1, u2 = step == 1 ? v3 : v2,
                                u3 = step == 1 ? v4 : v3;
                    float2 a;
                    a.x = Add(Add(Add(Mul(v0, cw0[0]), Mul(v1, cw0[1])), Mul(v2, cw0[2])), Mul(v3, cw0[3]));
                    a.y = Add(Add(Add(Mul(u0, cw1[0]), Mul(u1, cw1[1])), Mul(u2, cw1[2])), Mul(u3, cw1[3]));
                    if (pairAligned) {
                        *reinterpret_cast<float2*>(sA + r * g.wout + w) = a;
                    } else {
                        sA[r * g.wout + w] = a.x;
                        sA[r * g.wout + w + 1] = a.y;
                    }
                }
            } else {
                const int32_t q0 = ClampIdx(left1 - 1, g.win - 1), q1 = ClampIdx(left1, g.win - 1),
                              q2 = ClampIdx(left1 + 1, g.win - 1), q3 = ClampIdx(left1 + 2, g.win - 1);
                for (int32_t r = ty; r < nSrc; r += tyN) {
                    const float* row = sX + r * g.win;
                    sA[r * g.wout + w] = Add(Add(Add(Mul(row[o0], cw0[0]), Mul(row[o1], cw0[1])), Mul(row[o2], cw0[2])), Mul(row[o3], cw0[3]));
                    if (two) {
                        sA[r * g.wout + w + 1] = Add(Add(Add(Mul(row[q0], cw1[0]), Mul(row[q1], cw1[1])), Mul(row[q2], cw1[2])), Mul(row[q3], cw1[3]));
                    }
                }
            }
        }
        __syncthreads();
        // vertical combination, V adjacent outputs per thread
        T* py = y + (plane * g.hout + h0) * static_cast<int64_t>(g.wout);
        constexpr int C = V / 4 > 0 ? V / 4 : 1;
        constexpr int L = V < 4 ? V : 4;
        for (int32_t p = px_; p < packs; p += tile.pw) {
            for (int32_t r = py_; r < nOut; r += pyN) {
                const int32_t top = sTop[r];
                const float4 ch = *reinterpret_cast<const float4*>(sCh + 4 * r);
                const float* a0 = sA + (ClampIdx32(top - 1, g.hin - 1) - srcLo) * g.wout + p * V;
                const float* a1 = sA + (ClampIdx32(top, g.hin - 1) - srcLo) * g.wout + p * V;
                const float* a2 = sA + (ClampIdx32(top + 1, g.hin - 1) - srcLo) * g.wout + p * V;
                const float* a3 = sA + (ClampIdx32(top + 2, g.hin - 1) - srcLo) * g.wout + p * V;
                float out[V];
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    float r0[L], r1[L], r2[L], r3[L];
                    LoadPack<float, L>(a0 + c * L, r0);
                    LoadPack<float, L>(a1 + c * L, r1);
                    LoadPack<float, L>(a2 + c * L, r2);
                    LoadPack<float, L>(a3 + c * L, r3);
#pragma unroll
                    for (int v = 0; v < L; ++v) {
                        out[c * L + v] = Add(Add(Add(Mul(r0[v], ch.x), Mul(r1[v], ch.y)), Mul(r2[v], ch.z)), Mul(r3[v], ch.w));
                    }
                }
                StorePack<T, V>(py + static_cast<int64_t>(r) * g.wout + p * V, out);
            }
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

// One grad_input element by the reference's walk, with nothing cached: the coefficients of a column are evaluated
// again for every row. Used for elements whose column list does not fit the shared-memory lists of the kernel
// below (an extent of 1 makes every grads index a tap of the single element).
template <typename T>
__device__ float BwdElementDirect(const T* __restrict__ pg, const BicubicGeom& g, int32_t yh, int32_t yw, int32_t c,
                                  int64_t rowGo, float offset)
{
    const int32_t hStart = WalkStart(yh, g.invH, offset);
    const float rhStart = Sub(Mul(Add(static_cast<float>(hStart), offset), g.scaleH), offset);
    const bool borderH = yh == 0 || yh == g.hin - 1;
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
            fh = static_cast<long long>(floorf(rh));
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
    return add;
}

// The gather with the column side of the walk cached. A thread owns one element position of a grad_input row
// (column yw; for NHWC also its channel) and keeps it while the block moves over rows and planes. It first walks
// the grads columns once, exactly as the reference does, and stores every term it would add for one grads row as
// an entry (grads column, coefficient) in its own column of a shared-memory table: one entry per grads column for
// an interior yw, one per matching tap for a first or last yw. For each grads row h of the row walk it then has
// one coefficient (interior yh) or the matching tap coefficients in tap order (first or last yh), and adds
// (g * cH) * cW over the entries, grouped by grads column with the row taps outside the column taps. That is the
// order and the rounding of the reference's four walks, so the sum has the same bits.
// colsPB: element positions of a row that a block covers (its threads beyond that take further rows);
// borderOnly: the block's positions are those of the first and the last column only.
template <typename T, bool NHWC>
__global__ void __launch_bounds__(kThreads) Bicubic2dBwdListKernel(const T* __restrict__ go, T* __restrict__ gi, BicubicGeom g,
                                                                    int32_t maxW, int32_t colsPB, int32_t borderOnly)
{
    extern __shared__ float sList[];
    const int32_t nt = blockDim.x, tid = threadIdx.x;
    float* sCoef = sList;
    int32_t* sCol = reinterpret_cast<int32_t*>(sList + static_cast<size_t>(maxW) * nt);
    const int32_t inner = g.win * g.chan;
    const int32_t rowsPB = nt / colsPB;
    const int32_t rowLane = tid / colsPB;
    const int32_t pos = blockIdx.x * colsPB + (tid - rowLane * colsPB);
    if (rowLane >= rowsPB || pos >= (borderOnly ? 2 * g.chan : inner)) {
        return;
    }
    int32_t t = pos;
    if (borderOnly) {
        const int32_t side = NHWC ? pos / g.chan : pos;
        t = side == 0 ? pos : inner - 2 * g.chan + pos; // column 0 or column win - 1, same channel
    }
    const int32_t yw = NHWC ? t / g.chan : t;
    const int32_t c = NHWC ? t - yw * g.chan : 0;
    const int64_t planeGo = static_cast<int64_t>(g.hout) * g.wout * g.chan;
    const int64_t rowGo = static_cast<int64_t>(g.wout) * g.chan;
    const float offset = g.align ? 0.0f : 0.5f;
    const bool borderW = yw == 0 || yw == g.win - 1;

    // the column walk, once
    int32_t cnt = 0;
    bool overflow = false;
    const int32_t wStart = WalkStart(yw, g.invW, offset);
    {
        float rw = Sub(Mul(Add(static_cast<float>(wStart), offset), g.scaleW), offset);
        for (int32_t w = wStart; w < g.wout && !overflow; ++w, rw = BwdSrc(g.scaleW, w, g.align)) {
            if (borderW) {
                const long long fw = static_cast<long long>(floorf(rw));
                if (yw == 0 && fw > 1 && g.win > 1) {
                    break;
                }
                float cwTap[4];
                TapCoeff(Sub(rw, static_cast<float>(fw)), cwTap);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (ClampIdx(fw - 1 + j, g.win - 1) == yw) {
                        if (cnt < maxW) {
                            sCoef[cnt * nt + tid] = cwTap[j];
                            sCol[cnt * nt + tid] = w;
                            ++cnt;
                        } else {
                            overflow = true;
                        }
                    }
                }
            } else {
                if (!(rw < Add(static_cast<float>(yw), 2.0f))) {
                    break;
                }
                if (cnt < maxW) {
                    sCoef[cnt * nt + tid] = PointCoeff(fabsf(Sub(rw, static_cast<float>(yw))));
                    sCol[cnt * nt + tid] = w;
                    ++cnt;
                } else {
                    overflow = true;
                }
            }
        }
    }

    for (int64_t row = static_cast<int64_t>(blockIdx.y) * rowsPB + rowLane; row < g.rows;
         row += static_cast<int64_t>(gridDim.y) * rowsPB) {
        const int64_t plane = row / g.hin;
        const int32_t yh = static_cast<int32_t>(row - plane * g.hin);
        const T* pg = go + plane * planeGo;
        T* po = gi + row * inner;
        if (overflow) {
            po[t] = DType<T>::FromF(BwdElementDirect<T>(pg, g, yh, yw, c, rowGo, offset));
            continue;
        }
        const bool borderH = yh == 0 || yh == g.hin - 1;
        const int32_t hStart = WalkStart(yh, g.invH, offset);
        float rh = Sub(Mul(Add(static_cast<float>(hStart), offset), g.scaleH), offset);
        float add = 0.0f;
        for (int32_t h = hStart; h < g.hout; ++h, rh = BwdSrc(g.scaleH, h, g.align)) {
            const T* prow = pg + h * rowGo + c;
            if (!borderH) {
                if (!(rh < Add(static_cast<float>(yh), 2.0f))) {
                    break;
                }
                const float ch = PointCoeff(fabsf(Sub(rh, static_cast<float>(yh))));
                // one row coefficient: the entries in list order are already the reference's order
                for (int32_t k = 0; k < cnt; ++k) {
                    const float gv = DType<T>::Load(prow + static_cast<int64_t>(sCol[k * nt + tid]) * g.chan);
                    add = Add(add, Mul(Mul(gv, ch), sCoef[k * nt + tid]));
                }
                continue;
            }
            const long long fh = static_cast<long long>(floorf(rh));
            if (yh == 0 && fh > 1 && g.hin > 1) {
                break;
            }
            float chTap[4];
            TapCoeff(Sub(rh, static_cast<float>(fh)), chTap);
            float chv[4];
            int nH = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (ClampIdx(fh - 1 + i, g.hin - 1) == yh) {
                    // compacted in tap order without dynamic register indexing
                    chv[3] = chTap[i];
                    if (nH == 0) chv[0] = chTap[i];
                    if (nH == 1) chv[1] = chTap[i];
                    if (nH == 2) chv[2] = chTap[i];
                    ++nH;
                }
            }
            int32_t k = 0;
            while (k < cnt) {
                const int32_t w = sCol[k * nt + tid];
                int32_t k1 = k + 1;
                while (k1 < cnt && sCol[k1 * nt + tid] == w) {
                    ++k1;
                }
                const float gv = DType<T>::Load(prow + static_cast<int64_t>(w) * g.chan);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (i < nH) {
                        const float gc = Mul(gv, i == 3 ? chv[3] : (i == 2 ? chv[2] : (i == 1 ? chv[1] : chv[0])));
                        for (int32_t kk = k; kk < k1; ++kk) {
                            add = Add(add, Mul(gc, sCoef[kk * nt + tid]));
                        }
                    }
                }
                k = k1;
            }
        }
        po[t] = DType<T>::FromF(add);
    }
}

// The same gather for the interior columns (1 .. win - 2), whose walk has one coefficient per grads column and at
// most K columns (every up-scale factor up to (K - 1) / 4, and every down-scale): the list lives in registers and
// the loop over it is unrolled. The first and the last column go through the list kernel in a launch of their own.
// Terms, their order and their rounding are those of the list kernel.
template <typename T, bool NHWC, int K>
__global__ void __launch_bounds__(kThreads) Bicubic2dBwdRegKernel(const T* __restrict__ go, T* __restrict__ gi, BicubicGeom g)
{
    const int32_t inner = g.win * g.chan;
    const int32_t pos = blockIdx.x * blockDim.x + threadIdx.x;
    if (pos >= inner - 2 * g.chan) {
        return;
    }
    const int32_t t = pos + g.chan; // skip column 0
    const int32_t yw = NHWC ? t / g.chan : t;
    const int32_t c = NHWC ? t - yw * g.chan : 0;
    const int64_t planeGo = static_cast<int64_t>(g.hout) * g.wout * g.chan;
    const int64_t rowGo = static_cast<int64_t>(g.wout) * g.chan;
    const float offset = g.align ? 0.0f : 0.5f;

    float cw[K];
    int32_t cnt = 0;
    bool overflow = false;
    const int32_t wStart = WalkStart(yw, g.invW, offset);
    {
        bool done = false;
#pragma unroll
        for (int k = 0; k < K + 1; ++k) {
            const int32_t w = wStart + k;
            if (k < K) {
                cw[k] = 0.0f;
            }
            if (!done && w < g.wout) {
                const float rw = k == 0 ? Sub(Mul(Add(static_cast<float>(wStart), offset), g.scaleW), offset)
                                        : BwdSrc(g.scaleW, w, g.align);
                if (!(rw < Add(static_cast<float>(yw), 2.0f))) {
                    done = true;
                } else if (k == K) {
                    overflow = true;
                } else {
                    cw[k < K ? k : 0] = PointCoeff(fabsf(Sub(rw, static_cast<float>(yw))));
                    cnt = k + 1;
                }
            }
        }
    }
    const int32_t colStep = NHWC ? g.chan : 1; // a compile-time 1 for NCHW: the taps of a row are pw[0 .. K)

    for (int64_t row = blockIdx.y; row < g.rows; row += gridDim.y) {
        const int64_t plane = row / g.hin;
        const int32_t yh = static_cast<int32_t>(row - plane * g.hin);
        const T* pg = go + plane * planeGo;
        T* po = gi + row * inner;
        if (overflow) {
            po[t] = DType<T>::FromF(BwdElementDirect<T>(pg, g, yh, yw, c, rowGo, offset));
            continue;
        }
        const bool borderH = yh == 0 || yh == g.hin - 1; // uniform over the block
        const int32_t hStart = WalkStart(yh, g.invH, offset);
        float rh = Sub(Mul(Add(static_cast<float>(hStart), offset), g.scaleH), offset);
        float add = 0.0f;
        const T* pw0 = pg + c + static_cast<int64_t>(wStart) * colStep; // K * chan fits 32 bits (W * C does)
        if (!borderH) {
            for (int32_t h = hStart; h < g.hout; ++h, rh = BwdSrc(g.scaleH, h, g.align)) {
                if (!(rh < Add(static_cast<float>(yh), 2.0f))) {
                    break;
                }
                const float ch = PointCoeff(fabsf(Sub(rh, static_cast<float>(yh))));
                const T* pw = pw0 + h * rowGo;
                float gv[K];
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    gv[k] = k < cnt ? DType<T>::Load(pw + k * colStep) : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    gv[k] = Mul(Mul(gv[k], ch), cw[k]); // independent of the running sum: issued ahead of it
                }
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    if (k < cnt) {
                        add = Add(add, gv[k]);
                    }
                }
            }
        } else {
            for (int32_t h = hStart; h < g.hout; ++h, rh = BwdSrc(g.scaleH, h, g.align)) {
                const long long fh = static_cast<long long>(floorf(rh));
                if (yh == 0 && fh > 1 && g.hin > 1) {
                    break;
                }
                float chTap[4];
                TapCoeff(Sub(rh, static_cast<float>(fh)), chTap);
                bool hit[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    hit[i] = ClampIdx(fh - 1 + i, g.hin - 1) == yh;
                }
                const T* pw = pw0 + h * rowGo;
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    if (k < cnt) {
                        const float gvk = DType<T>::Load(pw + k * colStep);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (hit[i]) {
                                add = Add(add, Mul(Mul(gvk, chTap[i]), cw[k]));
                            }
                        }
                    }
                }
            }
        }
        po[t] = DType<T>::FromF(add);
    }
}

// ---- backward at exactly 2x (scales 0.5, align_corners = false), NCHW --------------------------------------------
// At this scale every source coordinate w / 2 - 0.25 is exact, so the walk of an interior grad_input index y visits
// the grads indices 2y - 3 .. 2y + 4 (those inside the image) and the coefficient of the k-th of them is the same
// number PointCoeff(|k / 2 - 1.75|) for every y. A block stages the grads rows of a band of grad_input rows in shared
// memory as fp32 (each grads value is loaded and converted once instead of sixteen times), with zero columns either
// side: a term whose grads column lies outside the image then adds a zero, which leaves a round-to-nearest sum that
// started from +0 unchanged, so the window of a column needs no bounds. A thread owns two adjacent grad_input
// columns of one row and reads their ten grads columns of a grads row as three 16-byte shared-memory loads. The
// first and last row and column, whose walk has up to three clamped taps per grads index, take their (index,
// coefficient) entries from four lists that the block builds with the reference's walk; the border columns are items
// of their own behind the pairs, so that their longer loop does not run in the warps of the interior. Terms, their
// (row, column, row tap, column tap) order and their rounding are those of the other two backward kernels.
// n / d for n * d < 2^32 as the high half of one 32-bit multiply: m = floor(2^32 / d) + 1 (the usual round-up
// reciprocal; exact because n * (m * d - 2^32) < 2^32 there). d = 1 has no 32-bit reciprocal and is tested for. The
// item loops below split an item index into (row, position) with it.
struct FastDiv {
    uint32_t m, d;
};
inline FastDiv MakeFastDiv(uint32_t d) { return FastDiv{d > 1 ? static_cast<uint32_t>((1ULL << 32) / d + 1) : 0u, d}; }
__device__ __forceinline__ uint32_t DivBy(uint32_t n, FastDiv f) { return f.d > 1 ? __umulhi(n, f.m) : n; }

constexpr int kX2Pad = 4;     // zero columns left of a staged grads row (the window of column 0 starts at -4)
constexpr int kX2Groups = 5;  // grads indices in the walk of a first or last index at 2x
constexpr int kX2Slots = 3;   // clamped taps of one grads index that fall on it (four only for an extent of 1)
constexpr int kX2Threads = 256;

// The walk of a first or last grad_input index in slot form: grads indices start .. start + 4, up to three tap
// coefficients each in tap order; bit 3m + t of mask says that slot t of group m holds a term.
constexpr int kX2Flat = 9;    // terms of such a walk when the extent is at least 2
struct X2BorderList {
    int32_t start;
    uint32_t mask;
    float coef[kX2Groups * kX2Slots];
    // the same terms one after the other in walk order, filled up with (column -1, 0): a term of the zero column
    // adds nothing, so a loop over all kX2Flat entries needs no test
    int32_t flatIdx[kX2Flat];
    float flatCoef[kX2Flat];
    int32_t terms;
};

struct X2BorderLists {
    X2BorderList l[4]; // 0 first column, 1 last column, 2 first row, 3 last row
    float interior[8]; // coefficient of the k-th grads index of an interior walk: PointCoeff(|k / 2 - 1.75|)
};

// The reference's walk for a first or last index at scale 0.5, on the host: this file's host code is compiled with
// floating-point contraction off, so every operation below rounds as the device's non-fused multiply and add do
// (and at this scale the coordinates and the fractions 0.25 / 0.75 are exact anyway).
namespace x2host {
inline float Conv1(float x) { return ((((kA + 2.0f) * x) - (kA + 3.0f)) * x) * x + 1.0f; }
inline float Conv2(float x) { return ((((kA * x) - 5.0f * kA) * x) + 8.0f * kA) * x - 4.0f * kA; }
inline float PointCoeff(float d) { return d <= 1.0f ? Conv1(d) : (d < 2.0f ? Conv2(d) : 0.0f); }
inline void FwdCoeff(float t, float (&c)[4])
{
    c[0] = Conv2(t + 1.0f);
    c[1] = Conv1(t);
    c[2] = Conv1(1.0f - t);
    c[3] = Conv2(2.0f - t);
}
inline X2BorderList BorderList(int32_t yIdx, int32_t in, int32_t out)
{
    X2BorderList list;
    const int32_t start = std::max(2 * yIdx - 3, 0); // ceil((y - 2 + 0.5) * 2 - 0.5), clamped at 0
    uint32_t mask = 0;
    for (int k = 0; k < kX2Groups * kX2Slots; ++k) {
        list.coef[k] = 0.0f;
    }
    for (int32_t o = start; o < out && o - start < kX2Groups; ++o) {
        const float r = (static_cast<float>(o) + 0.5f) * 0.5f - 0.5f;
        const long long f = static_cast<long long>(std::floor(r));
        if (yIdx == 0 && f > 1 && in > 1) {
            break;
        }
        const float t = r - static_cast<float>(f);
        const float u = 1.0f - t;
        const float tap[4] = {Conv2(t + 1.0f), Conv1(t), Conv1(u), Conv2(u + 1.0f)};
        int slot = 0;
        for (int j = 0; j < 4; ++j) {
            const long long idx = std::min<long long>(std::max<long long>(f - 1 + j, 0), in - 1);
            if (idx == yIdx && slot < kX2Slots) {
                list.coef[(o - start) * kX2Slots + slot] = tap[j];
                mask |= 1u << ((o - start) * kX2Slots + slot);
                ++slot;
            }
        }
    }
    list.start = start;
    list.mask = mask;
    list.terms = 0;
    for (int k = 0; k < kX2Flat; ++k) {
        list.flatIdx[k] = -1;
        list.flatCoef[k] = 0.0f;
    }
    for (int k = 0; k < kX2Groups * kX2Slots; ++k) {
        if (mask & (1u << k)) {
            if (list.terms < kX2Flat) {
                list.flatIdx[list.terms] = start + k / kX2Slots;
                list.flatCoef[list.terms] = list.coef[k];
            }
            ++list.terms;
        }
    }
    return list;
}
} // namespace x2host

// The four corners of a plane at 2x: both walks have clamped taps, so a grads value meets up to three row
// coefficients times up to three column coefficients, row taps outside column taps. One thread per plane and corner,
// the corner uniform over a block, so every slot test is uniform; grads straight from global memory.
template <typename T>
__device__ __forceinline__ void X2Corner(const T* __restrict__ go, T* __restrict__ gi, const BicubicGeom& g, int64_t plane,
                                         int corner, const X2BorderLists& lists)
{
    // corner: 0 (0, 0), 1 (0, win - 1), 2 (hin - 1, 0), 3 (hin - 1, win - 1)
    const X2BorderList& rows = lists.l[2 + (corner >> 1)];
    const X2BorderList& cols = lists.l[corner & 1];
    const uint32_t rmask = rows.mask, cmask = cols.mask;
    const T* pg = go + plane * (static_cast<int64_t>(g.hout) * g.wout);
    float add = 0.0f;
#pragma unroll
    for (int mr = 0; mr < kX2Groups; ++mr) {
        const uint32_t rbits = (rmask >> (mr * kX2Slots)) & 7u;
        if (rbits == 0) {
            continue;
        }
        const T* prow = pg + static_cast<int64_t>(rows.start + mr) * g.wout;
#pragma unroll
        for (int m = 0; m < kX2Groups; ++m) {
            const uint32_t cbits = (cmask >> (m * kX2Slots)) & 7u;
            if (cbits == 0) {
                continue;
            }
            const float gv = DType<T>::Load(prow + cols.start + m);
#pragma unroll
            for (int i = 0; i < kX2Slots; ++i) {
                if (rbits & (1u << i)) {
                    const float gch = Mul(gv, rows.coef[mr * kX2Slots + i]);
#pragma unroll
                    for (int t = 0; t < kX2Slots; ++t) {
                        if (cbits & (1u << t)) {
                            add = Add(add, Mul(gch, cols.coef[m * kX2Slots + t]));
                        }
                    }
                }
            }
        }
    }
    const int32_t yh = (corner >> 1) ? g.hin - 1 : 0, yw = (corner & 1) ? g.win - 1 : 0;
    gi[(plane * g.hin + yh) * g.win + yw] = DType<T>::FromF(add);
}

template <typename T>
__global__ void __launch_bounds__(kX2Threads) Bicubic2dBwdX2Kernel(const T* __restrict__ go, T* __restrict__ gi, BicubicGeom g,
                                                                   int32_t bandRows, int32_t bands, int32_t pitch,
                                                                   int32_t vecLoad, const X2BorderLists lists,
                                                                   int64_t planes, int32_t cornerBlocks)
{
    extern __shared__ __align__(16) float sG[]; // (2 * bandRows + 6) grads rows of `pitch` floats
    const X2BorderList* sL = lists.l;
    const int32_t tid = threadIdx.x, nt = blockDim.x;
    if (static_cast<int32_t>(blockIdx.x) < cornerBlocks) {
        // the first blocks of the grid take the corners of all planes (four blocks per nt planes); they are resident
        // next to band blocks from the start, so their chains of dependent additions cost no time of their own
        const int64_t cp = static_cast<int64_t>(blockIdx.x >> 2) * nt + tid;
        if (cp < planes) {
            X2Corner<T>(go, gi, g, cp, static_cast<int>(blockIdx.x & 3), lists);
        }
        return;
    }
    const uint32_t bandBlock = blockIdx.x - cornerBlocks;
    const int64_t plane = bandBlock / bands;
    const int32_t band = static_cast<int32_t>(bandBlock - plane * bands);
    const int32_t yhA = band * bandRows, yhB = min(yhA + bandRows, g.hin);
    const int32_t hBase = 2 * yhA - 3; // grads row of shared-memory row 0
    const int32_t hLo = max(hBase, 0), hHi = min(2 * (yhB - 1) + 4, g.hout - 1);
    const int32_t nRows = hHi - hLo + 1;

    const float* c = lists.interior;
    {
        // zero rows where the band's window leaves the image, zero columns either side of a row, as 8-byte stores (wout is even)
        const int32_t rowsTop = hLo - hBase, rowsAll = 2 * (yhB - yhA) + 6;
        const int32_t rowsZero = rowsAll - nRows; // above the first image row and below the last
        for (int32_t i = tid; i < rowsZero * (pitch / 4); i += nt) {
            const int32_t r = i / (pitch / 4), k = i - r * (pitch / 4);
            const int32_t row = r < rowsTop ? r : nRows + r;
            *reinterpret_cast<float4*>(sG + row * pitch + 4 * k) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        float* sRow0 = sG + (hLo - hBase) * pitch;
        const int32_t padPairs = (pitch - g.wout) / 2;
        for (int32_t i = tid; i < nRows * padPairs; i += nt) {
            const int32_t r = i / padPairs, k = i - r * padPairs;
            *reinterpret_cast<float2*>(sRow0 + r * pitch + (k < kX2Pad / 2 ? 2 * k : g.wout + 2 * k)) = make_float2(0.0f, 0.0f);
        }
        const T* pg = go + plane * (static_cast<int64_t>(g.hout) * g.wout) + static_cast<int64_t>(hLo) * g.wout;
        float* sBase = sRow0 + kX2Pad;
        // a thread keeps its position in a row and steps over rows: one division per thread instead of one per load
        if (vecLoad) {
            constexpr int VL = 16 / sizeof(T);
            const int32_t packs = g.wout / VL;
            const int32_t lanesPerRow = min(packs, nt), rowsPerPass = nt / lanesPerRow;
            const int32_t r0 = tid / lanesPerRow, p0 = tid - r0 * lanesPerRow;
            if (r0 < rowsPerPass) {
                for (int32_t r = r0; r < nRows; r += rowsPerPass) {
                    for (int32_t p = p0; p < packs; p += lanesPerRow) {
                        float v[VL];
                        LoadPackLdg<T, VL>(pg + r * g.wout + p * VL, v);
                        float4* dst = reinterpret_cast<float4*>(sBase + r * pitch + p * VL);
#pragma unroll
                        for (int m = 0; m < VL / 4; ++m) {
                            dst[m] = make_float4(v[4 * m], v[4 * m + 1], v[4 * m + 2], v[4 * m + 3]);
                        }
                    }
                }
            }
        } else {
            const int32_t lanesPerRow = min(g.wout, nt), rowsPerPass = nt / lanesPerRow;
            const int32_t r0 = tid / lanesPerRow, w0 = tid - r0 * lanesPerRow;
            if (r0 < rowsPerPass) {
                for (int32_t r = r0; r < nRows; r += rowsPerPass) {
                    for (int32_t w = w0; w < g.wout; w += lanesPerRow) {
                        sBase[r * pitch + w] = DType<T>::Load(pg + r * g.wout + w);
                    }
                }
            }
        }
    }
    __syncthreads();

    const int32_t pairs = (g.win + 1) / 2;
    const int32_t bandN = yhB - yhA;
    const int32_t nPair = bandN * pairs;
    const int32_t borderBase = (nPair + 31) & ~31;      // first columns from here, one per row of the band
    const int32_t borderBase1 = borderBase + ((bandN + 31) & ~31); // last columns: other warps, so that the slot
    const int32_t total = borderBase1 + bandN;                 // tests below are uniform over a warp
    T* pgi = gi + (plane * g.hin + yhA) * g.win;
    for (int32_t item = tid; item < total; item += nt) {
        if (item < nPair) {
            const int32_t r = item / pairs, q = item - r * pairs;
            const int32_t yh = yhA + r;
            const float* sw = sG + 4 * q; // grads column 4q - 4
            float a0 = 0.0f, a1 = 0.0f;
            if (yh != 0 && yh != g.hin - 1) {
                const float4* row = reinterpret_cast<const float4*>(sw + (2 * yh - 3 - hBase) * pitch);
#pragma unroll
                for (int j = 0; j < 8; ++j, row += pitch / 4) {
                    { // rows above or below the image are zero rows: their terms add nothing
                        const float4 A = row[0], B = row[1], C = row[2];
                        const float v[12] = {A.x, A.y, A.z, A.w, B.x, B.y, B.z, B.w, C.x, C.y, C.z, C.w};
                        float gc[10];
#pragma unroll
                        for (int k = 0; k < 10; ++k) {
                            gc[k] = Mul(v[1 + k], c[j]);
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            a0 = Add(a0, Mul(gc[k], c[k]));
                            a1 = Add(a1, Mul(gc[2 + k], c[k]));
                        }
                    }
                }
            } else {
                const X2BorderList& rows = sL[yh == 0 ? 2 : 3];
                const uint32_t mask = rows.mask;
#pragma unroll 1
                for (int m = 0; m < kX2Groups; ++m) {
                    const uint32_t bits = (mask >> (m * kX2Slots)) & 7u;
                    if (bits == 0) {
                        continue;
                    }
                    const float ch0 = rows.coef[m * kX2Slots], ch1 = rows.coef[m * kX2Slots + 1],
                                ch2 = rows.coef[m * kX2Slots + 2];
                    const float4* row = reinterpret_cast<const float4*>(sw + (rows.start + m - hBase) * pitch);
                    const float4 A = row[0], B = row[1], C = row[2];
                    const float v[12] = {A.x, A.y, A.z, A.w, B.x, B.y, B.z, B.w, C.x, C.y, C.z, C.w};
#pragma unroll
                    for (int k = 0; k < 8; ++k) { // slots fill in tap order, so bit 0 is set whenever the group is
                        a0 = Add(a0, Mul(Mul(v[1 + k], ch0), c[k]));
                        a1 = Add(a1, Mul(Mul(v[3 + k], ch0), c[k]));
                        if (bits & 2u) {
                            a0 = Add(a0, Mul(Mul(v[1 + k], ch1), c[k]));
                            a1 = Add(a1, Mul(Mul(v[3 + k], ch1), c[k]));
                        }
                        if (bits & 4u) {
                            a0 = Add(a0, Mul(Mul(v[1 + k], ch2), c[k]));
                            a1 = Add(a1, Mul(Mul(v[3 + k], ch2), c[k]));
                        }
                    }
                }
            }
            T* po = pgi + static_cast<int64_t>(r) * g.win;
            const int32_t yw0 = 2 * q;
            if (yw0 >= 1 && yw0 <= g.win - 2) {
                po[yw0] = DType<T>::FromF(a0);
            }
            if (yw0 + 1 <= g.win - 2) {
                po[yw0 + 1] = DType<T>::FromF(a1);
            }
        } else if (item >= borderBase) {
            // a first or last column of an interior row: the terms of its walk as one list
            const int32_t side = item >= borderBase1 ? 1 : 0;
            const int32_t r = item - (side ? borderBase1 : borderBase);
            if (r >= bandN) {
                continue;
            }
            const int32_t yh = yhA + r;
            if (yh == 0 || yh == g.hin - 1) {
                continue; // the four corners of a plane: the corner blocks
            }
            const X2BorderList& cols = sL[side];
            float add = 0.0f;
            int32_t wI[kX2Flat];
            float cw[kX2Flat];
#pragma unroll
            for (int e = 0; e < kX2Flat; ++e) {
                wI[e] = cols.flatIdx[e];
                cw[e] = cols.flatCoef[e];
            }
            const float* prow = sG + (2 * yh - 3 - hBase) * pitch + kX2Pad;
#pragma unroll
            for (int j = 0; j < 8; ++j, prow += pitch) {
#pragma unroll
                for (int e = 0; e < kX2Flat; ++e) {
                    add = Add(add, Mul(Mul(prow[wI[e]], c[j]), cw[e]));
                }
            }
            pgi[static_cast<int64_t>(r) * g.win + (side ? g.win - 1 : 0)] = DType<T>::FromF(add);
        }
    }
}

// ---- forward at exactly 2x (half-pixel coordinates, scales 0.5), NCHW ---------------------------------------------
// Output index 2i has the source coordinate i - 0.25 (window i - 2 .. i + 1, fraction 0.75), output index 2i + 1 has
// i + 0.25 (window i - 1 .. i + 2, fraction 0.25), all exact: two sets of four coefficients serve the whole image
// and come from the host. A block stages the source rows of a band (with the two rows above and below it, clamped)
// as fp32 with replicated columns either side, so that neither pass clamps an index; pass A forms the
// horizontal sums of every staged row, eight adjacent output columns per thread from eight source values (four
// 8-byte shared-memory loads, two 16-byte stores); pass B gives a thread four adjacent columns of the four output rows
// of two source rows: six 16-byte loads of sums, four stores. Sums and products in the order of the general kernels.
struct X2FwdCoef {
    float even[4]; // FwdCoeff(0.75): output indices 2i
    float odd[4];  // FwdCoeff(0.25): output indices 2i + 1
};

// FULL: every group of four output columns is whole and every row 8- or 16-byte aligned (one store per group).
template <typename T, bool FULL>
__global__ void __launch_bounds__(kX2Threads) Bicubic2dFwdX2Kernel(const T* __restrict__ x, T* __restrict__ y, BicubicGeom g,
                                                                   int32_t bandRows, int32_t bands, int32_t vecIn,
                                                                   int32_t vecOut, const X2FwdCoef cf, const FastDiv halfPacks,
                                                                   const FastDiv packsDiv)
{
    extern __shared__ __align__(16) float sm[];
    const int32_t tid = threadIdx.x, nt = blockDim.x;
    const int32_t pitchX = g.win + 4 + (g.win & 1); // two replicated columns left, two or three right (even pitch)
    const int32_t packs = (g.wout + 3) / 4, pitchH = 4 * packs; // an odd input width leaves the last pack half used
    const int64_t plane = blockIdx.x / bands;
    const int32_t band = static_cast<int32_t>(blockIdx.x - plane * bands);
    const int32_t rA = band * bandRows, rB = min(rA + bandRows, g.hin);
    const int32_t nSlots = rB - rA + 4; // slot s holds source row clamp(rA - 2 + s)
    float* sX = sm;
    float* sH = sm + (((bandRows + 4) * pitchX + 3) & ~3);
    const T* px = x + plane * (static_cast<int64_t>(g.hin) * g.win);
    {
        for (int32_t i = tid; i < 2 * nSlots; i += nt) { // the replicated columns
            const int32_t sl = i >> 1, right = i & 1;
            const int32_t row = ClampIdx32(rA - 2 + sl, g.hin - 1);
            const float v = DType<T>::Load(px + static_cast<int64_t>(row) * g.win + (right ? g.win - 1 : 0));
            if (right) {
                for (int32_t k = g.win + 2; k < pitchX; ++k) {
                    sX[sl * pitchX + k] = v;
                }
            } else {
                *reinterpret_cast<float2*>(sX + sl * pitchX) = make_float2(v, v);
            }
        }
        if (vecIn) {
            constexpr int VL = 16 / sizeof(T);
            const int32_t packs = g.win / VL;
            const int32_t lanesPerRow = min(packs, nt), rowsPerPass = nt / lanesPerRow;
            const int32_t s0 = tid / lanesPerRow, p0 = tid - s0 * lanesPerRow;
            if (s0 < rowsPerPass) {
                for (int32_t sl = s0; sl < nSlots; sl += rowsPerPass) {
                    const T* prow = px + static_cast<int64_t>(ClampIdx32(rA - 2 + sl, g.hin - 1)) * g.win;
                    for (int32_t pk = p0; pk < packs; pk += lanesPerRow) {
                        float v[VL];
                        LoadPackLdg<T, VL>(prow + pk * VL, v);
                        float2* dst = reinterpret_cast<float2*>(sX + sl * pitchX + 2 + pk * VL);
#pragma unroll
                        for (int m = 0; m < VL / 2; ++m) {
                            dst[m] = make_float2(v[2 * m], v[2 * m + 1]);
                        }
                    }
                }
            }
        } else {
            const int32_t lanesPerRow = min(g.win, nt), rowsPerPass = nt / lanesPerRow;
            const int32_t s0 = tid / lanesPerRow, w0 = tid - s0 * lanesPerRow;
            if (s0 < rowsPerPass) {
                for (int32_t sl = s0; sl < nSlots; sl += rowsPerPass) {
                    const T* prow = px + static_cast<int64_t>(ClampIdx32(rA - 2 + sl, g.hin - 1)) * g.win;
                    for (int32_t w = w0; w < g.win; w += lanesPerRow) {
                        sX[sl * pitchX + 2 + w] = DType<T>::Load(prow + w);
                    }
                }
            }
        }
    }
    __syncthreads();
    // Both passes use the packed fp32 operations: two sums that share their coefficients go through one instruction
    // per product and per addition (AddProduct2 keeps the product's own rounding), so the bits are the scalar ones.
    const F2 E0 = MakeF2(cf.even[0], cf.even[0]), E1 = MakeF2(cf.even[1], cf.even[1]), E2 = MakeF2(cf.even[2], cf.even[2]),
             E3 = MakeF2(cf.even[3], cf.even[3]);
    const F2 O0 = MakeF2(cf.odd[0], cf.odd[0]), O1 = MakeF2(cf.odd[1], cf.odd[1]), O2 = MakeF2(cf.odd[2], cf.odd[2]),
             O3 = MakeF2(cf.odd[3], cf.odd[3]);
    // ((t0 c0 + t1 c1) + t2 c2) + t3 c3 on both halves
    auto blend = [](F2 t0, F2 t1, F2 t2, F2 t3, F2 c0, F2 c1, F2 c2, F2 c3) {
        F2 acc = AddProduct2(Mul2(t1, c1), Mul2(t0, c0));
        acc = AddProduct2(Mul2(t2, c2), acc);
        return AddProduct2(Mul2(t3, c3), acc);
    };
    // pass A: eight adjacent sums of a staged row from eight source values (the second four only where they exist).
    // Output columns 4q and 4q + 2 share the even coefficients and have windows one source pixel apart, 4q + 1 and
    // 4q + 3 likewise with the odd ones: each pair is one packed chain, and a group of four sums is stored in the
    // order (0, 2, 1, 3), which pass B undoes when it stores.
    for (int32_t item = tid; item < nSlots * static_cast<int32_t>(halfPacks.d); item += nt) {
        const int32_t sl = DivBy(item, halfPacks), q = 2 * (item - sl * static_cast<int32_t>(halfPacks.d));
        if (sl >= nSlots || q >= packs) {
            continue; // cannot happen for item below the bound; keeps a wrong quotient from leaving the tiles
        }
        const float2* src = reinterpret_cast<const float2*>(sX + sl * pitchX + 2 * q); // source columns 2q - 2 ..
        const float2 a = src[0], b = src[1], c = src[2];
        const F2 A = MakeF2(a.x, a.y), B = MakeF2(b.x, b.y), C = MakeF2(c.x, c.y);
        const F2 AB = MakeF2(a.y, b.x), BC = MakeF2(b.y, c.x);
        F2* dst = reinterpret_cast<F2*>(sH + sl * pitchH + 4 * q);
        struct alignas(16) Quad {
            F2 lo, hi;
        };
        Quad h;
        h.lo = blend(A, AB, B, BC, E0, E1, E2, E3);  // columns 4q, 4q + 2
        h.hi = blend(AB, B, BC, C, O0, O1, O2, O3);  // columns 4q + 1, 4q + 3
        *reinterpret_cast<Quad*>(dst) = h;
        if (q + 1 < packs) {
            const float2 d = src[3];
            const F2 D = MakeF2(d.x, d.y), CD = MakeF2(c.y, d.x);
            h.lo = blend(B, BC, C, CD, E0, E1, E2, E3);
            h.hi = blend(BC, C, CD, D, O0, O1, O2, O3);
            *reinterpret_cast<Quad*>(dst + 2) = h;
        }
    }
    __syncthreads();
    // pass B: four adjacent columns of the four output rows of two source rows (two where the band ends)
    T* py = y + (plane * g.hout + 2 * rA) * static_cast<int64_t>(g.wout);
    const int32_t rows = rB - rA;
    const int32_t step = packs;
    // lo = columns (0, 2), hi = columns (1, 3) of the group; valid = columns of the group inside the row (4, or 2 in
    // the last group of a row whose width is not a multiple of 4); vecOut = elements per store the rows allow
    auto store = [&](T* dst, F2 lo, F2 hi, int32_t valid) {
        float vals[4];
        SplitF2(lo, vals[0], vals[2]);
        SplitF2(hi, vals[1], vals[3]);
        if (FULL) {
            StorePack<T, 4>(dst, vals);
        } else if (vecOut == 2) {
            const float a[2] = {vals[0], vals[1]}, b[2] = {vals[2], vals[3]};
            StorePack<T, 2>(dst, a);
            if (valid > 2) {
                StorePack<T, 2>(dst + 2, b);
            }
        } else {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                if (v < valid) {
                    dst[v] = DType<T>::FromF(vals[v]);
                }
            }
        }
    };
    for (int32_t item = tid; item < ((rows + 1) / 2) * packs; item += nt) {
        const int32_t r2 = DivBy(item, packsDiv), q = item - r2 * packs;
        const int32_t r = 2 * r2;
        if (r >= rows || q < 0 || q >= packs) {
            continue; // as in pass A
        }
        const float4* col = reinterpret_cast<const float4*>(sH + r * pitchH + 4 * q); // slots r .. r + 5
        const float4 R0 = col[0], R1 = col[step], R2 = col[2 * step], R3 = col[3 * step], R4 = col[4 * step];
        const F2 l0 = MakeF2(R0.x, R0.y), h0 = MakeF2(R0.z, R0.w), l1 = MakeF2(R1.x, R1.y), h1 = MakeF2(R1.z, R1.w),
                 l2 = MakeF2(R2.x, R2.y), h2 = MakeF2(R2.z, R2.w), l3 = MakeF2(R3.x, R3.y), h3 = MakeF2(R3.z, R3.w),
                 l4 = MakeF2(R4.x, R4.y), h4 = MakeF2(R4.z, R4.w);
        T* dst = py + static_cast<int64_t>(2 * r) * g.wout + 4 * q;
        const int32_t valid = FULL ? 4 : min(4, g.wout - 4 * q);
        store(dst, blend(l0, l1, l2, l3, E0, E1, E2, E3), blend(h0, h1, h2, h3, E0, E1, E2, E3), valid);
        store(dst + g.wout, blend(l1, l2, l3, l4, O0, O1, O2, O3), blend(h1, h2, h3, h4, O0, O1, O2, O3), valid);
        if (r + 1 < rows) {
            const float4 R5 = col[5 * step];
            const F2 l5 = MakeF2(R5.x, R5.y), h5 = MakeF2(R5.z, R5.w);
            store(dst + 2 * g.wout, blend(l1, l2, l3, l4, E0, E1, E2, E3), blend(h1, h2, h3, h4, E0, E1, E2, E3), valid);
            store(dst + 3 * g.wout, blend(l2, l3, l4, l5, O0, O1, O2, O3), blend(h2, h3, h4, h5, O0, O1, O2, O3), valid);
        }
    }
}

// Band height and block size of the 2x kernel. false: the kernel does not apply.
struct X2Launch {
    int32_t bandRows, bands, threads, pitch;
    size_t smem;
};
bool PlanBwdX2(const BicubicGeom& g, bool nhwc, X2Launch* out)
{
    if (nhwc || g.align || g.scaleH != 0.5f || g.scaleW != 0.5f || g.invH != 2.0f || g.invW != 2.0f ||
        g.hin < 2 || g.win < 2 || g.hout != 2 * g.hin || g.wout != 2 * g.win || g.wout > (1 << 20)) {
        return false;
    }
    const int32_t pitch = (g.wout + 12 + 3) & ~3;
    const int32_t pairs = (g.win + 1) / 2;
    // Bands as tall as 32 KB of staged rows allow (measured at 56 x 56 planes: taller bands stage fewer halo rows and
    // pay the per-block set-up less often, 301 us at 28 rows against 337 us at 14; a whole plane per block, 58 KB,
    // leaves too few blocks per SM: 341 us), equal over the plane; then the block size that wastes the fewest warp
    // slots over the passes of the item loop.
    const size_t rowBytes = static_cast<size_t>(pitch) * sizeof(float);
    int32_t bh = static_cast<int32_t>(std::min<int64_t>((32 * 1024 / rowBytes - 6) / 2, g.hin));
    if (bh < 1) {
        bh = 1;
    }
    if ((2 * bh + 6) * rowBytes > 48 * 1024) {
        return false;
    }
    const int32_t nb = (g.hin + bh - 1) / bh;
    bh = (g.hin + nb - 1) / nb;
    const int64_t warpItems = CeilDiv(static_cast<int64_t>(bh) * pairs, 32) + 2 * CeilDiv(bh, 32);
    double best = 0.0;
    for (int32_t threads = 128; threads <= kX2Threads; threads += 32) {
        const int64_t warps = threads / 32;
        const double fill = static_cast<double>(warpItems) / static_cast<double>(CeilDiv(warpItems, warps) * warps);
        if (fill > best) { // ties go to the smaller block: more blocks per SM to overlap staging with arithmetic
            best = fill;
            *out = X2Launch{bh, nb, threads, pitch, (2 * bh + 6) * rowBytes};
        }
    }
    const int64_t planes = g.rows / g.hin;
    return planes * out->bands + 4 * CeilDiv(planes, out->threads) <= INT32_MAX;
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
    const int64_t planes = nhwc ? sh.n : sh.n * sh.c;
    BicubicGeom g;
    g.rows = planes * sh.hout;
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
    const int64_t inner = static_cast<int64_t>(g.wout) * g.chan;
    if (schedule != 0) {
        const dim3 grid = RowGrid(g.rows, inner);
        OPSCV_DISPATCH_DT(dt, T, {
            if (nhwc) {
                Bicubic2dFwdCopyKernel<T, true><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(y), g);
            } else {
                Bicubic2dFwdCopyKernel<T, false><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(y), g);
            }
        });
        CountLaunch();
        return cudaGetLastError();
    }
    if (!nhwc && halfPixel && scaleH == 0.5f && scaleW == 0.5f && g.hout == 2 * g.hin && g.wout == 2 * g.win &&
        g.win <= (1 << 20)) {
        // exactly 2x: bands of source rows whose staged rows and horizontal sums take about 32 KB
        const size_t pitchX = static_cast<size_t>(g.win) + 4 + (g.win & 1), pitchH = (static_cast<size_t>(g.wout) + 3) / 4 * 4;
        const size_t slotBytes = (pitchX + pitchH) * sizeof(float);
        int32_t bh = static_cast<int32_t>(std::min<int64_t>(static_cast<int64_t>(32 * 1024 / slotBytes) - 4, g.hin));
        bh = std::max(bh, 1);
        const int32_t nb = (g.hin + bh - 1) / bh;
        bh = (g.hin + nb - 1) / nb;
        const size_t smem = ((static_cast<size_t>(bh + 4) * pitchX + 3) / 4 * 4 + static_cast<size_t>(bh + 4) * pitchH) * sizeof(float);
        if (smem <= 48 * 1024 && planes * nb <= INT32_MAX) {
            X2FwdCoef cf;
            x2host::FwdCoeff(0.75f, cf.even);
            x2host::FwdCoeff(0.25f, cf.odd);
            const int threads = 128; // measured at 56 x 56 planes: 101 us against 109 us with 256 (more blocks per SM overlap the three phases)
            OPSCV_DISPATCH_DT(dt, T, {
                const int vecIn = (g.win % (16 / sizeof(T)) == 0 && Aligned(x, 16)) ? 1 : 0;
                const int vecOut = (g.wout % 4 == 0 && Aligned(y, 4 * sizeof(T))) ? 4 : (Aligned(y, 2 * sizeof(T)) ? 2 : 1);
                auto k = vecOut == 4 ? Bicubic2dFwdX2Kernel<T, true> : Bicubic2dFwdX2Kernel<T, false>;
                k<<<static_cast<unsigned>(planes * nb), threads, smem, s>>>(
                    static_cast<const T*>(x), static_cast<T*>(y), g, bh, nb, vecIn, vecOut, cf,
                    MakeFastDiv(static_cast<uint32_t>(((g.wout + 3) / 4 + 1) / 2)), MakeFastDiv(static_cast<uint32_t>((g.wout + 3) / 4)));
            });
            CountLaunch();
            return cudaGetLastError();
        }
    }
    if (!nhwc) {
        // the shared-memory tile form: the largest band of output rows whose tiles fit 64 KB
        const int es = DtSize(dt);
        int v = 16 / es;
        while (v > 1 && (g.wout % v != 0 || !Aligned(y, static_cast<size_t>(v) * es))) {
            v >>= 1;
        }
        std::vector<int32_t> top(static_cast<size_t>(g.hout));
        for (int32_t H = 0; H < g.hout; ++H) {
            top[H] = FwdTop(H, g.scaleH, g.align, g.hin, nullptr);
        }
        auto clampRow = [&](int32_t r) { return std::min(std::max(r, 0), g.hin - 1); };
        BicubicTile tile{};
        size_t smem = 0;
        for (int32_t band = g.hout; band >= 4; band = (band + 1) / 2) {
            int32_t worst = 0;
            for (int32_t h0 = 0; h0 < g.hout; h0 += band) {
                const int32_t h1 = std::min(h0 + band, g.hout);
                worst = std::max(worst, clampRow(top[h1 - 1] + 2) - clampRow(top[h0] - 1) + 1);
            }
            const size_t need = (static_cast<size_t>(worst) * (static_cast<size_t>(g.wout) + g.win) + 5u * band) * sizeof(float);
            if (need <= 64u * 1024u) {
                tile.bandRows = band;
                tile.bands = static_cast<int32_t>(CeilDiv(g.hout, band));
                tile.maxSrc = worst;
                smem = need;
                break;
            }
            if (band == 4) {
                break;
            }
        }
        // a band must still be long enough to amortise the three extra source rows it loads
        if (smem != 0 && (tile.bandRows >= 16 || tile.bands == 1)) {
            int tw = 1; // one thread per pair of columns in the horizontal pass
            while (tw < (g.wout + 1) / 2 && tw < kThreads) {
                tw <<= 1;
            }
            int pw = 1;
            while (pw < g.wout / v && pw < kThreads) {
                pw <<= 1;
            }
            tile.tw = tw;
            tile.pw = pw;
            const int64_t items = planes * tile.bands;
            const int64_t perSm = std::max<int64_t>(1, std::min<int64_t>(8, (200u * 1024u) / smem));
            const unsigned grid = static_cast<unsigned>(std::min<int64_t>(items, static_cast<int64_t>(NumSMs()) * perSm * 4));
            cudaError_t attr = cudaSuccess;
            OPSCV_DISPATCH_DT(dt, T, {
                const T* px = static_cast<const T*>(x);
                T* py = static_cast<T*>(y);
                OPSCV_DISPATCH_VEC(v, V, {
                    if constexpr (V * sizeof(T) <= 16) {
                        if (smem > 48u * 1024u) {
                            attr = cudaFuncSetAttribute(Bicubic2dFwdTileKernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        static_cast<int>(smem));
                        }
                        if (attr == cudaSuccess) {
                            Bicubic2dFwdTileKernel<T, V><<<grid, kThreads, smem, s>>>(px, py, g, tile, items);
                        }
                    }
                });
            });
            if (attr != cudaSuccess) {
                return attr;
            }
            CountLaunch();
            return cudaGetLastError();
        }
    }
    // Two elements per thread for 16-bit tensors (4-byte stores) when rows allow it. Bands: enough (plane, band)
    // items to fill the device a few times over, but at least 16 output rows each, since every band starts by
    // computing four horizontal sums afresh.
    const int v = (DtSize(dt) == 2 && inner % 2 == 0 && Aligned(y, 4)) ? 2 : 1;
    // a block as wide as the row when the row is short, so that no warp of it is idle
    const int threads = static_cast<int>(std::min<int64_t>(kThreads, (CeilDiv(inner, v) + 31) / 32 * 32));
    const int64_t colBlocks = CeilDiv(CeilDiv(inner, v), threads);
    const int64_t want = static_cast<int64_t>(NumSMs()) * 8 * 4;
    int64_t bands = std::max<int64_t>(1, std::min<int64_t>(CeilDiv(want, std::max<int64_t>(planes * colBlocks, 1)),
                                                           std::max<int32_t>(sh.hout / 16, 1)));
    int32_t bandRows = static_cast<int32_t>(CeilDiv(sh.hout, bands));
    bandRows = std::min<int32_t>(bandRows, 2048); // 40 KB of row coefficients at most
    bands = CeilDiv(sh.hout, bandRows);
    const size_t smem = static_cast<size_t>(bandRows) * 5 * sizeof(float);
    g.rows = planes * bands;
    const dim3 grid(static_cast<unsigned>(colBlocks), static_cast<unsigned>(std::min<int64_t>(g.rows, 65535)), 1);
    OPSCV_DISPATCH_DT(dt, T, {
        const T* px = static_cast<const T*>(x);
        T* py = static_cast<T*>(y);
        if (nhwc) {
            if (v == 2) {
                Bicubic2dFwdKernel<T, true, 2><<<grid, threads, smem, s>>>(px, py, g, bandRows, static_cast<int32_t>(bands));
            } else {
                Bicubic2dFwdKernel<T, true, 1><<<grid, threads, smem, s>>>(px, py, g, bandRows, static_cast<int32_t>(bands));
            }
        } else {
            if (v == 2) {
                Bicubic2dFwdKernel<T, false, 2><<<grid, threads, smem, s>>>(px, py, g, bandRows, static_cast<int32_t>(bands));
            } else {
                Bicubic2dFwdKernel<T, false, 1><<<grid, threads, smem, s>>>(px, py, g, bandRows, static_cast<int32_t>(bands));
            }
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
    const int64_t inner = static_cast<int64_t>(g.win) * g.chan;
    const double perScale = invW > 0.0f ? static_cast<double>(invW) : 1.0;
    // columns of the longest interior walk: 4 / scale within two source pixels either side, one more for rounding
    const int64_t walk = static_cast<int64_t>(std::ceil(4.0 * perScale)) + 1;
    const bool split = walk <= 17 && sh.win > 2; // interior columns from registers, the two border columns apart
    // Entries of one column list: an interior column takes the grads columns of its walk, a first or last column
    // up to three taps of each column within two and a half source pixels (at most 6 / scale + a few). Lists that
    // would not fit make their thread fall back to the uncached walk, so the bound only has to be good, not safe;
    // a single-column image (every grads column is a tap) always falls back.
    int64_t maxW = static_cast<int64_t>(std::ceil(6.0 * perScale)) + 8;
    cudaError_t err = cudaSuccess;
    auto launchList = [&](bool borderOnly) {
        const int64_t positions = borderOnly ? 2LL * g.chan : inner;
        const int colsPB = static_cast<int>(std::min<int64_t>(kThreads, positions));
        const int threads = static_cast<int>(std::min<int64_t>(kThreads, (std::max<int64_t>(colsPB, 64) + 31) / 32 * 32));
        const int rowsPB = threads / colsPB;
        const int64_t cap = 96 * 1024 / (8 * threads);
        const int64_t entries = std::max<int64_t>(4, std::min<int64_t>(maxW, cap));
        const size_t smem = static_cast<size_t>(entries) * threads * 8;
        const int64_t gx = CeilDiv(positions, colsPB);
        const int64_t rowBlocks = CeilDiv(g.rows, rowsPB);
        const int64_t gyCap = std::max<int64_t>(static_cast<int64_t>(NumSMs()) * 32 / gx, 1);
        const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(std::min<int64_t>(std::min<int64_t>(rowBlocks, gyCap), 65535)), 1);
        OPSCV_DISPATCH_DT(dt, T, {
            auto kernel = nhwc ? Bicubic2dBwdListKernel<T, true> : Bicubic2dBwdListKernel<T, false>;
            if (smem > 48 * 1024) {
                err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            }
            if (err == cudaSuccess) {
                kernel<<<grid, threads, smem, s>>>(static_cast<const T*>(go), static_cast<T*>(gi), g,
                                                   static_cast<int32_t>(entries), colsPB, borderOnly ? 1 : 0);
            }
        });
        CountLaunch();
    };
    X2Launch x2;
    X2BorderLists lists;
    bool useX2 = PlanBwdX2(g, nhwc, &x2);
    if (useX2) {
        lists.l[0] = x2host::BorderList(0, g.win, g.wout);
        lists.l[1] = x2host::BorderList(g.win - 1, g.win, g.wout);
        lists.l[2] = x2host::BorderList(0, g.hin, g.hout);
        lists.l[3] = x2host::BorderList(g.hin - 1, g.hin, g.hout);
        for (const X2BorderList& l : lists.l) {
            useX2 = useX2 && l.terms <= kX2Flat;
        }
        for (int k = 0; k < 8; ++k) {
            lists.interior[k] = x2host::PointCoeff(std::fabs(0.5f * static_cast<float>(k) - 1.75f));
        }
    }
    if (useX2) {
        const int64_t planes = g.rows / g.hin;
        OPSCV_DISPATCH_DT(dt, T, {
            const int vec = (g.wout % (16 / sizeof(T)) == 0 && Aligned(go, 16)) ? 1 : 0;
            const int32_t cornerBlocks = 4 * static_cast<int32_t>(CeilDiv(planes, x2.threads));
            Bicubic2dBwdX2Kernel<T><<<static_cast<unsigned>(planes * x2.bands + cornerBlocks), x2.threads, x2.smem, s>>>(
                static_cast<const T*>(go), static_cast<T*>(gi), g, x2.bandRows, x2.bands, x2.pitch, vec, lists, planes,
                cornerBlocks);
        });
        CountLaunch();
        return cudaGetLastError();
    }
    if (!split) {
        launchList(false);
        return err != cudaSuccess ? err : cudaGetLastError();
    }
    {
        const int64_t positions = inner - 2LL * g.chan;
        const int threads = static_cast<int>(std::min<int64_t>(kThreads, (positions + 31) / 32 * 32));
        const int64_t gx = CeilDiv(positions, threads);
        const int64_t gyCap = std::max<int64_t>(static_cast<int64_t>(NumSMs()) * 32 / gx, 1);
        const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(std::min<int64_t>(std::min<int64_t>(g.rows, gyCap), 65535)), 1);
        OPSCV_DISPATCH_DT(dt, T, {
            const T* pgo = static_cast<const T*>(go);
            T* pgi = static_cast<T*>(gi);
            if (walk <= 9) {
                if (nhwc) {
                    Bicubic2dBwdRegKernel<T, true, 9><<<grid, threads, 0, s>>>(pgo, pgi, g);
                } else {
                    Bicubic2dBwdRegKernel<T, false, 9><<<grid, threads, 0, s>>>(pgo, pgi, g);
                }
            } else {
                if (nhwc) {
                    Bicubic2dBwdRegKernel<T, true, 17><<<grid, threads, 0, s>>>(pgo, pgi, g);
                } else {
                    Bicubic2dBwdRegKernel<T, false, 17><<<grid, threads, 0, s>>>(pgo, pgi, g);
                }
            }
        });
        CountLaunch();
    }
    launchList(true);
    return err != cudaSuccess ? err : cudaGetLastError();
}

} // namespace opscv
