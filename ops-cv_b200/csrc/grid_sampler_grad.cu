// GridSampler2DGrad: grad_input (N,C,H,W) and grad_grid (N,Ho,Wo,2) from grad_output (N,C,Ho,Wo), input and grid.
//
// grad_grid is a per-sample sum over channels; every mode computes it with one thread per sample walking the
// channels in order, so it is reproducible and equals the serial reference order.
//
// grad_input is a data-dependent scatter. Two modes:
//   * atomic (default): one thread per sample, channels inner, four fp32 atomics per channel into a zeroed fp32
//     accumulator (grad_input itself for fp32 tensors, workspace for 16-bit tensors, followed by one cast).
//   * deterministic (ACL_OPT_DETERMINISTIC): the scatter is turned into a gather with a fixed summation order.
//       1. count   - how many taps of every chunk of samples land on each input pixel (integer atomics: order-free).
//       2. scan    - prefix sums over chunks (per destination) and over destinations (per image): where each
//                    destination's segment starts, and where inside it each chunk appends.
//       3. fill    - one block per (image, chunk) appends the chunk's taps to the segments in the order in which
//                    the reference's deterministic kernel replays them (256-sample steps; inside a step tap NW, NE,
//                    SW, SE; inside a tap ascending sample index). Ranks inside a warp come from
//                    __match_any_sync and the warps of a block take turns, so no sort is needed.
//       4. gather  - per (image, channel group) the group's grad_output planes are staged in shared memory; one
//                    thread per destination pixel adds  weight * grad_output  over its segment in list order and
//                    writes grad_input once. (Planes too large for shared memory gather from global memory.)
//     The summation order per destination is fixed by the data alone, so results are bit-identical from run to
//     run, and equal to a serial replay in the reference's order. The segment lists are built once per call and
//     reused by all channels.
//
// Arithmetic: image/grid_sampler3_d_grad/op_kernel/arch35/grid_sampler3_d_grad_simt_base.h:51-184,
// image/grid_sampler2_d_grad/op_kernel/arch35/grid_sampler2_d_grad_simt.h:64-144,235-290. All arithmetic is fp32.
#include "grid_coords.cuh"
#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

inline uint64_t Align256(uint64_t v) { return (v + 255) & ~static_cast<uint64_t>(255); }

struct GradTaps {
    int32_t x0, y0;
    float ix, iy, mx, my;
    float tnw, tne, tsw, tse;
};

// Taps from source coordinates that SourceIndexSetGrad has already produced (t.ix, t.iy set by the caller).
__device__ __forceinline__ void FinishGradTaps(GradTaps& t, const GridShape& g)
{
    if (g.interp == 0) {
        t.x0 = static_cast<int32_t>(floorf(t.ix));
        t.y0 = static_cast<int32_t>(floorf(t.iy));
        const float xe = Sub(static_cast<float>(t.x0 + 1), t.ix), ye = Sub(static_cast<float>(t.y0 + 1), t.iy);
        const float xw = Sub(t.ix, static_cast<float>(t.x0)), yw = Sub(t.iy, static_cast<float>(t.y0));
        t.tnw = Mul(xe, ye);
        t.tne = Mul(xw, ye);
        t.tsw = Mul(xe, yw);
        t.tse = Mul(xw, yw);
    } else {
        t.x0 = static_cast<int32_t>(rintf(t.ix));
        t.y0 = static_cast<int32_t>(rintf(t.iy));
        t.tnw = 1.0f;
        t.tne = t.tsw = t.tse = 0.0f;
    }
}

__device__ __forceinline__ GradTaps MakeGradTaps(float gx, float gy, const GridShape& g)
{
    GradTaps t;
    t.ix = gs::SourceIndexSetGrad(gx, g.win, g.pad, g.align, &t.mx);
    t.iy = gs::SourceIndexSetGrad(gy, g.hin, g.pad, g.align, &t.my);
    FinishGradTaps(t, g);
    return t;
}

// Bicubic (interp == 2): only un-normalised coordinates (the 4 x 4 neighbourhood keeps negative positions and every
// neighbour goes through the padding mode on its own), taps visited x-outer, y-inner: tap = 4 * i + j is the
// neighbour (floor(ix) - 1 + i, floor(iy) - 1 + j) with weight cx[i] * cy[j]
// (image/grid_sampler2_d_grad/op_kernel/arch35/grid_sampler2_d_grad_simt.h:171-230).
struct CubicTaps {
    float ixF, iyF, mx, my;
    float cx[4], cy[4];
};
__device__ __forceinline__ CubicTaps MakeCubicTaps(float gx, float gy, const GridShape& g)
{
    CubicTaps t;
    const float ix = gs::UnnormalizeSetGrad(gx, g.win, g.align, &t.mx);
    const float iy = gs::UnnormalizeSetGrad(gy, g.hin, g.align, &t.my);
    t.ixF = floorf(ix);
    t.iyF = floorf(iy);
    gs::CubicCoefficients(t.cx, Sub(ix, t.ixF));
    gs::CubicCoefficients(t.cy, Sub(iy, t.iyF));
    return t;
}
__device__ __forceinline__ int32_t CubicDest(const CubicTaps& t, int tap, const GridShape& g)
{
    return gs::BoundedIndex(Add(Sub(t.ixF, 1.0f), static_cast<float>(tap >> 2)),
                            Add(Sub(t.iyF, 1.0f), static_cast<float>(tap & 3)), g.win, g.hin, g.pad, g.align);
}
__device__ __forceinline__ float CubicWeight(const CubicTaps& t, int tap)
{
    const int i = tap >> 2, j = tap & 3; // selected without dynamic indexing of the register arrays
    const float x = i == 0 ? t.cx[0] : (i == 1 ? t.cx[1] : (i == 2 ? t.cx[2] : t.cx[3]));
    const float y = j == 0 ? t.cy[0] : (j == 1 ? t.cy[1] : (j == 2 ? t.cy[2] : t.cy[3]));
    return Mul(x, y);
}

// Source coordinates of every sample, evaluated once instead of once per channel group (staged kernel).
template <typename T>
__global__ void __launch_bounds__(256)
    GridGradCoordsKernel(const T* __restrict__ grid, float2* __restrict__ rec, GridShape g, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; s < total; s += stride) {
        float mx, my;
        const float ix = gs::SourceIndexSetGrad(DType<T>::Load(grid + 2 * s), g.win, g.pad, g.align, &mx);
        const float iy = gs::SourceIndexSetGrad(DType<T>::Load(grid + 2 * s + 1), g.hin, g.pad, g.align, &my);
        rec[s] = make_float2(ix, iy);
    }
}

// One thread per sample; channels inner. ATOMIC_GI: scatter grad_input with fp32 atomics. WANT_GRID: grad_grid.
template <typename T, bool ATOMIC_GI, bool WANT_GRID>
__global__ void __launch_bounds__(kThreads)
    GridGradSampleKernel(const T* __restrict__ go, const T* __restrict__ x, const T* __restrict__ grid,
                         float* __restrict__ acc, T* __restrict__ ggrid, GridShape g, int64_t total)
{
    const int64_t inPlane = static_cast<int64_t>(g.hin) * g.win;
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; s < total; s += stride) {
        const int64_t n = s / outPlane;
        const int64_t p = s - n * outPlane;
        const GradTaps t = MakeGradTaps(DType<T>::Load(grid + 2 * s), DType<T>::Load(grid + 2 * s + 1), g);
        const T* gob = go + n * g.c * outPlane + p;
        const T* xb = x + n * g.c * inPlane;
        float* ab = acc + n * g.c * inPlane;
        if (g.interp == 0) {
            const bool bnw = gs::Within(t.y0, t.x0, g.hin, g.win), bne = gs::Within(t.y0, t.x0 + 1, g.hin, g.win);
            const bool bsw = gs::Within(t.y0 + 1, t.x0, g.hin, g.win),
                       bse = gs::Within(t.y0 + 1, t.x0 + 1, g.hin, g.win);
            const int64_t o = static_cast<int64_t>(t.y0) * g.win + t.x0;
            const float ye = Sub(static_cast<float>(t.y0 + 1), t.iy), xe = Sub(static_cast<float>(t.x0 + 1), t.ix);
            const float yw = Sub(t.iy, static_cast<float>(t.y0)), xw = Sub(t.ix, static_cast<float>(t.x0));
            float gix = 0.0f, giy = 0.0f;
            for (int64_t c = 0; c < g.c; ++c) {
                const float gv = DType<T>::Load(gob + c * outPlane);
                const int64_t base = c * inPlane + o;
                if (bnw) {
                    if (ATOMIC_GI) {
                        atomicAdd(ab + base, Mul(t.tnw, gv));
                    }
                    if (WANT_GRID) {
                        const float v = DType<T>::Load(xb + base);
                        gix = Sub(gix, Mul(Mul(v, ye), gv));
                        giy = Sub(giy, Mul(Mul(v, xe), gv));
                    }
                }
                if (bne) {
                    if (ATOMIC_GI) {
                        atomicAdd(ab + base + 1, Mul(t.tne, gv));
                    }
                    if (WANT_GRID) {
                        const float v = DType<T>::Load(xb + base + 1);
                        gix = Add(gix, Mul(Mul(v, ye), gv));
                        giy = Sub(giy, Mul(Mul(v, xw), gv));
                    }
                }
                if (bsw) {
                    if (ATOMIC_GI) {
                        atomicAdd(ab + base + g.win, Mul(t.tsw, gv));
                    }
                    if (WANT_GRID) {
                        const float v = DType<T>::Load(xb + base + g.win);
                        gix = Sub(gix, Mul(Mul(v, yw), gv));
                        giy = Add(giy, Mul(Mul(v, xe), gv));
                    }
                }
                if (bse) {
                    if (ATOMIC_GI) {
                        atomicAdd(ab + base + g.win + 1, Mul(t.tse, gv));
                    }
                    if (WANT_GRID) {
                        const float v = DType<T>::Load(xb + base + g.win + 1);
                        gix = Add(gix, Mul(Mul(v, yw), gv));
                        giy = Add(giy, Mul(Mul(v, xw), gv));
                    }
                }
            }
            if (WANT_GRID) {
                ggrid[2 * s] = DType<T>::FromF(Mul(t.mx, gix));
                ggrid[2 * s + 1] = DType<T>::FromF(Mul(t.my, giy));
            }
        } else if (g.interp == 2) {
            const float gxv = DType<T>::Load(grid + 2 * s), gyv = DType<T>::Load(grid + 2 * s + 1);
            const CubicTaps ct = MakeCubicTaps(gxv, gyv, g);
            float mxu, myu, gcx[4], gcy[4];
            const float ixu = gs::UnnormalizeSetGrad(gxv, g.win, g.align, &mxu);
            const float iyu = gs::UnnormalizeSetGrad(gyv, g.hin, g.align, &myu);
            gs::CubicCoefficientsGrad(gcx, Sub(ixu, ct.ixF));
            gs::CubicCoefficientsGrad(gcy, Sub(iyu, ct.iyF));
            float gix = 0.0f, giy = 0.0f;
            for (int64_t c = 0; c < g.c; ++c) {
                const float gv = DType<T>::Load(gob + c * outPlane);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int32_t o = CubicDest(ct, 4 * i + j, g);
                        if (ATOMIC_GI && o >= 0) { // grad_output * cx * cy, in this order (:216-217)
                            atomicAdd(ab + c * inPlane + o, Mul(Mul(gv, ct.cx[i]), ct.cy[j]));
                        }
                        if (WANT_GRID) {
                            const float v = o >= 0 ? DType<T>::Load(xb + c * inPlane + o) : 0.0f;
                            gix = Add(gix, Mul(Mul(Mul(v, gcx[i]), ct.cy[j]), gv));
                            giy = Add(giy, Mul(Mul(Mul(v, gcy[j]), ct.cx[i]), gv));
                        }
                    }
                }
            }
            if (WANT_GRID) {
                ggrid[2 * s] = DType<T>::FromF(Mul(ct.mx, gix));
                ggrid[2 * s + 1] = DType<T>::FromF(Mul(ct.my, giy));
            }
        } else {
            if (ATOMIC_GI && gs::Within(t.y0, t.x0, g.hin, g.win)) {
                const int64_t o = static_cast<int64_t>(t.y0) * g.win + t.x0;
                for (int64_t c = 0; c < g.c; ++c) {
                    atomicAdd(ab + c * inPlane + o, DType<T>::Load(gob + c * outPlane));
                }
            }
            if (WANT_GRID) {
                ggrid[2 * s] = DType<T>::FromF(0.0f);
                ggrid[2 * s + 1] = DType<T>::FromF(0.0f);
            }
        }
    }
}

// Copies `nch` planes of `count` elements each (plane k at src + k * planeStride) into shared memory interleaved by
// channel, tile[i] = {CG channels} (zeros past nch). The loads of several elements per thread (32 scalar loads at
// most) are issued before the first store, so a block that has an SM to itself does not pay one memory latency per
// element.
template <typename T, int CG>
__device__ __forceinline__ void StageInterleaved(Pack<T, CG>* tile, const T* __restrict__ src, int64_t planeStride,
                                                 int32_t nch, int32_t count)
{
    constexpr int kBatch = CG >= 8 ? 4 : 8;
    const int32_t step = blockDim.x;
    for (int32_t base = threadIdx.x; base < count; base += step * kBatch) {
        Pack<T, CG> v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int32_t i = base + u * step;
#pragma unroll
            for (int k = 0; k < CG; ++k) {
                v[u].v[k] = (i < count && k < nch) ? __ldg(src + k * planeStride + i) : DType<T>::FromF(0.0f);
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int32_t i = base + u * step;
            if (i < count) {
                tile[i] = v[u];
            }
        }
    }
}

// ---- deterministic mode --------------------------------------------------------------------------------------
struct Entry {
    int32_t sample; // pixel index inside the image's output plane
    float weight;
};

__device__ __forceinline__ int32_t TapDest(const GradTaps& t, int tap, const GridShape& g)
{
    const int32_t yy = t.y0 + (tap >> 1), xx = t.x0 + (tap & 1);
    if (g.interp != 0 && tap != 0) {
        return -1;
    }
    return gs::Within(yy, xx, g.hin, g.win) ? yy * g.win + xx : -1;
}

// The reference's deterministic kernel stages the contributions of 256 consecutive samples and lets one thread
// replay them tap by tap (grid_sampler2_d_grad_simt_det.h:78-106, VF_MAX_THREAD_NUM = 256), so per destination
// the order is: 256-sample step, then tap (NW, NE, SW, SE), then sample index. The lists keep that order.
constexpr int kDetStep = 256;

// counts[(n * chunks + c) * inPlane + d] = taps of the samples of chunk c of image n that land on destination d.
// A chunk is `chunkSamples` consecutive samples (a multiple of kDetStep).
// CUBIC: the bicubic variant (16 taps per sample); a template flag so that the bilinear / nearest kernels carry none
// of its registers.
template <typename T, bool CUBIC>
__global__ void __launch_bounds__(kThreads)
    DetCountKernel(const T* __restrict__ grid, int32_t* __restrict__ counts, GridShape g, int32_t chunks,
                   int32_t chunkSamples, int64_t total)
{
    const int64_t inPlane = static_cast<int64_t>(g.hin) * g.win;
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; s < total; s += stride) {
        const int64_t n = s / outPlane;
        const int64_t c = (s - n * outPlane) / chunkSamples;
        int32_t* cnt = counts + (n * chunks + c) * inPlane;
        if constexpr (CUBIC) {
            const CubicTaps ct = MakeCubicTaps(DType<T>::Load(grid + 2 * s), DType<T>::Load(grid + 2 * s + 1), g);
#pragma unroll
            for (int tap = 0; tap < 16; ++tap) {
                const int32_t d = CubicDest(ct, tap, g);
                if (d >= 0) {
                    atomicAdd(cnt + d, 1);
                }
            }
            continue;
        }
        const GradTaps t = MakeGradTaps(DType<T>::Load(grid + 2 * s), DType<T>::Load(grid + 2 * s + 1), g);
#pragma unroll
        for (int tap = 0; tap < 4; ++tap) {
            const int32_t d = TapDest(t, tap, g);
            if (d >= 0) {
                atomicAdd(cnt + d, 1);
            }
        }
    }
}

// Turns the per-chunk counts into list positions, in two steps.
// Column step (one thread per (image, destination)): counts[n][c][d] becomes the number of entries that earlier
// chunks append to destination d, and segStart[n][d] the destination's total.
__global__ void __launch_bounds__(kThreads)
    DetColumnKernel(int32_t* __restrict__ counts, int32_t* __restrict__ segStart, int64_t inPlane, int32_t chunks,
                    int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t n = i / inPlane;
        const int64_t d = i - n * inPlane;
        int32_t* cnt = counts + n * chunks * inPlane + d;
        int32_t run = 0;
        for (int32_t c0 = 0; c0 < chunks; c0 += 8) { // eight independent loads per trip, then the running sum
            int32_t t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                t[u] = c0 + u < chunks ? cnt[(c0 + u) * inPlane] : 0;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (c0 + u < chunks) {
                    cnt[(c0 + u) * inPlane] = run;
                    run += t[u];
                }
            }
        }
        segStart[n * (inPlane + 1) + d] = run;
    }
}

// Segment step (one block per image): exclusive prefix sum of the totals in place; segStart[n][inPlane] = number of
// entries of the image.
__global__ void __launch_bounds__(1024) DetScanKernel(int32_t* __restrict__ segStart, int64_t inPlane)
{
    __shared__ int32_t warpSums[32];
    __shared__ int32_t carry;
    int32_t* seg = segStart + static_cast<int64_t>(blockIdx.x) * (inPlane + 1);
    if (threadIdx.x == 0) {
        carry = 0;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t base = 0; base < inPlane; base += blockDim.x) {
        const int64_t d = base + threadIdx.x;
        const int32_t v = d < inPlane ? seg[d] : 0;
        int32_t incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) {
                incl += up;
            }
        }
        if (lane == 31) {
            warpSums[warp] = incl;
        }
        __syncthreads();
        if (warp == 0) {
            int32_t ws = lane < (blockDim.x >> 5) ? warpSums[lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int32_t up = __shfl_up_sync(0xffffffffu, ws, o);
                if (lane >= o) {
                    ws += up;
                }
            }
            warpSums[lane] = ws; // inclusive over warps
        }
        __syncthreads();
        const int32_t warpOffset = warp == 0 ? 0 : warpSums[warp - 1];
        const int32_t excl = carry + warpOffset + incl - v;
        if (d < inPlane) {
            seg[d] = excl;
        }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) {
            carry = excl + v;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        seg[inPlane] = carry;
    }
}

// One block of kDetStep threads per (image, chunk). The block appends the taps of its chunk to the destination
// segments in list order: 256-sample step by step; inside a step tap by tap; inside a tap the eight warps take turns
// (a barrier between turns), and inside a warp the rank among lanes with the same destination comes from
// __match_any_sync, so the position of every entry is a function of the data alone. The running positions live in
// shared memory when the plane fits (cursorInSmem), else in the chunk's own slice of the offsets array.
template <typename T, bool CUBIC>
__global__ void __launch_bounds__(kDetStep)
    DetFillKernel(const T* __restrict__ grid, int32_t* offsets, const int32_t* __restrict__ segStart,
                  Entry* __restrict__ entries, GridShape g, int32_t chunks, int32_t chunkSamples,
                  int64_t entriesPerImage, int32_t cursorInSmem)
{
    extern __shared__ int32_t cursorSmem[];
    const int32_t inPlane = g.hin * g.win;
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int64_t n = blockIdx.x / chunks;
    const int32_t c = static_cast<int32_t>(blockIdx.x - n * chunks);
    int32_t* off = offsets + (n * chunks + c) * static_cast<int64_t>(inPlane);
    // running position = start of the destination's segment + what earlier chunks append to it
    const int32_t* seg = segStart + n * (static_cast<int64_t>(inPlane) + 1);
    for (int32_t i = threadIdx.x; i < inPlane; i += blockDim.x) {
        if (cursorInSmem) {
            cursorSmem[i] = off[i] + seg[i];
        } else {
            off[i] += seg[i];
        }
    }
    __syncthreads();
    volatile int32_t* cur = cursorInSmem ? cursorSmem : off;
    Entry* ent = entries + n * entriesPerImage;
    const T* gb = grid + 2 * n * outPlane;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned lower = (1u << lane) - 1u;
    const int64_t p0 = static_cast<int64_t>(c) * chunkSamples, p1 = min(outPlane, p0 + chunkSamples);
    const int numTaps = CUBIC ? 16 : (g.interp == 0 ? 4 : 1);
    for (int64_t base = p0; base < p1; base += kDetStep) {
        const int64_t p = base + threadIdx.x;
        GradTaps t{};
        CubicTaps ct{};
        t.x0 = INT32_MIN / 2; // far out of bounds: a thread past the end has no tap in range
        t.y0 = INT32_MIN / 2;
        if (p < p1) {
            if constexpr (CUBIC) {
                ct = MakeCubicTaps(DType<T>::Load(gb + 2 * p), DType<T>::Load(gb + 2 * p + 1), g);
            } else {
                t = MakeGradTaps(DType<T>::Load(gb + 2 * p), DType<T>::Load(gb + 2 * p + 1), g);
            }
        }
        for (int tap = 0; tap < numTaps; ++tap) {
            int32_t d;
            float wgt;
            if constexpr (CUBIC) {
                d = p < p1 ? CubicDest(ct, tap, g) : -1;
                wgt = CubicWeight(ct, tap); // the deterministic kernel multiplies grad_output by cx * cy (:312-314)
            } else {
                d = TapDest(t, tap, g);
                wgt = tap == 0 ? t.tnw : (tap == 1 ? t.tne : (tap == 2 ? t.tsw : t.tse));
            }
            for (int turn = 0; turn < kDetStep / 32; ++turn) {
                if (warp == turn) {
                    // lanes without a tap get a key no other lane has: they match only themselves
                    const unsigned peers = __match_any_sync(0xffffffffu, d >= 0 ? d : -1 - lane);
                    int32_t start = 0;
                    if (d >= 0) {
                        start = cur[d];
                        ent[start + __popc(peers & lower)] = Entry{static_cast<int32_t>(p), wgt};
                    }
                    __syncwarp();
                    if (d >= 0 && (peers & lower) == 0) { // lowest lane of each group advances the position
                        cur[d] = start + __popc(peers);
                    }
                }
                __syncthreads();
            }
        }
    }
}

// Gather with grad_output staged in shared memory: one block per (image, group of CG channels) copies the group's
// grad_output planes into shared memory as tile[sample] = {CG channels}; then one thread per destination pixel adds
// weight * grad_output over the destination's segment, in list order, and writes grad_input once.
template <typename T, int CG>
__global__ void __launch_bounds__(1024)
    DetGatherStagedKernel(const T* __restrict__ go, const int32_t* __restrict__ segStart,
                          const Entry* __restrict__ entries, T* __restrict__ gi, GridShape g, int32_t groups,
                          int64_t entriesPerImage)
{
    extern __shared__ __align__(16) unsigned char stagedSmem[];
    using Vec = Pack<T, CG>;
    Vec* tile = reinterpret_cast<Vec*>(stagedSmem);
    const int32_t inPlane = g.hin * g.win, outPlane = g.hout * g.wout;
    const int64_t n = blockIdx.x / groups;
    const int32_t c0 = static_cast<int32_t>(blockIdx.x - n * groups) * CG;
    const int32_t nch = min(CG, static_cast<int32_t>(g.c) - c0);
    const T* gob = go + (n * g.c + c0) * outPlane;
    StageInterleaved<T, CG>(tile, gob, outPlane, nch, outPlane);
    __syncthreads();
    const int32_t* seg = segStart + n * (inPlane + 1);
    const Entry* ent = entries + n * entriesPerImage;
    T* gib = gi + (n * g.c + c0) * inPlane;
    for (int32_t d = threadIdx.x; d < inPlane; d += blockDim.x) {
        const int32_t a = __ldg(seg + d), b = __ldg(seg + d + 1);
        float acc[CG];
#pragma unroll
        for (int k = 0; k < CG; ++k) {
            acc[k] = 0.0f;
        }
        // Every lane walks its own segment, so the entry loads of a warp are scattered: 16-byte loads (two entries)
        // halve their count. Four pairs per trip are loaded before the first use; additions stay in list order.
        auto add = [&](int32_t sample, float wgt) {
            const Vec v = tile[sample];
            float vf[CG];
            UnpackToF<T, CG>(v, vf);
#pragma unroll
            for (int k = 0; k < CG; ++k) {
                acc[k] = Add(acc[k], Mul(wgt, vf[k]));
            }
        };
        int32_t e = a;
        if (e < b && (e & 1)) { // segments start at any entry; pairs are 16-byte aligned at even indices
            const int2 r = __ldg(reinterpret_cast<const int2*>(ent + e));
            add(r.x, __int_as_float(r.y));
            ++e;
        }
        constexpr int kPairs = 4;
        for (; e < b; e += 2 * kPairs) {
            int4 raw[kPairs];
#pragma unroll
            for (int u = 0; u < kPairs; ++u) {
                const int32_t q = e + 2 * u;
                if (q + 1 < b) {
                    raw[u] = __ldg(reinterpret_cast<const int4*>(ent + q));
                } else if (q < b) {
                    const int2 r = __ldg(reinterpret_cast<const int2*>(ent + q));
                    raw[u] = make_int4(r.x, r.y, 0, 0);
                } else {
                    raw[u] = make_int4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < kPairs; ++u) {
                const int32_t q = e + 2 * u;
                if (q < b) {
                    add(raw[u].x, __int_as_float(raw[u].y));
                }
                if (q + 1 < b) {
                    add(raw[u].z, __int_as_float(raw[u].w));
                }
            }
        }
#pragma unroll
        for (int k = 0; k < CG; ++k) {
            if (k < nch) {
                gib[static_cast<int64_t>(k) * inPlane + d] = DType<T>::FromF(acc[k]);
            }
        }
    }
}

// One thread per (image, channel group, destination pixel); consecutive threads -> consecutive destinations.
template <typename T, int CG>
__global__ void __launch_bounds__(kThreads)
    DetGatherKernel(const T* __restrict__ go, const int32_t* __restrict__ offsets, const Entry* __restrict__ entries,
                    T* __restrict__ gi, GridShape g, int32_t chanGroups, int64_t entriesPerImage, int64_t total)
{
    const int64_t inPlane = static_cast<int64_t>(g.hin) * g.win;
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t ng = idx / inPlane;
        const int64_t d = idx - ng * inPlane;
        const int64_t n = ng / chanGroups;
        const int32_t cg = static_cast<int32_t>(ng - n * chanGroups);
        const int64_t c0 = static_cast<int64_t>(cg) * CG;
        const int32_t* off = offsets + n * (inPlane + 1);
        const int32_t a = __ldg(off + d), b = __ldg(off + d + 1);
        const Entry* ent = entries + n * entriesPerImage;
        const T* gob = go + (n * g.c + c0) * outPlane;
        float acc[CG];
#pragma unroll
        for (int k = 0; k < CG; ++k) {
            acc[k] = 0.0f;
        }
        for (int32_t e = a; e < b; ++e) {
            const int2 raw = __ldg(reinterpret_cast<const int2*>(ent + e));
            const float wgt = __int_as_float(raw.y);
            const T* gs_ = gob + raw.x;
#pragma unroll
            for (int k = 0; k < CG; ++k) {
                if (c0 + k < g.c) {
                    acc[k] = Add(acc[k], Mul(wgt, DType<T>::Load(gs_ + k * outPlane)));
                }
            }
        }
        T* gib = gi + (n * g.c + c0) * inPlane + d;
#pragma unroll
        for (int k = 0; k < CG; ++k) {
            if (c0 + k < g.c) {
                gib[k * inPlane] = DType<T>::FromF(acc[k]);
            }
        }
    }
}

// ---- staged kernel (bilinear, atomic mode) ---------------------------------------------------------------------
// One block per (image, group of CG channels). Shared memory holds the group's grad_input planes as fp32
// accumulators, acc[k * inPlane + y * win + x] (planar: the lanes of a warp scatter to random pixels of ONE channel
// per instruction, and a planar plane spreads them over all 32 banks), and (for grad_grid) the group's input planes
// interleaved by channel, tile[y * win + x] = {CG channels}.
// Threads walk the output pixels of the image: grad_output is read coalesced, the scatter goes to shared-memory
// atomics, the input taps come from shared memory. At the end the accumulators are written to grad_input once, in
// the storage dtype: no zero-fill of grad_input, no global atomics on it, no fp32 staging buffer for 16-bit tensors.
// grad_grid needs the sum over ALL channels: every block adds its group's partial (gix, giy) to an fp32 buffer with
// one 8-byte global atomic per pixel (or, in the reproducible mode, stores it in the group's own slice of a partial
// buffer); GridGradFinishKernel adds the partials in group order, scales by the coordinate multipliers and stores.
template <typename T, int CG, bool WANT_IN, bool WANT_GRID>
__global__ void __launch_bounds__(1024)
    GridGradStagedKernel(const T* __restrict__ go, const T* __restrict__ x, const float2* __restrict__ rec,
                         T* __restrict__ gi, float2* __restrict__ ggAcc, GridShape g, int32_t groups,
                         int64_t partStride)
{
    extern __shared__ __align__(16) unsigned char stagedSmem[];
    using Vec = Pack<T, CG>;
    const int32_t inPlane = g.hin * g.win, outPlane = g.hout * g.wout;
    float* acc = reinterpret_cast<float*>(stagedSmem);
    Vec* tile = reinterpret_cast<Vec*>(stagedSmem + (WANT_IN ? static_cast<size_t>(inPlane) * CG * sizeof(float) : 0));
    const int64_t n = blockIdx.x / groups;
    const int32_t c0 = static_cast<int32_t>(blockIdx.x - n * groups) * CG;
    const int32_t nch = min(CG, static_cast<int32_t>(g.c) - c0);
    if (WANT_IN) {
        for (int32_t i = threadIdx.x; i < inPlane * CG; i += blockDim.x) {
            acc[i] = 0.0f;
        }
    }
    if (WANT_GRID) {
        StageInterleaved<T, CG>(tile, x + (n * g.c + c0) * inPlane, inPlane, nch, inPlane);
    }
    __syncthreads();
    const float2* rb = rec + n * outPlane;
    const T* gob = go + (n * g.c + c0) * outPlane;
    for (int32_t p = threadIdx.x; p < outPlane; p += blockDim.x) {
        const float2 r = __ldg(rb + p);
        GradTaps t;
        t.ix = r.x;
        t.iy = r.y;
        FinishGradTaps(t, g);
        float gv[CG];
#pragma unroll
        for (int k = 0; k < CG; ++k) {
            gv[k] = k < nch ? DType<T>::Load(gob + static_cast<int64_t>(k) * outPlane + p) : 0.0f;
        }
        const int32_t o = t.y0 * g.win + t.x0;
        const float ye = Sub(static_cast<float>(t.y0 + 1), t.iy), xe = Sub(static_cast<float>(t.x0 + 1), t.ix);
        const float yw = Sub(t.iy, static_cast<float>(t.y0)), xw = Sub(t.ix, static_cast<float>(t.x0));
        float gix = 0.0f, giy = 0.0f;
        // sx / sy: sign of the tap's term in d/dx and d/dy; fx / fy: the factor (ye or yw, xe or xw).
        auto tap = [&](bool in, int32_t off, float w, float fx, float fy, bool negX, bool negY) {
            if (!in) {
                return;
            }
            const int32_t d = o + off;
            float xf[CG] = {};
            if (WANT_GRID) {
                const Vec v = tile[d];
                UnpackToF<T, CG>(v, xf);
            }
#pragma unroll
            for (int k = 0; k < CG; ++k) {
                if (k < nch) {
                    if (WANT_IN) {
                        atomicAdd(acc + k * inPlane + d, Mul(w, gv[k]));
                    }
                    if (WANT_GRID) {
                        const float xv = xf[k];
                        const float tx = Mul(Mul(xv, fx), gv[k]), ty = Mul(Mul(xv, fy), gv[k]);
                        gix = negX ? Sub(gix, tx) : Add(gix, tx);
                        giy = negY ? Sub(giy, ty) : Add(giy, ty);
                    }
                }
            }
        };
        tap(gs::Within(t.y0, t.x0, g.hin, g.win), 0, t.tnw, ye, xe, true, true);
        tap(gs::Within(t.y0, t.x0 + 1, g.hin, g.win), 1, t.tne, ye, xw, false, true);
        tap(gs::Within(t.y0 + 1, t.x0, g.hin, g.win), g.win, t.tsw, yw, xe, true, false);
        tap(gs::Within(t.y0 + 1, t.x0 + 1, g.hin, g.win), g.win + 1, t.tse, yw, xw, false, false);
        if (WANT_GRID) {
            if (partStride > 0) { // reproducible mode: every group keeps its own partial sums
                ggAcc[(blockIdx.x - n * groups) * partStride + n * outPlane + p] = make_float2(gix, giy);
            } else {
                atomicAdd(ggAcc + n * outPlane + p, make_float2(gix, giy));
            }
        }
    }
    if (WANT_IN) {
        __syncthreads();
        T* gib = gi + (n * g.c + c0) * inPlane;
        for (int32_t i = threadIdx.x; i < inPlane; i += blockDim.x) {
#pragma unroll
            for (int k = 0; k < CG; ++k) {
                if (k < nch) {
                    gib[static_cast<int64_t>(k) * inPlane + i] = DType<T>::FromF(acc[k * inPlane + i]);
                }
            }
        }
    }
}

// grad_grid = multiplier * (sum over channels), from the fp32 sums of the staged kernel.
template <typename T>
__global__ void __launch_bounds__(kThreads)
    GridGradFinishKernel(const T* __restrict__ grid, const float2* __restrict__ ggAcc, T* __restrict__ ggrid,
                         GridShape g, int64_t total, int32_t parts, int64_t partStride)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; s < total; s += stride) {
        float mx, my;
        gs::SourceIndexSetGrad(DType<T>::Load(grid + 2 * s), g.win, g.pad, g.align, &mx);
        gs::SourceIndexSetGrad(DType<T>::Load(grid + 2 * s + 1), g.hin, g.pad, g.align, &my);
        float2 a = ggAcc[s];
        for (int32_t q = 1; q < parts; ++q) {
            const float2 b = ggAcc[q * partStride + s];
            a.x = Add(a.x, b.x);
            a.y = Add(a.y, b.y);
        }
        ggrid[2 * s] = DType<T>::FromF(Mul(mx, a.x));
        ggrid[2 * s + 1] = DType<T>::FromF(Mul(my, a.y));
    }
}

// Bytes of shared memory per block of the staged kernel for a group of cg channels.
inline size_t StagedBwdSmem(int es, int64_t inPlane, int cg, bool wantInput, bool wantGrid)
{
    return static_cast<size_t>(inPlane) * cg * ((wantInput ? 4 : 0) + (wantGrid ? es : 0));
}

// Group width for the staged kernel: the widest that fits the shared memory of an SM (0: none does).
inline int32_t StagedBwdGroup(int es, int64_t inPlane, int64_t c, bool wantInput, bool wantGrid)
{
    for (int cg = 16 / es; cg * es >= 4; cg /= 2) {
        if (StagedBwdSmem(es, inPlane, cg, wantInput, wantGrid) <= 220 * 1024 && (cg == 1 || cg / 2 < c)) {
            return cg;
        }
    }
    return 0;
}

template <typename T, int CG>
cudaError_t LaunchStagedBwd(const T* go, const T* x, const T* grid, T* gi, T* ggrid, float2* ggAcc, float2* rec,
                            GridShape g, bool wantInput, bool wantGrid, bool partials, cudaStream_t s)
{
    struct {
        bool wantInput, wantGrid;
    } plan{wantInput, wantGrid};
    const int64_t inPlane = static_cast<int64_t>(g.hin) * g.win, outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int32_t groups = static_cast<int32_t>(CeilDiv(g.c, CG));
    const size_t smem = StagedBwdSmem(sizeof(T), inPlane, CG, plan.wantInput, plan.wantGrid);
    const int threads = smem <= 110 * 1024 ? 512 : 1024;
    cudaError_t e = cudaSuccess;
    GridGradCoordsKernel<T><<<GridFor(g.n * outPlane, 256), 256, 0, s>>>(grid, rec, g, g.n * outPlane);
    CountLaunch();
    const int64_t partStride = partials ? g.n * outPlane : 0;
    if (plan.wantGrid && !partials) {
        e = cudaMemsetAsync(ggAcc, 0, static_cast<size_t>(g.n * outPlane) * sizeof(float2), s);
        if (e != cudaSuccess) {
            return e;
        }
        CountLaunch();
    }
    auto launch = [&](auto kernel) {
        if (smem > 48 * 1024) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (e != cudaSuccess) {
                return;
            }
        }
        kernel<<<static_cast<unsigned>(g.n * groups), threads, smem, s>>>(go, x, rec, gi, ggAcc, g, groups,
                                                                          partStride);
        CountLaunch();
        e = cudaGetLastError();
    };
    if (plan.wantInput && plan.wantGrid) {
        launch(GridGradStagedKernel<T, CG, true, true>);
    } else if (plan.wantInput) {
        launch(GridGradStagedKernel<T, CG, true, false>);
    } else {
        launch(GridGradStagedKernel<T, CG, false, true>);
    }
    if (e == cudaSuccess && plan.wantGrid) {
        const int64_t samples = g.n * outPlane;
        GridGradFinishKernel<T><<<GridFor(samples, kThreads), kThreads, 0, s>>>(grid, ggAcc, ggrid, g, samples,
                                                                                partials ? groups : 1, partStride);
        CountLaunch();
        e = cudaGetLastError();
    }
    return e;
}

} // namespace

GridGradPlan PlanGridSampler2DBwd(Dt dt, GridShape g, bool deterministic, bool wantInput, bool wantGrid)
{
    GridGradPlan p{};
    p.deterministic = deterministic;
    p.wantInput = wantInput;
    p.wantGrid = wantGrid;
    const uint64_t inPlane = static_cast<uint64_t>(g.hin) * g.win;
    const uint64_t outPlane = static_cast<uint64_t>(g.hout) * g.wout;
    // Staged kernel: bilinear, atomic mode, planes that fit shared memory, enough (image, group) blocks to occupy
    // the machine, and an image with at least as many output pixels as a plane has inputs.
    if (!deterministic && g.interp == 0 && (wantInput || wantGrid) && outPlane < (1ULL << 30)) {
        const int32_t cg = StagedBwdGroup(DtSize(dt), static_cast<int64_t>(inPlane), g.c, wantInput, wantGrid);
        if (cg > 0 && g.n * CeilDiv(g.c, cg) >= NumSMs() / 2 && outPlane * 2 >= inPlane &&
            g.n * CeilDiv(g.c, cg) < (1LL << 31)) {
            p.stagedGroup = cg;
            p.gridAccBytes = wantGrid ? Align256(static_cast<uint64_t>(g.n) * outPlane * 8) : 0;
            p.recBytes = Align256(static_cast<uint64_t>(g.n) * outPlane * 8);
            p.total = p.gridAccBytes + p.recBytes;
            return p;
        }
    }
    if (wantInput) {
        if (deterministic) {
            // Chunks of the sample sequence get their own append positions, so that they can be filled in
            // parallel. Start from one 256-sample step per chunk and coarsen while the positions
            // [N][chunks][inPlane] would exceed 256 MB.
            int64_t chunkSamples = kDetStep;
            int64_t chunks = CeilDiv(static_cast<int64_t>(outPlane), chunkSamples);
            while (chunks > 1 && static_cast<uint64_t>(g.n) * chunks * inPlane * 4 > (256ULL << 20)) {
                chunkSamples *= 2;
                chunks = CeilDiv(static_cast<int64_t>(outPlane), chunkSamples);
            }
            p.detChunks = static_cast<int32_t>(chunks);
            p.detChunkSamples = static_cast<int32_t>(chunkSamples);
            p.detCursorSmem = inPlane * 4 <= 200 * 1024;
            // gather with grad_output in shared memory: the widest channel vector whose planes fit (every block
            // reads the whole entry list of its image from L2, so fewer, wider groups win over more resident blocks)
            p.detGatherGroup = 0;
            const int es = DtSize(dt);
            for (int cg = 16 / es; cg * es >= 4 && outPlane < (1ULL << 30); cg /= 2) {
                if (outPlane * cg * es <= 220ULL * 1024 && (cg == 1 || cg / 2 < g.c)) {
                    p.detGatherGroup = cg;
                    break;
                }
            }
            // positions [N][chunks][inPlane] and segment starts [N][inPlane+1], then entries [N][4*outPlane]
            p.countBytes = Align256(static_cast<uint64_t>(g.n) * chunks * inPlane * 4) +
                           Align256(static_cast<uint64_t>(g.n) * (inPlane + 1) * 4);
            p.entryBytes = Align256(static_cast<uint64_t>(g.n) * (g.interp == 2 ? 16 : 4) * outPlane * sizeof(Entry));
        } else if (dt != Dt::F32) {
            p.accBytes = Align256(static_cast<uint64_t>(g.n) * g.c * inPlane * 4);
        }
    }
    if (deterministic && wantGrid && g.interp == 0 && outPlane < (1ULL << 30)) {
        // grad_grid from the staged kernel with per-group partial sums added in group order (needs
        // [groups][N * outPlane] float2; the per-sample kernel is the fallback)
        const int32_t cg = StagedBwdGroup(DtSize(dt), static_cast<int64_t>(inPlane), g.c, false, true);
        if (cg > 0 && g.n * CeilDiv(g.c, cg) >= NumSMs() / 2 && g.n * CeilDiv(g.c, cg) < (1LL << 31) &&
            static_cast<uint64_t>(CeilDiv(g.c, cg)) * g.n * outPlane * 8 <= (1ULL << 30)) {
            p.detGridGroup = cg;
            p.gridAccBytes = Align256(static_cast<uint64_t>(CeilDiv(g.c, cg)) * g.n * outPlane * 8);
            p.recBytes = Align256(static_cast<uint64_t>(g.n) * outPlane * 8);
        }
    }
    p.total = p.gridAccBytes + p.accBytes + p.countBytes + p.entryBytes + p.recBytes;
    return p;
}

cudaError_t GridSampler2DBwd(Dt dt, const void* go, const void* x, const void* grid, void* gi, void* ggrid,
                             GridShape g, const GridGradPlan& plan, void* workspace, cudaStream_t s)
{
    const int64_t inPlane = static_cast<int64_t>(g.hin) * g.win;
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int64_t samples = g.n * outPlane;
    const int64_t giElems = g.n * g.c * inPlane;
    cudaError_t e = cudaSuccess;
    char* ws = static_cast<char*>(workspace);
    // per-sample source coordinates of the staged kernels: always the last piece of the workspace
    float2* recs = plan.recBytes > 0 ? reinterpret_cast<float2*>(ws + plan.total - plan.recBytes) : nullptr;

    if (plan.stagedGroup > 0) {
        OPSCV_DISPATCH_DT(dt, T, {
            const T* pgo = static_cast<const T*>(go);
            const T* px = static_cast<const T*>(x);
            const T* pg = static_cast<const T*>(grid);
            T* pgi = static_cast<T*>(gi);
            T* pgg = static_cast<T*>(ggrid);
            float2* ggAcc = reinterpret_cast<float2*>(ws);
            constexpr int kMax = 16 / sizeof(T);
            if (plan.stagedGroup == kMax) {
                e = LaunchStagedBwd<T, kMax>(pgo, px, pg, pgi, pgg, ggAcc, recs, g, plan.wantInput, plan.wantGrid, false, s);
            } else if (plan.stagedGroup == kMax / 2) {
                e = LaunchStagedBwd<T, kMax / 2>(pgo, px, pg, pgi, pgg, ggAcc, recs, g, plan.wantInput, plan.wantGrid, false, s);
            } else {
                e = LaunchStagedBwd<T, kMax / 4>(pgo, px, pg, pgi, pgg, ggAcc, recs, g, plan.wantInput, plan.wantGrid, false, s);
            }
        });
        return e;
    }

    if (plan.deterministic && !plan.wantInput && plan.detGridGroup > 0) {
        OPSCV_DISPATCH_DT(dt, T, {
            const T* pgo = static_cast<const T*>(go);
            const T* px = static_cast<const T*>(x);
            const T* pg = static_cast<const T*>(grid);
            T* pgg = static_cast<T*>(ggrid);
            float2* parts = reinterpret_cast<float2*>(ws);
            constexpr int kMax = 16 / sizeof(T);
            if (plan.detGridGroup == kMax) {
                e = LaunchStagedBwd<T, kMax>(pgo, px, pg, nullptr, pgg, parts, recs, g, false, true, true, s);
            } else if (plan.detGridGroup == kMax / 2) {
                e = LaunchStagedBwd<T, kMax / 2>(pgo, px, pg, nullptr, pgg, parts, recs, g, false, true, true, s);
            } else {
                e = LaunchStagedBwd<T, kMax / 4>(pgo, px, pg, nullptr, pgg, parts, recs, g, false, true, true, s);
            }
        });
        return e;
    }

    if (!plan.deterministic || !plan.wantInput) {
        float* acc = nullptr;
        if (plan.wantInput) {
            acc = dt == Dt::F32 ? static_cast<float*>(gi) : reinterpret_cast<float*>(ws);
            e = cudaMemsetAsync(acc, 0, static_cast<size_t>(giElems) * sizeof(float), s);
            if (e != cudaSuccess) {
                return e;
            }
            CountLaunch();
        }
        OPSCV_DISPATCH_DT(dt, T, {
            const unsigned blocks = GridFor(samples, kThreads, 16);
            const T* pgo = static_cast<const T*>(go);
            const T* px = static_cast<const T*>(x);
            const T* pg = static_cast<const T*>(grid);
            T* pgg = static_cast<T*>(ggrid);
            if (plan.wantInput && plan.wantGrid) {
                GridGradSampleKernel<T, true, true><<<blocks, kThreads, 0, s>>>(pgo, px, pg, acc, pgg, g, samples);
            } else if (plan.wantInput) {
                GridGradSampleKernel<T, true, false><<<blocks, kThreads, 0, s>>>(pgo, px, pg, acc, pgg, g, samples);
            } else {
                GridGradSampleKernel<T, false, true><<<blocks, kThreads, 0, s>>>(pgo, px, pg, acc, pgg, g, samples);
            }
        });
        CountLaunch();
        e = cudaGetLastError();
        if (e != cudaSuccess) {
            return e;
        }
        if (plan.wantInput && dt != Dt::F32) {
            return CastFromF32(dt, gi, acc, giElems, s);
        }
        return cudaSuccess;
    }

    // deterministic grad_input
    const uint64_t posBytes = Align256(static_cast<uint64_t>(g.n) * plan.detChunks * inPlane * 4);
    int32_t* positions = reinterpret_cast<int32_t*>(ws);
    int32_t* segStart = reinterpret_cast<int32_t*>(ws + posBytes);
    Entry* entries = reinterpret_cast<Entry*>(ws + plan.countBytes);
    const int64_t entriesPerImage = (g.interp == 2 ? 16 : 4) * outPlane;
    e = cudaMemsetAsync(positions, 0, static_cast<size_t>(g.n) * plan.detChunks * inPlane * 4, s);
    if (e != cudaSuccess) {
        return e;
    }
    CountLaunch();
    OPSCV_DISPATCH_DT(dt, T, {
        const T* pgo = static_cast<const T*>(go);
        const T* px = static_cast<const T*>(x);
        const T* pg = static_cast<const T*>(grid);
        T* pgi = static_cast<T*>(gi);
        if (g.interp == 2) {
            DetCountKernel<T, true><<<GridFor(samples, kThreads), kThreads, 0, s>>>(pg, positions, g, plan.detChunks,
                                                                                    plan.detChunkSamples, samples);
        } else {
            DetCountKernel<T, false><<<GridFor(samples, kThreads), kThreads, 0, s>>>(pg, positions, g, plan.detChunks,
                                                                                     plan.detChunkSamples, samples);
        }
        DetColumnKernel<<<GridFor(g.n * inPlane, kThreads), kThreads, 0, s>>>(positions, segStart, inPlane,
                                                                              plan.detChunks, g.n * inPlane);
        DetScanKernel<<<static_cast<unsigned>(g.n), 1024, 0, s>>>(segStart, inPlane);
        const size_t cursorBytes = plan.detCursorSmem ? static_cast<size_t>(inPlane) * 4 : 0;
        auto fill = [&](auto kernel) {
            if (cursorBytes > 48 * 1024) {
                e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(cursorBytes));
            }
            if (e == cudaSuccess) {
                kernel<<<static_cast<unsigned>(g.n * plan.detChunks), kDetStep, cursorBytes, s>>>(
                    pg, positions, segStart, entries, g, plan.detChunks, plan.detChunkSamples, entriesPerImage,
                    plan.detCursorSmem ? 1 : 0);
            }
        };
        if (g.interp == 2) {
            fill(DetFillKernel<T, true>);
        } else {
            fill(DetFillKernel<T, false>);
        }
        CountLaunch(4);
        if (e == cudaSuccess && plan.detGatherGroup > 0) {
            auto gather = [&](auto kernel, int cg) {
                const size_t smem = static_cast<size_t>(outPlane) * cg * sizeof(T);
                if (smem > 48 * 1024) {
                    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
                    if (e != cudaSuccess) {
                        return;
                    }
                }
                const int32_t groups = static_cast<int32_t>(CeilDiv(g.c, cg));
                const int threads = smem <= 110 * 1024 ? 512 : 1024;
                kernel<<<static_cast<unsigned>(g.n * groups), threads, smem, s>>>(pgo, segStart, entries, pgi, g,
                                                                                  groups, entriesPerImage);
            };
            constexpr int kMax = 16 / sizeof(T);
            if (plan.detGatherGroup == kMax) {
                gather(DetGatherStagedKernel<T, kMax>, kMax);
            } else if (plan.detGatherGroup == kMax / 2) {
                gather(DetGatherStagedKernel<T, kMax / 2>, kMax / 2);
            } else {
                gather(DetGatherStagedKernel<T, kMax / 4>, kMax / 4);
            }
        } else if (e == cudaSuccess) {
            constexpr int CG = 8;
            const int32_t chanGroups = static_cast<int32_t>(CeilDiv(g.c, CG));
            const int64_t gatherTotal = g.n * chanGroups * inPlane;
            DetGatherKernel<T, CG><<<GridFor(gatherTotal, kThreads, 16), kThreads, 0, s>>>(
                pgo, segStart, entries, pgi, g, chanGroups, entriesPerImage, gatherTotal);
        }
        CountLaunch();
        if (e != cudaSuccess) {
            return e;
        }
        if (plan.wantGrid && plan.detGridGroup > 0) {
            float2* parts = reinterpret_cast<float2*>(ws + plan.countBytes + plan.entryBytes);
            T* pgg = static_cast<T*>(ggrid);
            constexpr int kMax = 16 / sizeof(T);
            if (plan.detGridGroup == kMax) {
                e = LaunchStagedBwd<T, kMax>(pgo, px, pg, pgi, pgg, parts, recs, g, false, true, true, s);
            } else if (plan.detGridGroup == kMax / 2) {
                e = LaunchStagedBwd<T, kMax / 2>(pgo, px, pg, pgi, pgg, parts, recs, g, false, true, true, s);
            } else {
                e = LaunchStagedBwd<T, kMax / 4>(pgo, px, pg, pgi, pgg, parts, recs, g, false, true, true, s);
            }
            if (e != cudaSuccess) {
                return e;
            }
        } else if (plan.wantGrid) {
            GridGradSampleKernel<T, false, true><<<GridFor(samples, kThreads, 16), kThreads, 0, s>>>(
                pgo, px, pg, nullptr, static_cast<T*>(ggrid), g, samples);
            CountLaunch();
        }
    });
    return cudaGetLastError();
}

} // namespace opscv
