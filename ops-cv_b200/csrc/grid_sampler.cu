// GridSampler2D forward (input NCHW, grid N x Ho x Wo x 2, output NCHW).
//
// Two kernels:
//   * staged kernel (bilinear, input plane small enough for shared memory): a block owns one image and a small
//     group of channels. It copies those channels' input planes from HBM into shared memory once, interleaved
//     by channel ([y][x][c]), then walks every output pixel of the image: the four taps of a pixel are four
//     16-byte shared-memory reads that serve all channels of the group, and the output stores are coalesced
//     along Wo. Random grids therefore cost HBM only the compulsory traffic (input once, grid, output once)
//     instead of one 32-byte sector per tap per channel.
//   * direct kernel (every mode, any size): one thread per output pixel and channel chunk, taps gathered from
//     global memory; coordinates are computed once per pixel and reused for the thread's channels.
//
// Arithmetic: image/grid_sampler2_d/op_kernel/arch35/grid_sampler2_d_simt.h:303-514 (see grid_coords.cuh).
#include "cp_async.cuh"
#include "grid_coords.cuh"
#include "launch_util.cuh"

#include <algorithm>

namespace opscv {
namespace {

constexpr int kThreads = 256;

struct BilinearTaps {
    int32_t x0, y0;
    float nw, ne, sw, se;
    bool nan;
};

__device__ __forceinline__ BilinearTaps MakeBilinearTaps(float gx, float gy, int32_t hin, int32_t win, int32_t pad,
                                                         int32_t align)
{
    BilinearTaps t;
    float ix = gs::ComputeSourceIndex(gx, win, pad, align);
    float iy = gs::ComputeSourceIndex(gy, hin, pad, align);
    t.nan = gs::IsNanOrInf(ix) || gs::IsNanOrInf(iy);
    ix = gs::SafeDowngradeToIntRange(ix);
    iy = gs::SafeDowngradeToIntRange(iy);
    const float ixF = floorf(ix), iyF = floorf(iy);
    t.x0 = static_cast<int32_t>(ixF);
    t.y0 = static_cast<int32_t>(iyF);
    const float xe = Sub(Add(ixF, 1.0f), ix), ye = Sub(Add(iyF, 1.0f), iy); // (x0 + 1 - ix), (y0 + 1 - iy)
    const float xw = Sub(ix, ixF), yw = Sub(iy, iyF);
    t.nw = Mul(xe, ye);
    t.ne = Mul(xw, ye);
    t.sw = Mul(xe, yw);
    t.se = Mul(xw, yw);
    return t;
}

// ---- direct kernel ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
    GridSamplerDirectKernel(const T* __restrict__ x, const T* __restrict__ grid, T* __restrict__ y, GridShape g,
                            int32_t chanChunks, int32_t chanPerChunk, int64_t total)
{
    const int64_t inPlane = static_cast<int64_t>(g.hin) * g.win;
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        // idx = (n * chanChunks + chunk) * outPlane + p : consecutive threads -> consecutive pixels
        const int64_t nc = idx / outPlane;
        const int64_t p = idx - nc * outPlane;
        const int64_t n = nc / chanChunks;
        const int32_t chunk = static_cast<int32_t>(nc - n * chanChunks);
        const int64_t c0 = static_cast<int64_t>(chunk) * chanPerChunk;
        const int64_t c1 = min(g.c, c0 + chanPerChunk);
        const int64_t s = n * outPlane + p;
        const float gx = DType<T>::Load(grid + 2 * s);
        const float gy = DType<T>::Load(grid + 2 * s + 1);
        const T* xb = x + (n * g.c + c0) * inPlane;
        T* yb = y + (n * g.c + c0) * outPlane + p;
        const int64_t nch = c1 - c0;
        if (g.interp == 0) {
            const BilinearTaps t = MakeBilinearTaps(gx, gy, g.hin, g.win, g.pad, g.align);
            if (t.nan) {
                const T nanv = DType<T>::FromF(__int_as_float(0x7fc00000));
                for (int64_t c = 0; c < nch; ++c) {
                    yb[c * outPlane] = nanv;
                }
                continue;
            }
            const bool bnw = gs::Within(t.y0, t.x0, g.hin, g.win), bne = gs::Within(t.y0, t.x0 + 1, g.hin, g.win);
            const bool bsw = gs::Within(t.y0 + 1, t.x0, g.hin, g.win),
                       bse = gs::Within(t.y0 + 1, t.x0 + 1, g.hin, g.win);
            const int64_t o = static_cast<int64_t>(t.y0) * g.win + t.x0;
            for (int64_t c = 0; c < nch; ++c) {
                const T* xc = xb + c * inPlane + o;
                float out = 0.0f;
                if (bnw) {
                    out = Add(out, Mul(DType<T>::Load(xc), t.nw));
                }
                if (bne) {
                    out = Add(out, Mul(DType<T>::Load(xc + 1), t.ne));
                }
                if (bsw) {
                    out = Add(out, Mul(DType<T>::Load(xc + g.win), t.sw));
                }
                if (bse) {
                    out = Add(out, Mul(DType<T>::Load(xc + g.win + 1), t.se));
                }
                yb[c * outPlane] = DType<T>::FromF(out);
            }
        } else if (g.interp == 1) {
            const float ix = gs::SafeDowngradeToIntRange(gs::ComputeSourceIndex(gx, g.win, g.pad, g.align));
            const float iy = gs::SafeDowngradeToIntRange(gs::ComputeSourceIndex(gy, g.hin, g.pad, g.align));
            const int32_t xn = gs::BankerRoundToInt(ix), yn = gs::BankerRoundToInt(iy);
            const bool in = gs::Within(yn, xn, g.hin, g.win);
            const int64_t o = static_cast<int64_t>(yn) * g.win + xn;
            const T zero = DType<T>::FromF(0.0f);
            for (int64_t c = 0; c < nch; ++c) {
                yb[c * outPlane] = in ? __ldg(xb + c * inPlane + o) : zero;
            }
        } else {
            const float ix = gs::UnnormalizeNoClip(gx, g.win, g.align);
            const float iy = gs::UnnormalizeNoClip(gy, g.hin, g.align);
            if (gs::IsNanOrInf(ix) || gs::IsNanOrInf(iy)) {
                const T nanv = DType<T>::FromF(__int_as_float(0x7fc00000));
                for (int64_t c = 0; c < nch; ++c) {
                    yb[c * outPlane] = nanv;
                }
                continue;
            }
            const float ixF = floorf(ix), iyF = floorf(iy);
            const float tx = Sub(ix, ixF), ty = Sub(iy, iyF);
            int32_t bx[4], by[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                bx[k] = gs::SafeFloatToInt32(
                    gs::ComputeCoordinates(Add(ixF, static_cast<float>(k - 1)), g.win, g.pad, g.align));
                by[k] = gs::SafeFloatToInt32(
                    gs::ComputeCoordinates(Add(iyF, static_cast<float>(k - 1)), g.hin, g.pad, g.align));
            }
            const float cx0 = gs::Cubic2(Add(tx, 1.0f)), cx1 = gs::Cubic1(tx), cx2 = gs::Cubic1(Sub(1.0f, tx)),
                        cx3 = gs::Cubic2(Sub(2.0f, tx));
            const float cy0 = gs::Cubic2(Add(ty, 1.0f)), cy1 = gs::Cubic1(ty), cy2 = gs::Cubic1(Sub(1.0f, ty)),
                        cy3 = gs::Cubic2(Sub(2.0f, ty));
            for (int64_t c = 0; c < nch; ++c) {
                const T* xc = xb + c * inPlane;
                float r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    r[j] = 0.0f;
                    if (by[j] >= 0 && by[j] < g.hin) {
                        const T* row = xc + static_cast<int64_t>(by[j]) * g.win;
                        float v[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            v[k] = (bx[k] >= 0 && bx[k] < g.win) ? DType<T>::Load(row + bx[k]) : 0.0f;
                        }
                        r[j] = gs::WeightedSum(cx0, cx1, cx2, cx3, v[0], v[1], v[2], v[3]);
                    }
                }
                yb[c * outPlane] = DType<T>::FromF(gs::WeightedSum(cy0, cy1, cy2, cy3, r[0], r[1], r[2], r[3]));
            }
        }
    }
}

// ---- staged kernel (bilinear, every padding mode) -------------------------------------------------------------
// Source coordinates are the same for all channels of a sample, so a prologue kernel evaluates them once per
// sample into a float2 record (ix, iy), already padded / reflected / range-limited; a NaN ix marks a sample whose
// coordinates were NaN or infinite (its outputs are NaN).
template <typename T>
__global__ void __launch_bounds__(kThreads)
    GridCoordsKernel(const T* __restrict__ grid, float2* __restrict__ rec, GridShape g, int64_t total)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; s < total; s += stride) {
        float ix = gs::ComputeSourceIndex(DType<T>::Load(grid + 2 * s), g.win, g.pad, g.align);
        float iy = gs::ComputeSourceIndex(DType<T>::Load(grid + 2 * s + 1), g.hin, g.pad, g.align);
        const bool bad = gs::IsNanOrInf(ix) || gs::IsNanOrInf(iy);
        ix = gs::SafeDowngradeToIntRange(ix);
        iy = gs::SafeDowngradeToIntRange(iy);
        rec[s] = bad ? make_float2(__int_as_float(0x7fc00000), 0.0f) : make_float2(ix, iy);
    }
}

// blockIdx.x = (image * groups + channel group) * split + part. A group is NV 16-byte vectors of channels
// (CG = NV * 16 / sizeof(T)). The block copies the group's input planes into shared memory as
// tile[((y + 2) * (win + 4) + x + 2) * NV + v], surrounded by a two-pixel border of zeros, then handles the output
// pixels [part * per, ...) of the image, one pixel per thread and trip. With the border, a tap outside the image
// reads a zero instead of being skipped: adding 0 * weight leaves the fp32 sum unchanged bit for bit (the
// weights are finite), so the kernel needs no bounds tests; tap positions are clamped into the border.
constexpr int kStageThreads = 512;
constexpr int kBorder = 2;

template <typename T, int NV>
__global__ void __launch_bounds__(kStageThreads, NV == 1 ? 3 : 1)
    GridSamplerStagedKernel(const T* __restrict__ x, const float2* __restrict__ rec, T* __restrict__ y, GridShape g,
                            int32_t groups, int32_t split, int32_t per)
{
    extern __shared__ __align__(16) unsigned char stagedSmem[];
    constexpr int LV = 16 / sizeof(T);
    constexpr int CG = NV * LV;
    using Vec = Pack<T, LV>;
    Vec* tile = reinterpret_cast<Vec*>(stagedSmem);
    const int32_t inPlane = g.hin * g.win, outPlane = g.hout * g.wout;
    const int32_t tw = g.win + 2 * kBorder, th = g.hin + 2 * kBorder;
    const int32_t part = blockIdx.x % split;
    const int64_t ng = blockIdx.x / split;
    const int64_t n = ng / groups;
    const int32_t c0 = static_cast<int32_t>(ng - n * groups) * CG;
    const int32_t nch = min(CG, static_cast<int32_t>(g.c) - c0);
    const T* xb = x + (n * g.c + c0) * inPlane;
    if constexpr (NV == 1) {
        // the zero border (two rows above and below, two columns left and right), then the planes as pixel records
        const Vec zero{};
        for (int32_t i = threadIdx.x; i < 2 * kBorder * tw; i += blockDim.x) {
            const int32_t r = i / tw;
            tile[(r < kBorder ? r : g.hin + r) * tw + (i - r * tw)] = zero;
        }
        for (int32_t i = threadIdx.x; i < g.hin * 2 * kBorder; i += blockDim.x) {
            const int32_t r = i / (2 * kBorder), c = i - r * (2 * kBorder);
            tile[(r + kBorder) * tw + (c < kBorder ? c : g.win + c)] = zero;
        }
        StageRecords<T>(tile + kBorder * tw + kBorder, tw, xb, inPlane, g.win, nch, g.hin, g.win, threadIdx.x, blockDim.x);
    } else {
    const int32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int32_t ty = warp; ty < th; ty += warps) {
        const int32_t sy = ty - kBorder;
        const bool rowIn = sy >= 0 && sy < g.hin;
        for (int32_t tx = lane; tx < tw; tx += 32) {
            const int32_t sx = tx - kBorder;
            const bool in = rowIn && sx >= 0 && sx < g.win;
            const T* src = xb + sy * g.win + sx;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                Vec q;
#pragma unroll
                for (int k = 0; k < LV; ++k) {
                    const int ch = v * LV + k;
                    q.v[k] = (in && ch < nch) ? __ldg(src + static_cast<int64_t>(ch) * inPlane) : DType<T>::FromF(0.0f);
                }
                tile[(ty * tw + tx) * NV + v] = q;
            }
        }
    }
    }
    __syncthreads();
    const int32_t p1 = min(outPlane, (part + 1) * per);
    const float2* rb = rec + n * outPlane;
    T* yb = y + (n * g.c + c0) * outPlane;
    for (int32_t p = part * per + threadIdx.x; p < p1; p += blockDim.x) {
        const float2 r = __ldg(rb + p);
        float out[CG];
        if (r.x != r.x) {
#pragma unroll
            for (int k = 0; k < CG; ++k) {
                out[k] = __int_as_float(0x7fc00000);
            }
        } else {
            const float ixF = floorf(r.x), iyF = floorf(r.y);
            const float xe = Sub(Add(ixF, 1.0f), r.x), ye = Sub(Add(iyF, 1.0f), r.y);
            const float xw = Sub(r.x, ixF), yw = Sub(r.y, iyF);
            const float wt[4] = {Mul(xe, ye), Mul(xw, ye), Mul(xe, yw), Mul(xw, yw)};
            const int32_t cx = min(max(static_cast<int32_t>(ixF), -kBorder), g.win);
            const int32_t cy = min(max(static_cast<int32_t>(iyF), -kBorder), g.hin);
            const Vec* t0 = tile + ((cy + kBorder) * tw + cx + kBorder) * NV;
#pragma unroll
            for (int k = 0; k < CG; ++k) {
                out[k] = 0.0f;
            }
#pragma unroll
            for (int tap = 0; tap < 4; ++tap) {
                const Vec* tp = t0 + ((tap >> 1) * tw + (tap & 1)) * NV;
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    const Vec q = tp[v];
                    float qv[LV];
                    UnpackToF<T, LV>(q, qv);
#pragma unroll
                    for (int k = 0; k < LV; ++k) {
                        out[v * LV + k] = Add(out[v * LV + k], Mul(qv[k], wt[tap]));
                    }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < CG; ++k) {
            if (k < nch) {
                yb[static_cast<int64_t>(k) * outPlane + p] = DType<T>::FromF(out[k]);
            }
        }
    }
}

// ---- windowed kernel (bilinear, fp32, planes too large for the plane-major staged kernel) -----------------------
// A block owns a 32 x 32 tile of output pixels of one image and walks all channels, four at a time. The source
// coordinates and tap weights of a pixel do not depend on the channel: a thread evaluates them once for its two
// pixels and keeps them in registers. The block then takes the bounding box of the tile's taps (smooth grids such as
// affine warps keep it small: a rotated, scaled square a little larger than the tile). For every group of four
// channels the box is copied from the four input planes into four small planes in shared memory, with 16-byte
// cp.async into one of two buffers while the previous group is sampled from the other, so the taps are shared-memory
// reads (neighbouring pixels of a smooth grid read neighbouring words: hardly any bank conflicts) and the copy of
// the next group overlaps the arithmetic of this one. 16-byte pieces of the box that lie outside the image are
// zero-filled (a tap there adds 0 * weight: the same fp32 sum as skipping it); rows are multiples of four pixels,
// which is why the kernel wants win % 4 == 0 and a 16-byte aligned input.
// A tile whose box does not fit a buffer (a grid that is not smooth) samples from global memory instead, like the
// direct kernel; the choice is made per tile from the data.
constexpr int kWinThreads = 512;
constexpr int kWinTile = 32;
constexpr int kWinChans = 4;
constexpr int32_t kWinCapFloats = 3400; // floats per staged plane: 2 buffers * 4 planes * 3400 * 4 B = 106 KiB
constexpr int kWinPieces = (kWinCapFloats / 4 + kWinThreads - 1) / kWinThreads; // 16-byte pieces a thread may own

__device__ __forceinline__ void CpAsync16Zfill(void* smem, const void* gmem, bool valid)
{
    const int srcBytes = valid ? 16 : 0; // 0 source bytes: the sixteen destination bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(smem))),
                 "l"(gmem), "r"(srcBytes)
                 : "memory");
}

__global__ void __launch_bounds__(kWinThreads, 2)
    GridSamplerWindowKernel(const float* __restrict__ x, const float* __restrict__ grid, float* __restrict__ y,
                            GridShape g, int32_t tilesX, int32_t tilesY, int32_t capFloats)
{
    extern __shared__ __align__(16) unsigned char stagedSmem[];
    __shared__ int32_t box[4]; // min x, max x, min y, max y of the clamped tap origins
    float* const bufBase = reinterpret_cast<float*>(stagedSmem); // two buffers of kWinChans * capFloats floats
    const int32_t inPlane = g.hin * g.win;
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int32_t tx = blockIdx.x % tilesX;
    const int32_t ty = (blockIdx.x / tilesX) % tilesY;
    const int64_t n = blockIdx.x / (tilesX * tilesY);
    const int32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        box[0] = INT32_MAX;
        box[1] = INT32_MIN;
        box[2] = INT32_MAX;
        box[3] = INT32_MIN;
    }
    __syncthreads();
    // The tile is 4 x 8 patches of 8 x 4 pixels; a warp takes the patches warp and warp + 16, a lane one pixel of
    // each (column lane % 8, row lane / 8 of the patch). The taps of a compact patch conflict on fewer shared-memory
    // banks than those of a 32 x 1 row (1.6 against 2.4 wavefronts per load for rotated grids, with the row pitch
    // chosen below), and a warp's stores are four full 32-byte sectors.
    float wt[2][4];
    int32_t cx[2], cy[2];
    int64_t outOff[2];
    bool live[2], bad[2];
    int32_t mnx = INT32_MAX, mxx = INT32_MIN, mny = INT32_MAX, mxy = INT32_MIN;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int32_t patch = warp + 16 * j;
        const int32_t ox = tx * kWinTile + (patch & 3) * 8 + (lane & 7);
        const int32_t oy = ty * kWinTile + (patch >> 2) * 4 + (lane >> 3);
        live[j] = ox < g.wout && oy < g.hout;
        bad[j] = false;
        cx[j] = cy[j] = 0;
        outOff[j] = static_cast<int64_t>(oy) * g.wout + ox;
        if (live[j]) {
            const int64_t s = n * outPlane + outOff[j];
            float ix = gs::ComputeSourceIndex(__ldg(grid + 2 * s), g.win, g.pad, g.align);
            float iy = gs::ComputeSourceIndex(__ldg(grid + 2 * s + 1), g.hin, g.pad, g.align);
            bad[j] = gs::IsNanOrInf(ix) || gs::IsNanOrInf(iy);
            ix = gs::SafeDowngradeToIntRange(ix);
            iy = gs::SafeDowngradeToIntRange(iy);
            const float ixF = floorf(ix), iyF = floorf(iy);
            const float xe = Sub(Add(ixF, 1.0f), ix), ye = Sub(Add(iyF, 1.0f), iy);
            const float xw = Sub(ix, ixF), yw = Sub(iy, iyF);
            wt[j][0] = Mul(xe, ye);
            wt[j][1] = Mul(xw, ye);
            wt[j][2] = Mul(xe, yw);
            wt[j][3] = Mul(xw, yw);
            // tap origins far outside the image are pulled to the two zero columns / rows beside it
            cx[j] = min(max(static_cast<int32_t>(ixF), -kBorder), g.win);
            cy[j] = min(max(static_cast<int32_t>(iyF), -kBorder), g.hin);
            if (!bad[j]) {
                mnx = min(mnx, cx[j]);
                mxx = max(mxx, cx[j]);
                mny = min(mny, cy[j]);
                mxy = max(mxy, cy[j]);
            }
        }
    }
    mnx = __reduce_min_sync(0xffffffffu, mnx);
    mxx = __reduce_max_sync(0xffffffffu, mxx);
    mny = __reduce_min_sync(0xffffffffu, mny);
    mxy = __reduce_max_sync(0xffffffffu, mxy);
    if (lane == 0) {
        atomicMin(&box[0], mnx);
        atomicMax(&box[1], mxx);
        atomicMin(&box[2], mny);
        atomicMax(&box[3], mxy);
    }
    __syncthreads();
    const bool any = box[1] >= box[0];
    // columns [wx0, wx0 + pitch) in whole 16-byte pieces (floor to a multiple of four: -4 holds the zero columns
    // -2, -1), rows [wy0, wy0 + wh)
    const int32_t wx0 = any ? (box[0] + 4) / 4 * 4 - 4 : 0, wy0 = any ? box[2] : 0;
    const int32_t needW = any ? (box[1] + 2 - wx0 + 3) / 4 * 4 : 4; // floats per row that are copied
    const int32_t pitch = needW + ((8 - needW % 16) + 16) % 16;       // row pitch: 8 or 24 modulo 32
    const int32_t wh = any ? box[3] - box[2] + 2 : 1;
    const int32_t wsize = pitch * wh;
    const float* xn = x + n * g.c * inPlane;
    float* yn = y + n * g.c * outPlane;
    const float nanv = __int_as_float(0x7fc00000);

    if (wsize > capFloats) {
        // not a smooth tile: taps from global memory, channel by channel
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (!live[j]) {
                continue;
            }
            const int32_t x0 = cx[j], y0 = cy[j];
            const bool bnw = gs::Within(y0, x0, g.hin, g.win), bne = gs::Within(y0, x0 + 1, g.hin, g.win);
            const bool bsw = gs::Within(y0 + 1, x0, g.hin, g.win), bse = gs::Within(y0 + 1, x0 + 1, g.hin, g.win);
            const int64_t o = static_cast<int64_t>(y0) * g.win + x0;
            for (int64_t c = 0; c < g.c; ++c) {
                const float* xc = xn + c * inPlane + o;
                float out = 0.0f;
                if (bnw) {
                    out = Add(out, Mul(__ldg(xc), wt[j][0]));
                }
                if (bne) {
                    out = Add(out, Mul(__ldg(xc + 1), wt[j][1]));
                }
                if (bsw) {
                    out = Add(out, Mul(__ldg(xc + g.win), wt[j][2]));
                }
                if (bse) {
                    out = Add(out, Mul(__ldg(xc + g.win + 1), wt[j][3]));
                }
                yn[c * outPlane + outOff[j]] = bad[j] ? nanv : out;
            }
        }
        return;
    }

    // byte offset of the thread's NW taps inside a staged plane
    uint32_t rec[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        rec[j] = (live[j] && !bad[j]) ? static_cast<uint32_t>((cy[j] - wy0) * pitch + (cx[j] - wx0)) * 4u : 0u;
    }
    // the two pixels' weights side by side: one packed multiply and one packed add per tap and channel
    // (a sample whose coordinates were NaN or infinite gets NaN weights: every one of its outputs is then NaN, which
    // is what the reference writes for it)
    F2 w2[4];
#pragma unroll
    for (int tap = 0; tap < 4; ++tap) {
        w2[tap] = MakeF2(bad[0] ? nanv : (live[0] ? wt[0][tap] : 0.0f), bad[1] ? nanv : (live[1] ? wt[1][tap] : 0.0f));
    }
    const int32_t groups = static_cast<int32_t>((g.c + kWinChans - 1) / kWinChans);
    // Copies. The box is the same for every channel, so a thread owns the same 16-byte pieces (row r, piece q) of the
    // box in every group: at most kWinPieces of them, whose source offset inside a plane, destination offset inside
    // a staged plane and in-image flag are evaluated once.
    const int32_t pieces = needW / 4;
    const int32_t total = wh * pieces;
    int32_t srcOff[kWinPieces];
    uint32_t dstOff[kWinPieces];
    int srcBytes[kWinPieces];
#pragma unroll
    for (int i = 0; i < kWinPieces; ++i) {
        const int32_t id = threadIdx.x + i * kWinThreads;
        const int32_t r = id / pieces, q = id - r * pieces;
        const int32_t sy = wy0 + r, sx = wx0 + 4 * q;
        const bool in = id < total && sy >= 0 && sy < g.hin && sx >= 0 && sx < g.win;
        srcBytes[i] = id < total ? (in ? 16 : 0) : -1; // -1: the thread has no such piece
        srcOff[i] = min(max(sy, 0), g.hin - 1) * g.win + min(max(sx, 0), g.win - 4);
        dstOff[i] = static_cast<uint32_t>(r * pitch + 4 * q) * 4u;
    }
    const uint32_t smemBase = static_cast<uint32_t>(__cvta_generic_to_shared(bufBase));
    const uint32_t planeBytes = static_cast<uint32_t>(pitch * wh) * 4u, pitchBytes = static_cast<uint32_t>(pitch) * 4u;
    auto stage = [&](int32_t grp, uint32_t dstBase) {
        const int32_t c0 = grp * kWinChans;
#pragma unroll
        for (int k = 0; k < kWinChans; ++k) {
            const bool chIn = c0 + k < g.c;
            const float* plane = xn + static_cast<int64_t>(chIn ? c0 + k : 0) * inPlane;
#pragma unroll
            for (int i = 0; i < kWinPieces; ++i) {
                if (srcBytes[i] >= 0) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dstBase + k * planeBytes + dstOff[i]),
                                 "l"(plane + srcOff[i]), "r"(chIn ? srcBytes[i] : 0)
                                 : "memory");
                }
            }
        }
        CpAsyncCommit();
    };
    const uint32_t bufBytes = static_cast<uint32_t>(kWinChans) * capFloats * 4u;
    float* yp0 = yn + outOff[0];
    float* yp1 = yn + outOff[1];
    stage(0, smemBase);
    for (int32_t grp = 0; grp < groups; ++grp) {
        if (grp + 1 < groups) {
            stage(grp + 1, smemBase + ((grp + 1) & 1) * bufBytes);
            CpAsyncWait<1>();
        } else {
            CpAsyncWait<0>();
        }
        __syncthreads();
        const unsigned char* ta = stagedSmem + (grp & 1) * bufBytes + rec[0];
        const unsigned char* tb = stagedSmem + (grp & 1) * bufBytes + rec[1];
        const int32_t c0 = grp * kWinChans;
#pragma unroll
        for (int k = 0; k < kWinChans; ++k) {
            auto tapv = [&](const unsigned char* t, uint32_t off) { return *reinterpret_cast<const float*>(t + off); };
            // acc = acc + v * w with two roundings, as the reference (see AddProduct2)
            F2 o = AddProduct2(Mul2(MakeF2(tapv(ta, 0), tapv(tb, 0)), w2[0]), MakeF2(0.0f, 0.0f)); // 0 + (-0) is +0
            o = AddProduct2(Mul2(MakeF2(tapv(ta, 4), tapv(tb, 4)), w2[1]), o);
            o = AddProduct2(Mul2(MakeF2(tapv(ta, pitchBytes), tapv(tb, pitchBytes)), w2[2]), o);
            o = AddProduct2(Mul2(MakeF2(tapv(ta, pitchBytes + 4), tapv(tb, pitchBytes + 4)), w2[3]), o);
            float o0, o1;
            SplitF2(o, o0, o1);
            if (c0 + k < g.c) { // written once and not read again by this kernel: streaming stores
                if (live[0]) {
                    __stcs(yp0, o0);
                }
                if (live[1]) {
                    __stcs(yp1, o1);
                }
            }
            ta += planeBytes;
            tb += planeBytes;
            yp0 += outPlane;
            yp1 += outPlane;
        }
        __syncthreads(); // the buffer is free for the copies of group grp + 2
    }
}

inline size_t StagedFwdSmem(int64_t hin, int64_t win, int nv)
{
    return static_cast<size_t>((hin + 2 * kBorder) * (win + 2 * kBorder)) * nv * 16;
}

template <typename T, int NV>
cudaError_t LaunchStaged(const T* x, const T* grid, T* y, float2* rec, GridShape g, cudaStream_t s)
{
    constexpr int CG = NV * 16 / static_cast<int>(sizeof(T));
    const int64_t outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int64_t samples = g.n * outPlane;
    GridCoordsKernel<T><<<GridFor(samples, kThreads), kThreads, 0, s>>>(grid, rec, g, samples);
    const int32_t groups = static_cast<int32_t>(CeilDiv(g.c, CG));
    const size_t smem = StagedFwdSmem(g.hin, g.win, NV);
    const int64_t slots = static_cast<int64_t>(NumSMs()) * std::max<int64_t>(1, (220 * 1024) / (smem + 1024));
    // Split the pixels of an image over several blocks only while that is needed for ~4 waves of blocks (every
    // part stages the planes again, from L2).
    int32_t split = 1;
    while (split < 8 && g.n * groups * split < 4 * slots && outPlane / (split * 2) >= 2048) {
        split *= 2;
    }
    const int32_t per = static_cast<int32_t>(CeilDiv(outPlane, split));
    auto kernel = GridSamplerStagedKernel<T, NV>;
    cudaError_t e = cudaSuccess;
    if (smem > 48 * 1024) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) {
            return e;
        }
    }
    kernel<<<static_cast<unsigned>(g.n * groups * split), kStageThreads, smem, s>>>(x, rec, y, g, groups, split, per);
    CountLaunch(2);
    return cudaGetLastError();
}

} // namespace

GridFwdPlan PlanGridSampler2DFwd(Dt dt, GridShape g)
{
    GridFwdPlan plan{};
    const int64_t inPlane = static_cast<int64_t>(g.hin) * g.win, outPlane = static_cast<int64_t>(g.hout) * g.wout;
    const int lanes = 16 / DtSize(dt);
    // Staging pays for bilinear sampling when an image has at least as many output pixels as a plane has inputs;
    // it needs planes that fit shared memory and 32-bit in-image offsets and block indices.
    if (g.interp != 0 || outPlane * 2 < inPlane || outPlane >= (1LL << 30) || g.c < lanes / 2 ||
        g.n * CeilDiv(g.c, lanes) * 8 >= (1LL << 31)) {
        return plan;
    }
    // At least two blocks per SM must fit, so that one block's staging overlaps another's sampling; larger planes
    // take the direct kernel. (Two channel vectors per pixel measured slower than one: the kernel is bound by
    // shared-memory wavefronts, not by the per-pixel coordinate work.)
    if (StagedFwdSmem(g.hin, g.win, 1) + 1024 <= 110 * 1024) {
        plan.vectors = 1;
    } else if (dt == Dt::F32 && g.c >= 4 && g.win % 4 == 0 && g.win >= 4 &&
               g.n * CeilDiv(g.hout, kWinTile) * CeilDiv(g.wout, kWinTile) < (1LL << 31)) {
        plan.windowed = 1; // larger planes: per-tile windows of the planes (no workspace)
    }
    if (plan.vectors > 0) {
        plan.recBytes = static_cast<uint64_t>(g.n) * outPlane * sizeof(float2);
    }
    return plan;
}

cudaError_t GridSampler2DFwd(Dt dt, const void* x, const void* grid, void* y, GridShape g, const GridFwdPlan& plan,
                             void* workspace, cudaStream_t s)
{
    const int64_t pixels = g.n * g.hout * static_cast<int64_t>(g.wout);
    if (plan.vectors > 0) {
        cudaError_t e = cudaSuccess;
        float2* rec = static_cast<float2*>(workspace);
        OPSCV_DISPATCH_DT(dt, T, {
            const T* px = static_cast<const T*>(x);
            const T* pg = static_cast<const T*>(grid);
            T* py = static_cast<T*>(y);
            if (plan.vectors == 2) {
                e = LaunchStaged<T, 2>(px, pg, py, rec, g, s);
            } else {
                e = LaunchStaged<T, 1>(px, pg, py, rec, g, s);
            }
        });
        return e;
    }
    if (plan.windowed != 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) { // 16-byte copies need an aligned input
        const int32_t tilesX = static_cast<int32_t>(CeilDiv(g.wout, kWinTile));
        const int32_t tilesY = static_cast<int32_t>(CeilDiv(g.hout, kWinTile));
        const size_t smem = static_cast<size_t>(kWinCapFloats) * 2 * kWinChans * sizeof(float);
        cudaError_t e = cudaFuncSetAttribute(GridSamplerWindowKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) {
            return e;
        }
        GridSamplerWindowKernel<<<static_cast<unsigned>(g.n * tilesX * tilesY), kWinThreads, smem, s>>>(
            static_cast<const float*>(x), static_cast<const float*>(grid), static_cast<float*>(y), g, tilesX, tilesY,
            kWinCapFloats);
        CountLaunch();
        return cudaGetLastError();
    }
    // Split channels across threads only as far as needed to fill the machine.
    const int64_t wanted = static_cast<int64_t>(NumSMs()) * 2048 * 2;
    int64_t chunks = CeilDiv(wanted, pixels > 0 ? pixels : 1);
    chunks = chunks < 1 ? 1 : (chunks > g.c ? g.c : chunks);
    const int32_t per = static_cast<int32_t>(CeilDiv(g.c, chunks));
    const int32_t chanChunks = static_cast<int32_t>(CeilDiv(g.c, per));
    const int64_t total = pixels * chanChunks;
    OPSCV_DISPATCH_DT(dt, T, {
        GridSamplerDirectKernel<T><<<GridFor(total, kThreads, 16), kThreads, 0, s>>>(
            static_cast<const T*>(x), static_cast<const T*>(grid), static_cast<T*>(y), g, chanChunks, per, total);
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
