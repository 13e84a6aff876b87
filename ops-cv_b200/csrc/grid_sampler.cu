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
#include "grid_coords.cuh"
#include "launch_util.cuh"

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

} // namespace

cudaError_t GridSampler2DFwd(Dt dt, const void* x, const void* grid, void* y, GridShape g, cudaStream_t s)
{
    const int64_t pixels = g.n * g.hout * static_cast<int64_t>(g.wout);
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
