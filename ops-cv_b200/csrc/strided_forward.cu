// UpsampleNearest2d / NearestExact2d forward on strided NCHW VIEWS for whole-number up-scales with a W factor of 2
// (the common 2x up-sample): the input may be a crop or a channel slice of a larger tensor, the output a crop or a
// channel slice of a larger buffer (an up-sample written straight into its place in a concatenation). Both views need
// a unit W stride; the N, C and H strides are free. The kernel is the dense replicate kernel with pitches: a thread
// loads VI adjacent input elements of a row once and stores the 2 * VI outputs they become into each of the rh output
// rows, as one 32-byte store when the row pitch keeps that alignment. No gather copy, no scatter copy.
#include <algorithm>

#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

template <typename T, int VI>
__global__ void __launch_bounds__(kThreads)
    NearestFwdX2PitchKernel(const T* __restrict__ x, ViewStrides si, T* __restrict__ y, ViewStrides so, int32_t hin,
                            int32_t win, int32_t rh, int64_t rowsIn)
{
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VI;
    if (t0 >= win) {
        return;
    }
    const bool small = rowsIn <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rowsIn; row += rowStep) {
        int64_t n; // row = (n, c, h) of the input
        int32_t c, h;
        SplitRow(row, hin, si.chan, small, n, c, h);
        const Pack<T, VI> in = *reinterpret_cast<const Pack<T, VI>*>(x + n * si.n + c * si.c + h * si.h + t0);
        constexpr int H = (2 * VI * sizeof(T) > 16) ? VI : 2 * VI; // elements per 16-byte half of the outputs
        Pack<T, H> out[2 * VI / H];
#pragma unroll
        for (int v = 0; v < VI; ++v) {
            out[(2 * v) / H].v[(2 * v) % H] = in.v[v];
            out[(2 * v + 1) / H].v[(2 * v + 1) % H] = in.v[v];
        }
        T* yr = y + n * so.n + c * so.c + static_cast<int64_t>(h) * rh * so.h + 2 * t0;
        for (int32_t b = 0; b < rh; ++b, yr += so.h) {
            if constexpr (2 * VI * sizeof(T) == 32) {
                Store32Bytes(yr, reinterpret_cast<const uint4&>(out[0]), reinterpret_cast<const uint4&>(out[1]));
            } else {
                *reinterpret_cast<Pack<T, H>*>(yr) = out[0];
            }
        }
    }
}

// The matching backward: grad_input (n, c, h, w) = sum of the rh x 2 window of grad_output, rows outer, columns inner,
// in fp32 (the order of the dense pool kernel and of the reference). grad_output may be a channel slice of the
// gradient of a concatenation, grad_input a slice or crop of a larger gradient buffer. Sides swapped: `big` is
// grad_output (2 * VO elements per thread and row), `small` is grad_input (VO elements).
template <typename T, int VO>
__global__ void __launch_bounds__(kThreads)
    NearestBwdX2PitchKernel(const T* __restrict__ go, ViewStrides big, T* __restrict__ gi, ViewStrides small_, int32_t hin,
                            int32_t win, int32_t rh, int64_t rowsIn)
{
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VO;
    if (t0 >= win) {
        return;
    }
    const bool small = rowsIn <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rowsIn; row += rowStep) {
        int64_t n; // row = (n, c, h) of grad_input
        int32_t c, h;
        SplitRow(row, hin, small_.chan, small, n, c, h);
        float acc[VO];
#pragma unroll
        for (int v = 0; v < VO; ++v) {
            acc[v] = 0.0f;
        }
        const T* gr = go + n * big.n + c * big.c + static_cast<int64_t>(h) * rh * big.h + 2 * t0;
        for (int32_t b = 0; b < rh; ++b, gr += big.h) {
            constexpr int H = (2 * VO * sizeof(T) > 16) ? VO : 2 * VO; // elements per 16-byte load
#pragma unroll
            for (int part = 0; part < 2 * VO / H; ++part) {
                float gv[H];
                LoadPackLdg<T, H>(gr + part * H, gv);
#pragma unroll
                for (int v = 0; v < H / 2; ++v) {
                    acc[part * (H / 2) + v] = Add(Add(acc[part * (H / 2) + v], gv[2 * v]), gv[2 * v + 1]);
                }
            }
        }
        StorePack<T, VO>(gi + n * small_.n + c * small_.c + h * small_.h + t0, acc);
    }
}

// Widest input pack: W extent, every pitch and both bases keep the alignment of the loads (VI elements) and of the
// stores (2 * VI elements).
int PitchVec(int es, int32_t win, const void* x, const ViewStrides& si, const void* y, const ViewStrides& so)
{
    for (int v = 16 / es; v >= 1; v >>= 1) {
        const int64_t a = v, b = 2 * v;
        if (win % a == 0 && si.n % a == 0 && si.c % a == 0 && si.h % a == 0 && Aligned(x, static_cast<size_t>(a) * es) &&
            so.n % b == 0 && so.c % b == 0 && so.h % b == 0 && Aligned(y, static_cast<size_t>(b) * es)) {
            return v;
        }
    }
    return 0;
}

} // namespace

bool NearestFwdX2PitchUsable(Dt dt, const void* x, ViewStrides si, const void* y, ViewStrides so, Shape4 sh)
{
    return si.w == 1 && so.w == 1 && PitchVec(DtSize(dt), sh.win, x, si, y, so) >= 1;
}

cudaError_t NearestFwdX2Pitch(Dt dt, const void* x, ViewStrides si, void* y, ViewStrides so, Shape4 sh, int32_t rh,
                              cudaStream_t s)
{
    const int vi = PitchVec(DtSize(dt), sh.win, x, si, y, so);
    if (vi < 1) {
        return cudaErrorInvalidValue;
    }
    const int64_t rowsIn = sh.n * sh.c * sh.hin;
    const RowLaunch rl = RowTiling(rowsIn, CeilDiv(static_cast<int64_t>(sh.win), vi), kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        OPSCV_DISPATCH_VEC(vi, VI, {
            if constexpr (VI * sizeof(T) <= 16) {
                NearestFwdX2PitchKernel<T, VI><<<rl.grid, rl.block, 0, s>>>(static_cast<const T*>(x), si, static_cast<T*>(y),
                                                                            so, sh.hin, sh.win, rh, rowsIn);
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv

namespace opscv {

bool NearestBwdX2PitchUsable(Dt dt, const void* go, ViewStrides big, const void* gi, ViewStrides small_, Shape4 sh)
{
    // the same alignment rule with the sides swapped: grad_input takes the role of the forward's input
    return big.w == 1 && small_.w == 1 && NearestFwdX2PitchUsable(dt, gi, small_, go, big, sh);
}

cudaError_t NearestBwdX2Pitch(Dt dt, const void* go, ViewStrides big, void* gi, ViewStrides small_, Shape4 sh, int32_t rh,
                              cudaStream_t s)
{
    const int es = DtSize(dt);
    int vo = 0;
    for (int v = 16 / es; v >= 1; v >>= 1) {
        const int64_t a = v, b = std::min<int64_t>(2 * v, 16 / es); // loads are at most 16 bytes each
        if (sh.win % a == 0 && small_.n % a == 0 && small_.c % a == 0 && small_.h % a == 0 &&
            Aligned(gi, static_cast<size_t>(a) * es) && big.n % b == 0 && big.c % b == 0 && big.h % b == 0 &&
            Aligned(go, static_cast<size_t>(b) * es)) {
            vo = v;
            break;
        }
    }
    if (vo < 1) {
        return cudaErrorInvalidValue;
    }
    const int64_t rowsIn = sh.n * sh.c * sh.hin;
    const RowLaunch rl = RowTiling(rowsIn, CeilDiv(static_cast<int64_t>(sh.win), vo), 256);
    OPSCV_DISPATCH_DT(dt, T, {
        OPSCV_DISPATCH_VEC(vo, VO, {
            if constexpr (VO * sizeof(T) <= 16) {
                NearestBwdX2PitchKernel<T, VO><<<rl.grid, rl.block, 0, s>>>(static_cast<const T*>(go), big, static_cast<T*>(gi),
                                                                            small_, sh.hin, sh.win, rh, rowsIn);
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
