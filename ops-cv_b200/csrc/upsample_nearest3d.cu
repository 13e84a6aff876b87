// UpsampleNearest3d / UpsampleNearestExact3d forward and backward on NCDHW and NDHWC tensors.
//
// Forward (image/upsample_nearest3d/op_kernel/arch35/upsample_nearest3d_simt_base.h:31-88): a pure copy,
// y[n, c, d, h, w] = x[n, c, sd(d), sh(h), sw(w)] with s(i) = min(floor((i [+ 0.5]) * scale), in - 1). A thread row of a
// block walks output rows (plane, d, h), finds the source row of each once, and each thread gathers a 16-byte pack of it
// (NCDHW: adjacent columns with their own source columns; NDHWC: adjacent channels of one pixel, one vector load).
// Backward (image/upsample_nearest3d_grad/op_kernel/arch35/upsample_nearest3d_grad_simt_base.h:33-58): every
// grad_input element sums its window [ceil(y * s [- 0.5]), ceil((y + 1) * s [- 0.5])) per axis in fp32, in d, h, w
// order, and is rounded once.
#include <algorithm>

#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ int32_t SrcIdx(int32_t i, float scale, int32_t exact, int32_t in)
{
    const float pos = exact ? Mul(Add(static_cast<float>(i), 0.5f), scale) : Mul(static_cast<float>(i), scale);
    const long long s = static_cast<long long>(floorf(pos));
    const long long last = in - 1;
    return static_cast<int32_t>(s < last ? s : last);
}

__device__ __forceinline__ int32_t WindowEdge(int32_t y, float scale, int32_t exact, int32_t limit)
{
    const float v = exact ? Sub(Mul(static_cast<float>(y), scale), 0.5f) : Mul(static_cast<float>(y), scale);
    long long e = static_cast<long long>(ceilf(v));
    e = e < 0 ? 0 : e;
    return static_cast<int32_t>(e < limit ? e : limit);
}

template <typename T, int V, bool CHANNELS_LAST>
__global__ void __launch_bounds__(kThreads) Nearest3dFwdKernel(const T* __restrict__ x, T* __restrict__ y, Nearest3dGeom g)
{
    const int64_t inner = static_cast<int64_t>(g.wo) * g.chan; // elements of an output row
    const int64_t rowIn = static_cast<int64_t>(g.wi) * g.chan;
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    if (t0 >= inner) {
        return;
    }
    const bool small = g.rows <= 0x7fffffffLL;
    // source offsets of this thread's pack inside a source row (the same for every row)
    int32_t off[CHANNELS_LAST ? 1 : V];
    if (CHANNELS_LAST) {
        const int32_t w = static_cast<int32_t>(t0 / g.chan);
        off[0] = SrcIdx(w, g.sw, g.exact, g.wi) * g.chan + static_cast<int32_t>(t0 - static_cast<int64_t>(w) * g.chan);
    } else {
#pragma unroll
        for (int v = 0; v < V; ++v) {
            off[CHANNELS_LAST ? 0 : v] = SrcIdx(static_cast<int32_t>(t0) + v, g.sw, g.exact, g.wi);
        }
    }
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < g.rows; row += rowStep) {
        int64_t plane; // row = (plane, d, h)
        int32_t d, h;
        SplitRow(row, g.ho, g.dout, small, plane, d, h);
        const int64_t srcRow = (plane * g.di + SrcIdx(d, g.sd, g.exact, g.di)) * g.hi + SrcIdx(h, g.sh, g.exact, g.hi);
        const T* px = x + srcRow * rowIn;
        T* py = y + row * inner + t0;
        if (CHANNELS_LAST) {
            *reinterpret_cast<Pack<T, V>*>(py) = *reinterpret_cast<const Pack<T, V>*>(px + off[0]);
        } else {
            Pack<T, V> p;
#pragma unroll
            for (int v = 0; v < V; ++v) {
                p.v[v] = __ldg(px + off[CHANNELS_LAST ? 0 : v]);
            }
            *reinterpret_cast<Pack<T, V>*>(py) = p;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) Nearest3dBwdKernel(const T* __restrict__ go, T* __restrict__ gi, Nearest3dGeom g)
{
    const int64_t inner = static_cast<int64_t>(g.wi) * g.chan; // elements of a grad_input row
    const int64_t rowGo = static_cast<int64_t>(g.wo) * g.chan;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= inner) {
        return;
    }
    const bool small = g.rows <= 0x7fffffffLL;
    const int32_t w = static_cast<int32_t>(t / g.chan);
    const int32_t c = static_cast<int32_t>(t - static_cast<int64_t>(w) * g.chan);
    const int32_t w0 = WindowEdge(w, g.sw, g.exact, g.wo), w1 = WindowEdge(w + 1, g.sw, g.exact, g.wo);
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < g.rows; row += rowStep) {
        int64_t plane; // row = (plane, d, h) of grad_input
        int32_t d, h;
        SplitRow(row, g.hi, g.di, small, plane, d, h);
        const int32_t d0 = WindowEdge(d, g.sd, g.exact, g.dout), d1 = WindowEdge(d + 1, g.sd, g.exact, g.dout);
        const int32_t h0 = WindowEdge(h, g.sh, g.exact, g.ho), h1 = WindowEdge(h + 1, g.sh, g.exact, g.ho);
        float acc = 0.0f;
        for (int32_t a = d0; a < d1; ++a) {
            for (int32_t b = h0; b < h1; ++b) {
                const T* pr = go + ((plane * g.dout + a) * g.ho + b) * rowGo + c;
                for (int32_t e = w0; e < w1; ++e) {
                    acc = Add(acc, DType<T>::Load(pr + static_cast<int64_t>(e) * g.chan));
                }
            }
        }
        gi[row * inner + t] = DType<T>::FromF(acc);
    }
}

// ---- whole-number up-scales on NCDHW tensors (g.rd, g.rh >= 1 and g.rw == 2, checked on the host against the index
// rules above): output (d, h, w) reads input (d / rd, h / rh, w / 2). A thread loads VI adjacent input elements of
// an input row once and stores the 2 * VI outputs they become into each of the rd * rh output rows; the backward
// loads 2 * VO adjacent grads of each of the rd * rh rows and adds them in (d, h, w) order, VO results per thread.
template <typename T, int VI>
__global__ void __launch_bounds__(kThreads) Nearest3dFwdX2Kernel(const T* __restrict__ x, T* __restrict__ y, Nearest3dGeom g)
{
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VI;
    if (t0 >= g.wi) {
        return;
    }
    const int64_t rowsIn = g.rows / (static_cast<int64_t>(g.rd) * g.rh); // (plane, d, h) of the input
    const bool small = rowsIn <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < rowsIn; row += rowStep) {
        int64_t plane;
        int32_t d, h;
        SplitRow(row, g.hi, g.di, small, plane, d, h);
        const Pack<T, VI> in = *reinterpret_cast<const Pack<T, VI>*>(x + row * g.wi + t0);
        // the 2 * VI outputs as one or two 16-byte stores
        constexpr int H = (2 * VI * sizeof(T) > 16) ? VI : 2 * VI;
        Pack<T, H> out[2 * VI / H];
#pragma unroll
        for (int v = 0; v < VI; ++v) {
            out[(2 * v) / H].v[(2 * v) % H] = in.v[v];
            out[(2 * v + 1) / H].v[(2 * v + 1) % H] = in.v[v];
        }
        for (int32_t a = 0; a < g.rd; ++a) {
            for (int32_t b = 0; b < g.rh; ++b) {
                const int64_t orow = (plane * g.dout + static_cast<int64_t>(d) * g.rd + a) * g.ho + static_cast<int64_t>(h) * g.rh + b;
                if constexpr (2 * VI * sizeof(T) == 32) {
                    // one 32-byte store: two 16-byte stores would each touch half of every sector of the warp
                    Store32Bytes(y + orow * g.wo + 2 * t0, reinterpret_cast<const uint4&>(out[0]),
                                 reinterpret_cast<const uint4&>(out[1]));
                } else {
                    *reinterpret_cast<Pack<T, H>*>(y + orow * g.wo + 2 * t0) = out[0];
                }
            }
        }
    }
}

template <typename T, int VO>
__global__ void __launch_bounds__(kThreads) Nearest3dBwdX2Kernel(const T* __restrict__ go, T* __restrict__ gi, Nearest3dGeom g)
{
    const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VO;
    if (t0 >= g.wi) {
        return;
    }
    const bool small = g.rows <= 0x7fffffffLL;
    const int64_t rowStep = static_cast<int64_t>(gridDim.y) * blockDim.y;
    for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < g.rows; row += rowStep) {
        int64_t plane; // row = (plane, d, h) of grad_input
        int32_t d, h;
        SplitRow(row, g.hi, g.di, small, plane, d, h);
        float acc[VO];
#pragma unroll
        for (int v = 0; v < VO; ++v) {
            acc[v] = 0.0f;
        }
        for (int32_t a = 0; a < g.rd; ++a) {
            for (int32_t b = 0; b < g.rh; ++b) {
                const int64_t orow = (plane * g.dout + static_cast<int64_t>(d) * g.rd + a) * g.ho + static_cast<int64_t>(h) * g.rh + b;
                // 2 * VO grads as one or two 16-byte loads
                constexpr int H = (2 * VO * sizeof(T) > 16) ? VO : 2 * VO; // elements per load
#pragma unroll
                for (int part = 0; part < 2 * VO / H; ++part) {
                    float gv[H];
                    LoadPackLdg<T, H>(go + orow * g.wo + 2 * t0 + part * H, gv);
#pragma unroll
                    for (int v = 0; v < H / 2; ++v) {
                        acc[part * (H / 2) + v] = Add(Add(acc[part * (H / 2) + v], gv[2 * v]), gv[2 * v + 1]);
                    }
                }
            }
        }
        StorePack<T, VO>(gi + row * g.wi + t0, acc);
    }
}

} // namespace

cudaError_t Nearest3dFwd(Dt dt, const void* x, void* y, Nearest3dGeom g, cudaStream_t s)
{
    const int64_t inner = static_cast<int64_t>(g.wo) * g.chan;
    const int es = DtSize(dt);
    const bool cl = g.chan > 1;
    if (!cl && g.rw == 2 && g.rd >= 1 && g.rh >= 1) {
        int vi = 16 / es; // a 16-byte load becomes 32 bytes of each output row, written as one 32-byte store
        while (vi > 1 && (g.wi % vi != 0 || !Aligned(x, static_cast<size_t>(vi) * es) ||
                          !Aligned(y, static_cast<size_t>(2 * vi) * es))) {
            vi >>= 1;
        }
        if (Aligned(y, static_cast<size_t>(2 * vi) * es)) {
            const int64_t rowsIn = g.rows / (static_cast<int64_t>(g.rd) * g.rh);
            const RowLaunch rl = RowTiling(rowsIn, CeilDiv(static_cast<int64_t>(g.wi), vi), kThreads);
            OPSCV_DISPATCH_DT(dt, T, {
                const T* px = static_cast<const T*>(x);
                T* py = static_cast<T*>(y);
                OPSCV_DISPATCH_VEC(vi, VI, {
                    if constexpr (VI * sizeof(T) <= 16) {
                        Nearest3dFwdX2Kernel<T, VI><<<rl.grid, rl.block, 0, s>>>(px, py, g);
                    }
                });
            });
            CountLaunch();
            return cudaGetLastError();
        }
    }
    // pack width: 16 bytes when rows keep that alignment; channels-last packs must not straddle a pixel
    int v = 16 / es;
    while (v > 1 && (inner % v != 0 || (cl && g.chan % v != 0) || !Aligned(y, static_cast<size_t>(v) * es) ||
                     (cl && (!Aligned(x, static_cast<size_t>(v) * es))))) {
        v >>= 1;
    }
    const RowLaunch rl = RowTiling(g.rows, CeilDiv(inner, v), kThreads);
    OPSCV_DISPATCH_DT(dt, T, {
        const T* px = static_cast<const T*>(x);
        T* py = static_cast<T*>(y);
        OPSCV_DISPATCH_VEC(v, V, {
            if constexpr (V * sizeof(T) <= 16) {
                if (cl) {
                    Nearest3dFwdKernel<T, V, true><<<rl.grid, rl.block, 0, s>>>(px, py, g);
                } else {
                    Nearest3dFwdKernel<T, V, false><<<rl.grid, rl.block, 0, s>>>(px, py, g);
                }
            }
        });
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t Nearest3dBwd(Dt dt, const void* go, void* gi, Nearest3dGeom g, cudaStream_t s)
{
    const int64_t inner = static_cast<int64_t>(g.wi) * g.chan;
    const int es = DtSize(dt);
    if (g.chan == 1 && g.rw == 2 && g.rd >= 1 && g.rh >= 1) {
        int vo = 16 / es; // 16 bytes of grad_input per store, read as 16-byte loads of grads
        while (vo > 1 && (g.wi % vo != 0 || !Aligned(gi, static_cast<size_t>(vo) * es) ||
                          !Aligned(go, std::min<size_t>(16, static_cast<size_t>(2 * vo) * es)))) {
            vo >>= 1;
        }
        if (Aligned(go, std::min<size_t>(16, static_cast<size_t>(2 * vo) * es))) {
            const RowLaunch rl = RowTiling(g.rows, CeilDiv(static_cast<int64_t>(g.wi), vo), kThreads);
            OPSCV_DISPATCH_DT(dt, T, {
                const T* pg = static_cast<const T*>(go);
                T* pi = static_cast<T*>(gi);
                OPSCV_DISPATCH_VEC(vo, VO, {
                    if constexpr (VO * sizeof(T) <= 16) {
                        Nearest3dBwdX2Kernel<T, VO><<<rl.grid, rl.block, 0, s>>>(pg, pi, g);
                    }
                });
            });
            CountLaunch();
            return cudaGetLastError();
        }
    }
    const RowLaunch rl = RowTiling(g.rows, inner, kThreads);
    OPSCV_DISPATCH_DT(dt, T, { Nearest3dBwdKernel<T><<<rl.grid, rl.block, 0, s>>>(static_cast<const T*>(go), static_cast<T*>(gi), g); });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
