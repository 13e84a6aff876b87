// UpsampleNearest2d forward and backward.
//
// Kernel schedules (chosen on the host from the exact index tables, see MakeNearestFwdPlan / MakeNearestBwdPlan):
//   * NCHW, integer up-scale factors (the common 2x / 4x case): input-major. A thread loads one 16-byte vector of
//     input, replicates its elements in registers and writes the RW * RH output vectors it feeds; the backward
//     loads RH 16-byte vectors of grads and reduces them to one output vector. Every global access is a
//     coalesced 16-byte access and nothing is read twice.
//   * NCHW, any other scale: output-major over shared memory. A block copies the input rows that its band of
//     output rows reads into shared memory (coalesced 16-byte loads, tile_stage.cuh); a thread owns one 16-byte
//     group of output columns, keeps their source columns in registers and walks down the rows of the band.
//   * NCHW rows too long to stage, or unaligned tensors: direct gather from global memory.
//   * NHWC: a gathered pixel is a contiguous run of channels, so taps are 16-byte global loads.
// The first version of the NCHW kernels gathered 2-byte elements straight from global memory and was bound by L1
// sector look-ups (ncu: l1tex throughput 85-95 %, 25 % of HBM peak); the schedules above remove that traffic.
//
// Reference arithmetic: image/resize_nearest_neighbor_v2/op_kernel/arch35/resize_nearest_neighbor_v2_simt.h:127-155
// (forward copy) and image/resize_nearest_neighbor_v2_grad/op_kernel/arch35/
// resize_nearest_neighbor_v2_grad_simt_determine.h:90-118 (backward: fp32 sum over the window, rows outer,
// columns inner, then one cast). All schedules keep that summation order, so results are bit-identical.
#include <algorithm>

#include "host_tables.h"
#include "launch_util.cuh"
#include "tile_stage.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;
constexpr int64_t kStageBudget = 24 * 1024; // staged bytes per block: keeps 8 blocks resident per SM

// ---- direct kernels (fallbacks; NHWC main path) ----------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdNCHWKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, const int32_t* __restrict__ sh, const int32_t* __restrict__ sw,
                         int64_t totalGroups)
{
    const int32_t groups = wout / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t row = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - row * groups);
        const int64_t p = row / hout;
        const int32_t h = static_cast<int32_t>(row - p * hout);
        const T* xr = x + (p * hin + __ldg(sh + h)) * static_cast<int64_t>(win);
        Pack<T, V> out;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            out.v[k] = __ldg(xr + __ldg(sw + g * V + k));
        }
        *reinterpret_cast<Pack<T, V>*>(y + row * wout + static_cast<int64_t>(g) * V) = out;
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdNHWCKernel(const T* __restrict__ x, T* __restrict__ y, int32_t c, int32_t hin, int32_t win,
                         int32_t hout, int32_t wout, const int32_t* __restrict__ sh,
                         const int32_t* __restrict__ sw, int64_t totalGroups)
{
    const int32_t groups = c / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t pix = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - pix * groups);
        const int64_t nh = pix / wout;
        const int32_t w = static_cast<int32_t>(pix - nh * wout);
        const int64_t n = nh / hout;
        const int32_t h = static_cast<int32_t>(nh - n * hout);
        const T* src = x + ((n * hin + __ldg(sh + h)) * win + __ldg(sw + w)) * static_cast<int64_t>(c) + g * V;
        *reinterpret_cast<Pack<T, V>*>(y + pix * c + static_cast<int64_t>(g) * V) =
            *reinterpret_cast<const Pack<T, V>*>(src);
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestBwdNCHWKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, RangeAxis th, RangeAxis tw, int64_t totalGroups)
{
    const int32_t groups = win / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t row = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - row * groups);
        const int64_t p = row / hin;
        const int32_t h = static_cast<int32_t>(row - p * hin);
        const int32_t hs = __ldg(th.start + h), he = __ldg(th.end + h);
        int32_t ws[V], we[V];
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            ws[k] = __ldg(tw.start + g * V + k);
            we[k] = __ldg(tw.end + g * V + k);
            acc[k] = 0.0f;
        }
        const T* gp = go + p * hout * static_cast<int64_t>(wout);
        for (int32_t i = hs; i < he; ++i) {
            const T* gr = gp + static_cast<int64_t>(i) * wout;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                for (int32_t j = ws[k]; j < we[k]; ++j) {
                    acc[k] = Add(acc[k], DType<T>::Load(gr + j));
                }
            }
        }
        StorePack<T, V>(gi + row * win + static_cast<int64_t>(g) * V, acc);
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestBwdNHWCKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t c, int32_t hin, int32_t win,
                         int32_t hout, int32_t wout, RangeAxis th, RangeAxis tw, int64_t totalGroups)
{
    const int32_t groups = c / V;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < totalGroups; gid += stride) {
        const int64_t pix = gid / groups;
        const int32_t g = static_cast<int32_t>(gid - pix * groups);
        const int64_t nh = pix / win;
        const int32_t w = static_cast<int32_t>(pix - nh * win);
        const int64_t n = nh / hin;
        const int32_t h = static_cast<int32_t>(nh - n * hin);
        const int32_t hs = __ldg(th.start + h), he = __ldg(th.end + h);
        const int32_t ws = __ldg(tw.start + w), we = __ldg(tw.end + w);
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            acc[k] = 0.0f;
        }
        for (int32_t i = hs; i < he; ++i) {
            for (int32_t j = ws; j < we; ++j) {
                float v[V];
                LoadPackLdg<T, V>(go + ((n * hout + i) * wout + j) * static_cast<int64_t>(c) + g * V, v);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    acc[k] = Add(acc[k], v[k]);
                }
            }
        }
        StorePack<T, V>(gi + pix * c + static_cast<int64_t>(g) * V, acc);
    }
}

// ---- NCHW, integer factors, input-major -------------------------------------------------------------------------
// Forward: out[h][w] = in[h / RH][w / RW]. grid.x = planes; a thread takes 16-byte input vectors of its plane.
// WIDE: the output rows are 32-byte aligned, so pairs of output vectors go out as one 32-byte store.
template <typename T, int RW, bool WIDE>
__global__ void __launch_bounds__(kThreads)
    NearestFwdReplicateKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t rh,
                              int64_t planes)
{
    constexpr int VI = 16 / sizeof(T);
    const int32_t vecsPerRow = win / VI;
    const int32_t vecsPerPlane = vecsPerRow * hin;
    const int32_t wout = win * RW;
    for (int64_t p = blockIdx.x; p < planes; p += gridDim.x) {
        const T* xp = x + p * hin * static_cast<int64_t>(win);
        T* yp = y + p * hin * static_cast<int64_t>(rh) * wout;
        for (int32_t v = threadIdx.x; v < vecsPerPlane; v += blockDim.x) {
            const int32_t r = v / vecsPerRow;
            const int32_t c0 = (v - r * vecsPerRow) * VI;
            const Pack<T, VI> in = *reinterpret_cast<const Pack<T, VI>*>(xp + static_cast<int64_t>(v) * VI);
            Pack<T, VI> out[RW];
#pragma unroll
            for (int o = 0; o < VI * RW; ++o) {
                out[o / VI].v[o % VI] = in.v[o / RW];
            }
            T* dst = yp + static_cast<int64_t>(r) * rh * wout + c0 * RW;
            for (int32_t i = 0; i < rh; ++i) {
#pragma unroll
                for (int q = 0; q < RW; ++q) {
                    if (WIDE && q + 1 < RW && q % 2 == 0) {
                        Store32Bytes(dst + q * VI, reinterpret_cast<const uint4&>(out[q]),
                                     reinterpret_cast<const uint4&>(out[q + 1]));
                    } else if (!(WIDE && q % 2 == 1)) {
                        *reinterpret_cast<Pack<T, VI>*>(dst + q * VI) = out[q];
                    }
                }
                dst += wout;
            }
        }
    }
}

// Backward: gi[y][x] = sum over the RH x RW block of grads, rows outer, columns inner (the reference's order).
// RH > 0: the row factor is known at compile time; the rows of a block are then loaded together before they are added.
template <typename T, int RW, int RH = 0>
__global__ void __launch_bounds__(kThreads)
    NearestBwdPoolKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t rh,
                         int64_t planes)
{
    constexpr int VI = 16 / sizeof(T); // grads elements per 16-byte load
    constexpr int VO = VI / RW;        // grad_input elements produced from them
    const int32_t wout = win * RW;
    const int32_t vecsPerRow = wout / VI;
    const int32_t vecsPerPlane = vecsPerRow * hin;
    for (int64_t p = blockIdx.x; p < planes; p += gridDim.x) {
        const T* gp = go + p * hin * static_cast<int64_t>(rh) * wout;
        T* op = gi + p * hin * static_cast<int64_t>(win);
        for (int32_t v = threadIdx.x; v < vecsPerPlane; v += blockDim.x) {
            const int32_t r = v / vecsPerRow;
            const int32_t cv = v - r * vecsPerRow;
            const T* src = gp + static_cast<int64_t>(r) * rh * wout + cv * VI;
            float acc[VO];
#pragma unroll
            for (int k = 0; k < VO; ++k) {
                acc[k] = 0.0f;
            }
            if constexpr (RH > 0) {
                float g[RH][VI];
#pragma unroll
                for (int i = 0; i < RH; ++i) {
                    LoadPackLdg<T, VI>(src + static_cast<int64_t>(i) * wout, g[i]);
                }
#pragma unroll
                for (int i = 0; i < RH; ++i) {
#pragma unroll
                    for (int k = 0; k < VO; ++k) {
#pragma unroll
                        for (int j = 0; j < RW; ++j) {
                            acc[k] = Add(acc[k], g[i][k * RW + j]);
                        }
                    }
                }
            } else {
                for (int32_t i = 0; i < rh; ++i) {
                    float g[VI];
                    LoadPackLdg<T, VI>(src, g);
#pragma unroll
                    for (int k = 0; k < VO; ++k) {
#pragma unroll
                        for (int j = 0; j < RW; ++j) {
                            acc[k] = Add(acc[k], g[k * RW + j]);
                        }
                    }
                    src += wout;
                }
            }
            StorePack<T, VO>(op + static_cast<int64_t>(r) * win + cv * VO, acc);
        }
    }
}

// ---- NCHW, any scale, shared-memory staged -----------------------------------------------------------------------
// grid = (planes, tiles per plane), block = (column threads, row threads); a tile is `tileRows` output rows of one plane, whose input rows
// [sh[h0], sh[h1-1]] are staged (the host sized the tile so that they fit).
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestFwdTileKernel(const T* __restrict__ x, T* __restrict__ y, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, const int32_t* __restrict__ sh, const int32_t* __restrict__ sw,
                         int32_t tileRows)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    const int64_t p = blockIdx.x;
    const int32_t tile = blockIdx.y;
    const int32_t h0 = tile * tileRows, h1 = min(hout, h0 + tileRows);
    const int32_t r0 = __ldg(sh + h0), r1 = __ldg(sh + h1 - 1) + 1;
    const T* plane = x + p * hin * static_cast<int64_t>(win);
    const T* src = StageSpan<T>(plane + static_cast<int64_t>(r0) * win, static_cast<int64_t>(r1 - r0) * win, smemRaw);
    __syncthreads();
    // blockDim = (column threads, row threads)
    const int32_t groups = wout / V;
    const int32_t colThreads = blockDim.x, rowThreads = blockDim.y;
    const int32_t cg0 = threadIdx.x, rc = threadIdx.y;
    T* yp = y + p * hout * static_cast<int64_t>(wout);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        int32_t col[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            col[k] = __ldg(sw + g * V + k);
        }
        T* dst = yp + static_cast<int64_t>(h0 + rc) * wout + g * V;
        for (int32_t h = h0 + rc; h < h1; h += rowThreads) {
            const T* row = src + (__ldg(sh + h) - r0) * win;
            Pack<T, V> out;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                out.v[k] = row[col[k]];
            }
            *reinterpret_cast<Pack<T, V>*>(dst) = out;
            dst += static_cast<int64_t>(rowThreads) * wout;
        }
    }
}

// A tile is `tileRows` grad_input rows of one plane; the grads rows of their windows are staged. Summation order
// per element: window rows outer, columns inner, in fp32.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
    NearestBwdTileKernel(const T* __restrict__ go, T* __restrict__ gi, int32_t hin, int32_t win, int32_t hout,
                         int32_t wout, RangeAxis th, RangeAxis tw, int32_t tileRows)
{
    extern __shared__ __align__(16) unsigned char smemRaw[];
    const int64_t p = blockIdx.x;
    const int32_t tile = blockIdx.y;
    const int32_t y0 = tile * tileRows, y1 = min(hin, y0 + tileRows);
    const int32_t r0 = __ldg(th.start + y0);
    const int32_t r1 = max(r0, __ldg(th.end + y1 - 1));
    const T* plane = go + p * hout * static_cast<int64_t>(wout);
    const T* src = StageSpan<T>(plane + static_cast<int64_t>(r0) * wout, static_cast<int64_t>(r1 - r0) * wout,
                                smemRaw);
    __syncthreads();
    // blockDim = (column threads, row threads)
    const int32_t groups = win / V;
    const int32_t colThreads = blockDim.x, rowThreads = blockDim.y;
    const int32_t cg0 = threadIdx.x, rc = threadIdx.y;
    T* gp = gi + p * hin * static_cast<int64_t>(win);
    for (int32_t g = cg0; g < groups; g += colThreads) {
        int32_t ws[V], we[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            ws[k] = __ldg(tw.start + g * V + k);
            we[k] = __ldg(tw.end + g * V + k);
        }
        for (int32_t yy = y0 + rc; yy < y1; yy += rowThreads) {
            const int32_t hs = __ldg(th.start + yy), he = __ldg(th.end + yy);
            float acc[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                acc[k] = 0.0f;
            }
            for (int32_t i = hs; i < he; ++i) {
                const T* row = src + (i - r0) * wout;
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    for (int32_t j = ws[k]; j < we[k]; ++j) {
                        acc[k] = Add(acc[k], DType<T>::ToF(row[j]));
                    }
                }
            }
            StorePack<T, V>(gp + static_cast<int64_t>(yy) * win + g * V, acc);
        }
    }
}

bool IsIntegerReplication(const std::vector<int32_t>& src, int32_t factor)
{
    for (size_t d = 0; d < src.size(); ++d) {
        if (src[d] != static_cast<int32_t>(d) / factor) {
            return false;
        }
    }
    return true;
}

bool IsIntegerPooling(const host::Ranges& r, int32_t factor)
{
    for (size_t y = 0; y < r.start.size(); ++y) {
        if (r.start[y] != static_cast<int32_t>(y) * factor || r.end[y] != static_cast<int32_t>(y + 1) * factor) {
            return false;
        }
    }
    return true;
}

} // namespace

NearestPlan MakeNearestFwdPlan(Dt dt, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw)
{
    NearestPlan plan{};
    plan.schedule = NearestPlan::kDirect;
    if (lay != kNCHW) {
        return plan;
    }
    const int es = DtSize(dt), vi = 16 / es;
    const std::vector<int32_t> srcH = host::NearestSrc(sh.hin, sh.hout, gh.scale, gh.exact != 0);
    const std::vector<int32_t> srcW = host::NearestSrc(sh.win, sh.wout, gw.scale, gw.exact != 0);
    const int32_t rh = sh.hout / sh.hin, rw = sh.wout / sh.win;
    if (sh.hout == rh * sh.hin && sh.wout == rw * sh.win && (rw == 2 || rw == 3 || rw == 4) && sh.win % vi == 0 &&
        IsIntegerReplication(srcH, rh) && IsIntegerReplication(srcW, rw)) {
        plan.schedule = NearestPlan::kInteger;
        plan.rh = rh;
        plan.rw = rw;
        return plan;
    }
    const int64_t rowBytes = static_cast<int64_t>(sh.win) * es;
    const int32_t budgetRows = static_cast<int32_t>(std::min<int64_t>(kStageBudget / rowBytes, sh.hin));
    auto need = [&](int32_t h0, int32_t h1) { return srcH[h1 - 1] - srcH[h0] + 1; };
    const int32_t tileRows = host::PickTileRows(sh.hout, budgetRows, need);
    if (tileRows > 0 && sh.n * sh.c < (1LL << 31) && CeilDiv(sh.hout, tileRows) <= 65535) {
        plan.schedule = NearestPlan::kTiled;
        plan.tileRows = tileRows;
        plan.bandRows = host::MaxBand(sh.hout, tileRows, need);
    }
    return plan;
}

NearestPlan MakeNearestBwdPlan(Dt dt, Layout lay, Shape4 sh, AxisGeom gh, AxisGeom gw)
{
    NearestPlan plan{};
    plan.schedule = NearestPlan::kDirect;
    if (lay != kNCHW) {
        return plan;
    }
    const int es = DtSize(dt), vi = 16 / es;
    const host::Ranges rH = host::NearestBwdRanges(sh.hin, sh.hout, gh.scale, gh.exact != 0);
    const host::Ranges rW = host::NearestBwdRanges(sh.win, sh.wout, gw.scale, gw.exact != 0);
    const int32_t rh = sh.hout / sh.hin, rw = sh.wout / sh.win;
    if (sh.hout == rh * sh.hin && sh.wout == rw * sh.win && (rw == 2 || rw == 4) && sh.wout % vi == 0 &&
        IsIntegerPooling(rH, rh) && IsIntegerPooling(rW, rw)) {
        plan.schedule = NearestPlan::kInteger;
        plan.rh = rh;
        plan.rw = rw;
        return plan;
    }
    const int64_t rowBytes = static_cast<int64_t>(sh.wout) * es;
    const int32_t budgetRows = static_cast<int32_t>(std::min<int64_t>(kStageBudget / rowBytes, sh.hout));
    auto need = [&](int32_t y0, int32_t y1) { return std::max(0, rH.end[y1 - 1] - rH.start[y0]); };
    const int32_t tileRows = host::PickTileRows(sh.hin, budgetRows, need);
    if (tileRows > 0 && sh.n * sh.c < (1LL << 31) && CeilDiv(sh.hin, tileRows) <= 65535) {
        plan.schedule = NearestPlan::kTiled;
        plan.tileRows = tileRows;
        plan.bandRows = host::MaxBand(sh.hin, tileRows, need);
    }
    return plan;
}

// The integer-factor kernels address everything arithmetically and need 16-byte aligned rows; when they apply
// the index tables are not read at all (the host then skips building them).
bool NearestFwdUsesInteger(Dt dt, Layout lay, const void* x, const void* y, Shape4 sh, const NearestPlan& plan)
{
    const int vi = 16 / DtSize(dt);
    return lay == kNCHW && plan.schedule == NearestPlan::kInteger && sh.wout % vi == 0 && Aligned(x, 16) &&
           Aligned(y, 16);
}

bool NearestBwdUsesInteger(Dt dt, Layout lay, const void* go, const void* gi, Shape4 sh, const NearestPlan& plan)
{
    const int vi = 16 / DtSize(dt);
    return lay == kNCHW && plan.schedule == NearestPlan::kInteger && sh.wout % vi == 0 && Aligned(go, 16) &&
           Aligned(gi, static_cast<size_t>(16 / plan.rw));
}

cudaError_t NearestFwd(Dt dt, Layout lay, const void* x, void* y, Shape4 sh, NearestAxis th, NearestAxis tw,
                       const NearestPlan& plan, cudaStream_t s)
{
    const int64_t planes = sh.n * sh.c;
    OPSCV_DISPATCH_DT(dt, T, {
        if (lay == kNCHW) {
            const int v = PickVec(sizeof(T), sh.wout, {y});
            if (NearestFwdUsesInteger(dt, lay, x, y, sh, plan)) {
                const unsigned blocks = static_cast<unsigned>(std::min<int64_t>(planes, 1 << 30));
                const T* px = static_cast<const T*>(x);
                T* py = static_cast<T*>(y);
                // 32-byte stores need 32-byte aligned output rows (a thread's first column is a multiple of 32 bytes)
                const bool wide = plan.rw != 3 && Aligned(y, 32) && (sh.wout * sizeof(T)) % 32 == 0;
                if (plan.rw == 2 && wide) {
                    NearestFwdReplicateKernel<T, 2, true><<<blocks, kThreads, 0, s>>>(px, py, sh.hin, sh.win, plan.rh, planes);
                } else if (plan.rw == 2) {
                    NearestFwdReplicateKernel<T, 2, false><<<blocks, kThreads, 0, s>>>(px, py, sh.hin, sh.win, plan.rh, planes);
                } else if (plan.rw == 3) {
                    NearestFwdReplicateKernel<T, 3, false><<<blocks, kThreads, 0, s>>>(px, py, sh.hin, sh.win, plan.rh, planes);
                } else if (wide) {
                    NearestFwdReplicateKernel<T, 4, true><<<blocks, kThreads, 0, s>>>(px, py, sh.hin, sh.win, plan.rh, planes);
                } else {
                    NearestFwdReplicateKernel<T, 4, false><<<blocks, kThreads, 0, s>>>(px, py, sh.hin, sh.win, plan.rh, planes);
                }
            } else {
                OPSCV_DISPATCH_VEC(v, V, {
                    if constexpr (V * sizeof(T) <= 16) {
                        if (plan.schedule != NearestPlan::kDirect && plan.tileRows > 0) {
                            const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hout, plan.tileRows));
                            const size_t smem = StageBytes(static_cast<int64_t>(plan.bandRows) * sh.win, sizeof(T));
                            const dim3 grid(static_cast<unsigned>(planes), static_cast<unsigned>(tiles));
                            NearestFwdTileKernel<T, V><<<grid, TileBlock(sh.wout / V, plan.tileRows, 8), smem, s>>>(
                                static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th.src,
                                tw.src, plan.tileRows);
                        } else {
                            const int64_t total = planes * sh.hout * (sh.wout / V);
                            NearestFwdNCHWKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                                static_cast<const T*>(x), static_cast<T*>(y), sh.hin, sh.win, sh.hout, sh.wout, th.src,
                                tw.src, total);
                        }
                    }
                });
            }
        } else {
            const int v = PickVec(sizeof(T), sh.c, {x, y});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    const int64_t total = sh.n * sh.hout * sh.wout * (sh.c / V);
                    NearestFwdNHWCKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(x), static_cast<T*>(y), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                        sh.hout, sh.wout, th.src, tw.src, total);
                }
            });
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t NearestBwd(Dt dt, Layout lay, const void* go, void* gi, Shape4 sh, RangeAxis th, RangeAxis tw,
                       const NearestPlan& plan, cudaStream_t s)
{
    const int64_t planes = sh.n * sh.c;
    OPSCV_DISPATCH_DT(dt, T, {
        if (lay == kNCHW) {
            const int v = PickVec(sizeof(T), sh.win, {gi});
            if (NearestBwdUsesInteger(dt, lay, go, gi, sh, plan)) {
                const unsigned blocks = static_cast<unsigned>(std::min<int64_t>(planes, 1 << 30));
                const T* pg = static_cast<const T*>(go);
                T* po = static_cast<T*>(gi);
                if (plan.rw == 2 && plan.rh == 2) {
                    NearestBwdPoolKernel<T, 2, 2><<<blocks, kThreads, 0, s>>>(pg, po, sh.hin, sh.win, plan.rh, planes);
                } else if (plan.rw == 2) {
                    NearestBwdPoolKernel<T, 2><<<blocks, kThreads, 0, s>>>(pg, po, sh.hin, sh.win, plan.rh, planes);
                } else {
                    NearestBwdPoolKernel<T, 4><<<blocks, kThreads, 0, s>>>(pg, po, sh.hin, sh.win, plan.rh, planes);
                }
            } else {
                OPSCV_DISPATCH_VEC(v, V, {
                    if constexpr (V * sizeof(T) <= 16) {
                        if (plan.schedule != NearestPlan::kDirect && plan.tileRows > 0) {
                            const int32_t tiles = static_cast<int32_t>(CeilDiv(sh.hin, plan.tileRows));
                            const size_t smem = StageBytes(static_cast<int64_t>(plan.bandRows) * sh.wout, sizeof(T));
                            const dim3 grid(static_cast<unsigned>(planes), static_cast<unsigned>(tiles));
                            NearestBwdTileKernel<T, V><<<grid, TileBlock(sh.win / V, plan.tileRows, 8), smem, s>>>(
                                static_cast<const T*>(go), static_cast<T*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th,
                                tw, plan.tileRows);
                        } else {
                            const int64_t total = planes * sh.hin * (sh.win / V);
                            NearestBwdNCHWKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                                static_cast<const T*>(go), static_cast<T*>(gi), sh.hin, sh.win, sh.hout, sh.wout, th,
                                tw, total);
                        }
                    }
                });
            }
        } else {
            const int v = PickVec(sizeof(T), sh.c, {go, gi});
            OPSCV_DISPATCH_VEC(v, V, {
                if constexpr (V * sizeof(T) <= 16) {
                    const int64_t total = sh.n * sh.hin * sh.win * (sh.c / V);
                    NearestBwdNHWCKernel<T, V><<<GridFor(total, kThreads), kThreads, 0, s>>>(
                        static_cast<const T*>(go), static_cast<T*>(gi), static_cast<int32_t>(sh.c), sh.hin, sh.win,
                        sh.hout, sh.wout, th, tw, total);
                }
            });
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
