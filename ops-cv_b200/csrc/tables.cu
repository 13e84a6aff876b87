// Per-axis index / weight tables. Shapes and scales are known on the host, but the tables are built by tiny
// kernels in stream order (no host->device copy whose source would have to outlive the call), into the caller's
// workspace. They are O(H + W), shared by all N*C planes, and stay resident in L1/L2 for the main kernels.
//
// Every expression keeps the operation order of the reference's arch35 SIMT kernels and uses the non-fusing
// intrinsics from common.cuh, so the integer tables (source indices, window bounds) and the fp32 weights can be
// checked bit for bit against a CPU statement of the same formulas.
#include <algorithm>
#include "common.cuh"
#include "kernels.h"
#include "lerp_entry.cuh"

namespace opscv {

namespace {

constexpr int kTableThreads = 128;

inline dim3 TableGrid(int32_t a, int32_t b)
{
    int32_t m = a > b ? a : b;
    if (m < 1) {
        m = 1;
    }
    return dim3(static_cast<unsigned>((m + kTableThreads - 1) / kTableThreads), 2, 1);
}

// ---- nearest ---------------------------------------------------------------------------------------------
// image/resize_nearest_neighbor_v2/op_kernel/arch35/resize_nearest_neighbor_v2_simt.h:104-124
// (align_corners = false, half_pixel_centers = false: src = min(floor(dst * scale), in - 1))
__global__ void NearestFwdTableKernel(AxisGeom gh, AxisGeom gw, NearestAxis th, NearestAxis tw)
{
    const AxisGeom g = blockIdx.y == 0 ? gh : gw;
    int32_t* src = blockIdx.y == 0 ? th.src : tw.src;
    const int32_t d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= g.out) {
        return;
    }
    // exact: half_pixel_centers = true, resize_nearest_neighbor_v2_simt.h:115-117
    const float pos = g.exact ? Add(static_cast<float>(d), 0.5f) : static_cast<float>(d);
    long long s = static_cast<long long>(floorf(Mul(pos, g.scale)));
    const long long last = g.in - 1;
    src[d] = static_cast<int32_t>(s < last ? s : last);
}

// image/resize_nearest_neighbor_v2_grad/op_kernel/arch35/resize_nearest_neighbor_v2_grad_simt_determine.h:79-88
// window of grads indices feeding grad_input index y: [min(ceil(y*inv), out), min(ceil((y+1)*inv), out))
__global__ void NearestBwdTableKernel(AxisGeom gh, AxisGeom gw, RangeAxis th, RangeAxis tw)
{
    const AxisGeom g = blockIdx.y == 0 ? gh : gw;
    const RangeAxis t = blockIdx.y == 0 ? th : tw;
    const int32_t y = blockIdx.x * blockDim.x + threadIdx.x;
    if (y >= g.in) {
        return;
    }
    long long a, b;
    if (g.exact) {
        // image/upsample_nearest_exact2d_grad/op_kernel/arch35/upsample_nearest_exact2d_grad_simt_base.h:33-43
        a = static_cast<long long>(ceilf(Sub(Mul(static_cast<float>(y), g.scale), 0.5f)));
        b = static_cast<long long>(ceilf(Sub(Mul(static_cast<float>(y + 1), g.scale), 0.5f)));
    } else {
        const float inv = Div(1.0f, g.scale);
        a = static_cast<long long>(ceilf(Mul(static_cast<float>(y), inv)));
        b = static_cast<long long>(ceilf(Mul(static_cast<float>(y + 1), inv)));
    }
    const long long lim = g.out;
    a = a < lim ? a : lim;
    b = b < lim ? b : lim;
    if (a < 0) {
        a = 0;
    }
    if (b < a) {
        b = a;
    }
    t.start[y] = static_cast<int32_t>(a);
    t.end[y] = static_cast<int32_t>(b);
}

// ---- bilinear --------------------------------------------------------------------------------------------
// variant 0: image/resize_bilinear_v2/op_kernel/arch35/resize_bilinear_v2_simt_nchw.h:110-133
// variant 1: image/resize_bilinear_v2_grad/op_kernel/arch35/resize_bilinear_v2_grad_simt.h:121-135
__global__ void LerpTableKernel(AxisGeom gh, AxisGeom gw, int halfPixel, int variant, LerpAxis th, LerpAxis tw)
{
    const AxisGeom g = blockIdx.y == 0 ? gh : gw;
    const LerpAxis t = blockIdx.y == 0 ? th : tw;
    const int32_t d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= g.out) {
        return;
    }
    int32_t lo, hi;
    float delta;
    LerpEntry(g, halfPixel, variant, d, lo, hi, delta);
    t.lo[d] = lo;
    t.hi[d] = hi;
    t.delta[d] = delta;
}

// The backward tables (variant 1) and their transposed ranges in one launch: blockIdx.y = 0, 1 write the tables of
// the two axes, 2, 3 the ranges. The range search evaluates table entries from the formula instead of reading
// them, so it does not have to wait for the table blocks; the entries are the same bits either way.
__global__ void LerpBwdTablesAndRangesKernel(AxisGeom gh, AxisGeom gw, int halfPixel, LerpAxis th, LerpAxis tw,
                                             RangeAxis rh, RangeAxis rw)
{
    const bool axisW = (blockIdx.y & 1) != 0;
    const AxisGeom g = axisW ? gw : gh;
    const int32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (blockIdx.y < 2) {
        const LerpAxis t = axisW ? tw : th;
        if (idx < g.out) {
            int32_t lo, hi;
            float delta;
            LerpEntry(g, halfPixel, 1, idx, lo, hi, delta);
            t.lo[idx] = lo;
            t.hi[idx] = hi;
            t.delta[idx] = delta;
        }
        return;
    }
    const RangeAxis r = axisW ? rw : rh;
    const int32_t y = idx;
    if (y >= g.in) {
        return;
    }
    int32_t lo, hi;
    float delta;
    // first i with hi[i] >= y
    int32_t a = 0, b = g.out;
    while (a < b) {
        const int32_t m = a + ((b - a) >> 1);
        LerpEntry(g, halfPixel, 1, m, lo, hi, delta);
        if (hi >= y) {
            b = m;
        } else {
            a = m + 1;
        }
    }
    const int32_t first = a;
    // first i with lo[i] > y
    a = first;
    b = g.out;
    while (a < b) {
        const int32_t m = a + ((b - a) >> 1);
        LerpEntry(g, halfPixel, 1, m, lo, hi, delta);
        if (lo > y) {
            b = m;
        } else {
            a = m + 1;
        }
    }
    r.start[y] = first;
    r.end[y] = a > first ? a : first;
}

// Transposed ranges for the gather backward. lo and hi are non-decreasing in the grads index, and hi <= lo + 1,
// so the grads indices that touch grad_input index y are the contiguous run {i : lo[i] <= y <= hi[i]}.
__global__ void LerpBwdRangeKernel(AxisGeom gh, AxisGeom gw, LerpAxis th, LerpAxis tw, RangeAxis rh, RangeAxis rw)
{
    const AxisGeom g = blockIdx.y == 0 ? gh : gw;
    const LerpAxis t = blockIdx.y == 0 ? th : tw;
    const RangeAxis r = blockIdx.y == 0 ? rh : rw;
    const int32_t y = blockIdx.x * blockDim.x + threadIdx.x;
    if (y >= g.in) {
        return;
    }
    // first i with hi[i] >= y
    int32_t a = 0, b = g.out;
    while (a < b) {
        const int32_t m = a + ((b - a) >> 1);
        if (t.hi[m] >= y) {
            b = m;
        } else {
            a = m + 1;
        }
    }
    const int32_t first = a;
    // first i with lo[i] > y
    a = first;
    b = g.out;
    while (a < b) {
        const int32_t m = a + ((b - a) >> 1);
        if (t.lo[m] > y) {
            b = m;
        } else {
            a = m + 1;
        }
    }
    r.start[y] = first;
    r.end[y] = a > first ? a : first;
}

// ---- bicubic, anti-aliased ------------------------------------------------------------------------------------
// image/upsample_bicubic2d_aa/op_kernel/arch35/upsample_bicubic2d_aa_simt_base.h:31-50 (Keys cubic, a = -0.5)
__device__ __forceinline__ float CubicFilterAA(float m)
{
    m = fabsf(m);
    if (m < 1.0f) {
        return Add(Mul(Mul(Sub(Mul(1.5f, m), 2.5f), m), m), 1.0f);
    } else if (m < 2.0f) {
        return Add(Mul(Sub(Mul(Add(Mul(-0.5f, m), 2.5f), m), 4.0f), m), 2.0f);
    }
    return 0.0f;
}

// image/upsample_bilinear2d_aa/op_kernel/arch35/upsample_bilinear2d_aa_simt_base.h:30-37 (triangle)
__device__ __forceinline__ float TriangleFilterAA(float m)
{
    m = fabsf(m);
    return m < 1.0f ? Sub(1.0f, m) : 0.0f;
}
__device__ __forceinline__ float FilterAA(int filter, float m)
{
    return filter == 0 ? CubicFilterAA(m) : TriangleFilterAA(m);
}

// upsample_bicubic2d_aa_simt_base.h:70-124 and upsample_bilinear2d_aa_simt_base.h:52-88: window
// [xmin, xmin+xsize), weights normalised by their sum. filter: 0 Keys cubic, 1 triangle.
__global__ void AATableKernel(AxisGeom gh, AxisGeom gw, float invH, float invW, float supH, float supW, AAAxis th,
                              AAAxis tw, int backward, int filter)
{
    const bool isH = blockIdx.y == 0;
    const AxisGeom g = isH ? gh : gw;
    const AAAxis t = isH ? th : tw;
    const float inv = isH ? invH : invW;
    const float support = isH ? supH : supW;
    const int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= g.out) {
        return;
    }
    // The backward kernel places the centre at 0.5 when the scale is 0 (align_corners with a single output,
    // upsample_bicubic2d_aa_grad_simt_base.h:38); the forward kernel does not (simt_base.h:72-73).
    float center = Mul(g.scale, Add(static_cast<float>(i), 0.5f));
    if (backward) {
        center = (g.scale > 0.0f) ? Mul(Add(static_cast<float>(i), 0.5f), g.scale) : 0.5f;
    }
    long long lo = static_cast<long long>(floorf(Add(Sub(center, support), 0.5f)));
    long long hi = static_cast<long long>(floorf(Add(Add(center, support), 0.5f)));
    lo = lo > 0 ? lo : 0;
    hi = hi < g.in ? hi : g.in;
    long long size = hi - lo;
    if (size < 0) {
        size = 0;
    }
    if (size > t.taps) { // cannot happen when taps is sized from the support; keeps the writes in bounds
        size = t.taps;
    }
    t.xmin[i] = static_cast<int32_t>(lo);
    t.xsize[i] = static_cast<int32_t>(size);
    float total = 0.0f;
    for (int32_t j = 0; j < size; ++j) {
        const float dist = Mul(Add(Sub(static_cast<float>(lo + j), center), 0.5f), inv);
        total = Add(total, FilterAA(filter, dist));
    }
    float* w = t.w + static_cast<int64_t>(i) * t.taps;
    for (int32_t j = 0; j < t.taps; ++j) {
        float wj = 0.0f;
        if (j < size) {
            const float dist = Mul(Add(Sub(static_cast<float>(lo + j), center), 0.5f), inv);
            wj = FilterAA(filter, dist);
            if (total != 0.0f) {
                wj = Div(wj, total);
            }
        }
        w[j] = wj;
    }
}

// Output indices whose window covers forward-input index y. xmin and xmin+xsize are non-decreasing in i.
__global__ void AABwdRangeKernel(AxisGeom gh, AxisGeom gw, AAAxis th, AAAxis tw, RangeAxis rh, RangeAxis rw)
{
    const bool isH = blockIdx.y == 0;
    const AxisGeom g = isH ? gh : gw;
    const AAAxis t = isH ? th : tw;
    const RangeAxis r = isH ? rh : rw;
    const int32_t y = blockIdx.x * blockDim.x + threadIdx.x;
    if (y >= g.in) {
        return;
    }
    int32_t a = 0, b = g.out;
    while (a < b) { // first i with xmin[i] + xsize[i] > y
        const int32_t m = a + ((b - a) >> 1);
        if (t.xmin[m] + t.xsize[m] > y) {
            b = m;
        } else {
            a = m + 1;
        }
    }
    const int32_t first = a;
    b = g.out;
    while (a < b) { // first i with xmin[i] > y
        const int32_t m = a + ((b - a) >> 1);
        if (t.xmin[m] > y) {
            b = m;
        } else {
            a = m + 1;
        }
    }
    r.start[y] = first;
    r.end[y] = a > first ? a : first;
}

} // namespace

cudaError_t BuildNearestFwdTables(AxisGeom h, AxisGeom w, NearestAxis th, NearestAxis tw, cudaStream_t s)
{
    NearestFwdTableKernel<<<TableGrid(h.out, w.out), kTableThreads, 0, s>>>(h, w, th, tw);
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BuildNearestBwdTables(AxisGeom h, AxisGeom w, RangeAxis th, RangeAxis tw, cudaStream_t s)
{
    NearestBwdTableKernel<<<TableGrid(h.in, w.in), kTableThreads, 0, s>>>(h, w, th, tw);
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BuildLerpTables(AxisGeom h, AxisGeom w, bool halfPixel, int variant, LerpAxis th, LerpAxis tw,
                            cudaStream_t s)
{
    LerpTableKernel<<<TableGrid(h.out, w.out), kTableThreads, 0, s>>>(h, w, halfPixel ? 1 : 0, variant, th, tw);
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BuildLerpBwdRanges(AxisGeom h, AxisGeom w, LerpAxis th, LerpAxis tw, RangeAxis rh, RangeAxis rw,
                               cudaStream_t s)
{
    LerpBwdRangeKernel<<<TableGrid(h.in, w.in), kTableThreads, 0, s>>>(h, w, th, tw, rh, rw);
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BuildLerpBwdTablesAndRanges(AxisGeom h, AxisGeom w, bool halfPixel, LerpAxis th, LerpAxis tw, RangeAxis rh,
                                        RangeAxis rw, cudaStream_t s)
{
    dim3 grid = TableGrid(std::max(h.out, h.in), std::max(w.out, w.in));
    grid.y = 4;
    LerpBwdTablesAndRangesKernel<<<grid, kTableThreads, 0, s>>>(h, w, halfPixel ? 1 : 0, th, tw, rh, rw);
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BuildAATables(AxisGeom h, AxisGeom w, float invH, float invW, float supH, float supW, AAAxis th,
                          AAAxis tw, bool backward, int filter, cudaStream_t s)
{
    AATableKernel<<<TableGrid(h.out, w.out), kTableThreads, 0, s>>>(h, w, invH, invW, supH, supW, th, tw,
                                                                    backward ? 1 : 0, filter);
    CountLaunch();
    return cudaGetLastError();
}

cudaError_t BuildAABwdRanges(AxisGeom h, AxisGeom w, AAAxis th, AAAxis tw, RangeAxis rh, RangeAxis rw,
                             cudaStream_t s)
{
    AABwdRangeKernel<<<TableGrid(h.in, w.in), kTableThreads, 0, s>>>(h, w, th, tw, rh, rw);
    CountLaunch();
    return cudaGetLastError();
}

} // namespace opscv
