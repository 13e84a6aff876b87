// GridSampler3D forward (bilinear, plus nearest) and GridSampler3DGrad (bilinear, nearest) on NCDHW and NDHWC tensors
// with a (N, Do, Ho, Wo, 3) grid of (x, y, z) points.
//
// Forward: image/grid_sample/op_kernel/arch35/grid_sampler_3d_bilinear_smit.h:58-184 and
// grid_sampler_bilinear_smit_common.h:37-91. A thread owns one output point of one image: it reads the grid point
// once, forms the eight weights, and walks the channels (stores of a warp are contiguous along the points).
// Backward: image/grid_sampler3_d_grad/op_kernel/arch35/grid_sampler3_d_grad_simt.h:43-300 with the coordinate
// helpers of grid_sampler3_d_grad_simt_base.h:46-168 (the ones the 2-D backward uses). grad_input is accumulated
// with fp32 atomics (in place for fp32 tensors, in a workspace that is cast afterwards for 16-bit ones); grad_grid
// is one thread's sum over the channels in the reference's corner and channel order.
#include <algorithm>

#include "grid_coords.cuh"
#include "launch_util.cuh"

namespace opscv {
namespace {

constexpr int kThreads = 256;

// grid_sampler_bilinear_smit_common.h:37-91
__device__ __forceinline__ float Clip3(float coord, int32_t size)
{
    coord = coord < 0 ? 0 : coord;
    coord = coord > (size - 1) ? static_cast<float>(size) - 1 : coord;
    if (isnan(coord) || isinf(coord)) {
        return 0.0f;
    }
    return coord;
}
__device__ __forceinline__ float Reflect3(float coord, int32_t twiceLow, int32_t twiceHigh)
{
    if (twiceLow == twiceHigh) {
        return 0.0f;
    }
    const float mn = Div(static_cast<float>(twiceLow), 2.0f);
    const float span = Div(static_cast<float>(twiceHigh - twiceLow), 2.0f);
    coord = fabsf(Sub(coord, mn));
    const float extra = fmodf(coord, span);
    const long long flips = static_cast<long long>(floorf(Div(coord, span)));
    return flips % 2 == 0 ? Add(extra, mn) : Add(Sub(span, extra), mn);
}
__device__ __forceinline__ float SourcePoint3(float gv, int32_t size, int32_t pad, int32_t align)
{
    float coord = align == 1 ? Mul(Div(Add(gv, 1.0f), 2.0f), static_cast<float>(size - 1))
                             : Div(Sub(Mul(Add(gv, 1.0f), static_cast<float>(size)), 1.0f), 2.0f);
    if (pad == 1) {
        coord = Clip3(coord, size);
    } else if (pad == 2) {
        coord = align ? Reflect3(coord, 0, 2 * (size - 1)) : Reflect3(coord, -1, 2 * size - 1);
        coord = Clip3(coord, size);
    }
    return isfinite(coord) ? coord : -100.0f;
}

__device__ __forceinline__ bool Inside3(float d, float h, float w, const Grid3dShape& g)
{
    return d >= 0 && h >= 0 && w >= 0 && d < g.di && h < g.hi && w < g.wi;
}

// CL: channels-last tensors (NDHWC): the channels of a voxel are contiguous, so a tap of a point is one contiguous run
// of C elements and the channel loop reads and writes V of them at a time; NCDHW: V = 1 and channels are a plane apart.
template <typename T, bool CL, int V>
__global__ void __launch_bounds__(kThreads) GridSampler3dFwdKernel(const T* __restrict__ x, const T* __restrict__ grid,
                                                                    T* __restrict__ y, Grid3dShape g)
{
    const int64_t outVol = static_cast<int64_t>(g.dout) * g.ho * g.wo, inVol = static_cast<int64_t>(g.di) * g.hi * g.wi;
    const int64_t total = g.n * outVol;
    const int64_t cs = CL ? 1 : inVol, vs = CL ? g.c : 1;       // channel / voxel stride of the input
    const int64_t ocs = CL ? 1 : outVol, ovs = CL ? g.c : 1;    // of the output
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int64_t n = idx / outVol, p = idx - n * outVol;
        const T* gp = grid + idx * 3;
        const float pw = SourcePoint3(DType<T>::Load(gp), g.wi, g.pad, g.align);
        const float ph = SourcePoint3(DType<T>::Load(gp + 1), g.hi, g.pad, g.align);
        const float pd = SourcePoint3(DType<T>::Load(gp + 2), g.di, g.pad, g.align);
        const T* xb = x + n * g.c * inVol;
        T* yb = y + n * g.c * outVol + p * ovs;
        if (g.interp == 1) { // nearest: the rounding of the backward kernel (rint)
            const float dn = rintf(pd), hn = rintf(ph), wn = rintf(pw);
            const bool in = Inside3(dn, hn, wn, g);
            const int64_t off = in ? ((static_cast<int64_t>(dn) * g.hi + static_cast<int64_t>(hn)) * g.wi + static_cast<int64_t>(wn)) * vs : 0;
            for (int64_t c = 0; c < g.c; c += V) {
                float v[V];
                if (in) {
                    LoadPack<T, V>(xb + c * cs + off, v);
                } else {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        v[k] = 0.0f;
                    }
                }
                StorePack<T, V>(yb + c * ocs, v);
            }
            continue;
        }
        const float df = floorf(pd), hf = floorf(ph), wf = floorf(pw);
        const float dd = Sub(pd, df), hd = Sub(ph, hf), wd = Sub(pw, wf);
        const float wd0 = Sub(1.0f, wd), hd0 = Sub(1.0f, hd), dd0 = Sub(1.0f, dd);
        float wt[8];
        int64_t off[8];
        bool in[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool east = (k & 1) != 0, south = (k & 2) != 0, back = (k & 4) != 0;
            wt[k] = Mul(Mul(east ? wd : wd0, south ? hd : hd0), back ? dd : dd0);
            const float d = back ? Add(df, 1.0f) : df, h = south ? Add(hf, 1.0f) : hf, w = east ? Add(wf, 1.0f) : wf;
            in[k] = Inside3(d, h, w, g);
            off[k] = in[k] ? ((static_cast<int64_t>(d) * g.hi + static_cast<int64_t>(h)) * g.wi + static_cast<int64_t>(w)) * vs : 0;
        }
        for (int64_t c = 0; c < g.c; c += V) {
            const T* xc = xb + c * cs;
            float acc[V], t[V];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (in[k]) {
                    LoadPack<T, V>(xc + off[k], t);
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        t[v] = 0.0f;
                    }
                }
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    acc[v] = k == 0 ? Mul(t[v], wt[0]) : Add(acc[v], Mul(t[v], wt[k]));
                }
            }
            StorePack<T, V>(yb + c * ocs, acc);
        }
    }
}

// Channels-last forward with the channel vectors of a point on adjacent lanes: thread t owns channel vector t % G of
// point t / G (G = C / V), so the G lanes of a point read each tap as one contiguous run of C elements and write the
// point's C outputs as one run. Every lane of a point evaluates the point's coordinates itself (a hundred
// instructions against eight 16-byte loads); the sums are those of the kernel above, in the same order.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads) GridSampler3dFwdLanesKernel(const T* __restrict__ x, const T* __restrict__ grid,
                                                                         T* __restrict__ y, Grid3dShape g, int32_t groups)
{
    const int64_t outVol = static_cast<int64_t>(g.dout) * g.ho * g.wo, inVol = static_cast<int64_t>(g.di) * g.hi * g.wi;
    const int64_t total = g.n * outVol * groups;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; t < total;
         t += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int64_t idx = t / groups;
        const int64_t c = (t - idx * groups) * V;
        const int64_t n = idx / outVol;
        const T* gp = grid + idx * 3;
        const float pw = SourcePoint3(DType<T>::Load(gp), g.wi, g.pad, g.align);
        const float ph = SourcePoint3(DType<T>::Load(gp + 1), g.hi, g.pad, g.align);
        const float pd = SourcePoint3(DType<T>::Load(gp + 2), g.di, g.pad, g.align);
        const T* xb = x + n * g.c * inVol + c;
        T* yp = y + idx * g.c + c;
        float acc[V], tv[V];
        if (g.interp == 1) {
            const float dn = rintf(pd), hn = rintf(ph), wn = rintf(pw);
            if (Inside3(dn, hn, wn, g)) {
                LoadPack<T, V>(xb + ((static_cast<int64_t>(dn) * g.hi + static_cast<int64_t>(hn)) * g.wi + static_cast<int64_t>(wn)) * g.c, acc);
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    acc[v] = 0.0f;
                }
            }
            StorePack<T, V>(yp, acc);
            continue;
        }
        const float df = floorf(pd), hf = floorf(ph), wf = floorf(pw);
        const float dd = Sub(pd, df), hd = Sub(ph, hf), wd = Sub(pw, wf);
        const float wd0 = Sub(1.0f, wd), hd0 = Sub(1.0f, hd), dd0 = Sub(1.0f, dd);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool east = (k & 1) != 0, south = (k & 2) != 0, back = (k & 4) != 0;
            const float wt = Mul(Mul(east ? wd : wd0, south ? hd : hd0), back ? dd : dd0);
            const float d = back ? Add(df, 1.0f) : df, h = south ? Add(hf, 1.0f) : hf, w = east ? Add(wf, 1.0f) : wf;
            if (Inside3(d, h, w, g)) {
                LoadPack<T, V>(xb + ((static_cast<int64_t>(d) * g.hi + static_cast<int64_t>(h)) * g.wi + static_cast<int64_t>(w)) * g.c, tv);
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    tv[v] = 0.0f;
                }
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                acc[v] = k == 0 ? Mul(tv[v], wt) : Add(acc[v], Mul(tv[v], wt));
            }
        }
        StorePack<T, V>(yp, acc);
    }
}

__device__ __forceinline__ void AtomicAddPack(float* p, const float (&v)[1]) { atomicAdd(p, v[0]); }
__device__ __forceinline__ void AtomicAddPack(float* p, const float (&v)[2])
{
    atomicAdd(reinterpret_cast<float2*>(p), make_float2(v[0], v[1])); // one 8-byte reduction (sm_90 and later)
}
__device__ __forceinline__ void AtomicAddPack(float* p, const float (&v)[4])
{
    atomicAdd(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3])); // one 16-byte reduction
}

template <typename T, bool CL, int V>
__global__ void __launch_bounds__(kThreads)
    GridSampler3dBwdKernel(const T* __restrict__ go, const T* __restrict__ x, const T* __restrict__ grid,
                           float* __restrict__ acc, T* __restrict__ ggrid, Grid3dShape g, int32_t wantInput,
                           int32_t wantGrid)
{
    const int64_t outVol = static_cast<int64_t>(g.dout) * g.ho * g.wo, inVol = static_cast<int64_t>(g.di) * g.hi * g.wi;
    const int64_t total = g.n * outVol;
    const int64_t cs = CL ? 1 : inVol, vs = CL ? g.c : 1;
    const int64_t ocs = CL ? 1 : outVol, ovs = CL ? g.c : 1;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int64_t n = idx / outVol, p = idx - n * outVol;
        const T* gp = grid + idx * 3;
        float mx = 0.0f, my = 0.0f, mz = 0.0f;
        const float ix = gs::SourceIndexSetGrad(DType<T>::Load(gp), g.wi, g.pad, g.align, &mx);
        const float iy = gs::SourceIndexSetGrad(DType<T>::Load(gp + 1), g.hi, g.pad, g.align, &my);
        const float iz = gs::SourceIndexSetGrad(DType<T>::Load(gp + 2), g.di, g.pad, g.align, &mz);
        const T* gob = go + n * g.c * outVol + p * ovs;
        const T* xb = x + n * g.c * inVol;
        float* ab = acc + n * g.c * inVol;
        auto inside = [&](int32_t d, int32_t h, int32_t w) {
            return d >= 0 && h >= 0 && w >= 0 && d < g.di && h < g.hi && w < g.wi;
        };
        if (g.interp == 1) {
            const int32_t xn = static_cast<int32_t>(rintf(ix)), yn = static_cast<int32_t>(rintf(iy)),
                          zn = static_cast<int32_t>(rintf(iz));
            if (wantInput && inside(zn, yn, xn)) {
                const int64_t off = ((static_cast<int64_t>(zn) * g.hi + yn) * g.wi + xn) * vs;
                for (int64_t c = 0; c < g.c; c += V) {
                    float gv[V];
                    LoadPack<T, V>(gob + c * ocs, gv);
                    AtomicAddPack(ab + c * cs + off, gv);
                }
            }
            if (wantGrid) {
                ggrid[idx * 3] = ggrid[idx * 3 + 1] = ggrid[idx * 3 + 2] = DType<T>::FromF(0.0f);
            }
            continue;
        }
        const int32_t x0 = static_cast<int32_t>(floorf(ix)), y0 = static_cast<int32_t>(floorf(iy)),
                      z0 = static_cast<int32_t>(floorf(iz));
        const float xe = Sub(static_cast<float>(x0 + 1), ix), xw = Sub(ix, static_cast<float>(x0));
        const float ye = Sub(static_cast<float>(y0 + 1), iy), yw = Sub(iy, static_cast<float>(y0));
        const float ze = Sub(static_cast<float>(z0 + 1), iz), zw = Sub(iz, static_cast<float>(z0));
        float wt[8];
        int64_t off[8];
        bool in[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool east = (k & 1) != 0, south = (k & 2) != 0, bottom = (k & 4) != 0;
            wt[k] = Mul(Mul(east ? xw : xe, south ? yw : ye), bottom ? zw : ze);
            const int32_t d = bottom ? z0 + 1 : z0, h = south ? y0 + 1 : y0, w = east ? x0 + 1 : x0;
            in[k] = inside(d, h, w);
            off[k] = in[k] ? ((static_cast<int64_t>(d) * g.hi + h) * g.wi + w) * vs : 0;
        }
        float gix = 0.0f, giy = 0.0f, giz = 0.0f;
        for (int64_t c = 0; c < g.c; c += V) {
            float gv[V];
            LoadPack<T, V>(gob + c * ocs, gv);
            float xv[8][V];
            if (wantGrid) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (in[k]) {
                        LoadPack<T, V>(xb + c * cs + off[k], xv[k]);
                    }
                }
            }
            if (wantInput) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (in[k]) {
                        float t[V];
#pragma unroll
                        for (int v = 0; v < V; ++v) {
                            t[v] = Mul(wt[k], gv[v]);
                        }
                        AtomicAddPack(ab + c * cs + off[k], t);
                    }
                }
            }
            if (wantGrid) { // channel by channel, corner by corner: the reference's order
#pragma unroll
                for (int v = 0; v < V; ++v) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        if (!in[k]) {
                            continue;
                        }
                        const bool east = (k & 1) != 0, south = (k & 2) != 0, bottom = (k & 4) != 0;
                        const float val = xv[k][v];
                        const float fx = east ? xw : xe, fy = south ? yw : ye, fz = bottom ? zw : ze;
                        const float tx = Mul(Mul(Mul(val, fy), fz), gv[v]), ty = Mul(Mul(Mul(val, fx), fz), gv[v]),
                                    tz = Mul(Mul(Mul(val, fx), fy), gv[v]);
                        gix = east ? Add(gix, tx) : Sub(gix, tx);
                        giy = south ? Add(giy, ty) : Sub(giy, ty);
                        giz = bottom ? Add(giz, tz) : Sub(giz, tz);
                    }
                }
            }
        }
        if (wantGrid) {
            ggrid[idx * 3] = DType<T>::FromF(Mul(mx, gix));
            ggrid[idx * 3 + 1] = DType<T>::FromF(Mul(my, giy));
            ggrid[idx * 3 + 2] = DType<T>::FromF(Mul(mz, giz));
        }
    }
}

// Channel vector of the channels-last kernels: 16 bytes of fp32 accumulator at most, C a multiple of it, pointers aligned.
int ChannelVec(const Grid3dShape& g, int es, std::initializer_list<const void*> ptrs, const float* acc)
{
    if (!g.cl) {
        return 1;
    }
    int v = 4;
    while (v > 1) {
        bool ok = g.c % v == 0 && (acc == nullptr || Aligned(acc, static_cast<size_t>(v) * sizeof(float)));
        for (const void* p : ptrs) {
            ok = ok && Aligned(p, static_cast<size_t>(v) * es);
        }
        if (ok) {
            break;
        }
        v >>= 1;
    }
    return v;
}

} // namespace

cudaError_t GridSampler3dFwd(Dt dt, const void* x, const void* grid, void* y, Grid3dShape g, cudaStream_t s)
{
    const int64_t total = g.n * g.dout * g.ho * g.wo;
    const int v = ChannelVec(g, DtSize(dt), {x, y}, nullptr);
    OPSCV_DISPATCH_DT(dt, T, {
        const T* px = static_cast<const T*>(x);
        const T* pg = static_cast<const T*>(grid);
        T* py = static_cast<T*>(y);
        const unsigned grid1 = GridFor(total, kThreads);
        if (!g.cl) {
            GridSampler3dFwdKernel<T, false, 1><<<grid1, kThreads, 0, s>>>(px, pg, py, g);
        } else if (v == 4) {
            const int32_t groups = static_cast<int32_t>(g.c / 4);
            GridSampler3dFwdLanesKernel<T, 4><<<GridFor(total * groups, kThreads), kThreads, 0, s>>>(px, pg, py, g, groups);
        } else if (v == 2) {
            const int32_t groups = static_cast<int32_t>(g.c / 2);
            GridSampler3dFwdLanesKernel<T, 2><<<GridFor(total * groups, kThreads), kThreads, 0, s>>>(px, pg, py, g, groups);
        } else {
            GridSampler3dFwdKernel<T, true, 1><<<grid1, kThreads, 0, s>>>(px, pg, py, g);
        }
    });
    CountLaunch();
    return cudaGetLastError();
}

// acc: fp32 grad_input accumulator of N * C * Di * Hi * Wi floats (the grad_input tensor itself for fp32), zeroed here.
cudaError_t GridSampler3dBwd(Dt dt, const void* go, const void* x, const void* grid, void* gi, void* ggrid, float* acc,
                             Grid3dShape g, bool wantInput, bool wantGrid, cudaStream_t s)
{
    const int64_t total = g.n * g.dout * g.ho * g.wo;
    const int64_t giElems = g.n * g.c * g.di * g.hi * g.wi;
    cudaError_t e = cudaSuccess;
    if (wantInput) {
        e = cudaMemsetAsync(acc, 0, static_cast<size_t>(giElems) * sizeof(float), s);
        CountLaunch();
        if (e != cudaSuccess) {
            return e;
        }
    }
    const int v = ChannelVec(g, DtSize(dt), {go, x}, acc);
    OPSCV_DISPATCH_DT(dt, T, {
        const T* pgo = static_cast<const T*>(go);
        const T* px = static_cast<const T*>(x);
        const T* pg = static_cast<const T*>(grid);
        T* pgg = static_cast<T*>(ggrid);
        const unsigned grid1 = GridFor(total, kThreads);
        const int32_t wi = wantInput ? 1 : 0, wg = wantGrid ? 1 : 0;
        if (!g.cl) {
            GridSampler3dBwdKernel<T, false, 1><<<grid1, kThreads, 0, s>>>(pgo, px, pg, acc, pgg, g, wi, wg);
        } else if (v == 4) {
            GridSampler3dBwdKernel<T, true, 4><<<grid1, kThreads, 0, s>>>(pgo, px, pg, acc, pgg, g, wi, wg);
        } else if (v == 2) {
            GridSampler3dBwdKernel<T, true, 2><<<grid1, kThreads, 0, s>>>(pgo, px, pg, acc, pgg, g, wi, wg);
        } else {
            GridSampler3dBwdKernel<T, true, 1><<<grid1, kThreads, 0, s>>>(pgo, px, pg, acc, pgg, g, wi, wg);
        }
    });
    CountLaunch();
    e = cudaGetLastError();
    if (e == cudaSuccess && wantInput && dt != Dt::F32) {
        e = CastFromF32(dt, gi, acc, giElems, s);
    }
    return e;
}

} // namespace opscv
