// Coordinate arithmetic of the 2-D grid sampler, forward and backward flavours, with the reference's operation
// order and explicit (non-fused) roundings.
#pragma once

#include "common.cuh"

namespace opscv {
namespace gs {

// ---- forward: image/grid_sampler2_d/op_kernel/arch35/grid_sampler2_d_simt.h:106-215 ----------------------------
__device__ __forceinline__ float UnnormalizeNoClip(float coord, int32_t size, int32_t align)
{
    if (align != 0) {
        return Mul(Div(Add(coord, 1.0f), 2.0f), static_cast<float>(size - 1));
    }
    const float scalingFactor = Div(static_cast<float>(size), 2.0f);
    return __fmaf_rn(scalingFactor, Add(coord, 1.0f), -0.5f); // the reference writes fmaf explicitly (:131)
}

__device__ __forceinline__ float ClipCoordinates(float coord, int32_t size)
{
    const float maxVal = static_cast<float>(size - 1);
    if (isnan(coord)) {
        return 0.0f;
    }
    return fminf(fmaxf(coord, 0.0f), maxVal);
}

__device__ __forceinline__ float ReflectCoordinates(float coord, float low, float twiceSpan)
{
    if (twiceSpan == 0.0f) {
        return 0.0f;
    }
    const float absIn = fabsf(Sub(coord, low));
    const float doubleFlips = truncf(Div(absIn, twiceSpan));
    const float product = Mul(doubleFlips, twiceSpan);
    const float extra = Sub(absIn, product);
    const float complement = Sub(twiceSpan, extra);
    return Add(fminf(extra, complement), low);
}

__device__ __forceinline__ float ComputeCoordinates(float coord, int32_t size, int32_t pad, int32_t align)
{
    if (pad == 1) {
        coord = ClipCoordinates(coord, size);
    } else if (pad == 2) {
        if (align != 0) {
            coord = ReflectCoordinates(coord, 0.0f, Mul(2.0f, static_cast<float>(size - 1)));
        } else {
            coord = ReflectCoordinates(coord, -0.5f, Mul(2.0f, static_cast<float>(size)));
        }
        coord = ClipCoordinates(coord, size);
    }
    return coord;
}

__device__ __forceinline__ float ComputeSourceIndex(float coord, int32_t size, int32_t pad, int32_t align)
{
    return ComputeCoordinates(UnnormalizeNoClip(coord, size, align), size, pad, align);
}

__device__ __forceinline__ float SafeDowngradeToIntRange(float x)
{
    if (x > 2147483646.0f || x < -2147483648.0f || isnan(x) || isinf(x)) {
        return -100.0f;
    }
    return x;
}

__device__ __forceinline__ bool IsNanOrInf(float x) { return isnan(x) || isinf(x); }

__device__ __forceinline__ int32_t BankerRoundToInt(float x)
{
    const float floorVal = floorf(x);
    const float frac = Sub(x, floorVal);
    if (frac < 0.5f) {
        return static_cast<int32_t>(floorVal);
    }
    if (frac > 0.5f) {
        return static_cast<int32_t>(floorVal) + 1;
    }
    const int32_t floorInt = static_cast<int32_t>(floorVal);
    return ((floorInt & 1) == 0) ? floorInt : floorInt + 1;
}

__device__ __forceinline__ bool Within(int32_t h, int32_t w, int32_t H, int32_t W)
{
    return h >= 0 && h < H && w >= 0 && w < W;
}

// Bicubic convolution coefficients, A = -0.75 (grid_sampler2_d_simt.h:272-291), separate roundings.
__device__ __forceinline__ float Cubic1(float x)
{
    const float t0 = Mul(1.25f, x);  // (A + 2) * x
    const float t1 = Sub(t0, 2.25f); // - (A + 3)
    const float t2 = Mul(t1, x);
    const float t3 = Mul(t2, x);
    return Add(t3, 1.0f);
}
__device__ __forceinline__ float Cubic2(float x)
{
    const float t0 = Mul(-0.75f, x);  // A * x
    const float t1 = Sub(t0, -3.75f); // - 5A
    const float t2 = Mul(t1, x);
    const float t3 = Add(t2, -6.0f); // + 8A
    const float t4 = Mul(t3, x);
    return Sub(t4, -3.0f); // - 4A
}
__device__ __forceinline__ int32_t SafeFloatToInt32(float f)
{
    if (f >= 0.0f && f < 2147483648.0f) {
        return static_cast<int32_t>(f);
    }
    return -1;
}
__device__ __forceinline__ float WeightedSum(float c0, float c1, float c2, float c3, float v0, float v1, float v2,
                                             float v3)
{
    float r = Mul(c0, v0);
    r = __fmaf_rn(c1, v1, r);
    r = __fmaf_rn(c2, v2, r);
    r = __fmaf_rn(c3, v3, r);
    return r;
}

// ---- backward: image/grid_sampler3_d_grad/op_kernel/arch35/grid_sampler3_d_grad_simt_base.h:51-184 --------------
__device__ __forceinline__ float UnnormalizeSetGrad(float coord, int32_t size, int32_t align, float* mult)
{
    if (align == 1) {
        coord = Mul(Div(Add(coord, 1.0f), 2.0f), static_cast<float>(size - 1));
        *mult = Div(static_cast<float>(size - 1), 2.0f);
    } else {
        coord = Div(Sub(Mul(Add(coord, 1.0f), static_cast<float>(size)), 1.0f), 2.0f);
        *mult = Div(static_cast<float>(size), 2.0f);
    }
    return coord;
}

__device__ __forceinline__ float ClipSetGrad(float coord, int32_t limit, float* g)
{
    if (coord <= 0.0f) {
        *g = 0.0f;
        return 0.0f;
    }
    const float mx = static_cast<float>(limit - 1);
    if (coord >= mx) {
        *g = 0.0f;
        return mx;
    }
    *g = 1.0f;
    return coord;
}

__device__ __forceinline__ float ReflectSetGrad(float coord, int32_t twiceLow, int32_t twiceHigh, float* g)
{
    if (twiceLow == twiceHigh) {
        *g = 0.0f;
        return 0.0f;
    }
    float mult;
    const float mn = Div(static_cast<float>(twiceLow), 2.0f);
    const float span = Div(static_cast<float>(twiceHigh - twiceLow), 2.0f);
    coord = Sub(coord, mn);
    if (coord < 0.0f) {
        mult = -1.0f;
        coord = -coord;
    } else {
        mult = 1.0f;
    }
    const float extra = fmodf(coord, span);
    const int32_t flips = static_cast<int32_t>(floorf(Div(coord, span)));
    if (flips % 2 == 0) {
        *g = mult;
        return Add(extra, mn);
    }
    *g = -mult;
    return Add(Sub(span, extra), mn);
}

__device__ __forceinline__ float SourceIndexSetGrad(float coord, int32_t size, int32_t pad, int32_t align, float* mult)
{
    float gc = 0.0f, gr = 0.0f;
    coord = UnnormalizeSetGrad(coord, size, align, mult);
    if (pad == 1) {
        coord = ClipSetGrad(coord, size, &gc);
        *mult = Mul(*mult, gc);
    } else if (pad == 2) {
        if (align) {
            coord = ReflectSetGrad(coord, 0, 2 * (size - 1), &gr);
        } else {
            coord = ReflectSetGrad(coord, -1, 2 * size - 1, &gr);
        }
        coord = ClipSetGrad(coord, size, &gc);
        *mult = Mul(Mul(*mult, gr), gc);
    }
    if (!isfinite(coord)) {
        coord = -100.0f;
    }
    return coord;
}

// ---- bicubic backward: image/grid_sampler3_d_grad/op_kernel/arch35/grid_sampler3_d_grad_simt_base.h:186-311 -------
// Derivatives of the four cubic coefficients with respect to t (A = -0.75), separate roundings.
__device__ __forceinline__ float Cubic2Slope(float x) // (3A x - 10A) x + 8A
{
    return Add(Mul(Sub(Mul(-2.25f, x), -7.5f), x), -6.0f);
}
__device__ __forceinline__ float Cubic1Slope(float x) // (3(A+2) x - 2(A+3)) x
{
    return Mul(Sub(Mul(3.75f, x), 4.5f), x);
}
__device__ __forceinline__ void CubicCoefficients(float (&c)[4], float t)
{
    c[0] = Cubic2(Add(t, 1.0f));
    c[1] = Cubic1(t);
    c[2] = Cubic1(Sub(1.0f, t));
    c[3] = Cubic2(Sub(2.0f, t));
}
__device__ __forceinline__ void CubicCoefficientsGrad(float (&c)[4], float t)
{
    c[0] = Cubic2Slope(Add(t, 1.0f));
    c[1] = Cubic1Slope(t);
    c[2] = -Cubic1Slope(Sub(1.0f, t));
    c[3] = -Cubic2Slope(Sub(2.0f, t));
}
// Pixel index that a neighbour coordinate maps to under the padding mode, or -1 (GetValueBounded / AddValueBounded:
// zeros tests the float coordinate, border clamps it, reflection reflects and clips; a coordinate that is not finite
// ends as -100 and is out of range).
__device__ __forceinline__ int32_t BoundedIndex(float x, float y, int32_t w, int32_t h, int32_t pad, int32_t align)
{
    if (pad == 0) {
        if (x < 0.0f || x >= static_cast<float>(w) || y < 0.0f || y >= static_cast<float>(h)) {
            return -1;
        }
    } else if (pad == 1) {
        x = x < 0.0f ? 0.0f : (x >= static_cast<float>(w) ? static_cast<float>(w) - 1.0f : x);
        y = y < 0.0f ? 0.0f : (y >= static_cast<float>(h) ? static_cast<float>(h) - 1.0f : y);
    } else {
        float gr, gc;
        if (align != 0) {
            x = ReflectSetGrad(x, 0, 2 * (w - 1), &gr);
            y = ReflectSetGrad(y, 0, 2 * (h - 1), &gr);
        } else {
            x = ReflectSetGrad(x, -1, 2 * w - 1, &gr);
            y = ReflectSetGrad(y, -1, 2 * h - 1, &gr);
        }
        x = ClipSetGrad(x, w, &gc);
        y = ClipSetGrad(y, h, &gc);
    }
    const int32_t ix = static_cast<int32_t>(isfinite(x) ? x : -100.0f);
    const int32_t iy = static_cast<int32_t>(isfinite(y) ? y : -100.0f);
    return (ix >= 0 && ix < w && iy >= 0 && iy < h) ? iy * w + ix : -1;
}

} // namespace gs

// ---- staging of channel-interleaved pixel records ------------------------------------------------------------------
// The plane-major grid-sampler kernels keep, per pixel, one 16-byte record holding LV = 16 / sizeof(T) channels.
// This copies LV planes of `rows` x `cols` elements (plane k at src + k * planeStride, rows `rowStride` elements
// apart) into records dst[(r * dstPitch + c)] (r, c relative to the caller's origin), channels past nch zero.
// Fast path (cols a multiple of LV, 16-byte aligned rows): a work item is LV consecutive pixels of one row; the
// thread reads them with one 16-byte load per channel, transposes the LV x LV block in registers and writes LV
// 16-byte records, instead of one scalar load per pixel and channel (for 16-bit types that was eight 2-byte loads
// per record and more instructions than the sampling itself when a plane is staged by several blocks).
template <typename T>
__device__ __forceinline__ void StageRecords(Pack<T, 16 / sizeof(T)>* dst, int32_t dstPitch, const T* __restrict__ src,
                                             int64_t planeStride, int32_t rowStride, int32_t nch, int32_t rows,
                                             int32_t cols, int32_t tid, int32_t nthreads)
{
    constexpr int LV = 16 / sizeof(T);
    using Vec = Pack<T, LV>;
    const bool fast = cols % LV == 0 && rowStride % LV == 0 && planeStride % LV == 0 &&
                      (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    if (fast) {
        const int32_t perRow = cols / LV;
        for (int32_t i = tid; i < rows * perRow; i += nthreads) {
            const int32_t r = i / perRow, q = i - r * perRow;
            const T* p = src + static_cast<int64_t>(r) * rowStride + q * LV;
            uint4* out = reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * dstPitch + q * LV);
            if constexpr (LV == 4) { // 4 x 4 words: pixel j takes word j of every channel
                uint4 in[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    in[k] = k < nch ? __ldg(reinterpret_cast<const uint4*>(p + k * planeStride)) : make_uint4(0, 0, 0, 0);
                }
                const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&in[0]);
                const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&in[1]);
                const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&in[2]);
                const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&in[3]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    out[j] = make_uint4(w0[j], w1[j], w2[j], w3[j]);
                }
            } else {
                // 8 x 8 halves in two passes of four channels (sixteen registers of input at a time): pixel j takes
                // half j of every channel, two channels per output word, so a pass writes half a record per pixel
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint4 in[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        in[k] = 4 * h + k < nch ? __ldg(reinterpret_cast<const uint4*>(p + (4 * h + k) * planeStride))
                                                : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint32_t o[2];
#pragma unroll
                        for (int c2 = 0; c2 < 2; ++c2) {
                            const uint32_t a = reinterpret_cast<const uint32_t*>(&in[2 * c2])[j >> 1];
                            const uint32_t b = reinterpret_cast<const uint32_t*>(&in[2 * c2 + 1])[j >> 1];
                            // low half of the word from channel 2*c2, high half from channel 2*c2 + 1 (of this pass)
                            o[c2] = (j & 1) ? __byte_perm(a, b, 0x7632) : __byte_perm(a, b, 0x5410);
                        }
                        reinterpret_cast<uint2*>(out + j)[h] = make_uint2(o[0], o[1]);
                    }
                }
            }
        }
        return;
    }
    for (int32_t i = tid; i < rows * cols; i += nthreads) {
        const int32_t r = i / cols, c = i - r * cols;
        const T* p = src + static_cast<int64_t>(r) * rowStride + c;
        Vec v;
#pragma unroll
        for (int k = 0; k < LV; ++k) {
            v.v[k] = k < nch ? __ldg(p + k * planeStride) : DType<T>::FromF(0.0f);
        }
        dst[static_cast<int64_t>(r) * dstPitch + c] = v;
    }
}

} // namespace opscv
