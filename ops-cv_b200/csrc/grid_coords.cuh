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

} // namespace gs
} // namespace opscv
