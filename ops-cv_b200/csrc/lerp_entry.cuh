// One entry of a bilinear index / weight table, shared by the table kernels and by the kernels that evaluate the
// few entries they need themselves instead of reading a table.
// variant 0: image/resize_bilinear_v2/op_kernel/arch35/resize_bilinear_v2_simt_nchw.h:110-133
// variant 1: image/resize_bilinear_v2_grad/op_kernel/arch35/resize_bilinear_v2_grad_simt.h:121-135
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace opscv {

// One table entry: source index pair and weight of destination index d.
__device__ __forceinline__ void LerpEntry(const AxisGeom& g, int halfPixel, int variant, int32_t d, int32_t& loOut,
                                          int32_t& hiOut, float& deltaOut)
{
    const long long last = g.in - 1;
    if (variant == 0) {
        float src;
        if (halfPixel) {
            src = Sub(Mul(Add(static_cast<float>(d), 0.5f), g.scale), 0.5f);
        } else {
            src = Mul(static_cast<float>(d), g.scale);
        }
        if (src < 0.0f) {
            src = 0.0f;
        }
        long long lo = (src > 0.0f) ? static_cast<long long>(floorf(src)) : 0;
        lo = lo < last ? lo : last;
        long long hi = (src > 0.0f) ? static_cast<long long>(ceilf(src)) : 0;
        hi = hi < last ? hi : last;
        loOut = static_cast<int32_t>(lo);
        hiOut = static_cast<int32_t>(hi);
        deltaOut = Sub(src, floorf(src));
    } else {
        const float offset = halfPixel ? 0.5f : 0.0f;
        float src = Sub(Mul(Add(static_cast<float>(d), offset), g.scale), offset);
        src = (src < 0.0f) ? 0.0f : src;
        long long lo = static_cast<long long>(floorf(src));
        lo = lo < last ? lo : last;
        const float delta = fminf(fmaxf(Sub(src, static_cast<float>(lo)), 0.0f), 1.0f);
        const long long hi = (lo < last) ? lo + 1 : lo;
        loOut = static_cast<int32_t>(lo);
        hiOut = static_cast<int32_t>(hi);
        deltaOut = delta;
    }
}

} // namespace opscv
