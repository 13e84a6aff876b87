// First- and second-phase entry points of the Upsample{Nearest,Bilinear,Bicubic2dAA} family. The first phase
// mirrors the reference's CheckParams functions (same checks, same order, same status codes; file:line cited at
// each function) and then freezes a launch plan into the executor: table builders, the resampling kernel, and
// the staging copies for strided views. Scales are computed here, on the host, with the expressions of the
// reference's arch35 tiling code.
#include <cfloat>
#include <cmath>
#include <cstring>

#include "host_common.h"
#include "host_tables.h"

using namespace opscv;

namespace {

struct Geom {
    int64_t n = 0, c = 0, h = 0, w = 0;
};

// View dims are [N,C,H,W] for NCHW / ND and [N,H,W,C] for NHWC.
Geom GeomOf(const aclTensor* t)
{
    Geom g;
    if (t->format == ACL_FORMAT_NHWC) {
        g.n = t->dims[0];
        g.h = t->dims[1];
        g.w = t->dims[2];
        g.c = t->dims[3];
    } else {
        g.n = t->dims[0];
        g.c = t->dims[1];
        g.h = t->dims[2];
        g.w = t->dims[3];
    }
    return g;
}

// common/stub/op_api/aclnn_kernels/common/op_error_check.h:112-141 (CheckNCDimValid)
bool CheckNCDimValid(const aclTensor* self, const aclTensor* out, const char* api)
{
    if (self->format != ACL_FORMAT_NCHW && self->format != ACL_FORMAT_NHWC) {
        Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output format only support [NCHW, NHWC]", api);
        return false;
    }
    const int cDim = self->format == ACL_FORMAT_NCHW ? 1 : 3;
    if (self->dims[0] != out->dims[0] || self->dims[cDim] != out->dims[cDim]) {
        Fail(ACLNN_ERR_PARAM_INVALID, "%s: N %ld/%ld or C %ld/%ld of input and output differ", api,
             (long)self->dims[0], (long)out->dims[0], (long)self->dims[cDim], (long)out->dims[cDim]);
        return false;
    }
    return true;
}

bool FitsInt32(const Geom& g) { return g.h <= INT32_MAX && g.w <= INT32_MAX && g.n >= 0 && g.c >= 0; }

aclnnStatus EmptySuccess(const char* api, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    *workspaceSize = 0;
    *executor = ex;
    return ACLNN_SUCCESS;
}

Shape4 MakeShape(const Geom& in, const Geom& out)
{
    Shape4 s;
    s.n = in.n;
    s.c = in.c;
    s.hin = static_cast<int32_t>(in.h);
    s.win = static_cast<int32_t>(in.w);
    s.hout = static_cast<int32_t>(out.h);
    s.wout = static_cast<int32_t>(out.w);
    return s;
}

struct TableAlloc {
    uint64_t off[4]; // workspace offsets, meaning depends on the table type
};

// A 4-D view that is not contiguous in its own format but is a dense tensor in the OTHER layout's memory order: an
// NCHW-format view [N, C, H, W] with the strides of an NHWC-contiguous tensor (what a channels-last framework tensor
// looks like through an NCHW handle), or an NHWC-format view [N, H, W, C] with NCHW-contiguous strides. `alt`
// receives the same memory described in that other format, contiguous.
bool PermutedDense(const aclTensor* t, aclTensor& alt)
{
    if (t->dims.size() != 4 || (t->format != ACL_FORMAT_NCHW && t->format != ACL_FORMAT_NHWC) || IsContiguous(t)) {
        return false;
    }
    const bool nchw = t->format == ACL_FORMAT_NCHW;
    const int64_t n = t->dims[0], c = t->dims[nchw ? 1 : 3], h = t->dims[nchw ? 2 : 1], w = t->dims[nchw ? 3 : 2];
    const int64_t sn = t->strides[0], sc = t->strides[nchw ? 1 : 3], sh = t->strides[nchw ? 2 : 1],
                  sw = t->strides[nchw ? 3 : 2];
    auto is = [](int64_t dim, int64_t stride, int64_t want) { return dim == 1 || stride == want; };
    alt = *t;
    if (nchw) { // memory order N, H, W, C
        if (!(is(c, sc, 1) && is(w, sw, c) && is(h, sh, w * c) && is(n, sn, h * w * c))) {
            return false;
        }
        alt.dims = {n, h, w, c};
        alt.strides = {h * w * c, w * c, c, 1};
        alt.format = ACL_FORMAT_NHWC;
    } else { // memory order N, C, H, W
        if (!(is(w, sw, 1) && is(h, sh, w) && is(c, sc, h * w) && is(n, sn, c * h * w))) {
            return false;
        }
        alt.dims = {n, c, h, w};
        alt.strides = {c * h * w, h * w, w, 1};
        alt.format = ACL_FORMAT_NCHW;
    }
    alt.storageDims = alt.dims;
    return true;
}

// Both tensors of a call are dense in the other layout: run that layout's kernels on the memory as it is instead
// of gathering the input into the workspace and scattering the output back (the reference's Contiguous / ViewCopy).
// Operators whose kernels exist for both layouts call this after their checks.
bool UseOtherLayout(const aclTensor*& a, const aclTensor*& b, aclTensor& altA, aclTensor& altB)
{
    if (a->format != b->format || !PermutedDense(a, altA) || !PermutedDense(b, altB)) {
        return false;
    }
    a = &altA;
    b = &altB;
    return true;
}

// ---- UpsampleNearest2d ----------------------------------------------------------------------------------------
// image/resize_nearest_neighbor_v2/op_host/arch35/resize_nearest_neighbor_v2_tiling_base.cpp:251-262
float NearestScale(int64_t in, int64_t out, float userScale)
{
    return userScale > 0.0f ? 1.0f / userScale : static_cast<float>(in) / static_cast<float>(out);
}

// image/resize_nearest_neighbor_v2/op_api/aclnn_upsample_nearest_2d.cpp:187-216 (CheckParams), :74-213 helpers
aclnnStatus CheckNearestFwd(const char* api, const aclTensor* self, const aclIntArray* outputSize,
                            const aclTensor* out)
{
    if (!DtypeSupported(self->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(self->dtype));
    }
    if (self->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from self dtype %s", api, DtypeName(out->dtype),
                    DtypeName(self->dtype));
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: outputSize must have 2 values, got %zu", api, outputSize->v.size());
    }
    if (self->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self must be 4-D, got %zu-D", api, self->dims.size());
    }
    if (self->dims[2] == 0 || self->dims[3] == 0 || outputSize->v[0] == 0 || outputSize->v[1] == 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes must be greater than 0", api);
    }
    if (self->dims[1] == 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: non-empty 4-D data tensor expected", api);
    }
    if (self->format != ACL_FORMAT_NCHW && self->format != ACL_FORMAT_NHWC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format %s of input not supported", api, FormatName(self->format));
    }
    if (self->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format of input (%s) and output (%s) must be equal", api,
                    FormatName(self->format), FormatName(out->format));
    }
    if (out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out must be 4-D, got %zu-D", api, out->dims.size());
    }
    if (!CheckNCDimValid(self, out, api)) {
        return ACLNN_ERR_PARAM_INVALID;
    }
    const Geom go = GeomOf(out);
    if (outputSize->v[0] != go.h || outputSize->v[1] != go.w) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: expected output size (H: %ld, W: %ld) but out tensor has (H: %ld, W: %ld)",
                    api, (long)outputSize->v[0], (long)outputSize->v[1], (long)go.h, (long)go.w);
    }
    if (!FitsInt32(GeomOf(self)) || !FitsInt32(go)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H and W must not exceed INT32_MAX", api);
    }
    return ACLNN_SUCCESS;
}

// Element strides of a four-dimensional NCHW view with no negative stride (an output view must also not overlap
// itself: no zero stride on a dimension longer than 1).
bool StridesOf(const aclTensor* t, bool output, ViewStrides* st)
{
    if (t->format == ACL_FORMAT_NHWC || t->dims.size() != 4 || t->strides.size() != 4) {
        return false;
    }
    for (size_t i = 0; i < 4; ++i) {
        if (t->strides[i] < 0 || (output && t->strides[i] == 0 && t->dims[i] > 1)) {
            return false;
        }
    }
    st->n = t->strides[0];
    st->c = t->strides[1];
    st->h = t->strides[2];
    st->w = t->strides[3];
    st->chan = static_cast<int32_t>(t->dims[1]);
    return true;
}

aclnnStatus PlanNearestFwd(const char* api, const aclTensor* self, const aclTensor* out, float userScaleH,
                           float userScaleW, uint64_t* workspaceSize, aclOpExecutor** executor, bool exact = false)
{
    aclTensor altSelf, altOut;
    UseOtherLayout(self, out, altSelf, altOut);
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const Geom gi = GeomOf(self), go = GeomOf(out);
    const Shape4 sh = MakeShape(gi, go);
    const Dt dt = ToDt(self->dtype);
    const Layout lay = self->format == ACL_FORMAT_NHWC ? kNHWC : kNCHW;
    const AxisGeom ah{sh.hin, sh.hout, NearestScale(gi.h, go.h, userScaleH), exact ? 1 : 0};
    const AxisGeom aw{sh.win, sh.wout, NearestScale(gi.w, go.w, userScaleW), exact ? 1 : 0};
    // A whole-number up-scale with a W factor of 2 between strided NCHW views (a crop or a channel slice on either
    // side) runs on the replicate kernel with pitches: no gather copy, no scatter copy.
    ViewStrides si{}, so{};
    if ((!IsContiguous(self) || !IsContiguous(out)) && StridesOf(self, false, &si) && StridesOf(out, true, &so) &&
        sh.wout == 2 * sh.win && sh.hout % sh.hin == 0) {
        const int32_t rh = sh.hout / sh.hin;
        const std::vector<int32_t> srcH = host::NearestSrc(sh.hin, sh.hout, ah.scale, exact);
        const std::vector<int32_t> srcW = host::NearestSrc(sh.win, sh.wout, aw.scale, exact);
        bool whole = true;
        for (int32_t d = 0; d < sh.hout && whole; ++d) {
            whole = srcH[d] == d / rh;
        }
        for (int32_t d = 0; d < sh.wout && whole; ++d) {
            whole = srcW[d] == d / 2;
        }
        char* px = static_cast<char*>(self->data) + self->offset * ElemSize(self->dtype);
        char* py = static_cast<char*>(out->data) + out->offset * ElemSize(out->dtype);
        if (whole && NearestFwdX2PitchUsable(dt, px, si, py, so, sh)) {
            ex->steps.push_back([=](char*, cudaStream_t s) { return NearestFwdX2Pitch(dt, px, si, py, so, sh, rh, s); });
            ex->workspaceSize = 0;
            *workspaceSize = 0;
            *executor = ex;
            return ACLNN_SUCCESS;
        }
    }
    const BufRef x = StageInput(self, ws, ex);
    const BufRef y = StageOutput(out, ws);
    const uint64_t offH = ws.Alloc(sizeof(int32_t) * static_cast<uint64_t>(sh.hout));
    const uint64_t offW = ws.Alloc(sizeof(int32_t) * static_cast<uint64_t>(sh.wout));
    const NearestPlan plan = MakeNearestFwdPlan(dt, lay, sh, ah, aw);
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        const NearestAxis th{reinterpret_cast<int32_t*>(w + offH)}, tw{reinterpret_cast<int32_t*>(w + offW)};
        if (!NearestFwdUsesInteger(dt, lay, x.At(w), y.At(w), sh, plan)) {
            const cudaError_t e = BuildNearestFwdTables(ah, aw, th, tw, s);
            if (e != cudaSuccess) {
                return e;
            }
        }
        return NearestFwd(dt, lay, x.At(w), y.At(w), sh, th, tw, plan, s);
    });
    FinishOutput(out, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

// ---- UpsampleNearest2dBackward --------------------------------------------------------------------------------
// image/upsample_nearest2d_grad/op_host/op_api/aclnn_upsample_nearest_2d_backward.cpp:147-166 (CheckParams)
aclnnStatus CheckBackwardCommon(const char* api, const aclTensor* gradOut, const aclIntArray* outputSize,
                                const aclIntArray* inputSize, const aclTensor* gradInput, bool allowF32ToAny)
{
    if (!DtypeSupported(gradOut->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(gradOut->dtype));
    }
    if (allowF32ToAny && gradOut->dtype == ACL_FLOAT) {
        if (!DtypeSupported(gradInput->dtype)) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s not supported", api, DtypeName(gradInput->dtype));
        }
    } else if (gradInput->dtype != gradOut->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from gradOut dtype %s", api,
                    DtypeName(gradInput->dtype), DtypeName(gradOut->dtype));
    }
    return ACLNN_SUCCESS;
    (void)outputSize;
    (void)inputSize;
}

aclnnStatus CheckBackwardShape(const char* api, const aclTensor* gradOut, const aclIntArray* outputSize,
                               const aclIntArray* inputSize, const aclTensor* gradInput, bool checkOutShape)
{
    if (gradOut->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut must be 4-D, got %zu-D", api, gradOut->dims.size());
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 2 values, got %zu", api, outputSize->v.size());
    }
    if (inputSize->v.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input_size must have 4 values, got %zu", api, inputSize->v.size());
    }
    if (gradInput->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out must be 4-D, got %zu-D", api, gradInput->dims.size());
    }
    const bool nhwc = gradOut->format == ACL_FORMAT_NHWC;
    const int64_t outH = outputSize->v[0], outW = outputSize->v[1];
    const int64_t batch = inputSize->v[0];
    const int64_t channels = nhwc ? inputSize->v[3] : inputSize->v[1];
    const int64_t inH = nhwc ? inputSize->v[1] : inputSize->v[2];
    const int64_t inW = nhwc ? inputSize->v[2] : inputSize->v[3];
    if (!(inH > 0 && inW > 0 && outH > 0 && outW > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID,
                    "%s: input and output sizes should be greater than 0, got input (H: %ld, W: %ld) output (H: %ld, W: %ld)",
                    api, (long)inH, (long)inW, (long)outH, (long)outW);
    }
    const int64_t fullOut[4] = {batch, nhwc ? outH : channels, nhwc ? outW : outH, nhwc ? channels : outW};
    const int64_t fullIn[4] = {batch, nhwc ? inH : channels, nhwc ? inW : inH, nhwc ? channels : inW};
    for (int i = 0; i < 4; ++i) {
        if (gradOut->dims[i] != fullOut[i]) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: expected grad_output.size(%d) = %ld but got %ld", api, i,
                        (long)fullOut[i], (long)gradOut->dims[i]);
        }
    }
    if (checkOutShape) {
        for (int i = 0; i < 4; ++i) {
            if (gradInput->dims[i] != fullIn[i]) {
                return Fail(ACLNN_ERR_PARAM_INVALID, "%s: expected out.size(%d) = %ld but got %ld", api, i,
                            (long)fullIn[i], (long)gradInput->dims[i]);
            }
        }
    }
    if (inH > INT32_MAX || inW > INT32_MAX || outH > INT32_MAX || outW > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H and W must not exceed INT32_MAX", api);
    }
    return ACLNN_SUCCESS;
}

// ---- UpsampleBilinear2d ---------------------------------------------------------------------------------------
// image/resize_bilinear_v2/op_host/arch35/resize_bilinear_v2_tiling_arch35.cpp:175-243
// BilinearScale: host_common.h (shared with the allocation-free entry point)

// image/resize_bilinear_v2_grad/op_host/arch35/resize_bilinear_v2_grad_tiling_arch35.cpp:352-384 (scatter form)
float BilinearGradScale(int64_t in, int64_t out, bool align, float userScale)
{
    if (align) {
        return out > 1 ? static_cast<float>(in - 1) / static_cast<float>(out - 1) : 0.0f;
    }
    return userScale > 0.0f ? 1.0f / userScale : static_cast<float>(in) / static_cast<float>(out);
}

struct LerpOffsets {
    uint64_t lo, hi, delta;
};
LerpOffsets AllocLerp(WsPlan& ws, int64_t n)
{
    LerpOffsets o;
    o.lo = ws.Alloc(4 * static_cast<uint64_t>(n));
    o.hi = ws.Alloc(4 * static_cast<uint64_t>(n));
    o.delta = ws.Alloc(4 * static_cast<uint64_t>(n));
    return o;
}
LerpAxis LerpAt(char* w, const LerpOffsets& o)
{
    return LerpAxis{reinterpret_cast<int32_t*>(w + o.lo), reinterpret_cast<int32_t*>(w + o.hi),
                    reinterpret_cast<float*>(w + o.delta)};
}
struct RangeOffsets {
    uint64_t start, end;
};
RangeOffsets AllocRange(WsPlan& ws, int64_t n)
{
    RangeOffsets o;
    o.start = ws.Alloc(4 * static_cast<uint64_t>(n));
    o.end = ws.Alloc(4 * static_cast<uint64_t>(n));
    return o;
}
RangeAxis RangeAt(char* w, const RangeOffsets& o)
{
    return RangeAxis{reinterpret_cast<int32_t*>(w + o.start), reinterpret_cast<int32_t*>(w + o.end)};
}

aclnnStatus PlanCopy(const char* api, const aclTensor* src, const aclTensor* dst, uint64_t* workspaceSize,
                     aclOpExecutor** executor)
{
    aclTensor altSrc, altDst;
    UseOtherLayout(src, dst, altSrc, altDst); // the same dense permutation on both sides: a flat copy
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef x = StageInput(src, ws, ex);
    const BufRef y = StageOutput(dst, ws);
    const uint64_t bytes = static_cast<uint64_t>(Numel(src)) * ElemSize(src->dtype);
    ex->steps.push_back([=](char* w, cudaStream_t s) { return CopyBytes(y.At(w), x.At(w), bytes, s); });
    FinishOutput(dst, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

// Shared by aclnnUpsampleBilinear2dBackward and ...BackwardV2 (both reach ResizeBilinearV2Grad on arch35).
aclnnStatus PlanBilinearBwd(const char* api, const aclTensor* gradOut, const aclIntArray* inputSize, bool alignCorners,
                            double scalesH, double scalesW, aclTensor* outParam, uint64_t* workspaceSize,
                            aclOpExecutor** executor)
{
    const aclTensor* out = outParam;
    aclTensor altGrad, altOut;
    UseOtherLayout(gradOut, out, altGrad, altOut);
    const Geom gg = GeomOf(gradOut), gi = GeomOf(out);
    (void)inputSize;
    if (gg.h == gi.h && gg.w == gi.w && gradOut->dtype == out->dtype) {
        // same spatial size: plain copy (aclnn_upsample_bilinear_2d_backward.cpp:252,299-301; all-copy tiling key)
        return PlanCopy(api, gradOut, out, workspaceSize, executor);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    Shape4 sh = MakeShape(gi, gg); // hin/win = grad_input extent, hout/wout = grads extent
    const Dt dtIn = ToDt(gradOut->dtype), dtOut = ToDt(out->dtype);
    const Layout lay = gradOut->format == ACL_FORMAT_NHWC ? kNHWC : kNCHW;
    const AxisGeom ah{sh.hin, sh.hout, BilinearGradScale(gi.h, gg.h, alignCorners, static_cast<float>(scalesH))};
    const AxisGeom aw{sh.win, sh.wout, BilinearGradScale(gi.w, gg.w, alignCorners, static_cast<float>(scalesW))};
    const bool halfPixel = !alignCorners;
    // The atomic scatter is used only on request (opscvSetBackwardAlgo(1)) and never in deterministic mode or
    // when the output dtype differs (the reference's IsMatchSimtDetermine, ..._grad_tiling_arch35.cpp:296-299).
    const bool atomic = GetBackwardAlgo() == 1 && GetDeterministic() == 0 && dtIn == dtOut;
    // A grad_output that is a pitched NCHW view (a channel slice of the gradient of a concatenation, unit W stride) is
    // read in place by the 2x gather kernel when grad_input is written in place too: no gather copy.
    ViewStrides gradsPitch{};
    bool pitched = false;
    if (!atomic && !IsContiguous(gradOut) && IsContiguous(out) && StridesOf(gradOut, false, &gradsPitch)) {
        const BilinearPlan probe = MakeBilinearBwdPlan(dtIn, lay, sh, ah, aw, halfPixel);
        pitched = BilinearBwdTakesPitch(dtIn, dtOut, lay,
                                        static_cast<char*>(gradOut->data) + gradOut->offset * ElemSize(gradOut->dtype),
                                        static_cast<char*>(out->data) + out->offset * ElemSize(out->dtype), sh, probe,
                                        gradsPitch);
    }
    BufRef g;
    if (pitched) {
        g.base = static_cast<char*>(gradOut->data) + gradOut->offset * ElemSize(gradOut->dtype);
    } else {
        g = StageInput(gradOut, ws, ex);
    }
    const BufRef y = StageOutput(out, ws);
    const LerpOffsets lh = AllocLerp(ws, sh.hout), lw = AllocLerp(ws, sh.wout);
    if (atomic) {
        const int64_t elems = gi.n * gi.c * gi.h * gi.w;
        const bool needAcc = dtOut != Dt::F32;
        const uint64_t accOff = needAcc ? ws.Alloc(static_cast<uint64_t>(elems) * 4) : 0;
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            const LerpAxis th = LerpAt(w, lh), tw = LerpAt(w, lw);
            cudaError_t e = BuildLerpTables(ah, aw, halfPixel, 1, th, tw, s);
            if (e != cudaSuccess) {
                return e;
            }
            float* acc = needAcc ? reinterpret_cast<float*>(w + accOff) : static_cast<float*>(y.At(w));
            return BilinearBwdAtomic(dtIn, dtOut, lay, g.At(w), y.At(w), acc, sh, th, tw, s);
        });
    } else {
        const RangeOffsets rh = AllocRange(ws, sh.hin), rw = AllocRange(ws, sh.win);
        const BilinearPlan plan = MakeBilinearBwdPlan(dtIn, lay, sh, ah, aw, halfPixel);
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            const LerpAxis th = LerpAt(w, lh), tw = LerpAt(w, lw);
            const RangeAxis qh = RangeAt(w, rh), qw = RangeAt(w, rw);
            // builds the tables and ranges if the kernel it picks reads them
            return BilinearBwdGather(dtIn, dtOut, lay, g.At(w), y.At(w), sh, th, tw, qh, qw, plan, s, true,
                                     pitched ? &gradsPitch : nullptr);
        });
    }
    FinishOutput(out, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

// ---- UpsampleBicubic2dAA --------------------------------------------------------------------------------------
struct AAGeom {
    float scale, inv, support;
    int32_t taps;
};
// Scale, inverse scale, support and widest window of one axis. `in` = forward input extent.
// Cubic (filter 0): image/upsample_bicubic2d_aa/op_host/upsample_bicubic2d_aa_tiling_arch35.cpp:139-168 (forward:
// originalScale is the API's scales value, used as 1.0f / float(scales)) and
// image/upsample_bicubic2d_aa_grad/op_host/upsample_bicubic2d_aa_grad_tiling_arch35.cpp:158-183 (backward: the API
// passes float(1.0 / scales), used as the scale itself); support 2 * scale when down-scaling, else 2.
// Triangle (filter 1): image/upsample_bilinear2d_aa/op_host/upsample_bilinear2d_aa_tiling_arch35.cpp:125-154 and
// image/upsample_bilinear2d_aa_backward/op_host/upsample_bilinear2d_aa_backward_tiling_arch35.cpp:143-171: both
// directions receive float(1.0 / scales) and use it as the scale; support scale when down-scaling, else 1.
AAGeom MakeAAGeom(int64_t in, int64_t out, bool align, double userScale, bool reciprocalInDouble, int filter = 0)
{
    AAGeom g;
    if (align) {
        g.scale = out > 1 ? static_cast<float>(in - 1) / static_cast<float>(out - 1) : 0.0f;
    } else if (!reciprocalInDouble) {
        const float original = userScale > 0 ? static_cast<float>(userScale) : 0.0f;
        g.scale = original > 0.0f ? 1.0f / original : static_cast<float>(in) / static_cast<float>(out);
    } else {
        const float original = userScale > 0 ? static_cast<float>(1.0 / userScale) : 0.0f;
        g.scale = original > 0.0f ? original : static_cast<float>(in) / static_cast<float>(out);
    }
    const float unit = filter == 0 ? 2.0f : 1.0f;
    g.inv = g.scale >= 1.0f ? 1.0f / g.scale : 1.0f;
    g.support = g.scale >= 1.0f ? unit * g.scale : unit;
    // window = floor(c + s + 0.5) - floor(c - s + 0.5) <= 2s + 1
    int64_t taps = static_cast<int64_t>(std::floor(2.0 * static_cast<double>(g.support))) + 2;
    taps = taps > in ? in : taps;
    g.taps = static_cast<int32_t>(taps < 1 ? 1 : taps);
    return g;
}

struct AAOffsets {
    uint64_t xmin, xsize, w;
};
AAOffsets AllocAA(WsPlan& ws, int64_t n, int32_t taps)
{
    AAOffsets o;
    o.xmin = ws.Alloc(4 * static_cast<uint64_t>(n));
    o.xsize = ws.Alloc(4 * static_cast<uint64_t>(n));
    o.w = ws.Alloc(4 * static_cast<uint64_t>(n) * static_cast<uint64_t>(taps));
    return o;
}
AAAxis AAAt(char* w, const AAOffsets& o, int32_t taps)
{
    return AAAxis{reinterpret_cast<int32_t*>(w + o.xmin), reinterpret_cast<int32_t*>(w + o.xsize),
                  reinterpret_cast<float*>(w + o.w), taps};
}

bool AAIsCopy(const Geom& in, const Geom& out, const AAGeom& h, const AAGeom& w)
{
    // upsample_bicubic2d_aa_tiling_arch35.cpp:115-125
    return out.h == in.h && out.w == in.w && std::fabs(h.scale - 1.0f) < 1e-6f && std::fabs(w.scale - 1.0f) < 1e-6f;
}

// ---- UpsampleBicubic2d (no antialiasing) ----------------------------------------------------------------------
// Schedule of the forward (image/resize_bicubic_v2/op_host/arch35/resize_bicubic_v2_tiling_arch35.cpp:484-522):
// 1 equal extents (copy), 3 a single output pixel of an align_corners call, 2 a single input pixel, 4 integer
// source positions (integer scales with align_corners, odd integer scales without), 0 the general kernel. The
// NHWC copy schedules of :391-420 give the results of 1 and 4.
bool IsIntegerScale(float s)
{
    const float back = static_cast<float>(static_cast<int32_t>(s));
    return std::fabs(s - back) < FLT_EPSILON;
}
int32_t BicubicFwdSchedule(const Geom& in, const Geom& out, bool align, float scaleH, float scaleW)
{
    const bool intH = IsIntegerScale(scaleH), intW = IsIntegerScale(scaleW);
    const bool odd = !align && intH && intW && static_cast<int32_t>(scaleH) % 2 == 1 &&
                     static_cast<int32_t>(scaleW) % 2 == 1;
    if (out.h == in.h && out.w == in.w) {
        return 1;
    }
    if (out.h == 1 && out.w == 1 && align) {
        return 3;
    }
    if (in.h == 1 && in.w == 1) {
        return 2;
    }
    return ((align && intH && intW) || odd) ? 4 : 0;
}

// Scale and inverse scale of the backward gather kernel
// (image/resize_bicubic_v2_grad/op_host/arch35/resize_bicubic_v2_grad_base_tiling_arch35.cpp:316-364, the
// isMatchDetermine branch). `in` = grad_input extent, `out` = grads extent.
struct BicubicGradScale {
    float scale, inverse;
};
BicubicGradScale MakeBicubicGradScale(int64_t in, int64_t out, bool align, float userScale)
{
    BicubicGradScale g;
    if (align && in > 1 && out > 1) {
        g.scale = static_cast<float>(in - 1) / static_cast<float>(out - 1);
        g.inverse = static_cast<float>(out - 1) / static_cast<float>(in - 1);
    } else if (!align && userScale > 0.0f) {
        g.scale = 1.0f / userScale;
        g.inverse = userScale;
    } else {
        g.scale = static_cast<float>(in) / static_cast<float>(out);
        g.inverse = static_cast<float>(out) / static_cast<float>(in);
    }
    return g;
}

} // namespace

static aclnnStatus PlanNearestBwd(const char* api, const aclTensor* gradOut, aclTensor* gradInput, float scaleH,
                                  float scaleW, bool exact, uint64_t* workspaceSize, aclOpExecutor** executor);
static aclnnStatus PlanNearestExactBwd(const char* api, const aclTensor* gradOutput, aclTensor* out, double scalesH,
                                       double scalesW, uint64_t* workspaceSize, aclOpExecutor** executor);

extern "C" {

// ===============================================================================================================
aclnnStatus aclnnUpsampleNearest2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                   aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleNearest2d";
    if (self == nullptr || outputSize == nullptr || out == nullptr || workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    const aclnnStatus st = CheckNearestFwd(api, self, outputSize, out);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (IsEmpty(self) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    // scales = nullptr in the reference call (aclnn_upsample_nearest_2d.cpp:271-272)
    return PlanNearestFwd(api, self, out, 0.0f, 0.0f, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleNearest2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                   const aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearest2d", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnUpsampleNearest2dV2GetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                     float scalesH, float scalesW, aclTensor* out,
                                                     uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleNearest2dV2";
    // aclnn_upsample_nearest_2d_v2.cpp:324-333: null check, then the empty shortcut, then CheckParams
    if (self == nullptr || out == nullptr || workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (IsEmpty(self) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (outputSize == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: outputSize is null", api);
    }
    const aclnnStatus st = CheckNearestFwd(api, self, outputSize, out);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    return PlanNearestFwd(api, self, out, scalesH, scalesW, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleNearest2dV2(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                     aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearest2dV2", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
aclnnStatus aclnnUpsampleNearest2dBackwardGetWorkspaceSize(const aclTensor* gradOut, const aclIntArray* outputSize,
                                                           const aclIntArray* inputSize, double scalesH,
                                                           double scalesW, aclTensor* gradInput,
                                                           uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleNearest2dBackward";
    if (gradOut == nullptr || outputSize == nullptr || inputSize == nullptr || gradInput == nullptr ||
        workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    // order: dtype, shape, N/C, elements (aclnn_upsample_nearest_2d_backward.cpp:147-166)
    aclnnStatus st = CheckBackwardCommon(api, gradOut, outputSize, inputSize, gradInput, false);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (gradOut->dims.size() != 4 || outputSize->v.size() != 2 || inputSize->v.size() != 4 ||
        gradInput->dims.size() != 4) {
        return CheckBackwardShape(api, gradOut, outputSize, inputSize, gradInput, false);
    }
    if (!CheckNCDimValid(gradInput, gradOut, api)) {
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (gradInput->format != gradOut->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut and gradInput must have the same format", api);
    }
    st = CheckBackwardShape(api, gradOut, outputSize, inputSize, gradInput, true);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (IsEmpty(gradOut) || IsEmpty(gradInput)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    const Geom gg = GeomOf(gradOut), gi = GeomOf(gradInput);
    if (gg.h == gi.h && gg.w == gi.w) {
        // all-copy schedule (resize_nearest_neighbor_v2_grad_tiling_base.cpp:449-452)
        return PlanCopy(api, gradOut, gradInput, workspaceSize, executor);
    }
    // scales reach the tiling as floats (aclnn_upsample_nearest_2d_backward.cpp:351-354)
    return PlanNearestBwd(api, gradOut, gradInput, NearestScale(gi.h, gg.h, static_cast<float>(scalesH)),
                          NearestScale(gi.w, gg.w, static_cast<float>(scalesW)), false, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleNearest2dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                           aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearest2dBackward", workspace, workspaceSize, executor, stream);
}

} // extern "C"

// Window tables and the gather kernel shared by UpsampleNearest2dBackward and UpsampleNearestExact2dBackward.
static aclnnStatus PlanNearestBwd(const char* api, const aclTensor* gradOut, aclTensor* gradInputParam, float scaleH,
                                  float scaleW, bool exact, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    const aclTensor* gradInput = gradInputParam;
    aclTensor altGrad, altIn;
    UseOtherLayout(gradOut, gradInput, altGrad, altIn);
    const Geom gg = GeomOf(gradOut), gi = GeomOf(gradInput);
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const Shape4 sh = MakeShape(gi, gg);
    const Dt dt = ToDt(gradOut->dtype);
    const Layout lay = gradOut->format == ACL_FORMAT_NHWC ? kNHWC : kNCHW;
    const AxisGeom ah{sh.hin, sh.hout, scaleH, exact ? 1 : 0};
    const AxisGeom aw{sh.win, sh.wout, scaleW, exact ? 1 : 0};
    // Whole-number windows (rh x 2) between strided NCHW views with unit W strides: the pool kernel with pitches, no
    // gather or scatter copy (grad_output as a channel slice of the gradient of a concatenation is the typical case).
    ViewStrides big{}, small{};
    if ((!IsContiguous(gradOut) || !IsContiguous(gradInput)) && gradOut->dtype == gradInput->dtype &&
        StridesOf(gradOut, false, &big) && StridesOf(gradInput, true, &small) && sh.wout == 2 * sh.win &&
        sh.hout % sh.hin == 0) {
        const int32_t fh = sh.hout / sh.hin;
        const host::Ranges wh = host::NearestBwdRanges(sh.hin, sh.hout, ah.scale, exact);
        const host::Ranges ww = host::NearestBwdRanges(sh.win, sh.wout, aw.scale, exact);
        bool whole = true;
        for (int32_t i = 0; i < sh.hin && whole; ++i) {
            whole = wh.start[i] == i * fh && wh.end[i] == (i + 1) * fh;
        }
        for (int32_t i = 0; i < sh.win && whole; ++i) {
            whole = ww.start[i] == 2 * i && ww.end[i] == 2 * i + 2;
        }
        char* pg = static_cast<char*>(gradOut->data) + gradOut->offset * ElemSize(gradOut->dtype);
        char* pi = static_cast<char*>(gradInput->data) + gradInput->offset * ElemSize(gradInput->dtype);
        if (whole && NearestBwdX2PitchUsable(dt, pg, big, pi, small, sh)) {
            ex->steps.push_back([=](char*, cudaStream_t s) { return NearestBwdX2Pitch(dt, pg, big, pi, small, sh, fh, s); });
            ex->workspaceSize = 0;
            *workspaceSize = 0;
            *executor = ex;
            return ACLNN_SUCCESS;
        }
    }
    const BufRef g = StageInput(gradOut, ws, ex);
    const BufRef y = StageOutput(gradInput, ws);
    const RangeOffsets rh = AllocRange(ws, sh.hin), rw = AllocRange(ws, sh.win);
    const NearestPlan plan = MakeNearestBwdPlan(dt, lay, sh, ah, aw);
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        const RangeAxis th = RangeAt(w, rh), tw = RangeAt(w, rw);
        if (!NearestBwdUsesInteger(dt, lay, g.At(w), y.At(w), sh, plan)) {
            const cudaError_t e = BuildNearestBwdTables(ah, aw, th, tw, s);
            if (e != cudaSuccess) {
                return e;
            }
        }
        return NearestBwd(dt, lay, g.At(w), y.At(w), sh, th, tw, plan, s);
    });
    FinishOutput(gradInput, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

extern "C" {

// ===============================================================================================================
// image/upsample_nearest/op_host/op_api/aclnn_upsample_nearest_exact2d.cpp:284-340: null check, empty tensors
// succeed, then CheckParams (:185-196: dtype, shape, elements, format); the regbase branch runs
// ResizeNearestNeighborV2 with half_pixel_centers = true and float(scales) (:249, :316-317).
aclnnStatus aclnnUpsampleNearestExact2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                        double scalesH, double scalesW, aclTensor* out,
                                                        uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleNearestExact2d";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (self == nullptr || outputSize == nullptr || out == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (IsEmpty(self) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (!DtypeSupported(self->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(self->dtype));
    }
    if (self->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from self dtype %s", api, DtypeName(out->dtype),
                    DtypeName(self->dtype));
    }
    if (self->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self must be 4-D, got %zu-D", api, self->dims.size());
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 2 values, got %zu", api, outputSize->v.size());
    }
    if (out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out must be 4-D, got %zu-D", api, out->dims.size());
    }
    if (self->format != ACL_FORMAT_NCHW && self->format != ACL_FORMAT_NHWC && self->format != ACL_FORMAT_ND) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format of self only supports NCHW, NHWC, ND, got %s", api,
                    FormatName(self->format));
    }
    if (self->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format of self (%s) and out (%s) must be equal", api,
                    FormatName(self->format), FormatName(out->format));
    }
    const Geom gi = GeomOf(self), go = GeomOf(out);
    const int64_t outH = outputSize->v[0], outW = outputSize->v[1];
    if (!(gi.h > 0 && gi.w > 0 && outH > 0 && outW > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    if (gi.n != go.n || gi.c != go.c) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: N %ld/%ld or C %ld/%ld of self and out differ", api, (long)gi.n,
                    (long)go.n, (long)gi.c, (long)go.c);
    }
    if (go.h != outH || go.w != outW) { // the reference leaves this to the kernel's shape inference
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out H/W (%ld, %ld) differ from output_size (%ld, %ld)", api,
                    (long)go.h, (long)go.w, (long)outH, (long)outW);
    }
    if (!FitsInt32(gi) || !FitsInt32(go)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H and W must not exceed INT32_MAX", api);
    }
    const float sH = scalesH > 0 ? static_cast<float>(scalesH) : 0.0f;
    const float sW = scalesW > 0 ? static_cast<float>(scalesW) : 0.0f;
    return PlanNearestFwd(api, self, out, sH, sW, workspaceSize, executor, true);
}

aclnnStatus aclnnUpsampleNearestExact2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                        aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearestExact2d", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// image/upsample_nearest_exact2d_grad/op_host/op_api/aclnn_upsample_nearest_exact2d_backward.cpp:178-240: null
// check, empty tensors succeed, CheckParams (:153-175: dtype, shape, N/C with NHWC rejected, negative scales,
// elements with the up-scale limit of 50); UpsampleNearestExact2dGrad with float(scales) (:215-228).
aclnnStatus aclnnUpsampleNearestExact2dBackwardGetWorkspaceSize(const aclTensor* gradOutput,
                                                                const aclIntArray* outputSize,
                                                                const aclIntArray* inputSize, double scalesH,
                                                                double scalesW, aclTensor* out,
                                                                uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleNearestExact2dBackward";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (gradOutput == nullptr || inputSize == nullptr || out == nullptr || outputSize == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (IsEmpty(gradOutput) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (!DtypeSupported(gradOutput->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOutput dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(gradOutput->dtype));
    }
    if (gradOutput->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from gradOutput dtype %s", api,
                    DtypeName(out->dtype), DtypeName(gradOutput->dtype));
    }
    if (gradOutput->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format of gradOutput (%s) and out (%s) must be equal", api,
                    FormatName(gradOutput->format), FormatName(out->format));
    }
    if (gradOutput->dims.size() != 4 || out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOutput and out must be 4-D", api);
    }
    if (inputSize->v.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input_size must have 4 values, got %zu", api, inputSize->v.size());
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 2 values, got %zu", api, outputSize->v.size());
    }
    if (gradOutput->format == ACL_FORMAT_NHWC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: only the NCHW and ND formats are supported", api);
    }
    if (gradOutput->dims[0] != out->dims[0] || gradOutput->dims[1] != out->dims[1]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: N and C of gradOutput and out differ", api);
    }
    if (scalesH < 0 || scalesW < 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales cannot be negative (w %f, h %f)", api, scalesW, scalesH);
    }
    const int64_t inH = inputSize->v[2], inW = inputSize->v[3];
    const Geom gg = GeomOf(gradOutput), gi = GeomOf(out);
    const double realH = scalesH > 0 ? 1.0 / scalesH : static_cast<double>(inH) / static_cast<double>(gg.h);
    const double realW = scalesW > 0 ? 1.0 / scalesW : static_cast<double>(inW) / static_cast<double>(gg.w);
    if (!(realH >= 0.02 && realW >= 0.02)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales are too large (h %f, w %f)", api, realH, realW);
    }
    if (!(inH > 0 && inW > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    if (gi.h != inH || gi.w != inW || gi.n != inputSize->v[0] || gi.c != inputSize->v[1] ||
        gg.h != outputSize->v[0] || gg.w != outputSize->v[1]) {
        // the reference's tiling rejects this (upsample_nearest_exact2d_grad_tiling_arch35.cpp:244-246)
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: tensor shapes differ from input_size / output_size", api);
    }
    if (!FitsInt32(gi) || !FitsInt32(gg)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H and W must not exceed INT32_MAX", api);
    }
    return PlanNearestExactBwd(api, gradOutput, out, scalesH, scalesW, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleNearestExact2dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearestExact2dBackward", workspace, workspaceSize, executor, stream);
}

} // extern "C"

// Checked 4-D tensors in, plan out; shared by the 2-D and the 1-D entry point.
static aclnnStatus PlanNearestExactBwd(const char* api, const aclTensor* gradOutput, aclTensor* out, double scalesH,
                                       double scalesW, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    const Geom gg = GeomOf(gradOutput), gi = GeomOf(out);
    // upsample_nearest_exact2d_grad_tiling_arch35.cpp:189-200: grads extent over grad_input extent, or the scale given
    const float userH = scalesH > 0 ? static_cast<float>(scalesH) : 0.0f;
    const float userW = scalesW > 0 ? static_cast<float>(scalesW) : 0.0f;
    const float sH = userH > 0.0f ? userH : static_cast<float>(gg.h) / static_cast<float>(gi.h);
    const float sW = userW > 0.0f ? userW : static_cast<float>(gg.w) / static_cast<float>(gi.w);
    if (gg.h == gi.h && gg.w == gi.w && std::fabs(sH - 1.0f) <= 1e-8f && std::fabs(sW - 1.0f) <= 1e-8f) {
        return PlanCopy(api, gradOutput, out, workspaceSize, executor); // :112-119
    }
    return PlanNearestBwd(api, gradOutput, out, sH, sW, true, workspaceSize, executor);
}

// (N, C, L) seen as (N, C, 1, L), as the reference's View3dAs4d does (aclnn_upsample_nearest_exact1d.cpp:45-62).
static aclTensor View3dAs4d(const aclTensor* t)
{
    aclTensor v = *t;
    v.dims = {t->dims[0], t->dims[1], 1, t->dims[2]};
    v.strides = {t->strides[0], t->strides[1], t->strides[2] * t->dims[2], t->strides[2]};
    v.format = ACL_FORMAT_NCHW;
    return v;
}

extern "C" {

// ===============================================================================================================
// image/upsample_nearest/op_host/op_api/aclnn_upsample_nearest_exact1d.cpp:166-226: CheckParams (:110-121: null,
// dtype, elements, shape), empty self succeeds, then the 2-D operator on the (N, C, 1, L) view with scales
// {1, float(scales)}; formats other than NCL / ND end in ACLNN_ERR_INNER_NULLPTR (:139-141, :213).
aclnnStatus aclnnUpsampleNearestExact1dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                        double scales, aclTensor* out, uint64_t* workspaceSize,
                                                        aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleNearestExact1d";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (self == nullptr || out == nullptr || outputSize == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (!DtypeSupported(self->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(self->dtype));
    }
    if (self->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from self dtype %s", api, DtypeName(out->dtype),
                    DtypeName(self->dtype));
    }
    if (self->dims.size() != 3 || out->dims.size() != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self and out must be 3-D, got %zu-D and %zu-D", api,
                    self->dims.size(), out->dims.size());
    }
    if (outputSize->v.size() != 1) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 1 value, got %zu", api, outputSize->v.size());
    }
    const int64_t outL = outputSize->v[0];
    if (!(self->dims[0] > 0 && self->dims[1] > 0 && self->dims[2] > 0 && outL > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    if (out->dims[0] != self->dims[0] || out->dims[1] != self->dims[1] || out->dims[2] != outL) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out shape differs from (N, C, output_size)", api);
    }
    if ((self->format != ACL_FORMAT_NCL && self->format != ACL_FORMAT_ND) || out->format != self->format) {
        return Fail(ACLNN_ERR_INNER_NULLPTR, "%s: only the NCL and ND formats are supported, got %s and %s", api,
                    FormatName(self->format), FormatName(out->format));
    }
    if (self->dims[2] > INT32_MAX || outL > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: L must not exceed INT32_MAX", api);
    }
    const aclTensor self4 = View3dAs4d(self);
    aclTensor out4 = View3dAs4d(out);
    const float s = scales > 0 ? static_cast<float>(scales) : 0.0f;
    return PlanNearestFwd(api, &self4, &out4, 1.0f, s, workspaceSize, executor, true);
}

aclnnStatus aclnnUpsampleNearestExact1d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                        aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearestExact1d", workspace, workspaceSize, executor, stream);
}

// image/upsample_nearest_exact2d_grad/op_host/op_api/aclnn_upsample_nearest_exact1d_backward.cpp: CheckParams (null,
// dtype, shape, N/C, negative scale, elements with the up-scale limit of 50), empty tensors succeed, then the 2-D
// backward on the (N, C, 1, L) views with scales {1, float(scales)}.
aclnnStatus aclnnUpsampleNearestExact1dBackwardGetWorkspaceSize(const aclTensor* gradOutput,
                                                                const aclIntArray* outputSize,
                                                                const aclIntArray* inputSize, double scales,
                                                                aclTensor* out, uint64_t* workspaceSize,
                                                                aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleNearestExact1dBackward";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (gradOutput == nullptr || inputSize == nullptr || out == nullptr || outputSize == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (!DtypeSupported(gradOutput->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOutput dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(gradOutput->dtype));
    }
    if (gradOutput->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from gradOutput dtype %s", api,
                    DtypeName(out->dtype), DtypeName(gradOutput->dtype));
    }
    if (gradOutput->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format of gradOutput (%s) and out (%s) must be equal", api,
                    FormatName(gradOutput->format), FormatName(out->format));
    }
    if (gradOutput->dims.size() != 3 || out->dims.size() != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOutput and out must be 3-D", api);
    }
    if (inputSize->v.size() != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input_size must have 3 values, got %zu", api, inputSize->v.size());
    }
    if (outputSize->v.size() != 1) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 1 value, got %zu", api, outputSize->v.size());
    }
    if (gradOutput->dims[0] != out->dims[0] || gradOutput->dims[1] != out->dims[1]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: N and C of gradOutput and out differ", api);
    }
    if (scales < 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales cannot be negative (%f)", api, scales);
    }
    const int64_t inL = inputSize->v[2], outL = gradOutput->dims[2];
    const double real = scales > 0 ? 1.0 / scales : (outL != 0 ? static_cast<double>(inL) / static_cast<double>(outL) : 0.0);
    if (!(real >= 0.02)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales is too large (%f)", api, real);
    }
    if (!(gradOutput->dims[0] > 0 && inL > 0 && gradOutput->dims[1] > 0 && outL > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    if (IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (out->dims[2] != inL || out->dims[0] != inputSize->v[0] || out->dims[1] != inputSize->v[1] ||
        outL != outputSize->v[0]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: tensor shapes differ from input_size / output_size", api);
    }
    if (inL > INT32_MAX || outL > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: L must not exceed INT32_MAX", api);
    }
    const aclTensor g4 = View3dAs4d(gradOutput);
    aclTensor out4 = View3dAs4d(out);
    return PlanNearestExactBwd(api, &g4, &out4, 1.0, scales, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleNearestExact1dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearestExact1dBackward", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// image/upsample_bilinear2d/op_host/op_api/aclnn_upsample_bilinear_2d.cpp:170-195 (CheckParams)
aclnnStatus aclnnUpsampleBilinear2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                    const bool alignCorners, const double scalesH,
                                                    const double scalesW, aclTensor* out, uint64_t* workspaceSize,
                                                    aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleBilinear2d";
    if (self == nullptr || out == nullptr) {
        return Fail(ACLNN_ERR_INNER_NULLPTR, "%s: self or out is null", api); // sic: 561103 (:175)
    }
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (!DtypeSupported(self->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(self->dtype));
    }
    if (self->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from self dtype %s", api, DtypeName(out->dtype),
                    DtypeName(self->dtype));
    }
    if (self->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format of input (%s) and output (%s) must be equal", api,
                    FormatName(self->format), FormatName(out->format));
    }
    if (self->format != ACL_FORMAT_NCHW && self->format != ACL_FORMAT_NHWC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format %s not supported", api, FormatName(self->format));
    }
    if (self->dims.size() != 4 || out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self and out must be 4-D", api);
    }
    if (!CheckNCDimValid(self, out, api)) {
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (scalesW < 0 || scalesH < 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales cannot be negative (w %f, h %f)", api, scalesW, scalesH);
    }
    if (outputSize == nullptr) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: outputSize must not be null", api);
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: outputSize size must be 2, got %zu", api, outputSize->v.size());
    }
    const Geom gi = GeomOf(self), go = GeomOf(out);
    if (outputSize->v[0] != go.h || outputSize->v[1] != go.w) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: expected output size (H: %ld, W: %ld) but out tensor has (H: %ld, W: %ld)",
                    api, (long)outputSize->v[0], (long)outputSize->v[1], (long)go.h, (long)go.w);
    }
    if (IsEmpty(self) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (!FitsInt32(gi) || !FitsInt32(go)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H and W must not exceed INT32_MAX", api);
    }
    const aclTensor* outT = out;
    aclTensor altSelf, altOut;
    UseOtherLayout(self, outT, altSelf, altOut);
    if (gi.h == go.h && gi.w == go.w) {
        // all-copy schedule (resize_bilinear_v2_tiling_arch35.cpp:245-252)
        return PlanCopy(api, self, outT, workspaceSize, executor);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const Shape4 sh = MakeShape(gi, go);
    const Dt dt = ToDt(self->dtype);
    const Layout lay = self->format == ACL_FORMAT_NHWC ? kNHWC : kNCHW;
    // scales reach the tiling as floats (aclnn_upsample_bilinear_2d.cpp:413)
    const AxisGeom ah{sh.hin, sh.hout, BilinearScale(gi.h, go.h, alignCorners, static_cast<float>(scalesH))};
    const AxisGeom aw{sh.win, sh.wout, BilinearScale(gi.w, go.w, alignCorners, static_cast<float>(scalesW))};
    const bool halfPixel = !alignCorners; // resize_bilinear_v2.cpp:99
    const LerpOffsets lh = AllocLerp(ws, sh.hout), lw = AllocLerp(ws, sh.wout);
    const BilinearPlan plan = MakeBilinearFwdPlan(dt, lay, sh, ah, aw, halfPixel);
    // Pitched NCHW views (a crop or a channel slice of a larger tensor, unit W stride, 16-byte aligned pitches) on either
    // side are read and written in place by the 2x-width kernel: no gather copy, no staged result, no scatter copy.
    ViewStrides si{}, so{};
    if ((!IsContiguous(self) || !IsContiguous(outT)) && StridesOf(self, false, &si) && StridesOf(outT, true, &so)) {
        char* px = static_cast<char*>(self->data) + self->offset * ElemSize(self->dtype);
        char* py = static_cast<char*>(outT->data) + outT->offset * ElemSize(outT->dtype);
        if (BilinearFwdTakesPitch(dt, lay, px, py, sh, plan, si, so)) {
            ex->steps.push_back([=](char* w, cudaStream_t s) {
                const LerpAxis th = LerpAt(w, lh), tw = LerpAt(w, lw);
                return BilinearFwd(dt, lay, px, py, sh, th, tw, plan, s, true, &so, &si);
            });
            ex->workspaceSize = ws.Size();
            *workspaceSize = ws.Size();
            *executor = ex;
            return ACLNN_SUCCESS;
        }
    }
    const BufRef x = StageInput(self, ws, ex);
    const BufRef y = StageOutput(outT, ws);
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        const LerpAxis th = LerpAt(w, lh), tw = LerpAt(w, lw);
        return BilinearFwd(dt, lay, x.At(w), y.At(w), sh, th, tw, plan, s, true); // builds the tables if it reads them
    });
    FinishOutput(outT, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnUpsampleBilinear2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                    aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBilinear2d", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// image/resize_bilinear_v2_grad/op_api/aclnn_upsample_bilinear_2d_backward.cpp:195-224 (CheckParams):
// null, shape, dtype, elements, N/C, format
aclnnStatus aclnnUpsampleBilinear2dBackwardGetWorkspaceSize(const aclTensor* gradOut, const aclIntArray* outputSize,
                                                            const aclIntArray* inputSize, bool alignCorners,
                                                            double scalesH, double scalesW, aclTensor* out,
                                                            uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleBilinear2dBackward";
    if (gradOut == nullptr || outputSize == nullptr || inputSize == nullptr || out == nullptr ||
        workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    aclnnStatus st = CheckBackwardShape(api, gradOut, outputSize, inputSize, out, true);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    st = CheckBackwardCommon(api, gradOut, outputSize, inputSize, out, true);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (!CheckNCDimValid(gradOut, out, api)) {
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (gradOut->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut and out must have the same format", api);
    }
    if (IsEmpty(gradOut)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    return PlanBilinearBwd(api, gradOut, inputSize, alignCorners, scalesH, scalesW, out, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleBilinear2dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                            aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBilinear2dBackward", workspace, workspaceSize, executor, stream);
}

// image/upsample_bilinear2d_grad/op_host/op_api/aclnn_upsample_bilinear_2d_backward_v2.cpp:190-213 (CheckParams):
// null, shape, format, elements, N/C, dtype
aclnnStatus aclnnUpsampleBilinear2dBackwardV2GetWorkspaceSize(const aclTensor* gradOut, const aclIntArray* outputSize,
                                                              const aclIntArray* inputSize, bool alignCorners,
                                                              double scalesH, double scalesW, aclTensor* out,
                                                              uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleBilinear2dBackwardV2";
    if (gradOut == nullptr || inputSize == nullptr || outputSize == nullptr || out == nullptr ||
        workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (gradOut->dims.size() != 4 || inputSize->v.size() != 4 || outputSize->v.size() != 2) {
        return CheckBackwardShape(api, gradOut, outputSize, inputSize, out, false);
    }
    if (out->format != ACL_FORMAT_NCHW && out->format != ACL_FORMAT_NHWC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format %s of out not supported", api, FormatName(out->format));
    }
    aclnnStatus st = CheckBackwardShape(api, gradOut, outputSize, inputSize, out, true);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (!CheckNCDimValid(gradOut, out, api)) {
        return ACLNN_ERR_PARAM_INVALID;
    }
    st = CheckBackwardCommon(api, gradOut, outputSize, inputSize, out, false);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (gradOut->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut and out must have the same format", api);
    }
    if (IsEmpty(gradOut) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    return PlanBilinearBwd(api, gradOut, inputSize, alignCorners, scalesH, scalesW, out, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleBilinear2dBackwardV2(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                              aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBilinear2dBackwardV2", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// The two anti-aliased forwards share one planner. filter 0: aclnnUpsampleBicubic2dAA
// (image/upsample_bicubic2d_aa/op_host/op_api/aclnn_upsample_bicubic2d_aa.cpp:145-162 CheckParams, :59-124);
// filter 1: aclnnUpsampleBilinear2dAA (image/upsample_bilinear2d_aa/op_host/op_api/aclnn_upsample_bilinear2d_aa.cpp
// :155-182 CheckParams: the same checks plus negative scales; :214-219 scale passing).
static aclnnStatus PlanAAForward(const char* api, int filter, const aclTensor* x, const aclIntArray* outputSize,
                                 const bool alignCorners, const double scalesH, const double scalesW, aclTensor* out,
                                 uint64_t* workspaceSize, aclOpExecutor** executor)
{
    if (workspaceSize == nullptr || executor == nullptr) { // OP_CHECK_COMM_INPUT (:168)
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (x == nullptr || outputSize == nullptr || out == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (!DtypeSupported(x->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: x dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(x->dtype));
    }
    if (x->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from x dtype %s", api, DtypeName(out->dtype),
                    DtypeName(x->dtype));
    }
    if (x->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: x must be 4-D, got %zu-D", api, x->dims.size());
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 2 values, got %zu", api, outputSize->v.size());
    }
    if (out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out must be 4-D, got %zu-D", api, out->dims.size());
    }
    if (filter == 1 && (scalesH < 0 || scalesW < 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales cannot be negative (w %f, h %f)", api, scalesW, scalesH);
    }
    const int64_t inH = x->dims[2], inW = x->dims[3], outH = outputSize->v[0], outW = outputSize->v[1];
    if (!(inH > 0 && inW > 0 && outH > 0 && outW > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID,
                    "%s: input and output sizes should be greater than 0, got input (H: %ld, W: %ld) output (H: %ld, W: %ld)",
                    api, (long)inH, (long)inW, (long)outH, (long)outW);
    }
    if (!(x->dims[1] > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: non-empty 4-D data tensor expected", api);
    }
    if (x->dims[0] != out->dims[0] || x->dims[1] != out->dims[1]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: N and C of x and out must be equal", api);
    }
    if (out->dims[2] != outH || out->dims[3] != outW) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out H/W (%ld, %ld) differ from output_size (%ld, %ld)", api,
                    (long)out->dims[2], (long)out->dims[3], (long)outH, (long)outW);
    }
    const bool fmtOk = (x->format == ACL_FORMAT_ND || x->format == ACL_FORMAT_NCHW) &&
                       (out->format == ACL_FORMAT_ND || out->format == ACL_FORMAT_NCHW);
    if (!fmtOk) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: storage format only supports NCHW, got %s and %s", api,
                    FormatName(x->format), FormatName(out->format));
    }
    if (inH > INT32_MAX || inW > INT32_MAX || outH > INT32_MAX || outW > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H and W must not exceed INT32_MAX", api);
    }
    if (IsEmpty(x) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    Geom gi{x->dims[0], x->dims[1], inH, inW}, go{x->dims[0], x->dims[1], outH, outW};
    const AAGeom ah = MakeAAGeom(inH, outH, alignCorners, scalesH, filter == 1, filter);
    const AAGeom aw = MakeAAGeom(inW, outW, alignCorners, scalesW, filter == 1, filter);
    if (AAIsCopy(gi, go, ah, aw)) {
        return PlanCopy(api, x, out, workspaceSize, executor);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef xin = StageInput(x, ws, ex);
    const BufRef y = StageOutput(out, ws);
    const Shape4 sh = MakeShape(gi, go);
    const Dt dt = ToDt(x->dtype);
    const AxisGeom gh{sh.hin, sh.hout, ah.scale}, gw{sh.win, sh.wout, aw.scale};
    const AAOffsets oh = AllocAA(ws, sh.hout, ah.taps), ow = AllocAA(ws, sh.wout, aw.taps);
    const AAFwdPlan plan = MakeAAFwdPlan(dt, sh, ah.scale, aw.taps);
    const RangeOffsets rh = AllocRange(ws, sh.hin), rw = AllocRange(ws, sh.win);
    const uint64_t wrowOff = ws.Alloc(plan.wrowBytes);
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        const AAAxis th = AAAt(w, oh, ah.taps), tw = AAAt(w, ow, aw.taps);
        const RangeAxis qh = RangeAt(w, rh), qw = RangeAt(w, rw);
        cudaError_t e = BuildAATables(gh, gw, ah.inv, aw.inv, ah.support, aw.support, th, tw, false, filter, s);
        if (e != cudaSuccess) {
            return e;
        }
        if (plan.stream) {
            e = BuildAABwdRanges(gh, gw, th, tw, qh, qw, s);
            if (e != cudaSuccess) {
                return e;
            }
        }
        return BicubicAAFwd(dt, xin.At(w), y.At(w), sh, th, tw, qh, reinterpret_cast<float*>(w + wrowOff), plan, s);
    });
    FinishOutput(out, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnUpsampleBicubic2dAAGetWorkspaceSize(const aclTensor* x, const aclIntArray* outputSize,
                                                     const bool alignCorners, const double scalesH,
                                                     const double scalesW, aclTensor* out, uint64_t* workspaceSize,
                                                     aclOpExecutor** executor)
{
    return PlanAAForward("aclnnUpsampleBicubic2dAA", 0, x, outputSize, alignCorners, scalesH, scalesW, out,
                         workspaceSize, executor);
}

aclnnStatus aclnnUpsampleBicubic2dAA(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                     aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBicubic2dAA", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// The two anti-aliased backwards share one planner. filter 0: aclnnUpsampleBicubic2dAAGrad
// (image/upsample_bicubic2d_aa_grad/op_host/op_api/aclnn_upsample_bicubic2d_aa_grad.cpp:159-181 CheckParams: null,
// dtype, scales, shape, N/C, elements); filter 1: aclnnUpsampleBilinear2dAABackward
// (image/upsample_bilinear2d_aa_backward/op_host/op_api/aclnn_upsample_bilinear2d_aa_backward.cpp:153-177, the same
// checks; :209-213 scale passing).
static aclnnStatus PlanAABackward(const char* api, int filter, const aclTensor* gradOutput,
                                  const aclIntArray* outputSize, const aclIntArray* inputSize, bool alignCorners,
                                  double scalesH, double scalesW, aclTensor* out, uint64_t* workspaceSize,
                                  aclOpExecutor** executor)
{
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (gradOutput == nullptr || inputSize == nullptr || out == nullptr || outputSize == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (!DtypeSupported(gradOutput->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOutput dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(gradOutput->dtype));
    }
    if (gradOutput->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from gradOutput dtype %s", api,
                    DtypeName(out->dtype), DtypeName(gradOutput->dtype));
    }
    if (scalesW < 0 || scalesH < 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales cannot be negative (w %f, h %f)", api, scalesW, scalesH);
    }
    if (gradOutput->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format of gradOutput (%s) and out (%s) must be equal", api,
                    FormatName(gradOutput->format), FormatName(out->format));
    }
    if (gradOutput->dims.size() != 4 || out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOutput and out must be 4-D", api);
    }
    if (inputSize->v.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input_size must have 4 values, got %zu", api, inputSize->v.size());
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 2 values, got %zu", api, outputSize->v.size());
    }
    if (gradOutput->format == ACL_FORMAT_NCHW && !CheckNCDimValid(gradOutput, out, api)) {
        return ACLNN_ERR_PARAM_INVALID;
    }
    const int64_t outN = gradOutput->dims[0], outC = gradOutput->dims[1], outH = gradOutput->dims[2],
                  outW = gradOutput->dims[3];
    const int64_t inH = inputSize->v[2], inW = inputSize->v[3];
    if (!(outN > 0 && inH > 0 && inW > 0 && outC > 0 && outH > 0 && outW > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    const bool fmtOk = (gradOutput->format == ACL_FORMAT_ND || gradOutput->format == ACL_FORMAT_NCHW);
    if (!fmtOk) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: storage format only supports NCHW, got %s", api,
                    FormatName(gradOutput->format));
    }
    if (outputSize->v[0] != outH || outputSize->v[1] != outW) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOutput H/W (%ld, %ld) differ from output_size (%ld, %ld)", api,
                    (long)outH, (long)outW, (long)outputSize->v[0], (long)outputSize->v[1]);
    }
    if (out->dims[0] != inputSize->v[0] || out->dims[1] != inputSize->v[1] || out->dims[2] != inH ||
        out->dims[3] != inW || out->dims[0] != outN || out->dims[1] != outC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out shape must equal input_size and share N, C with gradOutput", api);
    }
    if (inH > INT32_MAX || inW > INT32_MAX || outH > INT32_MAX || outW > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H and W must not exceed INT32_MAX", api);
    }
    if (IsEmpty(gradOutput) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    Geom gi{outN, outC, inH, inW}, gg{outN, outC, outH, outW};
    const AAGeom ah = MakeAAGeom(inH, outH, alignCorners, scalesH, true, filter);
    const AAGeom aw = MakeAAGeom(inW, outW, alignCorners, scalesW, true, filter);
    if (AAIsCopy(gi, gg, ah, aw)) {
        return PlanCopy(api, gradOutput, out, workspaceSize, executor);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef g = StageInput(gradOutput, ws, ex);
    const BufRef y = StageOutput(out, ws);
    const Shape4 sh = MakeShape(gi, gg);
    const Dt dt = ToDt(gradOutput->dtype);
    const AxisGeom gh{sh.hin, sh.hout, ah.scale}, gw{sh.win, sh.wout, aw.scale};
    const AAOffsets oh = AllocAA(ws, sh.hout, ah.taps), ow = AllocAA(ws, sh.wout, aw.taps);
    const bool atomic = GetBackwardAlgo() == 1 && GetDeterministic() == 0;
    // With scale == 0 (align_corners and a single output pixel) the reference's two backward kernels disagree on
    // the filter centre: the default (atomic) kernel uses 0.5, the deterministic one keeps the forward's 0
    // (upsample_bicubic2d_aa_grad_simt_base.h:38 vs ..._simt_base_deter.h:96). Follow whichever the mode selects.
    // The triangle-filter kernels (upsample_bilinear2d_aa_backward_simt_base.h:88,146) keep scale * (i + 0.5) in both.
    const bool bwdCentre = filter == 0 && GetDeterministic() == 0;
    if (atomic) {
        const int64_t elems = gi.n * gi.c * gi.h * gi.w;
        const bool needAcc = dt != Dt::F32;
        const uint64_t accOff = needAcc ? ws.Alloc(static_cast<uint64_t>(elems) * 4) : 0;
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            const AAAxis th = AAAt(w, oh, ah.taps), tw = AAAt(w, ow, aw.taps);
            cudaError_t e = BuildAATables(gh, gw, ah.inv, aw.inv, ah.support, aw.support, th, tw, bwdCentre, filter, s);
            if (e != cudaSuccess) {
                return e;
            }
            float* acc = needAcc ? reinterpret_cast<float*>(w + accOff) : static_cast<float*>(y.At(w));
            return BicubicAABwdAtomic(dt, g.At(w), y.At(w), acc, sh, th, tw, s);
        });
    } else {
        const RangeOffsets rh = AllocRange(ws, sh.hin), rw = AllocRange(ws, sh.win);
        const AABwdPlan plan = MakeAABwdPlan(dt, sh, ah.scale, aw.scale);
        const uint64_t wrowH = ws.Alloc(plan.wrowBytesH), wrowW = ws.Alloc(plan.wrowBytesW);
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            const AAAxis th = AAAt(w, oh, ah.taps), tw = AAAt(w, ow, aw.taps);
            const RangeAxis qh = RangeAt(w, rh), qw = RangeAt(w, rw);
            cudaError_t e = BuildAATables(gh, gw, ah.inv, aw.inv, ah.support, aw.support, th, tw, bwdCentre, filter, s);
            if (e != cudaSuccess) {
                return e;
            }
            e = BuildAABwdRanges(gh, gw, th, tw, qh, qw, s);
            if (e != cudaSuccess) {
                return e;
            }
            return BicubicAABwdGather(dt, g.At(w), y.At(w), sh, th, tw, qh, qw, reinterpret_cast<float*>(w + wrowH),
                                      reinterpret_cast<float*>(w + wrowW), plan, s);
        });
    }
    FinishOutput(out, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnUpsampleBicubic2dAAGradGetWorkspaceSize(const aclTensor* gradOutput, const aclIntArray* outputSize,
                                                         const aclIntArray* inputSize, bool alignCorners,
                                                         double scalesH, double scalesW, aclTensor* out,
                                                         uint64_t* workspaceSize, aclOpExecutor** executor)
{
    return PlanAABackward("aclnnUpsampleBicubic2dAAGrad", 0, gradOutput, outputSize, inputSize, alignCorners, scalesH,
                          scalesW, out, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleBicubic2dAAGrad(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                         aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBicubic2dAAGrad", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
aclnnStatus aclnnUpsampleBilinear2dAAGetWorkspaceSize(const aclTensor* input, const aclIntArray* outputSize,
                                                      bool alignCorners, double scalesH, double scalesW,
                                                      aclTensor* out, uint64_t* workspaceSize,
                                                      aclOpExecutor** executor)
{
    return PlanAAForward("aclnnUpsampleBilinear2dAA", 1, input, outputSize, alignCorners, scalesH, scalesW, out,
                         workspaceSize, executor);
}

aclnnStatus aclnnUpsampleBilinear2dAA(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                      aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBilinear2dAA", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnUpsampleBilinear2dAABackwardGetWorkspaceSize(const aclTensor* gradOutput,
                                                              const aclIntArray* outputSize,
                                                              const aclIntArray* inputSize, bool alignCorners,
                                                              double scalesH, double scalesW, aclTensor* out,
                                                              uint64_t* workspaceSize, aclOpExecutor** executor)
{
    return PlanAABackward("aclnnUpsampleBilinear2dAABackward", 1, gradOutput, outputSize, inputSize, alignCorners,
                          scalesH, scalesW, out, workspaceSize, executor);
}

aclnnStatus aclnnUpsampleBilinear2dAABackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                              aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBilinear2dAABackward", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// image/upsample_bicubic2d/op_host/op_api/aclnn_upsample_bicubic_2d.cpp:70-172 (CheckParams: null, dtype, format,
// shape), :233-276 (the first phase: checks, empty tensors succeed, ResizeBicubicV2 with float(scales))
aclnnStatus aclnnUpsampleBicubic2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                   const bool alignCorners, const double scalesH, const double scalesW,
                                                   aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleBicubic2d";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (outputSize == nullptr || self == nullptr || out == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (!DtypeSupported(self->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(self->dtype));
    }
    if (self->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from self dtype %s", api, DtypeName(out->dtype),
                    DtypeName(self->dtype));
    }
    if (self->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self (%s) and out (%s) must have the same format", api,
                    FormatName(self->format), FormatName(out->format));
    }
    if (out->format != ACL_FORMAT_NCHW && out->format != ACL_FORMAT_NHWC && out->format != ACL_FORMAT_ND) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the format must be NCHW, NHWC or ND, got %s", api,
                    FormatName(out->format));
    }
    if (self->dims.size() != 4 || out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self and out must be 4-D, got %zu-D and %zu-D", api,
                    self->dims.size(), out->dims.size());
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: outputSize must have 2 values, got %zu", api, outputSize->v.size());
    }
    const Geom gi = GeomOf(self);
    Geom go = gi;
    go.h = outputSize->v[0];
    go.w = outputSize->v[1];
    if (!(gi.c > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: non-empty 4-D data tensor expected", api);
    }
    if (!(gi.h > 0 && gi.w > 0 && go.h > 0 && go.w > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID,
                    "%s: size of H and W must be greater than 0, got input (H: %ld, W: %ld), output (H: %ld, W: %ld)",
                    api, (long)gi.h, (long)gi.w, (long)go.h, (long)go.w);
    }
    const Geom gOut = GeomOf(out);
    if (gOut.n != go.n || gOut.c != go.c || gOut.h != go.h || gOut.w != go.w) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out shape differs from (N, C, outputSize) of self", api);
    }
    if (!FitsInt32(gi) || !FitsInt32(go) || gi.w * gi.c > INT32_MAX || go.w * go.c > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H, W and W*C must not exceed INT32_MAX", api);
    }
    if (IsEmpty(self)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    const float sH = BilinearScale(gi.h, go.h, alignCorners, static_cast<float>(scalesH));
    const float sW = BilinearScale(gi.w, go.w, alignCorners, static_cast<float>(scalesW));
    const int32_t schedule = BicubicFwdSchedule(gi, go, alignCorners, sH, sW);
    if (schedule == 1) {
        return PlanCopy(api, self, out, workspaceSize, executor);
    }
    const aclTensor* outT = out;
    aclTensor altSelf, altOut;
    UseOtherLayout(self, outT, altSelf, altOut);
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef xin = StageInput(self, ws, ex);
    const BufRef y = StageOutput(outT, ws);
    const Shape4 sh = MakeShape(gi, go);
    const Dt dt = ToDt(self->dtype);
    const Layout lay = self->format == ACL_FORMAT_NHWC ? kNHWC : kNCHW;
    const bool halfPixel = !alignCorners;
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        return Bicubic2dFwd(dt, lay, xin.At(w), y.At(w), sh, sH, sW, halfPixel, schedule, s);
    });
    FinishOutput(outT, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnUpsampleBicubic2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                   aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBicubic2d", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// image/upsample_bicubic2d_grad/op_host/op_api/aclnn_upsample_bicubic_2d_backward.cpp:229-247 (CheckParams: null,
// elements, format, dtype), :317-366 (empty gradOut succeeds; ResizeBicubicV2Grad with float(scales))
aclnnStatus aclnnUpsampleBicubic2dBackwardGetWorkspaceSize(const aclTensor* gradOut, const aclIntArray* outputSize,
                                                           const aclIntArray* inputSize, const bool alignCorners,
                                                           double scalesH, double scalesW, aclTensor* gradInput,
                                                           uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnUpsampleBicubic2dBackward";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (inputSize == nullptr || gradInput == nullptr || gradOut == nullptr || outputSize == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (gradOut->dims.size() != 4 || gradInput->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut and gradInput must be 4-D, got %zu-D and %zu-D", api,
                    gradOut->dims.size(), gradInput->dims.size());
    }
    if (outputSize->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: outputSize must have two elements, got %zu", api,
                    outputSize->v.size());
    }
    if (inputSize->v.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: inputSize must have four elements, got %zu", api,
                    inputSize->v.size());
    }
    const bool nhwc = gradInput->format == ACL_FORMAT_NHWC;
    if (!nhwc && gradInput->format != ACL_FORMAT_NCHW && gradInput->format != ACL_FORMAT_ND) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format only supports NCHW, NHWC or ND, got %s", api,
                    FormatName(gradInput->format));
    }
    Geom gi, gg;
    gi.n = inputSize->v[0];
    gi.c = nhwc ? inputSize->v[3] : inputSize->v[1];
    gi.h = nhwc ? inputSize->v[1] : inputSize->v[2];
    gi.w = nhwc ? inputSize->v[2] : inputSize->v[3];
    gg = gi;
    gg.h = outputSize->v[0];
    gg.w = outputSize->v[1];
    if (!(gi.h > 0 && gi.w > 0 && gg.h > 0 && gg.w > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID,
                    "%s: size of H and W must be greater than 0, got input (H: %ld, W: %ld), output (H: %ld, W: %ld)",
                    api, (long)gi.h, (long)gi.w, (long)gg.h, (long)gg.w);
    }
    for (int i = 0; i < 4; ++i) {
        const int64_t wantOut = nhwc ? (i == 0 ? gi.n : i == 1 ? gg.h : i == 2 ? gg.w : gi.c)
                                     : (i == 0 ? gi.n : i == 1 ? gi.c : i == 2 ? gg.h : gg.w);
        if (gradOut->dims[i] != wantOut) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: dim %d of gradOut should be %ld, got %ld", api, i, (long)wantOut,
                        (long)gradOut->dims[i]);
        }
        if (gradInput->dims[i] != inputSize->v[i]) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: dim %d of gradInput should be %ld, got %ld", api, i,
                        (long)inputSize->v[i], (long)gradInput->dims[i]);
        }
    }
    if (gradOut->format != ACL_FORMAT_ND && gradOut->format != ACL_FORMAT_NCHW && gradOut->format != ACL_FORMAT_NHWC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: format only supports NCHW, NHWC or ND, got %s", api,
                    FormatName(gradOut->format));
    }
    if (gradOut->format != gradInput->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut (%s) and gradInput (%s) must have the same format", api,
                    FormatName(gradOut->format), FormatName(gradInput->format));
    }
    if (!DtypeSupported(gradOut->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(gradOut->dtype));
    }
    if (gradOut->dtype != gradInput->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradInput dtype %s differs from gradOut dtype %s", api,
                    DtypeName(gradInput->dtype), DtypeName(gradOut->dtype));
    }
    if (!FitsInt32(gi) || !FitsInt32(gg) || gi.w * gi.c > INT32_MAX || gg.w * gg.c > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: H, W and W*C must not exceed INT32_MAX", api);
    }
    if (IsEmpty(gradOut)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (gi.h == gg.h && gi.w == gg.w) { // resize_bicubic_v2_grad_all_copy_tiling_arch35.cpp:23-30
        return PlanCopy(api, gradOut, gradInput, workspaceSize, executor);
    }
    const aclTensor* inT = gradInput;
    aclTensor altGrad, altIn;
    UseOtherLayout(gradOut, inT, altGrad, altIn);
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef g = StageInput(gradOut, ws, ex);
    const BufRef y = StageOutput(inT, ws);
    const Shape4 sh = MakeShape(gi, gg);
    const Dt dt = ToDt(gradOut->dtype);
    const Layout lay = gradOut->format == ACL_FORMAT_NHWC ? kNHWC : kNCHW; // after the layout swap
    const BicubicGradScale bh = MakeBicubicGradScale(gi.h, gg.h, alignCorners, static_cast<float>(scalesH));
    const BicubicGradScale bw = MakeBicubicGradScale(gi.w, gg.w, alignCorners, static_cast<float>(scalesW));
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        return Bicubic2dBwd(dt, lay, g.At(w), y.At(w), sh, bh.scale, bw.scale, bh.inverse, bw.inverse, alignCorners, s);
    });
    FinishOutput(inT, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnUpsampleBicubic2dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                           aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleBicubic2dBackward", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
// image/resize_bilinear_v2/op_api/aclnn_resize.cpp:172-190 (CheckParams: null, mode, dtype, format, elements, shape),
// :245-278 (regbase branch: "nearest" runs ResizeNearestNeighborV2 without scales, align_corners or half-pixel
// centres, "bilinear" runs ResizeBilinearV2 with half-pixel centres). The output extent is the out tensor's, which the
// element check ties to floor(extent * scale) within 1e-5 of the scale.
aclnnStatus aclnnResizeGetWorkspaceSize(const aclTensor* self, const aclFloatArray* scales, const char* mode,
                                        aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnResize";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (self == nullptr || scales == nullptr || out == nullptr || mode == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    const bool nearest = std::strncmp(mode, "nearest", 7) == 0;
    if (!nearest && std::strncmp(mode, "bilinear", 8) != 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: mode %s is not nearest or bilinear", api, mode);
    }
    if (!DtypeSupported(self->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(self->dtype));
    }
    if (self->dtype != out->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from self dtype %s", api, DtypeName(out->dtype),
                    DtypeName(self->dtype));
    }
    if (self->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the format of self and out must be the same", api);
    }
    if (self->format != ACL_FORMAT_NCHW && self->format != ACL_FORMAT_NHWC) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the format of self must be NCHW or NHWC, got %s", api,
                    FormatName(self->format));
    }
    if (self->dims.size() != 4 || out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self and out must be 4-D", api);
    }
    if (scales->v.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales must have 4 values, got %zu", api, scales->v.size());
    }
    const Geom gi = GeomOf(self), go = GeomOf(out);
    if (gi.n != go.n || gi.c != go.c) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the batch or channel extent of self and out differ", api);
    }
    const bool nhwc = self->format == ACL_FORMAT_NHWC;
    const double sh = static_cast<double>(scales->v[nhwc ? 1 : 2]), sw = static_cast<double>(scales->v[nhwc ? 2 : 3]);
    const double eps = 1e-5;
    const int64_t hMax = static_cast<int64_t>(static_cast<double>(gi.h) * (sh + eps));
    const int64_t hMin = static_cast<int64_t>(static_cast<double>(gi.h) * (sh - eps));
    const int64_t wMax = static_cast<int64_t>(static_cast<double>(gi.w) * (sw + eps));
    const int64_t wMin = static_cast<int64_t>(static_cast<double>(gi.w) * (sw - eps));
    if (go.h < hMin || go.h > hMax) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the height of out (%ld) does not match %ld * %f", api, (long)go.h,
                    (long)gi.h, sh);
    }
    if (go.w < wMin || go.w > wMax) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the width of out (%ld) does not match %ld * %f", api, (long)go.w,
                    (long)gi.w, sw);
    }
    aclIntArray size;
    size.v = {go.h, go.w};
    const aclnnStatus st = nearest
                               ? aclnnUpsampleNearest2dGetWorkspaceSize(self, &size, out, workspaceSize, executor)
                               : aclnnUpsampleBilinear2dGetWorkspaceSize(self, &size, false, 0.0, 0.0, out,
                                                                         workspaceSize, executor);
    if (st == ACLNN_SUCCESS && *executor != nullptr) {
        (*executor)->api = api;
    }
    return st;
}

aclnnStatus aclnnResize(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    return RunExecutor("aclnnResize", workspace, workspaceSize, executor, stream);
}

// ===============================================================================================================
aclnnStatus opscvDebugAxisTable(int32_t kind, int64_t inSize, int64_t outSize, int32_t alignCorners, float userScale,
                                int32_t* i0, int32_t* i1, float* f0, int32_t* tapsOut)
{
    static const char* api = "opscvDebugAxisTable";
    if (inSize <= 0 || outSize <= 0 || inSize > INT32_MAX || outSize > INT32_MAX) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: sizes must be in [1, INT32_MAX]", api);
    }
    const int32_t in = static_cast<int32_t>(inSize), out = static_cast<int32_t>(outSize);
    AAGeom aa{};
    int aaFilter = 0;
    int64_t nInt = 0, nFloat = 0;
    switch (kind) {
        case 0: nInt = out; break;
        case 1: nInt = in; break;
        case 2: nInt = out; nFloat = out; break;
        case 3:
        case 4:
            aaFilter = kind == 4 ? 1 : 0;
            aa = MakeAAGeom(in, out, alignCorners != 0, userScale, aaFilter == 1, aaFilter);
            if (tapsOut != nullptr) {
                *tapsOut = aa.taps;
            }
            if (f0 == nullptr) {
                return ACLNN_SUCCESS;
            }
            nInt = out;
            nFloat = static_cast<int64_t>(out) * aa.taps;
            break;
        default: return Fail(ACLNN_ERR_PARAM_INVALID, "%s: unknown kind %d", api, kind);
    }
    if (i0 == nullptr || (kind != 0 && i1 == nullptr) || (nFloat > 0 && f0 == nullptr)) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null output array", api);
    }
    int32_t *d0 = nullptr, *d1 = nullptr;
    float* df = nullptr;
    cudaError_t e = cudaMalloc(&d0, sizeof(int32_t) * nInt);
    if (e == cudaSuccess) {
        e = cudaMalloc(&d1, sizeof(int32_t) * nInt);
    }
    if (e == cudaSuccess && nFloat > 0) {
        e = cudaMalloc(&df, sizeof(float) * nFloat);
    }
    if (e == cudaSuccess) {
        if (kind == 0) {
            const AxisGeom g{in, out, NearestScale(in, out, userScale)};
            e = BuildNearestFwdTables(g, g, NearestAxis{d0}, NearestAxis{d1}, nullptr);
        } else if (kind == 1) {
            const AxisGeom g{in, out, NearestScale(in, out, userScale)};
            // second table goes to scratch; only the first pair is returned
            int32_t *s0 = nullptr, *s1 = nullptr;
            e = cudaMalloc(&s0, sizeof(int32_t) * nInt);
            if (e == cudaSuccess) {
                e = cudaMalloc(&s1, sizeof(int32_t) * nInt);
            }
            if (e == cudaSuccess) {
                e = BuildNearestBwdTables(g, g, RangeAxis{d0, d1}, RangeAxis{s0, s1}, nullptr);
            }
            if (e == cudaSuccess) {
                e = cudaDeviceSynchronize();
            }
            cudaFree(s0);
            cudaFree(s1);
        } else if (kind == 2) {
            const AxisGeom g{in, out, BilinearScale(in, out, alignCorners != 0, userScale)};
            int32_t *s0 = nullptr, *s1 = nullptr;
            float* sf = nullptr;
            e = cudaMalloc(&s0, sizeof(int32_t) * nInt);
            if (e == cudaSuccess) {
                e = cudaMalloc(&s1, sizeof(int32_t) * nInt);
            }
            if (e == cudaSuccess) {
                e = cudaMalloc(&sf, sizeof(float) * nFloat);
            }
            if (e == cudaSuccess) {
                e = BuildLerpTables(g, g, alignCorners == 0, 0, LerpAxis{d0, d1, df}, LerpAxis{s0, s1, sf}, nullptr);
            }
            if (e == cudaSuccess) {
                e = cudaDeviceSynchronize();
            }
            cudaFree(s0);
            cudaFree(s1);
            cudaFree(sf);
        } else {
            const AxisGeom g{in, out, aa.scale};
            int32_t *s0 = nullptr, *s1 = nullptr;
            float* sf = nullptr;
            e = cudaMalloc(&s0, sizeof(int32_t) * nInt);
            if (e == cudaSuccess) {
                e = cudaMalloc(&s1, sizeof(int32_t) * nInt);
            }
            if (e == cudaSuccess) {
                e = cudaMalloc(&sf, sizeof(float) * nFloat);
            }
            if (e == cudaSuccess) {
                e = BuildAATables(g, g, aa.inv, aa.inv, aa.support, aa.support, AAAxis{d0, d1, df, aa.taps},
                                  AAAxis{s0, s1, sf, aa.taps}, false, aaFilter, nullptr);
            }
            if (e == cudaSuccess) {
                e = cudaDeviceSynchronize();
            }
            cudaFree(s0);
            cudaFree(s1);
            cudaFree(sf);
        }
    }
    if (e == cudaSuccess) {
        e = cudaDeviceSynchronize();
    }
    if (e == cudaSuccess) {
        e = cudaMemcpy(i0, d0, sizeof(int32_t) * nInt, cudaMemcpyDeviceToHost);
    }
    if (e == cudaSuccess && kind != 0) {
        e = cudaMemcpy(i1, d1, sizeof(int32_t) * nInt, cudaMemcpyDeviceToHost);
    }
    if (e == cudaSuccess && nFloat > 0) {
        e = cudaMemcpy(f0, df, sizeof(float) * nFloat, cudaMemcpyDeviceToHost);
    }
    cudaFree(d0);
    cudaFree(d1);
    cudaFree(df);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return Fail(ACLNN_ERR_RUNTIME_ERROR, "%s: CUDA error %d (%s)", api, static_cast<int>(e), cudaGetErrorString(e));
    }
    return ACLNN_SUCCESS;
}

} // extern "C"
