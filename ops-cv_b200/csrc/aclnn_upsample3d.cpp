// First- and second-phase entry points of the 3-D resamplers: UpsampleNearest3d, UpsampleNearestExact3d and
// UpsampleTrilinear3d, forward and backward, on NCDHW (or ND) and NDHWC tensors. Same structure as the 2-D entry
// points: the first phase repeats the reference's checks, computes the scales with the expressions of its arch35 tiling and freezes the
// launches into the executor.
#include <algorithm>
#include <cmath>

#include "host_common.h"
#include "host_tables.h"

using namespace opscv;

namespace {

struct Geom5 {
    int64_t n = 0, c = 0, d = 0, h = 0, w = 0;
};

// View dims are [N, C, D, H, W] for NCDHW / ND and [N, D, H, W, C] for NDHWC.
Geom5 Geom5Of(const aclTensor* t)
{
    Geom5 g;
    if (t->format == ACL_FORMAT_NDHWC) {
        g.n = t->dims[0];
        g.d = t->dims[1];
        g.h = t->dims[2];
        g.w = t->dims[3];
        g.c = t->dims[4];
    } else {
        g.n = t->dims[0];
        g.c = t->dims[1];
        g.d = t->dims[2];
        g.h = t->dims[3];
        g.w = t->dims[4];
    }
    return g;
}

aclnnStatus EmptyOk(const char* api, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    *workspaceSize = 0;
    *executor = ex;
    return ACLNN_SUCCESS;
}

bool FormatOk(aclFormat f) { return f == ACL_FORMAT_NCDHW || f == ACL_FORMAT_NDHWC || f == ACL_FORMAT_ND; }

bool Fits(const Geom5& g)
{
    return g.d <= INT32_MAX && g.h <= INT32_MAX && g.w <= INT32_MAX && g.c <= INT32_MAX && g.w * g.c <= INT32_MAX;
}

// image/upsample_nearest3d/op_host/upsample_nearest3d_tiling_arch35.cpp:372-386
float FwdScale(int64_t in, int64_t out, float user)
{
    return user > 0.0f ? 1.0f / user : static_cast<float>(in) / static_cast<float>(out);
}
// image/upsample_nearest3d_grad/op_host/upsample_nearest3d_grad_tiling_arch35.cpp:194-208
float BwdScale(int64_t gradsExtent, int64_t inputExtent, float user)
{
    return user > 0.0f ? user : static_cast<float>(gradsExtent) / static_cast<float>(inputExtent);
}

// Whole-number up-scale factor of one axis, or 0: out = r * in and every source index (forward) / window edge
// (backward) that the kernels' fp32 expressions give equals the integer rule d / r resp. r * y. Same operations in
// the same order as SrcIdx / WindowEdge in upsample_nearest3d.cu (this file is compiled without contraction).
int32_t WholeFactorFwd(int64_t in, int64_t out, float scale, bool exact)
{
    if (out % in != 0) {
        return 0;
    }
    const int64_t r = out / in;
    for (int64_t i = 0; i < out; ++i) {
        const float pos = exact ? (static_cast<float>(i) + 0.5f) * scale : static_cast<float>(i) * scale;
        const long long s = std::min<long long>(static_cast<long long>(std::floor(pos)), in - 1);
        if (s != i / r) {
            return 0;
        }
    }
    return static_cast<int32_t>(r);
}
int32_t WholeFactorBwd(int64_t in, int64_t out, float scale, bool exact)
{
    if (out % in != 0) {
        return 0;
    }
    const int64_t r = out / in;
    for (int64_t y = 0; y <= in; ++y) {
        const float v = exact ? static_cast<float>(y) * scale - 0.5f : static_cast<float>(y) * scale;
        long long e = static_cast<long long>(std::ceil(v));
        e = std::min<long long>(std::max<long long>(e, 0), out);
        if (e != r * y) {
            return 0;
        }
    }
    return static_cast<int32_t>(r);
}

// image/upsample_nearest3d/op_host/op_api/aclnn_upsample_nearest_3d.cpp:117-128 (CheckParams), :156-204; the exact
// variant adds the scale / size consistency check of aclnn_upsample_nearest_exact3d.cpp:129-160.
aclnnStatus PlanForward(const char* api, bool exact, const aclTensor* self, const aclIntArray* outputSize, double scalesD,
                        double scalesH, double scalesW, aclTensor* out, uint64_t* workspaceSize,
                        aclOpExecutor** executor)
{
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
    if (self->dims.size() != 5 || out->dims.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self and out must be 5-D, got %zu-D and %zu-D", api,
                    self->dims.size(), out->dims.size());
    }
    if (outputSize->v.size() != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 3 values, got %zu", api, outputSize->v.size());
    }
    if (!FormatOk(self->format) || self->format != out->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: formats must be equal and NCDHW, NDHWC or ND, got %s and %s", api,
                    FormatName(self->format), FormatName(out->format));
    }
    const Geom5 gi = Geom5Of(self), go = Geom5Of(out);
    const int64_t od = outputSize->v[0], oh = outputSize->v[1], ow = outputSize->v[2];
    if (!(gi.d > 0 && gi.h > 0 && gi.w > 0 && od > 0 && oh > 0 && ow > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    if (!(gi.c > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: non-empty 5-D data tensor expected", api);
    }
    if (go.n != gi.n || go.c != gi.c || go.d != od || go.h != oh || go.w != ow) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out shape differs from (N, C, output_size)", api);
    }
    if (exact && scalesD > 0 && scalesH > 0 && scalesW > 0) {
        const double eps = 1e-5;
        auto consistent = [&](int64_t in, int64_t o, double s) {
            const int64_t dst = static_cast<int64_t>(static_cast<double>(in) * s);
            const int64_t mx = static_cast<int64_t>(static_cast<double>(in) * (s + eps));
            const int64_t mn = static_cast<int64_t>(static_cast<double>(in) * (s - eps));
            return o == dst || (o >= mn && o <= mx);
        };
        if (!consistent(gi.d, od, scalesD) || !consistent(gi.h, oh, scalesH) || !consistent(gi.w, ow, scalesW)) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales conflict with output_size", api);
        }
    }
    if (!Fits(gi) || !Fits(go)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: D, H, W and W*C must not exceed INT32_MAX", api);
    }
    if (IsEmpty(self)) {
        return EmptyOk(api, workspaceSize, executor);
    }
    if (!ViewStageable(self) || !ViewStageable(out)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: a 5-D view must have two neighbouring dimensions that are contiguous "
                                             "with respect to each other", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef x = StageInput(self, ws, ex);
    const BufRef y = StageOutput(out, ws);
    const bool cl = self->format == ACL_FORMAT_NDHWC;
    Nearest3dGeom g;
    g.rows = (cl ? gi.n : gi.n * gi.c) * od * oh;
    g.di = static_cast<int32_t>(gi.d);
    g.hi = static_cast<int32_t>(gi.h);
    g.wi = static_cast<int32_t>(gi.w);
    g.dout = static_cast<int32_t>(od);
    g.ho = static_cast<int32_t>(oh);
    g.wo = static_cast<int32_t>(ow);
    g.chan = cl ? static_cast<int32_t>(gi.c) : 1;
    g.sd = FwdScale(gi.d, od, static_cast<float>(scalesD));
    g.sh = FwdScale(gi.h, oh, static_cast<float>(scalesH));
    g.sw = FwdScale(gi.w, ow, static_cast<float>(scalesW));
    g.exact = exact ? 1 : 0;
    g.rd = WholeFactorFwd(gi.d, od, g.sd, exact);
    g.rh = WholeFactorFwd(gi.h, oh, g.sh, exact);
    g.rw = WholeFactorFwd(gi.w, ow, g.sw, exact);
    const Dt dt = ToDt(self->dtype);
    ex->steps.push_back([=](char* w, cudaStream_t s) { return Nearest3dFwd(dt, x.At(w), y.At(w), g, s); });
    FinishOutput(out, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

// image/upsample_nearest3d_grad/op_host/op_api/aclnn_upsample_nearest_3d_backward.cpp:84-99 (CheckParams), :101-180;
// the exact variant (aclnn_upsample_nearest_exact3d_backward.cpp:172-190) also rejects negative scales and up-scale
// factors above 50. The user scales are used only when all three are positive.
aclnnStatus PlanBackward(const char* api, bool exact, const aclTensor* gradOut, const aclIntArray* outputSize,
                         const aclIntArray* inputSize, double scalesD, double scalesH, double scalesW,
                         aclTensor* gradInput, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (gradOut == nullptr || outputSize == nullptr || inputSize == nullptr || gradInput == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (!DtypeSupported(gradOut->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(gradOut->dtype));
    }
    if (gradOut->dtype != gradInput->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradInput dtype %s differs from gradOut dtype %s", api,
                    DtypeName(gradInput->dtype), DtypeName(gradOut->dtype));
    }
    if (gradOut->dims.size() != 5 || gradInput->dims.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut and gradInput must be 5-D", api);
    }
    if (outputSize->v.size() != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 3 values, got %zu", api, outputSize->v.size());
    }
    if (inputSize->v.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input_size must have 5 values, got %zu", api, inputSize->v.size());
    }
    if (!FormatOk(gradOut->format) || gradOut->format != gradInput->format) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: formats must be equal and NCDHW, NDHWC or ND, got %s and %s", api,
                    FormatName(gradOut->format), FormatName(gradInput->format));
    }
    if (exact && (scalesD < 0 || scalesH < 0 || scalesW < 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales cannot be negative", api);
    }
    const Geom5 gg = Geom5Of(gradOut), gi = Geom5Of(gradInput);
    const int64_t od = outputSize->v[0], oh = outputSize->v[1], ow = outputSize->v[2];
    if (!(gi.d > 0 && gi.h > 0 && gi.w > 0 && od > 0 && oh > 0 && ow > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    for (int i = 0; i < 5; ++i) {
        if (gradInput->dims[i] != inputSize->v[i]) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: dim %d of gradInput should be %ld, got %ld", api, i,
                        (long)inputSize->v[i], (long)gradInput->dims[i]);
        }
    }
    if (gg.n != gi.n || gg.c != gi.c || gg.d != od || gg.h != oh || gg.w != ow) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut shape differs from (N, C, output_size)", api);
    }
    if (exact) {
        auto real = [](int64_t in, int64_t o, double s) { return s > 0 ? 1.0 / s : static_cast<double>(in) / static_cast<double>(o); };
        if (!(real(gi.d, od, scalesD) >= 0.02 && real(gi.h, oh, scalesH) >= 0.02 && real(gi.w, ow, scalesW) >= 0.02)) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: scales are too large", api);
        }
    }
    if (!Fits(gi) || !Fits(gg)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: D, H, W and W*C must not exceed INT32_MAX", api);
    }
    if (IsEmpty(gradOut)) {
        return EmptyOk(api, workspaceSize, executor);
    }
    if (!ViewStageable(gradOut) || !ViewStageable(gradInput)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: a 5-D view must have two neighbouring dimensions that are contiguous "
                                             "with respect to each other", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef g0 = StageInput(gradOut, ws, ex);
    const BufRef y = StageOutput(gradInput, ws);
    const bool cl = gradOut->format == ACL_FORMAT_NDHWC;
    const bool user = scalesD > 0 && scalesH > 0 && scalesW > 0;
    Nearest3dGeom g;
    g.rows = (cl ? gi.n : gi.n * gi.c) * gi.d * gi.h;
    g.di = static_cast<int32_t>(gi.d);
    g.hi = static_cast<int32_t>(gi.h);
    g.wi = static_cast<int32_t>(gi.w);
    g.dout = static_cast<int32_t>(od);
    g.ho = static_cast<int32_t>(oh);
    g.wo = static_cast<int32_t>(ow);
    g.chan = cl ? static_cast<int32_t>(gi.c) : 1;
    g.sd = BwdScale(od, gi.d, user ? static_cast<float>(scalesD) : 0.0f);
    g.sh = BwdScale(oh, gi.h, user ? static_cast<float>(scalesH) : 0.0f);
    g.sw = BwdScale(ow, gi.w, user ? static_cast<float>(scalesW) : 0.0f);
    g.exact = exact ? 1 : 0;
    g.rd = WholeFactorBwd(gi.d, od, g.sd, exact);
    g.rh = WholeFactorBwd(gi.h, oh, g.sh, exact);
    g.rw = WholeFactorBwd(gi.w, ow, g.sw, exact);
    const Dt dt = ToDt(gradOut->dtype);
    ex->steps.push_back([=](char* w, cudaStream_t s) { return Nearest3dBwd(dt, g0.At(w), y.At(w), g, s); });
    FinishOutput(gradInput, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

// ---- UpsampleTrilinear3d -------------------------------------------------------------------------------------
// image/resize_upsample_trilinear/op_host/resize_upsample_trilinear_tiling_arch35.cpp:145-154; `cast` is
// float(1.0 / scales) when the caller gave all three scales, else 0
// (image/resize_upsample_trilinear/op_host/op_api/aclnn_upsample_trilinear_3d.cpp:333-351).
float TrilinearScale(bool align, int64_t in, int64_t out, float cast)
{
    if (out == in) {
        return 1.0f;
    }
    if (align) {
        return out > 1 ? static_cast<float>(in - 1) / static_cast<float>(out - 1) : 0.0f;
    }
    return cast > 0.0f ? cast : static_cast<float>(in) / static_cast<float>(out);
}

Trilinear3dGeom MakeTrilinearGeom(const Geom5& gi, int64_t od, int64_t oh, int64_t ow, bool cl, bool align,
                                  double scalesD, double scalesH, double scalesW)
{
    const bool user = scalesD > 0 && scalesH > 0 && scalesW > 0;
    Trilinear3dGeom g;
    g.rows = 0;
    g.di = static_cast<int32_t>(gi.d);
    g.hi = static_cast<int32_t>(gi.h);
    g.wi = static_cast<int32_t>(gi.w);
    g.dout = static_cast<int32_t>(od);
    g.ho = static_cast<int32_t>(oh);
    g.wo = static_cast<int32_t>(ow);
    g.chan = cl ? static_cast<int32_t>(gi.c) : 1;
    g.sd = TrilinearScale(align, gi.d, od, user ? static_cast<float>(1.0 / scalesD) : 0.0f);
    g.sh = TrilinearScale(align, gi.h, oh, user ? static_cast<float>(1.0 / scalesH) : 0.0f);
    g.sw = TrilinearScale(align, gi.w, ow, user ? static_cast<float>(1.0 / scalesW) : 0.0f);
    g.align = align ? 1 : 0;
    g.loop = 0;
    return g;
}

// image/resize_upsample_trilinear/op_host/op_api/aclnn_upsample_trilinear_3d.cpp:220-238 (CheckParams), :382-441.
aclnnStatus PlanTrilinearFwd(const char* api, const aclTensor* self, const aclIntArray* outputSize, bool alignCorners,
                             double scalesD, double scalesH, double scalesW, aclTensor* out, uint64_t* workspaceSize,
                             aclOpExecutor** executor)
{
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
    if (self->dims.size() != 5 || out->dims.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self and out must be 5-D, got %zu-D and %zu-D", api,
                    self->dims.size(), out->dims.size());
    }
    if (outputSize->v.size() != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 3 values, got %zu", api, outputSize->v.size());
    }
    if (!FormatOk(self->format)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input storage format must be NCDHW or NDHWC, got %s", api,
                    FormatName(self->format));
    }
    const bool cl = self->format == ACL_FORMAT_NDHWC;
    if ((out->format == ACL_FORMAT_NDHWC) != cl) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: self and out must have the same format, got %s and %s", api,
                    FormatName(self->format), FormatName(out->format));
    }
    const Geom5 gi = Geom5Of(self), go = Geom5Of(out);
    const int64_t od = outputSize->v[0], oh = outputSize->v[1], ow = outputSize->v[2];
    if (!(gi.d > 0 && gi.h > 0 && gi.w > 0 && od > 0 && oh > 0 && ow > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    if (!(gi.c > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: non-empty 5-D data tensor expected", api);
    }
    if (go.n != gi.n || go.c != gi.c || go.d != od || go.h != oh || go.w != ow) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out shape differs from (N, C, output_size)", api);
    }
    if (!Fits(gi) || !Fits(go)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: D, H, W and W*C must not exceed INT32_MAX", api);
    }
    if (IsEmpty(self)) {
        return EmptyOk(api, workspaceSize, executor);
    }
    if (!ViewStageable(self) || !ViewStageable(out)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: a 5-D view must have two neighbouring dimensions that are contiguous "
                                             "with respect to each other", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef x = StageInput(self, ws, ex);
    const BufRef y = StageOutput(out, ws);
    Trilinear3dGeom g = MakeTrilinearGeom(gi, od, oh, ow, cl, alignCorners, scalesD, scalesH, scalesW);
    g.rows = (cl ? gi.n : gi.n * gi.c) * od * oh;
    // The reference picks its loop by which scales are exactly 1.0f
    // (image/resize_upsample_trilinear/op_kernel/arch35/resize_upsample_trilinear_simt_base.h:37-60). Its one-axis
    // loops address the idle axes by the output coordinate, which only stands for equal extents; a unit scale on an
    // axis whose extents differ (a user scale of 1 against another output_size) runs the full loop here.
    const bool dEq = g.sd == 1.0f && gi.d == od, hEq = g.sh == 1.0f && gi.h == oh, wEq = g.sw == 1.0f && gi.w == ow;
    g.loop = (dEq && hEq && wEq) ? 4 : (hEq && wEq) ? 1 : (dEq && wEq) ? 2 : (dEq && hEq) ? 3 : 0;
    const Dt dt = ToDt(self->dtype);
    const uint64_t stageBytes = Trilinear3dFwdWorkspace(g, cl ? gi.n : gi.n * gi.c);
    const uint64_t stageOff = stageBytes > 0 ? ws.Alloc(stageBytes) : 0;
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        return Trilinear3dFwd(dt, x.At(w), y.At(w), stageBytes > 0 ? reinterpret_cast<float*>(w + stageOff) : nullptr, g, s);
    });
    FinishOutput(out, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

// image/upsample_trilinear3d_backward/op_host/op_api/aclnn_upsample_trilinear_3d_backward.cpp:130-148 (CheckParams),
// :177-240; scales: image/upsample_trilinear3d_backward/op_host/upsample_trilinear3d_backward_tiling_func.cpp:218-240.
aclnnStatus PlanTrilinearBwd(const char* api, const aclTensor* gradOut, const aclIntArray* outputSize,
                             const aclIntArray* inputSize, bool alignCorners, double scalesD, double scalesH,
                             double scalesW, aclTensor* gradInput, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (gradOut == nullptr || outputSize == nullptr || inputSize == nullptr || gradInput == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (!DtypeSupported(gradOut->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(gradOut->dtype));
    }
    if (gradOut->dtype != gradInput->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradInput dtype %s differs from gradOut dtype %s", api,
                    DtypeName(gradInput->dtype), DtypeName(gradOut->dtype));
    }
    if (gradOut->dims.size() != 5 || gradInput->dims.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut and gradInput must be 5-D", api);
    }
    if (outputSize->v.size() != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: output_size must have 3 values, got %zu", api, outputSize->v.size());
    }
    if (inputSize->v.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input_size must have 5 values, got %zu", api, inputSize->v.size());
    }
    if (!FormatOk(gradOut->format)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input storage format must be NCDHW or NDHWC, got %s", api,
                    FormatName(gradOut->format));
    }
    const bool cl = gradOut->format == ACL_FORMAT_NDHWC;
    if ((gradInput->format == ACL_FORMAT_NDHWC) != cl) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut and gradInput must have the same format, got %s and %s", api,
                    FormatName(gradOut->format), FormatName(gradInput->format));
    }
    // input_size is (N, C, D, H, W) whatever the format
    const int64_t od = outputSize->v[0], oh = outputSize->v[1], ow = outputSize->v[2];
    Geom5 gi;
    gi.n = inputSize->v[0];
    gi.c = inputSize->v[1];
    gi.d = inputSize->v[2];
    gi.h = inputSize->v[3];
    gi.w = inputSize->v[4];
    if (!(gi.d > 0 && gi.h > 0 && gi.w > 0 && od > 0 && oh > 0 && ow > 0)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and output sizes should be greater than 0", api);
    }
    const Geom5 gg = Geom5Of(gradOut), gv = Geom5Of(gradInput);
    if (gg.n != gi.n || gg.c != gi.c || gg.d != od || gg.h != oh || gg.w != ow) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradOut shape differs from (N, C, output_size)", api);
    }
    if (gv.n != gi.n || gv.c != gi.c || gv.d != gi.d || gv.h != gi.h || gv.w != gi.w) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gradInput shape differs from input_size", api);
    }
    if (!Fits(gi) || !Fits(gg)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: D, H, W and W*C must not exceed INT32_MAX", api);
    }
    if (IsEmpty(gradOut)) {
        return EmptyOk(api, workspaceSize, executor);
    }
    if (!ViewStageable(gradOut) || !ViewStageable(gradInput)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: a 5-D view must have two neighbouring dimensions that are contiguous "
                                             "with respect to each other", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef g0 = StageInput(gradOut, ws, ex);
    const BufRef y = StageOutput(gradInput, ws);
    Trilinear3dGeom g = MakeTrilinearGeom(gi, od, oh, ow, cl, alignCorners, scalesD, scalesH, scalesW);
    g.rows = (cl ? gi.n : gi.n * gi.c) * gi.d * gi.h;
    const int32_t ins[3] = {g.di, g.hi, g.wi}, outs[3] = {g.dout, g.ho, g.wo};
    const float sc[3] = {g.sd, g.sh, g.sw};
    int32_t taps[3];
    uint64_t offStart[3], offCount[3], offW[3];
    for (int a = 0; a < 3; ++a) {
        taps[a] = host::TrilinearBwdTaps(ins[a], outs[a], sc[a], alignCorners);
        offStart[a] = ws.Alloc(sizeof(int32_t) * static_cast<uint64_t>(ins[a]));
        offCount[a] = ws.Alloc(sizeof(int32_t) * static_cast<uint64_t>(ins[a]));
        offW[a] = ws.Alloc(sizeof(float) * static_cast<uint64_t>(ins[a]) * static_cast<uint64_t>(taps[a]));
    }
    const Dt dt = ToDt(gradOut->dtype);
    const uint64_t stageOff = ws.Alloc(Trilinear3dBwdWorkspace(g, cl ? gi.n : gi.n * gi.c));
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        TrilinearBwdTables t;
        for (int a = 0; a < 3; ++a) {
            t.start[a] = reinterpret_cast<int32_t*>(w + offStart[a]);
            t.count[a] = reinterpret_cast<int32_t*>(w + offCount[a]);
            t.w[a] = reinterpret_cast<float*>(w + offW[a]);
            t.taps[a] = taps[a];
        }
        const cudaError_t e = BuildTrilinearBwdTables(t, g, s);
        if (e != cudaSuccess) {
            return e;
        }
        return Trilinear3dBwd(dt, g0.At(w), y.At(w), reinterpret_cast<float*>(w + stageOff), g, t, s);
    });
    FinishOutput(gradInput, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

} // namespace

extern "C" {

aclnnStatus aclnnUpsampleNearest3dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize, double scalesD,
                                                   double scalesH, double scalesW, aclTensor* out,
                                                   uint64_t* workspaceSize, aclOpExecutor** executor)
{
    return PlanForward("aclnnUpsampleNearest3d", false, self, outputSize, scalesD, scalesH, scalesW, out, workspaceSize,
                       executor);
}
aclnnStatus aclnnUpsampleNearest3d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearest3d", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnUpsampleNearestExact3dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                        double scalesD, double scalesH, double scalesW, aclTensor* out,
                                                        uint64_t* workspaceSize, aclOpExecutor** executor)
{
    return PlanForward("aclnnUpsampleNearestExact3d", true, self, outputSize, scalesD, scalesH, scalesW, out,
                       workspaceSize, executor);
}
aclnnStatus aclnnUpsampleNearestExact3d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                        aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearestExact3d", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnUpsampleNearest3dBackwardGetWorkspaceSize(const aclTensor* gradOut, const aclIntArray* outputSize,
                                                           const aclIntArray* inputSize, double scalesD, double scalesH,
                                                           double scalesW, aclTensor* gradInput,
                                                           uint64_t* workspaceSize, aclOpExecutor** executor)
{
    return PlanBackward("aclnnUpsampleNearest3dBackward", false, gradOut, outputSize, inputSize, scalesD, scalesH,
                        scalesW, gradInput, workspaceSize, executor);
}
aclnnStatus aclnnUpsampleNearest3dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                           aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearest3dBackward", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnUpsampleNearestExact3dBackwardGetWorkspaceSize(const aclTensor* gradOut,
                                                                const aclIntArray* outputSize,
                                                                const aclIntArray* inputSize, double scalesD,
                                                                double scalesH, double scalesW, aclTensor* gradInput,
                                                                uint64_t* workspaceSize, aclOpExecutor** executor)
{
    return PlanBackward("aclnnUpsampleNearestExact3dBackward", true, gradOut, outputSize, inputSize, scalesD, scalesH,
                        scalesW, gradInput, workspaceSize, executor);
}
aclnnStatus aclnnUpsampleNearestExact3dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleNearestExact3dBackward", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnUpsampleTrilinear3dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                     bool alignCorners, double scalesD, double scalesH, double scalesW,
                                                     aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    return PlanTrilinearFwd("aclnnUpsampleTrilinear3d", self, outputSize, alignCorners, scalesD, scalesH, scalesW, out,
                            workspaceSize, executor);
}
aclnnStatus aclnnUpsampleTrilinear3d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                     aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleTrilinear3d", workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnUpsampleTrilinear3dBackwardGetWorkspaceSize(const aclTensor* gradOut, const aclIntArray* outputSize,
                                                             const aclIntArray* inputSize, bool alignCorners,
                                                             double scalesD, double scalesH, double scalesW,
                                                             aclTensor* gradInput, uint64_t* workspaceSize,
                                                             aclOpExecutor** executor)
{
    return PlanTrilinearBwd("aclnnUpsampleTrilinear3dBackward", gradOut, outputSize, inputSize, alignCorners, scalesD,
                            scalesH, scalesW, gradInput, workspaceSize, executor);
}
aclnnStatus aclnnUpsampleTrilinear3dBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                             aclrtStream stream)
{
    return RunExecutor("aclnnUpsampleTrilinear3dBackward", workspace, workspaceSize, executor, stream);
}

} // extern "C"
