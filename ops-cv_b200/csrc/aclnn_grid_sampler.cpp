// First- and second-phase entry points of GridSampler2D and GridSampler2DBackward.
#include "host_common.h"

using namespace opscv;

namespace {

bool FitsInt32Dims(const aclTensor* t)
{
    for (int64_t d : t->dims) {
        if (d > INT32_MAX) {
            return false;
        }
    }
    return true;
}

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

bool SameShape(const aclTensor* a, const aclTensor* b) { return a->dims == b->dims; }

GridShape MakeGridShape(const aclTensor* input, const aclTensor* grid, int64_t interp, int64_t pad, bool align)
{
    GridShape g;
    g.n = input->dims[0];
    g.c = input->dims[1];
    g.hin = static_cast<int32_t>(input->dims[2]);
    g.win = static_cast<int32_t>(input->dims[3]);
    g.hout = static_cast<int32_t>(grid->dims[1]);
    g.wout = static_cast<int32_t>(grid->dims[2]);
    g.interp = static_cast<int32_t>(interp);
    g.pad = static_cast<int32_t>(pad);
    g.align = align ? 1 : 0;
    return g;
}

} // namespace

extern "C" {

// image/grid_sample/op_api/aclnn_grid_sampler2d.cpp:159-175 (CheckParams): null, dtype, attr, shape
aclnnStatus aclnnGridSampler2DGetWorkspaceSize(const aclTensor* input, const aclTensor* grid,
                                               int64_t interpolationMode, int64_t paddingMode, bool alignCorners,
                                               aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnGridSampler2D";
    if (input == nullptr || grid == nullptr || out == nullptr || workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (grid->dtype != input->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: grid dtype %s differs from input dtype %s", api,
                    DtypeName(grid->dtype), DtypeName(input->dtype));
    }
    if (out->dtype != input->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: out dtype %s differs from input dtype %s", api,
                    DtypeName(out->dtype), DtypeName(input->dtype));
    }
    if (!DtypeSupported(input->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(input->dtype));
    }
    if (interpolationMode < 0 || interpolationMode > 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID,
                    "%s: interpolationMode %ld should be in {0 (bilinear), 1 (nearest), 2 (bicubic)}", api,
                    (long)interpolationMode);
    }
    if (paddingMode < 0 || paddingMode > 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: paddingMode %ld should be in {0 (zeros), 1 (border), 2 (reflection)}",
                    api, (long)paddingMode);
    }
    if (input->dims.size() != 4 || grid->dims.size() != 4 || out->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and out must be 4-D", api);
    }
    if (input->dims[0] != grid->dims[0] || input->dims[0] != out->dims[0]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and out must have the same batch size", api);
    }
    if (input->dims[1] != out->dims[1]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and out must have the same channel size", api);
    }
    if (grid->dims[1] != out->dims[2] || grid->dims[2] != out->dims[3]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: grid and out must have the same H and W", api);
    }
    if (input->dims[2] == 0 || input->dims[3] == 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input must have non-empty spatial dimensions", api);
    }
    if (grid->dims[3] != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: grid must have size 2 in its last dimension", api);
    }
    if (IsEmpty(input) || IsEmpty(grid) || IsEmpty(out)) {
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (!FitsInt32Dims(input) || !FitsInt32Dims(grid) ||
        input->dims[2] * input->dims[3] >= INT32_MAX) { // H*W < INT32_MAX (aclnnGridSampler2D.md, constraints)
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: extents exceed the supported range", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const BufRef x = StageInput(input, ws, ex);
    const BufRef gr = StageInput(grid, ws, ex);
    const BufRef y = StageOutput(out, ws);
    const GridShape g = MakeGridShape(input, grid, interpolationMode, paddingMode, alignCorners);
    const Dt dt = ToDt(input->dtype);
    const GridFwdPlan plan = PlanGridSampler2DFwd(dt, g);
    const uint64_t scratch = plan.recBytes > 0 ? ws.Alloc(plan.recBytes) : 0;
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        return GridSampler2DFwd(dt, x.At(w), gr.At(w), y.At(w), g, plan,
                                plan.recBytes > 0 ? static_cast<void*>(w + scratch) : nullptr, s);
    });
    FinishOutput(out, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnGridSampler2D(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    return RunExecutor("aclnnGridSampler2D", workspace, workspaceSize, executor, stream);
}

// image/grid_sampler2_d_grad/op_host/op_api/aclnn_grid_sampler2d_backward.cpp:214-250 and CheckParams :195-212
aclnnStatus aclnnGridSampler2DBackwardGetWorkspaceSize(const aclTensor* gradOutput, const aclTensor* input,
                                                       const aclTensor* grid, int64_t interpolationMode,
                                                       int64_t paddingMode, bool alignCorners,
                                                       const aclBoolArray* outputMask, aclTensor* inputGrad,
                                                       aclTensor* gridGrad, uint64_t* workspaceSize,
                                                       aclOpExecutor** executor)
{
    static const char* api = "aclnnGridSampler2DBackward";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (outputMask == nullptr) { // :231-235: successful no-op
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (gradOutput == nullptr || input == nullptr || grid == nullptr || inputGrad == nullptr || gridGrad == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null tensor argument", api);
    }
    if (gradOutput->dtype != input->dtype || grid->dtype != input->dtype || inputGrad->dtype != input->dtype ||
        gridGrad->dtype != input->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: all tensors must have the dtype of input (%s)", api,
                    DtypeName(input->dtype));
    }
    if (!DtypeSupported(input->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(input->dtype));
    }
    if (interpolationMode < 0 || interpolationMode > 2 || paddingMode < 0 || paddingMode > 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: interpolationMode %ld / paddingMode %ld out of range [0, 2]", api,
                    (long)interpolationMode, (long)paddingMode);
    }
    if (input->dims.size() != 4 || grid->dims.size() != 4 || gradOutput->dims.size() != 4) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and gradOutput must be 4-D", api);
    }
    if (input->dims[0] != grid->dims[0] || input->dims[0] != gradOutput->dims[0]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and gradOutput must have the same batch size", api);
    }
    if (input->dims[1] != gradOutput->dims[1]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and gradOutput must have the same channel size", api);
    }
    if (input->dims[2] == 0 || input->dims[3] == 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input must have non-empty spatial dimensions", api);
    }
    if (grid->dims[1] != gradOutput->dims[2] || grid->dims[2] != gradOutput->dims[3]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: grid and gradOutput must have the same H and W", api);
    }
    if (grid->dims[3] != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: grid must have size 2 in its last dimension", api);
    }
    if (!SameShape(inputGrad, input)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: inputGrad must have the shape of input", api);
    }
    if (!SameShape(gridGrad, grid)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: gridGrad must have the shape of grid", api);
    }
    if (outputMask->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: outputMask must have 2 values, got %zu", api, outputMask->v.size());
    }
    const bool wantInput = outputMask->v[0] != 0, wantGrid = outputMask->v[1] != 0;
    if (!wantInput && !wantGrid) { // :242-248
        return EmptySuccess(api, workspaceSize, executor);
    }
    if (!FitsInt32Dims(input) || !FitsInt32Dims(grid) || input->dims[2] * input->dims[3] >= INT32_MAX ||
        grid->dims[1] * grid->dims[2] >= INT32_MAX / 16) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: extents exceed the supported range", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    const GridShape g = MakeGridShape(input, grid, interpolationMode, paddingMode, alignCorners);
    const Dt dt = ToDt(input->dtype);
    if (IsEmpty(input) || IsEmpty(grid) || IsEmpty(gradOutput)) {
        // Nothing to sample from or no samples: the requested gradients are all zero.
        WsPlan ws;
        const BufRef gi = StageOutput(inputGrad, ws);
        const BufRef gg = StageOutput(gridGrad, ws);
        const uint64_t giBytes = static_cast<uint64_t>(Numel(inputGrad)) * ElemSize(input->dtype);
        const uint64_t ggBytes = static_cast<uint64_t>(Numel(gridGrad)) * ElemSize(input->dtype);
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            cudaError_t e = cudaSuccess;
            if (wantInput && giBytes > 0) {
                e = cudaMemsetAsync(gi.At(w), 0, giBytes, s);
            }
            if (e == cudaSuccess && wantGrid && ggBytes > 0) {
                e = cudaMemsetAsync(gg.At(w), 0, ggBytes, s);
            }
            return e;
        });
        if (wantInput) {
            FinishOutput(inputGrad, gi, ex);
        }
        if (wantGrid) {
            FinishOutput(gridGrad, gg, ex);
        }
        ex->workspaceSize = ws.Size();
        *workspaceSize = ws.Size();
        *executor = ex;
        return ACLNN_SUCCESS;
    }
    WsPlan ws;
    const BufRef go = StageInput(gradOutput, ws, ex);
    const BufRef x = StageInput(input, ws, ex);
    const BufRef gr = StageInput(grid, ws, ex);
    const BufRef gi = StageOutput(inputGrad, ws);
    const BufRef gg = StageOutput(gridGrad, ws);
    // deterministic flag: aclrtCtxGetSysParamOpt(ACL_OPT_DETERMINISTIC) at plan time (:180-186)
    const GridGradPlan plan = PlanGridSampler2DBwd(dt, g, GetDeterministic() != 0, wantInput, wantGrid);
    const uint64_t scratch = plan.total > 0 ? ws.Alloc(plan.total) : 0;
    ex->steps.push_back([=](char* w, cudaStream_t s) {
        return GridSampler2DBwd(dt, go.At(w), x.At(w), gr.At(w), gi.At(w), gg.At(w), g, plan,
                                plan.total > 0 ? static_cast<void*>(w + scratch) : nullptr, s);
    });
    if (wantInput) {
        FinishOutput(inputGrad, gi, ex);
    }
    if (wantGrid) {
        FinishOutput(gridGrad, gg, ex);
    }
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnGridSampler2DBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                       aclrtStream stream)
{
    return RunExecutor("aclnnGridSampler2DBackward", workspace, workspaceSize, executor, stream);
}

} // extern "C"
