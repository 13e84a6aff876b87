// First- and second-phase entry points of GridSampler3D and GridSampler3DBackward. NDHWC tensors are described as
// NCDHW views over the same memory and go through the staging copies (the reference transposes them as well).
#include "host_common.h"

using namespace opscv;

namespace {

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

// The tensor as an NCDHW view: an NDHWC tensor [N, D, H, W, C] is the same memory with permuted extents and strides.
aclTensor AsNcdhw(const aclTensor* t)
{
    aclTensor v = *t;
    if (t->format == ACL_FORMAT_NDHWC) {
        v.dims = {t->dims[0], t->dims[4], t->dims[1], t->dims[2], t->dims[3]};
        v.strides = {t->strides[0], t->strides[4], t->strides[1], t->strides[2], t->strides[3]};
        v.format = ACL_FORMAT_NCDHW;
    }
    return v;
}

bool Fits(const aclTensor& t)
{
    for (int64_t d : t.dims) {
        if (d > INT32_MAX) {
            return false;
        }
    }
    return true;
}

Grid3dShape MakeShape(const aclTensor& input, const aclTensor* grid, int64_t interp, int64_t pad, bool align)
{
    Grid3dShape g;
    g.n = input.dims[0];
    g.c = input.dims[1];
    g.di = static_cast<int32_t>(input.dims[2]);
    g.hi = static_cast<int32_t>(input.dims[3]);
    g.wi = static_cast<int32_t>(input.dims[4]);
    g.dout = static_cast<int32_t>(grid->dims[1]);
    g.ho = static_cast<int32_t>(grid->dims[2]);
    g.wo = static_cast<int32_t>(grid->dims[3]);
    g.interp = static_cast<int32_t>(interp);
    g.pad = static_cast<int32_t>(pad);
    g.align = align ? 1 : 0;
    return g;
}

// Shared shape rules (aclnn_grid_sampler3d.cpp:118-171): 5-D tensors, one batch size, grid (N, Do, Ho, Wo, 3), out
// (N, C, Do, Ho, Wo) in the input's layout.
aclnnStatus CheckShapes(const char* api, const aclTensor& in, const aclTensor* grid, const aclTensor& out)
{
    if (in.dims.size() != 5 || grid->dims.size() != 5 || out.dims.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and out must be 5-D", api);
    }
    if (in.dims[0] != grid->dims[0] || in.dims[0] != out.dims[0]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and out must have the same batch size", api);
    }
    if (in.dims[1] != out.dims[1]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input and out must have the same channel count", api);
    }
    if (grid->dims[1] != out.dims[2] || grid->dims[2] != out.dims[3] || grid->dims[3] != out.dims[4]) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: grid D/H/W differ from those of out", api);
    }
    if (grid->dims[4] != 3) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the last dimension of grid must be 3, got %ld", api,
                    (long)grid->dims[4]);
    }
    if (in.dims[2] <= 0 || in.dims[3] <= 0 || in.dims[4] <= 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: the spatial extents of input must be greater than 0", api);
    }
    return ACLNN_SUCCESS;
}

} // namespace

extern "C" {

// image/grid_sample/op_api/aclnn_grid_sampler3d.cpp:173-192 (CheckParams: null, dtype, format, attributes, shape).
// interpolationMode 0 (bilinear) is the reference's AI-core kernel; 1 (nearest) runs on its CPU fallback there and
// is computed here with the rounding of the backward kernel.
aclnnStatus aclnnGridSampler3DGetWorkspaceSize(const aclTensor* input, const aclTensor* grid, int64_t interpolationMode,
                                               int64_t paddingMode, bool alignCorners, aclTensor* out,
                                               uint64_t* workspaceSize, aclOpExecutor** executor)
{
    static const char* api = "aclnnGridSampler3D";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (input == nullptr || grid == nullptr || out == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (grid->dtype != input->dtype || out->dtype != input->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and out must have one dtype", api);
    }
    if (!DtypeSupported(input->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(input->dtype));
    }
    if (!FormatOk(input->format) || !FormatOk(out->format)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: formats must be NCDHW, NDHWC or ND, got %s and %s", api,
                    FormatName(input->format), FormatName(out->format));
    }
    if (paddingMode < 0 || paddingMode > 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: paddingMode %ld should be in [0, 2]", api, (long)paddingMode);
    }
    if (interpolationMode < 0 || interpolationMode > 1) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: interpolationMode %ld should be in [0, 1]", api,
                    (long)interpolationMode);
    }
    if (input->dims.size() != 5 || out->dims.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: input, grid and out must be 5-D", api);
    }
    aclTensor in5 = AsNcdhw(input), out5 = AsNcdhw(out);
    const aclnnStatus st = CheckShapes(api, in5, grid, out5);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (!Fits(in5) || !Fits(out5)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: extents must not exceed INT32_MAX", api);
    }
    if (IsEmpty(input) || IsEmpty(grid) || IsEmpty(out)) {
        return EmptyOk(api, workspaceSize, executor);
    }
    if (!ViewStageable(&in5) || !ViewStageable(grid) || !ViewStageable(&out5) || !ViewStageable(input) ||
        !ViewStageable(out)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: view not supported (more than four strided dimensions)", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    // channels-last tensors on both sides keep their layout (the kernels read a tap as a contiguous run of channels);
    // a mix of layouts goes through NCDHW views and the staging copies
    const bool cl = input->format == ACL_FORMAT_NDHWC && out->format == ACL_FORMAT_NDHWC;
    const aclTensor* xin = cl ? input : &in5;
    const aclTensor* yout = cl ? out : &out5;
    const BufRef x = StageInput(xin, ws, ex);
    const BufRef gr = StageInput(grid, ws, ex);
    const BufRef y = StageOutput(yout, ws);
    Grid3dShape g = MakeShape(in5, grid, interpolationMode, paddingMode, alignCorners);
    g.cl = cl ? 1 : 0;
    const Dt dt = ToDt(input->dtype);
    // NCDHW tensors with enough channels: a tap of a point costs a 32-byte sector per channel in that layout, so the
    // input is turned channels-last in the workspace (tiled transpose), sampled by the channels-last kernel, and the
    // result turned back: two extra passes over tensors that the gather reads eight times over.
    const int64_t inVol = static_cast<int64_t>(g.di) * g.hi * g.wi, outVol = static_cast<int64_t>(g.dout) * g.ho * g.wo;
    if (!cl && g.c >= 16 && g.c % 4 == 0) {
        const int es = ElemSize(input->dtype);
        const uint64_t xtOff = ws.Alloc(static_cast<uint64_t>(g.n) * g.c * inVol * es);
        const uint64_t ytOff = ws.Alloc(static_cast<uint64_t>(g.n) * g.c * outVol * es);
        Grid3dShape gc = g;
        gc.cl = 1;
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            cudaError_t e = TransposeBatched(es, x.At(w), w + xtOff, g.n, g.c, inVol, s);
            if (e != cudaSuccess) {
                return e;
            }
            e = GridSampler3dFwd(dt, w + xtOff, gr.At(w), w + ytOff, gc, s);
            if (e != cudaSuccess) {
                return e;
            }
            return TransposeBatched(es, w + ytOff, y.At(w), g.n, outVol, g.c, s);
        });
    } else {
        ex->steps.push_back([=](char* w, cudaStream_t s) { return GridSampler3dFwd(dt, x.At(w), gr.At(w), y.At(w), g, s); });
    }
    FinishOutput(yout, y, ex);
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnGridSampler3D(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    return RunExecutor("aclnnGridSampler3D", workspace, workspaceSize, executor, stream);
}

// image/grid_sampler3_d_grad/op_host/op_api/aclnn_grid_sampler3d_backward.cpp:146-160 (CheckParams), :183-310.
// grad_input is accumulated with atomics in both modes: the reference's ordered kernel
// (grid_sampler3_d_grad_simt_det.h) is not restated, so ACL_OPT_DETERMINISTIC does not change the 3-D backward.
aclnnStatus aclnnGridSampler3DBackwardGetWorkspaceSize(const aclTensor* gradOutput, const aclTensor* input,
                                                       const aclTensor* grid, int64_t interpolationMode,
                                                       int64_t paddingMode, bool alignCorners,
                                                       const aclBoolArray* outputMask, aclTensor* inputGrad,
                                                       aclTensor* gridGrad, uint64_t* workspaceSize,
                                                       aclOpExecutor** executor)
{
    static const char* api = "aclnnGridSampler3DBackward";
    if (workspaceSize == nullptr || executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspaceSize or executor is null", api);
    }
    if (outputMask == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: outputMask is null", api);
    }
    if (gradOutput == nullptr || input == nullptr || grid == nullptr || inputGrad == nullptr || gridGrad == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: null argument", api);
    }
    if (gradOutput->dtype != input->dtype || grid->dtype != input->dtype || inputGrad->dtype != input->dtype ||
        gridGrad->dtype != input->dtype) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: all tensors must have one dtype", api);
    }
    if (!DtypeSupported(input->dtype)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: dtype %s not supported (FLOAT, FLOAT16, BF16)", api,
                    DtypeName(input->dtype));
    }
    if (paddingMode < 0 || paddingMode > 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: paddingMode %ld should be in [0, 2]", api, (long)paddingMode);
    }
    if (interpolationMode < 0 || interpolationMode > 1) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: interpolationMode %ld should be in [0, 1]", api,
                    (long)interpolationMode);
    }
    if (!FormatOk(input->format) || !FormatOk(gradOutput->format) || !FormatOk(inputGrad->format)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: formats must be NCDHW, NDHWC or ND", api);
    }
    if (input->dims.size() != 5 || gradOutput->dims.size() != 5 || inputGrad->dims.size() != 5) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: tensors must be 5-D", api);
    }
    aclTensor in5 = AsNcdhw(input), go5 = AsNcdhw(gradOutput), gi5 = AsNcdhw(inputGrad);
    const aclnnStatus st = CheckShapes(api, in5, grid, go5);
    if (st != ACLNN_SUCCESS) {
        return st;
    }
    if (inputGrad->dims != input->dims || gridGrad->dims != grid->dims) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: inputGrad / gridGrad shapes differ from input / grid", api);
    }
    if (outputMask->v.size() != 2) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: outputMask must have 2 values, got %zu", api, outputMask->v.size());
    }
    if (!Fits(in5) || !Fits(go5)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: extents must not exceed INT32_MAX", api);
    }
    const bool wantInput = outputMask->v[0] != 0, wantGrid = outputMask->v[1] != 0;
    if (IsEmpty(gradOutput) || IsEmpty(input) || IsEmpty(grid) || (!wantInput && !wantGrid)) {
        return EmptyOk(api, workspaceSize, executor);
    }
    if (!ViewStageable(&in5) || !ViewStageable(grid) || !ViewStageable(&go5) || !ViewStageable(&gi5) ||
        !ViewStageable(gridGrad) || !ViewStageable(input) || !ViewStageable(gradOutput) || !ViewStageable(inputGrad)) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: view not supported (more than four strided dimensions)", api);
    }
    aclOpExecutor* ex = NewExecutor(api);
    if (ex == nullptr) {
        return Fail(ACLNN_ERR_INNER_CREATE_EXECUTOR, "%s: cannot create executor", api);
    }
    WsPlan ws;
    const bool cl = input->format == ACL_FORMAT_NDHWC && gradOutput->format == ACL_FORMAT_NDHWC &&
                    inputGrad->format == ACL_FORMAT_NDHWC;
    const aclTensor* goT = cl ? gradOutput : &go5;
    const aclTensor* xT = cl ? input : &in5;
    const aclTensor* giT = cl ? inputGrad : &gi5;
    const BufRef go = StageInput(goT, ws, ex);
    const BufRef x = StageInput(xT, ws, ex);
    const BufRef gr = StageInput(grid, ws, ex);
    const BufRef gi = StageOutput(giT, ws);
    const BufRef gg = StageOutput(gridGrad, ws);
    Grid3dShape g = MakeShape(in5, grid, interpolationMode, paddingMode, alignCorners);
    g.cl = cl ? 1 : 0;
    const Dt dt = ToDt(input->dtype);
    const bool needAcc = wantInput && dt != Dt::F32;
    const int64_t inVol = static_cast<int64_t>(g.di) * g.hi * g.wi, outVol = static_cast<int64_t>(g.dout) * g.ho * g.wo;
    if (!cl && g.c >= 16 && g.c % 4 == 0) {
        // as in the forward: channels-last copies of grad_output and input, the channels-last kernel (16-byte vector
        // reductions into an fp32 channels-last accumulator), and grad_input turned back to NCDHW
        const int es = ElemSize(input->dtype);
        const uint64_t gotOff = ws.Alloc(static_cast<uint64_t>(g.n) * g.c * outVol * es);
        const uint64_t xtOff = ws.Alloc(static_cast<uint64_t>(g.n) * g.c * inVol * es);
        const uint64_t accOff = wantInput ? ws.Alloc(static_cast<uint64_t>(g.n) * g.c * inVol * 4) : 0;
        const uint64_t gitOff = needAcc ? ws.Alloc(static_cast<uint64_t>(g.n) * g.c * inVol * es) : 0;
        Grid3dShape gc = g;
        gc.cl = 1;
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            cudaError_t e = TransposeBatched(es, go.At(w), w + gotOff, g.n, g.c, outVol, s);
            if (e == cudaSuccess) {
                e = TransposeBatched(es, x.At(w), w + xtOff, g.n, g.c, inVol, s);
            }
            if (e != cudaSuccess) {
                return e;
            }
            float* acc = reinterpret_cast<float*>(w + accOff);
            // 16-bit tensors: the kernel's cast pass writes a channels-last grad_input of the storage type
            void* giT = needAcc ? static_cast<void*>(w + gitOff) : static_cast<void*>(acc);
            e = GridSampler3dBwd(dt, w + gotOff, w + xtOff, gr.At(w), giT, gg.At(w), acc, gc, wantInput, wantGrid, s);
            if (e != cudaSuccess || !wantInput) {
                return e;
            }
            return TransposeBatched(es, giT, gi.At(w), g.n, inVol, g.c, s);
        });
    } else {
        const uint64_t accOff = needAcc ? ws.Alloc(static_cast<uint64_t>(Numel(input)) * 4) : 0;
        ex->steps.push_back([=](char* w, cudaStream_t s) {
            float* acc = needAcc ? reinterpret_cast<float*>(w + accOff) : static_cast<float*>(gi.At(w));
            return GridSampler3dBwd(dt, go.At(w), x.At(w), gr.At(w), gi.At(w), gg.At(w), acc, g, wantInput, wantGrid, s);
        });
    }
    if (wantInput) {
        FinishOutput(giT, gi, ex);
    }
    if (wantGrid) {
        FinishOutput(gridGrad, gg, ex);
    }
    ex->workspaceSize = ws.Size();
    *workspaceSize = ws.Size();
    *executor = ex;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnGridSampler3DBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                       aclrtStream stream)
{
    return RunExecutor("aclnnGridSampler3DBackward", workspace, workspaceSize, executor, stream);
}

} // extern "C"
