/*
 * aclnn_resample.h - the image-resampling entry points of hicann/ops-cv, served by hand-written CUDA kernels
 * for NVIDIA B200 (sm_100a).
 *
 * Every operator keeps the reference's two-phase protocol (docs/zh/context/two_phase_api.md):
 *
 *   1. aclnnXxxGetWorkspaceSize(...) validates the arguments, chooses the launch configuration, and returns
 *      the number of device bytes of workspace the caller must provide plus an executor. No GPU work happens.
 *   2. aclnnXxx(workspace, workspaceSize, executor, stream) enqueues the kernels on `stream` (a cudaStream_t)
 *      and returns without synchronising. The executor is consumed: it must not be passed to a second call.
 *
 * Argument meaning, dtype / format rules, the order of the checks and the status codes follow the reference
 * files cited at each declaration (paths relative to the reference repository). Arithmetic follows the
 * reference's "arch35" SIMT kernels: all interpolation is done in fp32 and rounded once to the storage dtype.
 * There is no CPU fallback: without a CUDA device the second-phase call returns ACLNN_ERR_RUNTIME_ERROR.
 *
 * Supported storage dtypes: ACL_FLOAT, ACL_FLOAT16, ACL_BF16. (The reference routes ACL_DOUBLE / ACL_UINT8 to
 * AI-CPU kernels; those dtypes are rejected here with ACLNN_ERR_PARAM_INVALID.)
 */
#ifndef ACLNN_RESAMPLE_H
#define ACLNN_RESAMPLE_H

#include "opscv_acl.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- UpsampleNearest2d ---------------------------------------------------------------------------------
 * Replaces image/resize_nearest_neighbor_v2/op_api/aclnn_upsample_nearest_2d.h:49-80
 * (implementation aclnn_upsample_nearest_2d.cpp:247-311; kernel resize_nearest_neighbor_v2_simt.h:104-155).
 * self/out: 4-D, NCHW or NHWC (same format, same dtype), out H,W == outputSize. src = min(floor(dst*in/out), in-1).
 */
ACLNN_API aclnnStatus aclnnUpsampleNearest2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                             aclTensor* out, uint64_t* workspaceSize,
                                                             aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearest2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                             const aclrtStream stream);

/* Replaces image/upsample_nearest3d/op_host/op_api/aclnn_upsample_nearest_2d_v2.h:38-55 (implementation
 * aclnn_upsample_nearest_2d_v2.cpp:316-400). Same as above with user scales: when scalesH/W > 0 the source
 * index uses 1/scales instead of in/out. */
ACLNN_API aclnnStatus aclnnUpsampleNearest2dV2GetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                               float scalesH, float scalesW, aclTensor* out,
                                                               uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearest2dV2(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                               aclrtStream stream);

/* Replaces image/upsample_nearest2d_grad/op_host/op_api/aclnn_upsample_nearest_2d_backward.h:40-59
 * (implementation aclnn_upsample_nearest_2d_backward.cpp:320-388; kernel
 * resize_nearest_neighbor_v2_grad_simt_determine.h:79-118). inputSize = {N,C,H,W} (or {N,H,W,C} for NHWC) of
 * gradInput; deterministic gather with fp32 accumulation. */
ACLNN_API aclnnStatus aclnnUpsampleNearest2dBackwardGetWorkspaceSize(const aclTensor* gradOut,
                                                                     const aclIntArray* outputSize,
                                                                     const aclIntArray* inputSize, double scalesH,
                                                                     double scalesW, aclTensor* gradInput,
                                                                     uint64_t* workspaceSize,
                                                                     aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearest2dBackward(void* workspace, uint64_t workspaceSize,
                                                     aclOpExecutor* executor, aclrtStream stream);

/* ---- UpsampleBilinear2d --------------------------------------------------------------------------------
 * Replaces image/upsample_bilinear2d/op_host/op_api/aclnn_upsample_bilinear_2d.h:24-34 (implementation
 * aclnn_upsample_bilinear_2d.cpp:384-467; kernel resize_bilinear_v2_simt_nchw.h:84-146 / _simt_nhwc.h:88-151).
 * Null self/out returns ACLNN_ERR_INNER_NULLPTR (561103) as the reference does (:175). */
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                              const bool alignCorners, const double scalesH,
                                                              const double scalesW, aclTensor* out,
                                                              uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBilinear2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                              aclrtStream stream);

/* Replaces image/resize_bilinear_v2_grad/op_api/aclnn_upsample_bilinear_2d_backward.h:23-32 (implementation
 * aclnn_upsample_bilinear_2d_backward.cpp:226-309; kernels resize_bilinear_v2_grad_simt.h:107-152 and
 * resize_bilinear_v2_grad_simt_determine.h:56-123). out dtype == gradOut dtype, or any supported dtype when
 * gradOut is fp32. */
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dBackwardGetWorkspaceSize(const aclTensor* gradOut,
                                                                      const aclIntArray* outputSize,
                                                                      const aclIntArray* inputSize,
                                                                      bool alignCorners, double scalesH,
                                                                      double scalesW, aclTensor* out,
                                                                      uint64_t* workspaceSize,
                                                                      aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dBackward(void* workspace, uint64_t workspaceSize,
                                                      aclOpExecutor* executor, aclrtStream stream);

/* Replaces image/upsample_bilinear2d_grad/op_host/op_api/aclnn_upsample_bilinear_2d_backward_v2.h:33-58
 * (implementation aclnn_upsample_bilinear_2d_backward_v2.cpp:354-446). Same kernels as above. */
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dBackwardV2GetWorkspaceSize(const aclTensor* gradOut,
                                                                        const aclIntArray* outputSize,
                                                                        const aclIntArray* inputSize,
                                                                        bool alignCorners, double scalesH,
                                                                        double scalesW, aclTensor* out,
                                                                        uint64_t* workspaceSize,
                                                                        aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dBackwardV2(void* workspace, uint64_t workspaceSize,
                                                        aclOpExecutor* executor, aclrtStream stream);

/* ---- UpsampleBicubic2dAA -------------------------------------------------------------------------------
 * Replaces image/upsample_bicubic2d_aa/op_host/op_api/aclnn_upsample_bicubic2d_aa.h:40-58 (implementation
 * aclnn_upsample_bicubic2d_aa.cpp:164-229; kernel upsample_bicubic2d_aa_simt_base.h:31-127; scale/support
 * upsample_bicubic2d_aa_tiling_arch35.cpp:139-168). NCHW (or ND) only; Keys cubic with a = -0.5, support
 * 2*scale when down-scaling. */
ACLNN_API aclnnStatus aclnnUpsampleBicubic2dAAGetWorkspaceSize(const aclTensor* x, const aclIntArray* outputSize,
                                                               const bool alignCorners, const double scalesH,
                                                               const double scalesW, aclTensor* out,
                                                               uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBicubic2dAA(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                               aclrtStream stream);

/* Replaces image/upsample_bicubic2d_aa_grad/op_host/op_api/aclnn_upsample_bicubic2d_aa_grad.h:39-58
 * (implementation aclnn_upsample_bicubic2d_aa_grad.cpp:183-232; kernels upsample_bicubic2d_aa_grad_simt_base.h:32-102
 * and upsample_bicubic2d_aa_grad_simt_base_deter.h:30-122). */
ACLNN_API aclnnStatus aclnnUpsampleBicubic2dAAGradGetWorkspaceSize(const aclTensor* gradOutput,
                                                                   const aclIntArray* outputSize,
                                                                   const aclIntArray* inputSize, bool alignCorners,
                                                                   double scalesH, double scalesW, aclTensor* out,
                                                                   uint64_t* workspaceSize,
                                                                   aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBicubic2dAAGrad(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                   aclrtStream stream);

/* ---- UpsampleNearestExact2d -------------------------------------------------------------------------------
 * Replaces image/upsample_nearest/op_host/op_api/aclnn_upsample_nearest_exact2d.h:42-60 (implementation
 * aclnn_upsample_nearest_exact2d.cpp:284-340, regbase branch: ResizeNearestNeighborV2 with half_pixel_centers = true;
 * index image/resize_nearest_neighbor_v2/op_kernel/arch35/resize_nearest_neighbor_v2_simt.h:115-123:
 * src = min(floor((dst + 0.5) * scale), in - 1)). NCHW, NHWC or ND. Same kernels as UpsampleNearest2d with the
 * other index table. */
ACLNN_API aclnnStatus aclnnUpsampleNearestExact2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                                  double scalesH, double scalesW, aclTensor* out,
                                                                  uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                  aclrtStream stream);

/* Replaces image/upsample_nearest_exact2d_grad/op_host/op_api/aclnn_upsample_nearest_exact2d_backward.h:39-56
 * (implementation aclnn_upsample_nearest_exact2d_backward.cpp:178-240; kernel
 * op_kernel/arch35/upsample_nearest_exact2d_grad_simt_base.h:33-139: grad_input[y] sums the grads window
 * [ceil(y * s - 0.5), ceil((y + 1) * s - 0.5)) in fp32). NCHW or ND. */
ACLNN_API aclnnStatus aclnnUpsampleNearestExact2dBackwardGetWorkspaceSize(const aclTensor* gradOutput,
                                                                          const aclIntArray* outputSize,
                                                                          const aclIntArray* inputSize,
                                                                          double scalesH, double scalesW,
                                                                          aclTensor* out, uint64_t* workspaceSize,
                                                                          aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact2dBackward(void* workspace, uint64_t workspaceSize,
                                                          aclOpExecutor* executor, aclrtStream stream);

/* The 1-D pair: (N, C, L) tensors in NCL or ND format, computed as the 2-D operator on the (N, C, 1, L) view with
 * scales {1, scales}. Replaces image/upsample_nearest/op_host/op_api/aclnn_upsample_nearest_exact1d.h
 * (implementation aclnn_upsample_nearest_exact1d.cpp:166-226) and
 * image/upsample_nearest_exact2d_grad/op_host/op_api/aclnn_upsample_nearest_exact1d_backward.h (implementation
 * aclnn_upsample_nearest_exact1d_backward.cpp, first phase). */
ACLNN_API aclnnStatus aclnnUpsampleNearestExact1dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                                  double scales, aclTensor* out,
                                                                  uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact1d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                  aclrtStream stream);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact1dBackwardGetWorkspaceSize(const aclTensor* gradOutput,
                                                                          const aclIntArray* outputSize,
                                                                          const aclIntArray* inputSize, double scales,
                                                                          aclTensor* out, uint64_t* workspaceSize,
                                                                          aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact1dBackward(void* workspace, uint64_t workspaceSize,
                                                          aclOpExecutor* executor, aclrtStream stream);

/* ---- UpsampleBilinear2dAA ----------------------------------------------------------------------------------
 * Replaces image/upsample_bilinear2d_aa/op_host/op_api/aclnn_upsample_bilinear2d_aa.h:38-49 (implementation
 * aclnn_upsample_bilinear2d_aa.cpp:184-252; kernel image/upsample_bilinear2d_aa/op_kernel/arch35/
 * upsample_bilinear2d_aa_simt_base.h:30-91; scale / support upsample_bilinear2d_aa_tiling_arch35.cpp:104-154).
 * NCHW (or ND) only; triangle filter, support `scale` when down-scaling. Same tables and kernels as
 * UpsampleBicubic2dAA with the other filter. */
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dAAGetWorkspaceSize(const aclTensor* input, const aclIntArray* outputSize,
                                                                bool alignCorners, double scalesH, double scalesW,
                                                                aclTensor* out, uint64_t* workspaceSize,
                                                                aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dAA(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                aclrtStream stream);

/* Replaces image/upsample_bilinear2d_aa_backward/op_host/op_api/aclnn_upsample_bilinear2d_aa_backward.h:40-56
 * (implementation aclnn_upsample_bilinear2d_aa_backward.cpp:179-250; kernels
 * upsample_bilinear2d_aa_backward_simt_base.h:74-126 atomic, :128-171 deterministic). */
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dAABackwardGetWorkspaceSize(const aclTensor* gradOutput,
                                                                        const aclIntArray* outputSize,
                                                                        const aclIntArray* inputSize,
                                                                        bool alignCorners, double scalesH,
                                                                        double scalesW, aclTensor* out,
                                                                        uint64_t* workspaceSize,
                                                                        aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBilinear2dAABackward(void* workspace, uint64_t workspaceSize,
                                                        aclOpExecutor* executor, aclrtStream stream);

/* ---- UpsampleBicubic2d (no antialiasing) ------------------------------------------------------------------
 * Replaces image/upsample_bicubic2d/op_host/op_api/aclnn_upsample_bicubic_2d.h:25-34 (implementation
 * aclnn_upsample_bicubic_2d.cpp:233-330, regbase branch; kernel
 * image/resize_bicubic_v2/op_kernel/arch35/resize_bicubic_v2_simt_base.h:23-171; schedules and scales
 * image/resize_bicubic_v2/op_host/arch35/resize_bicubic_v2_tiling_arch35.cpp:484-588). NCHW, NHWC or ND; cubic
 * convolution with A = -0.75 over four clamped taps per axis. */
ACLNN_API aclnnStatus aclnnUpsampleBicubic2dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                             const bool alignCorners, const double scalesH,
                                                             const double scalesW, aclTensor* out,
                                                             uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBicubic2d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                             aclrtStream stream);

/* Replaces image/upsample_bicubic2d_grad/op_host/op_api/aclnn_upsample_bicubic_2d_backward.h:24-33 (implementation
 * aclnn_upsample_bicubic_2d_backward.cpp:308-366, regbase branch; gather kernel
 * image/resize_bicubic_v2_grad/op_kernel/arch35/resize_bicubic_v2_grad_simt_determine.h:95-350, which the reference
 * runs when the deterministic option is set or an extent grows; its atomic kernel resize_bicubic_v2_grad_simt.h:108-146
 * adds the same terms in no fixed order). Always the gather here, so results do not change from run to run. */
ACLNN_API aclnnStatus aclnnUpsampleBicubic2dBackwardGetWorkspaceSize(const aclTensor* gradOut,
                                                                     const aclIntArray* outputSize,
                                                                     const aclIntArray* inputSize,
                                                                     const bool alignCorners, double scalesH,
                                                                     double scalesW, aclTensor* gradInput,
                                                                     uint64_t* workspaceSize,
                                                                     aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleBicubic2dBackward(void* workspace, uint64_t workspaceSize,
                                                     aclOpExecutor* executor, aclrtStream stream);

/* ---- UpsampleNearest3d / UpsampleNearestExact3d -------------------------------------------------------------
 * 5-D tensors in ACL_FORMAT_NCDHW (or ND) or ACL_FORMAT_NDHWC; outputSize = {D, H, W}.
 * Replace image/upsample_nearest3d/op_host/op_api/aclnn_upsample_nearest_3d.h (implementation
 * aclnn_upsample_nearest_3d.cpp:156-204; kernel op_kernel/arch35/upsample_nearest3d_simt_base.h:31-88),
 * image/upsample_nearest_exact3d/op_host/op_api/aclnn_upsample_nearest_exact3d.h:25-34 (the same kernel with the
 * half-pixel source index), image/upsample_nearest3d_grad/op_host/op_api/aclnn_upsample_nearest_3d_backward.h:25-33
 * (kernel op_kernel/arch35/upsample_nearest3d_grad_simt_base.h:33-58) and
 * image/upsample_nearest_exact3d_grad/op_host/op_api/aclnn_upsample_nearest_exact3d_backward.h:25-33. */
ACLNN_API aclnnStatus aclnnUpsampleNearest3dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                             double scalesD, double scalesH, double scalesW,
                                                             aclTensor* out, uint64_t* workspaceSize,
                                                             aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearest3d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                             aclrtStream stream);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact3dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                                  double scalesD, double scalesH, double scalesW,
                                                                  aclTensor* out, uint64_t* workspaceSize,
                                                                  aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact3d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                  aclrtStream stream);
ACLNN_API aclnnStatus aclnnUpsampleNearest3dBackwardGetWorkspaceSize(const aclTensor* gradOut,
                                                                     const aclIntArray* outputSize,
                                                                     const aclIntArray* inputSize, double scalesD,
                                                                     double scalesH, double scalesW,
                                                                     aclTensor* gradInput, uint64_t* workspaceSize,
                                                                     aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearest3dBackward(void* workspace, uint64_t workspaceSize,
                                                     aclOpExecutor* executor, aclrtStream stream);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact3dBackwardGetWorkspaceSize(const aclTensor* gradOut,
                                                                          const aclIntArray* outputSize,
                                                                          const aclIntArray* inputSize,
                                                                          double scalesD, double scalesH,
                                                                          double scalesW, aclTensor* gradInput,
                                                                          uint64_t* workspaceSize,
                                                                          aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleNearestExact3dBackward(void* workspace, uint64_t workspaceSize,
                                                          aclOpExecutor* executor, aclrtStream stream);

/* ---- UpsampleTrilinear3d / UpsampleTrilinear3dBackward ------------------------------------------------------------
 * Replace image/resize_upsample_trilinear/op_host/op_api/aclnn_upsample_trilinear_3d.h:25-34 (implementation
 * aclnn_upsample_trilinear_3d.cpp:382-455; kernel arithmetic
 * image/resize_upsample_trilinear/op_kernel/arch35/resize_upsample_trilinear_simt_base_common.h:47-188) and
 * image/upsample_trilinear3d_backward/op_host/op_api/aclnn_upsample_trilinear_3d_backward.h:25-36 (implementation
 * aclnn_upsample_trilinear_3d_backward.cpp:177-245; kernel
 * image/upsample_trilinear3d_backward/op_kernel/upsample_trilinear3d_backward.h:141-263). The three scales are the
 * output-per-input factors and are used only when all three are positive; inputSize is (N, C, D, H, W) in either
 * format. */
ACLNN_API aclnnStatus aclnnUpsampleTrilinear3dGetWorkspaceSize(const aclTensor* self, const aclIntArray* outputSize,
                                                               bool alignCorners, double scalesD, double scalesH,
                                                               double scalesW, aclTensor* out, uint64_t* workspaceSize,
                                                               aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleTrilinear3d(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                               aclrtStream stream);
ACLNN_API aclnnStatus aclnnUpsampleTrilinear3dBackwardGetWorkspaceSize(const aclTensor* gradOut,
                                                                       const aclIntArray* outputSize,
                                                                       const aclIntArray* inputSize, bool alignCorners,
                                                                       double scalesD, double scalesH, double scalesW,
                                                                       aclTensor* gradInput, uint64_t* workspaceSize,
                                                                       aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnUpsampleTrilinear3dBackward(void* workspace, uint64_t workspaceSize,
                                                       aclOpExecutor* executor, aclrtStream stream);

/* ---- GridSampler3D --------------------------------------------------------------------------------------------
 * Replaces image/grid_sample/op_api/aclnn_grid_sampler3d.h (implementation aclnn_grid_sampler3d.cpp:194-380; kernel
 * image/grid_sample/op_kernel/arch35/grid_sampler_3d_bilinear_smit.h:58-184) and
 * image/grid_sampler3_d_grad/op_host/op_api/aclnn_grid_sampler3d_backward.h (implementation
 * aclnn_grid_sampler3d_backward.cpp:183-310; kernel op_kernel/arch35/grid_sampler3_d_grad_simt.h:43-300).
 * input (N, C, D, H, W) in NCDHW / ND (or NDHWC with permuted extents), grid (N, Do, Ho, Wo, 3) holding (x, y, z),
 * out (N, C, Do, Ho, Wo). interpolationMode 0 bilinear, 1 nearest; paddingMode 0 zeros, 1 border, 2 reflection.
 * outputMask = {grad_input wanted, grad_grid wanted}. */
ACLNN_API aclnnStatus aclnnGridSampler3DGetWorkspaceSize(const aclTensor* input, const aclTensor* grid,
                                                         int64_t interpolationMode, int64_t paddingMode,
                                                         bool alignCorners, aclTensor* out, uint64_t* workspaceSize,
                                                         aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnGridSampler3D(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                         aclrtStream stream);
ACLNN_API aclnnStatus aclnnGridSampler3DBackwardGetWorkspaceSize(const aclTensor* gradOutput, const aclTensor* input,
                                                                 const aclTensor* grid, int64_t interpolationMode,
                                                                 int64_t paddingMode, bool alignCorners,
                                                                 const aclBoolArray* outputMask, aclTensor* inputGrad,
                                                                 aclTensor* gridGrad, uint64_t* workspaceSize,
                                                                 aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnGridSampler3DBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                 aclrtStream stream);

/* ---- Resize ---------------------------------------------------------------------------------------------------
 * Replaces image/resize_bilinear_v2/op_api/aclnn_resize.h:32-46 (implementation aclnn_resize.cpp:231-300, regbase
 * branch). `scales` holds one factor per dimension of `self` (4 values); `mode` starts with "nearest" or "bilinear".
 * nearest: UpsampleNearest2d; bilinear: UpsampleBilinear2d with align_corners = false. NCHW or NHWC. */
ACLNN_API aclnnStatus aclnnResizeGetWorkspaceSize(const aclTensor* self, const aclFloatArray* scales, const char* mode,
                                                  aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnResize(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                  aclrtStream stream);

/* ---- GridSampler2D -------------------------------------------------------------------------------------
 * Replaces image/grid_sample/op_api/aclnn_grid_sampler2d.h:53-82 (implementation aclnn_grid_sampler2d.cpp:266-340;
 * arithmetic image/grid_sampler2_d/op_kernel/arch35/grid_sampler2_d_simt.h:106-215,303-514).
 * input (N,C,H,W), grid (N,Ho,Wo,2), out (N,C,Ho,Wo), all one dtype. interpolationMode 0 bilinear, 1 nearest,
 * 2 bicubic; paddingMode 0 zeros, 1 border, 2 reflection. */
ACLNN_API aclnnStatus aclnnGridSampler2DGetWorkspaceSize(const aclTensor* input, const aclTensor* grid,
                                                         int64_t interpolationMode, int64_t paddingMode,
                                                         bool alignCorners, aclTensor* out, uint64_t* workspaceSize,
                                                         aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnGridSampler2D(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                         aclrtStream stream);

/* Replaces image/grid_sampler2_d_grad/op_host/op_api/aclnn_grid_sampler2d_backward.h:58-91 (implementation
 * aclnn_grid_sampler2d_backward.cpp:214-357; arithmetic image/grid_sampler3_d_grad/op_kernel/arch35/
 * grid_sampler3_d_grad_simt_base.h:51-184 and image/grid_sampler2_d_grad/op_kernel/arch35/
 * grid_sampler2_d_grad_simt.h:64-230,235-290). outputMask = {want inputGrad, want gridGrad}; a NULL mask or
 * {false,false} is a successful no-op. Atomic accumulation by default; bit-reproducible, in the summation order of
 * the reference's deterministic kernel (grid_sampler2_d_grad_simt_det.h), when ACL_OPT_DETERMINISTIC is set.
 * interpolationMode 0 bilinear, 1 nearest, 2 bicubic (A = -0.75, every neighbour of the 4 x 4 window through the
 * padding mode). */
ACLNN_API aclnnStatus aclnnGridSampler2DBackwardGetWorkspaceSize(const aclTensor* gradOutput, const aclTensor* input,
                                                                 const aclTensor* grid, int64_t interpolationMode,
                                                                 int64_t paddingMode, bool alignCorners,
                                                                 const aclBoolArray* outputMask, aclTensor* inputGrad,
                                                                 aclTensor* gridGrad, uint64_t* workspaceSize,
                                                                 aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnGridSampler2DBackward(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                 aclrtStream stream);

/* ---- Diagnostics (no counterpart in the reference) ------------------------------------------------------
 * Build on the device, with the same kernels the operators use, the per-axis index / weight tables and copy
 * them to HOST arrays, so that tests can compare the coordinate arithmetic bit for bit with a CPU statement of
 * the reference formulas. `kind`: 0 nearest forward source index (i0 = src[outSize]);
 * 1 nearest backward ranges (i0 = start[inSize], i1 = end[inSize]);
 * 2 bilinear forward (i0 = lo[outSize], i1 = hi[outSize], f0 = delta[outSize]);
 * 3 bicubic-AA forward (i0 = xmin[outSize], i1 = xsize[outSize], f0 = weights[outSize * taps], taps returned
 *   through *tapsOut; pass f0 == NULL to query taps only);
 * 4 bilinear-AA forward, laid out as kind 3.
 * Synchronises the device. Returns 0 or an aclnn status. */
ACLNN_API aclnnStatus opscvDebugAxisTable(int32_t kind, int64_t inSize, int64_t outSize, int32_t alignCorners,
                                          float userScale, int32_t* i0, int32_t* i1, float* f0, int32_t* tapsOut);

/* ---- allocation-free bilinear forward ------------------------------------------------------------------------
 * No counterpart in the reference (its entry points all take a workspace). For callers that can neither allocate
 * device memory nor pass a workspace at the point of the call: the per-axis tap tables live in a fixed 192 KiB
 * array inside the library's device image. Same arithmetic and kernels as aclnnUpsampleBilinear2d on contiguous
 * NCHW / NHWC data (dtype ACL_FLOAT, ACL_FLOAT16 or ACL_BF16); the work is enqueued on `stream`.
 * Limits and rules: outH and outW at most 8192 each (larger: ACLNN_ERR_PARAM_INVALID); the first call on a device
 * looks up the array's address and should be made before any stream capture on that device; all calls on a device
 * share the array, so calls that may overlap (different streams or unordered threads) must be serialised by the
 * caller. */
ACLNN_API aclnnStatus opscvUpsampleBilinear2dNoAlloc(const void* self, void* out, aclDataType dtype, aclFormat format,
                                                     int64_t n, int64_t c, int64_t inH, int64_t inW, int64_t outH,
                                                     int64_t outW, bool alignCorners, double scalesH, double scalesW,
                                                     aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* ACLNN_RESAMPLE_H */
