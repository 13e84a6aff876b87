/*
 * opscv_acl.h - the small part of the CANN "acl" object model that the aclnn resampling entry points need.
 *
 * In the reference these objects (aclTensor, aclIntArray, aclBoolArray, aclOpExecutor, aclrtStream) and their
 * constructors come from the CANN runtime / opbase packages, not from ops-cv itself; ops-cv only consumes them
 * (usage: image/upsample_bilinear2d/examples/test_aclnn_upsample_bilinear2d.cpp:55-72,
 * image/grid_sampler2_d_grad/examples/test_aclnn_grid_sampler2_d_backward.cpp:107-117; described in
 * docs/zh/context/data_structure.md and docs/zh/context/non_contiguous_tensor.md). This library supplies
 * source-compatible equivalents so that a caller of the reference's aclnn API links unchanged.
 *
 * On this library aclrtStream is a cudaStream_t and every data pointer is a CUDA device pointer.
 */
#ifndef OPSCV_ACL_H
#define OPSCV_ACL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#include <cstdbool>
extern "C" {
#else
#include <stdbool.h>
#endif

#define ACLNN_API __attribute__((visibility("default")))

typedef int32_t aclnnStatus;
typedef int aclError;

/* docs/zh/context/aclnn_return_code.md:8-30 */
#define ACLNN_SUCCESS 0
#define ACLNN_ERR_PARAM_NULLPTR 161001
#define ACLNN_ERR_PARAM_INVALID 161002
#define ACLNN_ERR_RUNTIME_ERROR 361001
#define ACLNN_ERR_INNER 561000
#define ACLNN_ERR_INNER_CREATE_EXECUTOR 561101
#define ACLNN_ERR_INNER_NULLPTR 561103
#define ACL_SUCCESS 0
#define ACL_ERROR_NONE 0
#define ACL_ERROR_INVALID_PARAM 100000

/* Values follow the public CANN acl_base.h so that callers compiled against it pass the same integers. */
typedef enum {
    ACL_DT_UNDEFINED = -1,
    ACL_FLOAT = 0,
    ACL_FLOAT16 = 1,
    ACL_INT8 = 2,
    ACL_INT32 = 3,
    ACL_UINT8 = 4,
    ACL_INT16 = 6,
    ACL_UINT16 = 7,
    ACL_UINT32 = 8,
    ACL_INT64 = 9,
    ACL_UINT64 = 10,
    ACL_DOUBLE = 11,
    ACL_BOOL = 12,
    ACL_BF16 = 27
} aclDataType;

typedef enum {
    ACL_FORMAT_UNDEFINED = -1,
    ACL_FORMAT_NCHW = 0,
    ACL_FORMAT_NHWC = 1,
    ACL_FORMAT_ND = 2,
    ACL_FORMAT_NDHWC = 27,
    ACL_FORMAT_NCDHW = 30,
    ACL_FORMAT_NCL = 47
} aclFormat;

typedef enum { ACL_OPT_DETERMINISTIC = 0 } aclSysParamOpt;

typedef struct aclTensor aclTensor;
typedef struct aclIntArray aclIntArray;
typedef struct aclBoolArray aclBoolArray;
typedef struct aclFloatArray aclFloatArray;
typedef struct aclOpExecutor aclOpExecutor;
typedef void* aclrtStream; /* a cudaStream_t */

/*
 * A tensor is a (viewDims, strides, offset) view over a device buffer; strides and offset are in elements.
 * For ACL_FORMAT_NHWC the view dims are ordered [N, H, W, C]. `tensorData` must stay valid until the
 * stream work that uses it has finished. Returns NULL on invalid arguments (NULL dims with a non-zero
 * rank, rank > 8, negative extents).
 */
ACLNN_API aclTensor* aclCreateTensor(const int64_t* viewDims, uint64_t viewDimsNum, aclDataType dataType,
                                     const int64_t* stride, int64_t offset, aclFormat format,
                                     const int64_t* storageDims, uint64_t storageDimsNum, void* tensorData);
ACLNN_API aclnnStatus aclDestroyTensor(const aclTensor* tensor);
ACLNN_API aclIntArray* aclCreateIntArray(const int64_t* value, uint64_t size);
ACLNN_API aclnnStatus aclDestroyIntArray(const aclIntArray* array);
ACLNN_API aclBoolArray* aclCreateBoolArray(const bool* value, uint64_t size);
ACLNN_API aclnnStatus aclDestroyBoolArray(const aclBoolArray* array);
ACLNN_API aclFloatArray* aclCreateFloatArray(const float* value, uint64_t size);
ACLNN_API aclnnStatus aclDestroyFloatArray(const aclFloatArray* array);
/* Number of values of `array` through *size; a non-zero status for a NULL argument. */
ACLNN_API aclnnStatus aclGetFloatArraySize(const aclFloatArray* array, uint64_t* size);

/* Frees an executor returned by a GetWorkspaceSize call that will not be passed to its second-phase call. */
ACLNN_API aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor* executor);

/* Text of the most recent failure on the calling thread ("" if none). The pointer stays valid until the
 * next failing call on the same thread. */
ACLNN_API const char* aclGetRecentErrMsg(void);

/*
 * Per-thread option store standing in for the CANN context options. ACL_OPT_DETERMINISTIC = 1 selects the
 * bit-reproducible backward kernels; the value is read by the first-phase call and frozen into the executor
 * (reference: aclrtCtxGetSysParamOpt in image/grid_sampler2_d_grad/op_host/op_api/aclnn_grid_sampler2d_backward.cpp:180-186,
 * context->GetDeterministic() in image/resize_bilinear_v2_grad/op_host/arch35/resize_bilinear_v2_grad_tiling_arch35.cpp:74).
 */
ACLNN_API aclError aclrtCtxSetSysParamOpt(aclSysParamOpt opt, int64_t value);
ACLNN_API aclError aclrtCtxGetSysParamOpt(aclSysParamOpt opt, int64_t* value);

/*
 * Library-specific knobs (no counterpart in the reference).
 *
 * opscvSetBackwardAlgo: how the non-deterministic backward of the separable resamplers (bilinear, bicubic-AA)
 * is computed on the calling thread. 0 (default) = gather kernels, which are both the fastest and
 * deterministic on this hardware; 1 = the scatter kernels with fp32 atomics (the reference's "atomic" schedule).
 * GridSampler2DBackward is not affected: it uses atomics unless ACL_OPT_DETERMINISTIC is set.
 */
ACLNN_API aclnnStatus opscvSetBackwardAlgo(int32_t algo);
ACLNN_API int32_t opscvGetBackwardAlgo(void);
/* Library version: major * 10000 + minor * 100 + patch. */
ACLNN_API int32_t opscvVersion(void);
/* Number of kernel launches this thread has enqueued through second-phase calls since the last reset. */
ACLNN_API uint64_t opscvGetLaunchCount(void);
ACLNN_API void opscvResetLaunchCount(void);
/* Number of bounded device-side waits on asynchronous copies that ran out on the current device since the library
 * was loaded (a kernel that gives up a wait abandons its block's work and counts here instead of hanging).
 * 0 in a healthy run; 0xffffffff if the counter cannot be read. Synchronises the device. */
ACLNN_API uint32_t opscvGetAsyncCopyTimeouts(void);

#ifdef __cplusplus
}
#endif
#endif /* OPSCV_ACL_H */
