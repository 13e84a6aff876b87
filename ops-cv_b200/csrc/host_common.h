// Host-side object model behind the public C types, and the helpers every aclnn entry point shares: error
// reporting, the executor (a frozen list of launch steps), workspace planning and strided-view staging.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <functional>
#include <vector>

#include "../../include/aclnn_resample.h"
#include "kernels.h"

struct aclTensor {
    std::vector<int64_t> dims;
    std::vector<int64_t> strides;
    std::vector<int64_t> storageDims;
    int64_t offset = 0;
    aclDataType dtype = ACL_FLOAT;
    aclFormat format = ACL_FORMAT_ND;
    void* data = nullptr;
};

struct aclIntArray {
    std::vector<int64_t> v;
};

struct aclBoolArray {
    std::vector<uint8_t> v;
};

struct aclFloatArray {
    std::vector<float> v;
};

namespace opscv {

using Step = std::function<cudaError_t(char* ws, cudaStream_t stream)>;

} // namespace opscv

struct aclOpExecutor {
    std::vector<opscv::Step> steps;
    uint64_t workspaceSize = 0;
    const char* api = "";
};

namespace opscv {

// ---- errors -------------------------------------------------------------------------------------------------
// Records a message for aclGetRecentErrMsg, logs it when OPSCV_LOG_LEVEL >= 1, and returns `code`.
aclnnStatus Fail(aclnnStatus code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void LogInfo(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

// ---- executor registry -----------------------------------------------------------------------------------------
// Live executors are tracked so that a second-phase call with a consumed or foreign pointer is rejected instead
// of dereferencing freed memory.
aclOpExecutor* NewExecutor(const char* api);
bool ReleaseExecutor(aclOpExecutor* e); // true if it was live (and is now deleted)
// The shared second phase: validates workspace/executor, runs the steps on `stream`, consumes the executor.
aclnnStatus RunExecutor(const char* api, void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                        aclrtStream stream);

// ---- tensor helpers ------------------------------------------------------------------------------------------
inline bool IsEmpty(const aclTensor* t)
{
    for (int64_t d : t->dims) {
        if (d == 0) {
            return true;
        }
    }
    return false;
}
inline int64_t Numel(const aclTensor* t)
{
    int64_t n = 1;
    for (int64_t d : t->dims) {
        n *= d;
    }
    return n;
}
bool IsContiguous(const aclTensor* t);
bool DtypeSupported(aclDataType d); // fp32 / fp16 / bf16
Dt ToDt(aclDataType d);
inline int ElemSize(aclDataType d) { return d == ACL_FLOAT ? 4 : 2; }
const char* DtypeName(aclDataType d);
const char* FormatName(aclFormat f);
int64_t GetDeterministic(); // thread-local ACL_OPT_DETERMINISTIC
int32_t GetBackwardAlgo();

// Forward source-coordinate scale of UpsampleBilinear2d
// (image/resize_bilinear_v2/op_host/arch35/resize_bilinear_v2_tiling_arch35.cpp:175-243).
inline float BilinearScale(int64_t in, int64_t out, bool align, float userScale)
{
    if (!align) {
        return userScale > 0.0f ? 1.0f / userScale : static_cast<float>(in) / static_cast<float>(out);
    }
    float s = static_cast<float>(in) / static_cast<float>(out);
    if (out > 1) {
        s = static_cast<float>(in - 1) / static_cast<float>(out - 1);
    }
    return s;
}

// ---- workspace planning ----------------------------------------------------------------------------------------
class WsPlan {
public:
    uint64_t Alloc(uint64_t bytes)
    {
        const uint64_t off = size_;
        size_ += (bytes + 255) & ~static_cast<uint64_t>(255);
        return off;
    }
    uint64_t Size() const { return size_; }

private:
    uint64_t size_ = 0;
};

// A device buffer that is either caller memory or a region of the workspace (resolved in the second phase).
struct BufRef {
    void* base = nullptr;
    uint64_t wsOff = 0;
    bool inWs = false;
    void* At(char* ws) const { return inWs ? static_cast<void*>(ws + wsOff) : base; }
};

// Input staging: returns a reference to contiguous data of `t`; for a strided view a gather-copy step into the
// workspace is appended to the executor first (the reference's l0op::Contiguous).
// False for a view of rank five or more that no merging of neighbouring dimensions brings down to four strided
// dimensions (the staging copies handle four).
bool ViewStageable(const aclTensor* t);
BufRef StageInput(const aclTensor* t, WsPlan& ws, aclOpExecutor* ex);
// Output staging: returns where the kernels must write; for a strided view that is a workspace buffer, and
// FinishOutput appends the scatter-copy back into the view (the reference's l0op::ViewCopy).
BufRef StageOutput(const aclTensor* t, WsPlan& ws);
void FinishOutput(const aclTensor* t, const BufRef& staged, aclOpExecutor* ex);

} // namespace opscv
