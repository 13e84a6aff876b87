// The acl object model (tensors, arrays, executors), error reporting and per-thread options.
#include <nvtx3/nvToolsExt.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_set>

#include "host_common.h"

namespace opscv {

namespace {

thread_local std::string g_lastError;
thread_local int64_t g_deterministic = 0;
thread_local int32_t g_backwardAlgo = 0;

int LogLevel()
{
    static const int level = [] {
        const char* e = std::getenv("OPSCV_LOG_LEVEL");
        return e ? std::atoi(e) : 0;
    }();
    return level;
}

std::mutex g_execMutex;
std::unordered_set<aclOpExecutor*>& LiveExecutors()
{
    static std::unordered_set<aclOpExecutor*> s;
    return s;
}

} // namespace

aclnnStatus Fail(aclnnStatus code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_lastError = "[" + std::to_string(code) + "] " + buf;
    if (LogLevel() >= 1) {
        fprintf(stderr, "[opscv][E] %s\n", g_lastError.c_str());
    }
    return code;
}

void LogInfo(const char* fmt, ...)
{
    if (LogLevel() < 2) {
        return;
    }
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    fprintf(stderr, "[opscv][I] %s\n", buf);
}

// NVTX ranges around the two phases of every call (the tracing hook of this library, as the reference's
// entry points log through its dfx macros): off unless OPSCV_NVTX is set to a non-zero value or OPSCV_LOG_LEVEL >= 2.
// nvtx3 is header-only and finds the profiler's injection library at run time; without a profiler a range is a
// few nanoseconds of no-op.
bool NvtxEnabled()
{
    static const bool on = [] {
        const char* e = std::getenv("OPSCV_NVTX");
        return (e != nullptr && std::atoi(e) != 0) || LogLevel() >= 2;
    }();
    return on;
}
struct NvtxRange {
    explicit NvtxRange(const char* name) : on(NvtxEnabled())
    {
        if (on) {
            nvtxRangePushA(name);
        }
    }
    ~NvtxRange()
    {
        if (on) {
            nvtxRangePop();
        }
    }
    bool on;
};

aclOpExecutor* NewExecutor(const char* api)
{
    const NvtxRange range(api); // phase 1: the executor is created at the end of validation and planning
    aclOpExecutor* e = new (std::nothrow) aclOpExecutor();
    if (e == nullptr) {
        return nullptr;
    }
    e->api = api;
    std::lock_guard<std::mutex> lock(g_execMutex);
    LiveExecutors().insert(e);
    return e;
}

bool ReleaseExecutor(aclOpExecutor* e)
{
    {
        std::lock_guard<std::mutex> lock(g_execMutex);
        auto it = LiveExecutors().find(e);
        if (it == LiveExecutors().end()) {
            return false;
        }
        LiveExecutors().erase(it);
    }
    delete e;
    return true;
}

aclnnStatus RunExecutor(const char* api, void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                        aclrtStream stream)
{
    if (executor == nullptr) {
        return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: executor is null", api);
    }
    {
        std::lock_guard<std::mutex> lock(g_execMutex);
        if (LiveExecutors().find(executor) == LiveExecutors().end()) {
            return Fail(ACLNN_ERR_PARAM_INVALID,
                        "%s: executor is not live (already consumed by a second-phase call, destroyed, or not "
                        "created by this library)",
                        api);
        }
    }
    if (std::strcmp(executor->api, api) != 0) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "%s: executor was created by %sGetWorkspaceSize", api, executor->api);
    }
    if (executor->workspaceSize > 0) {
        if (workspace == nullptr) {
            return Fail(ACLNN_ERR_PARAM_NULLPTR, "%s: workspace is null but %llu bytes are required", api,
                        static_cast<unsigned long long>(executor->workspaceSize));
        }
        if (workspaceSize < executor->workspaceSize) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: workspaceSize %llu is smaller than the required %llu", api,
                        static_cast<unsigned long long>(workspaceSize),
                        static_cast<unsigned long long>(executor->workspaceSize));
        }
        if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) {
            return Fail(ACLNN_ERR_PARAM_INVALID, "%s: workspace must be 256-byte aligned", api);
        }
    }
    aclnnStatus status = ACLNN_SUCCESS;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const NvtxRange range(api); // phase 2: the launches of this call
    for (auto& step : executor->steps) {
        const cudaError_t e = step(static_cast<char*>(workspace), s);
        if (e != cudaSuccess) {
            status = Fail(ACLNN_ERR_RUNTIME_ERROR, "%s: CUDA error %d (%s)", api, static_cast<int>(e),
                          cudaGetErrorString(e));
            break;
        }
    }
    LogInfo("%s: ran %zu steps, workspace %llu bytes, status %d", api, executor->steps.size(),
            static_cast<unsigned long long>(executor->workspaceSize), status);
    ReleaseExecutor(executor);
    return status;
}

bool IsContiguous(const aclTensor* t)
{
    int64_t expect = 1;
    for (int64_t i = static_cast<int64_t>(t->dims.size()) - 1; i >= 0; --i) {
        if (t->dims[i] != 1 && t->strides[i] != expect) {
            return false;
        }
        expect *= t->dims[i];
    }
    return true;
}

bool DtypeSupported(aclDataType d) { return d == ACL_FLOAT || d == ACL_FLOAT16 || d == ACL_BF16; }

Dt ToDt(aclDataType d) { return d == ACL_FLOAT ? Dt::F32 : (d == ACL_FLOAT16 ? Dt::F16 : Dt::BF16); }

const char* DtypeName(aclDataType d)
{
    switch (d) {
        case ACL_FLOAT: return "FLOAT";
        case ACL_FLOAT16: return "FLOAT16";
        case ACL_BF16: return "BF16";
        case ACL_DOUBLE: return "DOUBLE";
        case ACL_INT8: return "INT8";
        case ACL_INT16: return "INT16";
        case ACL_INT32: return "INT32";
        case ACL_INT64: return "INT64";
        case ACL_UINT8: return "UINT8";
        case ACL_BOOL: return "BOOL";
        default: return "UNKNOWN";
    }
}

const char* FormatName(aclFormat f)
{
    switch (f) {
        case ACL_FORMAT_NCHW: return "NCHW";
        case ACL_FORMAT_NHWC: return "NHWC";
        case ACL_FORMAT_ND: return "ND";
        case ACL_FORMAT_NCL: return "NCL";
        case ACL_FORMAT_NCDHW: return "NCDHW";
        case ACL_FORMAT_NDHWC: return "NDHWC";
        default: return "UNKNOWN";
    }
}

int64_t GetDeterministic() { return g_deterministic; }
int32_t GetBackwardAlgo() { return g_backwardAlgo; }

// The view as at most four (extent, stride) pairs: extents of 1 are dropped and neighbours that are contiguous with
// respect to each other are merged, which brings every 5-D view with at least one such pair down to four.
static bool CollapseView(const aclTensor* t, View4& v)
{
    std::vector<int64_t> dims, strides;
    for (size_t i = 0; i < t->dims.size(); ++i) {
        if (t->dims[i] == 1) {
            continue;
        }
        if (!dims.empty() && strides.back() == t->strides[i] * t->dims[i]) {
            dims.back() *= t->dims[i];
            strides.back() = t->strides[i];
        } else {
            dims.push_back(t->dims[i]);
            strides.push_back(t->strides[i]);
        }
    }
    if (dims.size() > 4) {
        return false;
    }
    const size_t rank = dims.size();
    for (size_t i = 0; i < 4; ++i) { // right-align
        const int64_t src = static_cast<int64_t>(i) - (4 - static_cast<int64_t>(rank));
        v.dim[i] = src >= 0 ? dims[src] : 1;
        v.stride[i] = src >= 0 ? strides[src] : 0;
    }
    return true;
}

bool ViewStageable(const aclTensor* t)
{
    View4 v;
    return IsContiguous(t) || CollapseView(t, v);
}

static View4 MakeView4(const aclTensor* t)
{
    View4 v{};
    CollapseView(t, v); // callers with tensors of rank above four check ViewStageable in their first phase
    return v;
}

BufRef StageInput(const aclTensor* t, WsPlan& ws, aclOpExecutor* ex)
{
    BufRef r;
    char* base = static_cast<char*>(t->data) + t->offset * ElemSize(t->dtype);
    if (IsContiguous(t)) {
        r.base = base;
        return r;
    }
    r.inWs = true;
    r.wsOff = ws.Alloc(static_cast<uint64_t>(Numel(t)) * ElemSize(t->dtype));
    const View4 v = MakeView4(t);
    const int elem = ElemSize(t->dtype);
    const uint64_t off = r.wsOff;
    ex->steps.push_back([=](char* w, cudaStream_t s) { return StridedCopy(elem, w + off, base, v, false, s); });
    return r;
}

BufRef StageOutput(const aclTensor* t, WsPlan& ws)
{
    BufRef r;
    if (IsContiguous(t)) {
        r.base = static_cast<char*>(t->data) + t->offset * ElemSize(t->dtype);
        return r;
    }
    r.inWs = true;
    r.wsOff = ws.Alloc(static_cast<uint64_t>(Numel(t)) * ElemSize(t->dtype));
    return r;
}

void FinishOutput(const aclTensor* t, const BufRef& staged, aclOpExecutor* ex)
{
    if (!staged.inWs) {
        return;
    }
    char* base = static_cast<char*>(t->data) + t->offset * ElemSize(t->dtype);
    const View4 v = MakeView4(t);
    const int elem = ElemSize(t->dtype);
    const uint64_t off = staged.wsOff;
    ex->steps.push_back([=](char* w, cudaStream_t s) { return StridedCopy(elem, w + off, base, v, true, s); });
}

} // namespace opscv

using namespace opscv;

extern "C" {

aclTensor* aclCreateTensor(const int64_t* viewDims, uint64_t viewDimsNum, aclDataType dataType,
                           const int64_t* stride, int64_t offset, aclFormat format, const int64_t* storageDims,
                           uint64_t storageDimsNum, void* tensorData)
{
    if (viewDimsNum > 8 || (viewDimsNum > 0 && viewDims == nullptr) || offset < 0) {
        Fail(ACLNN_ERR_PARAM_INVALID, "aclCreateTensor: invalid view description");
        return nullptr;
    }
    aclTensor* t = new (std::nothrow) aclTensor();
    if (t == nullptr) {
        return nullptr;
    }
    t->dims.assign(viewDims, viewDims + viewDimsNum);
    for (int64_t d : t->dims) {
        if (d < 0) {
            delete t;
            Fail(ACLNN_ERR_PARAM_INVALID, "aclCreateTensor: negative extent");
            return nullptr;
        }
    }
    if (stride != nullptr) {
        t->strides.assign(stride, stride + viewDimsNum);
    } else {
        t->strides.assign(viewDimsNum, 1);
        for (int64_t i = static_cast<int64_t>(viewDimsNum) - 2; i >= 0; --i) {
            t->strides[i] = t->strides[i + 1] * t->dims[i + 1];
        }
    }
    if (storageDims != nullptr) {
        t->storageDims.assign(storageDims, storageDims + storageDimsNum);
    }
    t->offset = offset;
    t->dtype = dataType;
    t->format = format;
    t->data = tensorData;
    return t;
}

aclnnStatus aclDestroyTensor(const aclTensor* tensor)
{
    delete tensor;
    return ACLNN_SUCCESS;
}

aclIntArray* aclCreateIntArray(const int64_t* value, uint64_t size)
{
    if (size > 0 && value == nullptr) {
        return nullptr;
    }
    aclIntArray* a = new (std::nothrow) aclIntArray();
    if (a != nullptr) {
        a->v.assign(value, value + size);
    }
    return a;
}

aclnnStatus aclDestroyIntArray(const aclIntArray* array)
{
    delete array;
    return ACLNN_SUCCESS;
}

aclBoolArray* aclCreateBoolArray(const bool* value, uint64_t size)
{
    if (size > 0 && value == nullptr) {
        return nullptr;
    }
    aclBoolArray* a = new (std::nothrow) aclBoolArray();
    if (a != nullptr) {
        a->v.resize(size);
        for (uint64_t i = 0; i < size; ++i) {
            a->v[i] = value[i] ? 1 : 0;
        }
    }
    return a;
}

aclFloatArray* aclCreateFloatArray(const float* value, uint64_t size)
{
    if (size > 0 && value == nullptr) {
        return nullptr;
    }
    aclFloatArray* a = new (std::nothrow) aclFloatArray();
    if (a != nullptr) {
        a->v.assign(value, value + size);
    }
    return a;
}

aclnnStatus aclDestroyFloatArray(const aclFloatArray* array)
{
    delete array;
    return ACLNN_SUCCESS;
}

aclnnStatus aclGetFloatArraySize(const aclFloatArray* array, uint64_t* size)
{
    if (array == nullptr || size == nullptr) {
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    *size = array->v.size();
    return ACLNN_SUCCESS;
}

aclnnStatus aclDestroyBoolArray(const aclBoolArray* array)
{
    delete array;
    return ACLNN_SUCCESS;
}

aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor* executor)
{
    if (executor == nullptr) {
        return ACLNN_SUCCESS;
    }
    return ReleaseExecutor(executor) ? ACLNN_SUCCESS :
                                       Fail(ACLNN_ERR_PARAM_INVALID, "aclDestroyAclOpExecutor: executor is not live");
}

const char* aclGetRecentErrMsg(void) { return g_lastError.c_str(); }

aclError aclrtCtxSetSysParamOpt(aclSysParamOpt opt, int64_t value)
{
    if (opt != ACL_OPT_DETERMINISTIC) {
        return ACL_ERROR_INVALID_PARAM;
    }
    g_deterministic = value != 0 ? 1 : 0;
    return ACL_SUCCESS;
}

aclError aclrtCtxGetSysParamOpt(aclSysParamOpt opt, int64_t* value)
{
    if (opt != ACL_OPT_DETERMINISTIC || value == nullptr) {
        return ACL_ERROR_INVALID_PARAM;
    }
    *value = g_deterministic;
    return ACL_SUCCESS;
}

aclnnStatus opscvSetBackwardAlgo(int32_t algo)
{
    if (algo != 0 && algo != 1) {
        return Fail(ACLNN_ERR_PARAM_INVALID, "opscvSetBackwardAlgo: algo must be 0 (gather) or 1 (atomic)");
    }
    g_backwardAlgo = algo;
    return ACLNN_SUCCESS;
}

int32_t opscvGetBackwardAlgo(void) { return g_backwardAlgo; }
int32_t opscvVersion(void) { return 100; }
uint64_t opscvGetLaunchCount(void) { return LaunchCount(); }
void opscvResetLaunchCount(void) { ResetLaunchCount(); }
uint32_t opscvGetAsyncCopyTimeouts(void) { return AsyncCopyTimeouts(); }

} // extern "C"
