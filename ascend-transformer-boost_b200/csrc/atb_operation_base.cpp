#include "atb_operation_base.h"
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <new>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <sys/stat.h>
#include <vector>

namespace atb {

// ---------------------------------------------------------------------------------- logging
namespace {
int g_logLevel = -1;
int LogLevelFromEnv()
{
    const char *e = std::getenv("ATB_LOG_LEVEL");
    if (e == nullptr) {
        return static_cast<int>(LogLevel::ERROR);
    }
    static const char *names[] = {"DEBUG", "INFO", "WARN", "ERROR", "NONE"};
    for (int i = 0; i < 5; ++i) {
        if (std::strcmp(e, names[i]) == 0) {
            return i;
        }
    }
    return static_cast<int>(LogLevel::ERROR);
}
} // namespace

void AtbLog(LogLevel level, const std::string &msg)
{
    if (g_logLevel < 0) {
        g_logLevel = LogLevelFromEnv();
    }
    if (static_cast<int>(level) >= g_logLevel && g_logLevel < static_cast<int>(LogLevel::NONE)) {
        static const char *names[] = {"DEBUG", "INFO", "WARN", "ERROR"};
        std::fprintf(stderr, "[atb][%s] %s\n", names[static_cast<int>(level)], msg.c_str());
    }
}

// ------------------------------------------------------------------------------------ Utils
std::string Utils::GetAtbVersion() { return "8.5.0-b200"; }

uint64_t Utils::GetTensorNumel(const TensorDesc &desc)
{
    if (desc.shape.dimNum == 0 || desc.shape.dimNum > MAX_DIM) {
        return 0;
    }
    uint64_t n = 1;
    for (uint64_t i = 0; i < desc.shape.dimNum; ++i) {
        const int64_t d = desc.shape.dims[i];
        if (d <= 0 || std::numeric_limits<uint64_t>::max() / static_cast<uint64_t>(d) < n) {
            return 0;
        }
        n *= static_cast<uint64_t>(d);
    }
    return n;
}
uint64_t Utils::GetTensorNumel(const Tensor &tensor) { return GetTensorNumel(tensor.desc); }

uint64_t Utils::GetTensorSize(const TensorDesc &desc)
{
    uint64_t item = 0;
    switch (desc.dtype) {
        case ACL_DT_UNDEFINED:
        case ACL_BOOL:
        case ACL_INT8:
        case ACL_UINT8:
            item = 1;
            break;
        case ACL_FLOAT16:
        case ACL_BF16:
        case ACL_INT16:
        case ACL_UINT16:
            item = 2;
            break;
        case ACL_FLOAT:
        case ACL_INT32:
        case ACL_UINT32:
            item = 4;
            break;
        case ACL_INT64:
        case ACL_UINT64:
        case ACL_DOUBLE:
            item = 8;
            break;
        default:
            return 0;
    }
    const uint64_t n = GetTensorNumel(desc);
    if (n == 0 || std::numeric_limits<uint64_t>::max() / n < item) {
        return 0;
    }
    return n * item;
}
uint64_t Utils::GetTensorSize(const Tensor &tensor) { return GetTensorSize(tensor.desc); }

void Utils::QuantParamConvert(const float *src, uint64_t *dest, uint64_t itemCount)
{
    if (src == nullptr || dest == nullptr) {
        return;
    }
    for (uint64_t i = 0; i < itemCount; ++i) {
        uint32_t bits;
        std::memcpy(&bits, &src[i], sizeof(bits));
        dest[i] = bits;
    }
}

Status Utils::SetLogLevel(const atb::LogLevel level)
{
    g_logLevel = static_cast<int>(level);
    return NO_ERROR;
}
Status Utils::ResetLogLevel()
{
    g_logLevel = LogLevelFromEnv();
    return NO_ERROR;
}

// ---------------------------------------------------------------------------------- Context
Status ContextImpl::SetExecuteStream(aclrtStream stream)
{
    streams_[0] = stream;
    return NO_ERROR;
}
aclrtStream ContextImpl::GetExecuteStream() const { return streams_[0]; }
Status ContextImpl::SetAsyncTilingCopyStatus(bool enable)
{
    asyncTilingCopy_ = enable;
    return NO_ERROR;
}
bool ContextImpl::GetAsyncTilingCopyStatus() const { return asyncTilingCopy_; }
Status ContextImpl::SetExecuteStreams(const std::vector<aclrtStream> &streams)
{
    if (streams.empty()) {
        return ERROR_INVALID_PARAM;
    }
    streams_ = streams;
    return NO_ERROR;
}
std::vector<aclrtStream> ContextImpl::GetExecuteStreams() { return streams_; }
namespace {
thread_local ExecuteType t_executeType = EXECUTE_NORMAL;
}
Status ContextImpl::SetExecuteType(ExecuteType type)
{
    t_executeType = type;
    return NO_ERROR;
}
ExecuteType ContextImpl::GetExecuteType() { return t_executeType; }
Status ContextImpl::SetLaunchMode(LaunchMode mode)
{
    mode_ = mode;
    return NO_ERROR;
}
LaunchMode ContextImpl::GetLaunchMode() { return mode_; }

Status CreateContext(Context **context)
{
    if (context == nullptr) {
        return ERROR_INVALID_PARAM;
    }
    *context = new (std::nothrow) ContextImpl();
    return *context == nullptr ? ERROR_OUT_OF_HOST_MEMORY : NO_ERROR;
}

Status DestroyContext(Context *context)
{
    delete context;
    return NO_ERROR;
}

Status DestroyOperation(Operation *operation)
{
    delete operation;
    return NO_ERROR;
}

// ---------------------------------------------------------------------------- OperationBase
bool TensorDescEqual(const TensorDesc &a, const TensorDesc &b)
{
    if (a.dtype != b.dtype || a.format != b.format || a.shape.dimNum != b.shape.dimNum) {
        return false;
    }
    for (uint64_t i = 0; i < a.shape.dimNum; ++i) {
        if (a.shape.dims[i] != b.shape.dims[i]) {
            return false;
        }
    }
    return true;
}

bool RsvIsZero(const uint8_t *rsv, size_t n)
{
    for (size_t i = 0; i < n; ++i) {
        if (rsv[i] != 0) {
            return false;
        }
    }
    return true;
}

namespace {
constexpr uint64_t kMaxTensorSize = 256ull << 30;

Status CheckTensorShape(const TensorDesc &desc)
{
    if (desc.shape.dimNum == 0 || desc.shape.dimNum > MAX_DIM) {
        return ERROR_INVALID_TENSOR_DIM;
    }
    const uint64_t size = Utils::GetTensorSize(desc);
    if (size == 0 || size > kMaxTensorSize) {
        return ERROR_INVALID_TENSOR_SIZE;
    }
    return NO_ERROR;
}
} // namespace

Status OperationBase::InferShape(const SVector<TensorDesc> &inTensorDescs, SVector<TensorDesc> &outTensorDescs) const
{
    try {
        if (inTensorDescs.size() != GetInputNum()) {
            return ERROR_INVALID_IN_TENSOR_NUM;
        }
        for (size_t i = 0; i < inTensorDescs.size(); ++i) {
            Status st = CheckTensorShape(inTensorDescs.at(i));
            if (st != NO_ERROR) {
                return st;
            }
        }
        Status st = InferShapeCheckImpl(inTensorDescs);
        if (st != NO_ERROR) {
            return st;
        }
        outTensorDescs.resize(GetOutputNum());
        return InferShapeImpl(inTensorDescs, outTensorDescs);
    } catch (...) {
        return ERROR_INTERNAL_ERROR;
    }
}

bool OperationBase::CheckIniMatch(const VariantPack &variantPack) const
{
    const size_t nIn = variantPack.inTensors.size(), nOut = variantPack.outTensors.size();
    for (const DtypeComb &comb : DtypeCombs()) {
        if (comb.size() != nIn + nOut) {
            continue;
        }
        bool ok = true;
        for (size_t i = 0; i < nIn + nOut && ok; ++i) {
            const Tensor &t = i < nIn ? variantPack.inTensors.at(i) : variantPack.outTensors.at(i - nIn);
            ok = t.desc.dtype == comb[i] && t.desc.format == ACL_FORMAT_ND;
        }
        if (ok) {
            return true;
        }
    }
    return false;
}

Status OperationBase::CheckVariantPack(const VariantPack &variantPack) const
{
    if (variantPack.inTensors.size() != GetInputNum() || variantPack.outTensors.size() != GetOutputNum()) {
        ATB_B200_LOG(ERROR, name_ + ": tensor count differs from GetInputNum/GetOutputNum");
        return ERROR_INVALID_IN_TENSOR_NUM;
    }
    for (size_t i = 0; i < variantPack.inTensors.size(); ++i) {
        Status st = CheckTensorShape(variantPack.inTensors.at(i).desc);
        if (st != NO_ERROR) {
            return st;
        }
    }
    for (size_t i = 0; i < variantPack.outTensors.size(); ++i) {
        Status st = CheckTensorShape(variantPack.outTensors.at(i).desc);
        if (st != NO_ERROR) {
            return st;
        }
    }
    if (!CheckIniMatch(variantPack)) {
        ATB_B200_LOG(ERROR, name_ + ": tensor dtype/format combination is not supported");
        return ERROR_INVALID_TENSOR_INI_MATCH;
    }
    return NO_ERROR;
}

namespace {
// A named range around Setup / Execute for timeline tools (NVTX is header-only and costs a few nanoseconds when no tool
// is attached).
struct TraceRange {
    explicit TraceRange(const std::string &name) { nvtxRangePushA(name.c_str()); }
    ~TraceRange() { nvtxRangePop(); }
};

// ATB_STREAM_SYNC_EVERY_OPERATION_ENABLE=1, as in the reference (src/atb/utils/config.cpp:36,
// src/atb/operation/operation_base.cpp:1059-1062): wait for the execute stream after every Execute, so that a device
// failure is reported by the operation that caused it.  Read at every call: a test can switch it.
// ATB_SAVE_TENSOR_DIR=<dir>: every Execute writes its input and output tensors before and after the launch, for parity
// triage, as the reference's Probe hooks do (src/atb/runner/runner.cpp:102-135, store_util.cpp:57-73):
//   <dir>/<execute count>_<operation name>/{before,after}/{intensor,outtensor}<i>.bin
// A file is one text line "dtype=<aclDataType> format=<aclFormat> dims=<d0,d1,..> bytes=<n>" and then the n raw bytes.
// The stream is synchronised around the launch while this is on.
void MakeDirs(const std::string &path)
{
    for (size_t i = 1; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            ::mkdir(path.substr(0, i).c_str(), 0755);
        }
    }
}

void SaveTensors(const SVector<Tensor> &tensors, const std::string &dir, const char *stem)
{
    std::vector<unsigned char> host;
    for (size_t i = 0; i < tensors.size(); ++i) {
        const Tensor &t = tensors.at(i);
        const unsigned char *src = static_cast<const unsigned char *>(t.hostData);
        if (t.deviceData != nullptr) {
            host.resize(t.dataSize);
            if (cudaMemcpy(host.data(), t.deviceData, t.dataSize, cudaMemcpyDeviceToHost) != cudaSuccess) {
                cudaGetLastError();
                continue;
            }
            src = host.data();
        }
        if (src == nullptr) {
            continue;
        }
        FILE *f = std::fopen((dir + "/" + stem + std::to_string(i) + ".bin").c_str(), "wb");
        if (f == nullptr) {
            continue;
        }
        std::string dims;
        for (uint64_t k = 0; k < t.desc.shape.dimNum; ++k) {
            dims += (k ? "," : "") + std::to_string(t.desc.shape.dims[k]);
        }
        std::fprintf(f, "dtype=%d format=%d dims=%s bytes=%llu\n", static_cast<int>(t.desc.dtype), static_cast<int>(t.desc.format),
                     dims.c_str(), static_cast<unsigned long long>(t.dataSize));
        std::fwrite(src, 1, t.dataSize, f);
        std::fclose(f);
    }
}

void SaveVariantPack(const VariantPack &pack, cudaStream_t stream, const std::string &dir)
{
    cudaStreamSynchronize(stream);
    MakeDirs(dir);
    SaveTensors(pack.inTensors, dir, "intensor");
    SaveTensors(pack.outTensors, dir, "outtensor");
}

bool StreamSyncEveryOperation()
{
    const char *e = std::getenv("ATB_STREAM_SYNC_EVERY_OPERATION_ENABLE");
    return e != nullptr && std::strcmp(e, "1") == 0;
}
} // namespace

Status OperationBase::Setup(const VariantPack &variantPack, uint64_t &workspaceSize, Context *context)
{
    TraceRange range(name_ + "::Setup");
    setupSuccess_ = false;
    try {
        Status st = CheckVariantPack(variantPack);
        if (st != NO_ERROR) {
            return st;
        }
        st = SetupCheckImpl(variantPack.inTensors, variantPack.outTensors);
        if (st != NO_ERROR) {
            return st;
        }
        if (context == nullptr || dynamic_cast<ContextImpl *>(context) == nullptr) {
            ATB_B200_LOG(ERROR, name_ + ": context is null or was not made by CreateContext");
            return ERROR_INVALID_PARAM;
        }
        uint64_t ws = 0;
        st = PlanImpl(variantPack, ws);
        if (st != NO_ERROR) {
            return st;
        }
        context_ = context;
        workspaceSize_ = ws;
        workspaceSize = ws;
        setupInDescs_.clear();
        setupOutDescs_.clear();
        for (size_t i = 0; i < variantPack.inTensors.size(); ++i) {
            setupInDescs_.push_back(variantPack.inTensors.at(i).desc);
        }
        for (size_t i = 0; i < variantPack.outTensors.size(); ++i) {
            setupOutDescs_.push_back(variantPack.outTensors.at(i).desc);
        }
        setupSuccess_ = true;
        if (context->GetExecuteStream() != nullptr) {
            AfterPlanImpl(context->GetExecuteStream());
        }
        return NO_ERROR;
    } catch (...) {
        return ERROR_OUT_OF_HOST_MEMORY;
    }
}

Status OperationBase::Execute(const VariantPack &variantPack, uint8_t *workspace, uint64_t workspaceSize,
                              Context *context)
{
    TraceRange range(name_ + "::Execute");
    try {
        if (!setupSuccess_) {
            ATB_B200_LOG(ERROR, name_ + ": Execute without a successful Setup");
            return ERROR_INVALID_PARAM;
        }
        if (context == nullptr || context != context_) {
            return ERROR_INVALID_PARAM;
        }
        aclrtStream stream = context->GetExecuteStream();
        if (stream == nullptr) {
            ATB_B200_LOG(ERROR, name_ + ": the context has no execute stream");
            return ERROR_INVALID_PARAM;
        }
        if (workspaceSize < workspaceSize_ || (workspaceSize_ != 0 && workspace == nullptr)) {
            return ERROR_INVALID_PARAM;
        }
        if (variantPack.inTensors.size() != setupInDescs_.size() ||
            variantPack.outTensors.size() != setupOutDescs_.size()) {
            return ERROR_INVALID_PARAM;
        }
        for (size_t i = 0; i < variantPack.inTensors.size(); ++i) {
            const Tensor &t = variantPack.inTensors.at(i);
            if (t.dataSize != Utils::GetTensorSize(setupInDescs_[i]) || (!t.deviceData && !t.hostData)) {
                return ERROR_INVALID_PARAM;
            }
        }
        for (size_t i = 0; i < variantPack.outTensors.size(); ++i) {
            const Tensor &t = variantPack.outTensors.at(i);
            if (t.dataSize != Utils::GetTensorSize(setupOutDescs_[i]) || (!t.deviceData && !t.hostData)) {
                return ERROR_INVALID_PARAM;
            }
        }
        const char *dumpDir = std::getenv("ATB_SAVE_TENSOR_DIR");
        std::string dumpBase;
        if (dumpDir != nullptr && dumpDir[0] != '\0') {
            dumpBase = std::string(dumpDir) + "/" + std::to_string(executeCount_) + "_" + name_;
            SaveVariantPack(variantPack, static_cast<cudaStream_t>(stream), dumpBase + "/before");
        }
        const Status st = LaunchImpl(variantPack, workspace, workspaceSize, stream);
        ++executeCount_;
        if (!dumpBase.empty()) {
            SaveVariantPack(variantPack, static_cast<cudaStream_t>(stream), dumpBase + "/after");
        }
        if (StreamSyncEveryOperation()) {
            const cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
            if (e != cudaSuccess) {
                ATB_B200_LOG(ERROR, name_ + ": stream sync fail: " + cudaGetErrorString(e));
            }
        }
        return st;
    } catch (...) {
        return ERROR_RT_FAIL;
    }
}

} // namespace atb
