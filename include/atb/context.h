// Execution context: owns nothing but the stream handle(s) the caller sets and a small pinned
// staging area for plan uploads.  Interface of include/atb/context.h:57-194 of the reference.
#ifndef ATB_CONTEXT_H
#define ATB_CONTEXT_H
#include <vector>
#include <acl/acl.h>
#include "atb/types.h"

namespace atb {
enum ExecuteType : int { EXECUTE_NORMAL = 0, EXECUTE_PRELAUNCH, EXECUTE_LAUNCH };
enum LaunchMode : int { KERNEL_LAUNCH_MODE = 0, GRAPH_LAUNCH_MODE };

class Context {
public:
    Context() = default;
    virtual ~Context() = default;
    virtual Status SetExecuteStream(aclrtStream stream) = 0;
    virtual aclrtStream GetExecuteStream() const = 0;
    virtual Status SetAsyncTilingCopyStatus(bool enable) = 0;
    virtual bool GetAsyncTilingCopyStatus() const = 0;
    virtual Status SetExecuteStreams(const std::vector<aclrtStream> &streams) = 0;
    virtual std::vector<aclrtStream> GetExecuteStreams() = 0;
    virtual Status SetExecuteType(ExecuteType type) = 0;
    virtual ExecuteType GetExecuteType() = 0;
    virtual Status SetLaunchMode(LaunchMode mode) = 0;
    virtual LaunchMode GetLaunchMode() = 0;
};

Status CreateContext(Context **context);
Status DestroyContext(Context *context);
} // namespace atb
#endif
