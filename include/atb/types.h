// Data types of the operator API: Status/ErrorType, Dims, TensorDesc, Tensor, VariantPack.
// Mirrors include/atb/types.h:29-141 of the reference (same names, field order and error codes);
// graph-composition types (Node, GraphParam) are outside the decode path and not provided.
#ifndef ATB_TYPES_H
#define ATB_TYPES_H
#include <cstdint>
#include <string>
#include <acl/acl.h>
#include "atb/svector.h"

namespace atb {
using Status = int32_t;
constexpr uint32_t MAX_DIM = 8;

enum ErrorType : int {
    NO_ERROR = 0,
    ERROR_INVALID_PARAM,
    ERROR_INVALID_GRAPH,
    ERROR_INTERNAL_ERROR,
    ERROR_RT_FAIL,
    ERROR_INVALID_IN_TENSOR_NUM,
    ERROR_INVALID_TENSOR_DTYPE,
    ERROR_INVALID_TENSOR_FORMAT,
    ERROR_INVALID_TENSOR_DIM,
    ERROR_INVALID_TENSOR_SIZE,
    ERROR_OPERATION_NULL_RUNNER,
    ERROR_GRAPH_INFERSHAPE_FUNC_FAIL,
    ERROR_CANN_ERROR,
    ERROR_INVALID_TENSOR_INI_MATCH,
    ERROR_INVALID_TENSOR_ADDR,
    ERROR_INVALID_TENSOR_NUM,
    ERROR_INVALID_TENSOR_DIM_NUM,
    ERROR_INVALID_SINGLE_OPERATION_PARAM,
    ERROR_GRAPH_NODE_RESHAPE_FUNC_FAIL,
    ERROR_INVALID_GRAPH_NODE_CHUNK,
    ERROR_INVALID_CONTEXT_ADDR,
    ERROR_INVALID_STREAM,
    ERROR_INVALID_WORKSPACE_SIZE,
    ERROR_INVALID_WORKSPACE_ADDR,
    ERROR_INVALID_OPERATION_ADDR,
    ERROR_HCCL_FAIL,
    ERROR_OUT_OF_DEVICE_MEMORY,
    ERROR_OUT_OF_HOST_MEMORY,
    ERROR_COMM_EMPTY,
    ERROR_COPY_HOST_MEMORY_FAIL
};

enum class LogLevel : int { DEBUG = 0, INFO, WARN, ERROR, NONE };

struct Dims {
    int64_t dims[MAX_DIM];
    uint64_t dimNum = 0;
};

struct TensorDesc {
    aclDataType dtype = ACL_DT_UNDEFINED;
    aclFormat format = ACL_FORMAT_UNDEFINED;
    Dims shape;
};

// deviceData is GPU memory (HBM); hostData, when set, is read during Setup only.
struct Tensor {
    TensorDesc desc;
    void *deviceData = nullptr;
    void *hostData = nullptr;
    uint64_t dataSize = 0;
};

struct VariantPack {
    SVector<Tensor> inTensors;
    SVector<Tensor> outTensors;
};
} // namespace atb
#endif
