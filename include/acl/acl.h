// Minimal stand-in for the CANN `acl/acl.h` names that ATB's public headers use
// (include/atb/types.h:16, include/atb/context.h:13 of the reference include <acl/acl.h>).
// On a CUDA box the stream handle is a cudaStream_t; the enum values are the public CANN ones so
// that serialized descriptors keep their meaning.
#ifndef ATB_B200_ACL_SHIM_H
#define ATB_B200_ACL_SHIM_H
#include <cstddef>
#include <cstdint>

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
    ACL_BF16 = 27,
} aclDataType;

typedef enum {
    ACL_FORMAT_UNDEFINED = -1,
    ACL_FORMAT_NCHW = 0,
    ACL_FORMAT_NHWC = 1,
    ACL_FORMAT_ND = 2,
    ACL_FORMAT_NC1HWC0 = 3,
    ACL_FORMAT_FRACTAL_Z = 4,
    ACL_FORMAT_FRACTAL_NZ = 29,
} aclFormat;

// The execute stream.  Holds a cudaStream_t.
typedef void *aclrtStream;

#endif
