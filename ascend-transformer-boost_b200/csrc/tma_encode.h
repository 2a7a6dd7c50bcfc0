// cuTensorMapEncodeTiled, looked up once through the runtime (the library links no libcuda).
#ifndef ATB_B200_TMA_ENCODE_H
#define ATB_B200_TMA_ENCODE_H
#include <cuda.h>

namespace atb_b200 {

using TmaEncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// nullptr when the driver does not export the entry point.
TmaEncodeFn tma_encode_fn();

} // namespace atb_b200
#endif
