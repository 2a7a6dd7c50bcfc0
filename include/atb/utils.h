// Tensor size helpers and log level control (include/atb/utils.h:25-98 of the reference).
#ifndef ATB_UTILS_H
#define ATB_UTILS_H
#include <cstdint>
#include <string>
#include "atb/types.h"

namespace atb {
class Utils {
public:
    static std::string GetAtbVersion();
    static uint64_t GetTensorSize(const Tensor &tensor);
    static uint64_t GetTensorSize(const TensorDesc &tensorDesc);
    static uint64_t GetTensorNumel(const Tensor &tensor);
    static uint64_t GetTensorNumel(const TensorDesc &tensorDesc);
    // Packs fp32 scales into the low 32 bits of uint64 words (the int64 descale encoding).
    static void QuantParamConvert(const float *src, uint64_t *dest, uint64_t itemCount);
    static Status SetLogLevel(const atb::LogLevel atbLogLevel);
    static Status ResetLogLevel();
};
} // namespace atb
#endif
