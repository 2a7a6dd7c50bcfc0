#include "tma_encode.h"
#include <cuda_runtime.h>
#include <mutex>

namespace atb_b200 {

TmaEncodeFn tma_encode_fn()
{
    static TmaEncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<TmaEncodeFn>(p);
        }
    });
    return fn;
}

} // namespace atb_b200
