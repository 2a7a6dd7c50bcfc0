// Small device helpers of the operator layer: conversion of descale tensors given in the
// int64-packed-fp32 or fp16 encodings into plain fp32, and device scratch allocation.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {
__global__ void convert_scales_kernel(const void *src, int kind, float *dst, uint64_t n)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) {
        return;
    }
    if (kind == 1) {
        const uint64_t w = static_cast<const uint64_t *>(src)[i];
        dst[i] = __uint_as_float((uint32_t)(w & 0xffffffffu));
    } else {
        dst[i] = __half2float(static_cast<const __half *>(src)[i]);
    }
}
} // namespace

extern "C" int atb_b200_internal_convert_scales(const void *src, int src_kind, float *dst, uint64_t n, void *stream)
{
    if (n == 0) {
        return 0;
    }
    convert_scales_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, src_kind, dst, n);
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int atb_b200_internal_device_alloc(void **p, uint64_t bytes)
{
    return cudaMalloc(p, bytes) == cudaSuccess ? 0 : 1;
}

extern "C" void atb_b200_internal_device_free(void *p) { cudaFree(p); }
