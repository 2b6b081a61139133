// Shared helpers for the sm_100a kernels behind the cmlb200 C-ABI.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "cmlb200.h"

extern "C" void cmlb200_set_error_(const char* fmt, ...);

#define CMLB_CUDA(call)                                                                      \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess) {                                                             \
            cmlb200_set_error_("%s:%d: %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
            return CMLB200_ECUDA;                                                            \
        }                                                                                    \
    } while (0)

#define CMLB_REQUIRE(cond, ...)                \
    do {                                       \
        if (!(cond)) {                         \
            cmlb200_set_error_(__VA_ARGS__);   \
            return CMLB200_EINVAL;             \
        }                                      \
    } while (0)

#define CMLB_LAUNCH_CHECK() CMLB_CUDA(cudaGetLastError())

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// The 16 NF4 code values of C-ML (src/core/quantization.c:195-198).
__device__ __constant__ float kNF4[16] = {-1.0f, -0.6962f, -0.5251f, -0.3949f, -0.2844f, -0.1848f,
                                          -0.0911f, 0.0f, 0.0796f, 0.1609f, 0.2461f, 0.3379f,
                                          0.4407f, 0.5626f, 0.7230f, 1.0f};

// fp16 bits -> fp32 exactly as C-ML's fp16_to_fp32 (src/core/gguf_quant.c:14-58) does it:
// IEEE-exact for normals, zeros, infinities and NaNs; a SUBNORMAL half comes out at half its
// IEEE value, because the reference counts one mantissa shift too many (:35-36). The IEEE
// widening of a subnormal half is a normal fp32 number, so the halving below is exact.
__device__ __forceinline__ float cml_half_to_float(uint16_t h) {
    const float f = __half2float(__ushort_as_half(h));
    return ((h & 0x7C00u) == 0) ? f * 0.5f : f;
}

static inline int cmlb_num_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}
