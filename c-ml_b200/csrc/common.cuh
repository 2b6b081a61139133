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

// Activation "digits" consumed by the integer-dot GEMV: per 32-element block of x a record of
// kXqWords 32-bit words: three planes of 8 words (signed 7-bit digits d0, d1, d2 of the 21-bit
// block-fixed-point value, 4 per word), the block scale (fp32 bits), the block sum (int32), 2 pad.
constexpr int kXqWords = 28;
constexpr int kXqFull = (1 << 20) - 1;

// One warp = one block: lane l holds element l. Writes the block's record at dst.
__device__ __forceinline__ void xq_emit_warp(float v, int lane, uint32_t* dst) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float inv = amax > 0.f ? (float)kXqFull / amax : 0.f;
    int X = __float2int_rn(v * inv);
    X = max(-kXqFull, min(kXqFull, X));
    const int d2 = ((X + 64) & 127) - 64;
    const int X1 = (X - d2) >> 7;
    const int d1 = ((X1 + 64) & 127) - 64;
    const int d0 = (X1 - d1) >> 7;
    int xsum = X;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) xsum += __shfl_xor_sync(0xffffffffu, xsum, o);
    uint32_t b0 = (uint32_t)(d0 & 0xFF) << (8 * (lane & 3)), b1 = (uint32_t)(d1 & 0xFF) << (8 * (lane & 3)),
             b2 = (uint32_t)(d2 & 0xFF) << (8 * (lane & 3));
#pragma unroll
    for (int o = 1; o < 4; o <<= 1) {
        b0 |= __shfl_xor_sync(0xffffffffu, b0, o);
        b1 |= __shfl_xor_sync(0xffffffffu, b1, o);
        b2 |= __shfl_xor_sync(0xffffffffu, b2, o);
    }
    if ((lane & 3) == 0) {
        dst[lane >> 2] = b0;
        dst[8 + (lane >> 2)] = b1;
        dst[16 + (lane >> 2)] = b2;
    }
    if (lane == 0) {
        dst[24] = __float_as_uint(amax / (float)kXqFull);
        dst[25] = (uint32_t)xsum;
    }
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
