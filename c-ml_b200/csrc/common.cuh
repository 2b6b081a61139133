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
// kXqWords 32-bit words: three planes of 8 words (signed 8-bit digits d0, d1, d2 of the 24-bit
// block-fixed-point value X = d0*65536 + d1*256 + d2, 4 elements per word), the block scale
// (fp32 bits) and 3 pad words (records stay 16-byte aligned; the 28-word stride is
// bank-conflict-free for 128-bit shared-memory reads by consecutive lanes).
constexpr int kXqWords = 28;
constexpr int kXqFull = 127 * 65536 + 127 * 256 + 127;      // largest |X| whose balanced digits all fit int8

// X = d0*65536 + d1*256 + d2 with d1, d2 in [-128, 127]; |X| <= kXqFull keeps d0 in [-127, 127].
__device__ __forceinline__ void xq_split(int X, int& d0, int& d1, int& d2) {
    d2 = ((X + 128) & 255) - 128;
    const int X1 = (X - d2) >> 8;
    d1 = ((X1 + 128) & 255) - 128;
    d0 = (X1 - d1) >> 8;
}

// One warp = one block: lane l holds element l. Writes the block's record at dst.
__device__ __forceinline__ void xq_emit_warp(float v, int lane, uint32_t* dst) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float inv = amax > 0.f ? (float)kXqFull / amax : 0.f;
    int X = __float2int_rn(v * inv);
    X = max(-kXqFull, min(kXqFull, X));
    int d0, d1, d2;
    xq_split(X, d0, d1, d2);
    const int sh = 8 * (lane & 3);
    uint32_t b0 = (uint32_t)(d0 & 0xFF) << sh, b1 = (uint32_t)(d1 & 0xFF) << sh, b2 = (uint32_t)(d2 & 0xFF) << sh;
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
    if (lane == 0) dst[24] = __float_as_uint(amax / (float)kXqFull);
}

// 8 lanes (sub = 0..7; gmask = their lane mask) turn the 32 values of one block, 4 per lane, into
// its record at dst (global or shared memory).
__device__ __forceinline__ void xq_emit_oct(const float (&e)[4], int sub, unsigned gmask, uint32_t* dst) {
    float amax = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o));
    const float inv = amax > 0.f ? (float)kXqFull / amax : 0.f;
    uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int X = __float2int_rn(e[i] * inv);
        X = max(-kXqFull, min(kXqFull, X));
        int d0, d1, d2;
        xq_split(X, d0, d1, d2);
        w0 |= (uint32_t)(d0 & 0xFF) << (8 * i);
        w1 |= (uint32_t)(d1 & 0xFF) << (8 * i);
        w2 |= (uint32_t)(d2 & 0xFF) << (8 * i);
    }
    dst[sub] = w0;
    dst[8 + sub] = w1;
    dst[16 + sub] = w2;
    if (sub == 0) dst[24] = __float_as_uint(amax / (float)kXqFull);
}

// Workspace of the tensor-parallel all-reduce over peer memory (one per rank, mapped into every
// other rank through CUDA IPC). Two independent channels: 0 = the stand-alone kernel
// (tp_allreduce.cu, kTpCtas slices), 1 = the epilogue of the decode GEMV (gemv_mma.cu, one slice
// per CTA of its grid). Per channel: a sequence counter per slice, a flag word per (peer, slice;
// channel 0 only) and two alternating inboxes with room for max_floats values from each of 8
// ranks (channel 1 stores 8-byte (value, sequence) packets there, so it holds max_floats / 2).
//   +0      u32 seq0[16]      +64    u32 status
//   +1024   u32 flags0[8][16]
//   +2048   u32 seq1[192]     +4096  u32 flags1[8][192]
//   +16384  float inbox[channel][parity][from][max_floats]
constexpr int kTpMaxRanks = 8;
constexpr int kTpCtas = 16;
constexpr int kTpGemvSlices = 192;
constexpr size_t kTpHeaderBytes = 16384;
struct TpPeers {
    uint8_t* ws[kTpMaxRanks];        // every rank's workspace as mapped in this process (ws[rank] = own)
    float* h;                        // the residual the sum is added to (GEMV epilogue channel)
    size_t max_floats;
    int tp, rank;                    // tp == 0: no all-reduce
    int spin_limit;                  // polls of a peer's flag or packet before the launch gives up
};
__device__ __forceinline__ uint32_t* tpws_seq(uint8_t* ws, int ch) { return reinterpret_cast<uint32_t*>(ws + (ch ? 2048 : 0)); }
__device__ __forceinline__ uint32_t* tpws_status(uint8_t* ws) { return reinterpret_cast<uint32_t*>(ws + 64); }
__device__ __forceinline__ uint32_t* tpws_flags(uint8_t* ws, int ch, int from) {
    return reinterpret_cast<uint32_t*>(ws + (ch ? 4096 : 1024)) + from * (ch ? kTpGemvSlices : kTpCtas);
}
__device__ __forceinline__ float* tpws_inbox(uint8_t* ws, int ch, int parity, int from, size_t max_floats) {
    return reinterpret_cast<float*>(ws + kTpHeaderBytes) + (((size_t)ch * 2 + parity) * kTpMaxRanks + from) * max_floats;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
constexpr int kTpSpinLimit = 1 << 22;
// The limit in force for the next launches (cmlb200_set_wait_limit, or CMLB200_WAIT_LIMIT in the
// environment, read once; kTpSpinLimit otherwise). Defined in tp_allreduce.cu.
int cmlb_tp_spin_limit();
// (value, sequence number) packets: one 8-byte store carries a result and the proof that it
// belongs to this all-reduce, so the receiver polls the data words themselves and no fence or
// separate flag is needed between ranks.
__device__ __forceinline__ void st_packet_sys(uint2* p, float v, uint32_t seq) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_packet_sys(const uint2* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

constexpr int kMaxDevices = 16;
// Index of the current device (0 when the query fails); keys every per-device cache below and
// in the launchers: function attributes, SM counts and scratch buffers belong to one device.
static inline int cmlb_device_index() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return dev;
}
static inline int cmlb_num_sms() {
    static int sms[kMaxDevices] = {};
    const int dev = cmlb_device_index();
    if (!sms[dev]) {
        if (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0) sms[dev] = 148;
    }
    return sms[dev];
}
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the current device only: `done`
// (one array per kernel instantiation, owned by the caller) remembers the largest size set on each.
template <typename Kern>
static inline cudaError_t cmlb_ensure_smem(Kern kern, size_t bytes, size_t (&done)[kMaxDevices]) {
    const int dev = cmlb_device_index();
    if (bytes <= done[dev]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) done[dev] = bytes;
    return e;
}
