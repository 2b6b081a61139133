// Per-tensor affine 8-bit quantisation (C-ML: src/core/quantization.c:8-192):
//   q = clamp(round(v / scale) + zero_point),  v' = (q - zero_point) * scale
// with round = half away from zero (roundf), the division and the two dequantisation operations in
// IEEE fp32, so the bytes and floats equal those of C-ML's scalar loops. HBM-bound element-wise
// kernels over grid-stride loops; the range scan reduces per warp and CTA, then one CTA combines
// the partial ranges.
#include <float.h>
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ void warp_minmax(float& lo, float& hi) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
}
__device__ __forceinline__ void block_minmax(float& lo, float& hi) {
    __shared__ float slo[THREADS / 32], shi[THREADS / 32];
    warp_minmax(lo, hi);
    if ((threadIdx.x & 31) == 0) { slo[threadIdx.x >> 5] = lo; shi[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        lo = threadIdx.x < THREADS / 32 ? slo[threadIdx.x] : FLT_MAX;
        hi = threadIdx.x < THREADS / 32 ? shi[threadIdx.x] : -FLT_MAX;
        warp_minmax(lo, hi);
    }
}

// partial[2 * b] / partial[2 * b + 1] = min / max of the elements CTA b scanned (FLT_MAX / -FLT_MAX when none)
__global__ void __launch_bounds__(THREADS) range_partial_kernel(const float* __restrict__ x, size_t n, float* __restrict__ partial) {
    float lo = FLT_MAX, hi = -FLT_MAX;
    const size_t stride = (size_t)gridDim.x * THREADS;
    for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < n; i += stride) {
        const float v = x[i];
        if (v < lo) lo = v;                 // the comparisons of src/core/quantization.c:18-22: a NaN never replaces a bound
        if (v > hi) hi = v;
    }
    block_minmax(lo, hi);
    if (threadIdx.x == 0) { partial[2 * blockIdx.x] = lo; partial[2 * blockIdx.x + 1] = hi; }
}
__global__ void __launch_bounds__(THREADS) range_final_kernel(const float* __restrict__ partial, int parts, float* __restrict__ out) {
    float lo = FLT_MAX, hi = -FLT_MAX;
    for (int i = threadIdx.x; i < parts; i += THREADS) {
        lo = fminf(lo, partial[2 * i]);
        hi = fmaxf(hi, partial[2 * i + 1]);
    }
    block_minmax(lo, hi);
    if (threadIdx.x == 0) { out[0] = lo; out[1] = hi; }
}

template <bool UNSIGNED>
__global__ void __launch_bounds__(THREADS) quantize8_kernel(const float* __restrict__ x, size_t n, float scale, int zero_point,
                                                            uint8_t* __restrict__ q) {
    const int lo = UNSIGNED ? 0 : -128, hi = UNSIGNED ? 255 : 127;
    const size_t stride = (size_t)gridDim.x * THREADS;
    for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < n; i += stride) {
        const float r = roundf(__fdiv_rn(x[i], scale));
        // Where the quotient leaves the int32 range (or is NaN) C-ML's cast is undefined; the compiled
        // x86 reference yields INT_MIN there and wraps the zero-point addition, and so does this.
        const int c = (r >= -2147483648.0f && r < 2147483648.0f) ? __float2int_rz(r) : (int)0x80000000;
        int v = (int)((unsigned)c + (unsigned)zero_point);
        v = v < lo ? lo : (v > hi ? hi : v);
        q[i] = (uint8_t)v;
    }
}

template <bool UNSIGNED>
__global__ void __launch_bounds__(THREADS) dequantize8_kernel(const uint8_t* __restrict__ q, size_t n, float scale, int zero_point,
                                                              float* __restrict__ out) {
    const float zp = (float)zero_point;
    const size_t stride = (size_t)gridDim.x * THREADS;
    for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < n; i += stride) {
        const float v = UNSIGNED ? (float)q[i] : (float)(int8_t)q[i];
        out[i] = __fmul_rn(__fsub_rn(v, zp), scale);
    }
}

int grid_for(size_t n) {
    size_t g = (n + THREADS - 1) / THREADS;
    const size_t cap = (size_t)cmlb_num_sms() * 8;
    return (int)(g > cap ? cap : (g ? g : 1));
}

}  // namespace

// min and max of x[0..n) into d_out[0..1]; d_scratch holds 2 * cmlb200_range_scratch_floats() floats.
extern "C" size_t cmlb200_range_scratch_floats(void) { return 2 * (size_t)cmlb_num_sms() * 8; }
extern "C" int cmlb200_range_f32(const float* d_x, size_t n, float* d_scratch, float* d_out, void* stream) {
    CMLB_REQUIRE(d_x && d_scratch && d_out && n > 0, "cmlb200_range_f32: bad argument");
    const int g = grid_for(n);
    range_partial_kernel<<<g, THREADS, 0, as_stream(stream)>>>(d_x, n, d_scratch);
    CMLB_LAUNCH_CHECK();
    range_final_kernel<<<1, THREADS, 0, as_stream(stream)>>>(d_scratch, g, d_out);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_quantize_8bit(const float* d_x, size_t n, float scale, int zero_point, int is_unsigned, void* d_q, void* stream) {
    CMLB_REQUIRE(d_x && d_q && n > 0, "cmlb200_quantize_8bit: bad argument");
    if (is_unsigned) quantize8_kernel<true><<<grid_for(n), THREADS, 0, as_stream(stream)>>>(d_x, n, scale, zero_point, (uint8_t*)d_q);
    else quantize8_kernel<false><<<grid_for(n), THREADS, 0, as_stream(stream)>>>(d_x, n, scale, zero_point, (uint8_t*)d_q);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_dequantize_8bit(const void* d_q, size_t n, float scale, int zero_point, int is_unsigned, float* d_out, void* stream) {
    CMLB_REQUIRE(d_q && d_out && n > 0, "cmlb200_dequantize_8bit: bad argument");
    if (is_unsigned) dequantize8_kernel<true><<<grid_for(n), THREADS, 0, as_stream(stream)>>>((const uint8_t*)d_q, n, scale, zero_point, d_out);
    else dequantize8_kernel<false><<<grid_for(n), THREADS, 0, as_stream(stream)>>>((const uint8_t*)d_q, n, scale, zero_point, d_out);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
