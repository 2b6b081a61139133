// Dequantisation to fp32, bit-exact with C-ML's CPU routines: one IEEE fp32
// multiply per element, integer arithmetic before it, no fast-math, no FTZ.
//   Q8_0: y = (float)q * d              (src/core/gguf_quant.c:114-125)
//   Q4_0: y = (float)(nibble - 8) * d   (src/core/gguf_quant.c:66-82)
//   NF4 : y = TABLE[idx] * absmax       (src/core/quantization.c:349-366)
// fp16 scales widen through cml_half_to_float (common.cuh), which reproduces C-ML's
// fp16_to_fp32 (src/core/gguf_quant.c:14-58) bit for bit, its subnormal quirk included.
#include "common.cuh"

namespace {

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return cml_half_to_float(h); }

// Raw GGUF blocks: 34-byte (Q8_0) or 18-byte (Q4_0) records, only 2-byte aligned.
template <int TYPE>
__global__ void dequant_blocks_kernel(const uint8_t* __restrict__ blocks, float* __restrict__ dst, size_t numel) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < numel; e += stride) {
        const size_t b = e >> 5;
        const int j = (int)(e & 31);
        if (TYPE == CMLB200_Q8_0) {
            const uint8_t* p = blocks + b * 34;
            const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(p));
            const int q = (int)(int8_t)p[2 + j];
            dst[e] = (float)q * d;
        } else {
            const uint8_t* p = blocks + b * 18;
            const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(p));
            const uint8_t byte = p[2 + (j & 15)];
            const int nib = (j < 16) ? (byte & 15) : (byte >> 4);
            dst[e] = (float)(nib - 8) * d;
        }
    }
}

// Repacked planes: one thread expands 16 quant bytes (128-bit load).
template <int TYPE>
__global__ void dequant_planes_kernel(const uint8_t* __restrict__ qs, const uint16_t* __restrict__ scales,
                                      float* __restrict__ dst, size_t nchunks) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < nchunks; c += stride) {
        const uint4 v = reinterpret_cast<const uint4*>(qs)[c];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        if (TYPE == CMLB200_Q8_0) {
            const float d = half_bits_to_float(scales[c >> 1]);   // 16 quants = half a block
            float* o = dst + c * 16;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int q = (int)(int8_t)((w[i >> 2] >> (8 * (i & 3))) & 0xFF);
                o[i] = (float)q * d;
            }
        } else {
            const float d = half_bits_to_float(scales[c]);        // 16 bytes = one block
            float* o = dst + c * 32;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xFF;
                o[i] = (float)((int)(byte & 15) - 8) * d;
                o[i + 16] = (float)((int)(byte >> 4) - 8) * d;
            }
        }
    }
}

__global__ void dequant_nf4_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                   int num_scales, int block, size_t numel, float* __restrict__ out) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t nbytes = (numel + 1) / 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += stride) {
        const uint8_t byte = packed[i];
        const size_t e0 = 2 * i, e1 = e0 + 1;
        size_t b0 = e0 / (size_t)block;
        if (b0 >= (size_t)num_scales) b0 = (size_t)num_scales - 1;
        out[e0] = kNF4[byte >> 4] * scales[b0];
        if (e1 < numel) {
            size_t b1 = e1 / (size_t)block;
            if (b1 >= (size_t)num_scales) b1 = (size_t)num_scales - 1;
            out[e1] = kNF4[byte & 15] * scales[b1];
        }
    }
}

// NF4 quantisation (src/core/quantization.c:213-312), two passes: block absmax, then codes.
__global__ void nf4_absmax_kernel(const float* __restrict__ x, size_t numel, int block, float* __restrict__ scales, size_t nblocks) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += stride) {
        size_t s = b * (size_t)block, e = s + (size_t)block;
        if (e > numel) e = numel;
        float amax = 0.f;
        for (size_t i = s; i < e; i++) { const float a = fabsf(x[i]); if (a > amax) amax = a; }
        scales[b] = amax < 1e-10f ? 1e-10f : amax;
    }
}
__device__ __forceinline__ int nf4_nearest(float v) {
    int best = 0;
    float bd = fabsf(v - kNF4[0]);
#pragma unroll
    for (int c = 1; c < 16; c++) {
        const float d = fabsf(v - kNF4[c]);
        if (d < bd) { bd = d; best = c; }
    }
    return best;
}
__global__ void nf4_codes_kernel(const float* __restrict__ x, size_t numel, int block, const float* __restrict__ scales,
                                 uint8_t* __restrict__ packed) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t nbytes = (numel + 1) / 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += stride) {
        int idx[2] = {0, 0};                               // the pad element of an odd tensor keeps code 0
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t e = 2 * i + h;
            if (e < numel) {
                float v = __fdiv_rn(x[e], scales[e / (size_t)block]);
                if (v > 1.0f) v = 1.0f;
                if (v < -1.0f) v = -1.0f;
                idx[h] = nf4_nearest(v);
            }
        }
        packed[i] = (uint8_t)((idx[0] << 4) | (idx[1] & 15));
    }
}

inline int grid_for(size_t work, int threads) {
    size_t g = (work + threads - 1) / threads;
    size_t cap = (size_t)cmlb_num_sms() * 16;
    return (int)(g < cap ? (g ? g : 1) : cap);
}

}  // namespace

extern "C" int cmlb200_gguf_dequantize(int type, const void* d_blocks, float* d_dst, size_t numel, void* stream) {
    CMLB_REQUIRE(d_blocks && d_dst && numel != 0, "cmlb200_gguf_dequantize: NULL pointer or numel == 0");
    CMLB_REQUIRE(type == CMLB200_Q4_0 || type == CMLB200_Q8_0, "cmlb200_gguf_dequantize: unsupported type %d", type);
    CMLB_REQUIRE(numel % 32 == 0, "cmlb200_gguf_dequantize: numel must be a multiple of the block size 32");
    const int threads = 256;
    if (type == CMLB200_Q8_0)
        dequant_blocks_kernel<CMLB200_Q8_0><<<grid_for(numel, threads), threads, 0, as_stream(stream)>>>(
            (const uint8_t*)d_blocks, d_dst, numel);
    else
        dequant_blocks_kernel<CMLB200_Q4_0><<<grid_for(numel, threads), threads, 0, as_stream(stream)>>>(
            (const uint8_t*)d_blocks, d_dst, numel);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_dequantize_nf4(const uint8_t* d_packed, const float* d_scales, int num_scales, int block,
                                      size_t numel, float* d_out, void* stream) {
    CMLB_REQUIRE(d_packed && d_scales && d_out, "cmlb200_dequantize_nf4: NULL argument");
    CMLB_REQUIRE(num_scales > 0 && block > 0 && numel != 0, "cmlb200_dequantize_nf4: invalid parameters");
    const int threads = 256;
    dequant_nf4_kernel<<<grid_for((numel + 1) / 2, threads), threads, 0, as_stream(stream)>>>(
        d_packed, d_scales, num_scales, block, numel, d_out);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_dequant_qmat(const cmlb200_qmat* W, float* d_dst, void* stream) {
    CMLB_REQUIRE(W && d_dst && W->qs && W->scales, "cmlb200_dequant_qmat: NULL argument");
    CMLB_REQUIRE(W->rows > 0 && W->cols > 0 && W->cols % 32 == 0, "cmlb200_dequant_qmat: bad shape %dx%d", W->rows, W->cols);
    const size_t numel = (size_t)W->rows * W->cols;
    const int threads = 256;
    switch (W->type) {
        case CMLB200_Q8_0:
            dequant_planes_kernel<CMLB200_Q8_0><<<grid_for(numel / 16, threads), threads, 0, as_stream(stream)>>>(
                (const uint8_t*)W->qs, (const uint16_t*)W->scales, d_dst, numel / 16);
            break;
        case CMLB200_Q4_0:
            dequant_planes_kernel<CMLB200_Q4_0><<<grid_for(numel / 32, threads), threads, 0, as_stream(stream)>>>(
                (const uint8_t*)W->qs, (const uint16_t*)W->scales, d_dst, numel / 32);
            break;
        case CMLB200_NF4: {
            CMLB_REQUIRE(W->block > 0 && numel % (size_t)W->block == 0, "cmlb200_dequant_qmat: bad NF4 block %d", W->block);
            return cmlb200_dequantize_nf4((const uint8_t*)W->qs, (const float*)W->scales,
                                          (int)(numel / (size_t)W->block), W->block, numel, d_dst, stream);
        }
        default:
            CMLB_REQUIRE(false, "cmlb200_dequant_qmat: unsupported type %d", W->type);
    }
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

extern "C" int cmlb200_quantize_nf4(const float* d_x, size_t numel, int block, uint8_t* d_packed, float* d_scales, void* stream) {
    CMLB_REQUIRE(d_x && d_packed && d_scales, "cmlb200_quantize_nf4: NULL argument");
    CMLB_REQUIRE(numel != 0 && block > 0, "cmlb200_quantize_nf4: invalid parameters");
    const size_t nblocks = (numel + (size_t)block - 1) / (size_t)block;
    nf4_absmax_kernel<<<grid_for(nblocks, 128), 128, 0, as_stream(stream)>>>(d_x, numel, block, d_scales, nblocks);
    CMLB_LAUNCH_CHECK();
    nf4_codes_kernel<<<grid_for((numel + 1) / 2, 256), 256, 0, as_stream(stream)>>>(d_x, numel, block, d_scales, d_packed);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
