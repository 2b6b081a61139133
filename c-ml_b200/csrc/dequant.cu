// Dequantisation to fp32, bit-exact with C-ML's CPU routines: one IEEE fp32
// multiply per element, integer arithmetic before it, no fast-math, no FTZ.
//   Q8_0: y = (float)q * d              (src/core/gguf_quant.c:114-125)
//   Q4_0: y = (float)(nibble - 8) * d   (src/core/gguf_quant.c:66-82)
//   NF4 : y = TABLE[idx] * absmax       (src/core/quantization.c:349-366)
//   Q4_1: y = (float)nibble * d + m                       (src/core/gguf_quant.c:90-112)
//   Q4_K: y = (float)q4 * (d * sc) - dmin * mn            (src/core/gguf_quant.c:151-196)
//   Q5_K: y = (float)q5 * (d * sc) - dmin * mn            (src/core/gguf_quant.c:211-270)
//   Q6_K: y = d * (float)scale8 * (float)(q6 - 32)        (src/core/gguf_quant.c:283-311)
//   (every product above is exact in fp32 -- at most 24 significant bits -- so contracting a
//   multiply-add into one instruction cannot change a result bit)
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

// The other block types C-ML reads (GGUF ids 3, 12, 13, 14), element by element in C-ML's own
// layout: Q4_K / Q5_K keep each 32-element sub-block in 16 consecutive bytes (low nibble =
// element k, high nibble = element k + 16 of the sub-block), which is C-ML's definition
// (src/core/gguf_quant.c:174-187), not ggml's 64-element interleave.
__device__ __forceinline__ void kquant_scale_min(const uint8_t* sc_raw, int i, int& sc, int& mn) {
    if (i < 4) { sc = sc_raw[i] & 0x3F; mn = sc_raw[i + 4] & 0x3F; }
    else {
        const int j = i - 4;
        sc = (sc_raw[j + 8] & 0x0F) | ((sc_raw[j] >> 6) << 4);
        mn = (sc_raw[j + 8] >> 4) | ((sc_raw[j + 4] >> 6) << 4);
    }
}

template <int GTYPE>
__global__ void dequant_other_kernel(const uint8_t* __restrict__ blocks, float* __restrict__ dst, size_t numel) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < numel; e += stride) {
        if (GTYPE == 3) {                                  // Q4_1: d, m, 16 bytes
            const uint8_t* p = blocks + (e >> 5) * 20;
            const int j = (int)(e & 31);
            const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(p));
            const float m = half_bits_to_float(*reinterpret_cast<const uint16_t*>(p + 2));
            const uint8_t byte = p[4 + (j & 15)];
            dst[e] = (float)((j < 16) ? (byte & 15) : (byte >> 4)) * d + m;
        } else if (GTYPE == 12 || GTYPE == 13) {           // Q4_K / Q5_K: d, dmin, scales[12], (qh[32],) qs[128]
            const uint8_t* p = blocks + (e >> 8) * (GTYPE == 12 ? 144 : 176);
            const int r = (int)(e & 255), i = r >> 5, k = r & 31;
            const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(p));
            const float dmin = half_bits_to_float(*reinterpret_cast<const uint16_t*>(p + 2));
            int sc, mn;
            kquant_scale_min(p + 4, i, sc, mn);
            const uint8_t* qs = p + (GTYPE == 12 ? 16 : 48);
            const uint8_t byte = qs[i * 16 + (k & 15)];
            int q = (k < 16) ? (byte & 15) : (byte >> 4);
            if (GTYPE == 13) q |= ((p[16 + (r >> 3)] >> (r & 7)) & 1) << 4;
            const float scale = d * (float)sc, mnv = dmin * (float)mn;
            dst[e] = (float)q * scale - mnv;
        } else {                                           // Q6_K: ql[128], qh[64], scales[16], d
            const uint8_t* p = blocks + (e >> 8) * 210;
            const int r = (int)(e & 255);
            const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(p + 208));
            const int low4 = (r & 1) ? (p[r >> 1] >> 4) : (p[r >> 1] & 15);
            const int high2 = (p[128 + (r >> 2)] >> (2 * (r & 3))) & 3;
            const float sc = (float)(int)(int8_t)p[192 + (r >> 4)];
            dst[e] = d * sc * (float)((low4 | (high2 << 4)) - 32);
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
    CMLB_REQUIRE(type == CMLB200_Q4_0 || type == CMLB200_Q8_0 || type == 3 || type == 12 || type == 13 || type == 14,
                 "cmlb200_gguf_dequantize: unsupported type %d", type);
    const size_t bs = (type == 12 || type == 13 || type == 14) ? 256 : 32;
    CMLB_REQUIRE(numel % bs == 0, "cmlb200_gguf_dequantize: numel must be a multiple of the block size %zu", bs);
    const int threads = 256;
    const dim3 grid = grid_for(numel, threads);
    cudaStream_t st = as_stream(stream);
    if (type == 3) dequant_other_kernel<3><<<grid, threads, 0, st>>>((const uint8_t*)d_blocks, d_dst, numel);
    else if (type == 12) dequant_other_kernel<12><<<grid, threads, 0, st>>>((const uint8_t*)d_blocks, d_dst, numel);
    else if (type == 13) dequant_other_kernel<13><<<grid, threads, 0, st>>>((const uint8_t*)d_blocks, d_dst, numel);
    else if (type == 14) dequant_other_kernel<14><<<grid, threads, 0, st>>>((const uint8_t*)d_blocks, d_dst, numel);
    else if (type == CMLB200_Q8_0)
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
