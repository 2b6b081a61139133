// Dequant-fused GEMV / skinny GEMM for decode (M <= 32), fp32 activations,
// fp32 accumulation: y[M,N] = x[M,K] . dequant(W[N,K])^T.
//
// Replaces "dequantize the whole weight to fp32, then run an fp32 matmul"
// (C-ML src/nn/qlora.c:264-317; src/core/gguf.c:271-295 followed by
// src/ops/ir/execution.c:989-1052 / 3090-3134). The weight is streamed once
// from HBM in its packed form with 128-bit loads; each lane expands its 16
// bytes in registers, multiplies with activations staged in shared memory,
// and rows are reduced with warp shuffles.
#include "common.cuh"

// gemv_dp4a.cu: the integer-dot kernels for Q4_0 / Q8_0 at small M
int cmlb200_gemv_dp4a_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                       const uint32_t* xq, float* y, int M, int epi, cudaStream_t st);
size_t cmlb200_xq_bytes_(int M, int K);
int cmlb200_x_digits_(const float* x, int M, int K, uint32_t* xq, cudaStream_t st);

// gemv_mma.cu: the tensor-core decode kernel (mma.sync int8) for up to 4 rows of x per launch
int cmlb200_gemv_mma_rows_(const cmlb200_qmat* W, int epi);
int cmlb200_gemv_mma_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                      const uint32_t* xq, float* y, int M, int epi, cudaStream_t st);

// gemv_mma8.cu: the same for 5 to 8 rows of x per launch (Q4_0)
bool cmlb200_gemv_mma8_ok_(const cmlb200_qmat* W, int epi);
int cmlb200_gemv_mma8_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps, float* y, int M,
                       int epi, cudaStream_t st);

// gemv_kquant.cu: Q4_1 / Q4_K / Q5_K / Q6_K weights straight from the GGUF block stream
bool cmlb200_is_kquant_type_(int type);
int cmlb200_gemv_kquant_(const cmlb200_qmat* W, const float* x, float* y, int M, int accumulate, cudaStream_t st);

// gemv_tc.cu: tcgen05 integer tensor-core path over the tile-major copy of the weight
int cmlb200_gemv_tc_(const cmlb200_qmat* W, const float* x, float* y, int M, int accumulate, cudaStream_t st);

namespace {

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };
constexpr int kDp4aMaxM = 2;     // up to here the CUDA-core integer-dot path is the faster one
constexpr int kMmaMaxM = 8;      // up to here the mma.sync kernel (4 rows of x per launch) beats the tcgen05 one

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kSegMaxFloats = 12288;  // activation floats staged per K segment (48 KB)

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    // weights are read exactly once: bypass L1 allocation
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Dot product of the 16 packed bytes in `v` with the matching activations.
// ELEMS = activations covered by 16 bytes: 16 (Q8_0) or 32 (Q4_0, NF4).
template <int TYPE>
__device__ __forceinline__ float dot16(const uint4& v, const float* __restrict__ xs) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float s = 0.f;
    if (TYPE == CMLB200_Q8_0) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + 4 * i);
            s = fmaf((float)(int)(int8_t)(w[i] & 0xFF), xv.x, s);
            s = fmaf((float)(int)(int8_t)((w[i] >> 8) & 0xFF), xv.y, s);
            s = fmaf((float)(int)(int8_t)((w[i] >> 16) & 0xFF), xv.z, s);
            s = fmaf((float)((int)w[i] >> 24), xv.w, s);
        }
    } else if (TYPE == CMLB200_Q4_0) {
        // byte j: low nibble -> element j, high nibble -> element j + 16
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 xl = *reinterpret_cast<const float4*>(xs + 4 * i);
            const float4 xh = *reinterpret_cast<const float4*>(xs + 16 + 4 * i);
            const uint32_t u = w[i];
            s = fmaf((float)((int)(u & 15) - 8), xl.x, s);
            s = fmaf((float)((int)((u >> 4) & 15) - 8), xh.x, s);
            s = fmaf((float)((int)((u >> 8) & 15) - 8), xl.y, s);
            s = fmaf((float)((int)((u >> 12) & 15) - 8), xh.y, s);
            s = fmaf((float)((int)((u >> 16) & 15) - 8), xl.z, s);
            s = fmaf((float)((int)((u >> 20) & 15) - 8), xh.z, s);
            s = fmaf((float)((int)((u >> 24) & 15) - 8), xl.w, s);
            s = fmaf((float)((int)(u >> 28) - 8), xh.w, s);
        }
    } else {
        // NF4: byte i -> element 2i (high nibble), 2i+1 (low nibble)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + 8 * i);
            const float4 xb = *reinterpret_cast<const float4*>(xs + 8 * i + 4);
            const uint32_t u = w[i];
            s = fmaf(kNF4[(u >> 4) & 15], xa.x, s);
            s = fmaf(kNF4[u & 15], xa.y, s);
            s = fmaf(kNF4[(u >> 12) & 15], xa.z, s);
            s = fmaf(kNF4[(u >> 8) & 15], xa.w, s);
            s = fmaf(kNF4[(u >> 20) & 15], xb.x, s);
            s = fmaf(kNF4[(u >> 16) & 15], xb.y, s);
            s = fmaf(kNF4[u >> 28], xb.z, s);
            s = fmaf(kNF4[(u >> 24) & 15], xb.w, s);
        }
    }
    return s;
}

template <int TYPE>
__device__ __forceinline__ float load_scale(const void* scales, size_t row, int K, int chunk, int nf4_block) {
    if (TYPE == CMLB200_Q8_0)
        return cml_half_to_float(reinterpret_cast<const uint16_t*>(scales)[row * (size_t)(K / 32) + (chunk >> 1)]);
    if (TYPE == CMLB200_Q4_0)
        return cml_half_to_float(reinterpret_cast<const uint16_t*>(scales)[row * (size_t)(K / 32) + chunk]);
    return reinterpret_cast<const float*>(scales)[(row * (size_t)K + (size_t)chunk * 32) / (size_t)nf4_block];
}

// One warp owns R consecutive rows (2R when SWIGLU pairs gate and up); its 32
// lanes split K in 16-byte chunks. MT activation rows are handled per pass.
template <int TYPE, int MT, int R, int EPI>
__global__ void __launch_bounds__(kThreads)
gemv_kernel(const uint8_t* __restrict__ qs, const void* __restrict__ scales,
            const uint8_t* __restrict__ qs2, const void* __restrict__ scales2,
            const float* __restrict__ x, float* __restrict__ y, int N, int K, int m0, int nf4_block, int kseg) {
    extern __shared__ __align__(16) float xs[];   // [MT][kseg]
    constexpr int ELEMS = (TYPE == CMLB200_Q8_0) ? 16 : 32;
    constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t row_bytes = (size_t)K * 16 / ELEMS;
    const int ngroups = (N + R - 1) / R;

    for (int g0 = blockIdx.x * kWarps; g0 < ngroups; g0 += gridDim.x * kWarps) {
        const int g = g0 + warp;
        float acc[NW][R][MT];
#pragma unroll
        for (int a = 0; a < NW; a++)
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int m = 0; m < MT; m++) acc[a][r][m] = 0.f;

        for (int k0 = 0; k0 < K; k0 += kseg) {
            const int klen = min(kseg, K - k0);
            __syncthreads();
            for (int m = 0; m < MT; m++)
                for (int i = threadIdx.x * 4; i < klen; i += kThreads * 4)
                    *reinterpret_cast<float4*>(xs + m * kseg + i) =
                        *reinterpret_cast<const float4*>(x + (size_t)(m0 + m) * K + k0 + i);
            __syncthreads();
            if (g < ngroups) {
                const int c0 = k0 / ELEMS, nchunks = klen / ELEMS;
                for (int c = lane; c < nchunks; c += 32) {
                    uint4 wv[NW][R];
                    float sc[NW][R];
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        const int row = min(g * R + r, N - 1);
                        wv[0][r] = ld_stream(qs + row * row_bytes + (size_t)(c0 + c) * 16);
                        sc[0][r] = load_scale<TYPE>(scales, row, K, c0 + c, nf4_block);
                        if (NW == 2) {
                            wv[1][r] = ld_stream(qs2 + row * row_bytes + (size_t)(c0 + c) * 16);
                            sc[1][r] = load_scale<TYPE>(scales2, row, K, c0 + c, nf4_block);
                        }
                    }
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const float* xp = xs + m * kseg + c * ELEMS;
#pragma unroll
                        for (int a = 0; a < NW; a++)
#pragma unroll
                            for (int r = 0; r < R; r++)
                                acc[a][r][m] = fmaf(sc[a][r], dot16<TYPE>(wv[a][r], xp), acc[a][r][m]);
                    }
                }
            }
        }
        if (g < ngroups) {
#pragma unroll
            for (int a = 0; a < NW; a++)
#pragma unroll
                for (int r = 0; r < R; r++)
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        float v = acc[a][r][m];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        acc[a][r][m] = v;
                    }
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int row = g * R + r;
                    if (row < N) {
#pragma unroll
                        for (int m = 0; m < MT; m++) {
                            float* out = y + (size_t)(m0 + m) * N + row;
                            if (EPI == EPI_STORE) *out = acc[0][r][m];
                            else if (EPI == EPI_ACCUM) *out += acc[0][r][m];
                            else {
                                const float gte = acc[0][r][m];
                                *out = (gte / (1.0f + expf(-gte))) * acc[1][r][m];   // silu(g) * u
                            }
                        }
                    }
                }
            }
        }
    }
}

template <int TYPE, int MT, int EPI>
int launch_gemv(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, float* y, int m0, cudaStream_t st) {
    constexpr int R = (EPI == EPI_SWIGLU) ? 1 : 2;
    const int N = W->rows, K = W->cols;
    int kseg = K;
    if ((size_t)kseg * MT > (size_t)kSegMaxFloats) kseg = (kSegMaxFloats / MT) / 64 * 64;
    const size_t smem = (size_t)kseg * MT * sizeof(float);
    auto kern = gemv_kernel<TYPE, MT, R, EPI>;
    static size_t attr_smem[kMaxDevices] = {};
    CMLB_CUDA(cmlb_ensure_smem(kern, (size_t)kSegMaxFloats * 4, attr_smem));
    const int ngroups = (N + R - 1) / R;
    int grid = (ngroups + kWarps - 1) / kWarps;
    const int cap = cmlb_num_sms() * 4;
    if (grid > cap) grid = cap;
    kern<<<grid, kThreads, smem, st>>>((const uint8_t*)W->qs, W->scales, W2 ? (const uint8_t*)W2->qs : nullptr,
                                        W2 ? W2->scales : nullptr, x, y, N, K, m0, W->block, kseg);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}

template <int TYPE, int EPI>
int gemv_type(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, float* y, int M, cudaStream_t st) {
    int m0 = 0, rc = 0;
    while (m0 < M && rc == 0) {
        const int left = M - m0;
        if (left >= 4) { rc = launch_gemv<TYPE, 4, EPI>(W, W2, x, y, m0, st); m0 += 4; }
        else if (left >= 2) { rc = launch_gemv<TYPE, 2, EPI>(W, W2, x, y, m0, st); m0 += 2; }
        else { rc = launch_gemv<TYPE, 1, EPI>(W, W2, x, y, m0, st); m0 += 1; }
    }
    return rc;
}

int check_qmat(const cmlb200_qmat* W, const char* who) {
    CMLB_REQUIRE(W && W->qs && (W->scales || cmlb200_is_kquant_type_(W->type)), "%s: NULL weight", who);
    CMLB_REQUIRE(W->rows > 0 && W->cols > 0 && W->cols % 32 == 0, "%s: weight shape %dx%d (cols must be a multiple of 32)", who, W->rows, W->cols);
    if (cmlb200_is_kquant_type_(W->type)) return CMLB200_OK;     // the block-stream kernel checks the rest
    CMLB_REQUIRE(W->type == CMLB200_Q4_0 || W->type == CMLB200_Q8_0 || W->type == CMLB200_NF4, "%s: unsupported weight type %d", who, W->type);
    if (W->type == CMLB200_NF4)
        CMLB_REQUIRE(W->block >= 32 && W->block % 32 == 0 && W->cols % W->block == 0,
                     "%s: NF4 block size %d must be a multiple of 32 that divides cols=%d", who, W->block, W->cols);
    CMLB_REQUIRE(((uintptr_t)W->qs & 15) == 0 && ((uintptr_t)W->scales & 3) == 0, "%s: weight planes must be 16-byte aligned", who);
    return CMLB200_OK;
}

template <int EPI>
int gemv_dispatch(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, float* y, int M, void* stream,
                  const char* who) {
    int rc = check_qmat(W, who);
    if (rc) return rc;
    if (EPI == EPI_SWIGLU) {
        rc = check_qmat(W2, who);
        if (rc) return rc;
        CMLB_REQUIRE(W2->type == W->type && W2->rows == W->rows && W2->cols == W->cols && W2->block == W->block,
                     "%s: gate and up weights must have the same type and shape", who);
    }
    CMLB_REQUIRE(x && y, "%s: NULL activation pointer", who);
    CMLB_REQUIRE(M >= 1 && M <= 32, "%s: M=%d outside the decode range 1..32", who, M);
    CMLB_REQUIRE(((uintptr_t)x & 15) == 0, "%s: x must be 16-byte aligned", who);
    cudaStream_t st = as_stream(stream);
    if (cmlb200_is_kquant_type_(W->type)) {
        CMLB_REQUIRE(EPI != EPI_SWIGLU, "%s: GGUF type %d has no fused SwiGLU kernel; use cmlb200_gemv twice and cmlb200_swiglu_f32", who, W->type);
        return cmlb200_gemv_kquant_(W, x, y, M, EPI == EPI_ACCUM, st);
    }
    const bool tc_ok = W->type != CMLB200_NF4 && M > kDp4aMaxM && W->tiles && EPI != EPI_SWIGLU && W->cols % 128 == 0 && ((uintptr_t)y & 15) == 0;
    if (W->type == CMLB200_Q4_0 && M > 2 && (M > 4 || cmlb200_gemv_mma_rows_(W, EPI) < M) && cmlb200_gemv_mma8_ok_(W, EPI)) {
        // eight rows of x per launch of the plane-major mma.sync kernel: the weight is streamed once per eight rows
        for (int m0 = 0; m0 < M && rc == 0; m0 += 8)
            rc = cmlb200_gemv_mma8_(W, W2, x + (size_t)m0 * W->cols, nullptr, 0.f, y + (size_t)m0 * W->rows, M - m0 < 8 ? M - m0 : 8, EPI, st);
        return rc;
    }
    if (W->type != CMLB200_NF4 && M <= kMmaMaxM) {
        // the mma.sync kernel streams the weight once per launch: take it while two launches cover M
        // (or when there is no tile-major copy for the tcgen05 kernel)
        const int per = cmlb200_gemv_mma_rows_(W, EPI);
        if (per > 0 && ((M + per - 1) / per <= 2 || !tc_ok)) return cmlb200_gemv_mma_(W, W2, x, nullptr, 0.f, nullptr, y, M, EPI, st);
    }
    if (W->type != CMLB200_NF4 && M > kDp4aMaxM && W->tiles && EPI != EPI_SWIGLU && W->cols % 128 == 0 &&
        ((uintptr_t)y & 15) == 0)
        return cmlb200_gemv_tc_(W, x, y, M, EPI == EPI_ACCUM, st);
    if (W->type != CMLB200_NF4 && M <= 4) return cmlb200_gemv_dp4a_(W, W2, x, nullptr, 0.f, nullptr, y, M, EPI, st);
    switch (W->type) {
        case CMLB200_Q8_0: return gemv_type<CMLB200_Q8_0, EPI>(W, W2, x, y, M, st);
        case CMLB200_Q4_0: return gemv_type<CMLB200_Q4_0, EPI>(W, W2, x, y, M, st);
        default: return gemv_type<CMLB200_NF4, EPI>(W, W2, x, y, M, st);
    }
}

}  // namespace

extern "C" int cmlb200_gemv(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, void* stream) {
    return gemv_dispatch<EPI_STORE>(W, nullptr, d_x, d_y, M, stream, "cmlb200_gemv");
}
extern "C" int cmlb200_gemv_accum(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, void* stream) {
    return gemv_dispatch<EPI_ACCUM>(W, nullptr, d_x, d_y, M, stream, "cmlb200_gemv_accum");
}
extern "C" int cmlb200_gemv_swiglu(const cmlb200_qmat* Wg, const cmlb200_qmat* Wu, const float* d_x, float* d_y,
                                   int M, void* stream) {
    return gemv_dispatch<EPI_SWIGLU>(Wg, Wu, d_x, d_y, M, stream, "cmlb200_gemv_swiglu");
}

// ---- host activations in, host result out ----------------------------------------------------
// C-ML's quantized Linear takes and returns host tensors (src/nn/qlora.c:264-317; the GGUF path
// dequantises to a host tensor and multiplies there, src/core/gguf.c:271-295). For a decode-sized call
// the two DMA copies and their bookkeeping cost several times the GEMV, so with page-locked host
// buffers the copies become two small kernels in the same programmatic-launch chain as the GEMV:
// one reads x from host memory over the bus into a device staging row (and lets the GEMV start
// prefetching weights meanwhile), one writes y from the device straight into the host buffer with
// 16-byte stores. Pageable buffers go through cudaMemcpyAsync. The call returns when y is in h_y.
// (Tried and not kept: digit records made straight from the host buffer, and the GEMV storing y
// straight into host memory; one launch fewer each, 0.5-1 us slower per call.)
namespace {
template <bool VEC>
__global__ void __launch_bounds__(256) host_stage_kernel(const float* __restrict__ src, float* __restrict__ dst, size_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        if (i < n / 4) reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    } else if (i < n) {
        dst[i] = src[i];
    }
}
int host_stage(const float* src, float* dst, size_t n, cudaStream_t st) {
    const bool vec = n % 4 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0;
    const size_t items = vec ? n / 4 : n;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((items + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (vec) CMLB_CUDA(cudaLaunchKernelEx(&cfg, host_stage_kernel<true>, src, dst, n));
    else CMLB_CUDA(cudaLaunchKernelEx(&cfg, host_stage_kernel<false>, src, dst, n));
    return CMLB200_OK;
}
struct HostStage { float* x; size_t xcap; float* y; size_t ycap; };
HostStage g_host_stage[kMaxDevices] = {};
int stage_reserve(float** buf, size_t* cap, size_t n) {
    if (n <= *cap) return CMLB200_OK;
    if (*buf) { CMLB_CUDA(cudaDeviceSynchronize()); CMLB_CUDA(cudaFree(*buf)); *buf = nullptr; *cap = 0; }
    CMLB_CUDA(cudaMalloc(reinterpret_cast<void**>(buf), n * sizeof(float)));
    *cap = n;
    return CMLB200_OK;
}
// The address a kernel can use for a page-locked host pointer, nullptr for pageable memory.
const float* device_view(const float* h) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, h) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return a.type == cudaMemoryTypeHost ? static_cast<const float*>(a.devicePointer) : nullptr;
}
}  // namespace

extern "C" int cmlb200_gemv_host(const cmlb200_qmat* W, const float* h_x, float* h_y, int M, void* stream) {
    int rc = check_qmat(W, "cmlb200_gemv_host");
    if (rc) return rc;
    CMLB_REQUIRE(h_x && h_y, "cmlb200_gemv_host: NULL activation pointer");
    CMLB_REQUIRE(M >= 1 && M <= 32, "cmlb200_gemv_host: M=%d outside the decode range 1..32", M);
    HostStage& s = g_host_stage[cmlb_device_index()];
    const size_t nx = (size_t)M * W->cols, ny = (size_t)M * W->rows;
    if ((rc = stage_reserve(&s.x, &s.xcap, nx)) || (rc = stage_reserve(&s.y, &s.ycap, ny))) return rc;
    cudaStream_t st = as_stream(stream);
    const float* vx = device_view(h_x);
    float* vy = const_cast<float*>(device_view(h_y));
    if (vx) { if ((rc = host_stage(vx, s.x, nx, st))) return rc; }
    else CMLB_CUDA(cudaMemcpyAsync(s.x, h_x, nx * sizeof(float), cudaMemcpyHostToDevice, st));
    if ((rc = gemv_dispatch<EPI_STORE>(W, nullptr, s.x, s.y, M, stream, "cmlb200_gemv_host"))) return rc;
    if (vy) { if ((rc = host_stage(s.y, vy, ny, st))) return rc; }
    else CMLB_CUDA(cudaMemcpyAsync(h_y, s.y, ny * sizeof(float), cudaMemcpyDeviceToHost, st));
    CMLB_CUDA(cudaStreamSynchronize(st));
    return CMLB200_OK;
}

// ---- NF4 linear for shapes outside the vectorised kernels (any in_features, any block size, blocks
// that straddle rows): the quantized Linear of src/nn/qlora.c:264-317 element by element, one warp
// per output value. Element e = n*K + k of the flat [out, in] weight is TABLE[nibble(e)] times
// scales[min(e / block, num_scales - 1)], even e in the high nibble (src/core/quantization.c:349-366).
namespace {
__global__ void __launch_bounds__(256)
nf4_linear_general_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales, int num_scales, int block,
                          const float* __restrict__ x, float* __restrict__ y, int M, int N, int K) {
    const int lane = threadIdx.x & 31;
    const long long out = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (out >= (long long)M * N) return;
    const int m = (int)(out / N), n = (int)(out % N);
    float s = 0.f;
    for (int k = lane; k < K; k += 32) {
        const size_t e = (size_t)n * K + k;
        const uint8_t b = packed[e >> 1];
        const int idx = (e & 1) ? (b & 15) : (b >> 4);
        size_t bi = e / (size_t)block;
        if (bi >= (size_t)num_scales) bi = (size_t)num_scales - 1;
        s = fmaf(x[(size_t)m * K + k], kNF4[idx] * scales[bi], s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) y[out] = s;
}
}  // namespace

extern "C" int cmlb200_linear_nf4_general(const uint8_t* d_packed, const float* d_scales, int num_scales, int block, int rows, int cols,
                                          const float* d_x, int M, float* d_y, void* stream) {
    CMLB_REQUIRE(d_packed && d_scales && d_x && d_y, "cmlb200_linear_nf4_general: NULL argument");
    CMLB_REQUIRE(num_scales > 0 && block > 0 && rows > 0 && cols > 0 && M > 0, "cmlb200_linear_nf4_general: bad shape (rows=%d cols=%d M=%d block=%d)", rows, cols, M, block);
    const long long outs = (long long)M * rows;
    nf4_linear_general_kernel<<<(unsigned)((outs + 7) / 8), 256, 0, as_stream(stream)>>>(d_packed, d_scales, num_scales, block, d_x, d_y, M, rows, cols);
    CMLB_LAUNCH_CHECK();
    return CMLB200_OK;
}
