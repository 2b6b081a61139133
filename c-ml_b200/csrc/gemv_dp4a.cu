// Decode GEMV for Q4_0 / Q8_0 at M <= 4, built to stay under the instruction-issue budget
// that HBM speed leaves per weight (about 3 lane-operations per 4-bit weight on B200).
//
// A straight fp32 path needs ~4 operations per weight just to turn a nibble into a float and
// multiply it. Here the activation vector is re-expressed as block-fixed-point: for every
// 32-element block of x (the same blocks the weights are quantized in)
//     x_k  ~=  s_b * X_k,   X_k a signed 16-bit integer,  s_b = max|x_block| / 32639,
// and X_k is split into two signed 8-bit digits X_k = d0*256 + d1 held as int8x4 words. The
// block dot product  sum_k q_k * X_k  then is two exact integer dot products on dp4a (4
// multiply-adds per lane-operation), recombined in fp32 and scaled by d_b * s_b;
// blocks are accumulated in fp32. Q4_0 nibbles are turned into the signed bytes 16*(q-8) with
// one shift and two 3-input logic operations per 8 weights, so the "-8" offset costs nothing
// and the factor 16 is taken out once per output. The only approximation is the rounding of x
// to 16 bits relative to its block maximum (relative output error of a few 1e-5), far inside
// the 2e-3 tolerance of this path.
//
// Replaces, like gemv.cu, C-ML's dequantize-then-fp32-matmul (src/core/gguf.c:271-295 +
// src/ops/ir/execution.c:989-1052, 3090-3134).
//
// This file holds the register-path kernel, which takes any K % 32 == 0: each warp loads its rows
// straight from global memory and digits come from a record array. The tensor-core kernel in
// gemv_mma.cu takes the shapes it can (K % 256 == 0 and a digit table that fits shared memory) and
// is tried first.
#include "common.cuh"

int cmlb200_x_digits_(const float* x, int M, int K, uint32_t* xq, cudaStream_t st);
// gemv_mma.cu: the tensor-core kernel for the shapes it takes
bool cmlb200_gemv_mma_ok_(const cmlb200_qmat* W, int epi, int M);
int cmlb200_gemv_mma_rows_(const cmlb200_qmat* W, int epi);
int cmlb200_gemv_mma_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                      const uint32_t* xq, float* y, int M, int epi, cudaStream_t st);
// gemv_mma8.cu: its sibling for 5 to 8 rows of x in one launch (Q4_0, fp32 x)
bool cmlb200_gemv_mma8_ok_(const cmlb200_qmat* W, int epi);
int cmlb200_gemv_mma8_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps, float* y, int M,
                       int epi, cudaStream_t st);

namespace {

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int XW = kXqWords;      // words per block of x digits: 3 planes x 8 words + scale + 3 pad
constexpr int XFULL = kXqFull;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ldg_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// x[M][K] (fp32) -> xq[M][K/32][XW] (global scratch). One launch serves every GEMV that
// consumes the same activations (q/k/v projections, gate/up).
__global__ void __launch_bounds__(256) x_digits_kernel(const float* __restrict__ x, int M, int K, uint32_t* __restrict__ xq) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int nblk = K / 32;
    const int sub = threadIdx.x & 7;                  // 8 lanes share a block, 4 elements each
    const int item = (blockIdx.x * 256 + threadIdx.x) >> 3;
    if (item < nblk * M) {                            // whole groups of 8 lanes enter or skip together
        const float4 v = *reinterpret_cast<const float4*>(x + (size_t)item * 32 + sub * 4);
        const float e[4] = {v.x, v.y, v.z, v.w};
        xq_emit_oct(e, sub, 0xffu << (threadIdx.x & 24), xq + (size_t)item * XW);
    }
}

// The three digit planes of one block record, as 24 registers.
__device__ __forceinline__ void load_digits(const uint32_t* __restrict__ xb, uint32_t (&d)[24]) {
#pragma unroll
    for (int i = 0; i < 6; i++) {
        const uint4 v = *reinterpret_cast<const uint4*>(xb + 4 * i);
        d[4 * i] = v.x; d[4 * i + 1] = v.y; d[4 * i + 2] = v.z; d[4 * i + 3] = v.w;
    }
}

// Integer part of one block dot product: sum_k w_k * X_k with w = q (Q8_0) or 16*(q-8) (Q4_0),
// exact in the three int32 digit sums and combined in fp32 (|sum| < 2^35).
template <int TYPE>
__device__ __forceinline__ float block_dot(const uint4& q0, const uint4& q1, const uint32_t (&d)[24]) {
    int s0 = 0, s1 = 0, s2 = 0, t0 = 0, t1 = 0, t2 = 0;
    if (TYPE == CMLB200_Q4_0) {
        const uint32_t w[4] = {q0.x, q0.y, q0.z, q0.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // nibble n in the top half of a byte, top bit flipped, reads as the int8 16*(n-8)
            const int lo = (int)(((w[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u);   // elements 4i..4i+3
            const int hi = (int)((w[i] & 0xF0F0F0F0u) ^ 0x80808080u);          // elements 16+4i..16+4i+3
            s0 = __dp4a(lo, (int)d[i], s0);      t0 = __dp4a(hi, (int)d[4 + i], t0);
            s1 = __dp4a(lo, (int)d[8 + i], s1);  t1 = __dp4a(hi, (int)d[12 + i], t1);
            s2 = __dp4a(lo, (int)d[16 + i], s2); t2 = __dp4a(hi, (int)d[20 + i], t2);
        }
    } else {
        const int w[8] = {(int)q0.x, (int)q0.y, (int)q0.z, (int)q0.w, (int)q1.x, (int)q1.y, (int)q1.z, (int)q1.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            s0 = __dp4a(w[i], (int)d[i], s0);      t0 = __dp4a(w[4 + i], (int)d[4 + i], t0);
            s1 = __dp4a(w[i], (int)d[8 + i], s1);  t1 = __dp4a(w[4 + i], (int)d[12 + i], t1);
            s2 = __dp4a(w[i], (int)d[16 + i], s2); t2 = __dp4a(w[4 + i], (int)d[20 + i], t2);
        }
    }
    return fmaf((float)(s0 + t0), 65536.0f, (float)(((s1 + t1) << 8) + (s2 + t2)));
}
template <int TYPE> constexpr float kDotUnit = (TYPE == CMLB200_Q4_0) ? 0.0625f : 1.0f;

// U block-steps of R rows are loaded together (U*R 128-bit loads in flight per lane); for
// K = 4096 and Q4_0 that is the warp's entire share of its rows, requested in one burst.
template <int TYPE, int MT, int R, int U, int EPI, bool QUIRK>
__global__ void __launch_bounds__(THREADS)
gemv_dp4a_kernel(const uint8_t* __restrict__ qs, const uint16_t* __restrict__ scales,
                 const uint8_t* __restrict__ qs2, const uint16_t* __restrict__ scales2,
                 const uint32_t* __restrict__ xq, float* __restrict__ y, int N, int K, int m0, int rows_per_warp) {
    extern __shared__ __align__(16) uint32_t xd[];     // [MT][K/32][XW]
    constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr int QB = (TYPE == CMLB200_Q8_0) ? 32 : 16;   // quant bytes per block
    constexpr int QV = QB / 16;                            // 128-bit loads per block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = K / 32;
    const size_t row_bytes = (size_t)nblk * QB;

    // contiguous row range of this warp
    const long long gw = (long long)blockIdx.x * WARPS + warp;
    const int row_begin = (int)min((long long)N, gw * rows_per_warp);
    const int row_end = min(N, row_begin + rows_per_warp);

    uint4 q[NW][U][R][QV];
    uint16_t dh[NW][U][R];
    auto load_step = [&](int r0, int b0) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int b = b0 + 32 * u;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int row = r0 + r;
                if (b < nblk && row < row_end) {
                    const uint8_t* p = qs + (size_t)row * row_bytes + (size_t)b * QB;
#pragma unroll
                    for (int v = 0; v < QV; v++) q[0][u][r][v] = ldg_stream(p + 16 * v);
                    dh[0][u][r] = ldg_u16(scales + (size_t)row * nblk + b);
                    if (NW == 2) {
                        const uint8_t* p2 = qs2 + (size_t)row * row_bytes + (size_t)b * QB;
#pragma unroll
                        for (int v = 0; v < QV; v++) q[1][u][r][v] = ldg_stream(p2 + 16 * v);
                        dh[1][u][r] = ldg_u16(scales2 + (size_t)row * nblk + b);
                    }
                } else {
#pragma unroll
                    for (int a = 0; a < NW; a++) {
#pragma unroll
                        for (int v = 0; v < QV; v++) q[a][u][r][v] = make_uint4(0, 0, 0, 0);
                        dh[a][u][r] = 0;        // scale 0 -> contributes nothing
                    }
                }
            }
        }
    };

    // Weights do not depend on the preceding kernel: request the first burst before the
    // dependency wait; activations are only touched after it.
    if (row_begin < row_end) load_step(row_begin, lane);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    {   // activation digits of rows m0..m0+MT-1: one contiguous run of the scratch
        const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)m0 * nblk * XW);
        uint4* dst = reinterpret_cast<uint4*>(xd);
        for (int i = threadIdx.x; i < MT * nblk * (XW / 4); i += THREADS) dst[i] = src[i];
    }
    __syncthreads();

    for (int r0 = row_begin; r0 < row_end; r0 += R) {
        float acc[NW][R][MT];
#pragma unroll
        for (int a = 0; a < NW; a++)
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int m = 0; m < MT; m++) acc[a][r][m] = 0.f;

        for (int b0 = lane; b0 < nblk; b0 += 32 * U) {
            if (r0 != row_begin || b0 != lane) load_step(r0, b0);
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int b = min(b0 + 32 * u, nblk - 1);       // out-of-range steps carry scale 0
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    const uint32_t* xb = xd + ((size_t)m * nblk + b) * XW;
                    const float xs = __uint_as_float(xb[24]) * kDotUnit<TYPE>;
                    uint32_t dg[24];
                    load_digits(xb, dg);
#pragma unroll
                    for (int a = 0; a < NW; a++)
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const float t = block_dot<TYPE>(q[a][u][r][0], q[a][u][r][QV - 1], dg);
                            const float d = QUIRK ? cml_half_to_float(dh[a][u][r]) : __half2float(__ushort_as_half(dh[a][u][r]));
                            acc[a][r][m] = fmaf(t, d * xs, acc[a][r][m]);
                        }
                }
            }
        }
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
                const int row = r0 + r;
                if (row < row_end) {
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        float* out = y + (size_t)(m0 + m) * N + row;
                        if (EPI == EPI_STORE) *out = acc[0][r][m];
                        else if (EPI == EPI_ACCUM) *out += acc[0][r][m];
                        else {
                            const float g = acc[0][r][m];
                            *out = (g / (1.0f + expf(-g))) * acc[1][r][m];
                        }
                    }
                }
            }
        }
    }
}

// Scratch for the activation digits of the plain entry points: one fixed 1 MiB buffer per
// device, allocated on first use and never moved (so captured CUDA graphs stay valid).
constexpr size_t kScratchBytes = 1u << 20;
uint32_t* g_scratch[16] = {};

int library_scratch(uint32_t** out) {
    int dev = 0;
    CMLB_CUDA(cudaGetDevice(&dev));
    CMLB_REQUIRE(dev >= 0 && dev < 16, "device index %d out of range", dev);
    if (!g_scratch[dev]) CMLB_CUDA(cudaMalloc((void**)&g_scratch[dev], kScratchBytes));
    *out = g_scratch[dev];
    return CMLB200_OK;
}

template <typename Kern, typename... Args>
int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CMLB_CUDA(cudaLaunchKernelEx(&cfg, kern, args...));
    return CMLB200_OK;
}

template <int TYPE, int MT, int EPI, bool QUIRK>
int launch(const cmlb200_qmat* W, const cmlb200_qmat* W2, const uint32_t* xq, float* y, int m0, cudaStream_t st) {
    constexpr int R = (EPI == EPI_SWIGLU) ? 2 : 4;
    constexpr int U = (TYPE == CMLB200_Q8_0) ? 1 : 2;
    const int N = W->rows, K = W->cols;
    const size_t smem = (size_t)(K / 32) * MT * XW * sizeof(uint32_t);
    CMLB_REQUIRE(smem <= 200 * 1024, "cmlb200_gemv: K=%d too large for the shared-memory activation digits", K);
    auto kern = gemv_dp4a_kernel<TYPE, MT, R, U, EPI, QUIRK>;
    static size_t attr_smem[kMaxDevices] = {};
    if (smem > 48 * 1024) CMLB_CUDA(cmlb_ensure_smem(kern, smem, attr_smem));
    // One group of R rows per warp while that keeps the grid within ~8 CTAs per SM; beyond
    // that, more rows per warp (a multiple of R).
    int rows_per_warp = R;
    const long long slots = (long long)cmlb_num_sms() * 8 * WARPS;
    while ((long long)(N + rows_per_warp - 1) / rows_per_warp > slots) rows_per_warp += R;
    const int nwarps = (N + rows_per_warp - 1) / rows_per_warp;
    const int grid = (nwarps + WARPS - 1) / WARPS;
    return launch_pdl(kern, dim3(grid), dim3(THREADS), smem, st, (const uint8_t*)W->qs, (const uint16_t*)W->scales,
                      W2 ? (const uint8_t*)W2->qs : (const uint8_t*)nullptr,
                      W2 ? (const uint16_t*)W2->scales : (const uint16_t*)nullptr, xq, y, N, K, m0, rows_per_warp);
}

int rmsnorm_digits_(const float* x, const __half* w, int rows, int dim, float eps, float* out, uint32_t* xq, cudaStream_t st);

// Rows of x are taken two at a time (one launch streams the weight once for both), then one.
// x != NULL: fp32 activations, RMS-normalised with nw first when nw != NULL, turned into digit
// records in `ws`; else xq holds the digit records.
template <int TYPE, int EPI, bool QUIRK>
int run_type(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const __half* nw, float eps, const uint32_t* xq,
             uint32_t* ws, float* y, int M, cudaStream_t st) {
    if (x) {
        const int rc = nw ? rmsnorm_digits_(x, nw, M, W->cols, eps, nullptr, ws, st) : cmlb200_x_digits_(x, M, W->cols, ws, st);
        if (rc) return rc;
        xq = ws;
    }
    int m0 = 0, rc = 0;
    while (m0 < M && rc == 0) {
        if (M - m0 >= 2) { rc = launch<TYPE, 2, EPI, QUIRK>(W, W2, xq, y, m0, st); m0 += 2; }
        else { rc = launch<TYPE, 1, EPI, QUIRK>(W, W2, xq, y, m0, st); m0 += 1; }
    }
    return rc;
}

template <int TYPE, bool QUIRK>
int run_epi(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const __half* nw, float eps, const uint32_t* xq, uint32_t* ws,
            float* y, int M, int epi, cudaStream_t st) {
    switch (epi) {
        case EPI_STORE: return run_type<TYPE, EPI_STORE, QUIRK>(W, W2, x, nw, eps, xq, ws, y, M, st);
        case EPI_ACCUM: return run_type<TYPE, EPI_ACCUM, QUIRK>(W, W2, x, nw, eps, xq, ws, y, M, st);
        default: return run_type<TYPE, EPI_SWIGLU, QUIRK>(W, W2, x, nw, eps, xq, ws, y, M, st);
    }
}

}  // namespace

size_t cmlb200_xq_bytes_(int M, int K) { return (size_t)M * (K / 32) * XW * sizeof(uint32_t); }

// Activation digits for M rows of K floats into caller-provided scratch.
int cmlb200_x_digits_(const float* x, int M, int K, uint32_t* xq, cudaStream_t st) {
    const int items = M * (K / 32);
    return launch_pdl(x_digits_kernel, dim3((items * 8 + 255) / 256), dim3(256), 0, st, x, M, K, xq);
}

// Internal entry used by gemv.cu's dispatcher (arguments already validated there).
// epi: 0 store, 1 accumulate, 2 swiglu (W2 = up projection). xq = digit records (then x is
// ignored), or NULL to work from the fp32 activations x, RMS-normalised with the fp16 weight
// norm_w first when that is not NULL.
int cmlb200_gemv_dp4a_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                       const uint32_t* xq, float* y, int M, int epi, cudaStream_t st) {
    // more rows of x than one launch of the 4-row kernel takes for this shape: the 8-row kernel streams the weight once
    if (!xq && M > 2 && M <= 8 && (M > 4 || cmlb200_gemv_mma_rows_(W, epi) < M) && cmlb200_gemv_mma8_ok_(W, epi)) return cmlb200_gemv_mma8_(W, W2, x, norm_w, eps, y, M, epi, st);
    if (cmlb200_gemv_mma_ok_(W, epi, M)) return cmlb200_gemv_mma_(W, W2, xq ? nullptr : x, norm_w, eps, xq, y, M, epi, st);
    uint32_t* ws = nullptr;
    if (xq) x = nullptr;
    else {                            // the register kernel reads digits from the library's scratch
        int rc = library_scratch(&ws);
        if (rc) return rc;
        CMLB_REQUIRE(cmlb200_xq_bytes_(M, W->cols) <= kScratchBytes, "cmlb200_gemv: M*K too large for the built-in activation scratch");
    }
    const __half* nw = reinterpret_cast<const __half*>(norm_w);
    const bool quirk = (W->flags & CMLB200_QMAT_SUBNORMAL_SCALES) || (W2 && (W2->flags & CMLB200_QMAT_SUBNORMAL_SCALES));
    const bool q8 = W->type == CMLB200_Q8_0;
    if (quirk) return q8 ? run_epi<CMLB200_Q8_0, true>(W, W2, x, nw, eps, xq, ws, y, M, epi, st) : run_epi<CMLB200_Q4_0, true>(W, W2, x, nw, eps, xq, ws, y, M, epi, st);
    return q8 ? run_epi<CMLB200_Q8_0, false>(W, W2, x, nw, eps, xq, ws, y, M, epi, st) : run_epi<CMLB200_Q4_0, false>(W, W2, x, nw, eps, xq, ws, y, M, epi, st);
}

// ---- allocation-free variant -------------------------------------------------------------------
// Some hosts of this library must not allocate device memory once they are running: an inference
// server that has handed the whole GPU to its own arena, a real-time loop that may not take the
// allocator's lock, a sandboxed plug-in whose CUDA allocation calls are filtered. For them the
// activation digits of the decode GEMV live in a fixed array that is part of the library image
// (every GPU that loads the library carries these 512 KiB until the process exits).
constexpr size_t kStaticScratchBytes = 512u << 10;
static __device__ __align__(256) uint32_t g_static_xq[kStaticScratchBytes / sizeof(uint32_t)];

// `g_static_xq` as written in host code is only the host-side handle of the symbol, never a
// device address; the address a kernel may use is looked up once per device, with that device
// current, and cached here.
static uint32_t* g_static_xq_ptr[16] = {};

static int static_scratch(uint32_t** out) {
    int dev = 0;
    CMLB_CUDA(cudaGetDevice(&dev));
    CMLB_REQUIRE(dev >= 0 && dev < 16, "cmlb200_gemv_noalloc: device index %d out of range", dev);
    if (!g_static_xq_ptr[dev]) {
        void* p = nullptr;
        CMLB_CUDA(cudaGetSymbolAddress(&p, g_static_xq));
        g_static_xq_ptr[dev] = static_cast<uint32_t*>(p);
    }
    *out = g_static_xq_ptr[dev];
    return CMLB200_OK;
}

extern "C" int cmlb200_gemv_noalloc(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, void* stream) {
    CMLB_REQUIRE(W && W->qs && W->scales && d_x && d_y, "cmlb200_gemv_noalloc: NULL argument");
    CMLB_REQUIRE(W->type == CMLB200_Q4_0 || W->type == CMLB200_Q8_0, "cmlb200_gemv_noalloc: weight type %d is not Q4_0 or Q8_0", W->type);
    CMLB_REQUIRE(W->rows > 0 && W->cols > 0 && W->cols % 32 == 0, "cmlb200_gemv_noalloc: weight shape %dx%d (cols must be a multiple of 32)", W->rows, W->cols);
    CMLB_REQUIRE(M >= 1 && M <= 4, "cmlb200_gemv_noalloc: M=%d outside 1..4", M);
    CMLB_REQUIRE(((uintptr_t)W->qs & 15) == 0 && ((uintptr_t)d_x & 15) == 0, "cmlb200_gemv_noalloc: weight planes and x must be 16-byte aligned");
    const size_t need = cmlb200_xq_bytes_(M, W->cols);
    CMLB_REQUIRE(need <= kStaticScratchBytes,
                 "cmlb200_gemv_noalloc: M*cols = %d*%d needs %zu bytes of activation scratch, the built-in array holds %zu "
                 "(M*cols <= 149796); use cmlb200_gemv for larger problems",
                 M, W->cols, need, kStaticScratchBytes);
    uint32_t* xq = nullptr;
    int rc = static_scratch(&xq);
    if (rc) return rc;
    // Every word a later kernel reads is rewritten here for this call's x, so nothing in the
    // array has to start at zero and the previous call's contents are harmless.
    rc = cmlb200_x_digits_(d_x, M, W->cols, xq, as_stream(stream));
    if (rc) return rc;
    return cmlb200_gemv_dp4a_(W, nullptr, nullptr, nullptr, 0.f, xq, d_y, M, EPI_STORE, as_stream(stream));
}

// ---- digits produced by the kernel that makes the activations ------------------------------------
// In the LLaMA decode step the GEMV input comes out of RMSNorm; producing the digit planes there
// saves a launch per projection group (Q/K/V share one set, gate/up another).
namespace {

// RMSNorm (src/nn/llama.c:71-124) of one row per CTA; writes the normalised row as fp32 (if asked)
// and as digit records. dim % 32 == 0.
__global__ void __launch_bounds__(1024)
rmsnorm_digits_kernel(const float* __restrict__ x, const __half* __restrict__ w, int dim, float eps, float* __restrict__ out,
                      uint32_t* __restrict__ xq) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)r * dim;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < dim; i += 4096) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) tot += red[i];
    const float inv = 1.0f / sqrtf(tot / (float)dim + eps);
    const int sub = threadIdx.x & 7;
    const unsigned gmask = 0xffu << (threadIdx.x & 24);
    const int nblk = dim / 32;
    for (int b = threadIdx.x >> 3; b < nblk; b += 128) {
        const int i = b * 32 + sub * 4;
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        const float e[4] = {v.x * inv * __half2float(w[i]), v.y * inv * __half2float(w[i + 1]),
                            v.z * inv * __half2float(w[i + 2]), v.w * inv * __half2float(w[i + 3])};
        if (out) *reinterpret_cast<float4*>(out + (size_t)r * dim + i) = make_float4(e[0], e[1], e[2], e[3]);
        xq_emit_oct(e, sub, gmask, xq + ((size_t)r * nblk + b) * XW);
    }
}

}  // namespace

namespace {
int rmsnorm_digits_(const float* x, const __half* w, int rows, int dim, float eps, float* out, uint32_t* xq, cudaStream_t st) {
    return launch_pdl(rmsnorm_digits_kernel, dim3(rows), dim3(1024), 0, st, x, w, dim, eps, out, xq);
}
}  // namespace

extern "C" size_t cmlb200_xq_bytes(int M, int K) { return cmlb200_xq_bytes_(M, K); }

extern "C" int cmlb200_x_digits(const float* d_x, int M, int K, void* d_xq, void* stream) {
    CMLB_REQUIRE(d_x && d_xq && M >= 1 && K > 0 && K % 32 == 0, "cmlb200_x_digits: bad argument");
    CMLB_REQUIRE(((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_xq & 15) == 0, "cmlb200_x_digits: pointers must be 16-byte aligned");
    return cmlb200_x_digits_(d_x, M, K, (uint32_t*)d_xq, as_stream(stream));
}

extern "C" int cmlb200_rmsnorm_digits(const float* d_x, const uint16_t* d_w_f16, int rows, int dim, float eps, float* d_out_f32,
                                      void* d_xq, void* stream) {
    CMLB_REQUIRE(d_x && d_w_f16 && d_xq && rows >= 1 && dim > 0 && dim % 32 == 0, "cmlb200_rmsnorm_digits: bad argument");
    CMLB_REQUIRE(((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_xq & 15) == 0 && ((uintptr_t)d_out_f32 & 15) == 0,
                 "cmlb200_rmsnorm_digits: pointers must be 16-byte aligned");
    return rmsnorm_digits_(d_x, (const __half*)d_w_f16, rows, dim, eps, d_out_f32, (uint32_t*)d_xq, as_stream(stream));
}

// epi: 0 store, 1 accumulate into y, 2 SwiGLU of (W, W2)
extern "C" int cmlb200_gemv_xq(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* d_xq, float* d_y, int M, int epi,
                               void* stream) {
    CMLB_REQUIRE(W && W->qs && W->scales && d_xq && d_y, "cmlb200_gemv_xq: NULL argument");
    CMLB_REQUIRE(W->type == CMLB200_Q4_0 || W->type == CMLB200_Q8_0, "cmlb200_gemv_xq: weight type %d is not Q4_0 or Q8_0", W->type);
    CMLB_REQUIRE(W->rows > 0 && W->cols > 0 && W->cols % 32 == 0, "cmlb200_gemv_xq: bad weight shape %dx%d", W->rows, W->cols);
    CMLB_REQUIRE(M >= 1 && M <= 4 && epi >= 0 && epi <= 2, "cmlb200_gemv_xq: M=%d must be 1..4 and epi=%d one of 0, 1, 2", M, epi);
    if (epi == EPI_SWIGLU)
        CMLB_REQUIRE(W2 && W2->qs && W2->scales && W2->type == W->type && W2->rows == W->rows && W2->cols == W->cols,
                     "cmlb200_gemv_xq: SwiGLU needs a second weight of the same type and shape");
    return cmlb200_gemv_dp4a_(W, epi == EPI_SWIGLU ? W2 : nullptr, nullptr, nullptr, 0.f, (const uint32_t*)d_xq, d_y, M, epi, as_stream(stream));
}

// y (= | += | swiglu) from rms_norm(x, norm_w, eps) without a separate normalisation launch.
extern "C" int cmlb200_gemv_rmsnorm(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* d_x, const uint16_t* d_norm_w_f16, float eps,
                                    float* d_y, int M, int epi, void* stream) {
    CMLB_REQUIRE(W && W->qs && W->scales && d_x && d_norm_w_f16 && d_y, "cmlb200_gemv_rmsnorm: NULL argument");
    CMLB_REQUIRE(W->type == CMLB200_Q4_0 || W->type == CMLB200_Q8_0, "cmlb200_gemv_rmsnorm: weight type %d is not Q4_0 or Q8_0", W->type);
    CMLB_REQUIRE(W->rows > 0 && W->cols > 0 && W->cols % 32 == 0, "cmlb200_gemv_rmsnorm: bad weight shape %dx%d", W->rows, W->cols);
    CMLB_REQUIRE(M >= 1 && M <= 8 && epi >= 0 && epi <= 2, "cmlb200_gemv_rmsnorm: M=%d must be 1..8 and epi=%d one of 0, 1, 2", M, epi);
    CMLB_REQUIRE(((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_norm_w_f16 & 7) == 0, "cmlb200_gemv_rmsnorm: x must be 16-byte, norm_w 8-byte aligned");
    if (epi == EPI_SWIGLU)
        CMLB_REQUIRE(W2 && W2->qs && W2->scales && W2->type == W->type && W2->rows == W->rows && W2->cols == W->cols,
                     "cmlb200_gemv_rmsnorm: SwiGLU needs a second weight of the same type and shape");
    return cmlb200_gemv_dp4a_(W, epi == EPI_SWIGLU ? W2 : nullptr, d_x, d_norm_w_f16, eps, nullptr, d_y, M, epi, as_stream(stream));
}
