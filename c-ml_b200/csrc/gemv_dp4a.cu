// Decode GEMV for Q4_0 / Q8_0 at M <= 4, built to stay under the instruction-issue budget
// that HBM speed leaves per weight (about 3 lane-operations per 4-bit weight on B200).
//
// A straight fp32 path needs ~4 operations per weight just to turn a nibble into a float and
// multiply it. Here the activation vector is re-expressed as block-fixed-point: for every
// 32-element block of x (the same blocks the weights are quantized in)
//     x_k  ~=  s_b * X_k,   X_k a signed 16-bit integer,  s_b = max|x_block| / 32639,
// and X_k is split into two signed 8-bit digits X_k = d0*256 + d1 held as int8x4 words. The
// block dot product  sum_k q_k * X_k  then is two exact integer dot products on dp4a (4
// multiply-adds per lane-operation), recombined in int32 and scaled by d_b * s_b in fp32;
// blocks are accumulated in fp32. Q4_0 nibbles are turned into the signed bytes 16*(q-8) with
// one shift and two 3-input logic operations per 8 weights, so the "-8" offset costs nothing
// and the factor 16 is taken out once per output. The only approximation is the rounding of x
// to 16 bits relative to its block maximum (relative output error of a few 1e-5), far inside
// the 2e-3 tolerance of this path.
//
// Replaces, like gemv.cu, C-ML's dequantize-then-fp32-matmul (src/core/gguf.c:271-295 +
// src/ops/ir/execution.c:989-1052, 3090-3134).
//
// Two kernels:
//   * gemv_stream_kernel (K % 256 == 0): one persistent CTA per SM. Every warp runs its own
//     ring of NBUF shared-memory buffers filled by bulk copies (cp.async.bulk + mbarrier), one
//     buffer = R weight rows x up to KC blocks with their scales, so each SM keeps
//     WARPS*NBUF buffers in flight from launch to exit; the digits of x sit in shared memory
//     and are either produced in the kernel from fp32 x or copied from a record array made by
//     the kernel that produced the activations. Weight copies are issued before
//     griddepcontrol.wait (programmatic dependent launch), x is touched only after it.
//   * gemv_dp4a_kernel (any K % 32 == 0): register path, each warp loads its rows straight
//     from global memory; digits come from a record array.
#include "common.cuh"

int cmlb200_x_digits_(const float* x, int M, int K, uint32_t* xq, cudaStream_t st);
// gemv_mma.cu: the tensor-core kernel for the shapes it takes
bool cmlb200_gemv_mma_ok_(const cmlb200_qmat* W, int epi, int M);
int cmlb200_gemv_mma_(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const uint16_t* norm_w, float eps,
                      const uint32_t* xq, float* y, int M, int epi, cudaStream_t st);

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

// ---- streaming kernel ---------------------------------------------------------------------------
constexpr int SPIN_LIMIT = 1 << 22;
__device__ int g_stream_status = 0;          // 0 ok; else 1 + index of the buffer whose wait expired

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the phase did not complete within SPIN_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < SPIN_LIMIT; i++)
        if (mbar_try(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

#ifdef CMLB200_TRACE
// Diagnostic build only: per CTA and launch, global-timer stamps at kernel entry, after the
// dependency wait, after the digits are in place and at exit.
__device__ unsigned long long g_trace[16][160][4];
__device__ unsigned int g_trace_cnt[160];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRACE_SLOT() unsigned tr_slot = 0; if (threadIdx.x == 0) { tr_slot = atomicAdd(&g_trace_cnt[blockIdx.x], 1u) % 16; }
#define TRACE(k) if (threadIdx.x == 0) g_trace[tr_slot][blockIdx.x][k] = gtime();
#else
#define TRACE_SLOT()
#define TRACE(k)
#endif

template <int TYPE, int NW, int R, bool DREG>
struct StreamCfg {
    static constexpr int QB = (TYPE == CMLB200_Q8_0) ? 32 : 16;      // quant bytes per block
    static constexpr int KC = 128;                                   // blocks per buffer and row
    static constexpr int QS_BYTES = NW * R * KC * QB;
    static constexpr int BUF_BYTES = QS_BYTES + NW * R * KC * 2;     // + fp16 scales
    // shared memory left for the rings once the digit records are placed
    static constexpr int BUDGET = DREG ? 200 * 1024 : 150 * 1024;
    static constexpr int SW0 = DREG ? 12 : 16;
    static constexpr int SW = (BUDGET / (SW0 * BUF_BYTES) >= 2) ? SW0 : 8;       // warps per CTA
    static constexpr int NBUF = (BUDGET / (SW * BUF_BYTES) >= 4) ? 4 : BUDGET / (SW * BUF_BYTES);
    static_assert(NBUF >= 2, "ring too small");
    static constexpr int BAR_BYTES = 128 * ((SW * NBUF * 8 + 127) / 128);
    __host__ __device__ static size_t digit_bytes(int MT, int nblk) { return 128 * (((size_t)MT * nblk * XW * 4 + 127) / 128); }
};

// xin: digit records [MT][K/32][XW] (XMODE 0), fp32 activations [MT][K] (XMODE 1), or fp32
// activations to be RMS-normalised with the fp16 weight nw first (XMODE 2; src/nn/llama.c:71-124:
// x * (1 / sqrt(mean(x^2) + eps)) * w, every CTA normalising its own copy). y: [MT][N].
// Work unit = (group of R consecutive rows, chunk of KC blocks); warp w of the grid owns groups
// w, w + total_warps, ... and walks their chunks in order. Buffer i of a warp holds its unit i,
// i + NBUF, ...; the warp refills a buffer as soon as all its lanes have finished reading it.
// DREG (MT == 1 and K <= 32*KC): each lane keeps the digits of its own blocks in registers for
// the whole kernel, so the inner loop reads only weights from shared memory.
template <int TYPE, int MT, int R, int EPI, bool QUIRK, int XMODE, bool DREG>
__global__ void __launch_bounds__(StreamCfg<TYPE, (EPI == EPI_SWIGLU) ? 2 : 1, R, DREG>::SW * 32, 1)
gemv_stream_kernel(const uint8_t* __restrict__ qs, const uint16_t* __restrict__ scales,
                   const uint8_t* __restrict__ qs2, const uint16_t* __restrict__ scales2,
                   const void* __restrict__ xin, const __half* __restrict__ nw, float eps, float* __restrict__ y, int N, int K) {
    constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
    using C = StreamCfg<TYPE, NW, R, DREG>;
    constexpr int QB = C::QB, KC = C::KC, QV = QB / 16, SW = C::SW, NBUF = C::NBUF, NJ = KC / 32;
    static_assert(!DREG || MT == 1, "register-resident digits are for one row of x");
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = K / 32;
    const int nch = (nblk + KC - 1) / KC;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                       // [SW][NBUF]
    uint32_t* xd = reinterpret_cast<uint32_t*>(smem + C::BAR_BYTES);          // [MT][nblk][XW]
    uint8_t* ring = smem + C::BAR_BYTES + C::digit_bytes(MT, nblk) + (size_t)warp * NBUF * C::BUF_BYTES;
    const uint32_t bar0 = smem_u32(bars + warp * NBUF);
    const uint32_t ring0 = smem_u32(ring);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    TRACE_SLOT();
    TRACE(0);
    if (threadIdx.x == 0) {
        for (int i = 0; i < SW * NBUF; i++) mbar_init(smem_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int groups = (N + R - 1) / R;
    const int total_warps = gridDim.x * SW;
    const int gw = warp * gridDim.x + blockIdx.x;
    const int my_groups = gw < groups ? (groups - gw + total_warps - 1) / total_warps : 0;
    const int n_it = my_groups * nch;
    const size_t row_bytes = (size_t)nblk * QB;

    // fill buffer `buf` with unit `it`
    auto issue = [&](int it, int buf) {
        const int gi = it / nch, c = it - gi * nch;
        const int row0 = (gw + gi * total_warps) * R;
        const int nb = min(KC, nblk - c * KC);
        const int nrows = min(R, N - row0);
        const uint32_t bar = bar0 + 8 * buf, dst = ring0 + buf * C::BUF_BYTES;
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)(NW * nrows * nb * (QB + 2)));
        __syncwarp();
        if (lane < 2 * NW * R) {
            const int what = lane & 1, ar = lane >> 1, a = ar / R, r = ar - a * R;     // what: 0 quants, 1 scales
            if (r < nrows) {
                const int row = row0 + r;
                if (what == 0)
                    bulk_g2s(dst + ar * (KC * QB), (a ? qs2 : qs) + (size_t)row * row_bytes + (size_t)c * KC * QB, (uint32_t)(nb * QB), bar);
                else
                    bulk_g2s(dst + C::QS_BYTES + ar * (KC * 2), (a ? scales2 : scales) + (size_t)row * nblk + (size_t)c * KC, (uint32_t)(nb * 2), bar);
            }
        }
    };

    // Weights do not depend on the preceding kernel: fill the ring before the dependency wait.
    for (int i = 0; i < NBUF && i < n_it; i++) issue(i, i);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    TRACE(1);

    if (XMODE != 0) {      // digits of x, 8 lanes per block
        const float* x = static_cast<const float*>(xin);
        float inv[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) inv[m] = 1.f;
        if (XMODE == 2) {
            __shared__ float red[SW][MT];
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float ss = 0.f;
                for (int i = threadIdx.x * 4; i < K; i += SW * 128) {
                    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + i);
                    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) red[warp][m] = ss;
            }
            __syncthreads();
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < SW; w++) tot += red[w][m];
                inv[m] = 1.0f / sqrtf(tot / (float)K + eps);
            }
        }
        const int sub = threadIdx.x & 7;
        const unsigned gmask = 0xffu << (threadIdx.x & 24);
#pragma unroll
        for (int m = 0; m < MT; m++)
            for (int b = threadIdx.x >> 3; b < nblk; b += SW * 4) {
                const int i = b * 32 + sub * 4;
                const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + i);
                float e[4] = {v.x, v.y, v.z, v.w};
                if (XMODE == 2) {
                    const uint2 wr = *reinterpret_cast<const uint2*>(nw + i);
                    const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&wr.x));
                    const float2 w23 = __half22float2(*reinterpret_cast<const __half2*>(&wr.y));
                    e[0] = e[0] * inv[m] * w01.x; e[1] = e[1] * inv[m] * w01.y;
                    e[2] = e[2] * inv[m] * w23.x; e[3] = e[3] * inv[m] * w23.y;
                }
                xq_emit_oct(e, sub, gmask, xd + ((size_t)m * nblk + b) * XW);
            }
    } else {
        const uint4* src = static_cast<const uint4*>(xin);
        uint4* dst = reinterpret_cast<uint4*>(xd);
        for (int i = threadIdx.x; i < MT * nblk * (XW / 4); i += SW * 32) dst[i] = src[i];
    }
    __syncthreads();
    TRACE(2);

    uint32_t dg[DREG ? NJ : 1][24];
    float xsr[DREG ? NJ : 1];
    if (DREG) {
#pragma unroll
        for (int j = 0; j < (DREG ? NJ : 1); j++) {
            const int b = min(lane + 32 * j, nblk - 1);
            load_digits(xd + (size_t)b * XW, dg[j]);
            xsr[j] = __uint_as_float(xd[(size_t)b * XW + 24]);
        }
    }

    float acc[NW][R][MT];
#pragma unroll
    for (int a = 0; a < NW; a++)
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int m = 0; m < MT; m++) acc[a][r][m] = 0.f;

    int it = 0;
    bool ok = true;
    for (; it < n_it; it++) {
        const int buf = it % NBUF;
        if (!mbar_wait(bar0 + 8 * buf, (uint32_t)(it / NBUF) & 1u)) { ok = false; break; }
        const int gi = it / nch, c = it - gi * nch;
        const uint8_t* bq = ring + (size_t)buf * C::BUF_BYTES;
        const uint16_t* bs = reinterpret_cast<const uint16_t*>(bq + C::QS_BYTES);
        const int nb = min(KC, nblk - c * KC);
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int b = lane + 32 * j;
            if (b < nb) {
                uint4 q[NW * R][QV];
                uint16_t dh[NW * R];
#pragma unroll
                for (int ar = 0; ar < NW * R; ar++) {
#pragma unroll
                    for (int v = 0; v < QV; v++) q[ar][v] = *reinterpret_cast<const uint4*>(bq + ar * (KC * QB) + b * QB + 16 * v);
                    dh[ar] = bs[ar * KC + b];
                }
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    uint32_t dl[24];
                    float xsl = 0.f;
                    if (!DREG) {
                        const uint32_t* xb = xd + ((size_t)m * nblk + c * KC + b) * XW;
                        load_digits(xb, dl);
                        xsl = __uint_as_float(xb[24]);
                    }
                    const uint32_t (&dd)[24] = DREG ? dg[DREG ? j : 0] : dl;
                    const float xs = DREG ? xsr[DREG ? j : 0] : xsl;
#pragma unroll
                    for (int a = 0; a < NW; a++)
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const float t = block_dot<TYPE>(q[a * R + r][0], q[a * R + r][QV - 1], dd);
                            const float d = QUIRK ? cml_half_to_float(dh[a * R + r]) : __half2float(__ushort_as_half(dh[a * R + r]));
                            acc[a][r][m] = fmaf(t, d * xs, acc[a][r][m]);
                        }
                }
            }
        }
        __syncwarp();                                       // every lane is done with this buffer
        if (it + NBUF < n_it) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(it + NBUF, buf);
        }
        if (c == nch - 1) {                                 // last chunk of the group: reduce and write
            const int row0 = (gw + gi * total_warps) * R;
#pragma unroll
            for (int a = 0; a < NW; a++)
#pragma unroll
                for (int r = 0; r < R; r++)
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        float v = acc[a][r][m];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        acc[a][r][m] = v * kDotUnit<TYPE>;
                    }
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    if (row0 + r < N) {
#pragma unroll
                        for (int m = 0; m < MT; m++) {
                            float* out = y + (size_t)m * N + row0 + r;
                            if (EPI == EPI_STORE) *out = acc[0][r][m];
                            else if (EPI == EPI_ACCUM) *out += acc[0][r][m];
                            else {
                                const float g = acc[0][r][m];
                                *out = (g / (1.0f + expf(-g))) * acc[NW - 1][r][m];
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int a = 0; a < NW; a++)
#pragma unroll
                for (int r = 0; r < R; r++)
#pragma unroll
                    for (int m = 0; m < MT; m++) acc[a][r][m] = 0.f;
        }
    }
    if (!ok) {
        // A copy never landed. Record it, then give the copies still addressed to this warp's
        // buffers one more bounded chance to finish before the CTA's shared memory is released.
        if (lane == 0) atomicCAS(&g_stream_status, 0, 1 + it % NBUF);
        for (int k = it; k < n_it && k < it + NBUF; k++) (void)mbar_wait(bar0 + 8 * (k % NBUF), (uint32_t)(k / NBUF) & 1u);
    }
#ifdef CMLB200_TRACE
    __syncthreads();
    TRACE(3);
#endif
}

template <int TYPE, int MT, int EPI, bool QUIRK, int XMODE, bool DREG>
int launch_stream_cfg(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, cudaStream_t st) {
    constexpr int NW = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr int R = (DREG || EPI == EPI_SWIGLU) ? 1 : 2;
    using C = StreamCfg<TYPE, NW, R, DREG>;
    const int N = W->rows, K = W->cols, nblk = K / 32;
    const size_t smem = C::BAR_BYTES + C::digit_bytes(MT, nblk) + (size_t)C::SW * C::NBUF * C::BUF_BYTES;
    auto kern = gemv_stream_kernel<TYPE, MT, R, EPI, QUIRK, XMODE, DREG>;
    static size_t attr_smem = 0;
    if (smem > attr_smem) {
        CMLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem = smem;
    }
    const int groups = (N + R - 1) / R;
    const int grid = min(cmlb_num_sms(), (groups + C::SW - 1) / C::SW);
    return launch_pdl(kern, dim3(grid), dim3(C::SW * 32), smem, st, (const uint8_t*)W->qs, (const uint16_t*)W->scales,
                      W2 ? (const uint8_t*)W2->qs : (const uint8_t*)nullptr,
                      W2 ? (const uint16_t*)W2->scales : (const uint16_t*)nullptr, xin, nw, eps, y, N, K);
}

template <int TYPE, int MT, int EPI, bool QUIRK, int XMODE>
int launch_stream(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* xin, const __half* nw, float eps, float* y, cudaStream_t st) {
    if (MT == 1 && W->cols <= 32 * 128) return launch_stream_cfg<TYPE, 1, EPI, QUIRK, XMODE, true>(W, W2, xin, nw, eps, y, st);
    return launch_stream_cfg<TYPE, MT, EPI, QUIRK, XMODE, false>(W, W2, xin, nw, eps, y, st);
}

// The streaming kernel needs 16-byte aligned row chunks of the scale plane (K % 256 == 0) and
// room for the digits of MT rows of x next to the rings.
inline bool stream_ok(const cmlb200_qmat* W, int MT) {
    return W->cols % 256 == 0 && (size_t)MT * (W->cols / 32) * XW * 4 <= 80 * 1024 &&
           ((uintptr_t)W->qs & 15) == 0 && ((uintptr_t)W->scales & 15) == 0;
}

template <int TYPE, int MT, int EPI, bool QUIRK>
int launch(const cmlb200_qmat* W, const cmlb200_qmat* W2, const uint32_t* xq, float* y, int m0, cudaStream_t st) {
    constexpr int R = (EPI == EPI_SWIGLU) ? 2 : 4;
    constexpr int U = (TYPE == CMLB200_Q8_0) ? 1 : 2;
    const int N = W->rows, K = W->cols;
    const size_t smem = (size_t)(K / 32) * MT * XW * sizeof(uint32_t);
    CMLB_REQUIRE(smem <= 200 * 1024, "cmlb200_gemv: K=%d too large for the shared-memory activation digits", K);
    auto kern = gemv_dp4a_kernel<TYPE, MT, R, U, EPI, QUIRK>;
    static size_t attr_smem = 0;
    if (smem > 48 * 1024 && smem > attr_smem) {
        CMLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem = smem;
    }
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
// x != NULL: fp32 activations, RMS-normalised with nw first when nw != NULL (digits made in the
// streaming kernel, or in `ws` for the register kernel); else xq holds the digit records.
template <int TYPE, int EPI, bool QUIRK>
int run_type(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* x, const __half* nw, float eps, const uint32_t* xq,
             uint32_t* ws, float* y, int M, cudaStream_t st) {
    const int N = W->rows, K = W->cols, nblk = K / 32;
    auto digits_to_ws = [&]() -> int {
        const int rc = nw ? rmsnorm_digits_(x, nw, M, K, eps, nullptr, ws, st) : cmlb200_x_digits_(x, M, K, ws, st);
        xq = ws;
        x = nullptr;
        return rc;
    };
    if (x && !stream_ok(W, 1)) {
        const int rc = digits_to_ws();
        if (rc) return rc;
    }
    int m0 = 0, rc = 0;
    while (m0 < M && rc == 0) {
        const int mt = (M - m0 >= 2) ? 2 : 1;
        float* ym = y + (size_t)m0 * N;
        if (stream_ok(W, mt)) {
            if (x && nw) {
                const float* xm = x + (size_t)m0 * K;
                rc = mt == 2 ? launch_stream<TYPE, 2, EPI, QUIRK, 2>(W, W2, xm, nw, eps, ym, st) : launch_stream<TYPE, 1, EPI, QUIRK, 2>(W, W2, xm, nw, eps, ym, st);
            } else if (x) {
                const float* xm = x + (size_t)m0 * K;
                rc = mt == 2 ? launch_stream<TYPE, 2, EPI, QUIRK, 1>(W, W2, xm, nullptr, 0.f, ym, st) : launch_stream<TYPE, 1, EPI, QUIRK, 1>(W, W2, xm, nullptr, 0.f, ym, st);
            } else {
                const uint32_t* qm = xq + (size_t)m0 * nblk * XW;
                rc = mt == 2 ? launch_stream<TYPE, 2, EPI, QUIRK, 0>(W, W2, qm, nullptr, 0.f, ym, st) : launch_stream<TYPE, 1, EPI, QUIRK, 0>(W, W2, qm, nullptr, 0.f, ym, st);
            }
        } else {
            if (!xq) {       // shape fits the streaming kernel for one row but not two: digits on demand
                rc = digits_to_ws();
                if (rc) return rc;
            }
            rc = mt == 2 ? launch<TYPE, 2, EPI, QUIRK>(W, W2, xq, y, m0, st) : launch<TYPE, 1, EPI, QUIRK>(W, W2, xq, y, m0, st);
        }
        m0 += mt;
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
    if (cmlb200_gemv_mma_ok_(W, epi, M)) return cmlb200_gemv_mma_(W, W2, xq ? nullptr : x, norm_w, eps, xq, y, M, epi, st);
    uint32_t* ws = nullptr;
    if (xq) x = nullptr;
    else if (!stream_ok(W, 2)) {      // the register kernel may be needed: it reads digits from the library's scratch
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

// Device-side health word of the streaming kernel: 0 while every bounded wait has completed.
extern "C" int cmlb200_gemv_status(int* status, int reset) {
    CMLB_REQUIRE(status, "cmlb200_gemv_status: NULL argument");
    CMLB_CUDA(cudaDeviceSynchronize());
    CMLB_CUDA(cudaMemcpyFromSymbol(status, g_stream_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        CMLB_CUDA(cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int)));
    }
    return CMLB200_OK;
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
