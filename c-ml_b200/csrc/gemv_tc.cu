// Decode GEMV / skinny GEMM (M <= 32) for Q4_0 and Q8_0 on the tcgen05 integer tensor cores.
//
//   y[M,N] = x[M,K] . dequant(W[N,K])^T,  fp32 activations in, fp32 out.
//
// Why tensor cores for a GEMV: at HBM speed a B200 SM has a budget of about three
// lane-operations per 4-bit weight, and any CUDA-core path spends more than that on turning
// nibbles into numbers and multiplying them. Here the multiply-accumulate of a whole 32-element
// quantization block of 128 weight rows is ONE tcgen05.mma (kind::i8, 128 x NCOLS x 32):
//   * A operand = the quants themselves. Q8_0 bytes go from HBM to shared memory by bulk copy
//     and are consumed as they are; Q4_0 nibbles are split into two byte planes (one AND, one
//     shift+AND per word) on the way.
//   * B operand = the activations as exact small integers: per 32-block of x,
//         x_k ~= s_b * X_k,  X_k signed 21 bit,  X_k = d0*2^14 + d1*2^7 + d2  (7-bit digits),
//     one int8 column per digit (x_digits_tc_kernel writes them once per activation vector).
//   * D = exact int32 block dot products in tensor memory. The epilogue warps read them with
//     tcgen05.ld, recombine the digits, apply the block's fp16 scale d and the activation scale
//     s_b in fp32 and accumulate over the blocks of a row in fp32 registers.
// The only approximation is the 21-bit rounding of x relative to its block maximum
// (<= 2^-21 * max|x_block| per element).
//
// Weights are stored tile-major ("units"): for row tile t (128 rows) and block column b, one
// contiguous unit holds the 128 rows' quants of that block followed by their 128 fp16 scales
//   Q4_0: 128 x 16 B quants | 128 x 2 B scales            = 2304 B
//   Q8_0: 128 x 16 B (k 0..15) | 128 x 16 B (k 16..31) | scales = 4352 B
// so that a pipeline stage (BC consecutive units) is a single cp.async.bulk, and the Q8_0 unit
// already is the canonical K-major (no-swizzle) operand layout of the MMA.
// Work is split by contiguous ranges of stages (stream-K): every SM streams an equal share of
// the weight bytes; rows whose blocks are shared between two CTAs are combined with fp32
// atomics into y, which the digit kernel zeroes first.
//
// Replaces C-ML's dequantize-then-fp32-matmul (src/core/gguf.c:271-295 followed by
// src/ops/ir/execution.c:989-1052 / 3090-3134). No cluster multicast; every mbarrier wait is
// bounded and reports through cmlb200_gemm_status.
#include <string.h>
#include "common.cuh"

__device__ int g_tc_status = 0;   // 0 = ok; otherwise the code of the bounded wait that expired

namespace {

constexpr int ROWS = 128;
constexpr int XFULL = (1 << 20) - 1;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

template <int TYPE> struct Unit {
    static constexpr int qs_bytes = (TYPE == CMLB200_Q8_0) ? 4096 : 2048;
    static constexpr int bytes = qs_bytes + 256;
};
// B payload of one block column: NCOLS int8 columns x 32 k-bytes in two 16-byte k-planes, then
// MP activation scales (fp32) and MP block sums (int32).
template <int NCOLS> struct Pay {
    static constexpr int MP = NCOLS == 8 ? 2 : NCOLS == 16 ? 8 : NCOLS == 32 ? 16 : 32;
    static constexpr int tile = NCOLS * 32;
    static constexpr int bytes = tile + 8 * MP;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        if (mbar_try(bar, parity)) return true;
        if (it > 4096) {
            if (*abort_flag) return false;
            __nanosleep(32);
        }
    }
    *abort_flag = code;
    atomicCAS(&g_tc_status, 0, code);
    return false;
}
// one lane polls, the whole warp learns the verdict
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, bool ok) {
    int okl = ok ? 1 : 0;
    if (ok && (threadIdx.x & 31) == 0) okl = mbar_wait(bar, parity, abort_flag, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, okl, 0) != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// K-major, no swizzle: 8-row x 16-byte core matrices; rows of a core matrix 16 B apart, 8-row
// groups `sbo` bytes apart, the two 16-byte k-halves `lbo` bytes apart.
__device__ __forceinline__ uint64_t make_desc_none(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, 0, 0;\n"      // p = false: D is overwritten
                 " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int NV>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, int (&r)[NV]);
template <> __device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, int (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
}
template <> __device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, int (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
template <> __device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, int (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// ---- activations -> B payloads [bcol][ k-plane c ][ column n ][16 B] + scales + block sums.
// Column n = 3*m + j holds digit j of activation row m. One thread writes one 16-byte chunk
// (b, c, n); it re-derives the block maximum from the 32 floats of its block (served by L1).
// The same launch zeroes y (the GEMV accumulates into it with atomics) when asked to.
template <int NCOLS>
__global__ void __launch_bounds__(256)
x_digits_tc_kernel(const float* __restrict__ x, int M, int K, uint8_t* __restrict__ pay, float* __restrict__ y_zero,
                   size_t y_count) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    using P = Pay<NCOLS>;
    const int nblk = K / 32;
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (y_zero) {
        for (size_t i = gid; i < y_count; i += (size_t)gridDim.x * blockDim.x) y_zero[i] = 0.f;
    }
    const size_t chunks = (size_t)nblk * 2 * NCOLS;
    if (gid >= chunks) return;
    const int b = (int)(gid / (2 * NCOLS));
    const int c = (int)((gid / NCOLS) & 1), n = (int)(gid % NCOLS);
    uint8_t* dst = pay + (size_t)b * P::bytes + (size_t)c * (NCOLS * 16) + (size_t)n * 16;
    const int m = n / 3, j = n - 3 * m;
    uint4 outv = make_uint4(0, 0, 0, 0);
    if (m < M) {
        const float4* xp = reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)b * 32);
        float v[32];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float4 t = xp[i];
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w))));
        }
        const float inv = amax > 0.f ? (float)XFULL / amax : 0.f;
        uint32_t w[4] = {0, 0, 0, 0};
        int xsum = 0;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            int X = __float2int_rn(v[i] * inv);
            X = max(-XFULL, min(XFULL, X));
            xsum += X;
            const int d2 = ((X + 64) & 127) - 64;
            const int X1 = (X - d2) >> 7;
            const int d1 = ((X1 + 64) & 127) - 64;
            const int d0 = (X1 - d1) >> 7;
            const int dj = j == 0 ? d0 : (j == 1 ? d1 : d2);
            if ((i >> 4) == c) w[(i & 15) >> 2] |= (uint32_t)(dj & 0xFF) << (8 * (i & 3));
        }
        outv = make_uint4(w[0], w[1], w[2], w[3]);
        if (c == 0 && j == 0) {
            float* meta = reinterpret_cast<float*>(pay + (size_t)b * P::bytes + P::tile);
            meta[m] = amax / (float)XFULL;
            reinterpret_cast<int*>(meta)[P::MP + m] = xsum;
        }
    }
    *reinterpret_cast<uint4*>(dst) = outv;
}

// ---- the GEMV. grid = one CTA per SM; CTA c owns stages [c*G/grid, (c+1)*G/grid) where a stage
// is BC consecutive units of one row tile.
template <int TYPE, int NCOLS, int BC, int ST>
struct Smem {
    using U = Unit<TYPE>;
    using P = Pay<NCOLS>;
    static constexpr int raw_stage = BC * U::bytes;
    static constexpr int pay_stage = BC * P::bytes;
    static constexpr int a_stage = (TYPE == CMLB200_Q4_0) ? BC * 4096 : 0;
    static constexpr int raw_off = 0;
    static constexpr int pay_off = raw_off + ST * raw_stage;
    static constexpr int a_off = (pay_off + ST * pay_stage + 127) / 128 * 128;
    static constexpr int bar_off = a_off + ST * a_stage;
    static constexpr int total = bar_off + 8 * (4 * ST) + 32;
    static constexpr int tmem_cols_needed = ST * BC * NCOLS;
};

template <int TYPE, int NCOLS, int BC, int ST, int MMAX>
__global__ void __launch_bounds__(512, 1)
gemv_tc_kernel(const uint8_t* __restrict__ wt, const uint8_t* __restrict__ pay, float* __restrict__ y, int N, int nblk,
               int M, int total_stages, int dbg) {
    using L = Smem<TYPE, NCOLS, BC, ST>;
    using U = Unit<TYPE>;
    using P = Pay<NCOLS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + L::bar_off;
    auto full = [&](int s) { return bars + 8 * s; };
    auto aready = [&](int s) { return bars + 8 * (ST + s); };
    auto dready = [&](int s) { return bars + 8 * (2 * ST + s); };
    auto empty = [&](int s) { return bars + 8 * (3 * ST + s); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::bar_off + 8 * (4 * ST));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::bar_off + 8 * (4 * ST) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int spt = nblk / BC;                                    // stages per row tile
    const int g0 = (int)((long long)blockIdx.x * total_stages / gridDim.x);
    const int g1 = (int)((long long)(blockIdx.x + 1) * total_stages / gridDim.x);
    const int nst = g1 - g0;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < L::tmem_cols_needed) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; s++) {
            mbar_init(full(s), 1);
            mbar_init(aready(s), 4);
            mbar_init(dready(s), 1);
            mbar_init(empty(s), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer: one bulk copy of weights + one of activation payloads per stage
        if (lane == 0) {
            // Weights never depend on the preceding kernel: fill the ring before the
            // dependency wait; the activation payloads follow after it.
            const int pre = min(nst, ST);
            for (int i = 0; i < pre; i++) {
                mbar_expect_tx(full(i), (uint32_t)(L::raw_stage + L::pay_stage));
                bulk_g2s(sbase + L::raw_off + i * L::raw_stage, wt + (size_t)(g0 + i) * L::raw_stage, L::raw_stage, full(i));
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            for (int i = 0; i < pre; i++) {
                const int j = (g0 + i) % spt;
                bulk_g2s(sbase + L::pay_off + i * L::pay_stage, pay + (size_t)j * L::pay_stage, L::pay_stage, full(i));
            }
            int issued = pre;
            for (int i = ST; i < nst; i++) {
                const int s = i % ST;
                if (!mbar_wait(empty(s), ((i / ST) & 1) ^ 1, abort_flag, 11)) break;
                mbar_expect_tx(full(s), (uint32_t)(L::raw_stage + L::pay_stage));
                bulk_g2s(sbase + L::raw_off + s * L::raw_stage, wt + (size_t)(g0 + i) * L::raw_stage, L::raw_stage, full(s));
                bulk_g2s(sbase + L::pay_off + s * L::pay_stage, pay + (size_t)((g0 + i) % spt) * L::pay_stage, L::pay_stage, full(s));
                issued = i + 1;
            }
            for (int i = max(0, issued - ST); i < issued; i++)      // drain: no copy may outlive the CTA
                mbar_wait(full(i % ST), (i / ST) & 1, abort_flag, 12);
        } else {
            asm volatile("griddepcontrol.wait;" ::: "memory");
        }
    } else if (warp == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // ---------------- MMA issuer: one 128 x NCOLS x 32 integer MMA per unit
        if (lane == 0) {
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NCOLS >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
            for (int i = 0; i < nst; i++) {
                const int s = i % ST;
                const uint32_t ph = (i / ST) & 1;
                if (!mbar_wait(TYPE == CMLB200_Q4_0 ? aready(s) : full(s), ph, abort_flag, 13)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (dbg == 1 || dbg == 2) { mbar_arrive(dready(s)); continue; }
#pragma unroll
                for (int bc = 0; bc < BC; bc++) {
                    const uint32_t a_addr = (TYPE == CMLB200_Q4_0) ? sbase + L::a_off + s * L::a_stage + bc * 4096
                                                                   : sbase + L::raw_off + s * L::raw_stage + bc * U::bytes;
                    const uint64_t adesc = make_desc_none(a_addr, 2048, 128);
                    const uint64_t bdesc = make_desc_none(sbase + L::pay_off + s * L::pay_stage + bc * P::bytes, NCOLS * 16, 128);
                    umma_i8(tmem_base + (uint32_t)((s * BC + bc) * NCOLS), adesc, bdesc, idesc);
                }
                umma_commit(dready(s));
            }
        }
    } else if ((warp >= 4 && warp < 8) || warp >= 12) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // ---------------- epilogue: lane = weight row of the tile. Two warp sets (4..7 and
        // 12..15) take alternate stages so that one set's TMEM round trip overlaps the other's.
        const int set = warp >= 12 ? 1 : 0;
        const int q = warp & 3;
        const int r = q * 32 + lane;
        float acc[MMAX];
#pragma unroll
        for (int m = 0; m < MMAX; m++) acc[m] = 0.f;
        int cur_tile = -1;
        auto flush = [&](int tile) {
            const int row = tile * ROWS + r;
            if (tile >= 0 && row < N) {
#pragma unroll
                for (int m = 0; m < MMAX; m++)
                    if (m < M) atomicAdd(y + (size_t)m * N + row, acc[m]);
            }
#pragma unroll
            for (int m = 0; m < MMAX; m++) acc[m] = 0.f;
        };
        bool ok = true;
        for (int i = set; i < nst; i += 2) {
            const int s = i % ST;
            const uint32_t ph = (i / ST) & 1;
            const int tile = (g0 + i) / spt;
            if (tile != cur_tile) { flush(cur_tile); cur_tile = tile; }
            static_assert(3 * MMAX <= NCOLS, "digit columns exceed the MMA width");
            ok = warp_wait(dready(s), ph, abort_flag, 14, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (dbg) { __syncwarp(); if (lane == 0) mbar_arrive(empty(s)); continue; }
            int v[BC][NCOLS];
#pragma unroll
            for (int bc = 0; bc < BC; bc++)
                tmem_ld<NCOLS>(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((s * BC + bc) * NCOLS), v[bc]);
            float d[BC];
#pragma unroll
            for (int bc = 0; bc < BC; bc++)
                d[bc] = cml_half_to_float(*reinterpret_cast<const uint16_t*>(smem + L::raw_off + s * L::raw_stage + bc * U::bytes + U::qs_bytes + 2 * r));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int bc = 0; bc < BC; bc++) {
                const float* meta = reinterpret_cast<const float*>(smem + L::pay_off + s * L::pay_stage + bc * P::bytes + P::tile);
                const int* xsum = reinterpret_cast<const int*>(meta) + P::MP;
#pragma unroll
                for (int m = 0; m < MMAX; m++) {             // columns 3m..3m+2 = digits of activation row m
                    float t;
                    if (TYPE == CMLB200_Q4_0) t = (float)(v[bc][3 * m] * 16384 + v[bc][3 * m + 1] * 128 + v[bc][3 * m + 2] - 8 * xsum[m]);
                    else t = fmaf((float)v[bc][3 * m], 16384.0f, (float)(v[bc][3 * m + 1] * 128 + v[bc][3 * m + 2]));
                    acc[m] = fmaf(t, d[bc] * meta[m], acc[m]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));
        }
        flush(cur_tile);
    } else if (TYPE == CMLB200_Q4_0 && warp >= 8 && warp < 12) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // ---------------- nibble split: row r's 16 packed bytes -> low-nibble plane, high-nibble plane
        const int r = (warp - 8) * 32 + lane;
        bool ok = true;
        for (int i = 0; i < nst; i++) {
            const int s = i % ST;
            ok = warp_wait(full(s), (i / ST) & 1, abort_flag, 15, ok);
            if (!ok) break;
            if (dbg == 1) { __syncwarp(); if (lane == 0) mbar_arrive(aready(s)); continue; }
#pragma unroll
            for (int bc = 0; bc < BC; bc++) {
                const uint4 v = *reinterpret_cast<const uint4*>(smem + L::raw_off + s * L::raw_stage + bc * U::bytes + r * 16);
                uint8_t* a = smem + L::a_off + s * L::a_stage + bc * 4096 + r * 16;
                *reinterpret_cast<uint4*>(a) = make_uint4(v.x & 0x0F0F0F0Fu, v.y & 0x0F0F0F0Fu, v.z & 0x0F0F0F0Fu, v.w & 0x0F0F0F0Fu);
                *reinterpret_cast<uint4*>(a + 2048) = make_uint4((v.x >> 4) & 0x0F0F0F0Fu, (v.y >> 4) & 0x0F0F0F0Fu,
                                                                 (v.z >> 4) & 0x0F0F0F0Fu, (v.w >> 4) & 0x0F0F0F0Fu);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(aready(s));
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

constexpr size_t kPayScratchBytes = 4u << 20;
uint8_t* g_pay[16] = {};

int pay_scratch(uint8_t** out) {
    int dev = 0;
    CMLB_CUDA(cudaGetDevice(&dev));
    CMLB_REQUIRE(dev >= 0 && dev < 16, "device index %d out of range", dev);
    if (!g_pay[dev]) CMLB_CUDA(cudaMalloc((void**)&g_pay[dev], kPayScratchBytes));
    *out = g_pay[dev];
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

template <int TYPE, int NCOLS, int BC, int ST, int MMAX>
int run(const cmlb200_qmat* W, const float* x, float* y, int M, bool accumulate, cudaStream_t st, int dbg = 0) {
    using L = Smem<TYPE, NCOLS, BC, ST>;
    using P = Pay<NCOLS>;
    static_assert(L::tmem_cols_needed <= 512, "tensor memory ring too large");
    static_assert(L::total + 128 <= 227 * 1024, "shared memory ring too large");
    const int N = W->rows, K = W->cols, nblk = K / 32;
    CMLB_REQUIRE(nblk % BC == 0, "cmlb200_gemv: cols=%d must be a multiple of %d on the tensor-core path", K, 32 * BC);
    uint8_t* pay = nullptr;
    int rc = pay_scratch(&pay);
    if (rc) return rc;
    CMLB_REQUIRE((size_t)nblk * P::bytes <= kPayScratchBytes, "cmlb200_gemv: cols=%d too large for the activation scratch", K);
    const size_t chunks = (size_t)nblk * 2 * NCOLS;
    const size_t ycount = accumulate ? 0 : (size_t)M * N;
    size_t want = chunks > ycount / 4 ? chunks : ycount / 4;
    int dgrid = (int)((want + 255) / 256);
    rc = launch_pdl(x_digits_tc_kernel<NCOLS>, dim3(dgrid), dim3(256), 0, st, x, M, K, pay, accumulate ? (float*)nullptr : y, ycount);
    if (rc) return rc;
    const int ntiles = (N + ROWS - 1) / ROWS;
    const int total_stages = ntiles * (nblk / BC);
    int grid = cmlb_num_sms();
    if (grid > total_stages) grid = total_stages;
    auto kern = gemv_tc_kernel<TYPE, NCOLS, BC, ST, MMAX>;
    const int smem = L::total + 128;
    static bool attr_done = false;
    if (!attr_done) {
        CMLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_done = true;
    }
    return launch_pdl(kern, dim3(grid), dim3(512), (size_t)smem, st, (const uint8_t*)W->qs,
                      (const uint8_t*)pay, y, N, nblk, M, total_stages, dbg);
}

template <int TYPE>
int run_type(const cmlb200_qmat* W, const float* x, float* y, int M, bool accumulate, cudaStream_t st, int dbg = 0) {
    // NCOLS = 3 digit columns per activation row, rounded up to what the MMA accepts
    if (M <= 2) return run<TYPE, 8, 4, (TYPE == CMLB200_Q4_0 ? 6 : 8), 2>(W, x, y, M, accumulate, st, dbg);
    if (M <= 5) return run<TYPE, 16, 4, (TYPE == CMLB200_Q4_0 ? 6 : 6), 5>(W, x, y, M, accumulate, st);
    if (M <= 10) return run<TYPE, 32, 2, (TYPE == CMLB200_Q4_0 ? 8 : 8), 10>(W, x, y, M, accumulate, st);
    // larger M: chunks of 10 rows
    int rc = 0;
    for (int m0 = 0; m0 < M && rc == 0; m0 += 10) {
        const int mc = M - m0 < 10 ? M - m0 : 10;
        rc = run<TYPE, 32, 2, 8, 10>(W, x + (size_t)m0 * W->cols, y + (size_t)m0 * W->rows, mc, accumulate, st);
    }
    return rc;
}

}  // namespace

// Tile-major repack on the host: GGUF blocks [rows][cols/32] -> units [tile][bcol].
extern "C" size_t cmlb200_tiles_bytes(int type, int rows, int cols) {
    if (rows <= 0 || cols <= 0 || cols % 32) return 0;
    const size_t unit = type == CMLB200_Q8_0 ? 4352 : type == CMLB200_Q4_0 ? 2304 : 0;
    return unit * (size_t)((rows + ROWS - 1) / ROWS) * (size_t)(cols / 32);
}

extern "C" int cmlb200_repack_tiles(int type, const void* h_blocks, int rows, int cols, void* h_tiles) {
    CMLB_REQUIRE(h_blocks && h_tiles, "cmlb200_repack_tiles: NULL argument");
    CMLB_REQUIRE(type == CMLB200_Q4_0 || type == CMLB200_Q8_0, "cmlb200_repack_tiles: type %d is not a GGUF block type on this path", type);
    CMLB_REQUIRE(rows > 0 && cols > 0 && cols % 32 == 0, "cmlb200_repack_tiles: cols (%d) must be a positive multiple of 32", cols);
    const int nblk = cols / 32, ntiles = (rows + ROWS - 1) / ROWS;
    const int bb = type == CMLB200_Q8_0 ? 34 : 18;
    const size_t unit = type == CMLB200_Q8_0 ? 4352 : 2304;
    const size_t qsb = unit - 256;
    const uint8_t* src = (const uint8_t*)h_blocks;
    uint8_t* dst = (uint8_t*)h_tiles;
    memset(dst, 0, unit * (size_t)ntiles * nblk);
    for (int row = 0; row < rows; row++) {
        const int t = row / ROWS, r = row % ROWS;
        for (int b = 0; b < nblk; b++) {
            const uint8_t* blk = src + ((size_t)row * nblk + b) * bb;
            uint8_t* u = dst + ((size_t)t * nblk + b) * unit;
            memcpy(u + qsb + 2 * r, blk, 2);
            if (type == CMLB200_Q4_0) memcpy(u + r * 16, blk + 2, 16);
            else { memcpy(u + r * 16, blk + 2, 16); memcpy(u + 2048 + r * 16, blk + 18, 16); }
        }
    }
    return CMLB200_OK;
}

extern "C" int cmlb200_unrepack_tiles(int type, const void* h_tiles, int rows, int cols, void* h_blocks) {
    CMLB_REQUIRE(h_blocks && h_tiles, "cmlb200_unrepack_tiles: NULL argument");
    CMLB_REQUIRE(type == CMLB200_Q4_0 || type == CMLB200_Q8_0, "cmlb200_unrepack_tiles: type %d is not a GGUF block type on this path", type);
    CMLB_REQUIRE(rows > 0 && cols > 0 && cols % 32 == 0, "cmlb200_unrepack_tiles: cols (%d) must be a positive multiple of 32", cols);
    const int nblk = cols / 32;
    const int bb = type == CMLB200_Q8_0 ? 34 : 18;
    const size_t unit = type == CMLB200_Q8_0 ? 4352 : 2304;
    const size_t qsb = unit - 256;
    const uint8_t* src = (const uint8_t*)h_tiles;
    uint8_t* dst = (uint8_t*)h_blocks;
    for (int row = 0; row < rows; row++) {
        const int t = row / ROWS, r = row % ROWS;
        for (int b = 0; b < nblk; b++) {
            uint8_t* blk = dst + ((size_t)row * nblk + b) * bb;
            const uint8_t* u = src + ((size_t)t * nblk + b) * unit;
            memcpy(blk, u + qsb + 2 * r, 2);
            if (type == CMLB200_Q4_0) memcpy(blk + 2, u + r * 16, 16);
            else { memcpy(blk + 2, u + r * 16, 16); memcpy(blk + 18, u + 2048 + r * 16, 16); }
        }
    }
    return CMLB200_OK;
}

// y[M, rows] (=|+=) x[M, cols] . W^T with W in the tile-major layout (W->qs; W->scales unused).
extern "C" int cmlb200_gemv_tiles(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, int accumulate, void* stream) {
    CMLB_REQUIRE(W && W->qs && d_x && d_y, "cmlb200_gemv_tiles: NULL argument");
    CMLB_REQUIRE(W->type == CMLB200_Q4_0 || W->type == CMLB200_Q8_0, "cmlb200_gemv_tiles: unsupported weight type %d", W->type);
    CMLB_REQUIRE(W->rows > 0 && W->cols > 0 && W->cols % 128 == 0, "cmlb200_gemv_tiles: cols=%d must be a positive multiple of 128", W->cols);
    CMLB_REQUIRE(M >= 1 && M <= 32, "cmlb200_gemv_tiles: M=%d outside the decode range 1..32", M);
    CMLB_REQUIRE(((uintptr_t)W->qs & 15) == 0 && ((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_y & 15) == 0,
                 "cmlb200_gemv_tiles: pointers must be 16-byte aligned");
    cudaStream_t st = as_stream(stream);
    if (W->type == CMLB200_Q8_0) return run_type<CMLB200_Q8_0>(W, d_x, d_y, M, accumulate != 0, st);
    return run_type<CMLB200_Q4_0>(W, d_x, d_y, M, accumulate != 0, st);
}

extern "C" int cmlb200_gemv_tiles_status(int* status, int reset) {
    CMLB_REQUIRE(status, "cmlb200_gemv_tiles_status: NULL argument");
    CMLB_CUDA(cudaDeviceSynchronize());
    CMLB_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        CMLB_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
    }
    return CMLB200_OK;
}

// Experiment hook (not declared in the public header): dbg = 1 copies only, 2 adds the nibble
// split, 3 adds the MMAs; results are meaningless for dbg != 0.
extern "C" int cmlb200_gemv_tiles_dbg_(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, int dbg, void* stream) {
    cudaStream_t st = as_stream(stream);
    if (W->type == CMLB200_Q8_0) return run_type<CMLB200_Q8_0>(W, d_x, d_y, M, false, st, dbg);
    return run_type<CMLB200_Q4_0>(W, d_x, d_y, M, false, st, dbg);
}
