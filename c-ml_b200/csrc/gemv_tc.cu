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
//     one int8 column per digit (built in shared memory by every CTA for M <= 2, or once per
//     activation matrix by x_digits_tc_kernel into a scratch buffer for larger M).
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
// the weight bytes. A row tile whose blocks are shared between CTAs is finished by the CTA that
// owns its first stage: the others leave their partial sums in a scratch slot and raise a flag
// (they reach that point early, the finisher late, so the bounded wait is short); the result is
// deterministic and needs no zero-initialised output.
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
constexpr uint32_t SPIN_LIMIT = 1u << 21;

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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, int stage = -1) {
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        if (mbar_try(bar, parity)) return true;
        if (it > 4096) {
            if (*abort_flag) return false;
            __nanosleep(32);
        }
    }
    *abort_flag = code;
    (void)stage;
    atomicCAS(&g_tc_status, 0, code);
    return false;
}
// Every lane waits on the barrier itself (each reader of bytes that a bulk copy wrote has to observe
// the barrier's phase on its own); the verdict is then made warp-uniform.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, bool ok, int stage = -1) {
    bool mine = ok;
    if (ok) {
        mine = false;
        for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
            if (mbar_try(bar, parity)) { mine = true; break; }
            if (it > 4096) {
                if (*abort_flag) break;
                __nanosleep(32);
            }
        }
        if (!mine && !*abort_flag) { *abort_flag = code; atomicCAS(&g_tc_status, 0, code); }
    }
    (void)stage;
    return __all_sync(0xffffffffu, mine);
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


// Writes the digits of 4 consecutive activations (elements 4*sub..4*sub+3 of block `b`, row m)
// into a payload laid out as [k-plane c][column n][16 B] + scales + block sums. Called by groups
// of 8 lanes (sub = 0..7) that share one (block, row) pair; `gmask` names the group's lanes.
template <int NCOLS>
__device__ __forceinline__ void write_digits(uint8_t* payload, const float4 v, int m, int sub, unsigned gmask) {
    using P = Pay<NCOLS>;
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o));
    const float inv = amax > 0.f ? (float)XFULL / amax : 0.f;
    const float e[4] = {v.x, v.y, v.z, v.w};
    uint32_t w0 = 0, w1 = 0, w2 = 0;
    int xsum = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int X = __float2int_rn(e[i] * inv);
        X = max(-XFULL, min(XFULL, X));
        xsum += X;
        const int d2 = ((X + 64) & 127) - 64;
        const int X1 = (X - d2) >> 7;
        const int d1 = ((X1 + 64) & 127) - 64;
        const int d0 = (X1 - d1) >> 7;
        w0 |= (uint32_t)(d0 & 0xFF) << (8 * i);
        w1 |= (uint32_t)(d1 & 0xFF) << (8 * i);
        w2 |= (uint32_t)(d2 & 0xFF) << (8 * i);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) xsum += __shfl_xor_sync(gmask, xsum, o);
    uint32_t* dst = reinterpret_cast<uint32_t*>(payload + (sub >> 2) * (NCOLS * 16) + (3 * m) * 16 + (sub & 3) * 4);
    dst[0] = w0;
    dst[4] = w1;       // next column: +16 bytes
    dst[8] = w2;
    if (sub == 0) {
        float* meta = reinterpret_cast<float*>(payload + P::tile);
        meta[m] = amax / (float)XFULL;
        reinterpret_cast<int*>(meta)[P::MP + m] = xsum;
    }
}

// ---- activations -> B payloads in a global scratch buffer, one payload per block column
// (used when M is too large to rebuild the payloads inside every CTA).
template <int NCOLS>
__global__ void __launch_bounds__(256)
x_digits_tc_kernel(const float* __restrict__ x, int M, int K, uint8_t* __restrict__ pay) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    using P = Pay<NCOLS>;
    const int nblk = K / 32;
    const int gid = blockIdx.x * 256 + threadIdx.x;
    // unused columns must read as zero
    for (int i = gid; i < nblk * (P::bytes / 16); i += gridDim.x * 256) {
        const int b = i / (P::bytes / 16), ch = i % (P::bytes / 16);
        const int n = ch % NCOLS;
        if (ch < 2 * NCOLS && n >= 3 * M) reinterpret_cast<uint4*>(pay + (size_t)b * P::bytes)[ch] = make_uint4(0, 0, 0, 0);
    }
    const int item = gid >> 3, sub = gid & 7;
    if (item < nblk * M) {
        const int b = item / M, m = item - b * M;
        const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)b * 32 + sub * 4);
        write_digits<NCOLS>(pay + (size_t)b * P::bytes, v, m, sub, 0xffu << (threadIdx.x & 24));
    }
}

enum { EPI_STORE = 0, EPI_ACCUM = 1 };
constexpr int TBCAP = 160;          // block columns whose payloads a CTA can keep in shared memory

template <int TYPE, int NCOLS, int BC, int RS, int AS, int MMAX, bool INLINE>
struct Smem {
    using U = Unit<TYPE>;
    using P = Pay<NCOLS>;
    static constexpr int raw_stage = BC * U::bytes;
    static constexpr int pay_stage = INLINE ? 0 : BC * P::bytes;
    static constexpr int a_stage = (TYPE == CMLB200_Q4_0) ? BC * 4096 : 0;
    static constexpr int raw_off = 0;
    static constexpr int pay_off = raw_off + RS * raw_stage;
    static constexpr int a_off = (pay_off + RS * pay_stage + 127) / 128 * 128;
    static constexpr int table_off = a_off + AS * a_stage;
    static constexpr int red_off = table_off + (INLINE ? TBCAP * P::bytes : 0);
    static constexpr int bar_off = red_off + ROWS * MMAX * 4;
    static constexpr int total = bar_off + 8 * (2 * RS + 3 * AS) + 64;
    static constexpr int tmem_cols_needed = AS * BC * NCOLS;
    static constexpr int threads = (TYPE == CMLB200_Q4_0) ? 640 : 512;
};

// grid = one CTA per SM; CTA c owns stages [c*G/grid, (c+1)*G/grid) where a stage is BC
// consecutive units (block columns) of one 128-row tile.
//   warp 0       producer: one bulk copy per stage into a ring of RS raw stages
//   warp 1       allocates tensor memory; one lane issues the MMAs
//   warps 4-7, 12-15   two epilogue sets taking alternate stages
//   warps 8-11, 16-19  (Q4_0) two nibble-split sets taking alternate stages, ring of AS planes
template <int TYPE, int NCOLS, int BC, int RS, int AS, int MMAX, bool INLINE>
__global__ void __launch_bounds__((TYPE == CMLB200_Q4_0) ? 640 : 512, 1)
gemv_tc_kernel(const uint8_t* __restrict__ wt, const uint8_t* __restrict__ pay, const float* __restrict__ x,
               float* __restrict__ y, float* __restrict__ slots, int* __restrict__ flags, int N, int K, int M,
               int total_stages, int epi) {
    using L = Smem<TYPE, NCOLS, BC, RS, AS, MMAX, INLINE>;
    using U = Unit<TYPE>;
    using P = Pay<NCOLS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + L::bar_off;
    auto full = [&](int s) { return bars + 8 * s; };
    auto rempty = [&](int s) { return bars + 8 * (RS + s); };
    auto aready = [&](int s) { return bars + 8 * (2 * RS + s); };
    auto dready = [&](int s) { return bars + 8 * (2 * RS + AS + s); };
    auto aempty = [&](int s) { return bars + 8 * (2 * RS + 2 * AS + s); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::bar_off + 8 * (2 * RS + 3 * AS));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::bar_off + 8 * (2 * RS + 3 * AS) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = K / 32;
    const int spt = nblk / BC;                                    // stages per row tile
    auto start_of = [&](int cta) { return (int)((long long)cta * total_stages / gridDim.x); };
    const int g0 = start_of(blockIdx.x), g1 = start_of(blockIdx.x + 1);
    const int nst = g1 - g0;
    const int tb_first = (g0 % spt) * BC;                         // first block column of the payload table
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < L::tmem_cols_needed) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; s++) { mbar_init(full(s), 1); mbar_init(rempty(s), 4); }
        for (int s = 0; s < AS; s++) { mbar_init(aready(s), 4); mbar_init(dready(s), 1); mbar_init(aempty(s), 4); }
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
        // ---------------- producer. Weights never depend on the preceding kernel, so the ring is
        // filled before the dependency wait; anything derived from activations comes after it.
        if (lane == 0) {
            constexpr uint32_t stage_tx = (uint32_t)(L::raw_stage + L::pay_stage);
            const int pre = min(nst, RS);
            for (int i = 0; i < pre; i++) {
                mbar_expect_tx(full(i), stage_tx);
                bulk_g2s(sbase + L::raw_off + i * L::raw_stage, wt + (size_t)(g0 + i) * L::raw_stage, L::raw_stage, full(i));
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            if (!INLINE)
                for (int i = 0; i < pre; i++)
                    bulk_g2s(sbase + L::pay_off + i * L::pay_stage, pay + (size_t)((g0 + i) % spt) * L::pay_stage, L::pay_stage, full(i));
            int issued = pre;
            for (int i = RS; i < nst; i++) {
                const int s = i % RS;
                if (!mbar_wait(rempty(s), ((i / RS) & 1) ^ 1, abort_flag, 11, i)) break;
                mbar_expect_tx(full(s), stage_tx);
                bulk_g2s(sbase + L::raw_off + s * L::raw_stage, wt + (size_t)(g0 + i) * L::raw_stage, L::raw_stage, full(s));
                if (!INLINE)
                    bulk_g2s(sbase + L::pay_off + s * L::pay_stage, pay + (size_t)((g0 + i) % spt) * L::pay_stage, L::pay_stage, full(s));
                issued = i + 1;
            }
            for (int i = max(0, issued - RS); i < issued; i++)      // drain: no copy may outlive the CTA
                mbar_wait(full(i % RS), (i / RS) & 1, abort_flag, 12, i);
        } else {
            asm volatile("griddepcontrol.wait;" ::: "memory");
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (INLINE) {
            // Every CTA rebuilds the digit payloads of the block columns it will meet (a
            // contiguous run of at most TBCAP columns, modulo the row length).
            constexpr int NT = L::threads - 32;
            const int t = threadIdx.x - 32;
            const int need = min(nblk, nst * BC);
            uint4* tab = reinterpret_cast<uint4*>(smem + L::table_off);
            for (int i = t; i < need * (P::bytes / 16); i += NT) tab[i] = make_uint4(0, 0, 0, 0);
            asm volatile("bar.sync 3, %0;" ::"n"(NT) : "memory");
            for (int item = t >> 3; item < ((need * M + 3) & ~3); item += NT / 8) {   // whole warps iterate together
                if (item < need * M) {
                    const int slot = item / M, m = item - slot * M;
                    int b = tb_first + slot;
                    if (b >= nblk) b -= nblk;
                    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)b * 32 + (t & 7) * 4);
                    write_digits<NCOLS>(smem + L::table_off + slot * P::bytes, v, m, t & 7, 0xffu << (t & 24));
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 3, %0;" ::"n"(NT) : "memory");
        }
        // shared-memory address of the payload of stage i, block column bc
        auto pay_ptr = [&](int i, int bc) -> uint32_t {
            if (INLINE) {
                int slot = ((g0 + i) % spt) * BC + bc - tb_first;
                if (slot < 0) slot += nblk;
                return (uint32_t)(L::table_off + slot * P::bytes);
            }
            return (uint32_t)(L::pay_off + (i % RS) * L::pay_stage + bc * P::bytes);
        };

        if (warp == 1) {
            // ---------------- MMA issuer: one 128 x NCOLS x 32 integer MMA per unit
            if (lane == 0) {
                const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NCOLS >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
                for (int i = 0; i < nst; i++) {
                    const int rs = i % RS, as = i % AS;
                    bool ok;
                    if (TYPE == CMLB200_Q4_0) ok = mbar_wait(aready(as), (i / AS) & 1, abort_flag, 13, i);
                    else ok = mbar_wait(full(rs), (i / RS) & 1, abort_flag, 19, i) && mbar_wait(aempty(as), ((i / AS) & 1) ^ 1, abort_flag, 16, i);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int bc = 0; bc < BC; bc++) {
                        const uint32_t a_addr = (TYPE == CMLB200_Q4_0) ? sbase + L::a_off + as * L::a_stage + bc * 4096
                                                                       : sbase + L::raw_off + rs * L::raw_stage + bc * U::bytes;
                        const uint64_t adesc = make_desc_none(a_addr, 2048, 128);
                        const uint64_t bdesc = make_desc_none(sbase + pay_ptr(i, bc), NCOLS * 16, 128);
                        umma_i8(tmem_base + (uint32_t)((as * BC + bc) * NCOLS), adesc, bdesc, idesc);
                    }
                    umma_commit(dready(as));
                }
            }
        } else if ((warp >= 4 && warp < 8) || (warp >= 12 && warp < 16)) {
            // ---------------- epilogue: lane = weight row of the tile
            const int set = warp >= 12 ? 1 : 0;
            const int q = warp & 3;
            const int r = q * 32 + lane;
            float* red = reinterpret_cast<float*>(smem + L::red_off);
            bool ok = true;
            const int tile_first = nst > 0 ? g0 / spt : 0, tile_last = nst > 0 ? (g1 - 1) / spt : -1;
            for (int T = tile_first; T <= tile_last; T++) {
                const int seg_b = max(g0, T * spt), seg_e = min(g1, (T + 1) * spt);
                float acc[MMAX];
#pragma unroll
                for (int m = 0; m < MMAX; m++) acc[m] = 0.f;
                int i0 = seg_b - g0;
                if ((i0 & 1) != set) i0++;
                for (int i = i0; i < seg_e - g0 && ok; i += 2) {
                    const int rs = i % RS, as = i % AS;
                    ok = warp_wait(dready(as), (i / AS) & 1, abort_flag, 14, ok, i);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    static_assert(3 * MMAX <= NCOLS, "digit columns exceed the MMA width");
                    int v[BC][NCOLS];
#pragma unroll
                    for (int bc = 0; bc < BC; bc++)
                        tmem_ld<NCOLS>(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((as * BC + bc) * NCOLS), v[bc]);
                    float d[BC];
#pragma unroll
                    for (int bc = 0; bc < BC; bc++)
                        d[bc] = cml_half_to_float(*reinterpret_cast<const uint16_t*>(smem + L::raw_off + rs * L::raw_stage + bc * U::bytes + U::qs_bytes + 2 * r));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int bc = 0; bc < BC; bc++) {
                        const float* meta = reinterpret_cast<const float*>(smem + pay_ptr(i, bc) + P::tile);
                        const int* xsum = reinterpret_cast<const int*>(meta) + P::MP;
#pragma unroll
                        for (int m = 0; m < MMAX; m++) {         // columns 3m..3m+2 = digits of activation row m
                            float t;
                            if (TYPE == CMLB200_Q4_0) t = (float)(v[bc][3 * m] * 16384 + v[bc][3 * m + 1] * 128 + v[bc][3 * m + 2] - 8 * xsum[m]);
                            else t = fmaf((float)v[bc][3 * m], 16384.0f, (float)(v[bc][3 * m + 1] * 128 + v[bc][3 * m + 2]));
                            acc[m] = fmaf(t, d[bc] * meta[m], acc[m]);
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(rempty(rs)); mbar_arrive(aempty(as)); }
                }
                // ---- finish the segment: set 1 hands its partial sums to set 0 ...
                if (set == 1) {
#pragma unroll
                    for (int m = 0; m < MMAX; m++) red[m * ROWS + r] = acc[m];
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (set == 0) {
#pragma unroll
                    for (int m = 0; m < MMAX; m++) acc[m] += red[m * ROWS + r];
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (set == 0) {
                    const int row = T * ROWS + r;
                    if (seg_b == T * spt) {
                        // ... this CTA owns the tile's first stage: collect the partial sums of the
                        // CTAs that own its later stages, then write the result
                        for (int cc = blockIdx.x + 1; cc < (int)gridDim.x && start_of(cc) < (T + 1) * spt; cc++) {
                            int seen = 0;
                            if (lane == 0) {
                                for (uint32_t it = 0; it < SPIN_LIMIT && !seen; ++it) {
                                    seen = *reinterpret_cast<volatile int*>(flags + cc);
                                    if (!seen && it > 1024) __nanosleep(64);
                                }
                                if (!seen) atomicCAS(&g_tc_status, 0, 17);
                            }
                            __syncwarp();
                            __threadfence();
#pragma unroll
                            for (int m = 0; m < MMAX; m++)
                                if (m < M) acc[m] += __ldcg(slots + ((size_t)cc * MMAX + m) * ROWS + r);
                            asm volatile("bar.sync 2, 128;" ::: "memory");
                            if (threadIdx.x == 128) *reinterpret_cast<volatile int*>(flags + cc) = 0;
                        }
                        if (row < N) {
#pragma unroll
                            for (int m = 0; m < MMAX; m++)
                                if (m < M) {
                                    float* out = y + (size_t)m * N + row;
                                    *out = (epi == EPI_ACCUM) ? *out + acc[m] : acc[m];
                                }
                        }
                    } else {
                        // ... otherwise leave the partial sums for the owner and raise the flag
#pragma unroll
                        for (int m = 0; m < MMAX; m++)
                            if (m < M) __stcg(slots + ((size_t)blockIdx.x * MMAX + m) * ROWS + r, acc[m]);
                        __threadfence();
                        asm volatile("bar.sync 2, 128;" ::: "memory");
                        if (threadIdx.x == 128) *reinterpret_cast<volatile int*>(flags + blockIdx.x) = 1;
                    }
                }
            }
        } else if (TYPE == CMLB200_Q4_0 && ((warp >= 8 && warp < 12) || warp >= 16)) {
            // ---------------- nibble split: row r's 16 packed bytes -> low-nibble plane, high-nibble plane
            const int set = warp >= 16 ? 1 : 0;
            const int r = (warp & 3) * 32 + lane;
            bool ok = true;
            for (int i = set; i < nst; i += 2) {
                const int rs = i % RS, as = i % AS;
                ok = warp_wait(full(rs), (i / RS) & 1, abort_flag, 15, ok, i);
                ok = warp_wait(aempty(as), ((i / AS) & 1) ^ 1, abort_flag, 18, ok, i);
                if (!ok) break;
                uint4 v[BC];
#pragma unroll
                for (int bc = 0; bc < BC; bc++)
                    v[bc] = *reinterpret_cast<const uint4*>(smem + L::raw_off + rs * L::raw_stage + bc * U::bytes + r * 16);
#pragma unroll
                for (int bc = 0; bc < BC; bc++) {
                    uint8_t* a = smem + L::a_off + as * L::a_stage + bc * 4096 + r * 16;
                    *reinterpret_cast<uint4*>(a) = make_uint4(v[bc].x & 0x0F0F0F0Fu, v[bc].y & 0x0F0F0F0Fu, v[bc].z & 0x0F0F0F0Fu, v[bc].w & 0x0F0F0F0Fu);
                    *reinterpret_cast<uint4*>(a + 2048) = make_uint4((v[bc].x >> 4) & 0x0F0F0F0Fu, (v[bc].y >> 4) & 0x0F0F0F0Fu,
                                                                     (v[bc].z >> 4) & 0x0F0F0F0Fu, (v[bc].w >> 4) & 0x0F0F0F0Fu);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(aready(as));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// Per-device scratch of the plain entry point: digit payloads (large M), stream-K partial
// sums and their flags. Allocated once, never moved, so captured CUDA graphs stay valid.
constexpr size_t kPayBytes = 4u << 20;
constexpr int kMaxGrid = 256, kSlotFloats = kMaxGrid * 10 * ROWS;
struct Scratch { uint8_t* pay; float* slots; int* flags; };
Scratch g_scratch[16] = {};

int get_scratch(Scratch** out) {
    int dev = 0;
    CMLB_CUDA(cudaGetDevice(&dev));
    CMLB_REQUIRE(dev >= 0 && dev < 16, "device index %d out of range", dev);
    Scratch& s = g_scratch[dev];
    if (!s.pay) {
        uint8_t* base = nullptr;
        const size_t bytes = kPayBytes + (size_t)kSlotFloats * 4 + kMaxGrid * 4;
        CMLB_CUDA(cudaMalloc((void**)&base, bytes));
        CMLB_CUDA(cudaMemset(base, 0, bytes));
        s.pay = base;
        s.slots = reinterpret_cast<float*>(base + kPayBytes);
        s.flags = reinterpret_cast<int*>(base + kPayBytes + (size_t)kSlotFloats * 4);
    }
    *out = &s;
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

template <int TYPE, int NCOLS, int BC, int RS, int AS, int MMAX, bool INLINE>
int run_cfg(const cmlb200_qmat* W, const float* x, float* y, int M, int epi, Scratch* sc, int grid, int total_stages,
            cudaStream_t st) {
    using L = Smem<TYPE, NCOLS, BC, RS, AS, MMAX, INLINE>;
    // Two warp sets take alternate stages; with even ring depths a ring slot is always served by
    // the same set, so every mbarrier has one in-order waiter and its 1-bit phase parity cannot
    // alias (an odd depth lets one set run two phases ahead of the other).
    static_assert(RS % 2 == 0 && AS % 2 == 0, "ring depths must be even");
    static_assert(L::tmem_cols_needed <= 512, "tensor memory ring too large");
    static_assert(L::total + 128 <= 227 * 1024, "shared memory ring too large");
    static_assert(MMAX <= 10, "scratch slots hold at most 10 activation rows");
    auto kern = gemv_tc_kernel<TYPE, NCOLS, BC, RS, AS, MMAX, INLINE>;
    const int smem = L::total + 128;
    static size_t attr_smem[kMaxDevices] = {};
    CMLB_CUDA(cmlb_ensure_smem(kern, (size_t)smem, attr_smem));
    return launch_pdl(kern, dim3(grid), dim3(L::threads), (size_t)smem, st, (const uint8_t*)W->qs, (const uint8_t*)sc->pay, x, y,
                      sc->slots, sc->flags, W->rows, W->cols, M, total_stages, epi);
}

template <int TYPE, int NCOLS, int BC, int RS, int AS, int MMAX>
int run(const cmlb200_qmat* W, const float* x, float* y, int M, int epi, cudaStream_t st) {
    using P = Pay<NCOLS>;
    const int N = W->rows, K = W->cols, nblk = K / 32;
    CMLB_REQUIRE(nblk % BC == 0, "cmlb200_gemv_tiles: cols=%d must be a multiple of %d", K, 32 * BC);
    Scratch* sc = nullptr;
    int rc = get_scratch(&sc);
    if (rc) return rc;
    const int ntiles = (N + ROWS - 1) / ROWS;
    const int total_stages = ntiles * (nblk / BC);
    int grid = cmlb_num_sms();
    if (grid > kMaxGrid) grid = kMaxGrid;
    if (grid > total_stages) grid = total_stages;
    const int nst_max = (total_stages + grid - 1) / grid;
    const int need = nblk < nst_max * BC ? nblk : nst_max * BC;
    if (NCOLS == 8 && need <= TBCAP)
        return run_cfg<TYPE, NCOLS, BC, RS, AS, MMAX, (NCOLS == 8)>(W, x, y, M, epi, sc, grid, total_stages, st);
    CMLB_REQUIRE((size_t)nblk * P::bytes <= kPayBytes, "cmlb200_gemv_tiles: cols=%d too large for the activation scratch", K);
    rc = launch_pdl(x_digits_tc_kernel<NCOLS>, dim3((nblk * M * 8 + 255) / 256), dim3(256), 0, st, x, M, K, sc->pay);
    if (rc) return rc;
    return run_cfg<TYPE, NCOLS, BC, (NCOLS == 8 ? RS - 2 : RS), AS, MMAX, false>(W, x, y, M, epi, sc, grid, total_stages, st);
}

template <int TYPE>
int run_type(const cmlb200_qmat* W, const float* x, float* y, int M, int epi, cudaStream_t st) {
    constexpr bool Q4 = TYPE == CMLB200_Q4_0;
    // NCOLS = 3 digit columns per activation row, rounded up to what the MMA accepts
    if (M <= 2) return run<TYPE, 8, 4, 8, 4, 2>(W, x, y, M, epi, st);
    if (M <= 5) return run<TYPE, 16, 4, (Q4 ? 8 : 6), 4, 5>(W, x, y, M, epi, st);
    int rc = 0;                                               // larger M: chunks of up to 10 rows
    for (int m0 = 0; m0 < M && rc == 0; m0 += 10) {
        const int mc = M - m0 < 10 ? M - m0 : 10;
        rc = run<TYPE, 32, 2, (Q4 ? 12 : 10), 4, 10>(W, x + (size_t)m0 * W->cols, y + (size_t)m0 * W->rows, mc, epi, st);
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

// Used by cmlb200_gemv's dispatcher: same as cmlb200_gemv_tiles on W->tiles.
int cmlb200_gemv_tc_(const cmlb200_qmat* W, const float* x, float* y, int M, int accumulate, cudaStream_t st) {
    cmlb200_qmat T = *W;
    T.qs = W->tiles;
    if (W->type == CMLB200_Q8_0) return run_type<CMLB200_Q8_0>(&T, x, y, M, accumulate ? EPI_ACCUM : EPI_STORE, st);
    return run_type<CMLB200_Q4_0>(&T, x, y, M, accumulate ? EPI_ACCUM : EPI_STORE, st);
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
    if (W->type == CMLB200_Q8_0) return run_type<CMLB200_Q8_0>(W, d_x, d_y, M, accumulate ? EPI_ACCUM : EPI_STORE, st);
    return run_type<CMLB200_Q4_0>(W, d_x, d_y, M, accumulate ? EPI_ACCUM : EPI_STORE, st);
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

