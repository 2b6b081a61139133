// Prefill dequant-GEMM on the 5th-generation tensor cores (sm_100a):
//   Y[M,N] (bf16) = X[M,K] (bf16) . dequant(W[N,K])^T, fp32 accumulation in tensor memory.
//
// Replaces C-ML's "dequantize the whole weight to an fp32 temporary, then a scalar
// triple loop" (src/nn/qlora.c:264-317) and its dequantize-at-load + fp32 matmul
// (src/core/gguf.c:271-295, src/ops/ir/execution.c:989-1052).
//
// One CTA owns a tile of 128 weight rows (the MMA "M" side, operand A) by MT <= 256 (or 512: two MMAs
// per K step into two accumulators, so that a weight slab is expanded once for 512 activation rows;
// chosen where a cost model says it saves CTA waves)
// activation rows (the MMA "N" side, operand B) and walks K in slabs of 64:
//   warp 0      one lane issues TMA tensor loads of the bf16 activation slab (128B swizzle)
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128 x MT x 16, kind::f16)
//   warps 2..17 expand the packed weights to bf16 and store them in the canonical K-major
//               128B-swizzled layout the MMA reads. Expanding a slab is a chain of dependent
//               steps (wait, load, convert, store, fence, signal) of about a microsecond whatever
//               the number of threads sharing it, so the sixteen warps form four groups and
//               group g takes slabs g, g+4, g+8, ...: four slabs are in flight at once.
//               Afterwards the same warps are the epilogue: tcgen05.ld the fp32 accumulators,
//               round to bf16 and write Y
//   warp 18     one lane issues TMA tensor loads of the PACKED weights (a [128 rows x 32 or 64
//               byte] box per slab, into a ring) and of their scales (a [128 rows x 8 slabs]
//               box per 8 slabs), so that no warp gathers 128 different cache lines per slab
// Expansion cost decides this kernel (a slab of 8192 weights per 128 x 256 x 64 MMA group):
//   Q4_0  no table: a byte permute drops two nibbles into the mantissas of two bf16 halves
//         (0x43nn = 128 + n), one packed subtract gives n - 8 exactly, one packed multiply
//         applies the block scale: 15 instructions per 8 weights, nothing read from shared memory
//   NF4   one 4-byte table entry per packed BYTE (both code values as bf16), the table kept in
//         8 copies so that lanes rarely meet in a bank, one packed multiply by the block scale
//   Q8_0  convert, multiply in fp32, round once
// Q4_0 and NF4 therefore round twice (scale or code value to bf16, then the product); the path's
// tolerance is 1e-2 of the largest output. No cluster multicast is used. Every wait on an
// mbarrier is bounded; on expiry the CTA raises a status flag (cmlb200_gemm_status), waits for
// its copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include "common.cuh"

namespace {

constexpr int BN = 128;             // weight rows per CTA (MMA M)
constexpr int BK = 64;              // K slab: 64 bf16 = one 128-byte swizzle row
constexpr int DQ_WARPS = 16;
constexpr int DQ_GROUPS = 4;                    // slabs being expanded at once
constexpr int GROUP_WARPS = DQ_WARPS / DQ_GROUPS;
constexpr int DQ_THREADS = DQ_WARPS * 32;
constexpr int THREADS = 64 + DQ_THREADS + 32;
constexpr int A_BYTES = BN * BK * 2;            // 16 KB
constexpr int B_HALF = 256 * BK * 2;            // 32 KB: 256 activation rows, what one MMA instruction takes
constexpr int SC_SLABS = 8;                     // slabs per scale box (4 bytes per row and slab)
constexpr int SC_BYTES = BN * SC_SLABS * 4;     // 4 KB
constexpr uint32_t SPIN_LIMIT = 1u << 22;

// WIDE: tiles of up to 512 activation rows (two MMA instructions per K step on the same expanded
// weight slab, accumulators side by side in all 512 columns of tensor memory): the expansion, which
// decides this kernel, is paid once per 512 instead of once per 256 activation rows. The activation
// ring then holds two 64 KB stages; the narrow form keeps as many activation as weight stages.
template <int TYPE, bool WIDE> struct Cfg {
    static constexpr int RAWB = (TYPE == CMLB200_Q8_0) ? 64 : 32;       // packed bytes per row and slab
    // The expanded-weight (A) stages and the packed-weight ring have exactly one slot per expansion
    // group: group g then only ever reuses slot g, whose previous user was its own previous slab, so a
    // parity wait can never be two phases away from the barrier (with fewer slots than groups a fast
    // group could see "phase complete" for a phase that has not begun: a first Q8_0 configuration
    // with three stages had that flaw).
    static constexpr int STAGES = DQ_GROUPS;
    static constexpr int RSTAGES = DQ_GROUPS;
    // activation (B) stages: producer and consumer are one thread each and move in lockstep
    static constexpr int BSTAGES = WIDE ? 2 : (TYPE == CMLB200_Q8_0 ? 3 : 4);
    static constexpr int B_STAGE = WIDE ? 2 * B_HALF : B_HALF;
    static constexpr int RAW_STAGE = BN * RAWB;
    static constexpr int LUT_BYTES = (TYPE == CMLB200_NF4) ? 8 * 256 * 4 : 0;
    // offsets from the 1024-byte aligned base
    static constexpr int a_off = 0;
    static constexpr int b_off = STAGES * A_BYTES;
    static constexpr int raw_off = b_off + BSTAGES * B_STAGE;
    static constexpr int sc_off = raw_off + RSTAGES * RAW_STAGE;
    static constexpr int lut_off = sc_off + 2 * SC_BYTES;
    static constexpr int bar_off = lut_off + LUT_BYTES;
    static constexpr int nbars = 2 * STAGES + 2 * BSTAGES + 1 + 2 * RSTAGES + 2;
    static constexpr int total = bar_off + 8 * nbars + 32;
};

__device__ int g_gemm_status = 0;   // 0 = ok; otherwise a code identifying the wait that expired

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
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and raises the abort flag) when the limit is hit or when
// another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        if (mbar_try(bar, parity)) return true;
        if (it > 1024) {
            if (*abort_flag) return false;
            __nanosleep(32);
        }
    }
    *abort_flag = code;
    atomicCAS(&g_gemm_status, 0, code);
    return false;
}
// Every lane waits on the barrier itself (each reader of bytes that a tensor load wrote has to
// observe the barrier's phase on its own); the verdict is then made warp-uniform so that no lane
// is left behind at a __syncwarp.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, bool ok) {
    bool mine = ok;
    if (ok) {
        mine = false;
        for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
            if (mbar_try(bar, parity)) { mine = true; break; }
            if (it > 1024) {
                if (*abort_flag) break;
                __nanosleep(32);
            }
        }
        if (!mine && !*abort_flag) { *abort_flag = code; atomicCAS(&g_gemm_status, 0, code); }
    }
    return __all_sync(0xffffffffu, mine);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
    // K-major, 128-byte swizzle: 8-row groups 1024 B apart (SBO), LBO unused (=1), version 1
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t bf162_mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf162_sub(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Expand the 32 weights this thread owns (row n, K offset k0 + 32*h) into four 16-byte
// chunks of bf16, in element order. `raw`: the thread's packed bytes (16, or 32 for Q8_0).
template <int TYPE>
__device__ __forceinline__ void expand32(const uint4 (&raw)[2], float scale, const uint32_t* lut, int lane, uint4 (&out)[4]) {
    if (TYPE == CMLB200_Q8_0) {
        const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t o[4];
#pragma unroll
            for (int p = 0; p < 4; p++) {
                const uint32_t word = w[2 * c + (p >> 1)];
                const int sh = (p & 1) * 16;
                const float a = (float)(int)(int8_t)((word >> sh) & 0xFF) * scale;
                const float b = (float)(int)(int8_t)((word >> (sh + 8)) & 0xFF) * scale;
                o[p] = pack_bf16(a, b);
            }
            out[c] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else if (TYPE == CMLB200_NF4) {
        // word i = bytes 4i..4i+3 = elements 8i..8i+7; lut[byte] = (bf16 of the high-nibble code, of the low-nibble code)
        const uint32_t w[4] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w};
        const uint32_t s2 = pack_bf16(scale, scale);
        const uint32_t* tab = lut + (lane & 7);
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t o[4];
#pragma unroll
            for (int p = 0; p < 4; p++) o[p] = bf162_mul(tab[((w[c] >> (8 * p)) & 0xFF) << 3], s2);
            out[c] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else {
        // Q4_0: byte j -> element j (low nibble) and j+16 (high nibble). 0x43nn as bf16 is 128 + n.
        const uint32_t w[4] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w};
        const uint32_t s2 = pack_bf16(scale, scale);
        const uint32_t bias = 0x43084308u;                 // (136, 136): 128 + n - 136 = n - 8
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t l4 = w[i] & 0x0F0F0F0Fu, h4 = (w[i] >> 4) & 0x0F0F0F0Fu;
            lo[2 * i] = bf162_mul(bf162_sub(__byte_perm(l4, 0x43434343u, 0x4140), bias), s2);
            lo[2 * i + 1] = bf162_mul(bf162_sub(__byte_perm(l4, 0x43434343u, 0x4342), bias), s2);
            hi[2 * i] = bf162_mul(bf162_sub(__byte_perm(h4, 0x43434343u, 0x4140), bias), s2);
            hi[2 * i + 1] = bf162_mul(bf162_sub(__byte_perm(h4, 0x43434343u, 0x4342), bias), s2);
        }
        out[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        out[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
        out[2] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        out[3] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
    }
}

// What happens to a finished output value (the sum over all of K) at flat index i of [M, N]:
//   GEMM_OUT_BF16    stored as bf16                         (the plain product)
//   GEMM_OUT_F32     stored as fp32                         (Q/K/V: RoPE and attention read fp32)
//   GEMM_ACC_F32     added to an fp32 array                 (attention-out and FFN-down onto the residual,
//                                                            src/nn/llama.c:523-530, 538-543)
//   GEMM_SWIGLU_BF16 silu(gate[i]) * value stored as bf16   (the up projection finishing SwiGLU,
//                                                            src/nn/llama.c:126-155; gate may be the output array)
enum { GEMM_OUT_BF16 = 0, GEMM_OUT_F32 = 1, GEMM_ACC_F32 = 2, GEMM_SWIGLU_BF16 = 3 };
__device__ __forceinline__ void epilogue_store(void* out, const __nv_bfloat16* gate, int mode, size_t i, float v) {
    if (mode == GEMM_OUT_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else if (mode == GEMM_OUT_F32) static_cast<float*>(out)[i] = v;
    else if (mode == GEMM_ACC_F32) static_cast<float*>(out)[i] += v;
    else {
        const float g = __bfloat162float(gate[i]);
        static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * v);
    }
}

// grid = (ceil(N/128), ceil(M/MT), splits); MT <= 256, or 512 in the WIDE form. With splits > 1 each z-slice covers a K range and
// writes fp32 partial sums [split][M][N] to `partial`; a second kernel reduces them.
// SCTMA: the scales come as 4 bytes per row and slab (two fp16 of Q4_0 / Q8_0, or one fp32 of NF4
// with block 64) through the tensor map `smap`; otherwise every expansion thread loads its own.
template <int TYPE, bool SCTMA, bool WIDE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
            const __grid_constant__ CUtensorMap smap, const void* __restrict__ scales, void* __restrict__ out,
            const __nv_bfloat16* __restrict__ gate, int mode, float* __restrict__ partial, int M, int N, int K, int MT,
            int nf4_block, int kb_per_split) {
    using C = Cfg<TYPE, WIDE>;
    constexpr int STAGES = C::STAGES, BST = C::BSTAGES, RS = C::RSTAGES, RAWB = C::RAWB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + C::bar_off;
    // barrier slots (8 B each)
    constexpr int NB0 = 2 * STAGES + 2 * BST;
    auto full_a = [&](int s) { return bars + 8 * s; };
    auto empty = [&](int s) { return bars + 8 * (STAGES + s); };
    auto full_b = [&](int s) { return bars + 8 * (2 * STAGES + s); };
    // (slots 2 * STAGES + BST .. 2 * STAGES + 2 * BST - 1 of the barrier area are spare)
    const uint32_t accum_bar = bars + 8 * NB0;
    auto raw_full = [&](int s) { return bars + 8 * (NB0 + 1 + s); };
    auto raw_empty = [&](int s) { return bars + 8 * (NB0 + 1 + RS + s); };
    auto sc_full = [&](int s) { return bars + 8 * (NB0 + 1 + 2 * RS + s); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::bar_off + 8 * C::nbars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::bar_off + 8 * C::nbars + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * MT;
    const int total_kb = (K + BK - 1) / BK;          // K % 64 == 32: the last slab's upper half is zero
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(total_kb, kb_begin + kb_per_split);
    const int nkb = kb_end - kb_begin;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < MT) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full_a(s), GROUP_WARPS); mbar_init(empty(s), 1); }
        for (int s = 0; s < BST; s++) mbar_init(full_b(s), 1);
        mbar_init(accum_bar, 1);
        for (int s = 0; s < RS; s++) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), GROUP_WARPS); }
        for (int s = 0; s < 2; s++) mbar_init(sc_full(s), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (TYPE == CMLB200_NF4 && threadIdx.x >= 64 && threadIdx.x < 64 + 256) {
        // byte -> (high-nibble code, low-nibble code) as two bf16, eight copies interleaved
        uint32_t* lut = reinterpret_cast<uint32_t*>(smem + C::lut_off);
        const int b = threadIdx.x - 64;
        const uint32_t e = pack_bf16(kNF4[b >> 4], kNF4[b & 15]);
#pragma unroll
        for (int c = 0; c < 8; c++) lut[b * 8 + c] = e;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer: activation slabs (operand B) ----------------
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < nkb; i++) {
                const int s = i % BST;
                // stage s was last read by the MMAs of slab i - BST, whose completion the issuer signals
                // on that slab's weight-stage barrier (one commit per slab serves both rings)
                if (i >= BST && !mbar_wait(empty((i - BST) % STAGES), ((i - BST) / STAGES) & 1, abort_flag, 1)) break;
                mbar_expect_tx(full_b(s), (uint32_t)MT * BK * 2);
                tma_load_2d(sbase + C::b_off + s * C::B_STAGE, &xmap, (kb_begin + i) * BK, m0, full_b(s));
                if (WIDE && MT > 256)                              // rows 256.. of the tile: the second MMA's operand
                    tma_load_2d(sbase + C::b_off + s * C::B_STAGE + B_HALF, &xmap, (kb_begin + i) * BK, m0 + 256, full_b(s));
                issued = i + 1;
            }
            // never leave a bulk copy in flight behind an exiting CTA
            for (int i = max(0, issued - BST); i < issued; i++)
                mbar_wait(full_b(i % BST), (i / BST) & 1, abort_flag, 2);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const int n_lo = MT < 256 ? MT : 256, n_hi = MT - n_lo;       // activation rows of the first / second MMA
            const uint32_t ibase = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 4) << 24);
            const uint32_t idesc = ibase | ((uint32_t)(n_lo >> 3) << 17), idesc_hi = ibase | ((uint32_t)(n_hi >> 3) << 17);
            bool ok = true;
            for (int i = 0; i < nkb && ok; i++) {
                const int s = i % STAGES, sb = i % BST;
                ok = mbar_wait(full_a(s), (i / STAGES) & 1, abort_flag, 3) && mbar_wait(full_b(sb), (i / BST) & 1, abort_flag, 4);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t adesc = make_desc_sw128(sbase + C::a_off + s * A_BYTES);
                const uint64_t bdesc = make_desc_sw128(sbase + C::b_off + sb * C::B_STAGE);
                const uint64_t bdesc_hi = make_desc_sw128(sbase + C::b_off + sb * C::B_STAGE + B_HALF);
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++) {  // advance 32 bytes inside the swizzle row per K=16 step
                    umma_f16(tmem_base, adesc + (uint64_t)(2 * kk), bdesc + (uint64_t)(2 * kk), idesc, (i | kk) ? 1u : 0u);
                    if (WIDE && n_hi > 0)
                        umma_f16(tmem_base + 256u, adesc + (uint64_t)(2 * kk), bdesc_hi + (uint64_t)(2 * kk), idesc_hi, (i | kk) ? 1u : 0u);
                }
                umma_commit(empty(s));
            }
            umma_commit(accum_bar);   // arrives once every MMA issued so far has retired
        }
    } else if (warp == 2 + DQ_WARPS) {
        // ---------------- TMA producer: packed weights and their scales ----------------
        if (lane == 0) {
            int issued = 0, sc_issued = 0;
            const int c_first = kb_begin / SC_SLABS;
            for (int i = 0; i < nkb; i++) {
                // Slot of slab i - RS free: its group has read that slab's bytes AND its scales. Waits
                // happen in slab order, so by now every slab up to i - RS is done with the scale box
                // that the box loaded below replaces (it ended at least RS + 1 slabs ago).
                const int rs = i % RS;
                if (!mbar_wait(raw_empty(rs), ((i / RS) & 1) ^ 1, abort_flag, 8)) break;
                if (SCTMA && (i == 0 || (kb_begin + i) % SC_SLABS == 0)) {
                    const int cs = sc_issued & 1;
                    mbar_expect_tx(sc_full(cs), SC_BYTES);
                    tma_load_2d(sbase + C::sc_off + cs * SC_BYTES, &smap, (c_first + sc_issued) * (SC_SLABS * 4), n0, sc_full(cs));
                    sc_issued++;
                }
                mbar_expect_tx(raw_full(rs), C::RAW_STAGE);
                tma_load_2d(sbase + C::raw_off + rs * C::RAW_STAGE, &wmap, (kb_begin + i) * RAWB, n0, raw_full(rs));
                issued = i + 1;
            }
            for (int i = max(0, issued - RS); i < issued; i++) mbar_wait(raw_full(i % RS), (i / RS) & 1, abort_flag, 9);
            for (int c = max(0, sc_issued - 2); c < sc_issued; c++) mbar_wait(sc_full(c & 1), (c >> 1) & 1, abort_flag, 10);
        }
    } else {
        // ---------------- weight expansion (operand A), then epilogue ----------------
        // group = which slabs (i % 4), tg = thread within the group; a thread expands two (row, half)
        // items of its group's slab: rows tg/2 and 64 + tg/2, half tg & 1
        const int dqw = warp - 2, grp = dqw % DQ_GROUPS, tg = (dqw / DQ_GROUPS) * 32 + lane;
        const int h = tg & 1;
        const int row_blocks = K / 32;
        const uint32_t* lut = reinterpret_cast<const uint32_t*>(smem + C::lut_off);
        const int c_first = kb_begin / SC_SLABS;
        int chunk_seen = -1;

        bool ok = true;
        for (int i = grp; i < nkb; i += DQ_GROUPS) {
            const int kb = kb_begin + i;
            const size_t kblk = (size_t)kb * 2 + h;               // 32-element block index in the row
            const bool in_row = kblk < (size_t)row_blocks;
            // scales that do not come by tensor load are fetched before the waits, which hide part of the latency
            float scale[2] = {0.f, 0.f};
            if (!SCTMA && in_row) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int n = min(n0 + 64 * e + (tg >> 1), N - 1);
                    if (TYPE == CMLB200_NF4) scale[e] = reinterpret_cast<const float*>(scales)[((size_t)n * K + kblk * 32) / (size_t)nf4_block];
                    else scale[e] = cml_half_to_float(reinterpret_cast<const uint16_t*>(scales)[(size_t)n * row_blocks + kblk]);
                }
            }
            const int rs = i % RS;
            ok = warp_wait(raw_full(rs), (i / RS) & 1, abort_flag, 11, ok);
            const int cl = kb / SC_SLABS - c_first, cs = cl & 1;
            if (SCTMA && cl != chunk_seen) { ok = warp_wait(sc_full(cs), (cl >> 1) & 1, abort_flag, 12, ok); chunk_seen = cl; }
            if (!ok) break;
            uint4 raw[2][2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const uint8_t* src = smem + C::raw_off + rs * C::RAW_STAGE + (64 * e + (tg >> 1)) * RAWB + h * (RAWB / 2);
                raw[e][0] = *reinterpret_cast<const uint4*>(src);
                if (RAWB == 64) raw[e][1] = *reinterpret_cast<const uint4*>(src + 16);
                if (SCTMA) {
                    const uint32_t sw = *reinterpret_cast<const uint32_t*>(smem + C::sc_off + cs * SC_BYTES + (64 * e + (tg >> 1)) * (SC_SLABS * 4) + (kb % SC_SLABS) * 4);
                    if (TYPE == CMLB200_NF4) scale[e] = __uint_as_float(sw);
                    else scale[e] = cml_half_to_float((uint16_t)(h ? (sw >> 16) : (sw & 0xFFFF)));
                }
            }
            uint4 out[2][4];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                if (in_row) expand32<TYPE>(raw[e], scale[e], lut, lane, out[e]);
                else {                                            // past the end of the row: zeros meet the zero-filled activations
#pragma unroll
                    for (int c = 0; c < 4; c++) out[e][c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            // The slot is handed back only now, after the arithmetic above has consumed every loaded
            // register. Signalling right behind the load instructions is not enough: the arrival can
            // overtake loads that are still queued in a busy shared-memory pipe, the producer then
            // refills the slot, and those loads return the bytes of a later slab (seen as whole 16-row
            // bands carrying the weights of slab i + ring depth, more often with the NF4 table traffic).
            __syncwarp();
            if (lane == 0) mbar_arrive(raw_empty(rs));
            const int s = i % STAGES;
            ok = warp_wait(empty(s), ((i / STAGES) & 1) ^ 1, abort_flag, 5, ok);
            if (!ok) break;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int r = 64 * e + (tg >> 1);
                uint8_t* arow = smem + C::a_off + s * A_BYTES + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
                for (int c = 0; c < 4; c++)
                    *reinterpret_cast<uint4*>(arow + (((4 * h + c) ^ (r & 7)) << 4)) = out[e][c];
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(full_a(s));
        }

        // ---- epilogue: D[n][m] (lane = weight row, column = activation row) -> Y[m][n]
        ok = warp_wait(accum_bar, 0, abort_flag, 6, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int q = warp & 3;                 // the TMEM lane quadrant this warp may read
            const int part = (warp - 2) >> 2;       // four warps share a quadrant and split the columns
            const int nrow = n0 + q * 32 + lane;
            for (int c0 = part * 32; c0 < MT; c0 += 32 * GROUP_WARPS) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (nrow < N) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int m = m0 + c0 + j;
                        if (m < M && c0 + j < MT) {
                            if (partial) partial[((size_t)blockIdx.z * M + m) * N + nrow] = __uint_as_float(v[j]);
                            else epilogue_store(out, gate, mode, (size_t)m * N + nrow, __uint_as_float(v[j]));
                        }
                    }
                }
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

__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out, const __nv_bfloat16* __restrict__ gate,
                                     int mode, size_t mn, int splits) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += stride) {
        float s = 0.f;
        for (int z = 0; z < splits; z++) s += partial[(size_t)z * mn + i];
        epilogue_store(out, gate, mode, i, s);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encoder(EncodeTiledFn* out) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        CMLB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        CMLB_REQUIRE(p && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available in this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    *out = fn;
    return CMLB200_OK;
}

// Scratch for split-K partial sums, grown on demand, one per device in use.
struct Workspace { float* ptr; size_t bytes; };
Workspace g_ws[16] = {};

// K splits for a grid of gx x gy tiles: few tiles are split so that every SM gets a CTA, with at
// least 8 slabs per CTA.
inline int auto_splits(int gx, int gy, int total_kb, int sms) {
    int splits = 1;
    while (gx * gy * splits * 2 <= sms && total_kb / (splits * 2) >= 8) splits *= 2;
    return splits;
}

// Estimated time (us) of one launch with tiles of mt activation rows: per 64-wide K slab a 256-row
// tile takes SLAB_N us (bound by the weight expansion), a 512-row tile SLAB_W (bound by the 64 KB of
// activations it pulls from L2), plus 8 us per wave of CTAs for pipeline fill and epilogue, plus
// the split-K partial sums going out and back in at about 5 TB/s.
constexpr double SLAB_N = 0.6, SLAB_W = 0.95;     // fitted to 4096x4096, 11008x4096, 4096x11008 at M = 512 .. 4096
inline double tile_cost_us(int M, int N, int K, int mt, int sms) {
    const int gx = (N + BN - 1) / BN, gy = (M + mt - 1) / mt, total_kb = (K + BK - 1) / BK;
    const int splits = auto_splits(gx, gy, total_kb, sms);
    const int waves = (gx * gy * splits + sms - 1) / sms;
    return waves * ((double)((total_kb + splits - 1) / splits) * (mt > 256 ? SLAB_W : SLAB_N) + 8.0) +
           (splits > 1 ? (double)splits * M * N * 8.0 / 5e6 : 0.0);
}

template <int TYPE>
int launch_gemm(const cmlb200_qmat* W, const uint16_t* x, void* y, const uint16_t* gate, int mode, int M, float* ws, int splits_forced,
                cudaStream_t st) {
    const int N = W->rows, K = W->cols;
    // more than 256 activation rows: 512-row tiles (the weight slab is expanded once for both halves)
    const bool wide = M > 256 && splits_forced <= 0 && Cfg<TYPE, true>::total + 1024 <= 227 * 1024 &&
                      tile_cost_us(M, N, K, 512, cmlb_num_sms()) < tile_cost_us(M, N, K, 256, cmlb_num_sms());    // (Q8_0's 8 KB packed slabs leave no room for it)
    const int MT = wide ? 512 : (M >= 256 ? 256 : ((M + 15) / 16) * 16);
    EncodeTiledFn enc;
    int rc = get_encoder(&enc);
    if (rc) return rc;
    CUtensorMap xmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)(MT > 256 ? 256 : MT)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)x, dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CMLB_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d (x must be 16-byte aligned, K*2 a multiple of 16)", (int)cr);
    // the packed weights as bytes [N][row_bytes], a box of 128 rows by one slab's bytes
    using C = Cfg<TYPE, false>;
    CUtensorMap wmap, smap;
    const cuuint64_t row_bytes = (cuuint64_t)K * C::RAWB / BK;
    const cuuint64_t wdims[2] = {row_bytes, (cuuint64_t)N};
    const cuuint64_t wstr[1] = {row_bytes};
    const cuuint32_t wbox[2] = {(cuuint32_t)C::RAWB, (cuuint32_t)BN};
    cr = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, W->qs, wdims, wstr, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CMLB_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled (weights) failed with %d", (int)cr);
    // scales as bytes [N][4 per slab] when every row and slab has exactly four of them on a 16-byte row pitch:
    // the two fp16 of Q4_0 / Q8_0, or the fp32 of NF4 with block 64; K % 256 == 0
    const bool sctma = K % 256 == 0 && ((uintptr_t)W->scales & 15) == 0 && (TYPE != CMLB200_NF4 || W->block == 64);
    smap = wmap;
    if (sctma) {
        const cuuint64_t sdims[2] = {(cuuint64_t)K / 16, (cuuint64_t)N};
        const cuuint64_t sstr[1] = {(cuuint64_t)K / 16};
        const cuuint32_t sbox[2] = {(cuuint32_t)(SC_SLABS * 4), (cuuint32_t)BN};
        cr = enc(&smap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, W->scales, sdims, sstr, sbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        CMLB_REQUIRE(cr == CUDA_SUCCESS, "cuTensorMapEncodeTiled (scales) failed with %d", (int)cr);
    }

    const int gx = (N + BN - 1) / BN, gy = (M + MT - 1) / MT;
    const int total_kb = (K + BK - 1) / BK;
    int splits = 1;
    if (splits_forced > 0) splits = splits_forced;
    else {
        splits = auto_splits(gx, gy, total_kb, cmlb_num_sms());
    }
    if (splits > total_kb) splits = total_kb;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    splits = (total_kb + kb_per_split - 1) / kb_per_split;
    float* partial = nullptr;
    if (splits > 1) {
        const size_t need = (size_t)splits * M * N * sizeof(float);
        if (ws) partial = ws;
        else {
            int dev = 0;
            CMLB_CUDA(cudaGetDevice(&dev));
            CMLB_REQUIRE(dev < 16, "device index %d out of range", dev);
            if (g_ws[dev].bytes < need) {
                if (g_ws[dev].ptr) CMLB_CUDA(cudaFree(g_ws[dev].ptr));
                g_ws[dev].ptr = nullptr;
                g_ws[dev].bytes = 0;
                CMLB_CUDA(cudaMalloc((void**)&g_ws[dev].ptr, need));
                g_ws[dev].bytes = need;
            }
            partial = g_ws[dev].ptr;
        }
    }
    static_assert(Cfg<TYPE, false>::total + 1024 <= 227 * 1024, "the stages do not fit shared memory");
    static size_t attr[4][kMaxDevices] = {};
#define GEMM_LAUNCH(SC, WD, slot)                                                                                                     \
    do {                                                                                                                             \
        auto kern = gemm_kernel<TYPE, SC, WD>;                                                                                       \
        const int smem = Cfg<TYPE, WD>::total + 1024;                                                                                \
        CMLB_CUDA(cmlb_ensure_smem(kern, (size_t)smem, attr[slot]));                                                                 \
        kern<<<dim3(gx, gy, splits), THREADS, smem, st>>>(xmap, wmap, smap, W->scales, y, (const __nv_bfloat16*)gate, mode, partial, M, N, \
                                                          K, MT, W->block, kb_per_split);                                           \
    } while (0)
    constexpr bool kWideFits = Cfg<TYPE, true>::total + 1024 <= 227 * 1024;
    if (sctma && wide) GEMM_LAUNCH(true, kWideFits, 0);
    else if (sctma) GEMM_LAUNCH(true, false, 1);
    else if (wide) GEMM_LAUNCH(false, kWideFits, 2);
    else GEMM_LAUNCH(false, false, 3);
#undef GEMM_LAUNCH
    CMLB_LAUNCH_CHECK();
    if (splits > 1) {
        const size_t mn = (size_t)M * N;
        int grid = (int)((mn + 255) / 256);
        if (grid > cmlb_num_sms() * 8) grid = cmlb_num_sms() * 8;
        splitk_reduce_kernel<<<grid, 256, 0, st>>>(partial, y, (const __nv_bfloat16*)gate, mode, mn, splits);
        CMLB_LAUNCH_CHECK();
    }
    return CMLB200_OK;
}

int gemm_entry(const cmlb200_qmat* W, const uint16_t* x, void* y, const uint16_t* gate, int mode, int M, float* ws, int splits, void* stream) {
    CMLB_REQUIRE(W && W->qs && W->scales && x && y, "cmlb200_gemm_bf16: NULL argument");
    CMLB_REQUIRE(mode >= GEMM_OUT_BF16 && mode <= GEMM_SWIGLU_BF16 && (mode != GEMM_SWIGLU_BF16 || gate), "cmlb200_gemm_bf16_ex: bad output mode %d", mode);
    CMLB_REQUIRE(M >= 1, "cmlb200_gemm_bf16: M=%d must be positive", M);
    CMLB_REQUIRE(W->rows > 0 && W->cols > 0 && W->cols % 32 == 0, "cmlb200_gemm_bf16: cols=%d must be a positive multiple of 32", W->cols);
    CMLB_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)W->qs & 15) == 0 && ((uintptr_t)W->scales & 3) == 0,
                 "cmlb200_gemm_bf16: x and the weight planes must be 16-byte aligned");
    cudaStream_t st = as_stream(stream);
    switch (W->type) {
        case CMLB200_Q8_0: return launch_gemm<CMLB200_Q8_0>(W, x, y, gate, mode, M, ws, splits, st);
        case CMLB200_Q4_0: return launch_gemm<CMLB200_Q4_0>(W, x, y, gate, mode, M, ws, splits, st);
        case CMLB200_NF4:
            CMLB_REQUIRE(W->block >= 32 && W->block % 32 == 0 && W->cols % W->block == 0,
                         "cmlb200_gemm_bf16: NF4 block size %d must be a multiple of 32 that divides cols", W->block);
            return launch_gemm<CMLB200_NF4>(W, x, y, gate, mode, M, ws, splits, st);
        default: CMLB_REQUIRE(false, "cmlb200_gemm_bf16: unsupported weight type %d", W->type);
    }
    return CMLB200_EINVAL;
}

}  // namespace

extern "C" int cmlb200_gemm_bf16(const cmlb200_qmat* W, const uint16_t* d_x_bf16, uint16_t* d_y_bf16, int M, void* stream) {
    return gemm_entry(W, d_x_bf16, d_y_bf16, nullptr, GEMM_OUT_BF16, M, nullptr, 0, stream);
}

extern "C" int cmlb200_gemm_bf16_ex(const cmlb200_qmat* W, const uint16_t* d_x_bf16, int M, int mode, void* d_out, const uint16_t* d_gate_bf16,
                                    void* stream) {
    return gemm_entry(W, d_x_bf16, d_out, d_gate_bf16, mode, M, nullptr, 0, stream);
}

extern "C" int cmlb200_gemm_bf16_splitk(const cmlb200_qmat* W, const uint16_t* d_x_bf16, uint16_t* d_y_bf16, int M,
                                        int splits, void* stream) {
    CMLB_REQUIRE(splits >= 1, "cmlb200_gemm_bf16_splitk: splits must be >= 1");
    return gemm_entry(W, d_x_bf16, d_y_bf16, nullptr, GEMM_OUT_BF16, M, nullptr, splits, stream);
}

extern "C" int cmlb200_gemm_status(int* status, int reset) {
    CMLB_REQUIRE(status, "cmlb200_gemm_status: NULL argument");
    CMLB_CUDA(cudaDeviceSynchronize());
    CMLB_CUDA(cudaMemcpyFromSymbol(status, g_gemm_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        CMLB_CUDA(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
    }
    return CMLB200_OK;
}
