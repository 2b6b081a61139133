// Tensor-parallel "residual += sum over ranks of partial" for decode-sized rows, over peer
// memory: h += all_reduce_sum(partial). Replaces C-ML's cml_tp_all_reduce_sum after the
// row-parallel projections (src/distributed/tensor_parallel.c:195-260, which goes through
// ncclAllReduce on host buffers, src/distributed/nccl_backend.c:219-240) for the 16-64 KB messages
// of a decode step, where the collective's launch and protocol latency is the whole cost.
//
// One launch per rank and all-reduce, no library call:
//   1. every CTA pushes its slice of the local partial into the inbox each peer keeps for this
//      rank (plain remote stores over NVLink), fences, and stores the sequence number of this
//      all-reduce into the peer's flag word for (this rank, this CTA);
//   2. it waits until the flag words of all peers for its slice show the same sequence number
//      (bounded spin; on expiry a status word is set and the launch returns without touching h);
//   3. it adds the partials of all ranks in rank order (its own from local memory, the others
//      from its inboxes) onto h. The order is the same on every rank, so all ranks hold
//      bit-identical h afterwards.
// Sequence numbers live in device memory and count up by themselves, so the launch can sit in a
// captured CUDA graph. Inboxes alternate between two buffers: a peer can only start all-reduce
// s+2 after this rank has started s+1, i.e. after it finished reading the inbox of s.
//
// The workspace layout (one per rank, mapped into every other rank through CUDA IPC) is in
// common.cuh; this file uses channel 0.
#include <stdlib.h>
#include <string.h>
#include "common.cuh"

namespace {

constexpr int CTAS = kTpCtas;
constexpr int MAX_TP = kTpMaxRanks;

__global__ void __launch_bounds__(256)
tp_allreduce_add_kernel(float* __restrict__ h, const float* __restrict__ partial, int n4, TpPeers peers) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tp = peers.tp, rank = peers.rank;
    const size_t max_floats = peers.max_floats;
    uint8_t* mine = peers.ws[rank];
    const int c = blockIdx.x;
    const uint32_t seq = tpws_seq(mine, 0)[c] + 1;            // this all-reduce; every CTA keeps its own count
    const int parity = (int)(seq & 1u);
    // slice of this CTA, in float4
    const int per = (n4 + CTAS - 1) / CTAS;
    const int lo = min(n4, c * per), hi = min(n4, lo + per);
    const float4* __restrict__ src = reinterpret_cast<const float4*>(partial);
    constexpr int U = 4;                     // independent 16-byte pieces in flight per thread
    const int bs = blockDim.x;

    // 1. push
    for (int q = 0; q < tp; q++) {
        if (q == rank) continue;
        float4* __restrict__ dst = reinterpret_cast<float4*>(tpws_inbox(peers.ws[q], 0, parity, rank, max_floats));
        for (int i = lo + (int)threadIdx.x; i < hi; i += bs * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; u++) if (i + u * bs < hi) v[u] = src[i + u * bs];
#pragma unroll
            for (int u = 0; u < U; u++) if (i + u * bs < hi) dst[i + u * bs] = v[u];
        }
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < tp && (int)threadIdx.x != rank) st_release_sys(tpws_flags(peers.ws[threadIdx.x], 0, rank) + c, seq);

    // 2. wait for every peer's slice
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < tp && (int)threadIdx.x != rank) {
        const uint32_t* f = tpws_flags(mine, 0, threadIdx.x) + c;
        int i = 0;
        while ((int32_t)(ld_acquire_sys(f) - seq) < 0 && ++i < peers.spin_limit) {}
        if (i >= peers.spin_limit) { ok = 0; atomicExch(tpws_status(mine), 1u + threadIdx.x); }
    }
    __syncthreads();
    if (threadIdx.x == 0) tpws_seq(mine, 0)[c] = seq;
    if (!ok) return;

    // 3. sum in rank order onto h
    float4* __restrict__ out = reinterpret_cast<float4*>(h);
    for (int i = lo + (int)threadIdx.x; i < hi; i += bs * U) {
        float4 acc[U], o[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i + u * bs < hi) o[u] = out[i + u * bs];
        }
        for (int q = 0; q < tp; q++) {
            const float4* __restrict__ in = (q == rank) ? src : reinterpret_cast<const float4*>(tpws_inbox(mine, 0, parity, q, max_floats));
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; u++) if (i + u * bs < hi) v[u] = in[i + u * bs];
#pragma unroll
            for (int u = 0; u < U; u++)
                if (i + u * bs < hi) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
        }
#pragma unroll
        for (int u = 0; u < U; u++)
            if (i + u * bs < hi) {
                o[u].x += acc[u].x; o[u].y += acc[u].y; o[u].z += acc[u].z; o[u].w += acc[u].w;
                out[i + u * bs] = o[u];
            }
    }
}


// ---- prompt-sized messages -------------------------------------------------------------------
// The kernel above sends every rank's whole partial to every peer, which is right for the 16-512 KB
// of a decode step. A prompt's row-parallel projection leaves 16-64 MB per rank; for that size the
// sum is split by rank ("reduce-scatter, then all-gather", all inside one launch per rank):
//   1. every CTA pushes, for each peer q, its share of slice q of the local partial into the inbox A
//      that q keeps for this rank, fences, and raises flag A;
//   2. it waits for flag A of all peers, sums its share of this rank's own slice in rank order
//      (the local partial and the inboxes), adds the sum onto h and pushes it into the inbox B of
//      every peer, fences, and raises flag B;
//   3. it waits for flag B of all peers and adds their summed slices onto h.
// Each slice is summed by one rank, in rank order, so all ranks end with bit-identical h. A rank
// sends 2 (tp - 1) / tp of the message over NVLink instead of tp - 1 times the message.
// Element i of a slice belongs to CTA (i / 256) % gridDim.x on every rank (all ranks launch the same
// number of CTAs), so CTA c only ever depends on CTA c of its peers; the inboxes alternate with the
// parity of the sequence number as above. Every loop first loads several independent 16-byte
// pieces and then stores them: the copies are bound by how many loads are in flight, not by
// arithmetic. The workspace is a second allocation with its own header:
//   +64 u32 status   +1024 u32 seq[128]   +4096 u32 flagA[8][128]   +8192 u32 flagB[8][128]
//   +16384 float4 inbox[A|B][parity][from < tp][region4]
// With EMU the ranks are blockIdx.y of ONE cooperative launch over buffers of one GPU: the way to
// exercise the protocol where only one device is at hand (launches that wait on one another must
// not be separate launches on the same GPU).
constexpr int kBulkCtas = 128;           // flag words per rank and flag kind; a launch uses at most this many CTAs
constexpr int kBulkThreads = 256;
constexpr int kBulkUnroll = 4;
struct BulkArgs {
    uint8_t* ws[MAX_TP];
    float* h[MAX_TP];               // [0] only, unless emulating
    const float* partial[MAX_TP];
    size_t region4;                 // float4 per (inbox, parity, from) region
    int n4, tp, rank, spin_limit;
};
__device__ __forceinline__ uint32_t* bulk_seq(uint8_t* ws) { return reinterpret_cast<uint32_t*>(ws + 1024); }
__device__ __forceinline__ uint32_t* bulk_flag(uint8_t* ws, int which, int from) {
    return reinterpret_cast<uint32_t*>(ws + 4096 + 4096 * which) + from * kBulkCtas;
}
__device__ __forceinline__ float4* bulk_inbox(uint8_t* ws, int which, int parity, int from, int tp, size_t region4) {
    return reinterpret_cast<float4*>(ws + kTpHeaderBytes) + (((size_t)which * 2 + parity) * tp + from) * region4;
}
__device__ __forceinline__ void add4(float4& a, const float4 b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }

// All peers' flag words for CTA c reach seq, or the launch records which peer it gave up on.
__device__ __forceinline__ bool bulk_wait(uint8_t* mine, int which, int tp, int rank, int c, uint32_t seq, int spin_limit, int* ok) {
    if ((int)threadIdx.x < tp && (int)threadIdx.x != rank) {
        const uint32_t* f = bulk_flag(mine, which, threadIdx.x) + c;
        int i = 0;
        while ((int32_t)(ld_acquire_sys(f) - seq) < 0 && ++i < spin_limit) {}
        if (i >= spin_limit) { *ok = 0; atomicExch(tpws_status(mine), 1u + threadIdx.x); }
    }
    __syncthreads();
    return *ok != 0;
}

template <bool EMU>
__global__ void __launch_bounds__(kBulkThreads)
tp_allreduce_bulk_kernel(BulkArgs a) {
    if (!EMU) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int tp = a.tp, rank = EMU ? (int)blockIdx.y : a.rank;
    uint8_t* mine = a.ws[rank];
    const int c = blockIdx.x, t = threadIdx.x;
    const uint32_t seq = bulk_seq(mine)[c] + 1;
    const int parity = (int)(seq & 1u);
    const int per = (a.n4 + tp - 1) / tp;                      // float4 per slice
    const float4* __restrict__ src = reinterpret_cast<const float4*>(a.partial[EMU ? rank : 0]);
    float4* __restrict__ h4 = reinterpret_cast<float4*>(a.h[EMU ? rank : 0]);
    const int step = (int)gridDim.x * kBulkThreads;
    constexpr int U = kBulkUnroll;
    __shared__ int ok;
    if (t == 0) ok = 1;

    // 1. slice q of the local partial -> rank q
    for (int d = 1; d < tp; d++) {
        const int q = (rank + d) % tp;
        const int lo = min(a.n4, q * per), len = min(a.n4, lo + per) - lo;
        float4* __restrict__ dst = bulk_inbox(a.ws[q], 0, parity, rank, tp, a.region4);
        for (int i = c * kBulkThreads + t; i < len; i += step * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; u++) if (i + u * step < len) v[u] = src[lo + i + u * step];
#pragma unroll
            for (int u = 0; u < U; u++) if (i + u * step < len) dst[i + u * step] = v[u];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (t < tp && t != rank) st_release_sys(bulk_flag(a.ws[t], 0, rank) + c, seq);

    // 2. this rank's slice: sum in rank order, add onto h, hand the sum to every peer
    const bool got_a = bulk_wait(mine, 0, tp, rank, c, seq, a.spin_limit, &ok);
    if (got_a) {
        const int lo = min(a.n4, rank * per), len = min(a.n4, lo + per) - lo;
        for (int i = c * kBulkThreads + t; i < len; i += step * U) {
            float4 acc[U], o[U];
#pragma unroll
            for (int u = 0; u < U; u++) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int q = 0; q < tp; q++) {
                const float4* __restrict__ in = q == rank ? src + lo : bulk_inbox(mine, 0, parity, q, tp, a.region4);
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; u++) if (i + u * step < len) v[u] = __ldcg(in + i + u * step);
#pragma unroll
                for (int u = 0; u < U; u++) if (i + u * step < len) add4(acc[u], v[u]);
            }
#pragma unroll
            for (int u = 0; u < U; u++) if (i + u * step < len) o[u] = h4[lo + i + u * step];
            for (int d = 1; d < tp; d++) {
                float4* __restrict__ dst = bulk_inbox(a.ws[(rank + d) % tp], 1, parity, rank, tp, a.region4);
#pragma unroll
                for (int u = 0; u < U; u++) if (i + u * step < len) dst[i + u * step] = acc[u];
            }
#pragma unroll
            for (int u = 0; u < U; u++) if (i + u * step < len) { add4(o[u], acc[u]); h4[lo + i + u * step] = o[u]; }
        }
    }
    __threadfence_system();
    __syncthreads();
    // after an expired wait no flag B goes out: the peers' own waits expire and set their status words
    if (got_a && t < tp && t != rank) st_release_sys(bulk_flag(a.ws[t], 1, rank) + c, seq);

    // 3. the other ranks' summed slices
    const bool got_b = got_a && bulk_wait(mine, 1, tp, rank, c, seq, a.spin_limit, &ok);
    if (got_b) {
        for (int d = 1; d < tp; d++) {
            const int q = (rank + d) % tp;
            const int lo = min(a.n4, q * per), len = min(a.n4, lo + per) - lo;
            const float4* __restrict__ in = bulk_inbox(mine, 1, parity, q, tp, a.region4);
            for (int i = c * kBulkThreads + t; i < len; i += step * U) {
                float4 v[U], o[U];
#pragma unroll
                for (int u = 0; u < U; u++) if (i + u * step < len) { v[u] = __ldcg(in + i + u * step); o[u] = h4[lo + i + u * step]; }
#pragma unroll
                for (int u = 0; u < U; u++) if (i + u * step < len) { add4(o[u], v[u]); h4[lo + i + u * step] = o[u]; }
            }
        }
    }
    if (t == 0) bulk_seq(mine)[c] = seq;
}

int bulk_args(BulkArgs* a, size_t n, int tp, void* const* ws, size_t max_floats, const char* who) {
    CMLB_REQUIRE(ws, "%s: NULL argument", who);
    CMLB_REQUIRE(tp >= 2 && tp <= MAX_TP, "%s: tp=%d (must be 2..8)", who, tp);
    CMLB_REQUIRE(max_floats > 0 && max_floats % 4 == 0, "%s: max_floats=%zu must be a positive multiple of 4", who, max_floats);
    CMLB_REQUIRE(n > 0 && n % 4 == 0 && n <= max_floats && n / 4 <= 0x7fffffff, "%s: n=%zu must be a multiple of 4 and at most %zu", who, n, max_floats);
    for (int r = 0; r < tp; r++) {
        CMLB_REQUIRE(ws[r], "%s: workspace of rank %d missing", who, r);
        a->ws[r] = static_cast<uint8_t*>(ws[r]);
    }
    a->region4 = (max_floats / 4 + tp - 1) / tp;
    a->n4 = (int)(n / 4);
    a->tp = tp;
    a->spin_limit = cmlb_tp_spin_limit();
    return CMLB200_OK;
}

}  // namespace

// Workspace of the prompt-sized all-reduce for messages of up to max_floats values over tp ranks.
extern "C" size_t cmlb200_tp_ar_bulk_workspace_bytes(size_t max_floats, int tp) {
    if (tp < 2 || tp > MAX_TP) return 0;
    const size_t region4 = (max_floats / 4 + tp - 1) / tp;
    return kTpHeaderBytes + 2 * 2 * (size_t)tp * region4 * sizeof(float4);
}

// h[0..n) += sum over ranks of partial[0..n), for n of prompt size. ws[r] = rank r's bulk workspace
// as mapped in this process (zero-filled once before the first call on any rank; tp and max_floats
// fixed for the life of the workspace). Every rank must make the same sequence of calls.
extern "C" int cmlb200_tp_allreduce_bulk_add(float* d_h, const float* d_partial, size_t n, int tp, int rank, void* const* ws,
                                             size_t max_floats, void* stream) {
    CMLB_REQUIRE(d_h && d_partial, "cmlb200_tp_allreduce_bulk_add: NULL argument");
    CMLB_REQUIRE(rank >= 0 && rank < tp, "cmlb200_tp_allreduce_bulk_add: rank %d outside 0..%d", rank, tp - 1);
    CMLB_REQUIRE(((uintptr_t)d_h & 15) == 0 && ((uintptr_t)d_partial & 15) == 0, "cmlb200_tp_allreduce_bulk_add: buffers must be 16-byte aligned");
    BulkArgs a = {};
    if (int rc = bulk_args(&a, n, tp, ws, max_floats, "cmlb200_tp_allreduce_bulk_add")) return rc;
    a.rank = rank;
    a.h[0] = d_h;
    a.partial[0] = d_partial;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cmlb_num_sms() < kBulkCtas ? cmlb_num_sms() : kBulkCtas);      // the same on every rank of one box
    cfg.blockDim = dim3(kBulkThreads);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CMLB_CUDA(cudaLaunchKernelEx(&cfg, tp_allreduce_bulk_kernel<false>, a));
    return CMLB200_OK;
}

// The same exchange with all tp ranks on ONE device, as one cooperative launch (every CTA of every
// rank resident at once): d_h[r], d_partial[r], ws[r] are rank r's buffers on the current device.
// For checking the protocol on a single GPU; a real job runs one process per GPU and the call above.
extern "C" int cmlb200_tp_allreduce_bulk_emulate(float* const* d_h, const float* const* d_partial, size_t n, int tp, void* const* ws,
                                                 size_t max_floats, void* stream) {
    CMLB_REQUIRE(d_h && d_partial, "cmlb200_tp_allreduce_bulk_emulate: NULL argument");
    BulkArgs a = {};
    if (int rc = bulk_args(&a, n, tp, ws, max_floats, "cmlb200_tp_allreduce_bulk_emulate")) return rc;
    for (int r = 0; r < tp; r++) {
        CMLB_REQUIRE(d_h[r] && d_partial[r] && ((uintptr_t)d_h[r] & 15) == 0 && ((uintptr_t)d_partial[r] & 15) == 0,
                     "cmlb200_tp_allreduce_bulk_emulate: buffers of rank %d missing or not 16-byte aligned", r);
        a.h[r] = d_h[r];
        a.partial[r] = d_partial[r];
    }
    int per_sm = 0;
    CMLB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tp_allreduce_bulk_kernel<true>, kBulkThreads, 0));
    int ctas = per_sm * cmlb_num_sms() / tp;             // per rank, as many as stay resident together
    if (ctas > kBulkCtas) ctas = kBulkCtas;
    CMLB_REQUIRE(ctas >= 1, "cmlb200_tp_allreduce_bulk_emulate: %d ranks do not fit on the device at once", tp);
    void* args[] = {&a};
    CMLB_CUDA(cudaLaunchCooperativeKernel((const void*)tp_allreduce_bulk_kernel<true>, dim3(ctas, tp), dim3(kBulkThreads), args, 0, as_stream(stream)));
    return CMLB200_OK;
}

extern "C" size_t cmlb200_tp_ar_workspace_bytes(size_t max_floats) {
    return kTpHeaderBytes + 2 * 2 * (size_t)MAX_TP * max_floats * sizeof(float);
}

// h[0..n) += sum over ranks of partial[0..n). ws[r] = rank r's workspace as mapped in this process
// (ws[rank] is this rank's own, zero-filled once before the first call on any rank). n % 4 == 0,
// n <= max_floats, tp <= 8. Every rank must make the same sequence of calls.
extern "C" int cmlb200_tp_allreduce_add(float* d_h, const float* d_partial, size_t n, int tp, int rank, void* const* ws, size_t max_floats,
                                        void* stream) {
    CMLB_REQUIRE(d_h && d_partial && ws, "cmlb200_tp_allreduce_add: NULL argument");
    CMLB_REQUIRE(tp >= 2 && tp <= MAX_TP && rank >= 0 && rank < tp, "cmlb200_tp_allreduce_add: tp=%d rank=%d (tp must be 2..8)", tp, rank);
    CMLB_REQUIRE(n > 0 && n % 4 == 0 && n <= max_floats, "cmlb200_tp_allreduce_add: n=%zu must be a multiple of 4 and at most %zu", n, max_floats);
    CMLB_REQUIRE(((uintptr_t)d_h & 15) == 0 && ((uintptr_t)d_partial & 15) == 0, "cmlb200_tp_allreduce_add: buffers must be 16-byte aligned");
    TpPeers p = {};
    for (int r = 0; r < tp; r++) {
        CMLB_REQUIRE(ws[r], "cmlb200_tp_allreduce_add: workspace of rank %d missing", r);
        p.ws[r] = static_cast<uint8_t*>(ws[r]);
    }
    p.tp = tp; p.rank = rank; p.max_floats = max_floats; p.h = d_h;
    p.spin_limit = cmlb_tp_spin_limit();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CTAS);
    cfg.blockDim = dim3(256);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CMLB_CUDA(cudaLaunchKernelEx(&cfg, tp_allreduce_add_kernel, d_h, d_partial, (int)(n / 4), p));
    return CMLB200_OK;
}

// Nonzero once a wait of the kernel above (or of the decode GEMV's all-reduce epilogue) expired
// on this rank: 1 + the peer it waited for.
extern "C" int cmlb200_tp_ar_status(const void* own_ws, int* status) {
    CMLB_REQUIRE(own_ws && status, "cmlb200_tp_ar_status: NULL argument");
    uint32_t v = 0;
    CMLB_CUDA(cudaMemcpy(&v, static_cast<const uint8_t*>(own_ws) + 64, sizeof v, cudaMemcpyDeviceToHost));
    *status = (int)v;
    return CMLB200_OK;
}
extern "C" int cmlb200_tp_ar_status_reset(void* own_ws) {
    CMLB_REQUIRE(own_ws, "cmlb200_tp_ar_status_reset: NULL argument");
    CMLB_CUDA(cudaMemset(static_cast<uint8_t*>(own_ws) + 64, 0, sizeof(uint32_t)));
    return CMLB200_OK;
}

namespace { int g_wait_limit = 0; }      // 0: not set yet
int cmlb_tp_spin_limit() {
    if (g_wait_limit <= 0) {
        const char* e = getenv("CMLB200_WAIT_LIMIT");
        const long v = e ? strtol(e, nullptr, 10) : 0;
        g_wait_limit = (v > 0 && v <= kTpSpinLimit) ? (int)v : kTpSpinLimit;
    }
    return g_wait_limit;
}
extern "C" int cmlb200_set_wait_limit(int polls) {
    CMLB_REQUIRE(polls >= 0 && polls <= kTpSpinLimit, "cmlb200_set_wait_limit: %d outside 0..%d", polls, kTpSpinLimit);
    g_wait_limit = polls > 0 ? polls : kTpSpinLimit;
    return CMLB200_OK;
}

// CUDA IPC plumbing for the workspaces (64-byte handles travel between ranks by any means).
extern "C" int cmlb200_ipc_get_handle(void* d_ptr, void* handle64) {
    CMLB_REQUIRE(d_ptr && handle64, "cmlb200_ipc_get_handle: NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    CMLB_CUDA(cudaIpcGetMemHandle(&h, d_ptr));
    memcpy(handle64, &h, 64);
    return CMLB200_OK;
}
extern "C" int cmlb200_ipc_open(const void* handle64, void** d_ptr) {
    CMLB_REQUIRE(handle64 && d_ptr, "cmlb200_ipc_open: NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    CMLB_CUDA(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return CMLB200_OK;
}
extern "C" int cmlb200_ipc_close(void* d_ptr) {
    if (d_ptr) CMLB_CUDA(cudaIpcCloseMemHandle(d_ptr));
    return CMLB200_OK;
}
