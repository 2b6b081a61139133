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
    const float4* src = reinterpret_cast<const float4*>(partial);

    // 1. push
    for (int q = 0; q < tp; q++) {
        if (q == rank) continue;
        float4* dst = reinterpret_cast<float4*>(tpws_inbox(peers.ws[q], 0, parity, rank, max_floats));
        for (int i = lo + (int)threadIdx.x; i < hi; i += blockDim.x) dst[i] = src[i];
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
    float4* out = reinterpret_cast<float4*>(h);
    for (int i = lo + (int)threadIdx.x; i < hi; i += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < tp; q++) {
            const float4 v = (q == rank) ? src[i] : reinterpret_cast<const float4*>(tpws_inbox(mine, 0, parity, q, max_floats))[i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float4 o = out[i];
        o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
        out[i] = o;
    }
}

}  // namespace

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
