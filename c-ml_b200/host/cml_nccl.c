/*
 * NCCL through dlopen, for the tensor-parallel all-reduce after the row-parallel projections
 * (C-ML loads NCCL the same way, src/distributed/nccl_backend.c:476-479, but passes host
 * pointers on the default stream, :219-240; here the buffers are device memory and the
 * collective runs on the model's own stream so that it can sit inside a captured CUDA graph).
 * Library search order: $CML_NCCL_LIB, libnccl.so.2, libnccl.so.
 */
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

typedef struct { char internal[128]; } nccl_uid;
typedef int (*fn_get_uid)(nccl_uid*);
typedef int (*fn_init_rank)(void**, int, nccl_uid, int);
typedef int (*fn_allreduce)(const void*, void*, size_t, int, int, void*, void*);
typedef int (*fn_allgather)(const void*, void*, size_t, int, void*, void*);
typedef int (*fn_destroy)(void*);
typedef const char* (*fn_errstr)(int);

static struct {
    void* lib;
    fn_get_uid get_uid;
    fn_init_rank init_rank;
    fn_allreduce allreduce;
    fn_allgather allgather;
    fn_destroy destroy;
    fn_errstr errstr;
} g_nccl;

static int load_nccl(void) {
    if (g_nccl.lib) return 0;
    const char* names[] = {getenv("CML_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (int i = 0; i < 3 && !g_nccl.lib; i++)
        if (names[i] && names[i][0]) g_nccl.lib = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!g_nccl.lib) {
        LOG_ERROR("NCCL: no libnccl found (set CML_NCCL_LIB to its path): %s", dlerror());
        return -1;
    }
    g_nccl.get_uid = (fn_get_uid)dlsym(g_nccl.lib, "ncclGetUniqueId");
    g_nccl.init_rank = (fn_init_rank)dlsym(g_nccl.lib, "ncclCommInitRank");
    g_nccl.allreduce = (fn_allreduce)dlsym(g_nccl.lib, "ncclAllReduce");
    g_nccl.allgather = (fn_allgather)dlsym(g_nccl.lib, "ncclAllGather");
    g_nccl.destroy = (fn_destroy)dlsym(g_nccl.lib, "ncclCommDestroy");
    g_nccl.errstr = (fn_errstr)dlsym(g_nccl.lib, "ncclGetErrorString");
    if (!g_nccl.get_uid || !g_nccl.init_rank || !g_nccl.allreduce || !g_nccl.destroy) {
        LOG_ERROR("NCCL: the loaded library lacks a required symbol");
        dlclose(g_nccl.lib);
        memset(&g_nccl, 0, sizeof g_nccl);
        return -1;
    }
    return 0;
}

static int check(int rc, const char* what) {
    if (rc == 0) return 0;
    LOG_ERROR("NCCL: %s failed: %s", what, g_nccl.errstr ? g_nccl.errstr(rc) : "unknown error");
    return -1;
}

int cml_nccl_unique_id(void* id128) {
    if (!id128 || load_nccl()) return -1;
    return check(g_nccl.get_uid((nccl_uid*)id128), "ncclGetUniqueId");
}

int cml_nccl_init(void** comm, int nranks, int rank, const void* id128) {
    if (!comm || !id128 || load_nccl()) return -1;
    nccl_uid id;
    memcpy(&id, id128, sizeof id);
    return check(g_nccl.init_rank(comm, nranks, id, rank), "ncclCommInitRank");
}

int cml_nccl_allreduce_sum_f32(void* comm, float* d_buf, size_t count, void* stream) {
    if (!comm || !d_buf) return -1;
    return check(g_nccl.allreduce(d_buf, d_buf, count, 7 /* ncclFloat32 */, 0 /* ncclSum */, comm, stream), "ncclAllReduce");
}

/* Every rank contributes `bytes` bytes at d_send; d_recv receives nranks * bytes in rank order. */
int cml_nccl_allgather_bytes(void* comm, const void* d_send, void* d_recv, size_t bytes, void* stream) {
    if (!comm || !d_send || !d_recv || !g_nccl.allgather) return -1;
    return check(g_nccl.allgather(d_send, d_recv, bytes, 0 /* ncclInt8 */, comm, stream), "ncclAllGather");
}

void cml_nccl_destroy(void* comm) {
    if (comm && g_nccl.destroy) g_nccl.destroy(comm);
}
