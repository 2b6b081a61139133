/* Internal helpers shared by the C11 host sources (not part of the public API). */
#ifndef CML_INTERNAL_H
#define CML_INTERNAL_H

#include "cml_quant_api.h"
#include "cmlb200.h"

/* Logs the cmlb200 error text and evaluates to true when a C-ABI call failed. */
#define CML_DEV_FAIL(call, who) ((call) != CMLB200_OK ? (LOG_ERROR("%s: %s", (who), cmlb200_last_error()), 1) : 0)

Tensor* cml_tensor_alloc(DType dtype, const int* shape, int ndim, bool zero);

/* GGUF reader internals used by the model loader. */
typedef struct GGUFTensorInfo {
    char* name;
    int ndim;
    int64_t shape[8];
    GGUFTensorType type;
    uint64_t offset;
    size_t data_size;
} GGUFTensorInfo;
const GGUFTensorInfo* cml_gguf_find(GGUFContext* ctx, const char* name);
/* Raw bytes of a tensor exactly as stored in the file (malloc'd, caller frees). */
void* cml_gguf_read_raw(GGUFContext* ctx, const GGUFTensorInfo* info);

/* fp16 <-> fp32 on the host (IEEE, round to nearest even) for norm / embedding tensors. */
uint16_t cml_f32_to_f16(float f);
float cml_f16_to_f32(uint16_t h);

/* NCCL, loaded with dlopen (src/distributed/nccl_backend.c:476-479 does the same). */
int cml_nccl_unique_id(void* id128);
int cml_nccl_init(void** comm, int nranks, int rank, const void* id128);
int cml_nccl_allreduce_sum_f32(void* comm, float* d_buf, size_t count, void* stream);
int cml_nccl_allgather_bytes(void* comm, const void* d_send, void* d_recv, size_t bytes, void* stream);
void cml_nccl_destroy(void* comm);

#endif
