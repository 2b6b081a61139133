/*
 * C-ML's tensor-parallel building blocks (include/distributed/tensor_parallel.h:12-59,
 * src/distributed/tensor_parallel.c) for fp32 weights, as stand-alone entry points: the shards are
 * host tensors cut exactly as C-ML cuts them, the forward passes (y = x . W_shard^T + b) and the sum
 * over partial results run on the device. The quantized model does its own sharding
 * (cml_tp_shard_qblocks) and all-reduce (cml_llama.c); these are for callers that build their own
 * layers out of the blocks.
 */
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

#define FAIL(call, who) CML_DEV_FAIL(call, who)

/* src/distributed/tensor_parallel.c:25-101 */
Tensor* cml_tp_shard_weight(Tensor* weight, int dim, int tp_size, int tp_rank) {
    if (!weight) { LOG_ERROR("cml_tp_shard_weight: weight is NULL"); return NULL; }
    if (weight->ndim != 2) { LOG_ERROR("cml_tp_shard_weight: expected 2-D weight, got ndim=%d", weight->ndim); return NULL; }
    if (dim != 0 && dim != 1) { LOG_ERROR("cml_tp_shard_weight: dim must be 0 or 1, got %d", dim); return NULL; }
    if (tp_size <= 0 || tp_rank < 0 || tp_rank >= tp_size) { LOG_ERROR("cml_tp_shard_weight: invalid tp_size=%d or tp_rank=%d", tp_size, tp_rank); return NULL; }
    const int rows = weight->shape[0], cols = weight->shape[1];
    if (dim == 0 && rows % tp_size != 0) { LOG_ERROR("cml_tp_shard_weight: rows (%d) not divisible by tp_size (%d)", rows, tp_size); return NULL; }
    if (dim == 1 && cols % tp_size != 0) { LOG_ERROR("cml_tp_shard_weight: cols (%d) not divisible by tp_size (%d)", cols, tp_size); return NULL; }
    const float* src = (const float*)weight->data;
    if (!src) { LOG_ERROR("cml_tp_shard_weight: failed to get weight data"); return NULL; }
    if (dim == 0) {
        const int shape[2] = {rows / tp_size, cols};
        Tensor* shard = cml_tensor_alloc(DTYPE_FLOAT32, shape, 2, false);
        if (!shard) { LOG_ERROR("cml_tp_shard_weight: allocation failed"); return NULL; }
        const size_t n = (size_t)shape[0] * cols;
        memcpy(shard->data, src + (size_t)tp_rank * n, n * sizeof(float));
        return shard;
    }
    const int sc = cols / tp_size;
    const int shape[2] = {rows, sc};
    Tensor* shard = cml_tensor_alloc(DTYPE_FLOAT32, shape, 2, false);
    if (!shard) { LOG_ERROR("cml_tp_shard_weight: allocation failed"); return NULL; }
    for (int r = 0; r < rows; r++)
        memcpy((float*)shard->data + (size_t)r * sc, src + (size_t)r * cols + (size_t)tp_rank * sc, (size_t)sc * sizeof(float));
    return shard;
}

static Tensor* bias_slice(const Tensor* full_bias, int offset, int n, const char* who) {
    if (!full_bias->data) { LOG_ERROR("%s: failed to get bias data", who); return NULL; }
    const int shape[1] = {n};
    Tensor* b = cml_tensor_alloc(DTYPE_FLOAT32, shape, 1, false);
    if (!b) { LOG_ERROR("%s: failed to create bias tensor", who); return NULL; }
    memcpy(b->data, (const float*)full_bias->data + offset, (size_t)n * sizeof(float));
    return b;
}

/* y[batch, N] = x[batch, K] . w[N, K]^T (+ bias) on the device */
static Tensor* linear_device(const Tensor* input, const Tensor* weight, const Tensor* bias, const char* who) {
    const int M = input->shape[0], K = input->shape[1], N = weight->shape[0];
    if (!input->data || !weight->data) { LOG_ERROR("%s: failed to get data pointers", who); return NULL; }
    const int oshape[2] = {M, N};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, oshape, 2, false);
    void *d_x = NULL, *d_w = NULL, *d_b = NULL, *d_y = NULL;
    int ok = out != NULL;
    ok = ok && !FAIL(cmlb200_malloc(&d_x, (size_t)M * K * 4), who) && !FAIL(cmlb200_malloc(&d_w, (size_t)N * K * 4), who) &&
         !FAIL(cmlb200_malloc(&d_y, (size_t)M * N * 4), who);
    ok = ok && !FAIL(cmlb200_memcpy_h2d(d_x, input->data, (size_t)M * K * 4, NULL), who) &&
         !FAIL(cmlb200_memcpy_h2d(d_w, weight->data, (size_t)N * K * 4, NULL), who);
    if (ok && bias && bias->data)
        ok = !FAIL(cmlb200_malloc(&d_b, (size_t)N * 4), who) && !FAIL(cmlb200_memcpy_h2d(d_b, bias->data, (size_t)N * 4, NULL), who);
    ok = ok && !FAIL(cmlb200_linear_f32((const float*)d_x, (const float*)d_w, (const float*)d_b, M, N, K, (float*)d_y, NULL), who);
    ok = ok && !FAIL(cmlb200_memcpy_d2h(out->data, d_y, (size_t)M * N * 4, NULL), who) && !FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_x); cmlb200_free(d_w); cmlb200_free(d_b); cmlb200_free(d_y);
    if (!ok) { tensor_free(out); return NULL; }
    return out;
}

/* src/distributed/tensor_parallel.c:103-260 */
CMLColumnParallelLinear* cml_column_parallel_create(Tensor* full_weight, Tensor* full_bias, int tp_size, int tp_rank) {
    if (!full_weight) { LOG_ERROR("cml_column_parallel_create: full_weight is NULL"); return NULL; }
    if (full_weight->ndim != 2) { LOG_ERROR("cml_column_parallel_create: expected 2-D weight, got ndim=%d", full_weight->ndim); return NULL; }
    if (tp_size <= 0 || tp_rank < 0 || tp_rank >= tp_size) { LOG_ERROR("cml_column_parallel_create: invalid tp_size=%d or tp_rank=%d", tp_size, tp_rank); return NULL; }
    const int out_features = full_weight->shape[0], in_features = full_weight->shape[1];
    if (out_features % tp_size != 0) { LOG_ERROR("cml_column_parallel_create: out_features (%d) not divisible by tp_size (%d)", out_features, tp_size); return NULL; }
    CMLColumnParallelLinear* cp = (CMLColumnParallelLinear*)calloc(1, sizeof *cp);
    if (!cp) { LOG_ERROR("cml_column_parallel_create: allocation failed"); return NULL; }
    cp->in_features = in_features;
    cp->out_features = out_features;
    cp->tp_size = tp_size;
    cp->tp_rank = tp_rank;
    cp->weight = cml_tp_shard_weight(full_weight, 0, tp_size, tp_rank);
    if (!cp->weight) { LOG_ERROR("cml_column_parallel_create: failed to shard weight"); free(cp); return NULL; }
    if (full_bias) {
        const int so = out_features / tp_size;
        cp->bias = bias_slice(full_bias, tp_rank * so, so, "cml_column_parallel_create");
        if (!cp->bias) { tensor_free(cp->weight); free(cp); return NULL; }
    }
    return cp;
}

void cml_column_parallel_free(CMLColumnParallelLinear* cp) {
    if (!cp) return;
    tensor_free(cp->weight);
    tensor_free(cp->bias);
    free(cp);
}

Tensor* cml_column_parallel_forward(CMLColumnParallelLinear* cp, Tensor* input) {
    if (!cp || !input) { LOG_ERROR("cml_column_parallel_forward: NULL argument"); return NULL; }
    if (input->ndim != 2) { LOG_ERROR("cml_column_parallel_forward: expected 2-D input, got ndim=%d", input->ndim); return NULL; }
    if (input->shape[1] != cp->in_features) {
        LOG_ERROR("cml_column_parallel_forward: input in_features (%d) != expected (%d)", input->shape[1], cp->in_features);
        return NULL;
    }
    return linear_device(input, cp->weight, cp->bias, "cml_column_parallel_forward");
}

/* src/distributed/tensor_parallel.c:262-400: the weight is cut along the input dimension, the bias
 * stays whole on rank 0 only, and the caller sums the partial outputs over the ranks. */
CMLRowParallelLinear* cml_row_parallel_create(Tensor* full_weight, Tensor* full_bias, int tp_size, int tp_rank) {
    if (!full_weight) { LOG_ERROR("cml_row_parallel_create: full_weight is NULL"); return NULL; }
    if (full_weight->ndim != 2) { LOG_ERROR("cml_row_parallel_create: expected 2-D weight, got ndim=%d", full_weight->ndim); return NULL; }
    if (tp_size <= 0 || tp_rank < 0 || tp_rank >= tp_size) { LOG_ERROR("cml_row_parallel_create: invalid tp_size=%d or tp_rank=%d", tp_size, tp_rank); return NULL; }
    const int out_features = full_weight->shape[0], in_features = full_weight->shape[1];
    if (in_features % tp_size != 0) { LOG_ERROR("cml_row_parallel_create: in_features (%d) not divisible by tp_size (%d)", in_features, tp_size); return NULL; }
    CMLRowParallelLinear* rp = (CMLRowParallelLinear*)calloc(1, sizeof *rp);
    if (!rp) { LOG_ERROR("cml_row_parallel_create: allocation failed"); return NULL; }
    rp->in_features = in_features;
    rp->out_features = out_features;
    rp->tp_size = tp_size;
    rp->tp_rank = tp_rank;
    rp->weight = cml_tp_shard_weight(full_weight, 1, tp_size, tp_rank);
    if (!rp->weight) { LOG_ERROR("cml_row_parallel_create: failed to shard weight"); free(rp); return NULL; }
    if (full_bias && tp_rank == 0) {
        rp->bias = bias_slice(full_bias, 0, out_features, "cml_row_parallel_create");
        if (!rp->bias) { tensor_free(rp->weight); free(rp); return NULL; }
    }
    return rp;
}

void cml_row_parallel_free(CMLRowParallelLinear* rp) {
    if (!rp) return;
    tensor_free(rp->weight);
    tensor_free(rp->bias);
    free(rp);
}

Tensor* cml_row_parallel_forward(CMLRowParallelLinear* rp, Tensor* input) {
    if (!rp || !input) { LOG_ERROR("cml_row_parallel_forward: NULL argument"); return NULL; }
    if (input->ndim != 2) { LOG_ERROR("cml_row_parallel_forward: expected 2-D input, got ndim=%d", input->ndim); return NULL; }
    const int expected_in = rp->in_features / rp->tp_size;
    if (input->shape[1] != expected_in) {
        LOG_ERROR("cml_row_parallel_forward: input in_features (%d) != expected (%d)", input->shape[1], expected_in);
        return NULL;
    }
    return linear_device(input, rp->weight, rp->bias, "cml_row_parallel_forward");
}

/* Element-wise sum of same-shaped partial results, in list order. */
Tensor* cml_tp_all_reduce_sum(Tensor** partials, int num_parts) {
    if (!partials || num_parts <= 0) { LOG_ERROR("cml_tp_all_reduce_sum: invalid arguments"); return NULL; }
    for (int i = 0; i < num_parts; i++) {
        if (!partials[i] || !partials[i]->data) { LOG_ERROR("cml_tp_all_reduce_sum: partial %d is NULL", i); return NULL; }
        if (partials[i]->numel != partials[0]->numel || partials[i]->ndim != partials[0]->ndim) {
            LOG_ERROR("cml_tp_all_reduce_sum: shape mismatch at partial %d", i);
            return NULL;
        }
    }
    const size_t n = partials[0]->numel;
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, partials[0]->shape, partials[0]->ndim, false);
    void *d_acc = NULL, *d_in = NULL;
    const char* who = "cml_tp_all_reduce_sum";
    int ok = out != NULL && !FAIL(cmlb200_malloc(&d_acc, n * 4), who) && !FAIL(cmlb200_malloc(&d_in, n * 4), who) &&
             !FAIL(cmlb200_memcpy_h2d(d_acc, partials[0]->data, n * 4, NULL), who);
    for (int i = 1; i < num_parts && ok; i++)
        ok = !FAIL(cmlb200_memcpy_h2d(d_in, partials[i]->data, n * 4, NULL), who) &&
             !FAIL(cmlb200_add_f32((float*)d_acc, (const float*)d_in, n, NULL), who);
    ok = ok && !FAIL(cmlb200_memcpy_d2h(out->data, d_acc, n * 4, NULL), who) && !FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_acc); cmlb200_free(d_in);
    if (!ok) { tensor_free(out); return NULL; }
    return out;
}
