// Device plumbing of the cmlb200 C-ABI: errors, memory, copies, streams.
#include <stdarg.h>
#include <string.h>
#include "common.cuh"

static thread_local char g_err[512] = "";

extern "C" void cmlb200_set_error_(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

extern "C" const char* cmlb200_last_error(void) { return g_err; }

extern "C" int cmlb200_device_count(int* count) {
    CMLB_REQUIRE(count, "cmlb200_device_count: NULL argument");
    CMLB_CUDA(cudaGetDeviceCount(count));
    return CMLB200_OK;
}
extern "C" int cmlb200_set_device(int device) {
    CMLB_CUDA(cudaSetDevice(device));
    return CMLB200_OK;
}
extern "C" int cmlb200_malloc(void** d_ptr, size_t bytes) {
    CMLB_REQUIRE(d_ptr, "cmlb200_malloc: NULL argument");
    *d_ptr = nullptr;
    CMLB_CUDA(cudaMalloc(d_ptr, bytes ? bytes : 1));
    return CMLB200_OK;
}
extern "C" int cmlb200_free(void* d_ptr) {
    if (d_ptr) CMLB_CUDA(cudaFree(d_ptr));
    return CMLB200_OK;
}
extern "C" int cmlb200_host_alloc_pinned(void** h_ptr, size_t bytes) {
    CMLB_REQUIRE(h_ptr, "cmlb200_host_alloc_pinned: NULL argument");
    *h_ptr = nullptr;
    CMLB_CUDA(cudaMallocHost(h_ptr, bytes ? bytes : 1));
    return CMLB200_OK;
}
extern "C" int cmlb200_host_free_pinned(void* h_ptr) {
    if (h_ptr) CMLB_CUDA(cudaFreeHost(h_ptr));
    return CMLB200_OK;
}
extern "C" int cmlb200_memcpy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream) {
    CMLB_REQUIRE(d_dst && h_src, "cmlb200_memcpy_h2d: NULL argument");
    CMLB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_memcpy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream) {
    CMLB_REQUIRE(h_dst && d_src, "cmlb200_memcpy_d2h: NULL argument");
    CMLB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_memcpy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream) {
    CMLB_REQUIRE(d_dst && d_src, "cmlb200_memcpy_d2d: NULL argument");
    CMLB_CUDA(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_memset(void* d_dst, int value, size_t bytes, void* stream) {
    CMLB_REQUIRE(d_dst, "cmlb200_memset: NULL argument");
    CMLB_CUDA(cudaMemsetAsync(d_dst, value, bytes, as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_stream_create(void** stream) {
    CMLB_REQUIRE(stream, "cmlb200_stream_create: NULL argument");
    cudaStream_t s;
    CMLB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return CMLB200_OK;
}
extern "C" int cmlb200_stream_destroy(void* stream) {
    if (stream) CMLB_CUDA(cudaStreamDestroy(as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_stream_sync(void* stream) {
    CMLB_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_device_sync(void) {
    CMLB_CUDA(cudaDeviceSynchronize());
    return CMLB200_OK;
}

extern "C" int cmlb200_graph_begin(void* stream) {
    CMLB_CUDA(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeRelaxed));
    return CMLB200_OK;
}
extern "C" int cmlb200_graph_end(void* stream, void** graph_exec) {
    CMLB_REQUIRE(graph_exec, "cmlb200_graph_end: NULL argument");
    cudaGraph_t g = nullptr;
    CMLB_CUDA(cudaStreamEndCapture(as_stream(stream), &g));
    cudaGraphExec_t e = nullptr;
    cudaError_t err = cudaGraphInstantiate(&e, g, 0);
    cudaGraphDestroy(g);
    CMLB_CUDA(err);
    *graph_exec = e;
    return CMLB200_OK;
}
extern "C" int cmlb200_graph_launch(void* graph_exec, void* stream) {
    CMLB_REQUIRE(graph_exec, "cmlb200_graph_launch: NULL argument");
    CMLB_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_graph_destroy(void* graph_exec) {
    if (graph_exec) CMLB_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
    return CMLB200_OK;
}
extern "C" int cmlb200_event_create(void** event) {
    CMLB_REQUIRE(event, "cmlb200_event_create: NULL argument");
    cudaEvent_t e;
    CMLB_CUDA(cudaEventCreate(&e));
    *event = e;
    return CMLB200_OK;
}
extern "C" int cmlb200_event_record(void* event, void* stream) {
    CMLB_CUDA(cudaEventRecord((cudaEvent_t)event, as_stream(stream)));
    return CMLB200_OK;
}
extern "C" int cmlb200_event_elapsed_ms(void* start, void* stop, float* ms) {
    CMLB_REQUIRE(ms, "cmlb200_event_elapsed_ms: NULL argument");
    CMLB_CUDA(cudaEventSynchronize((cudaEvent_t)stop));
    CMLB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return CMLB200_OK;
}
extern "C" int cmlb200_event_destroy(void* event) {
    if (event) CMLB_CUDA(cudaEventDestroy((cudaEvent_t)event));
    return CMLB200_OK;
}
