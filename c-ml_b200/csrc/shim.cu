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
