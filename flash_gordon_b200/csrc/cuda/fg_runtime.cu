// CUDA runtime plumbing behind the C host layer: device selection, streams,
// allocations and copies.  No kernels here.  Each function returns the
// cudaError_t as int so the C side needs no CUDA headers.
#include <cuda_runtime.h>

#include "fg_kernels.h"

extern "C" int fgk_device_count(int *count) { return (int)cudaGetDeviceCount(count); }

extern "C" int fgk_set_device(int device) { return (int)cudaSetDevice(device); }

extern "C" int fgk_device_sm_count(int device, int *sm_count) {
    return (int)cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, device);
}

extern "C" int fgk_stream_create(void **stream) {
    cudaStream_t s = nullptr;
    const cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    *stream = s;
    return (int)e;
}

extern "C" int fgk_stream_destroy(void *stream) {
    return (int)cudaStreamDestroy(static_cast<cudaStream_t>(stream));
}

extern "C" int fgk_stream_synchronize(void *stream) {
    return (int)cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
}

extern "C" int fgk_malloc(void **pointer, size_t bytes) { return (int)cudaMalloc(pointer, bytes); }

extern "C" int fgk_free(void *pointer) { return (int)cudaFree(pointer); }

extern "C" int fgk_host_alloc(void **pointer, size_t bytes) {
    return (int)cudaHostAlloc(pointer, bytes, cudaHostAllocDefault);
}

extern "C" int fgk_host_free(void *pointer) { return (int)cudaFreeHost(pointer); }

extern "C" int fgk_memset_async(void *pointer, int value, size_t bytes, void *stream) {
    return (int)cudaMemsetAsync(pointer, value, bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int fgk_copy_to_device_async(void *device, const void *host, size_t bytes, void *stream) {
    return (int)cudaMemcpyAsync(device, host, bytes, cudaMemcpyHostToDevice,
                                static_cast<cudaStream_t>(stream));
}

extern "C" int fgk_copy_to_host_async(void *host, const void *device, size_t bytes, void *stream) {
    return (int)cudaMemcpyAsync(host, device, bytes, cudaMemcpyDeviceToHost,
                                static_cast<cudaStream_t>(stream));
}

extern "C" const char *fgk_error_string(int cuda_error) {
    return cudaGetErrorString(static_cast<cudaError_t>(cuda_error));
}
