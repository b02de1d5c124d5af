// Device runtime behind the C ABI: device/queue, buffers, begin/submit, copies.
// Counterpart of the reference's src/metal.cpp (device, one queue, buffer allocation,
// begin/submit); there is no pipeline cache because kernels are linked in.
#include "common.cuh"

#include <mutex>
#include <new>

namespace miori_b200 {

static thread_local char t_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace miori_b200

using namespace miori_b200;

struct miori_device {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    bool open_scope = false;
    std::mutex mu;  // two host threads may enqueue concurrently (reference src/server.cpp:294)
};

struct miori_buffer {
    miori_device* dev = nullptr;
    void* ptr = nullptr;
    size_t bytes = 0;
    bool shared = false;
};

MIORI_API const char* miori_last_error(void) { return t_err; }
MIORI_API const char* miori_version(void) { return "miori_b200 0.1 sm_100a"; }

MIORI_API int miori_device_open(int ordinal, miori_device** out) {
    if (!out) return fail(MIORI_E_INVALID, "miori_device_open: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(MIORI_E_CUDA, "no CUDA device: %s", cudaGetErrorString(e));
    if (ordinal < 0 || ordinal >= count)
        return fail(MIORI_E_INVALID, "device ordinal %d out of range (have %d)", ordinal, count);
    MIORI_CUDA(cudaSetDevice(ordinal));
    cudaDeviceProp prop;
    MIORI_CUDA(cudaGetDeviceProperties(&prop, ordinal));
    if (prop.major != 10)
        return fail(MIORI_E_INVALID, "device %d is sm_%d%d; this library is built for sm_100a only",
                    ordinal, prop.major, prop.minor);
    miori_device* d = new (std::nothrow) miori_device;
    if (!d) return fail(MIORI_E_NOMEM, "out of host memory");
    d->ordinal = ordinal;
    e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete d;
        return cuda_fail(e, "cudaStreamCreateWithFlags");
    }
    *out = d;
    return MIORI_OK;
}

MIORI_API int miori_device_close(miori_device* dev) {
    if (!dev) return MIORI_OK;
    cudaSetDevice(dev->ordinal);
    cudaStreamSynchronize(dev->stream);
    cudaStreamDestroy(dev->stream);
    delete dev;
    return MIORI_OK;
}

MIORI_API void* miori_device_stream(miori_device* dev) { return dev ? (void*)dev->stream : nullptr; }
MIORI_API int miori_device_ordinal(miori_device* dev) { return dev ? dev->ordinal : -1; }

MIORI_API int miori_buffer_alloc(miori_device* dev, size_t bytes, int shared, miori_buffer** out) {
    if (!dev || !out) return fail(MIORI_E_INVALID, "miori_buffer_alloc: null argument");
    *out = nullptr;
    if (bytes == 0) return fail(MIORI_E_INVALID, "miori_buffer_alloc: zero bytes");
    MIORI_CUDA(cudaSetDevice(dev->ordinal));
    miori_buffer* b = new (std::nothrow) miori_buffer;
    if (!b) return fail(MIORI_E_NOMEM, "out of host memory");
    cudaError_t e = shared ? cudaMallocManaged(&b->ptr, bytes, cudaMemAttachGlobal)
                           : cudaMalloc(&b->ptr, bytes);
    if (e != cudaSuccess) {
        delete b;
        (void)cudaGetLastError();
        return fail(MIORI_E_NOMEM, "buffer allocation of %zu bytes failed: %s", bytes,
                    cudaGetErrorString(e));
    }
    b->dev = dev;
    b->bytes = bytes;
    b->shared = shared != 0;
    *out = b;
    return MIORI_OK;
}

MIORI_API int miori_buffer_free(miori_buffer* buf) {
    if (!buf) return MIORI_OK;
    cudaSetDevice(buf->dev->ordinal);
    cudaError_t e = cudaFree(buf->ptr);
    delete buf;
    if (e != cudaSuccess) return cuda_fail(e, "cudaFree");
    return MIORI_OK;
}

MIORI_API void* miori_buffer_contents(miori_buffer* buf) {
    return (buf && buf->shared) ? buf->ptr : nullptr;
}
MIORI_API void* miori_buffer_device_ptr(miori_buffer* buf) { return buf ? buf->ptr : nullptr; }
MIORI_API size_t miori_buffer_length(miori_buffer* buf) { return buf ? buf->bytes : 0; }

MIORI_API int miori_buffer_prefetch(miori_buffer* buf, int to_device) {
    if (!buf) return fail(MIORI_E_INVALID, "miori_buffer_prefetch: null buffer");
    if (!buf->shared) return MIORI_OK;
    MIORI_CUDA(cudaSetDevice(buf->dev->ordinal));
    cudaMemLocation loc;
    loc.type = to_device ? cudaMemLocationTypeDevice : cudaMemLocationTypeHost;
    loc.id = to_device ? buf->dev->ordinal : 0;
    MIORI_CUDA(cudaMemPrefetchAsync_v2(buf->ptr, buf->bytes, loc, 0, buf->dev->stream));
    return MIORI_OK;
}

MIORI_API int miori_begin(miori_device* dev) {
    if (!dev) return fail(MIORI_E_INVALID, "miori_begin: null device");
    std::lock_guard<std::mutex> lk(dev->mu);
    MIORI_CUDA(cudaSetDevice(dev->ordinal));
    dev->open_scope = true;
    return MIORI_OK;
}

MIORI_API int miori_submit(miori_device* dev, int wait) {
    if (!dev) return fail(MIORI_E_INVALID, "miori_submit: null device");
    std::lock_guard<std::mutex> lk(dev->mu);
    dev->open_scope = false;
    if (wait) {
        MIORI_CUDA(cudaSetDevice(dev->ordinal));
        MIORI_CUDA(cudaStreamSynchronize(dev->stream));
    }
    return MIORI_OK;
}

MIORI_API int miori_host_alloc(size_t bytes, void** out) {
    if (!out || bytes == 0) return fail(MIORI_E_INVALID, "miori_host_alloc: bad argument");
    cudaError_t e = cudaMallocHost(out, bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(MIORI_E_NOMEM, "pinned allocation of %zu bytes failed: %s", bytes,
                    cudaGetErrorString(e));
    }
    return MIORI_OK;
}
MIORI_API int miori_host_free(void* p) {
    if (p) MIORI_CUDA(cudaFreeHost(p));
    return MIORI_OK;
}
MIORI_API int miori_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
    if (!dst || !src) return fail(MIORI_E_INVALID, "miori_memcpy_h2d: null pointer");
    MIORI_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return MIORI_OK;
}
MIORI_API int miori_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
    if (!dst || !src) return fail(MIORI_E_INVALID, "miori_memcpy_d2h: null pointer");
    MIORI_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return MIORI_OK;
}
MIORI_API int miori_stream_sync(void* stream) {
    MIORI_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return MIORI_OK;
}
