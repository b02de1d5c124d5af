// Shared host/device helpers for the miori_b200 CUDA library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/miori_b200.h"
#include "tune.h"

#define MIORI_API extern "C" __attribute__((visibility("default")))

namespace miori_b200 {

// Records the calling thread's last error message and returns `code`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

inline int cuda_fail(cudaError_t e, const char* what) {
    return fail(MIORI_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define MIORI_CUDA(call)                                                  \
    do {                                                                  \
        cudaError_t e__ = (call);                                         \
        if (e__ != cudaSuccess) return miori_b200::cuda_fail(e__, #call); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device ordinal).
int sm_count();

// Launch helper: grid/block/smem on `stream`, optionally with the programmatic
// dependent launch attribute so that the kernel may begin before its predecessor ends.
template <class... KArgs, class... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Device-side record of kernel-internal failures (bounded waits that expired).
// word 0: error count, word 1: code of the first failure, word 2/3: detail.
__device__ unsigned int g_device_error[4];

#ifdef __CUDACC__
__device__ __forceinline__ void device_error(unsigned code, unsigned d0, unsigned d1) {
    if (atomicAdd(&g_device_error[0], 1u) == 0u) {
        g_device_error[1] = code;
        g_device_error[2] = d0;
        g_device_error[3] = d1;
    }
}

// Programmatic dependent launch controls (no-ops when the launch is not programmatic).
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_prior() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- shared-memory barriers (mbarrier) and bounded waits -------------------------------
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // ~1 s at boost clock

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the CTA is aborting (this or another role gave up); on
// expiry it raises the CTA's abort flag and records a device error with code `where`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort,
                                          uint32_t where) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (*abort) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort = 1u;
            device_error(0x6E00u | where, blockIdx.x, parity);
            return false;
        }
    }
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t v16) {
    return __uint_as_float(v16 << 16);
}
__device__ __forceinline__ float bf16lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16hi(uint32_t pair) {
    return __uint_as_float(pair & 0xFFFF0000u);
}
// RNE fp32 -> bf16 bits for finite inputs, the reference's rule (src/cpu_ref.h:16-23).
__device__ __forceinline__ uint32_t float_to_bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return u >> 16;
}
#endif

}  // namespace miori_b200
