// The steps either side of a projection in the reference's decode graph (src/engine.cpp:389-413,
// 484-502): RMSNorm in front of it, SiLU x up or post-norm + residual behind it, and the 8-bit
// embedding gather that shares its table with the LM head.  Each is a small HBM- or latency-bound
// kernel; the RMSNorm also exists fused into the GEMV's activation staging (gemv_umma.cuh).
//   rmsnorm        shaders/ops.metal:86-115   y = bf16(x * rsqrt(mean(x^2) + eps) * w)
//   silu_mul       shaders/ops.metal:129-139  out = bf16(g / (1 + exp(-g)) * up)
//   post_norm_add  shaders/ops.metal:605-631  out = x + src * rsqrt(mean(src^2) + eps) * w
//   embed8         shaders/ops.metal:170-197  out[t][k] = bf16(code * scale + bias) of row tokens[t]
#include "common.cuh"
#include "norm.cuh"

namespace miori_b200 {
namespace neighbors {

__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w, uint16_t* __restrict__ y,
               uint32_t n, float eps) {
    __shared__ float part[NORM_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait_prior();
    const float* row = x + (size_t)blockIdx.x * n;
    const float inv = rsqrtf(row_sum_squares<0, false>(row, n, part) / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += NORM_THREADS)
        y[(size_t)blockIdx.x * n + i] = (uint16_t)float_to_bf16_bits(row[i] * inv * bf16_bits_to_float(w[i]));
}

__global__ void __launch_bounds__(NORM_THREADS)
post_norm_add_kernel(const float* __restrict__ x, const float* __restrict__ src,
                     const uint16_t* __restrict__ w, float* __restrict__ out, uint32_t n, float eps) {
    __shared__ float part[NORM_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait_prior();
    const size_t at = (size_t)blockIdx.x * n;
    post_norm_add_row<0, false>(x + at, src + at, w, out + at, n, eps, part);
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up, uint16_t* __restrict__ out,
                size_t n) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float g = gate[i];
        const float s = g / (1.0f + expf(-g));
        out[i] = (uint16_t)float_to_bf16_bits(s * up[i]);
    }
}

// One CTA per token: dequantize row tokens[t] of the 8-bit table.  A thread handles 16 codes (one
// 16-byte load), so a warp reads 512 contiguous bytes; fp32 multiply then add (unfused, like the
// cache build), integer round-to-nearest-even to bf16: bit-exact with src/cpu_ref.h:16-23,36-45.
__global__ void __launch_bounds__(128)
embed8_kernel(const uint4* __restrict__ q, const uint16_t* __restrict__ s, const uint16_t* __restrict__ b,
              const uint32_t* __restrict__ tokens, uint16_t* __restrict__ out, uint32_t K, uint32_t gshift,
              uint32_t rows) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const uint32_t tok = tokens[blockIdx.x];
    if (tok >= rows) return;  // an id outside the table leaves its output row untouched
    const uint32_t ng = K >> gshift;
    const uint4* qrow = q + (size_t)tok * (K / 16u);
    for (uint32_t c = threadIdx.x; c < K / 16u; c += blockDim.x) {
        const uint4 w = __ldg(qrow + c);
        const uint32_t g = (c * 16u) >> gshift;
        const float sc = bf16_bits_to_float(s[(size_t)tok * ng + g]);
        const float bi = bf16_bits_to_float(b[(size_t)tok * ng + g]);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const float v0 = __fadd_rn(__fmul_rn((float)((ww[i] >> (8 * j)) & 0xFFu), sc), bi);
                const float v1 = __fadd_rn(__fmul_rn((float)((ww[i] >> (8 * j + 8)) & 0xFFu), sc), bi);
                o[i * 2 + j / 2] = float_to_bf16_bits(v0) | (float_to_bf16_bits(v1) << 16);
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * K + (size_t)c * 16u);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

// Largest element of a vector and its index (ties: the lowest index, as the host loop of
// src/engine.cpp:740-747 finds it).  A thread-block cluster of up to 8 CTAs shares the vector:
// 16-byte loads, a shuffle and shared-memory reduction per CTA, then every CTA hands its
// candidate to CTA 0 through distributed shared memory and CTA 0's first thread holds the result.
struct Best {
    float v;
    uint32_t i;
};
constexpr int ARGMAX_THREADS = 1024, ARGMAX_CLUSTER = 8;
__device__ __forceinline__ Best better(Best a, Best b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// This CTA's best over its slice of v[0, n): elements are compared in index order inside a thread
// and ties across threads go to the lower index, so the result is the first maximum.
template <bool BF16>
__device__ __forceinline__ Best block_argmax(const void* __restrict__ v, uint32_t n, uint32_t index0,
                                             Best* warp_best) {
    constexpr uint32_t PER = BF16 ? 8u : 4u;  // elements per 16-byte load
    const uint32_t nct = cluster_nctarank(), cr = cluster_ctarank();
    // slices of whole 16-byte pieces; the last CTA also takes the ragged tail
    const uint32_t pieces = n / PER, per_cta = (pieces + nct - 1u) / nct;
    const uint32_t p0 = min(cr * per_cta, pieces), p1 = min(p0 + per_cta, pieces);
    Best me = {-INFINITY, 0xFFFFFFFFu};
    const bool vec_ok = (reinterpret_cast<uintptr_t>(v) & 15u) == 0;
    if (vec_ok) {
        const uint4* v4 = static_cast<const uint4*>(v);
        for (uint32_t p = p0 + threadIdx.x; p < p1; p += blockDim.x) {
            const uint4 w = __ldg(v4 + p);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            const uint32_t i0 = index0 + p * PER;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (BF16) {
                    me = better(me, Best{bf16lo(ww[k]), i0 + 2u * k});
                    me = better(me, Best{bf16hi(ww[k]), i0 + 2u * k + 1u});
                } else {
                    me = better(me, Best{__uint_as_float(ww[k]), i0 + (uint32_t)k});
                }
            }
        }
    }
    // scalar part: everything when v is not 16-byte aligned (CTA 0 of the cluster walks it all),
    // else the tail past the last whole piece (last CTA)
    uint32_t s0 = n, s1 = n;
    if (!vec_ok) { if (cr == 0u) s0 = 0u; }
    else if (cr == nct - 1u) s0 = pieces * PER;
    for (uint32_t i = s0 + threadIdx.x; i < s1; i += blockDim.x) {
        const float f = BF16 ? bf16_bits_to_float(static_cast<const uint16_t*>(v)[i])
                             : static_cast<const float*>(v)[i];
        me = better(me, Best{f, index0 + i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xFFFFFFFFu, me.v, o);
        other.i = __shfl_xor_sync(0xFFFFFFFFu, me.i, o);
        me = better(me, other);
    }
    if ((threadIdx.x & 31u) == 0) warp_best[threadIdx.x >> 5] = me;
    __syncthreads();
    Best all = warp_best[0];
    for (uint32_t w = 1; w < blockDim.x / 32u; ++w) all = better(all, warp_best[w]);
    return all;
}
// Cluster-wide result, valid in thread 0 of CTA 0 of the cluster.  Every thread of every CTA of
// the cluster must call it (it contains cluster barriers).  cta_best: ARGMAX_CLUSTER entries of
// shared memory, at the same offset in every CTA.
template <bool BF16>
__device__ __forceinline__ Best cluster_argmax(const void* __restrict__ v, uint32_t n, uint32_t index0,
                                               Best* warp_best, Best* cta_best) {
    const Best mine = block_argmax<BF16>(v, n, index0, warp_best);
    const uint32_t nct = cluster_nctarank(), cr = cluster_ctarank();
    if (nct == 1u) return mine;
    if (threadIdx.x == 0) {
        uint32_t remote;  // cta_best[cr] in CTA 0's shared memory
        asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(smem_addr(cta_best + cr)));
        asm volatile("st.shared::cluster.v2.u32 [%0], {%1, %2};" ::"r"(remote), "r"(__float_as_uint(mine.v)), "r"(mine.i)
                     : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    Best all = mine;
    if (cr == 0u && threadIdx.x == 0)
        for (uint32_t c = 1; c < nct; ++c) all = better(all, cta_best[c]);
    return all;
}
template <bool BF16>
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const void* __restrict__ v, uint32_t n, uint32_t index0, uint32_t* __restrict__ out_index,
              float* __restrict__ out_value) {
    __shared__ Best warp_best[32];
    __shared__ __align__(8) Best cta_best[ARGMAX_CLUSTER];
    pdl_launch_dependents();
    pdl_wait_prior();
    const Best all = cluster_argmax<BF16>(v, n, index0, warp_best, cta_best);
    if (cluster_ctarank() == 0u && threadIdx.x == 0) {
        *out_index = all.i;
        if (out_value) *out_value = all.v;
    }
}
// CTAs for a vector of n elements: one per 8192 elements, at most a cluster of 8.
inline unsigned argmax_ctas(uint32_t n) {
    const unsigned c = (n + 8191u) / 8192u;
    return c >= 8u ? 8u : c >= 4u ? 4u : c >= 2u ? 2u : 1u;
}
// Launch with `ctas` CTAs forming one cluster.
template <class... KArgs, class... Args>
inline cudaError_t launch_cluster(void (*kernel)(KArgs...), unsigned ctas, unsigned threads, cudaStream_t stream,
                                  bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = ctas;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace neighbors
}  // namespace miori_b200

using namespace miori_b200;

MIORI_API int miori_rmsnorm(const void* x, const void* gamma, void* y, uint32_t rows, uint32_t n, float eps,
                            uint32_t flags, void* stream) {
    if (!x || !gamma || !y) return fail(MIORI_E_INVALID, "miori_rmsnorm: null pointer");
    if (rows == 0 || n == 0) return fail(MIORI_E_INVALID, "miori_rmsnorm: empty shape rows=%u n=%u", rows, n);
    const cudaError_t e = launch(neighbors::rmsnorm_kernel, dim3(rows), dim3(neighbors::NORM_THREADS), 0,
                                 (cudaStream_t)stream, (flags & MIORI_LAUNCH_PDL) != 0,
                                 static_cast<const float*>(x), static_cast<const uint16_t*>(gamma),
                                 static_cast<uint16_t*>(y), n, eps);
    if (e != cudaSuccess) return cuda_fail(e, "miori_rmsnorm launch");
    return MIORI_OK;
}

MIORI_API int miori_post_norm_add(const void* x, const void* src, const void* gamma, void* out, uint32_t rows,
                                  uint32_t n, float eps, uint32_t flags, void* stream) {
    if (!x || !src || !gamma || !out) return fail(MIORI_E_INVALID, "miori_post_norm_add: null pointer");
    if (rows == 0 || n == 0) return fail(MIORI_E_INVALID, "miori_post_norm_add: empty shape rows=%u n=%u", rows, n);
    const cudaError_t e = launch(neighbors::post_norm_add_kernel, dim3(rows), dim3(neighbors::NORM_THREADS), 0,
                                 (cudaStream_t)stream, (flags & MIORI_LAUNCH_PDL) != 0,
                                 static_cast<const float*>(x), static_cast<const float*>(src),
                                 static_cast<const uint16_t*>(gamma), static_cast<float*>(out), n, eps);
    if (e != cudaSuccess) return cuda_fail(e, "miori_post_norm_add launch");
    return MIORI_OK;
}

MIORI_API int miori_silu_mul(const void* gate, const void* up, void* out, size_t n, uint32_t flags, void* stream) {
    if (!gate || !up || !out) return fail(MIORI_E_INVALID, "miori_silu_mul: null pointer");
    if (n == 0) return fail(MIORI_E_INVALID, "miori_silu_mul: empty vector");
    const unsigned blocks = (unsigned)std::min<size_t>((n + 255) / 256, (size_t)sm_count() * 8);
    const cudaError_t e = launch(neighbors::silu_mul_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
                                 (flags & MIORI_LAUNCH_PDL) != 0, static_cast<const float*>(gate),
                                 static_cast<const float*>(up), static_cast<uint16_t*>(out), n);
    if (e != cudaSuccess) return cuda_fail(e, "miori_silu_mul launch");
    return MIORI_OK;
}

MIORI_API int miori_embed8(const void* q, const void* s, const void* b, const void* tokens, void* out,
                           uint32_t T, uint32_t rows, uint32_t K, uint32_t group, uint32_t flags, void* stream) {
    if (!q || !s || !b || !tokens || !out) return fail(MIORI_E_INVALID, "miori_embed8: null pointer");
    if (group != 32 && group != 64) return fail(MIORI_E_INVALID, "miori_embed8: group must be 32 or 64 (got %u)", group);
    if (T == 0 || rows == 0 || K == 0 || K % group != 0 || K % 16 != 0)
        return fail(MIORI_E_INVALID, "miori_embed8: bad shape T=%u rows=%u K=%u group=%u", T, rows, K, group);
    if (!aligned16(q) || !aligned16(out)) return fail(MIORI_E_INVALID, "miori_embed8: q and out must be 16-byte aligned");
    const cudaError_t e = launch(neighbors::embed8_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream,
                                 (flags & MIORI_LAUNCH_PDL) != 0, static_cast<const uint4*>(q),
                                 static_cast<const uint16_t*>(s), static_cast<const uint16_t*>(b),
                                 static_cast<const uint32_t*>(tokens), static_cast<uint16_t*>(out), K,
                                 group == 32 ? 5u : 6u, rows);
    if (e != cudaSuccess) return cuda_fail(e, "miori_embed8 launch");
    return MIORI_OK;
}

MIORI_API int miori_argmax(const void* v, uint32_t n, uint32_t flags, void* out_index, void* out_value,
                           void* stream) {
    if (!v || !out_index) return fail(MIORI_E_INVALID, "miori_argmax: null pointer");
    if (n == 0) return fail(MIORI_E_INVALID, "miori_argmax: empty vector");
    cudaError_t e;
    if (flags & MIORI_OUT_BF16)
        e = neighbors::launch_cluster(neighbors::argmax_kernel<true>, neighbors::argmax_ctas(n),
                                      neighbors::ARGMAX_THREADS, (cudaStream_t)stream,
                                      (flags & MIORI_LAUNCH_PDL) != 0, v, n, 0u, static_cast<uint32_t*>(out_index),
                                      static_cast<float*>(out_value));
    else
        e = neighbors::launch_cluster(neighbors::argmax_kernel<false>, neighbors::argmax_ctas(n),
                                      neighbors::ARGMAX_THREADS, (cudaStream_t)stream,
                                      (flags & MIORI_LAUNCH_PDL) != 0, v, n, 0u, static_cast<uint32_t*>(out_index),
                                      static_cast<float*>(out_value));
    if (e != cudaSuccess) return cuda_fail(e, "miori_argmax launch");
    return MIORI_OK;
}
