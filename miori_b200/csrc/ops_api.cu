// C ABI launch entries: argument validation, path selection, enqueue.
#include "common.cuh"
#include "dequant.cuh"
#include "gemv_mma.cuh"
#include "gemv_simt.cuh"
#include "gemv_tma.cuh"
#include "gemv_umma.cuh"
#include "gemv_cache.cuh"

using namespace miori_b200;

namespace {

int check_quant_args(const char* op, const void* q, const void* s, const void* b, uint32_t N,
                     uint32_t K, uint32_t group) {
    if (!q || !s || !b) return fail(MIORI_E_INVALID, "%s: null weight pointer", op);
    if (group != 32 && group != 64)
        return fail(MIORI_E_INVALID, "%s: group must be 32 or 64 (got %u)", op, group);
    if (N == 0 || K == 0) return fail(MIORI_E_INVALID, "%s: empty shape N=%u K=%u", op, N, K);
    if (K % group != 0)
        return fail(MIORI_E_INVALID, "%s: K=%u is not a multiple of the group %u", op, K, group);
    if (!aligned16(q) || !aligned16(s) || !aligned16(b))
        return fail(MIORI_E_INVALID, "%s: q, s and b must be 16-byte aligned", op);
    return MIORI_OK;
}

template <int BITS>
int gemv_entry(const char* op, const void* q, const void* s, const void* b, const void* x, void* y,
               uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags, void* stream) {
    int rc = check_quant_args(op, q, s, b, N, K, group);
    if (rc) return rc;
    if (!x || !y) return fail(MIORI_E_INVALID, "%s: null activation pointer", op);
    if (M == 0 || M > 32) return fail(MIORI_E_INVALID, "%s: M=%u outside 1..32", op, M);
    if (!aligned16(x)) return fail(MIORI_E_INVALID, "%s: x must be 16-byte aligned", op);
    const bool force_exact = (flags & MIORI_GEMV_EXACT) != 0;
    const bool force_simt = (flags & MIORI_TUNE_GEMV_SIMT) != 0;  // tuning override: shape-agnostic SIMT path
    const bool no_bulk = (flags & MIORI_TUNE_GEMV_LDG) != 0;     // tuning override: register-streaming kernel
    // The tcgen05 kernel (integer tensor cores, fp32 dequantization with an exact inner sum for
    // every M).  By default it takes the 8-bit weights from three activation rows up: there the
    // mma.sync kernel needs a second column set (M = 3, 4) or does not apply at all (M > 4 would
    // fall to the multi-pass scalar kernel), and any batch wider than four rows when the caller
    // asks for fp32 dequantization (MIORI_GEMV_EXACT), and long streams of 4-bit weights in groups
    // of 64 (four 128-row tiles per SM and more, up to four activation rows), where it runs two
    // CTAs per SM and measured 14-17 % faster (at group 32 it drains twice the accumulator columns
    // and measured 7-30 % slower, so those stay on the mma.sync kernel).  Elsewhere the mma.sync kernel with its shorter
    // pipeline measured faster and stays the default; MIORI_TUNE_GEMV_UMMA forces this one.
    const bool long_stream4 = BITS == 4 && M <= 4 && group == 64 && (N + 127u) / 128u >= 4u * (uint32_t)sm_count();
    const bool umma_default = (BITS == 8 && M >= 3) || (force_exact && M > 4) || long_stream4;
    if (!force_simt && !no_bulk && !(flags & MIORI_TUNE_GEMV_MMASYNC) &&
        (umma_default || (flags & MIORI_TUNE_GEMV_UMMA))) {
        rc = gemvumma::try_launch<BITS>(q, s, b, x, y, N, K, M, group, flags, (cudaStream_t)stream);
        if (rc <= 0) return rc;  // launched (0) or failed (<0); 1 = not eligible
    }
    if (!force_simt && !(force_exact && M > 4)) {
        if (!no_bulk) {
            rc = gemvtma::try_launch<BITS>(q, s, b, x, y, N, K, M, group, flags, (cudaStream_t)stream);
            if (rc <= 0) return rc;  // launched (0) or failed (<0); 1 = not eligible
        }
        if (gemvmma::supported<BITS>(K, M, force_exact))
            return gemvmma::launch<BITS>(q, s, b, x, y, N, K, M, group, flags, (cudaStream_t)stream);
    }
    if ((size_t)K * 2 * 4 > 200 * 1024)
        return fail(MIORI_E_INVALID, "%s: K=%u too large for the activation staging", op, K);
    return launch_gemv_simt<BITS>(q, s, b, x, y, N, K, M, group, flags, (cudaStream_t)stream);
}

}  // namespace

MIORI_API int miori_gemv4(const void* q, const void* s, const void* b, const void* x, void* y,
                          uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
                          void* stream) {
    return gemv_entry<4>("miori_gemv4", q, s, b, x, y, N, K, M, group, flags, stream);
}

MIORI_API int miori_gemv8(const void* q, const void* s, const void* b, const void* x, void* y,
                          uint32_t N, uint32_t K, uint32_t M, uint32_t group, uint32_t flags,
                          void* stream) {
    return gemv_entry<8>("miori_gemv8", q, s, b, x, y, N, K, M, group, flags, stream);
}

namespace {
template <int BITS>
int gemv_rmsnorm_entry(const char* op, const void* q, const void* s, const void* b, const void* x,
                       const void* gamma, float eps, void* y, uint32_t N, uint32_t K, uint32_t M,
                       uint32_t group, uint32_t flags, void* stream) {
    int rc = check_quant_args(op, q, s, b, N, K, group);
    if (rc) return rc;
    if (!x || !y || !gamma) return fail(MIORI_E_INVALID, "%s: null activation, weight or output pointer", op);
    if (M == 0 || M > 32) return fail(MIORI_E_INVALID, "%s: M=%u outside 1..32", op, M);
    if (!aligned16(x) || !aligned16(gamma)) return fail(MIORI_E_INVALID, "%s: x and gamma must be 16-byte aligned", op);
    // 4-bit weights, up to four rows, fp32 out, K within one slab: the TMA + mma.sync kernel with the norm
    // in its staging pass (1.2-1.6 us faster than the pair of kernels; the tcgen05 kernel is slower than
    // the pair there).  Longer rows and long streams go to the tcgen05 kernel (8192 -> 2048: 8.3 us
    // against 10.3); the private flags force either.
    if constexpr (BITS == 4) {
        const bool long_stream = group == 64 && (N + 127u) / 128u >= 4u * (uint32_t)sm_count();
        if (M <= 4 && !(flags & (MIORI_OUT_BF16 | MIORI_TUNE_GEMV_UMMA)) &&
            ((!long_stream && K <= 2048u) || (flags & MIORI_TUNE_GEMV_MMASYNC))) {
            gemvtma::Shard sh;
            sh.pre.gamma = static_cast<const uint16_t*>(gamma);
            sh.pre.eps = eps;
            rc = gemvtma::try_launch<4>(q, s, b, x, y, N, K, M, group, flags, (cudaStream_t)stream, sh);
            if (rc <= 0) return rc;  // launched (0) or failed (<0); 1 = not eligible: the tcgen05 kernel may be
        }
    }
    gemvumma::Placement pl;
    pl.gamma = gamma;
    pl.eps = eps;
    rc = gemvumma::try_launch<BITS>(q, s, b, x, y, N, K, M, group, flags, (cudaStream_t)stream, pl);
    if (rc == 1)
        return fail(MIORI_E_INVALID, "%s: shape N=%u K=%u M=%u group=%u is outside the fused kernel's range "
                    "(run miori_rmsnorm and the plain GEMV instead)", op, N, K, M, group);
    return rc;
}
}  // namespace

MIORI_API int miori_gemv4_silu(const void* q, const void* s, const void* b, const void* x, void* y, uint32_t N,
                               uint32_t K, uint32_t M, uint32_t group, uint32_t flags, void* stream) {
    const char* op = "miori_gemv4_silu";
    int rc = check_quant_args(op, q, s, b, N, K, group);
    if (rc) return rc;
    if (!x || !y) return fail(MIORI_E_INVALID, "%s: null activation pointer", op);
    // 17..32 staged rows do not fit the kernel's shared memory at any K
    if (M == 0 || M > 16) return fail(MIORI_E_INVALID, "%s: M=%u outside 1..16", op, M);
    if (!aligned16(x)) return fail(MIORI_E_INVALID, "%s: x must be 16-byte aligned", op);
    if (N % 16 != 0)
        return fail(MIORI_E_INVALID, "%s: N=%u (gate rows then up rows) must be a multiple of 16", op, N);
    gemvtma::Shard sh;
    sh.gated = true;
    rc = gemvtma::try_launch<4>(q, s, b, x, y, N, K, M, group, flags | MIORI_OUT_BF16, (cudaStream_t)stream, sh);
    if (rc == 1)
        return fail(MIORI_E_INVALID, "%s: shape N=%u K=%u M=%u group=%u is outside the fused kernel's range "
                    "(run the plain GEMV and miori_silu_mul instead)", op, N, K, M, group);
    return rc;
}

MIORI_API int miori_gemv4_rmsnorm_silu(const void* q, const void* s, const void* b, const void* x,
                                       const void* gamma, float eps, void* y, uint32_t N, uint32_t K, uint32_t M,
                                       uint32_t group, uint32_t flags, void* stream) {
    const char* op = "miori_gemv4_rmsnorm_silu";
    int rc = check_quant_args(op, q, s, b, N, K, group);
    if (rc) return rc;
    if (!x || !y || !gamma) return fail(MIORI_E_INVALID, "%s: null activation, weight or output pointer", op);
    if (M == 0 || M > 4) return fail(MIORI_E_INVALID, "%s: M=%u outside 1..4", op, M);
    if (!aligned16(x) || !aligned16(gamma)) return fail(MIORI_E_INVALID, "%s: x and gamma must be 16-byte aligned", op);
    if (N % 16 != 0)
        return fail(MIORI_E_INVALID, "%s: N=%u (gate rows then up rows) must be a multiple of 16", op, N);
    gemvtma::Shard sh;
    sh.gated = true;
    sh.pre.gamma = static_cast<const uint16_t*>(gamma);
    sh.pre.eps = eps;
    rc = gemvtma::try_launch<4>(q, s, b, x, y, N, K, M, group, flags | MIORI_OUT_BF16, (cudaStream_t)stream, sh);
    if (rc == 1)
        return fail(MIORI_E_INVALID, "%s: shape N=%u K=%u M=%u group=%u is outside the fused kernel's range "
                    "(run miori_rmsnorm and miori_gemv4_silu instead)", op, N, K, M, group);
    return rc;
}

MIORI_API int miori_gemv4_post_norm_add(const void* q, const void* s, const void* b, const void* x,
                                        const void* residual, const void* gamma, float eps, void* counter,
                                        void* out, uint32_t N, uint32_t K, uint32_t M, uint32_t group,
                                        uint32_t flags, void* stream) {
    const char* op = "miori_gemv4_post_norm_add";
    int rc = check_quant_args(op, q, s, b, N, K, group);
    if (rc) return rc;
    if (!x || !residual || !gamma || !counter || !out) return fail(MIORI_E_INVALID, "%s: null pointer", op);
    if (M == 0 || M > 4) return fail(MIORI_E_INVALID, "%s: M=%u outside 1..4", op, M);
    if (!aligned16(x)) return fail(MIORI_E_INVALID, "%s: x must be 16-byte aligned", op);
    if (flags & MIORI_OUT_BF16) return fail(MIORI_E_INVALID, "%s: the output is fp32", op);
    if (out == residual) return fail(MIORI_E_INVALID, "%s: out must not be the residual", op);
    gemvtma::Shard sh;
    sh.post.residual = static_cast<const float*>(residual);
    sh.post.gamma = static_cast<const uint16_t*>(gamma);
    sh.post.arrivals = static_cast<unsigned int*>(counter);
    sh.post.eps = eps;
    rc = gemvtma::try_launch<4>(q, s, b, x, out, N, K, M, group, flags, (cudaStream_t)stream, sh);
    if (rc == 1)
        return fail(MIORI_E_INVALID, "%s: shape N=%u K=%u M=%u group=%u is outside the fused kernel's range "
                    "(run the plain GEMV and miori_post_norm_add instead)", op, N, K, M, group);
    return rc;
}

MIORI_API int miori_gemv4_rmsnorm(const void* q, const void* s, const void* b, const void* x, const void* gamma,
                                  float eps, void* y, uint32_t N, uint32_t K, uint32_t M, uint32_t group,
                                  uint32_t flags, void* stream) {
    return gemv_rmsnorm_entry<4>("miori_gemv4_rmsnorm", q, s, b, x, gamma, eps, y, N, K, M, group, flags, stream);
}
MIORI_API int miori_gemv8_rmsnorm(const void* q, const void* s, const void* b, const void* x, const void* gamma,
                                  float eps, void* y, uint32_t N, uint32_t K, uint32_t M, uint32_t group,
                                  uint32_t flags, void* stream) {
    return gemv_rmsnorm_entry<8>("miori_gemv8_rmsnorm", q, s, b, x, gamma, eps, y, N, K, M, group, flags, stream);
}

MIORI_API int miori_gemv_bf16_cache(const void* x, const void* cache, void* y, uint32_t M, uint32_t N, uint32_t K,
                                    uint32_t flags, void* stream) {
    const char* op = "miori_gemv_bf16_cache";
    if (!x || !cache || !y) return fail(MIORI_E_INVALID, "%s: null pointer", op);
    if (M == 0 || M > 32) return fail(MIORI_E_INVALID, "%s: M=%u outside 1..32", op, M);
    if (N == 0 || K == 0 || K % 8 != 0)
        return fail(MIORI_E_INVALID, "%s: N=%u K=%u (K must be a positive multiple of 8)", op, N, K);
    if (!aligned16(x) || !aligned16(cache) || !aligned16(y))
        return fail(MIORI_E_INVALID, "%s: x, cache and y must be 16-byte aligned", op);
    const int rc = gemvcache::try_launch(x, cache, y, M, N, K, flags, (cudaStream_t)stream);
    if (rc == 1)
        return fail(MIORI_E_INVALID, "%s: K=%u is beyond the kernel's 8192 (use miori_gemm_bf16_cache)", op, K);
    return rc;
}

// Where miori_linear4 sends a projection: 0 = packed-weight GEMV, 1 = narrow-batch kernel on the
// bf16 cache, 2 = tcgen05 GEMM on the bf16 cache.  Measured on B200 in chains of dependent
// launches (us per launch, 2048 -> 3072 / 2048 -> 2048 / 8192 -> 2048 / 2048 -> 16384):
//   M = 8:  packed 4.4 / 3.9 / 8.9 / 10.5, narrow 4.1 / 3.2 / 7.6 / 11.8
//   M = 16: packed 5.3 / 4.7 / 82 / 12.6,  narrow 4.4 / 3.3 / 9.2 / 12.1,  GEMM 8.9 / 7.6 / 12.6 / 15.9
//   M = 32: packed 10.8 / 7.1 / 162 / 32,  narrow 5.6 / 4.4 / 14.6 / 17.4, GEMM 8.6 / 7.8 / 12.8 / 16.0
// Up to four rows stay on the packed weights with fp32 dequantization, as in the reference
// (src/batch.cpp:223-230 cuts over to the cache above four rows).  Above that the cache is used
// when given: by the narrow-batch kernel while the projection is short (at most two 16-row tiles
// per SM: its launch is cheap, but it streams four times the bytes and its mma.sync rate caps it
// on long streams) and for 9..16 rows of any width, else by the packed GEMV up to 8 rows, else by
// the tensor-core GEMM.
static int linear4_route(uint32_t M, uint32_t N, uint32_t K, bool has_cache) {
    if (M <= 4 || !has_cache) return 0;
    const uint32_t tiles = (N + 15u) / 16u, slabs = (K + 511u) / 512u;
    const uint32_t nt = M <= 8 ? 1u : M <= 16 ? 2u : 4u;
    const uint32_t frags = (slabs <= 1 ? 1u : slabs <= 2 ? 2u : slabs <= 4 ? 4u : slabs <= 8 ? 8u : 16u) * nt;
    const bool short_proj = tiles <= 2u * (uint32_t)sm_count();
    if (slabs <= 16u && K % 8 == 0) {
        // activations resident in registers: short projections, and 9..16 rows of any width
        if (frags <= (uint32_t)gemvcache::MAX_FRAGS && (short_proj || nt == 2u)) return 1;
        // activations streamed per tile (long rows): pays up to 16 rows on short projections
        // (8192 -> 2048 at 16 rows: 9.2 us against 12.6 us for the GEMM; at 32 rows 14.6 against 12.8)
        if (frags > (uint32_t)gemvcache::MAX_FRAGS && short_proj && nt == 2u) return 1;
    }
    if (M <= 8) return 0;
    return 2;
}

MIORI_API int miori_linear4_route(uint32_t M, uint32_t N, uint32_t K, int has_cache) {
    return linear4_route(M, N, K, has_cache != 0);
}

MIORI_API int miori_linear4(const void* q, const void* s, const void* b, const void* cache,
                            const void* x, void* y, uint32_t N, uint32_t K, uint32_t M,
                            uint32_t group, uint32_t flags, void* workspace, size_t workspace_bytes,
                            void* stream) {
    switch (linear4_route(M, N, K, cache != nullptr)) {
    case 1:
        return miori_gemv_bf16_cache(x, cache, y, M, N, K, flags, stream);
    case 2:
        return miori_gemm_bf16_cache_ws(x, cache, y, M, N, K, flags, workspace, workspace_bytes, stream);
    default:
        return miori_gemv4(q, s, b, x, y, N, K, M, group, flags, stream);
    }
}

MIORI_API int miori_dequant4_rowmajor(const void* q, const void* s, const void* b, void* out,
                                      uint32_t N, uint32_t K, uint32_t group, void* stream) {
    int rc = check_quant_args("miori_dequant4_rowmajor", q, s, b, N, K, group);
    if (rc) return rc;
    if (!out || !aligned16(out))
        return fail(MIORI_E_INVALID, "miori_dequant4_rowmajor: out null or not 16-byte aligned");
    return launch_dequant_rowmajor<4>(q, s, b, out, N, K, group, (cudaStream_t)stream);
}

MIORI_API int miori_dequant8_rowmajor(const void* q, const void* s, const void* b, void* out,
                                      uint32_t N, uint32_t K, uint32_t group, void* stream) {
    int rc = check_quant_args("miori_dequant8_rowmajor", q, s, b, N, K, group);
    if (rc) return rc;
    if (!out || !aligned16(out))
        return fail(MIORI_E_INVALID, "miori_dequant8_rowmajor: out null or not 16-byte aligned");
    return launch_dequant_rowmajor<8>(q, s, b, out, N, K, group, (cudaStream_t)stream);
}

// The GEMM reads B through TMA as a K-major [N][K] bf16 matrix, so the cache is simply the
// row-major dequantized tensor; the accessors keep the layout private to this library.
MIORI_API size_t miori_cache_bytes(uint32_t N, uint32_t K) { return (size_t)N * K * 2; }

MIORI_API int miori_dequant4_cache(const void* q, const void* s, const void* b, void* cache,
                                   uint32_t N, uint32_t K, uint32_t group, void* stream) {
    int rc = check_quant_args("miori_dequant4_cache", q, s, b, N, K, group);
    if (rc) return rc;
    if (!cache || !aligned16(cache))
        return fail(MIORI_E_INVALID, "miori_dequant4_cache: cache null or not 16-byte aligned");
    return launch_dequant_rowmajor<4>(q, s, b, cache, N, K, group, (cudaStream_t)stream);
}

MIORI_API int miori_cache_to_rowmajor(const void* cache, void* out, uint32_t N, uint32_t K,
                                      void* stream) {
    if (!cache || !out) return fail(MIORI_E_INVALID, "miori_cache_to_rowmajor: null pointer");
    MIORI_CUDA(cudaMemcpyAsync(out, cache, (size_t)N * K * 2, cudaMemcpyDeviceToDevice,
                               (cudaStream_t)stream));
    return MIORI_OK;
}

MIORI_API int miori_device_error_poll(void) {
    unsigned int rec[4] = {0, 0, 0, 0};
    if (cudaMemcpyFromSymbol(rec, g_device_error, sizeof(rec)) != cudaSuccess) return 0;
    if (rec[0] == 0) return 0;
    const unsigned int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_device_error, zero, sizeof(zero));
    fail(MIORI_E_DEVICE, "kernel reported %u internal error(s); first code=%u detail=%u,%u", rec[0],
         rec[1], rec[2], rec[3]);
    return (int)rec[0];
}

#ifdef MIORI_TMA_TRACE
// Profiling build only: read and reset the TMA GEMV's %globaltimer marks.
MIORI_API int miori_debug_tma_marks(unsigned long long* out4096) {
    if (cudaMemcpyFromSymbol(out4096, gemvtma::g_tma_marks, 4096 * sizeof(unsigned long long)) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(out4096 + 4096, gemvtma::g_tma_pmarks, 2048 * sizeof(unsigned long long)) != cudaSuccess) return -1;
    const unsigned int zero[4] = {0, 0, 0, 0};
    return cudaMemcpyToSymbol(gemvtma::g_tma_launch, zero, sizeof(zero)) == cudaSuccess ? 0 : -1;
}
#endif
#ifdef MIORI_UMMA_TRACE
// Profiling build only: read and clear the tcgen05 GEMV's cycle counters.
MIORI_API int miori_debug_umma_trace(long long* out32) {
    long long zero[32] = {};
    if (cudaMemcpyFromSymbol(out32, gemvumma::g_umma_trace, sizeof(zero)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(gemvumma::g_umma_trace, zero, sizeof(zero));
    return 0;
}
MIORI_API int miori_debug_umma_events(unsigned int* out1024) {
    return cudaMemcpyFromSymbol(out1024, gemvumma::g_umma_ev, 1024 * sizeof(unsigned int)) == cudaSuccess ? 0 : -1;
}
#endif
