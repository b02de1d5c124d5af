/*
 * CPU oracle for the quantized-matmul path (TEST INFRASTRUCTURE, not product code).
 *
 * A plain-C restatement of the reference's CPU checker and of the arithmetic its
 * Metal kernels define.  Only the tests, the smoke check and the CPU-baseline leg
 * of the benchmark may load this library; the CUDA library never does.
 *
 * Parity status: pinned.  The reference ships no golden vectors for this path, so
 * the pin is (a) hand-computed known answers (word 0x76543210, s=0.5, b=-1) and
 * (b) equality with the reference's own src/cpu_ref.h compiled unmodified into
 * oracle/_ref (see ref_bridge.cpp), exercised by tests/test_oracle.py and frozen
 * in tests/golden/.
 *
 * Every function names the reference lines it follows (paths inside the reference
 * project).  The group size is a parameter: 32 is what the reference hard-codes
 * (config/m6.h:48, src/cpu_ref.h:30-32); 64 is the same formula with the constant
 * changed.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define MO_API __attribute__((visibility("default")))

/* ---- minimal static-chunk parallel-for over pthreads (no OpenMP runtime needed) ---- */
static int g_threads = 0;
typedef void (*mo_body_fn)(int64_t lo, int64_t hi, void* ctx);
typedef struct { mo_body_fn fn; void* ctx; int64_t lo, hi; } mo_task;
static void* mo_trampoline(void* p) {
    mo_task* t = (mo_task*)p;
    t->fn(t->lo, t->hi, t->ctx);
    return NULL;
}
static int mo_threads(void) {
    if (g_threads > 0) return g_threads;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (n > 256 ? 256 : (int)n);
}
static void mo_parallel_for(int64_t lo, int64_t hi, mo_body_fn fn, void* ctx) {
    int T = mo_threads();
    if (hi - lo < T) T = (int)(hi - lo > 0 ? hi - lo : 1);
    if (T <= 1) { fn(lo, hi, ctx); return; }
    pthread_t th[256];
    mo_task tk[256];
    const int64_t span = hi - lo;
    for (int i = 0; i < T; ++i) {
        tk[i].fn = fn; tk[i].ctx = ctx;
        tk[i].lo = lo + span * i / T;
        tk[i].hi = lo + span * (i + 1) / T;
        if (pthread_create(&th[i], NULL, mo_trampoline, &tk[i]) != 0) {
            /* could not spawn: run this chunk inline */
            th[i] = 0;
            fn(tk[i].lo, tk[i].hi, ctx);
        }
    }
    for (int i = 0; i < T; ++i)
        if (th[i]) pthread_join(th[i], NULL);
}

/* src/cpu_ref.h:9-14 -- widen bf16 to fp32 by placing it in the high half. */
static inline float bf16_to_float(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* src/cpu_ref.h:16-23 -- round-to-nearest-even, no NaN/Inf special case. */
static inline uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

MO_API float mo_bf16_to_float(uint16_t v) { return bf16_to_float(v); }
MO_API uint16_t mo_float_to_bf16(float f) { return float_to_bf16(f); }

MO_API void mo_bf16_to_float_n(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = bf16_to_float(in[i]);
}
MO_API void mo_float_to_bf16_n(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = float_to_bf16(in[i]);
}

/*
 * src/cpu_ref.h:25-34 (4-bit) and :36-45 (8-bit): one dequantized weight.
 * q is [N][K*bits/32] uint32, low nibble / low byte first; s and b are
 * [N][K/group] bf16.  Result is float(q)*scale + bias evaluated in fp32 as a
 * separate multiply and add (build with -ffp-contract=off).
 */
static inline float dequant_elem(int bits, const uint32_t* q, const uint16_t* s,
                                 const uint16_t* b, int64_t n, int64_t k, int64_t K,
                                 int64_t group) {
    const int per = 32 / bits;
    const uint32_t* qrow = q + (uint64_t)n * (uint64_t)(K / per);
    const uint32_t word = qrow[k / per];
    const uint32_t qv = (word >> (bits * (k % per))) & ((1u << bits) - 1u);
    const int64_t g = k / group;
    const float sc = bf16_to_float(s[(uint64_t)n * (K / group) + g]);
    const float bi = bf16_to_float(b[(uint64_t)n * (K / group) + g]);
    return (float)qv * sc + bi;
}

MO_API float mo_dequant_elem(int bits, const uint32_t* q, const uint16_t* s, const uint16_t* b,
                             int64_t n, int64_t k, int64_t K, int64_t group) {
    return dequant_elem(bits, q, s, b, n, k, K, group);
}

/*
 * GEMV reference as the reference's own test computes it, src/main.cpp:67-86:
 * a double-precision dot of dequant{4,8}_elem with the bf16-rounded activations.
 * x is [M][K] bf16 and y is [M][N] double (M=1 is the reference's test; rows are
 * independent, shaders/batch.metal:142-144).  Rows n0..n1-1 only.
 */
typedef struct {
    int bits;
    const uint32_t* q; const uint16_t* s; const uint16_t* b; const uint16_t* x;
    double* y; int64_t N, K, M, group;
} gemv_ctx;
static void gemv_body(int64_t lo, int64_t hi, void* p) {
    const gemv_ctx* c = (const gemv_ctx*)p;
    for (int64_t n = lo; n < hi; ++n) {
        for (int64_t m = 0; m < c->M; ++m) {
            double ref = 0.0;
            const uint16_t* xr = c->x + (uint64_t)m * c->K;
            for (int64_t k = 0; k < c->K; ++k) {
                const float wv = dequant_elem(c->bits, c->q, c->s, c->b, n, k, c->K, c->group);
                ref += (double)wv * (double)bf16_to_float(xr[k]);
            }
            c->y[(uint64_t)m * c->N + n] = ref;
        }
    }
}
MO_API void mo_gemv(int bits, const uint32_t* q, const uint16_t* s, const uint16_t* b,
                    const uint16_t* x, double* y, int64_t N, int64_t K, int64_t M,
                    int64_t group, int64_t n0, int64_t n1) {
    gemv_ctx c = {bits, q, s, b, x, y, N, K, M, group};
    mo_parallel_for(n0, n1, gemv_body, &c);
}

/*
 * bf16 weight cache.  Row-major: shaders/ops.metal:142-166 (dequant4) and :754-779
 * (dequant8): out[n][k] = bf16(float(q)*scale + bias), RNE.  Tile-major (tile=1):
 * the reference's [N/64][K][64] layout, shaders/gemm_mpp.metal:9-34, where element
 * (n,k) lives at tile n/64, row k, column n%64; same value per element (:31-32).
 */
typedef struct {
    int bits, tile;
    const uint32_t* q; const uint16_t* s; const uint16_t* b; uint16_t* out;
    int64_t N, K, group;
} deq_ctx;
static void deq_body(int64_t lo, int64_t hi, void* p) {
    const deq_ctx* c = (const deq_ctx*)p;
    for (int64_t n = lo; n < hi; ++n)
        for (int64_t k = 0; k < c->K; ++k) {
            const uint16_t v =
                float_to_bf16(dequant_elem(c->bits, c->q, c->s, c->b, n, k, c->K, c->group));
            if (c->tile)
                c->out[(uint64_t)(n / 64) * c->K * 64 + (uint64_t)k * 64 + (n % 64)] = v;
            else
                c->out[(uint64_t)n * c->K + k] = v;
        }
}
MO_API void mo_dequant_rowmajor(int bits, const uint32_t* q, const uint16_t* s,
                                const uint16_t* b, uint16_t* out, int64_t N, int64_t K,
                                int64_t group) {
    deq_ctx c = {bits, 0, q, s, b, out, N, K, group};
    mo_parallel_for(0, N, deq_body, &c);
}
MO_API void mo_dequant_tile(const uint32_t* q, const uint16_t* s, const uint16_t* b,
                            uint16_t* out, int64_t N, int64_t K, int64_t group) {
    deq_ctx c = {4, 1, q, s, b, out, N, K, group};
    mo_parallel_for(0, N, deq_body, &c);
}

/*
 * GEMM semantics, shaders/gemm_mpp.metal:36-54 with src/ops.cpp:341:
 * C[M][N] = A[M][K] (bf16, row-major, lda=K) x B^T, B being the bf16 cache.
 * The reference delegates the arithmetic to a closed library, so this is the
 * exact product accumulated in double over the row-major cache Bc[N][K].
 * Only rows m0..m1-1 are produced.
 */
static inline double dot_bf16(const uint16_t* a, const uint16_t* w, int64_t K) {
    double acc = 0.0;
    for (int64_t k = 0; k < K; ++k)
        acc += (double)bf16_to_float(a[k]) * (double)bf16_to_float(w[k]);
    return acc;
}
typedef struct {
    const uint16_t* A; const uint16_t* Bc; double* C; int64_t N, K, m0;
} gemm_ctx;
static void gemm_body(int64_t lo, int64_t hi, void* p) {
    const gemm_ctx* c = (const gemm_ctx*)p;
    for (int64_t i = lo; i < hi; ++i) {
        const int64_t m = c->m0 + i / c->N, n = i % c->N;
        c->C[(uint64_t)m * c->N + n] =
            dot_bf16(c->A + (uint64_t)m * c->K, c->Bc + (uint64_t)n * c->K, c->K);
    }
}
MO_API void mo_gemm_bf16(const uint16_t* A, const uint16_t* Bc, double* C, int64_t M,
                         int64_t N, int64_t K, int64_t m0, int64_t m1) {
    (void)M;
    gemm_ctx c = {A, Bc, C, N, K, m0};
    mo_parallel_for(0, (m1 - m0) * N, gemm_body, &c);
}

/* One sampled GEMM entry (used to spot-check full-size products). */
MO_API double mo_gemm_bf16_entry(const uint16_t* A, const uint16_t* Bc, int64_t K, int64_t m,
                                 int64_t n) {
    return dot_bf16(A + (uint64_t)m * K, Bc + (uint64_t)n * K, K);
}

/*
 * Input generator (NOT part of the reference, which only consumes pre-quantized
 * safetensors, src/weights.cpp:48-62): MLX-style affine quantization of fp32
 * weights along K.  scale=(max-min)/qmax and bias=min are stored as bf16 (RNE);
 * q=round((w-bias)/scale) clamped to [0,qmax] is computed against the stored
 * values.  A constant group gets scale 1, q 0.
 */
typedef struct {
    int bits; const float* W; uint32_t* q; uint16_t* s; uint16_t* b; int64_t K, group;
} quant_ctx;
static void quant_body(int64_t lo, int64_t hi, void* p) {
    const quant_ctx* c = (const quant_ctx*)p;
    const int bits = c->bits, per = 32 / bits;
    const float qmax = (float)((1 << bits) - 1);
    const int64_t K = c->K, group = c->group, ng = K / group;
    for (int64_t n = lo; n < hi; ++n) {
        memset(c->q + (uint64_t)n * (K / per), 0, (size_t)(K / per) * 4);
        for (int64_t g = 0; g < ng; ++g) {
            const float* w = c->W + (uint64_t)n * K + g * group;
            float mn = w[0], mx = w[0];
            for (int64_t j = 1; j < group; ++j) {
                mn = w[j] < mn ? w[j] : mn;
                mx = w[j] > mx ? w[j] : mx;
            }
            float sc = (mx - mn) / qmax;
            if (!(sc > 0.0f)) sc = 1.0f;
            const uint16_t sb = float_to_bf16(sc), bb = float_to_bf16(mn);
            c->s[(uint64_t)n * ng + g] = sb;
            c->b[(uint64_t)n * ng + g] = bb;
            const float scr = bf16_to_float(sb), bir = bf16_to_float(bb);
            for (int64_t j = 0; j < group; ++j) {
                float v = nearbyintf((w[j] - bir) / scr);
                v = v < 0.0f ? 0.0f : (v > qmax ? qmax : v);
                const int64_t k = g * group + j;
                c->q[(uint64_t)n * (K / per) + k / per] |= ((uint32_t)v) << (bits * (k % per));
            }
        }
    }
}
MO_API void mo_quantize(int bits, const float* W, uint32_t* q, uint16_t* s, uint16_t* b,
                        int64_t N, int64_t K, int64_t group) {
    quant_ctx c = {bits, W, q, s, b, K, group};
    mo_parallel_for(0, N, quant_body, &c);
}

/*
 * The steps either side of a projection, restated from the reference's shaders in plain
 * fp32 as they compute them (sums of squares in double, so that the checker does not depend
 * on a reduction order).
 *   rmsnorm        shaders/ops.metal:86-115   y = bf16(x * rsqrt(mean(x^2) + eps) * w)
 *   silu_mul       shaders/ops.metal:129-139  out = bf16(g / (1 + exp(-g)) * up)
 *   post_norm_add  shaders/ops.metal:605-631  out = x + src * rsqrt(mean(src^2) + eps) * w
 *   embed8         shaders/ops.metal:170-197  out[t][k] = bf16(code * scale + bias) of row tokens[t]
 */
MO_API void mo_rmsnorm(const float* x, const uint16_t* w, uint16_t* y, int64_t rows, int64_t n,
                       float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (int64_t i = 0; i < n; ++i) ss += (double)x[r * n + i] * (double)x[r * n + i];
        const float inv = 1.0f / sqrtf((float)(ss / (double)n) + eps);
        for (int64_t i = 0; i < n; ++i)
            y[r * n + i] = float_to_bf16(x[r * n + i] * inv * bf16_to_float(w[i]));
    }
}
MO_API void mo_silu_mul(const float* gate, const float* up, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const float g = gate[i];
        const float s = g / (1.0f + expf(-g));
        out[i] = float_to_bf16(s * up[i]);
    }
}
MO_API void mo_post_norm_add(const float* x, const float* src, const uint16_t* w, float* out,
                             int64_t rows, int64_t n, float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (int64_t i = 0; i < n; ++i) ss += (double)src[r * n + i] * (double)src[r * n + i];
        const float inv = 1.0f / sqrtf((float)(ss / (double)n) + eps);
        for (int64_t i = 0; i < n; ++i)
            out[r * n + i] = x[r * n + i] + src[r * n + i] * inv * bf16_to_float(w[i]);
    }
}
MO_API void mo_embed8(const uint32_t* q, const uint16_t* s, const uint16_t* b, const uint32_t* tokens,
                      uint16_t* out, int64_t T, int64_t K, int64_t group) {
    for (int64_t t = 0; t < T; ++t)
        for (int64_t k = 0; k < K; ++k)
            out[t * K + k] = float_to_bf16(dequant_elem(8, q, s, b, (int64_t)tokens[t], k, K, group));
}

MO_API int mo_num_threads(void) { return mo_threads(); }
MO_API void mo_set_threads(int n) { g_threads = n > 0 ? (n > 256 ? 256 : n) : 0; }
