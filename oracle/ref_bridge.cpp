// Bridge that compiles the reference's own CPU checker (src/cpu_ref.h, included
// from where the reference lies, never copied) into oracle/_ref/libmiori_cpuref.so.
// TEST INFRASTRUCTURE: used to validate oracle/miori_oracle.c and, at group 32, as
// the timed CPU baseline.  The loops around dequant{4,8}_elem follow the reference's
// test procedure in src/main.cpp:67-86 (double-precision dot with bf16-rounded x).
#include "cpu_ref.h"

#include <cstddef>
#include <cstdint>
#include <algorithm>
#include <thread>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
int g_threads = 0;
int threads() {
    if (g_threads > 0) return g_threads;
    const unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}
template <class F>
void parallel_rows(int64_t lo, int64_t hi, F body) {
    const int T = (int)std::max<int64_t>(1, std::min<int64_t>(threads(), hi - lo));
    if (T == 1) { body(lo, hi); return; }
    std::vector<std::thread> th;
    const int64_t span = hi - lo;
    for (int i = 0; i < T; ++i)
        th.emplace_back(body, lo + span * i / T, lo + span * (i + 1) / T);
    for (auto& t : th) t.join();
}
miori::Tensor make_tensor(const void* p, int64_t rows, int64_t cols, size_t elem) {
    miori::Tensor t;
    t.shape = {rows, cols};
    t.ptr = static_cast<const uint8_t*>(p);
    t.begin = 0;
    t.end = static_cast<uint64_t>(rows) * static_cast<uint64_t>(cols) * elem;
    return t;
}
}  // namespace

REF_API float ref_bf16_to_float(uint16_t v) { return miori::bf16_to_float(v); }
REF_API uint16_t ref_float_to_bf16(float f) { return miori::float_to_bf16(f); }

REF_API float ref_dequant_elem(int bits, const uint32_t* q, const uint16_t* s, const uint16_t* b,
                               int64_t N, int64_t n, int64_t k, int64_t K) {
    const int per = 32 / bits;
    miori::Tensor tq = make_tensor(q, N, K / per, 4);
    miori::Tensor ts = make_tensor(s, N, K / 32, 2);
    miori::Tensor tb = make_tensor(b, N, K / 32, 2);
    return bits == 8 ? miori::dequant8_elem(tq, ts, tb, n, k, K)
                     : miori::dequant4_elem(tq, ts, tb, n, k, K);
}

// y[m][n] = sum_k dequant_elem(n,k) * bf16(x[m][k]) in double, rows n0..n1-1.
REF_API void ref_gemv(int bits, const uint32_t* q, const uint16_t* s, const uint16_t* b,
                      const uint16_t* x, double* y, int64_t N, int64_t K, int64_t M, int64_t n0,
                      int64_t n1) {
    const int per = 32 / bits;
    const miori::Tensor tq = make_tensor(q, N, K / per, 4);
    const miori::Tensor ts = make_tensor(s, N, K / 32, 2);
    const miori::Tensor tb = make_tensor(b, N, K / 32, 2);
    parallel_rows(n0, n1, [&](int64_t lo, int64_t hi) {
    for (int64_t n = lo; n < hi; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            double ref = 0.0;
            for (int64_t k = 0; k < K; ++k) {
                const float wv = bits == 8 ? miori::dequant8_elem(tq, ts, tb, n, k, K)
                                           : miori::dequant4_elem(tq, ts, tb, n, k, K);
                ref += (double)wv * (double)miori::bf16_to_float(x[(uint64_t)m * K + k]);
            }
            y[(uint64_t)m * N + n] = ref;
        }
    }
    });
}

// out[n][k] = float_to_bf16(dequant_elem(n,k)), row-major.
REF_API void ref_dequant_rowmajor(int bits, const uint32_t* q, const uint16_t* s,
                                  const uint16_t* b, uint16_t* out, int64_t N, int64_t K) {
    const int per = 32 / bits;
    const miori::Tensor tq = make_tensor(q, N, K / per, 4);
    const miori::Tensor ts = make_tensor(s, N, K / 32, 2);
    const miori::Tensor tb = make_tensor(b, N, K / 32, 2);
    parallel_rows(0, N, [&](int64_t lo, int64_t hi) {
    for (int64_t n = lo; n < hi; ++n)
        for (int64_t k = 0; k < K; ++k) {
            const float wv = bits == 8 ? miori::dequant8_elem(tq, ts, tb, n, k, K)
                                       : miori::dequant4_elem(tq, ts, tb, n, k, K);
            out[(uint64_t)n * K + k] = miori::float_to_bf16(wv);
        }
    });
}

REF_API int ref_num_threads(void) { return threads(); }
REF_API void ref_set_threads(int n) { g_threads = n > 0 ? n : 0; }
