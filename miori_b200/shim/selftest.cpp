// C entry points that drive the operator shim the way the reference's own test commands do
// (reference src/main.cpp:44-87 test-gemv4/8, :1403-1443 test-mpp-tile), for the Python
// tests: host arrays in, host arrays out, everything in between through miori::Metal,
// miori::Weights and the miori:: operators.
#include "ops.h"

#include <cstring>
#include <exception>
#include <initializer_list>
#include <stdexcept>
#include <string>

namespace {
thread_local std::string g_err;
}

extern "C" __attribute__((visibility("default"))) const char* miori_shim_last_error() {
    return g_err.c_str();
}

// y[B][N] = gemv{4,8}[_b](W, x[B][K]) with group-32 weights given as host arrays.
extern "C" __attribute__((visibility("default"))) int miori_shim_test_gemv(
    int bits, const uint32_t* q, const uint16_t* s, const uint16_t* b, const uint16_t* x, float* y,
    uint32_t N, uint32_t K, uint32_t B) {
    using namespace miori;
    try {
        Metal m;
        std::string err;
        if (!m.init("", err)) throw std::runtime_error(err);
        Weights w;
        const size_t qb = (size_t)N * K * bits / 8, sb = (size_t)N * (K / kGroup) * 2;
        if (!w.reserve(m, qb + 2 * sb + 1024, err)) throw std::runtime_error(err);
        const Tensor& tq = w.add("w.weight", "U32", {(int64_t)N, (int64_t)(K * bits / 32)}, q, qb);
        const Tensor& ts = w.add("w.scales", "BF16", {(int64_t)N, (int64_t)(K / kGroup)}, s, sb);
        const Tensor& tb = w.add("w.biases", "BF16", {(int64_t)N, (int64_t)(K / kGroup)}, b, sb);
        MTL::Buffer* bx = m.new_buffer((size_t)B * K * 2);
        MTL::Buffer* by = m.new_buffer((size_t)B * N * 4);
        std::memcpy(bx->contents(), x, (size_t)B * K * 2);
        auto* cb = m.begin();
        auto* e = cb->computeCommandEncoder();
        if (bits == 8) {
            if (B == 1) gemv8(m, e, w, tq, ts, tb, bx, by, N, K);
            else gemv8_b(m, e, w, tq, ts, tb, bx, by, N, K, B);
        } else {
            if (B == 1) gemv4(m, e, w, tq, ts, tb, bx, by, N, K);
            else gemv4_b(m, e, w, tq, ts, tb, bx, by, N, K, B);
        }
        e->endEncoding();
        m.submit(cb, true);
        std::memcpy(y, by->contents(), (size_t)B * N * 4);
        bx->release();
        by->release();
        return 0;
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return -1;
    }
}

// Cache build + prefill GEMM: C32 = gemm_mpp32(A[:M]), C64 = gemm_mpp(A[:M]), both [M][N] f32,
// against dequant_tile(W) placed at a 256-byte-aligned offset of one cache buffer, as the
// reference's engine registers its projections (src/engine.cpp:139-151).
extern "C" __attribute__((visibility("default"))) int miori_shim_test_prefill(
    const uint32_t* q, const uint16_t* s, const uint16_t* b, const uint16_t* A, float* C32,
    float* C64, uint32_t M, uint32_t N, uint32_t K) {
    using namespace miori;
    try {
        Metal m;
        std::string err;
        if (!m.init("", err)) throw std::runtime_error(err);
        Weights w;
        const size_t qb = (size_t)N * K / 2, sb = (size_t)N * (K / kGroup) * 2;
        if (!w.reserve(m, qb + 2 * sb + 1024, err)) throw std::runtime_error(err);
        const Tensor& tq = w.add("p.weight", "U32", {(int64_t)N, (int64_t)(K / 8)}, q, qb);
        const Tensor& ts = w.add("p.scales", "BF16", {(int64_t)N, (int64_t)(K / kGroup)}, s, sb);
        const Tensor& tb = w.add("p.biases", "BF16", {(int64_t)N, (int64_t)(K / kGroup)}, b, sb);
        const uint32_t off = 4096;  // a non-zero, 256-byte-aligned cache offset
        MTL::Buffer* cache = m.new_buffer(off + (size_t)N * K * 2, false);
        MTL::Buffer* bA = m.new_buffer((size_t)M * K * 2);
        MTL::Buffer* b32 = m.new_buffer((size_t)M * N * 4);
        MTL::Buffer* b64 = m.new_buffer((size_t)M * N * 4);
        std::memcpy(bA->contents(), A, (size_t)M * K * 2);
        auto* cb = m.begin();
        auto* e = cb->computeCommandEncoder();
        dequant_tile(m, e, w, tq, ts, tb, cache, N, K, off);
        gemm_mpp32(m, e, bA, cache, b32, M, N, K, off);
        gemm_mpp(m, e, bA, cache, b64, M, N, K, off);
        e->endEncoding();
        m.submit(cb, true);
        std::memcpy(C32, b32->contents(), (size_t)M * N * 4);
        std::memcpy(C64, b64->contents(), (size_t)M * N * 4);
        cache->release();
        bA->release();
        b32->release();
        b64->release();
        return 0;
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return -1;
    }
}

// The reference's test-gemm-naive procedure (src/main.cpp:561-610): C = A x B^T on bf16 operands
// with row pitches and byte offsets into larger buffers, result read back through contents().
extern "C" __attribute__((visibility("default"))) int miori_shim_test_naive(
    const uint16_t* A, const uint16_t* B, float* C, uint32_t M, uint32_t N, uint32_t K, uint32_t lda,
    uint32_t ldb, uint32_t ldc) {
    using namespace miori;
    try {
        Metal m;
        std::string err;
        if (!m.init("", err)) throw std::runtime_error(err);
        const uint32_t aoff = 512, boff = 1024, coff = 256;  // byte offsets, as the engines pass them
        MTL::Buffer* bA = m.new_buffer(aoff + (size_t)M * lda * 2);
        MTL::Buffer* bB = m.new_buffer(boff + (size_t)N * ldb * 2);
        MTL::Buffer* bC = m.new_buffer(coff + (size_t)M * ldc * 4);
        std::memcpy((char*)bA->contents() + aoff, A, (size_t)M * lda * 2);
        std::memcpy((char*)bB->contents() + boff, B, (size_t)N * ldb * 2);
        std::memset(bC->contents(), 0, coff + (size_t)M * ldc * 4);
        auto* cb = m.begin();
        auto* e = cb->computeCommandEncoder();
        gemm_naive(m, e, bA, bB, bC, M, N, K, lda, ldb, ldc, aoff, boff, coff);
        e->endEncoding();
        m.submit(cb, true);
        std::memcpy(C, (char*)bC->contents() + coff, (size_t)M * ldc * 4);
        bA->release();
        bB->release();
        bC->release();
        return 0;
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return -1;
    }
}

// The neighbours of a projection through the operator API, one decode step's worth: embed8 picks
// token rows out of the 8-bit table (bf16 [T][K]), rmsnorm normalises an fp32 row block against a
// bf16 weight vector, silu_mul gates (reference src/ops.h:16-24, 35-37).
extern "C" __attribute__((visibility("default"))) int miori_shim_test_neighbors(
    const uint32_t* q8, const uint16_t* s8, const uint16_t* b8, uint32_t rows8, const int32_t* tokens,
    uint32_t T, uint16_t* emb_out, const float* x, const uint16_t* gamma, uint16_t* norm_out,
    uint32_t rows, uint32_t K, float eps, const float* gate, const float* up, uint16_t* act_out, uint32_t n_act) {
    using namespace miori;
    try {
        Metal m;
        std::string err;
        if (!m.init("", err)) throw std::runtime_error(err);
        Weights w;
        const size_t qb = (size_t)rows8 * K, sb = (size_t)rows8 * (K / kGroup) * 2;
        if (!w.reserve(m, qb + 2 * sb + (size_t)K * 2 + 2048, err)) throw std::runtime_error(err);
        const Tensor& tq = w.add("e.weight", "U32", {(int64_t)rows8, (int64_t)(K / 4)}, q8, qb);
        const Tensor& ts = w.add("e.scales", "BF16", {(int64_t)rows8, (int64_t)(K / kGroup)}, s8, sb);
        const Tensor& tb = w.add("e.biases", "BF16", {(int64_t)rows8, (int64_t)(K / kGroup)}, b8, sb);
        const Tensor& tg = w.add("n.weight", "BF16", {(int64_t)K}, gamma, (size_t)K * 2);
        MTL::Buffer* btok = m.new_buffer((size_t)T * 4);
        MTL::Buffer* bemb = m.new_buffer((size_t)T * K * 2);
        MTL::Buffer* bx = m.new_buffer((size_t)rows * K * 4);
        MTL::Buffer* bn = m.new_buffer((size_t)rows * K * 2);
        MTL::Buffer* bg = m.new_buffer((size_t)n_act * 4);
        MTL::Buffer* bu = m.new_buffer((size_t)n_act * 4);
        MTL::Buffer* ba = m.new_buffer((size_t)n_act * 2);
        std::memcpy(btok->contents(), tokens, (size_t)T * 4);
        std::memcpy(bx->contents(), x, (size_t)rows * K * 4);
        std::memcpy(bg->contents(), gate, (size_t)n_act * 4);
        std::memcpy(bu->contents(), up, (size_t)n_act * 4);
        auto* cb = m.begin();
        auto* e = cb->computeCommandEncoder();
        embed8(m, e, w, tq, ts, tb, btok, bemb, T, K);
        rmsnorm(m, e, bx, w, tg, bn, rows, K, eps);
        silu_mul(m, e, bg, bu, ba, n_act);
        e->endEncoding();
        m.submit(cb, true);
        std::memcpy(emb_out, bemb->contents(), (size_t)T * K * 2);
        std::memcpy(norm_out, bn->contents(), (size_t)rows * K * 2);
        std::memcpy(act_out, ba->contents(), (size_t)n_act * 2);
        for (MTL::Buffer* b : {btok, bemb, bx, bn, bg, bu, ba}) b->release();
        return 0;
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return -1;
    }
}
