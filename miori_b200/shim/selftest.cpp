// C entry points that drive the operator shim the way the reference's own test commands do
// (reference src/main.cpp:44-87 test-gemv4/8, :1403-1443 test-mpp-tile), for the Python
// tests: host arrays in, host arrays out, everything in between through miori::Metal,
// miori::Weights and the miori:: operators.
#include "fused_ops.h"
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

// The feed-forward block of a decode step (reference src/engine.cpp:388-399: rmsnorm, w1, w3,
// silu_mul, w2, post-norm added onto the residual in place) through the operator API, three ways:
// the reference's six operators; the gate + up weights as one tensor with the activation as the
// GEMV's epilogue; the norm in front of that GEMV as well.  q13/s13/b13 hold w1's F rows followed by
// w3's; every variant starts from its own copy of the residual x and leaves the new residual there.
extern "C" __attribute__((visibility("default"))) int miori_shim_test_ffn(
    const uint32_t* q13, const uint16_t* s13, const uint16_t* b13, const uint32_t* q2, const uint16_t* s2,
    const uint16_t* b2, const uint16_t* gamma_in, const uint16_t* gamma_post, const float* x, uint32_t F,
    uint32_t H, float eps, float* out_six_ops, float* out_gated, float* out_normed_gated) {
    using namespace miori;
    try {
        Metal m;
        std::string err;
        if (!m.init("", err)) throw std::runtime_error(err);
        Weights w;
        const size_t q13b = (size_t)2 * F * H / 2, s13b = (size_t)2 * F * (H / kGroup) * 2;
        const size_t q2b = (size_t)H * F / 2, s2b = (size_t)H * (F / kGroup) * 2;
        if (!w.reserve(m, q13b + 2 * s13b + q2b + 2 * s2b + (size_t)4 * H + 4096, err)) throw std::runtime_error(err);
        const Tensor& tq13 = w.add("w13.weight", "U32", {(int64_t)2 * F, (int64_t)(H / 8)}, q13, q13b);
        const Tensor& ts13 = w.add("w13.scales", "BF16", {(int64_t)2 * F, (int64_t)(H / kGroup)}, s13, s13b);
        const Tensor& tb13 = w.add("w13.biases", "BF16", {(int64_t)2 * F, (int64_t)(H / kGroup)}, b13, s13b);
        const Tensor& tq2 = w.add("w2.weight", "U32", {(int64_t)H, (int64_t)(F / 8)}, q2, q2b);
        const Tensor& ts2 = w.add("w2.scales", "BF16", {(int64_t)H, (int64_t)(F / kGroup)}, s2, s2b);
        const Tensor& tb2 = w.add("w2.biases", "BF16", {(int64_t)H, (int64_t)(F / kGroup)}, b2, s2b);
        const Tensor& tgi = w.add("ffn_norm.weight", "BF16", {(int64_t)H}, gamma_in, (size_t)H * 2);
        const Tensor& tgp = w.add("post_ffn_norm.weight", "BF16", {(int64_t)H}, gamma_post, (size_t)H * 2);
        // w1 and w3 as the halves of the fused tensors (rows are contiguous)
        auto half = [&](const Tensor& t, int which) {
            Tensor h = t;
            const uint64_t mid = t.begin + (t.end - t.begin) / 2;
            h.shape[0] = t.shape[0] / 2;
            if (which == 0) h.end = mid; else h.begin = mid;
            return h;
        };
        const Tensor q1 = half(tq13, 0), s1 = half(ts13, 0), b1 = half(tb13, 0);
        const Tensor q3 = half(tq13, 1), s3 = half(ts13, 1), b3 = half(tb13, 1);
        MTL::Buffer* xs[3];
        for (auto& bx : xs) {
            bx = m.new_buffer((size_t)H * 4);
            std::memcpy(bx->contents(), x, (size_t)H * 4);
        }
        MTL::Buffer* h = m.new_buffer((size_t)H * 2);
        MTL::Buffer* fg = m.new_buffer((size_t)F * 4);
        MTL::Buffer* fu = m.new_buffer((size_t)F * 4);
        MTL::Buffer* fact = m.new_buffer((size_t)F * 2);
        MTL::Buffer* down = m.new_buffer((size_t)H * 4);
        auto* cb = m.begin();
        auto* e = cb->computeCommandEncoder();
        // the reference's operators
        rmsnorm(m, e, xs[0], w, tgi, h, 1, H, eps);
        gemv4(m, e, w, q1, s1, b1, h, fg, F, H);
        gemv4(m, e, w, q3, s3, b3, h, fu, F, H);
        silu_mul(m, e, fg, fu, fact, F);
        gemv4(m, e, w, tq2, ts2, tb2, fact, down, H, F);
        postnorm_add(m, e, xs[0], down, w, tgp, xs[0], 1, H, eps);
        // gate + up in one launch with the activation
        rmsnorm(m, e, xs[1], w, tgi, h, 1, H, eps);
        gemv4_silu(m, e, w, tq13, ts13, tb13, h, fact, 2 * F, H);
        gemv4(m, e, w, tq2, ts2, tb2, fact, down, H, F);
        postnorm_add(m, e, xs[1], down, w, tgp, xs[1], 1, H, eps);
        // and with the norm in front
        gemv4_rmsnorm_silu(m, e, w, tq13, ts13, tb13, xs[2], tgi, eps, fact, 2 * F, H);
        gemv4(m, e, w, tq2, ts2, tb2, fact, down, H, F);
        postnorm_add(m, e, xs[2], down, w, tgp, xs[2], 1, H, eps);
        e->endEncoding();
        m.submit(cb, true);
        std::memcpy(out_six_ops, xs[0]->contents(), (size_t)H * 4);
        std::memcpy(out_gated, xs[1]->contents(), (size_t)H * 4);
        std::memcpy(out_normed_gated, xs[2]->contents(), (size_t)H * 4);
        for (MTL::Buffer* b : {xs[0], xs[1], xs[2], h, fg, fu, fact, down}) b->release();
        return 0;
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return -1;
    }
}
