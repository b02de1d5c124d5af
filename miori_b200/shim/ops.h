// The hot-path subset of Miori's operator API (reference src/ops.h), same names, argument
// order and meaning, re-pointed at the CUDA kernels of libmiori_b200.so.  Every op only
// enqueues work on the encoder's stream and returns void, as the reference's ops only encode
// a dispatch; invalid arguments surface as std::runtime_error (the reference throws from
// Metal::pso / new_buffer at the equivalent points).  The quantization group is the
// reference's kGroup = 32 (config/m6.h:48).
#pragma once
#include "metal.h"
#include "weights.h"

#include <cstdint>

namespace miori {

constexpr uint32_t kGroup = 32;

// reference src/ops.h:8-10 -- y[N] (f32) = dequant4(W[N][K]) . x[K] (bf16)
void gemv4(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
           const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K);
// reference src/ops.h:12-14 -- 8-bit weights (embedding / LM head)
void gemv8(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
           const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K);
// reference src/ops.h:26-28 -- row-major bf16 [N][K] at byte offset boff of out
void dequant4(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
              const Tensor& s, const Tensor& b, MTL::Buffer* out, uint32_t N, uint32_t K,
              uint32_t boff = 0);
// reference src/ops.h:90-92 -- the cache layout consumed by gemm_mpp* (private to the pair)
void dequant_tile(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
                  const Tensor& s, const Tensor& b, MTL::Buffer* out, uint32_t N, uint32_t K,
                  uint32_t boff = 0);
// reference src/ops.h:94-96 -- C[M][N] (f32) = A[M][K] (bf16) x cache^T
void gemm_mpp(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
              MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t boff = 0);
// reference src/ops.h:101-103 -- byte offsets into A, B and C
void gemm_mpp_off(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
                  MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t aoff, uint32_t boff,
                  uint32_t coff);
// reference src/ops.h:105-107, 126-128 -- tuning variants of gemv4 (same result contract)
void gemv4x4(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K);
void gemv4x2(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K);
// reference src/ops.h:113-115 -- q, s, b in buffers of their own
void gemv4_raw(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* q, MTL::Buffer* s,
               MTL::Buffer* b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K);
// reference src/ops.h:135-138 -- byte offsets for weights, x and y
void gemv8_off(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* wbuf, uint32_t qoff,
               uint32_t soff, uint32_t boff, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K,
               uint32_t xoff, uint32_t yoff);
// reference src/ops.h:164-171 -- B input rows share one pass over W.  The reference accepts
// B <= 4 only and always touches four rows; here 1 <= B <= 32 and exactly B rows are touched.
void gemv4_b(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K,
             uint32_t B);
void gemv8_b(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K,
             uint32_t B);
// reference src/ops.h:176-179
void gemv8_b_off(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
                 const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N,
                 uint32_t K, uint32_t B, uint32_t xoff, uint32_t yoff);
// reference src/ops.h:203-205 -- row-major bf16 [N][K] from 8-bit weights
void dequant8(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
              const Tensor& s, const Tensor& b, MTL::Buffer* out, uint32_t N, uint32_t K);
// reference src/ops.h:30-33 -- C[M][N] (f32) = A[M][K] (bf16) x B[N][K]^T (bf16), row pitches in
// elements, byte offsets into the three buffers
void gemm_naive(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
                MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t lda, uint32_t ldb,
                uint32_t ldc, uint32_t aoff = 0, uint32_t boff = 0, uint32_t coff = 0);
// reference src/ops.h:16-18 -- y (bf16) = x (f32) * rsqrt(mean(x^2) + eps) * gamma, row by row
void rmsnorm(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* x, const Weights& w,
             const Tensor& gamma, MTL::Buffer* y, uint32_t rows, uint32_t n, float eps);
// reference src/ops.h:23-24 -- out (bf16) = silu(gate) * up, both f32
void silu_mul(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* gate, MTL::Buffer* up,
              MTL::Buffer* out, uint32_t n);
// reference src/ops.h:35-37 -- rows tokens[t] of the 8-bit table as bf16 [T][K]
void embed8(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
            const Tensor& s, const Tensor& b, MTL::Buffer* tokens, MTL::Buffer* out, uint32_t T,
            uint32_t K);
// reference src/ops.h:109-111 -- out (f32) = x + src * rsqrt(mean(src^2) + eps) * gamma, row by row;
// out may be x (the engine updates its residual stream in place, src/engine.cpp:384-386)
void postnorm_add(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* x, MTL::Buffer* src, const Weights& w,
                  const Tensor& gamma, MTL::Buffer* out, uint32_t rows, uint32_t n, float eps);

// reference src/ops.h:207-209 -- the small-M tile shape; same kernel, same result per row
void gemm_mpp32(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
                MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t boff = 0);

}  // namespace miori
