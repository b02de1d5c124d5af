// Operators beyond the reference's src/ops.h, in its style: the fusions the reference planned
// (docs/MILESTONES.md:87: gate + up weights concatenated, SiLU x up as an epilogue, the norm in front
// of a projection), for B <= 4 rows of a decode step.  ops.h stays a strict mirror of the reference's
// header; an engine that wants these includes this file as well.
#pragma once
#include "ops.h"

namespace miori {

// y (bf16 [B][N/2]) = silu(W1 x) * (W3 x) for q/s/b holding w1's N/2 rows followed by w3's: replaces
// gemv4 on w1, gemv4 on w3 and silu_mul (src/engine.cpp:393-395) with one launch, bit for bit
void gemv4_silu(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q, const Tensor& s,
                const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K, uint32_t B = 1);
// y (f32 [B][N]) = W * bf16(rmsnorm(x)), x f32: replaces rmsnorm followed by gemv4 where the norm's
// output has no other reader
void gemv4_rmsnorm(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q, const Tensor& s,
                   const Tensor& b, MTL::Buffer* x, const Tensor& gamma, float eps, MTL::Buffer* y, uint32_t N,
                   uint32_t K, uint32_t B = 1);
// both at once around the gate + up projection: rmsnorm, w1, w3 and silu_mul in one launch
void gemv4_rmsnorm_silu(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
                        const Tensor& s, const Tensor& b, MTL::Buffer* x, const Tensor& gamma, float eps,
                        MTL::Buffer* y, uint32_t N, uint32_t K, uint32_t B = 1);

}  // namespace miori
