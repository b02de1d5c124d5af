// int4 / int8 -> bf16 weight cache build.  out = bf16(float(code)*scale + bias) evaluated
// exactly as the reference does (src/cpu_ref.h:16-23,33,44): an fp32 multiply, an fp32 add
// (kept unfused so that overflow behaves identically) and the integer RNE to bf16.
//
// HBM-bound: 0.5625-1.125 B read and 2 B written per weight.  One thread converts eight
// consecutive weights of a row (one or two packed words) and stores them as one 16-byte
// vector, so every warp reads 128/256 contiguous bytes and writes 512.
#pragma once
#include "common.cuh"

namespace miori_b200 {

template <int BITS>
__global__ void __launch_bounds__(256)
dequant_rowmajor_kernel(const uint32_t* __restrict__ q, const uint16_t* __restrict__ s,
                        const uint16_t* __restrict__ b, uint4* __restrict__ out, uint32_t N,
                        uint32_t K, uint32_t gshift) {
    const uint64_t units = (uint64_t)N * (K >> 3);  // 8 weights per unit
    const uint32_t upr = K >> 3;                    // units per row
    const uint32_t ng = K >> gshift;
    pdl_launch_dependents();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < units;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / upr), u = (uint32_t)(i - (uint64_t)row * upr);
        const uint32_t g = (u << 3) >> gshift;
        const float sc = bf16_bits_to_float(__ldg(s + (size_t)row * ng + g));
        const float bi = bf16_bits_to_float(__ldg(b + (size_t)row * ng + g));
        uint32_t code[8];
        if (BITS == 4) {
            const uint32_t w = __ldg(q + i);
#pragma unroll
            for (int j = 0; j < 8; ++j) code[j] = (w >> (4 * j)) & 0xFu;
        } else {
            const uint2 w = __ldg(reinterpret_cast<const uint2*>(q) + i);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                code[j] = (w.x >> (8 * j)) & 0xFFu;
                code[4 + j] = (w.y >> (8 * j)) & 0xFFu;
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float q0 = __uint_as_float(0x4B000000u | code[2 * p]) - 8388608.0f;
            const float q1 = __uint_as_float(0x4B000000u | code[2 * p + 1]) - 8388608.0f;
            const float f0 = __fadd_rn(__fmul_rn(q0, sc), bi);
            const float f1 = __fadd_rn(__fmul_rn(q1, sc), bi);
            o[p] = float_to_bf16_bits(f0) | (float_to_bf16_bits(f1) << 16);
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

template <int BITS>
int launch_dequant_rowmajor(const void* q, const void* s, const void* b, void* out, uint32_t N,
                            uint32_t K, uint32_t group, cudaStream_t stream) {
    const uint64_t units = (uint64_t)N * (K >> 3);
    uint64_t blocks = (units + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    cudaError_t e = launch(dequant_rowmajor_kernel<BITS>, dim3((unsigned)blocks), dim3(256), 0,
                           stream, false, reinterpret_cast<const uint32_t*>(q),
                           reinterpret_cast<const uint16_t*>(s),
                           reinterpret_cast<const uint16_t*>(b), reinterpret_cast<uint4*>(out), N,
                           K, group == 32 ? 5u : 6u);
    if (e != cudaSuccess) return cuda_fail(e, "dequant_rowmajor launch");
    return MIORI_OK;
}

}  // namespace miori_b200
