// Kernel-selection overrides carried in the `flags` argument of the launch entries, for tests
// and A/B timing only: every choice computes the same result, the default heuristics pick among
// them by shape.  Private to this library and its tests (not part of the C ABI contract).
#pragma once
#define MIORI_TUNE_GEMM_NARROW 0x100u   // GEMM: 128x128 tiles
#define MIORI_TUNE_GEMM_WIDE 0x200u     // GEMM: 128x256 tiles, one CTA per tile
#define MIORI_TUNE_GEMV_SIMT 0x400u     // GEMV: the scalar-FMA kernel
#define MIORI_TUNE_GEMV_LDG 0x800u      // GEMV: mma.sync kernel fed by plain loads (no TMA)
#define MIORI_TUNE_GEMV_MMASYNC 0x1000u // GEMV: the mma.sync kernel with the TMA ring instead of tcgen05
#define MIORI_TUNE_GEMV_TILED 0x2000u   // GEMV (mma.sync kernel): tiled TMA even where linear bulk copies fit
#define MIORI_TUNE_GEMM_PAIR 0x4000u    // GEMM: two-CTA (cta_group::2) kernel
#define MIORI_TUNE_GEMM_NOPAIR 0x8000u  // GEMM: never the two-CTA kernel
#define MIORI_TUNE_UMMA_SPLIT_SHIFT 16  // GEMV (tcgen05 kernel): bits 16..19 = forced K split (1, 2, 4, 8)
#define MIORI_TUNE_GEMM_SPLIT_SHIFT 16  // GEMM: bits 16..19 = forced K split count (1..15; needs the workspace for it)
#define MIORI_TUNE_GEMV_UMMA 0x100000u  // GEMV: the tcgen05 kernel even where the heuristics prefer another
