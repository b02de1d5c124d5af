// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled) without linking
// libcuda: the entry point comes from the CUDA runtime.
#pragma once
#include "common.cuh"

#include <cuda.h>

namespace miori_b200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Row-major 2-D tensor [rows][inner] of `dtype` elements (`esize` bytes each), box
// [box_rows][box_inner], zero fill outside the tensor.  Rows are row_pitch_elems apart (0: dense).
// The row pitch in bytes must be a multiple of 16 and the base 16-byte aligned.
inline int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype,
                        uint32_t esize, uint64_t inner, uint64_t rows, uint32_t box_inner,
                        uint32_t box_rows, CUtensorMapSwizzle swizzle, uint64_t row_pitch_elems = 0) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MIORI_E_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {(row_pitch_elems ? row_pitch_elems : inner) * esize};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MIORI_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return MIORI_OK;
}

// Row-major 3-D tensor [d2][d1][d0] (d0 innermost, rows row_pitch_elems apart, 0: dense), box
// [1][box1][box0], no fill (used for stores, which clip at the tensor's edges).  The row pitch and
// the slice pitch in bytes must be multiples of 16 and the base 16-byte aligned.
inline int make_tmap_3d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype,
                        uint32_t esize, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t box0,
                        uint32_t box1, CUtensorMapSwizzle swizzle, uint64_t row_pitch_elems = 0) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MIORI_E_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
    const uint64_t pitch = row_pitch_elems ? row_pitch_elems : d0;
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {pitch * esize, pitch * d1 * esize};
    const cuuint32_t box[3] = {box0, box1, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, dtype, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MIORI_E_CUDA, "cuTensorMapEncodeTiled (3-D) failed (%d)", (int)r);
    return MIORI_OK;
}

#ifdef __CUDACC__
// 2-D tiled TMA load into shared memory; c0 is the innermost (element) coordinate, whose
// byte offset must be a multiple of 16.  Completion is counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// 3-D tiled TMA store from shared memory (bulk-group completion).  c0 is the innermost
// coordinate (byte offset a multiple of 16, never negative); elements outside the tensor are
// not written.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int c0, int c1, int c2,
                                             uint32_t src) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
        ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(src)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// wait until at most N of this thread's bulk groups still read their shared-memory source
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// wait until every bulk group of this thread has completed (its writes are performed)
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
#endif

}  // namespace miori_b200
