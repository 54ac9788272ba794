// Tensor-map (TMA) helpers shared by the kernels that stage tiles with
// cp.async.bulk.tensor: a host-side encoder reached through the runtime's driver
// entry point (no link-time dependency on the driver library) and the device-side
// 2-D tile load, each into the issuing CTA only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef CUresult (*mb_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);

static inline mb_encode_fn mb_tensor_map_encoder() {
    static mb_encode_fn fn = nullptr;
    if (fn == nullptr) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<mb_encode_fn>(sym);
    }
    return fn;
}

// Row-major 2-D array [rows][row_elems] with a row pitch of pitch_bytes; a box
// of box_cols x box_rows elements; elements outside the array read as zero.
static inline bool mb_make_map_2d(CUtensorMap *map, CUtensorMapDataType type, const void *ptr, size_t rows,
                                  size_t row_elems, size_t pitch_bytes, unsigned box_cols, unsigned box_rows,
                                  CUtensorMapSwizzle swizzle) {
    mb_encode_fn enc = mb_tensor_map_encoder();
    if (enc == nullptr) return false;
    cuuint64_t dims[2] = {(cuuint64_t)row_elems, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, type, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// General form: `rank` dimensions (innermost first) with byte strides for dimensions 1..rank-1
// and a box extent per dimension.  Elements outside the array read as zero and are not
// fetched, which lets a box be wider than the array in a dimension on purpose (padding rows
// of the shared-memory tile).
static inline bool mb_make_map_nd(CUtensorMap *map, CUtensorMapDataType type, const void *ptr, unsigned rank,
                                  const size_t *dims, const size_t *strides_bytes, const unsigned *box,
                                  CUtensorMapSwizzle swizzle) {
    mb_encode_fn enc = mb_tensor_map_encoder();
    if (enc == nullptr || rank < 2 || rank > 5) return false;
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], estr[5];
    for (unsigned i = 0; i < rank; ++i) {
        d[i] = (cuuint64_t)dims[i];
        b[i] = box[i];
        estr[i] = 1;
        if (i > 0) st[i - 1] = (cuuint64_t)strides_bytes[i - 1];
    }
    return enc(map, type, rank, const_cast<void *>(ptr), d, st, b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#ifdef __CUDACC__
// Tile whose first element is (x, y) -> this CTA's shared memory; completion is
// counted in bytes on the mbarrier.  x * element size must be a multiple of 16.
__device__ __forceinline__ void mb_tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, void *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(map), "r"(x), "r"(y),
        "r"((unsigned)__cvta_generic_to_shared(bar))
        : "memory");
}

// Same copy with an L2 eviction-priority hint.  `mb_l2_evict_first()` marks data read once
// per launch (a streamed cache), so that it does not push longer-lived lines (weights,
// activations, code) out of L2.
__device__ __forceinline__ unsigned long long mb_l2_evict_first() {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ unsigned long long mb_l2_evict_last() {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void mb_tma_load_2d_hint(void *dst, const CUtensorMap *map, int x, int y, void *bar,
                                                    unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(map), "r"(x), "r"(y),
        "r"((unsigned)__cvta_generic_to_shared(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void mb_tma_load_3d_hint(void *dst, const CUtensorMap *map, int c0, int c1, int c2, void *bar,
                                                    unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(map), "r"(c0), "r"(c1),
        "r"(c2), "r"((unsigned)__cvta_generic_to_shared(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void mb_tma_load_4d_hint(void *dst, const CUtensorMap *map, int c0, int c1, int c2, int c3,
                                                    void *bar, unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(map), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3), "r"((unsigned)__cvta_generic_to_shared(bar)), "l"(policy)
        : "memory");
}
#endif
