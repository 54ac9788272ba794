// Pieces shared by the kernels that walk a KV cache in 32-row TMA tiles: the mbarrier
// helpers with bounded waits, one chunk's scores and weighted values inside a warp, the
// ordered merge of per-chunk partials and the int8 quantization of a merged row.
#pragma once

#include "common.cuh"
#include "tma.cuh"

#include <float.h>

namespace {

constexpr int CHUNK = 32;
constexpr int FAST_THREADS = 128;
constexpr int MERGE_MAX = 128;      // most chunks one stream may have (4096 rows)
constexpr unsigned SPIN_LIMIT = 1u << 24;
constexpr int ROWS_SMEM_MAX = 225 * 1024;

__device__ __forceinline__ unsigned smem_addr(const void *ptr) {
    return (unsigned)__cvta_generic_to_shared(ptr);
}
__device__ __forceinline__ void mbar_init(void *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
                 "r"(bytes)
                 : "memory");
}
// Bounded wait for phase `parity`; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(void *bar, unsigned parity, unsigned limit) {
    for (unsigned i = 0; i < limit; ++i) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Merge one head's per-chunk partials (max, sum, weighted V[hw]) in chunk index order:
// M = max m_s, w_s = exp(m_s - M), L = sum l_s w_s, O = sum acc_s w_s, out = O / L, the
// sums as fma chains over s.  One warp; `ph` is in shared memory unless GLOBAL.
template <bool GLOBAL, typename Emit>
__device__ __forceinline__ void merge_chunks(const float *ph, int ns, int hw, int lane, float *wts, Emit emit) {
    auto ld = [](const float *q) { return GLOBAL ? __ldcg(q) : *q; };
    const int pitch = hw + 2;
    for (int s = lane; s < ns; s += 32) wts[s] = ld(ph + (long)s * pitch);
    __syncwarp();
    float M = -FLT_MAX;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, wts[s]);
    __syncwarp();
    for (int s = lane; s < ns; s += 32) wts[s] = exp_ref<false>(wts[s] - M);
    __syncwarp();
    float L = 0.0f;
    for (int s = 0; s < ns; ++s) L = fmaf(ld(ph + (long)s * pitch + 1), wts[s], L);
    for (int d = lane; d < hw; d += 32) {
        float O = 0.0f;
#pragma unroll 4
        for (int s = 0; s < ns; ++s) O = fmaf(ld(ph + (long)s * pitch + 2 + d), wts[s], O);
        emit(d, L > 0.0f ? O / L : 0.0f);
    }
}

// merge_chunks for one dimension d by one thread: the same operations in the same order
// (M, then per chunk w = exp(m - M), L and O as fma chains over the chunk index).
__device__ __forceinline__ float merge_dim(const float *ph, int ns, int hw, int d) {
    const int pitch = hw + 2;
    float M = -FLT_MAX;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, ph[(long)s * pitch]);
    float L = 0.0f, O = 0.0f;
    for (int s = 0; s < ns; ++s) {
        const float w = exp_ref<false>(ph[(long)s * pitch] - M);
        L = fmaf(ph[(long)s * pitch + 1], w, L);
        O = fmaf(ph[(long)s * pitch + 2 + d], w, O);
    }
    return L > 0.0f ? O / L : 0.0f;
}

// Quantize one merged row (already in `vals`, shared) to int8: shared by the
// per-stream tail of the kernel below.
__device__ __forceinline__ void quantize_shared_row(const float *vals, int width, int8_t *qrow,
                                                    float *sx_out, float *red) {
    float amax = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) amax = fmaxf(amax, fabsf(vals[i]));
    amax = block_max1(amax, red);   // callers pass scratch no thread is still reading
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int v = round_half_away(__fmul_rn(vals[i], inv));
        qrow[i] = (int8_t)min(127, max(-127, v));
    }
    if (threadIdx.x == 0) *sx_out = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
}

// The same quantization by one warp (`vals` and `qrow` in shared memory).
__device__ __forceinline__ void quantize_row_warp(const float *vals, int width, int8_t *qrow, float *sx_out, int lane) {
    float amax = 0.0f;
    for (int i = lane; i < width; i += 32) amax = fmaxf(amax, fabsf(vals[i]));
    amax = warp_max(amax);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = lane; i < width; i += 32) {
        const int v = round_half_away(__fmul_rn(vals[i], inv));
        qrow[i] = (int8_t)min(127, max(-127, v));
    }
    if (lane == 0) *sx_out = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
}

// Scores of one 32-row chunk for one head, one warp.  TPP lanes share a row (a float4 of
// the head each), 32 / TPP rows per step, TPP steps.  Each lane first forms its four-term
// partial for all TPP rows it touches, then the TPP lanes of a row group exchange halves
// (TPP - 1 shuffles in all, independent within a round) so that lane (sub, li) ends with
// the full dot product of row li * (32 / TPP) + sub.  Returns that score, unscaled.
template <int TPP>
__device__ __forceinline__ float chunk_scores(const float *Ks, int pitch, float4 qv, int sub, int li) {
    constexpr int RPS = 32 / TPP;
    float a[TPP];
#pragma unroll
    for (int t = 0; t < TPP; ++t) {
        const float4 kv = *reinterpret_cast<const float4 *>(Ks + (long)(t * RPS + sub) * pitch + 4 * li);
        float x = 0.0f;
        x = fmaf(qv.x, kv.x, x); x = fmaf(qv.y, kv.y, x);
        x = fmaf(qv.z, kv.z, x); x = fmaf(qv.w, kv.w, x);
        a[t] = x;
    }
#pragma unroll
    for (int o = TPP / 2; o >= 1; o >>= 1) {
        const bool upper = (li & o) != 0;     // this lane keeps the rows whose index has bit o set
#pragma unroll
        for (int t = 0; t < o; ++t) {
            const float send = upper ? a[t] : a[t + o];
            const float keep = upper ? a[t + o] : a[t];
            a[t] = keep + __shfl_xor_sync(MB_FULL, send, o);
        }
    }
    return a[0];
}

// Weighted V rows of one chunk for one head: lane (sub, li) adds rows t * (32 / TPP) + sub
// for its float4 of the head, weights from the lane that owns each row's score; the row
// sub-groups are then added up across the warp.
template <int TPP>
__device__ __forceinline__ float4 chunk_values(const float *Vs, int pitch, float e, int sub, int li) {
    constexpr int RPS = 32 / TPP;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < TPP; ++t) {
        const float w = __shfl_sync(MB_FULL, e, sub * TPP + t);
        const float4 vv = *reinterpret_cast<const float4 *>(Vs + (long)(t * RPS + sub) * pitch + 4 * li);
        acc.x = fmaf(w, vv.x, acc.x); acc.y = fmaf(w, vv.y, acc.y);
        acc.z = fmaf(w, vv.z, acc.z); acc.w = fmaf(w, vv.w, acc.w);
    }
#pragma unroll
    for (int o = TPP; o < 32; o <<= 1) {
        acc.x += __shfl_xor_sync(MB_FULL, acc.x, o); acc.y += __shfl_xor_sync(MB_FULL, acc.y, o);
        acc.z += __shfl_xor_sync(MB_FULL, acc.z, o); acc.w += __shfl_xor_sync(MB_FULL, acc.w, o);
    }
    return acc;
}

}  // namespace
