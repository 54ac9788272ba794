// Batched f16-weight products on the 5th-generation tensor cores (tcgen05, kind::f16).
//
//   out[b][r] = epilogue( sum_k W[r][k] * x[b][k] + bias[r] )       W in f16, x and the sum in f32
//
// for 16 or more streams stepped together: one pass over the weight serves every lane.  The
// reference keeps the activations in f32 and only the weights in f16 (matvec_f16,
// src/qmat.c:319-377).  A tensor-core operand has to be f16, so every activation is split
// into two halves that add up to it to 22 bits,
//   hi = f16(x), lo = f16(x - hi),
// and both go through the MMA as separate lanes of the N dimension: a tile of 16 streams is
// N = 32 columns (16 hi, 16 lo), accumulated in f32 in tensor memory, and the epilogue adds a
// stream's two columns.  The weights need no conversion at all: TMA brings them in as they
// lie in memory.  The result agrees with the SIMT kernel of gemv.cu to f32 rounding of the
// sums (about 1e-6 of a row; the reference's own bound for this format is 1e-3,
// src/qmat.c:1064-1104); it is not bit-identical to it, so with f16 weights a stream's
// hidden rows at 16 or more lanes match its rows at fewer lanes to that rounding only.
//
// One CTA = 128 weight rows x 16 streams over all of K, through a ring of eight stages of
// [128 rows x 128 B] of W (64 halves) and [32 rows x 128 B] of the split activations, each
// stage filled by two TMA copies that complete on its mbarrier; one thread issues four
// tcgen05.mma (M128 N32 K16) per stage and commits the stage's release; the four warps read
// their 32 accumulator rows with tcgen05.ld and run the epilogue.  The first weight stages
// are requested before the programmatic-dependency wait.  Every wait is bounded (status bits
// 8 and 16, as in gemm_tc.cu).
#include "common.cuh"
#include "launch.h"

#include "tc_common.cuh"

#include <cuda_fp16.h>
#include <string.h>

namespace {

constexpr int F_THREADS = 128;
constexpr int F_TM = 128;             // weight rows per tile
constexpr int F_BN = 16;              // streams per tile (N = 2 * F_BN columns)
constexpr int F_KC = 128;             // K bytes per stage: 64 halves
constexpr int F_STAGES = 8;
constexpr int FA_BYTES = F_TM * F_KC;         // 16 KB
constexpr int FB_BYTES = 2 * F_BN * F_KC;     // 4 KB
constexpr int F_TMEM_COLS = 32;
constexpr size_t F_SMEM = (size_t)F_STAGES * (FA_BYTES + FB_BYTES) + 1024;

struct F16P {
    const float *bias;
    float *out;
    const int *n_active;
    int *status;
    const uint32_t *tanh_tab;
    long n, k, out_stride;
    int batch, epilogue, strict;
};

// x[b][k] (f32) -> hi plane and lo plane of halves, [rows_alloc][k] each.
__global__ void __launch_bounds__(256)
k_split_f16(const float *__restrict__ x, __half *__restrict__ hi, __half *__restrict__ lo, int k,
            const int *__restrict__ n_active) {
    const int live = mb_lane_count(n_active);
    mb_pdl_wait();
    mb_pdl_trigger();
    const int b = blockIdx.x;
    if (b >= live) return;
    const float *row = x + (long)b * k;
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const float v = row[i];
        const __half h = __float2half_rn(v);
        hi[(long)b * k + i] = h;
        lo[(long)b * k + i] = __float2half_rn(__fsub_rn(v, __half2float(h)));
    }
}

__global__ void __launch_bounds__(F_THREADS)
k_gemm_f16_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, F16P p) {
    extern __shared__ unsigned char smem_f16[];
    __shared__ __align__(8) unsigned long long full_bar[F_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[F_STAGES];
    __shared__ __align__(8) unsigned long long done_bar;
    __shared__ uint32_t s_tmem;
    __shared__ unsigned s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = blockIdx.y * F_BN;
    const long m0 = (long)blockIdx.x * F_TM;
    const int nchunks = (int)((p.k * 2 + F_KC - 1) / F_KC);
    unsigned char *base = smem_f16 + ((1024u - (saddr(smem_f16) & 1023u)) & 1023u);
    unsigned char *As = base;                                    // [stage][128 rows][128 B]
    unsigned char *Bs = base + (size_t)F_STAGES * FA_BYTES;      // [stage][hi 16 rows | lo 16 rows][128 B]
    if (threadIdx.x == 0) {
        for (int s = 0; s < F_STAGES; ++s) {
            bar_init(&full_bar[s], 1u);
            bar_init(&empty_bar[s], 1u);
        }
        bar_init(&done_bar, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_fail = 0u;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&s_tmem)), "r"(F_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const unsigned stage_bytes = (unsigned)(FA_BYTES + FB_BYTES);
    const int first = min(nchunks, F_STAGES);
    // weights are written by no preceding launch: their first stages are requested before the wait
    if (warp == 0 && lane == 0) {
        for (int c = 0; c < first; ++c) {
            bar_expect(&full_bar[c], stage_bytes);
            tma_load_2d(As + (size_t)c * FA_BYTES, &map_w, c * F_KC, (int)m0, &full_bar[c]);
        }
    }
    const int nb = min(p.batch, mb_lane_count(p.n_active));
    if (warp == 0 && lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    mb_pdl_wait();
    mb_pdl_trigger();
    // the split activations of a stage: one copy of 128 B x 16 streams x 2 planes
    auto load_x = [&](int c, int s) {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(saddr(Bs + (size_t)s * FB_BYTES)), "l"(&map_x), "r"(c * F_KC), "r"(b0), "r"(0),
            "r"(saddr(&full_bar[s]))
            : "memory");
    };
    if (b0 >= nb) {
        // no live stream in this tile: let the requested stages land, then give the TMEM back
        if (warp == 0 && lane == 0) {
            for (int c = 0; c < first; ++c) {
                load_x(c, c);
                bar_wait(&full_bar[c], 0u, TC_SPIN);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 0)
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(F_TMEM_COLS) : "memory");
        return;
    }
    if (warp == 0 && lane == 0) {
        for (int c = 0; c < first; ++c) load_x(c, c);
        for (int c = first; c < nchunks; ++c) {
            const int s = c % F_STAGES;
            if (!bar_wait(&empty_bar[s], (unsigned)((c / F_STAGES - 1) & 1), TC_SPIN)) {
                s_fail = 1u;
                if (p.status != nullptr) atomicOr(p.status, 8);
                break;
            }
            bar_expect(&full_bar[s], stage_bytes);
            tma_load_2d(As + (size_t)s * FA_BYTES, &map_w, c * F_KC, (int)m0, &full_bar[s]);
            load_x(c, s);
        }
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = instr_desc_f16(F_TM, 2 * F_BN);
        for (int c = 0; c < nchunks; ++c) {
            const int s = c % F_STAGES;
            if (!bar_wait(&full_bar[s], (unsigned)((c / F_STAGES) & 1), TC_SPIN)) {
                s_fail = 1u;
                if (p.status != nullptr) atomicOr(p.status, 8);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = smem_desc_sw128(saddr(As + (size_t)s * FA_BYTES));
            const uint64_t db = smem_desc_sw128(saddr(Bs + (size_t)s * FB_BYTES));
#pragma unroll
            for (int kk = 0; kk < F_KC / 32; ++kk)            // 16 halves = 32 K-bytes per instruction
                mma_f16(tmem, da + 2u * kk, db + 2u * kk, idesc, (c | kk) != 0 ? 1u : 0u);
            mma_commit(&empty_bar[s]);
        }
        mma_commit(&done_bar);
    }
    const long row = m0 + warp * 32 + lane;
    const bool row_ok = row < p.n;
    const float bias = (row_ok && p.bias != nullptr) ? __ldg(p.bias + row) : 0.0f;
    float prior[F_BN];
#pragma unroll
    for (int j = 0; j < F_BN; ++j) {
        const int b = b0 + j;
        prior[j] = (p.epilogue == MB_EPI_RESIDUAL && row_ok && b < nb) ? p.out[(long)b * p.out_stride + row] : 0.0f;
    }
    const bool done = bar_wait(&done_bar, 0u, TC_SPIN);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool good = done && s_fail == 0u;
    if (!done && threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, 16);
    if (!good) {
        // a wait ran out: give copies still in flight one more bounded chance to land before
        // this CTA's shared memory is released
        if (threadIdx.x == 0)
            for (int s = 0; s < F_STAGES && s < nchunks; ++s) bar_wait(&full_bar[s], 0u, TC_SPIN >> 4);
    } else {
        float v[32];
        tmem_ld32f(tmem + ((uint32_t)(warp * 32) << 16), v);
        if (row_ok) {
#pragma unroll
            for (int j = 0; j < F_BN; ++j) {
                const int b = b0 + j;
                if (b < nb) {
                    float y = __fadd_rn(v[j], v[F_BN + j]);           // hi part + lo part
                    if (p.bias != nullptr) y = __fadd_rn(y, bias);
                    float *dst = p.out + (long)b * p.out_stride + row;
                    if (p.epilogue == MB_EPI_RESIDUAL) *dst = __fadd_rn(prior[j], y);
                    else if (p.epilogue == MB_EPI_GELU)
                        *dst = p.strict ? gelu_tanh<true>(y, p.tanh_tab) : gelu_tanh<false>(y, nullptr);
                    else *dst = y;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(F_TMEM_COLS) : "memory");
}

}  // namespace

extern "C" int mb_gemm_tc_f16_init(void) {
    return (int)cudaFuncSetAttribute(k_gemm_f16_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F_SMEM);
}

// Halves the split buffer must hold for `rows_alloc` streams of at most k_max activations.
extern "C" size_t mb_gemm_tc_f16_split_halves(size_t rows_alloc, size_t k_max) { return 2u * rows_alloc * k_max; }

extern "C" int mb_gemm_tc_f16_supported(size_t n, size_t k, size_t batch) {
    return n > 0 && batch >= 16 && k >= 64 && (k % 8u) == 0;
}

extern "C" int mb_gemm_tc_f16(const mb_gemv_args *a, void *split, size_t rows_alloc, int *status, mb_stream stream) {
    if (a == nullptr || a->qtype != MB_F16 || !mb_gemm_tc_f16_supported(a->n, a->k, a->batch) || a->x == nullptr ||
        a->out == nullptr || split == nullptr || rows_alloc < a->batch || (((uintptr_t)a->w | (uintptr_t)split) & 15u) != 0)
        return (int)cudaErrorInvalidValue;
    __half *hi = static_cast<__half *>(split);
    __half *lo = hi + rows_alloc * a->k;
    cudaStream_t s = (cudaStream_t)stream;
    mb_launch(k_split_f16, dim3((unsigned)a->batch), dim3(256), 0, s, a->x, hi, lo, (int)a->k, a->n_active);
    int rc = mb_check_launch();
    if (rc != 0) return rc;
    CUtensorMap map_w, map_x;
    // weights: [n][2k bytes]; box 128 B x 128 rows.  activations: (2k bytes, rows_alloc streams,
    // 2 planes); box 128 B x 16 streams x both planes.  128-byte swizzle for both.
    if (!mb_make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->w, a->n, a->k * 2u, a->k * 2u, (unsigned)F_KC, F_TM,
                        CU_TENSOR_MAP_SWIZZLE_128B))
        return (int)cudaErrorInvalidValue;
    const size_t dims[3] = {a->k * 2u, rows_alloc, 2u};
    const size_t strides[2] = {a->k * 2u, rows_alloc * a->k * 2u};
    const unsigned box[3] = {(unsigned)F_KC, (unsigned)F_BN, 2u};
    if (!mb_make_map_nd(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, hi, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
        return (int)cudaErrorInvalidValue;
    F16P p;
    memset(&p, 0, sizeof(p));
    p.bias = a->bias; p.out = a->out; p.n_active = a->n_active; p.status = status; p.tanh_tab = a->tanh_tab;
    p.n = (long)a->n; p.k = (long)a->k; p.out_stride = (long)a->out_stride;
    p.batch = (int)a->batch; p.epilogue = a->epilogue; p.strict = a->strict;
    const unsigned m_tiles = (unsigned)((a->n + F_TM - 1) / F_TM);
    const unsigned b_tiles = (unsigned)((a->batch + F_BN - 1) / F_BN);
    mb_launch(k_gemm_f16_tc, dim3(m_tiles, b_tiles), dim3(F_THREADS), F_SMEM, s, map_w, map_x, p);
    return mb_check_launch();
}
