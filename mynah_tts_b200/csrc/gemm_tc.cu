// Batched int8 weight products on the 5th-generation tensor cores (tcgen05).
//
//   out[b][r] = epilogue( (sum_k W[r][k] * qx[b][k]) * scales[r] * sx[b] + bias[r] )
//
// for 16 or more streams stepped together: one pass over the weight serves every
// lane (the weight-stationary batching of src/qmat.c:681-735 in mynah-tts).  The
// sum is an exact int32, so the result has the same bits as the SIMT kernel in
// gemv.cu and as the reference, whatever the batch.
//
// One CTA = one tile of 128 weight rows x BN lanes over a range of K:
//   * TMA (cp.async.bulk.tensor, 128-byte swizzle, into this CTA only) brings
//     [128 rows x 128 K-bytes] of W and [BN lanes x 128 K-bytes] of the quantized
//     activations into shared memory, one stage per 128-byte K chunk, each
//     stage completing on its own mbarrier;
//   * one thread issues tcgen05.mma kind::i8 (M=128, N=BN, K=32), four per
//     stage, accumulating int32 in tensor memory (TMEM);
//   * after tcgen05.commit signals completion, the four warps read their 32 TMEM
//     lanes (= weight rows) with tcgen05.ld and apply the epilogue.
// Grid: (row tiles, lane tiles).  A CTA walks the whole K range through a ring of
// eight stages: a stage is refilled as soon as tcgen05.commit reports that the
// MMAs reading it have finished.
//
// Long K (more chunks than stages, the feed-forward down product): a thread-block
// cluster of KS CTAs along K shares one output tile.  Each CTA walks 1/KS of the chunks,
// few enough that all its weight stages are requested before the dependency wait, and the
// CTAs of ranks 1.. write their int32 accumulators into rank 0's shared memory (distributed
// shared memory, then a release-arrive on rank 0's mbarrier); rank 0 adds them to its own
// and runs the epilogue.  Integer sums: the bits do not depend on the split.  (Splitting K
// with integer atomics in global memory was measured at twice the time of an unsplit
// launch and was dropped.)
//
// The first weight stages are requested BEFORE the programmatic-dependency wait: weights
// are never written by a preceding launch, so they can land while it finishes.
//
// Every wait is bounded: if a barrier does not complete within the limit the
// CTA raises a status bit, waits once more for its copies, frees its TMEM and
// returns.
#include "common.cuh"
#include "launch.h"

#include "tma.cuh"
#include "tc_common.cuh"

#include <stdlib.h>
#include <string.h>

namespace {

constexpr int TC_THREADS = 128;
constexpr int TM = 128;             // weight rows per tile (MMA M)
constexpr int BN = 16;              // lanes per tile (MMA N)
constexpr int KC = 128;             // K bytes per stage (one swizzle row)
constexpr int MAX_STAGES = 8;
constexpr int A_BYTES = TM * KC;    // 16 KB
constexpr int B_BYTES = BN * KC;    // 2 KB
constexpr int TMEM_COLS = 32;       // smallest allocation; BN <= 32 columns used

struct TcP {
    const float *scales, *bias, *sx;
    float *out;
    const int *n_active;
    int *status;
    const uint32_t *tanh_tab;
    long n, k, out_stride;
    int batch, epilogue, strict;
    int ksplit;          // CTAs of a cluster that share one output tile along K
};

// NS = stages of the ring (compile time: a run-time count was measured 30 us per step slower).
// Six stages (109 KB) hold all of k = 768 and let two CTAs share an SM: used for grids of
// more CTAs than SMs (the 512-CTA logit-head product), where it halves the waves.
template <bool SPLIT, int NS = MAX_STAGES>
__global__ void __launch_bounds__(TC_THREADS)
k_gemm_i8_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcP p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[MAX_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[MAX_STAGES];
    __shared__ __align__(8) unsigned long long done_bar;
    __shared__ __align__(8) unsigned long long part_bar;     // split K: arrivals of the other ranks
    __shared__ uint32_t s_tmem;
    __shared__ unsigned s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = blockIdx.y * BN;
    const long m0 = (long)blockIdx.x * TM;
    const int all_chunks = (int)((p.k + KC - 1) / KC);
    // split K: this CTA's share of the chunks (the launcher makes them divide evenly)
    const int nks = SPLIT ? p.ksplit : 1;
    const int ks = SPLIT ? (int)cluster_rank() : 0;
    const int nchunks = all_chunks / nks, c_first = ks * nchunks;
    // operands need 1024-byte alignment for the 128-byte swizzle
    unsigned char *base = smem_raw + ((1024u - (saddr(smem_raw) & 1023u)) & 1023u);
    unsigned char *As = base;                               // [stage][128 rows][128 B]
    unsigned char *Bs = base + (size_t)NS * A_BYTES; // [stage][BN rows][128 B]
    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            bar_init(&full_bar[s], 1u);
            bar_init(&empty_bar[s], 1u);
        }
        bar_init(&done_bar, 1u);
        if (SPLIT) bar_init(&part_bar, (unsigned)((nks - 1) * TC_THREADS));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_fail = 0u;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // split K: rank 0's arrival barrier is initialized before any rank can reach it
    if (SPLIT) cluster_sync_all();

    // Weights do not depend on the launches before this one: their first stages are
    // requested before the dependency wait, so they land while the predecessor finishes.
    const unsigned stage_bytes = (unsigned)(A_BYTES + B_BYTES);
    const int first = min(nchunks, NS);             // stages that need no release to fill
    if (warp == 0 && lane == 0) {
        for (int c = 0; c < first; ++c) {
            bar_expect(&full_bar[c], stage_bytes);
            tma_load_2d(As + (size_t)c * A_BYTES, &map_w, (c_first + c) * KC, (int)m0, &full_bar[c]);
        }
    }
    const int nb = min(p.batch, mb_lane_count(p.n_active));
    // the activation map is first used behind the wait: its descriptor is fetched now
    if (warp == 0 && lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    mb_pdl_wait();
    mb_pdl_trigger();
    if (b0 >= nb) {
        // no live lane in this tile: let the requested weight stages land (the activation
        // halves are sent too, so each barrier completes), then give the TMEM back
        if (warp == 0 && lane == 0) {
            for (int c = 0; c < first; ++c) {
                tma_load_2d(Bs + (size_t)c * B_BYTES, &map_x, (c_first + c) * KC, b0, &full_bar[c]);
                bar_wait(&full_bar[c], 0u, TC_SPIN);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 0)
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
        return;
    }
    if (warp == 0 && lane == 0) {
        // the activation halves of the first stages, then the rest of the K walk:
        // chunk c goes to stage c % 8 once the MMAs of chunk c - 8 released it
        for (int c = 0; c < first; ++c) tma_load_2d(Bs + (size_t)c * B_BYTES, &map_x, (c_first + c) * KC, b0, &full_bar[c]);
        for (int c = first; c < nchunks; ++c) {
            const int s = c % NS;
            if (!bar_wait(&empty_bar[s], (unsigned)((c / NS - 1) & 1), TC_SPIN)) {
                s_fail = 1u;
                if (p.status != nullptr) atomicOr(p.status, 8);
                break;
            }
            bar_expect(&full_bar[s], stage_bytes);
            tma_load_2d(As + (size_t)s * A_BYTES, &map_w, (c_first + c) * KC, (int)m0, &full_bar[s]);
            tma_load_2d(Bs + (size_t)s * B_BYTES, &map_x, (c_first + c) * KC, b0, &full_bar[s]);
        }
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = instr_desc_i8(TM, BN);
        for (int c = 0; c < nchunks; ++c) {
            const int s = c % NS;
            if (!bar_wait(&full_bar[s], (unsigned)((c / NS) & 1), TC_SPIN)) {
                s_fail = 1u;
                if (p.status != nullptr) atomicOr(p.status, 8);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = smem_desc_sw128(saddr(As + (size_t)s * A_BYTES));
            const uint64_t db = smem_desc_sw128(saddr(Bs + (size_t)s * B_BYTES));
#pragma unroll
            for (int kk = 0; kk < KC / 32; ++kk)          // 32 K-bytes per instruction: +2 in 16-byte units
                mma_i8(tmem, da + 2u * kk, db + 2u * kk, idesc, (c | kk) != 0 ? 1u : 0u);
            mma_commit(&empty_bar[s]);                       // stage s is free once these MMAs are done
        }
        mma_commit(&done_bar);                               // arrives when every MMA above has finished
    }
    // scale and bias of this thread's row, the lane scales and (residual epilogue) the
    // values to add to, all fetched while the tensor cores work: loads issued one by one
    // between the stores below would each pay a full memory round trip
    const long row = m0 + warp * 32 + lane;
    const bool row_ok = row < p.n;
    const float ws = row_ok ? __ldg(p.scales + row) : 0.0f;
    const float bias = (row_ok && p.bias != nullptr) ? __ldg(p.bias + row) : 0.0f;
    float lane_scale[BN], prior[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) {
        const int b = b0 + j;
        lane_scale[j] = b < nb ? p.sx[b] : 0.0f;
        prior[j] = (p.epilogue == MB_EPI_RESIDUAL && row_ok && b < nb) ? p.out[(long)b * p.out_stride + row] : 0.0f;
    }
    const bool done = bar_wait(&done_bar, 0u, TC_SPIN);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool good = done && s_fail == 0u;
    if (!done && threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, 16);
    if (!good) {
        // a wait ran out: give copies still in flight one more bounded chance to land
        // before this CTA's shared memory is released
        if (threadIdx.x == 0)
            for (int s = 0; s < NS && s < nchunks; ++s) bar_wait(&full_bar[s], 0u, TC_SPIN >> 4);
        if (SPLIT && ks != 0) remote_arrive(remote_saddr(&part_bar, 0u));   // rank 0 need not wait for the limit
    } else {
        int v[16];
        tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16), v);
        bool whole = true;                                   // v holds the sum over all of K
        if (SPLIT) {
            // partial sums of ranks 1.. in rank 0's shared memory: [rank - 1][lane j][weight row]
            int *parts = reinterpret_cast<int *>(Bs + (size_t)NS * B_BYTES);
            if (ks != 0) {
                const unsigned dst = remote_saddr(parts + ((size_t)(ks - 1) * BN) * TM + threadIdx.x, 0u);
#pragma unroll
                for (int j = 0; j < BN; ++j) remote_store(dst + (unsigned)(j * TM * 4), v[j]);
                remote_arrive(remote_saddr(&part_bar, 0u));
                whole = false;
            } else if (bar_wait_cluster(&part_bar, 0u, TC_SPIN)) {
                for (int z = 1; z < nks; ++z)
#pragma unroll
                    for (int j = 0; j < BN; ++j) v[j] += parts[((size_t)(z - 1) * BN + j) * TM + threadIdx.x];
            } else {
                whole = false;
                if (p.status != nullptr) atomicOr(p.status, 16);
            }
        }
        if (row_ok && whole && p.epilogue == MB_EPI_GELU && p.strict) {
            // host-libm GELU: the table words of all lanes are requested before the first
            // double-precision tanh, so the lookups overlap instead of queueing one by one
            float y[BN], c[BN];
            uint32_t word[BN];
#pragma unroll
            for (int j = 0; j < BN; ++j) {
                y[j] = __fmul_rn(__fmul_rn((float)v[j], ws), lane_scale[j]);
                if (p.bias != nullptr) y[j] = __fadd_rn(y[j], bias);
                c[j] = gelu_tanh_arg(y[j]);
                word[j] = b0 + j < nb ? mb_tanh_fetch(c[j], p.tanh_tab) : 0x88888888u;
            }
#pragma unroll
            for (int j = 0; j < BN; ++j)
                if (b0 + j < nb) p.out[(long)(b0 + j) * p.out_stride + row] = gelu_tanh_finish(y[j], c[j], word[j], p.tanh_tab != nullptr);
        } else if (row_ok && whole) {
#pragma unroll
            for (int j = 0; j < BN; ++j) {
                const int b = b0 + j;
                if (b < nb) {
                    float y = __fmul_rn(__fmul_rn((float)v[j], ws), lane_scale[j]);
                    if (p.bias != nullptr) y = __fadd_rn(y, bias);
                    float *dst = p.out + (long)b * p.out_stride + row;
                    if (p.epilogue == MB_EPI_RESIDUAL) *dst = __fadd_rn(prior[j], y);
                    else if (p.epilogue == MB_EPI_GELU) *dst = gelu_tanh<false>(y, nullptr);
                    else *dst = y;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    // split K: rank 0's shared memory stays allocated until every rank is past its stores
    if (SPLIT) cluster_sync_all();
}

// ------------------------------------------------------------------ int4 weights
// The same tile for int4 weights in groups of 32 (src/qmat.c:154-185): per group an exact
// int32 dot, scaled by the group's f32 scale and added up in group order.  A group is one
// K = 32 MMA, so every group gets its own accumulator in tensor memory:
//   * TMA brings [128 rows x 64 packed bytes] of W (128 elements, 4 groups) and
//     [16 lanes x 128 B] of the int8 activations per stage;
//   * the CTA's 512 threads unpack four stages at a time, a quarter of a weight row each:
//     low nibble = even k, minus 8, written as int8 in the 128-byte-swizzled operand
//     layout; one proxy fence and one barrier hand them to the MMA thread;
//   * four MMAs per stage (accumulate off), each into its own 16 columns; the 16 groups of
//     a pass fill the 256 allocated columns, then all threads read them back with
//     tcgen05.ld and fold them into f32 sums, group by group, and the next pass reuses
//     the columns.
// Same bits as the SIMT kernel's int4 path.
constexpr int I4_PASS_CHUNKS = 4;         // stages per pass (4 groups each): 16 accumulators
constexpr int I4_STAGES = 2 * I4_PASS_CHUNKS;   // packed stages in flight: this pass and the next
constexpr int I4_THREADS = 512;
constexpr int P_BYTES = TM * 64;          // packed weights of a stage, 8 KB
constexpr int I4_COLS = 256;              // 16 accumulators of 16 columns

__device__ __forceinline__ void tmem_ld4_nowait(uint32_t taddr, int (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr)
                 : "memory");
}

// Threads: t / 4 is the weight row a thread unpacks (a quarter of a stage's 64 packed bytes
// each).  Tensor memory is read per warp: warp w reaches rows 32 * (w % 4) .. + 31 of the
// tile, and takes lanes (columns) 4 * (w / 4) .. + 3 of every group's accumulator.
// A pass = up to four stages: wait for them, unpack them, one proxy fence and one barrier,
// sixteen MMAs, one commit; then every thread reads its accumulators and the stages are
// refilled for the pass after the next.
__global__ void __launch_bounds__(I4_THREADS)
k_gemm_i4_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcP p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[I4_STAGES];
    __shared__ __align__(8) unsigned long long pass_bar;
    __shared__ uint32_t s_tmem;
    __shared__ unsigned s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = blockIdx.y * BN;
    const long m0 = (long)blockIdx.x * TM;
    const int nchunks = (int)(p.k / KC);                    // k is a multiple of 128 here
    unsigned char *base = smem_raw + ((1024u - (saddr(smem_raw) & 1023u)) & 1023u);
    unsigned char *Ap = base;                                   // [4][128 rows][128 B] unpacked, swizzled
    unsigned char *Bs = Ap + (size_t)I4_PASS_CHUNKS * A_BYTES;  // [stage][16 lanes][128 B] swizzled
    unsigned char *Pk = Bs + (size_t)I4_STAGES * B_BYTES;       // [stage][128 rows][64 B] packed
    if (threadIdx.x == 0) {
        for (int s = 0; s < I4_STAGES; ++s) bar_init(&full_bar[s], 1u);
        bar_init(&pass_bar, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_fail = 0u;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&s_tmem)), "r"(I4_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const unsigned stage_bytes = (unsigned)(P_BYTES + B_BYTES);
    const int first = min(nchunks, I4_STAGES);
    if (threadIdx.x == 0) {                                 // weights: before the dependency wait
        for (int c = 0; c < first; ++c) {
            bar_expect(&full_bar[c], stage_bytes);
            tma_load_2d(Pk + (size_t)c * P_BYTES, &map_w, c * (KC / 2), (int)m0, &full_bar[c]);
        }
    }
    mb_pdl_wait();
    mb_pdl_trigger();
    const int nb = p.n_active != nullptr ? min(p.batch, *p.n_active) : p.batch;
    if (b0 >= nb) {
        if (threadIdx.x == 0) {
            for (int c = 0; c < first; ++c) {
                tma_load_2d(Bs + (size_t)c * B_BYTES, &map_x, c * KC, b0, &full_bar[c]);
                bar_wait(&full_bar[c], 0u, TC_SPIN);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 0)
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(I4_COLS) : "memory");
        return;
    }
    if (threadIdx.x == 0)
        for (int c = 0; c < first; ++c) tma_load_2d(Bs + (size_t)c * B_BYTES, &map_x, c * KC, b0, &full_bar[c]);
    auto wait = [&](void *bar, unsigned parity, int bit) {
        if (*reinterpret_cast<volatile unsigned *>(&s_fail) != 0u) return false;
        if (bar_wait(bar, parity, TC_SPIN)) return true;
        s_fail = 1u;
        if (p.status != nullptr) atomicOr(p.status, bit);
        return false;
    };
    // unpacking role
    const int urow = threadIdx.x >> 2, uq = threadIdx.x & 3, usw = urow & 7;
    // accumulation / epilogue role
    const long row = m0 + (warp & 3) * 32 + lane;
    const int col0 = (warp >> 2) * 4;                       // this thread's 4 lanes of the tile
    const bool row_ok = row < p.n;
    const long groups = p.k / 32;
    const float *gscale = p.scales + (row_ok ? row : 0) * groups;
    const uint32_t idesc = instr_desc_i8(TM, BN);
    const uint32_t tbase = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)col0;
    float accf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int pass = 0;
    for (int p0 = 0; p0 < nchunks; p0 += I4_PASS_CHUNKS, ++pass) {
        const int pend = min(nchunks, p0 + I4_PASS_CHUNKS);
        for (int c = p0; c < pend; ++c) {
            const int s = c % I4_STAGES;
            if (wait(&full_bar[s], (unsigned)((c / I4_STAGES) & 1), 8)) {
                // ---- unpack 16 packed bytes (32 elements) of row urow ----------------------
                const int4 pk = *reinterpret_cast<const int4 *>(Pk + (size_t)s * P_BYTES + (size_t)urow * 64 + uq * 16);
                unsigned char *dstrow = Ap + (size_t)(c - p0) * A_BYTES + (size_t)urow * 128;
                const unsigned w[4] = {(unsigned)pk.x, (unsigned)pk.y, (unsigned)pk.z, (unsigned)pk.w};
                unsigned o[8];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const unsigned lo = w[t] & 0x0f0f0f0fu, hi = (w[t] >> 4) & 0x0f0f0f0fu;
                    o[2 * t] = __vsub4(__byte_perm(lo, hi, 0x5140), 0x08080808u);
                    o[2 * t + 1] = __vsub4(__byte_perm(lo, hi, 0x7362), 0x08080808u);
                }
                *reinterpret_cast<int4 *>(dstrow + (((2 * uq) ^ usw) << 4)) = make_int4((int)o[0], (int)o[1], (int)o[2], (int)o[3]);
                *reinterpret_cast<int4 *>(dstrow + (((2 * uq + 1) ^ usw) << 4)) = make_int4((int)o[4], (int)o[5], (int)o[6], (int)o[7]);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMAs read these bytes
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 32) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (*reinterpret_cast<volatile unsigned *>(&s_fail) == 0u) {
                for (int c = p0; c < pend; ++c) {
                    const uint64_t da = smem_desc_sw128(saddr(Ap + (size_t)(c - p0) * A_BYTES));
                    const uint64_t db = smem_desc_sw128(saddr(Bs + (size_t)(c % I4_STAGES) * B_BYTES));
#pragma unroll
                    for (int g = 0; g < KC / 32; ++g)
                        mma_i8(tmem + (uint32_t)(((c - p0) * (KC / 32) + g) * BN), da + 2u * g, db + 2u * g, idesc, 0u);
                }
            }
            mma_commit(&pass_bar);                           // arrives when every MMA so far has finished
        }
        const bool done = wait(&pass_bar, (unsigned)(pass & 1), 16);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (threadIdx.x == 0 && done) {
            // the pass's stages are free: refill them for the pass after the next
            for (int c = p0; c < pend; ++c) {
                const int cn = c + I4_STAGES;
                if (cn < nchunks) {
                    const int s = c % I4_STAGES;
                    bar_expect(&full_bar[s], stage_bytes);
                    tma_load_2d(Pk + (size_t)s * P_BYTES, &map_w, cn * (KC / 2), (int)m0, &full_bar[s]);
                    tma_load_2d(Bs + (size_t)s * B_BYTES, &map_x, cn * KC, b0, &full_bar[s]);
                }
            }
        }
        if (done) {
            // all of the pass's accumulators for this thread's row and 4 lanes, then one wait;
            // folded into the f32 sums in group order
            const int ngroups = (pend - p0) * (KC / 32);
            int v[I4_PASS_CHUNKS * (KC / 32)][4];
#pragma unroll
            for (int g = 0; g < I4_PASS_CHUNKS * (KC / 32); ++g)
                if (g < ngroups) tmem_ld4_nowait(tbase + (uint32_t)(g * BN), v[g]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row_ok) {
#pragma unroll
                for (int g = 0; g < I4_PASS_CHUNKS * (KC / 32); ++g)
                    if (g < ngroups) {
                        const float gs = gscale[(long)p0 * (KC / 32) + g];
#pragma unroll
                        for (int j = 0; j < 4; ++j) accf[j] = __fadd_rn(accf[j], __fmul_rn((float)v[g][j], gs));
                    }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();                                     // accumulators and the unpacked tiles are free
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    const bool good = *reinterpret_cast<volatile unsigned *>(&s_fail) == 0u;
    if (!good) {
        // a wait ran out: give copies still in flight one more bounded chance to land before
        // this CTA's shared memory is released
        if (threadIdx.x == 0)
            for (int s = 0; s < I4_STAGES && s < nchunks; ++s) bar_wait(&full_bar[s], 0u, TC_SPIN >> 4);
    } else if (row_ok) {
        const float bias = p.bias != nullptr ? __ldg(p.bias + row) : 0.0f;
        float prior[4], lane_scale[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int b = b0 + col0 + j;
            lane_scale[j] = b < nb ? p.sx[b] : 0.0f;
            prior[j] = (p.epilogue == MB_EPI_RESIDUAL && b < nb) ? p.out[(long)b * p.out_stride + row] : 0.0f;
        }
        float y4[4], c4[4];
        uint32_t word4[4];
        const bool gelu_host = p.epilogue == MB_EPI_GELU && p.strict;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            y4[j] = __fmul_rn(accf[j], lane_scale[j]);
            if (p.bias != nullptr) y4[j] = __fadd_rn(y4[j], bias);
            c4[j] = gelu_tanh_arg(y4[j]);
            // the four table words are requested together (see the int8 kernel)
            word4[j] = (gelu_host && b0 + col0 + j < nb) ? mb_tanh_fetch(c4[j], p.tanh_tab) : 0x88888888u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int b = b0 + col0 + j;
            if (b < nb) {
                const float y = y4[j];
                float *dst = p.out + (long)b * p.out_stride + row;
                if (p.epilogue == MB_EPI_RESIDUAL) *dst = __fadd_rn(prior[j], y);
                else if (p.epilogue == MB_EPI_GELU)
                    *dst = p.strict ? gelu_tanh_finish(y, c4[j], word4[j], p.tanh_tab != nullptr) : gelu_tanh<false>(y, nullptr);
                else *dst = y;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(I4_COLS) : "memory");
}

constexpr size_t TC4_SMEM = (size_t)I4_PASS_CHUNKS * A_BYTES + (size_t)I4_STAGES * (B_BYTES + P_BYTES) + 1024;

// [rows][k] bytes, row-major; box = 128 K-bytes x box_rows rows, 128-byte swizzle.
bool make_map(CUtensorMap *map, const void *ptr, size_t rows, size_t k, unsigned box_rows) {
    return mb_make_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, ptr, rows, k, k, (unsigned)KC, box_rows,
                          CU_TENSOR_MAP_SWIZZLE_128B);
}

constexpr size_t TC_SMEM = (size_t)MAX_STAGES * (A_BYTES + B_BYTES) + 1024;
constexpr int KS_MAX = 4;            // most CTAs per cluster along K
constexpr size_t TC_SMEM_SPLIT = TC_SMEM + (size_t)(KS_MAX - 1) * BN * TM * sizeof(int);

}  // namespace

// MYNAH_B200_NO_KSPLIT=1 keeps every product on one CTA per tile (for A/B measurements).
static int mb_gemm_tc_split_enabled() {
    const char *e = getenv("MYNAH_B200_NO_KSPLIT");
    return (e != nullptr && strcmp(e, "0") != 0) ? 0 : 1;
}

extern "C" int mb_gemm_tc_init(void) {
    int rc = (int)cudaFuncSetAttribute(k_gemm_i8_tc<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_gemm_i8_tc<false, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_gemm_i8_tc<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_SPLIT);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_gemm_i4_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC4_SMEM);
    return rc;
}

// Shapes the tensor-core path takes: int8 weights, k a multiple of 16 (TMA row
// stride), 16-byte aligned operands.
extern "C" int mb_gemm_tc_supported(int qtype, size_t n, size_t k, size_t batch) {
    // int4: whole 4-group stages; measured against the SIMT kernel the unpack-and-fold passes
    // pay off from about 48 lanes (64 lanes: 1742 vs 1935 us per step; 32 lanes: 1624 vs 1488)
    if (qtype == MB_INT4) return n > 0 && batch >= 48 && k >= 128 && (k % 128u) == 0;
    return qtype == MB_INT8 && n > 0 && batch >= 16 && k >= 16 && (k % 16u) == 0;
}

// qx_rows_alloc: rows the activation buffer really holds (>= batch), so a lane
// tile never reads past the allocation.
extern "C" int mb_gemm_tc(const mb_gemv_args *a, size_t qx_rows_alloc, int *status, mb_stream stream) {
    if (a == nullptr || !mb_gemm_tc_supported(a->qtype, a->n, a->k, a->batch) || a->qx == nullptr ||
        a->sx == nullptr || a->scales == nullptr || a->out == nullptr ||
        (((uintptr_t)a->w | (uintptr_t)a->qx) & 15u) != 0)
        return (int)cudaErrorInvalidValue;
    CUtensorMap map_w, map_x;
    const bool int4 = a->qtype == MB_INT4;
    // int4: [n][k/2] packed bytes, box = 64 bytes x 128 rows, unswizzled (the threads unpack it)
    const bool w_ok = int4 ? mb_make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->w, a->n, a->k / 2u, a->k / 2u,
                                            (unsigned)(KC / 2), TM, CU_TENSOR_MAP_SWIZZLE_NONE)
                           : make_map(&map_w, a->w, a->n, a->k, TM);
    if (!w_ok || !make_map(&map_x, a->qx, qx_rows_alloc > a->batch ? qx_rows_alloc : a->batch, a->k, BN))
        return (int)cudaErrorInvalidValue;
    TcP p;
    p.scales = a->scales; p.bias = a->bias; p.sx = a->sx; p.out = a->out;
    p.n_active = a->n_active; p.status = status;
    p.tanh_tab = a->tanh_tab;
    p.n = (long)a->n; p.k = (long)a->k; p.out_stride = (long)a->out_stride;
    p.batch = (int)a->batch; p.epilogue = a->epilogue; p.strict = a->strict;
    p.ksplit = 1;
    const unsigned m_tiles = (unsigned)((a->n + TM - 1) / TM);
    const unsigned b_tiles = (unsigned)((a->batch + BN - 1) / BN);
    if (int4)
        mb_launch(k_gemm_i4_tc, dim3(dim3(m_tiles, b_tiles)), dim3(I4_THREADS), TC4_SMEM, (cudaStream_t)stream, map_w, map_x, p);
    else {
        // more chunks than stages: the widest split along K (up to KS_MAX) that lets every CTA
        // request all its weight stages at once, while the whole grid still fits the SMs
        const unsigned chunks = (unsigned)((a->k + KC - 1) / KC);
        unsigned ks = 1;
        if (chunks > (unsigned)MAX_STAGES && (a->k % KC) == 0 && mb_gemm_tc_split_enabled())
            for (unsigned c = (unsigned)KS_MAX; c >= 2 && ks == 1; --c)
                if (chunks % c == 0 && chunks / c <= (unsigned)MAX_STAGES && m_tiles * b_tiles * c <= 132u) ks = c;
        if (ks > 1) {
            p.ksplit = (int)ks;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(m_tiles, b_tiles, ks);
            cfg.blockDim = dim3(TC_THREADS);
            cfg.dynamicSmemBytes = TC_SMEM_SPLIT;
            cfg.stream = (cudaStream_t)stream;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = ks;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = mb_pdl_enabled() ? 2u : 1u;
            const int rc = (int)cudaLaunchKernelEx(&cfg, k_gemm_i8_tc<true>, map_w, map_x, p);
            return rc != 0 ? rc : mb_check_launch();
        }
        if (m_tiles * b_tiles > 148u && chunks <= 6u)
            mb_launch(k_gemm_i8_tc<false, 6>, dim3(dim3(m_tiles, b_tiles)), dim3(TC_THREADS),
                      (size_t)6 * (A_BYTES + B_BYTES) + 1024, (cudaStream_t)stream, map_w, map_x, p);
        else
            mb_launch(k_gemm_i8_tc<false>, dim3(dim3(m_tiles, b_tiles)), dim3(TC_THREADS), TC_SMEM, (cudaStream_t)stream, map_w, map_x, p);
    }
    return mb_check_launch();
}
