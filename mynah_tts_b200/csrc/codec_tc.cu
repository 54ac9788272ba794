// The codec's residual-layer convolutions on the 5th-generation tensor cores (tcgen05,
// kind::f16), fast mode only: strict mode keeps one sequential f32 sum per output sample
// (codec.cu), which no tensor-core accumulation order reproduces.
//
//   out[o][t] = bias[o] + sum_k sum_i W[o][i][k] * x[i][t - (K-1-k) * dilation]
//
// is one accumulation over (tap k, channel chunk) of products  X_k [128 times x 64 channels]
// . W_k^T [64 channels x N output channels]: the tile of X for tap k is the same channel-major
// slab of the activation shifted by the tap's delay, so TMA fetches it at row t0 - delay and
// fills rows before the start of the signal with zeros (the causal padding).  Operands are
// f16, so both sides are split in two halves that add up to the f32 value to about 22 bits,
//   hi = f16(v), lo = f16(v - hi),
// and three MMAs per K step (hi.hi + lo.hi + hi.lo) accumulate in f32 in tensor memory.  The
// weights are scaled by a power of two at pack time so that their lo halves stay normal
// numbers; the epilogue undoes it exactly.
//
// Layouts.  Activations that feed a convolution live as two f16 planes [time][Cp] (channels
// contiguous, Cp = channels rounded up to 64, pad columns zero) written by the producer's
// epilogue (k_conv1d_tc itself, or k_snake_planes at the start of a branch).  Weights:
// [plane][tap][rows = tiles * N][Cp] f16.  Everything else (residual stream, branch sum) stays
// f32 [channels][time] as in codec.cu.
//
// One CTA = 128 times x N output channels (N <= 112, a multiple of 16) through a ring of
// stages of { X hi, X lo: 16 KB each; W hi, W lo: N x 128 B each }, each filled by two TMA
// copies; one thread issues 12 tcgen05.mma (M128 N K16) per stage; sixteen warps (four per 32
// accumulator rows, each a quarter of the columns) read them with tcgen05.ld and run the same epilogue as the SIMT kernel (bias,
// residual, half-Snake copy for the next convolution, branch sum).  Every wait is bounded
// (status bits 8 and 16).
#include "common.cuh"
#include "launch.h"
#include "libm_parity.cuh"

#include "tc_common.cuh"

#include <cuda_fp16.h>
#include <string.h>

namespace {

constexpr int CT_THREADS = 512;            // 16 warps: warp w reads accumulator rows 32 (w % 4) .. +31, column groups w / 4, w / 4 + 4, ..
constexpr int CT_TM = 128;                 // times per tile
constexpr int CT_KC = 128;                 // bytes of channels per stage row: 64 halves
constexpr int CT_A_BYTES = CT_TM * CT_KC;  // one plane of the activation tile
constexpr int CT_MAX_STAGES = 6;

struct ConvTcP {
    const float *bias, *res, *alpha, *alpha2;
    float *out, *acc;
    __half *act_hi, *act_lo;     // planes [L][cp_out] of half-Snake(v), or NULL
    int *status;
    float inv_scale;             // 1 / the power of two the weights were scaled by
    int oc, L, K, dil, n_tile, chunks, stages, cp_out, acc_mode;
};

__device__ __forceinline__ float snake_fast(float v, int c, int snake_ch, const float *alpha) {
    if (c < snake_ch) {
        const float a = alpha[c];
        const float sn = sinf(a * v);
        return v + sn * sn * (1.0f / (a + 1e-9f));
    }
    return v < 0.0f ? v * 0.01f : v;
}

__device__ __forceinline__ void tmem_ld16f(uint32_t taddr, float (&v)[16]) {
    int r[16];
    tmem_ld16(taddr, r);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __int_as_float(r[i]);
}

__global__ void __launch_bounds__(CT_THREADS)
k_conv1d_tc(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, ConvTcP p) {
    extern __shared__ unsigned char smem_ct[];
    __shared__ __align__(8) unsigned long long full_bar[CT_MAX_STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[CT_MAX_STAGES];
    __shared__ __align__(8) unsigned long long done_bar;
    __shared__ uint32_t s_tmem;
    __shared__ unsigned s_fail;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * CT_TM;
    const int ntile = blockIdx.y;
    const int N = p.n_tile;
    const int b_bytes = N * CT_KC;                           // one plane of the weight tile
    const unsigned stage_bytes = (unsigned)(2 * CT_A_BYTES + 2 * b_bytes);
    const int nsteps = p.K * p.chunks;
    const int S = p.stages;
    const uint32_t tmem_cols = N <= 32 ? 32u : (N <= 64 ? 64u : 128u);
    unsigned char *base = smem_ct + ((1024u - (saddr(smem_ct) & 1023u)) & 1023u);
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            bar_init(&full_bar[s], 1u);
            bar_init(&empty_bar[s], 1u);
        }
        bar_init(&done_bar, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_fail = 0u;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&s_tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    mb_pdl_wait();
    mb_pdl_trigger();
    // stage s: [X hi 16 KB][X lo 16 KB][W hi N*128][W lo N*128]
    auto load_step = [&](int c, int s) {
        const int tap = c / p.chunks, chunk = c - tap * p.chunks;
        const int delay = (p.K - 1 - tap) * p.dil;
        unsigned char *dst = base + (size_t)s * stage_bytes;
        bar_expect(&full_bar[s], stage_bytes);
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(saddr(dst)), "l"(&map_x), "r"(chunk * CT_KC), "r"(t0 - delay), "r"(0),
            "r"(saddr(&full_bar[s]))
            : "memory");
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(saddr(dst + 2 * CT_A_BYTES)), "l"(&map_w), "r"(chunk * CT_KC),
            "r"(ntile * N), "r"(tap), "r"(0), "r"(saddr(&full_bar[s]))
            : "memory");
    };
    if (warp == 0 && lane == 0) {
        for (int c = 0; c < nsteps; ++c) {
            const int s = c % S;
            if (c >= S && !bar_wait(&empty_bar[s], (unsigned)((c / S - 1) & 1), TC_SPIN)) {
                s_fail = 1u;
                if (p.status != nullptr) atomicOr(p.status, 8);
                break;
            }
            load_step(c, s);
        }
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = instr_desc_f16(CT_TM, N);
        for (int c = 0; c < nsteps; ++c) {
            const int s = c % S;
            if (!bar_wait(&full_bar[s], (unsigned)((c / S) & 1), TC_SPIN)) {
                s_fail = 1u;
                if (p.status != nullptr) atomicOr(p.status, 8);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char *st = base + (size_t)s * stage_bytes;
            const uint64_t xh = smem_desc_sw128(saddr(st));
            const uint64_t xl = smem_desc_sw128(saddr(st + CT_A_BYTES));
            const uint64_t wh = smem_desc_sw128(saddr(st + 2 * CT_A_BYTES));
            const uint64_t wl = smem_desc_sw128(saddr(st + 2 * CT_A_BYTES + b_bytes));
#pragma unroll
            for (int kk = 0; kk < CT_KC / 32; ++kk) {            // 16 halves = 32 K-bytes per instruction
                mma_f16(tmem, xh + 2u * kk, wh + 2u * kk, idesc, (c | kk) != 0 ? 1u : 0u);
                mma_f16(tmem, xl + 2u * kk, wh + 2u * kk, idesc, 1u);
                mma_f16(tmem, xh + 2u * kk, wl + 2u * kk, idesc, 1u);
            }
            mma_commit(&empty_bar[s]);
        }
        mma_commit(&done_bar);
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
            for (int s = 0; s < S && s < nsteps; ++s) bar_wait(&full_bar[s], 0u, TC_SPIN >> 4);
    } else {
        const int quad = warp & 3;
        const int t = t0 + quad * 32 + lane;
        const bool t_ok = t < p.L;
        const int snake_ch = p.oc / 2;
        for (int g = warp >> 2; g < N / 16; g += CT_THREADS / 128) {
            float v[16];
            tmem_ld16f(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(g * 16), v);
            const int o0 = ntile * N + g * 16;
            // every global read of the group first (the pointers may alias, so the compiler
            // would otherwise keep each read behind the previous column's store)
            float r[16], s[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const bool ok = t_ok && o0 + j < p.oc;
                const size_t at = (size_t)(o0 + j) * p.L + t;
                r[j] = (ok && p.res != nullptr) ? p.res[at] : 0.0f;
                s[j] = (ok && p.acc_mode >= 2) ? p.acc[at] : 0.0f;
            }
            __align__(16) __half hi[16], lo[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int o = o0 + j;
                float a = 0.0f;
                if (o < p.oc && t_ok) {
                    const size_t at = (size_t)o * p.L + t;
                    const float y = r[j] + (v[j] * p.inv_scale + p.bias[o]);
                    if (p.out != nullptr) p.out[at] = y;
                    if (p.alpha != nullptr) a = snake_fast(y, o, snake_ch, p.alpha);
                    if (p.acc_mode == 1) {
                        p.acc[at] = y;
                    } else if (p.acc_mode == 2) {
                        p.acc[at] = s[j] + y;
                    } else if (p.acc_mode == 3) {
                        float s3 = (s[j] + y) / 3.0f;
                        if (p.alpha2 != nullptr) s3 = snake_fast(s3, o, snake_ch, p.alpha2);
                        p.acc[at] = s3;
                    }
                }
                hi[j] = __float2half_rn(a);
                lo[j] = __float2half_rn(a - __half2float(hi[j]));
            }
            if (p.act_hi != nullptr && t_ok && o0 < p.cp_out) {
                uint4 *dh = reinterpret_cast<uint4 *>(p.act_hi + (size_t)t * p.cp_out + o0);
                uint4 *dl = reinterpret_cast<uint4 *>(p.act_lo + (size_t)t * p.cp_out + o0);
                dh[0] = reinterpret_cast<const uint4 *>(hi)[0];
                dh[1] = reinterpret_cast<const uint4 *>(hi)[1];
                dl[0] = reinterpret_cast<const uint4 *>(lo)[0];
                dl[1] = reinterpret_cast<const uint4 *>(lo)[1];
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// f32 [C][L] -> half-Snake -> f16 planes [L][cp] (channels contiguous), through a 32 x 32 tile.
__global__ void __launch_bounds__(256)
k_snake_planes(const float *__restrict__ in, const float *__restrict__ alpha, __half *__restrict__ hi,
               __half *__restrict__ lo, int C, int L, int cp) {
    __shared__ float tile[32][33];
    mb_pdl_wait();
    mb_pdl_trigger();
    const int t0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 8 rows per pass
    for (int r = ty; r < 32; r += 8) {
        const int c = c0 + r, t = t0 + tx;
        tile[r][tx] = (c < C && t < L) ? snake_fast(in[(size_t)c * L + t], c, C / 2, alpha) : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int t = t0 + r, c = c0 + tx;
        if (t < L && c < cp) {
            const float v = tile[tx][r];
            const __half h = __float2half_rn(v);
            hi[(size_t)t * cp + c] = h;
            lo[(size_t)t * cp + c] = __float2half_rn(v - __half2float(h));
        }
    }
}

// [oc][ic][K] f32 -> planes [2][K][rows][cp] f16 of scale * w (zero where no channel).
__global__ void k_pack_conv_weight_tc(const float *__restrict__ w, __half *__restrict__ packed, int oc, int ic, int K,
                                      int rows, int cp, float scale) {
    const size_t plane = (size_t)K * rows * cp;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < plane; idx += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % cp);
        const int o = (int)((idx / cp) % rows);
        const int k = (int)(idx / ((size_t)cp * rows));
        const float v = (o < oc && i < ic) ? w[((size_t)o * ic + i) * K + k] * scale : 0.0f;
        const __half h = __float2half_rn(v);
        packed[idx] = h;
        packed[plane + idx] = __float2half_rn(v - __half2float(h));
    }
}

}  // namespace

extern "C" int mb_codec_tc_init(void) {
    return (int)cudaFuncSetAttribute(k_conv1d_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
}

// Output channels per tile, tiles, and padded channel count of a convolution with `oc` outputs.
extern "C" void mb_codec_tc_shape(size_t oc, size_t *n_tile, size_t *tiles, size_t *cp) {
    const size_t n = oc > 112u ? 112u : (oc + 15u) / 16u * 16u;
    *n_tile = n;
    *tiles = (oc + n - 1u) / n;
    *cp = (oc + 63u) / 64u * 64u;
}

extern "C" size_t mb_codec_tc_packed_halves(size_t oc, size_t ic, size_t kernel) {
    size_t n, tiles, cp_o, cp_i;
    mb_codec_tc_shape(oc, &n, &tiles, &cp_o);
    cp_i = (ic + 63u) / 64u * 64u;
    return 2u * kernel * tiles * n * cp_i;
}

extern "C" int mb_codec_tc_pack_weight(const float *w, void *packed, size_t oc, size_t ic, size_t kernel, float scale,
                                       mb_stream stream) {
    size_t n, tiles, cp_o;
    mb_codec_tc_shape(oc, &n, &tiles, &cp_o);
    const size_t cp_i = (ic + 63u) / 64u * 64u;
    k_pack_conv_weight_tc<<<512, 256, 0, (cudaStream_t)stream>>>(w, static_cast<__half *>(packed), (int)oc, (int)ic, (int)kernel,
                                                                 (int)(tiles * n), (int)cp_i, scale);
    return mb_check_launch();
}

extern "C" int mb_codec_snake_planes(const float *in, const float *alpha, void *hi, void *lo, size_t channels, size_t length,
                                     mb_stream stream) {
    if (channels == 0 || length == 0) return (int)cudaErrorInvalidValue;
    const size_t cp = (channels + 63u) / 64u * 64u;
    mb_launch(k_snake_planes, dim3((unsigned)((length + 31u) / 32u), (unsigned)(cp / 32u)), dim3(256), 0, (cudaStream_t)stream, in,
              alpha, static_cast<__half *>(hi), static_cast<__half *>(lo), (int)channels, (int)length, (int)cp);
    return mb_check_launch();
}

extern "C" int mb_codec_conv1d_tc(const mb_codec_conv_tc_args *a, mb_stream stream) {
    if (a == nullptr || a->x_planes == nullptr || a->w_packed == nullptr || a->bias == nullptr || a->ic == 0 || a->oc == 0 ||
        a->length == 0 || a->kernel == 0 || a->dilation == 0 || (a->alpha != nullptr && a->act_planes == nullptr) ||
        (a->acc_mode != 0 && a->acc == nullptr) || a->scale <= 0.0f ||
        (((uintptr_t)a->x_planes | (uintptr_t)a->w_packed | (uintptr_t)a->act_planes) & 15u) != 0)
        return (int)cudaErrorInvalidValue;
    size_t n, tiles, cp_o;
    mb_codec_tc_shape(a->oc, &n, &tiles, &cp_o);
    const size_t cp_i = (a->ic + 63u) / 64u * 64u, L = a->length, rows = tiles * n;
    CUtensorMap map_x, map_w;
    // activations: (channel bytes, time, plane); box 128 B x 128 times x both planes
    const size_t xdims[3] = {cp_i * 2u, L, 2u};
    const size_t xstrides[2] = {cp_i * 2u, a->x_plane_stride * 2u};
    const unsigned xbox[3] = {(unsigned)CT_KC, (unsigned)CT_TM, 2u};
    // weights: (channel bytes, output row, tap, plane); box 128 B x N rows x 1 tap x both planes
    const size_t wdims[4] = {cp_i * 2u, rows, a->kernel, 2u};
    const size_t wstrides[3] = {cp_i * 2u, rows * cp_i * 2u, a->kernel * rows * cp_i * 2u};
    const unsigned wbox[4] = {(unsigned)CT_KC, (unsigned)n, 1u, 2u};
    if (!mb_make_map_nd(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->x_planes, 3, xdims, xstrides, xbox, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !mb_make_map_nd(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->w_packed, 4, wdims, wstrides, wbox, CU_TENSOR_MAP_SWIZZLE_128B))
        return (int)cudaErrorInvalidValue;
    ConvTcP p;
    memset(&p, 0, sizeof(p));
    p.bias = a->bias; p.res = a->res; p.alpha = a->alpha; p.alpha2 = a->alpha2; p.out = a->out; p.acc = a->acc;
    p.act_hi = static_cast<__half *>(a->act_planes);
    p.act_lo = p.act_hi != nullptr ? p.act_hi + a->act_plane_stride : nullptr;
    p.status = a->status;
    p.inv_scale = 1.0f / a->scale;
    p.oc = (int)a->oc; p.L = (int)L; p.K = (int)a->kernel; p.dil = (int)a->dilation; p.n_tile = (int)n;
    p.chunks = (int)(cp_i / 64u);
    p.cp_out = (int)cp_o;
    p.acc_mode = a->acc_mode;
    const size_t stage_bytes = 2u * CT_A_BYTES + 2u * n * CT_KC;
    size_t stages = (224u * 1024u) / stage_bytes;
    if (stages > CT_MAX_STAGES) stages = CT_MAX_STAGES;
    const size_t steps = a->kernel * (cp_i / 64u);
    if (stages > steps) stages = steps;
    if (stages < 1) return (int)cudaErrorInvalidValue;
    p.stages = (int)stages;
    const size_t smem = stages * stage_bytes + 1024u;
    mb_launch(k_conv1d_tc, dim3((unsigned)((L + CT_TM - 1) / CT_TM), (unsigned)tiles), dim3(CT_THREADS), smem, (cudaStream_t)stream,
              map_x, map_w, p);
    return mb_check_launch();
}
