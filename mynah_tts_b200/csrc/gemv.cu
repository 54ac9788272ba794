// Quantized matrix-vector products of the decode step (SIMT path, batch-generic):
//   out[b][r] = epilogue( dot(W[r,:], act[b,:]) * scales + bias )
// for int8 per-row weights, int4 group-of-32 weights, f16 and f32 weights, in
// the byte layouts the reference's quantizers produce.
//
// Numerics (reference: src/qmat.c:136-185, 191-304, 319-377):
//   int8  the int32 sum is exact, so any summation order gives the reference's
//         bits; then (float)s * ws * sx (+ bias), each product rounded to f32.
//   int4  per group an exact int32 sum; the f32 accumulation over groups runs in
//         group order exactly as the reference's scalar kernel, so the result
//         is bit-identical given the same quantized activation.
//   f16/f32  tree reduction with fused multiply-adds: agrees with the reference
//         to rounding error only (its own tolerance for these modes is 1e-3).
//
// Work split: a row's packed bytes are cut into 16-byte chunks; LPR lanes
// (a power of two dividing the chunk count) share one row, so every warp-wide
// load instruction reads whole contiguous 16-byte pieces of 32/LPR consecutive
// rows.  Activations of a tile of BT streams are staged in shared memory once
// per CTA; batch tiles are spread over grid.z (the weight stream is read once per
// tile, from L2 after the first).
#include <float.h>

#include "common.cuh"
#include "launch.h"

#include <cuda_fp16.h>

#include <type_traits>

namespace {

constexpr int WARPS = 4;
constexpr int MAX_PRELOAD = 6;

struct GemvP {
    const unsigned char *w;
    const float *scales;
    const float *bias;
    const int8_t *qx;
    const float *sx;
    const float *x;
    float *out;
    const int *n_active;
    const uint32_t *tanh_tab;
    long n, k;
    long out_stride;
    int batch;
    int epilogue;
    int lpr, cpl;       // lanes per row, 16-byte chunks per lane
    int iters;          // consecutive row groups one warp walks
    long row_bytes;
    long w_gs, scale_gs, act_gs, out_gs;  // group strides (elements of the respective arrays)
    int fuse;                             // MB_FUSE_*: make the activations from the f32 row fx
    const float *fx, *fuse_gain;
    float fuse_eps;
};

template <bool STRICT>
__device__ __forceinline__ void store_out(const GemvP &p, float *out, long row, int b, float v) {
    float *dst = out + (long)b * p.out_stride + row;
    if (p.epilogue == MB_EPI_RESIDUAL) *dst = __fadd_rn(*dst, v);
    else if (p.epilogue == MB_EPI_GELU) *dst = gelu_tanh<STRICT>(v, p.tanh_tab);
    else *dst = v;
}

__device__ __forceinline__ uint4 ldg16(const unsigned char *ptr) {
    return __ldg(reinterpret_cast<const uint4 *>(ptr));
}
// The same load, kept where the source puts it (the compiler may otherwise sink a read-only
// load to its first use, behind the dependency wait).
__device__ __forceinline__ uint4 ldg16_pinned(const unsigned char *ptr) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

// EARLY (int8, one row group per warp): the first weight pieces are requested before the
// dependency wait.  A kernel of its own: the extra registers would cost the streaming form
// two resident CTAs per SM.
template <int QT, int BT, bool STRICT, bool EARLY>
__global__ void __launch_bounds__(WARPS * 32) k_gemv(GemvP p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long grp = blockIdx.y;
    const unsigned char *w = p.w + grp * p.w_gs;
    const float *scales = p.scales == nullptr ? nullptr : p.scales + grp * p.scale_gs;
    float *out = p.out + grp * p.out_gs;
    const int LPR = p.lpr, CPL = p.cpl, RPW = 32 / LPR;
    const int sub = lane / LPR, li = lane % LPR;
    const long k = p.k;
    constexpr bool QUANT = (QT == MB_INT8 || QT == MB_INT4);
    const long act_bytes = QUANT ? k : k * 4;
    unsigned char *act = smem;                         // [BT][act_bytes]
    float *pbuf = reinterpret_cast<float *>(smem + (size_t)BT * act_bytes);  // int4 only

    __shared__ float fuse_red[96];
    __shared__ float fuse_sx;
    __shared__ float fuse_stat[2];
    // Constants are requested before the dependency wait, so they land while the preceding
    // launch finishes: this warp's first weight pieces (int8) and the fused norm's gain.
    uint4 wpre[MAX_PRELOAD];
    constexpr bool early_weights = EARLY && QT == MB_INT8;
    if (early_weights) {
        const long row0 = (((long)blockIdx.x * p.iters) * WARPS + warp) * RPW + sub;
        const unsigned char *wrow0 = w + (row0 < p.n ? row0 : 0) * p.row_bytes;
#pragma unroll
        for (int u = 0; u < MAX_PRELOAD; ++u)
            if (u < CPL) wpre[u] = ldg16_pinned(wrow0 + (long)(li + u * LPR) * 16);
    }
    float *fuse_gain_s = reinterpret_cast<float *>(smem + ((act_bytes + 15) & ~(long)15)) + k;
    if (QT == MB_INT8 && BT == 1 && p.fuse == MB_FUSE_LN)
        for (int i = threadIdx.x; i < k; i += blockDim.x) fuse_gain_s[i] = __ldg(p.fuse_gain + i);
    const int nb = min(p.batch, mb_lane_count(p.n_active));
    mb_pdl_wait();
    mb_pdl_trigger();
    // one batch tile per CTA (grid.z): tiles past the live lanes leave at once
    for (int b0 = blockIdx.z * BT; b0 < nb; b0 = nb) {
        // ---- stage the activation tile ------------------------------------
        if (QT == MB_INT8 && BT == 1 && p.fuse != MB_FUSE_NONE) {
            // one lane: this CTA makes the quantized row itself from the f32 row (loads of a
            // batch before its stores), with the routines the stand-alone kernels use
            float *rowf = reinterpret_cast<float *>(smem + ((act_bytes + 15) & ~(long)15));
            for (int base = threadIdx.x; base < k; base += blockDim.x * 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = base + u * blockDim.x;
                    if (i < k) v[u] = p.fx[i];
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = base + u * blockDim.x;
                    if (i < k) rowf[i] = v[u];
                }
            }
            __syncthreads();
            // (strict: the reference's sequential sums, squares behind the gain; the plain
            // quantization is exact in either mode)
            const float sxv = p.fuse == MB_FUSE_LN
                                  ? (STRICT ? mb_ln_block_strict(rowf, (int)k, fuse_gain_s, nullptr, p.fuse_eps, fuse_gain_s + k,
                                                                 fuse_stat, fuse_red, nullptr, true, reinterpret_cast<int8_t *>(act))
                                            : mb_ln_block<2>(rowf, (int)k, fuse_gain_s, nullptr, p.fuse_eps, fuse_red, nullptr, true,
                                                             reinterpret_cast<int8_t *>(act)))
                                  : mb_quant_block(rowf, (int)k, fuse_red, reinterpret_cast<int8_t *>(act));
            if (threadIdx.x == 0) fuse_sx = sxv;
        } else if (QUANT) {
            const int8_t *src = p.qx + grp * p.act_gs;
            if (QT == MB_INT8) {
                const int per = (int)(k / 16);
                for (int i = threadIdx.x; i < BT * per; i += blockDim.x) {
                    const int b = i / per, c = i % per;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (b0 + b < nb)
                        v = *reinterpret_cast<const uint4 *>(src + (long)(b0 + b) * k + c * 16);
                    reinterpret_cast<uint4 *>(act)[(long)b * per + c] = v;
                }
            } else {
                // de-interleave each 8-byte span into (even bytes, odd bytes): a packed
                // int4 word holds its even-index weights in the low nibbles.
                const int per = (int)(k / 8);
                for (int i = threadIdx.x; i < BT * per; i += blockDim.x) {
                    const int b = i / per, c = i % per;
                    uint2 v = make_uint2(0, 0);
                    if (b0 + b < nb)
                        v = *reinterpret_cast<const uint2 *>(src + (long)(b0 + b) * k + c * 8);
                    const uint2 o = make_uint2(__byte_perm(v.x, v.y, 0x6420),
                                               __byte_perm(v.x, v.y, 0x7531));
                    reinterpret_cast<uint2 *>(act)[(long)b * per + c] = o;
                }
            }
        } else {
            const float *src = p.x + grp * p.act_gs;
            const int per = (int)(k / 4);
            for (int i = threadIdx.x; i < BT * per; i += blockDim.x) {
                const int b = i / per, c = i % per;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (b0 + b < nb)
                    v = *reinterpret_cast<const float4 *>(src + (long)(b0 + b) * k + c * 4);
                reinterpret_cast<float4 *>(act)[(long)b * per + c] = v;
            }
        }
        __syncthreads();

        // ---- dot products: a warp walks `iters` row groups; the unrolled loop keeps
        // the weight loads of two groups in flight -------------------------------
        // PRE: the first weight pieces were requested before the dependency wait (a launch
        // whose warps walk one row group each: latency bound; a streaming launch keeps the
        // plain loop, whose loads of two groups overlap)
        auto row_group = [&](int it, auto PRE) {
        const long wgroup = ((long)blockIdx.x * p.iters + it) * WARPS + warp;
        const long row = wgroup * RPW + sub;
        const bool row_ok = row < p.n;
        const unsigned char *wrow = w + (row_ok ? row : 0) * p.row_bytes;
        if (QT == MB_INT8) {
            int acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0;
            if (row_ok) {
                for (int i0 = 0; i0 < CPL; i0 += MAX_PRELOAD) {
                    uint4 wv[MAX_PRELOAD];
#pragma unroll
                    for (int u = 0; u < MAX_PRELOAD; ++u) {
                        if (i0 + u < CPL) {
                            if (decltype(PRE)::value && i0 == 0) wv[u] = wpre[u];
                            else wv[u] = ldg16(wrow + (long)(li + (i0 + u) * LPR) * 16);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < MAX_PRELOAD; ++u) {
                        if (i0 + u < CPL) {
                            const int c = li + (i0 + u) * LPR;
#pragma unroll
                            for (int b = 0; b < BT; ++b) {
                                const uint4 xv = reinterpret_cast<const uint4 *>(act + (long)b * k)[c];
                                int a = acc[b];
                                a = __dp4a((int)wv[u].x, (int)xv.x, a);
                                a = __dp4a((int)wv[u].y, (int)xv.y, a);
                                a = __dp4a((int)wv[u].z, (int)xv.z, a);
                                a = __dp4a((int)wv[u].w, (int)xv.w, a);
                                acc[b] = a;
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < BT; ++b)
                for (int o = LPR >> 1; o > 0; o >>= 1) acc[b] += __shfl_xor_sync(MB_FULL, acc[b], o);
            if (row_ok && li == 0) {
                const float ws = scales[row];
                const float bias = p.bias == nullptr ? 0.0f : p.bias[row];
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    if (b0 + b < nb) {
                        const float lane_sx = (BT == 1 && p.fuse != MB_FUSE_NONE) ? fuse_sx : p.sx[grp * p.batch + b0 + b];
                        float v = __fmul_rn(__fmul_rn((float)acc[b], ws), lane_sx);
                        if (p.bias != nullptr) v = __fadd_rn(v, bias);
                        store_out<STRICT>(p, out, row, b0 + b, v);
                    }
                }
            }
        } else if (QT == MB_INT4) {
            const long groups = k / 32;
            float *wp = pbuf + (size_t)warp * 32 * CPL * BT;   // [RPW][groups][BT]
            if (row_ok) {
                for (int i0 = 0; i0 < CPL; i0 += MAX_PRELOAD) {
                    uint4 wv[MAX_PRELOAD];
#pragma unroll
                    for (int u = 0; u < MAX_PRELOAD; ++u)
                        if (i0 + u < CPL) wv[u] = ldg16(wrow + (long)(li + (i0 + u) * LPR) * 16);
#pragma unroll
                    for (int u = 0; u < MAX_PRELOAD; ++u) {
                        if (i0 + u < CPL) {
                            const int g = li + (i0 + u) * LPR;   // chunk index == group index
                            const float gs = scales[row * groups + g];
                            const unsigned ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                            int lo[4], hi[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                lo[j] = (int)__vsub4(ww[j] & 0x0f0f0f0fu, 0x08080808u);
                                hi[j] = (int)__vsub4((ww[j] >> 4) & 0x0f0f0f0fu, 0x08080808u);
                            }
#pragma unroll
                            for (int b = 0; b < BT; ++b) {
                                const uint4 *xp = reinterpret_cast<const uint4 *>(act + (long)b * k) + 2 * g;
                                const uint4 x0 = xp[0], x1 = xp[1];
                                int gi = 0;
                                gi = __dp4a(lo[0], (int)x0.x, gi);
                                gi = __dp4a(hi[0], (int)x0.y, gi);
                                gi = __dp4a(lo[1], (int)x0.z, gi);
                                gi = __dp4a(hi[1], (int)x0.w, gi);
                                gi = __dp4a(lo[2], (int)x1.x, gi);
                                gi = __dp4a(hi[2], (int)x1.y, gi);
                                gi = __dp4a(lo[3], (int)x1.z, gi);
                                gi = __dp4a(hi[3], (int)x1.w, gi);
                                wp[((long)sub * groups + g) * BT + b] = __fmul_rn((float)gi, gs);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            // ordered accumulation over groups, one (row, stream) pair per lane
            for (int j = lane; j < RPW * BT; j += 32) {
                const int r = j / BT, b = j % BT;
                const long orow = wgroup * RPW + r;
                if (orow < p.n && b0 + b < nb) {
                    float a = 0.0f;
                    for (long g = 0; g < groups; ++g) a = __fadd_rn(a, wp[((long)r * groups + g) * BT + b]);
                    float v = __fmul_rn(a, p.sx[grp * p.batch + b0 + b]);
                    if (p.bias != nullptr) v = __fadd_rn(v, p.bias[orow]);
                    store_out<STRICT>(p, out, orow, b0 + b, v);
                }
            }
            __syncwarp();
        } else {
            float acc[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[b] = 0.0f;
            if (row_ok) {
                for (int i0 = 0; i0 < CPL; i0 += MAX_PRELOAD) {
                    uint4 wv[MAX_PRELOAD];
#pragma unroll
                    for (int u = 0; u < MAX_PRELOAD; ++u)
                        if (i0 + u < CPL) wv[u] = ldg16(wrow + (long)(li + (i0 + u) * LPR) * 16);
#pragma unroll
                    for (int u = 0; u < MAX_PRELOAD; ++u) {
                        if (i0 + u < CPL) {
                            const int c = li + (i0 + u) * LPR;
                            if (QT == MB_F16) {
                                const __half2 *h = reinterpret_cast<const __half2 *>(&wv[u]);
                                const float2 w0 = __half22float2(h[0]), w1 = __half22float2(h[1]);
                                const float2 w2 = __half22float2(h[2]), w3 = __half22float2(h[3]);
#pragma unroll
                                for (int b = 0; b < BT; ++b) {
                                    const float4 *xp = reinterpret_cast<const float4 *>(act + (long)b * k * 4) + 2 * c;
                                    const float4 xa = xp[0], xb = xp[1];
                                    float a = acc[b];
                                    a = fmaf(w0.x, xa.x, a); a = fmaf(w0.y, xa.y, a);
                                    a = fmaf(w1.x, xa.z, a); a = fmaf(w1.y, xa.w, a);
                                    a = fmaf(w2.x, xb.x, a); a = fmaf(w2.y, xb.y, a);
                                    a = fmaf(w3.x, xb.z, a); a = fmaf(w3.y, xb.w, a);
                                    acc[b] = a;
                                }
                            } else {
                                const float4 wf = *reinterpret_cast<const float4 *>(&wv[u]);
#pragma unroll
                                for (int b = 0; b < BT; ++b) {
                                    const float4 xa = reinterpret_cast<const float4 *>(act + (long)b * k * 4)[c];
                                    float a = acc[b];
                                    a = fmaf(wf.x, xa.x, a); a = fmaf(wf.y, xa.y, a);
                                    a = fmaf(wf.z, xa.z, a); a = fmaf(wf.w, xa.w, a);
                                    acc[b] = a;
                                }
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < BT; ++b)
                for (int o = LPR >> 1; o > 0; o >>= 1) acc[b] += __shfl_xor_sync(MB_FULL, acc[b], o);
            if (row_ok && li == 0) {
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    if (b0 + b < nb) {
                        float v = acc[b];
                        if (p.bias != nullptr) v = __fadd_rn(v, p.bias[row]);
                        store_out<STRICT>(p, out, row, b0 + b, v);
                    }
                }
            }
        }
        };   // row_group
        if (early_weights) {
            row_group(0, std::true_type{});   // the launcher gives this form iters == 1
        } else {
#pragma unroll 2
            for (int it = 0; it < p.iters; ++it) row_group(it, std::false_type{});
        }
    }
}

// Shapes whose packed rows are not a whole number of 16-byte chunks: one thread
// per (row, stream), sequential over k.  Cold path (tiny self-test shapes).
template <int QT, bool STRICT>
__global__ void k_gemv_generic(GemvP p) {
    mb_pdl_wait();
    mb_pdl_trigger();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int nb = p.n_active != nullptr ? min(p.batch, *p.n_active) : p.batch;
    const long row = idx % p.n;
    const int b = (int)(idx / p.n);
    if (b >= nb) return;
    const long k = p.k;
    float v;
    if (QT == MB_INT8) {
        const int8_t *w = reinterpret_cast<const int8_t *>(p.w) + row * k;
        const int8_t *q = p.qx + (long)b * k;
        int s = 0;
        for (long j = 0; j < k; ++j) s += (int)w[j] * (int)q[j];
        v = __fmul_rn(__fmul_rn((float)s, p.scales[row]), p.sx[b]);
    } else if (QT == MB_INT4) {
        const unsigned char *w = p.w + row * (k / 2);
        const int8_t *q = p.qx + (long)b * k;
        float a = 0.0f;
        for (long g = 0; g < k / 32; ++g) {
            int gi = 0;
            for (int j = 0; j < 32; j += 2) {
                const unsigned char byte = w[g * 16 + j / 2];
                gi += ((int)(byte & 0x0f) - 8) * (int)q[g * 32 + j] +
                      ((int)(byte >> 4) - 8) * (int)q[g * 32 + j + 1];
            }
            a = __fadd_rn(a, __fmul_rn((float)gi, p.scales[row * (k / 32) + g]));
        }
        v = __fmul_rn(a, p.sx[b]);
    } else if (QT == MB_F16) {
        const __half *w = reinterpret_cast<const __half *>(p.w) + row * k;
        const float *x = p.x + (long)b * k;
        float a = 0.0f;
        for (long j = 0; j < k; ++j) a = fmaf(__half2float(w[j]), x[j], a);
        v = a;
    } else {
        const float *w = reinterpret_cast<const float *>(p.w) + row * k;
        const float *x = p.x + (long)b * k;
        float a = 0.0f;
        for (long j = 0; j < k; ++j) a = __fadd_rn(a, __fmul_rn(w[j], x[j]));
        v = a;
    }
    if (p.bias != nullptr) v = __fadd_rn(v, p.bias[row]);
    store_out<STRICT>(p, p.out, row, b, v);
}

template <int QT, int BT, bool STRICT>
int launch_tiled(const GemvP &p, size_t groups, cudaStream_t s) {
    const int rpw = 32 / p.lpr;
    const long wgroups = (p.n + rpw - 1) / rpw;
    const long blocks1 = (wgroups + WARPS - 1) / WARPS;
    const long btiles = (p.batch + BT - 1) / BT;
    // enough CTAs to cover the SMs about four times; beyond that a warp walks several
    // row groups so a CTA moves tens of KB instead of a few
    long it = blocks1 * (long)groups * btiles / 600;
    it = it < 1 ? 1 : (it > 8 ? 8 : it);
    GemvP q = p;
    q.iters = (int)it;
    const unsigned blocks = (unsigned)((blocks1 + it - 1) / it);
    const bool quant = (QT == MB_INT8 || QT == MB_INT4);
    size_t smem = (size_t)BT * (quant ? p.k : p.k * 4);
    if (QT == MB_INT4) smem += (size_t)WARPS * 32 * p.cpl * BT * sizeof(float);
    if (p.fuse != MB_FUSE_NONE) smem += 16u + (STRICT ? 3u : 2u) * (size_t)p.k * sizeof(float);   /* the f32 row, the gain, (strict) the squares */
    if (smem > 160u * 1024u) return (int)cudaErrorInvalidValue;
    if (QT == MB_INT8 && it == 1)
        mb_launch(k_gemv<QT, BT, STRICT, QT == MB_INT8>, dim3(blocks, (unsigned)groups, (unsigned)btiles), dim3(WARPS * 32), smem, s, q);
    else
        mb_launch(k_gemv<QT, BT, STRICT, false>, dim3(blocks, (unsigned)groups, (unsigned)btiles), dim3(WARPS * 32), smem, s, q);
    return mb_check_launch();
}

// Strict f32 product at streaming speed: out[b][r] = ((w[r][0]*x[b][0] + w[r][1]*x[b][1]) + ...)
// with every product and sum rounded, in index order -- the reference's scalar build
// (src/backend.c:283-291, src/kernels.c:40-44).  The order binds each output's own sum, not
// how the weights reach the threads: a CTA owns 32 weight rows and up to 4 lanes; the rows'
// next 64 floats are fetched by all 128 threads with coalesced 16-byte loads into registers
// while the chains run over the current 64 (shared memory, row pitch 65 so that the 32 rows
// a warp reads fall into 32 banks), sixteen values staged in registers ahead of their adds.
constexpr int SEQ_ROWS = 32, SEQ_LANES = 4, SEQ_KC = 64, SEQ_PITCH = SEQ_KC + 1;

// ARGMAX: the rows are the logit heads ([tables * vocab][k]) and nothing is stored: the
// constrained first-on-ties pick of every (stream, table) is made on the fly, the fused
// projection + argmax of the reference's f32 greedy path (mynah_qmat_greedy_argmax,
// src/qmat.c:453-536; serial kernel src/kernels.c:116-139).  A warp holds 32 consecutive
// vocabulary entries of one stream: it reduces them to one candidate, and the last of the
// table's vocab / 32 warps to arrive (a counter per stream and table) reduces the candidates
// in index order.
struct SeqArgmaxP {
    int vocab, codebook_size, eos_id, tables;
    const int *allow_eos;
    float *cand_v;            // [batch][tables][vocab / 32]
    unsigned *cand_i;
    unsigned *counters;       // [batch][tables], zero between launches
    unsigned *tokens, *codes; // [batch][tables]
    int *eos_flag;            // [batch]
};

__device__ __forceinline__ void seq_better(float &v, unsigned &i, float ov, unsigned oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

template <bool ARGMAX>
__global__ void __launch_bounds__(SEQ_ROWS * SEQ_LANES) k_gemv_f32_seq(GemvP p, SeqArgmaxP q) {
    __shared__ float ws[SEQ_ROWS * SEQ_PITCH];
    __shared__ __align__(16) float xs[SEQ_LANES * SEQ_KC];
    const int nb = min(p.batch, mb_lane_count(p.n_active));
    mb_pdl_wait();
    mb_pdl_trigger();
    const int b0 = blockIdx.y * SEQ_LANES;
    if (b0 >= nb) return;
    const long r0 = (long)blockIdx.x * SEQ_ROWS;
    const int tid = threadIdx.x, r = tid % SEQ_ROWS, lb = tid / SEQ_ROWS;
    const long k = p.k;
    const float *w = reinterpret_cast<const float *>(p.w);
    const int nchunks = (int)((k + SEQ_KC - 1) / SEQ_KC);
    // this thread's share of a weight chunk: 32 rows x 16 pieces of 16 bytes = 512 pieces, 4 each
    float4 wreg[4], xreg;
    auto fetch = [&](int c) {
        const long k0 = (long)c * SEQ_KC;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + u * SEQ_ROWS * SEQ_LANES, rr = i >> 4, pc = i & 15;
            const long row = r0 + rr, col = k0 + 4 * pc;
            wreg[u] = (row < p.n && col < k) ? __ldg(reinterpret_cast<const float4 *>(w + row * k + col))
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // activations of the CTA's lanes: 4 lanes x 16 pieces = 64 pieces, threads 0..63
        xreg = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tid < SEQ_LANES * 16) {
            const int l = tid >> 4, pc = tid & 15;
            const long col = k0 + 4 * pc;
            if (b0 + l < nb && col < k) xreg = *reinterpret_cast<const float4 *>(p.x + (long)(b0 + l) * k + col);
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + u * SEQ_ROWS * SEQ_LANES, rr = i >> 4, pc = i & 15;
            float *dst = ws + rr * SEQ_PITCH + 4 * pc;
            dst[0] = wreg[u].x; dst[1] = wreg[u].y; dst[2] = wreg[u].z; dst[3] = wreg[u].w;
        }
        if (tid < SEQ_LANES * 16) *reinterpret_cast<float4 *>(xs + 4 * tid) = xreg;
    };
    fetch(0);
    stash();
    __syncthreads();
    float a = 0.0f;
    const bool mine = r0 + r < p.n && b0 + lb < nb;
    for (int c = 0; c < nchunks; ++c) {
        if (c + 1 < nchunks) fetch(c + 1);              // in flight while the chains run
        const int len = (int)min((long)SEQ_KC, k - (long)c * SEQ_KC);
        if (mine) {
            const float *wr = ws + r * SEQ_PITCH;
            const float *xr = xs + lb * SEQ_KC;
            for (int j0 = 0; j0 < len; j0 += 16) {
                float wv[16], xv[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) wv[j] = wr[j0 + j];
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                    const float4 t = *reinterpret_cast<const float4 *>(xr + j0 + 4 * j4);
                    xv[4 * j4] = t.x; xv[4 * j4 + 1] = t.y; xv[4 * j4 + 2] = t.z; xv[4 * j4 + 3] = t.w;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (j0 + j < len) a = __fadd_rn(a, __fmul_rn(wv[j], xv[j]));
            }
        }
        __syncthreads();
        if (c + 1 < nchunks) {
            stash();
            __syncthreads();
        }
    }
    if (ARGMAX) {
        // warp lb = stream b0 + lb, lane r = vocabulary entry (r0 + r) % vocab of table (r0 + r) / vocab
        const int b = b0 + lb;
        if (b >= nb) return;                               // whole warp
        const long row = r0 + r;
        const int table = (int)(r0 / q.vocab), chunk = (int)((r0 % q.vocab) / SEQ_ROWS), nchunk = q.vocab / SEQ_ROWS;
        const int idx = (int)(row % q.vocab);
        const int allow = q.allow_eos != nullptr ? q.allow_eos[b] : 0;
        float v = -FLT_MAX;
        unsigned vi = 0xffffffffu;
        if (row < p.n && (idx < q.codebook_size || (allow && idx == q.eos_id))) {
            float y = a;
            if (p.bias != nullptr) y = __fadd_rn(y, p.bias[row]);
            if (y > -FLT_MAX) { v = y; vi = (unsigned)idx; }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1)
            seq_better(v, vi, __shfl_xor_sync(MB_FULL, v, m), __shfl_xor_sync(MB_FULL, vi, m));
        const size_t slot = ((size_t)b * q.tables + table);
        unsigned ticket = 0;
        if (r == 0) {
            q.cand_v[slot * nchunk + chunk] = v;
            q.cand_i[slot * nchunk + chunk] = vi;
            __threadfence();
            ticket = atomicAdd(q.counters + slot, 1u);
        }
        ticket = __shfl_sync(MB_FULL, ticket, 0);
        if (ticket != (unsigned)(nchunk - 1)) return;
        __threadfence();
        v = -FLT_MAX;
        vi = 0xffffffffu;
        for (int c = r; c < nchunk; c += 32)
            seq_better(v, vi, __ldcg(q.cand_v + slot * nchunk + c), __ldcg(q.cand_i + slot * nchunk + c));
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1)
            seq_better(v, vi, __shfl_xor_sync(MB_FULL, v, m), __shfl_xor_sync(MB_FULL, vi, m));
        if (r == 0) {
            q.counters[slot] = 0u;
            const unsigned tok = vi == 0xffffffffu ? 0u : vi;
            q.tokens[slot] = tok;
            if (q.codes != nullptr) q.codes[slot] = tok < (unsigned)q.codebook_size ? tok : 0u;
            if (q.eos_flag != nullptr && tok == (unsigned)q.eos_id) atomicOr(&q.eos_flag[b], 1);
        }
        return;
    }
    if (!mine) return;
    if (p.bias != nullptr) a = __fadd_rn(a, p.bias[r0 + r]);
    store_out<true>(p, p.out, r0 + r, b0 + lb, a);
}

template <int QT, bool STRICT>
int launch_qt(const GemvP &p, size_t groups, bool tiled, cudaStream_t s) {
    // Strict f32: the reference's scalar build sums a row's products one after another
    // (src/kernels.c:40-44); only the one-thread-per-output kernel keeps that order.
    if (STRICT && QT == MB_F32 && groups == 1 && (p.k % 4) == 0 &&
        ((reinterpret_cast<uintptr_t>(p.w) | reinterpret_cast<uintptr_t>(p.x)) & 15u) == 0) {
        const dim3 grid((unsigned)((p.n + SEQ_ROWS - 1) / SEQ_ROWS), (unsigned)((p.batch + SEQ_LANES - 1) / SEQ_LANES));
        mb_launch(k_gemv_f32_seq<false>, grid, dim3(SEQ_ROWS * SEQ_LANES), 0, s, p, SeqArgmaxP{});
        return mb_check_launch();
    }
    if (!tiled || (STRICT && QT == MB_F32 && groups == 1)) {
        if (groups != 1) return (int)cudaErrorInvalidValue;
        const long total = p.n * p.batch;
        mb_launch(k_gemv_generic<QT, STRICT>, dim3((unsigned)((total + 127) / 128)), dim3(128), 0, s, p);
        return mb_check_launch();
    }
    const bool quant = (QT == MB_INT8 || QT == MB_INT4);
    const size_t act_row = quant ? (size_t)p.k : (size_t)p.k * 4;
    // widest batch tile whose activations fit comfortably in shared memory
    if (p.batch >= 8 && 8 * act_row <= 64u * 1024u) return launch_tiled<QT, 8, STRICT>(p, groups, s);
    if (p.batch >= 4 && 4 * act_row <= 64u * 1024u) return launch_tiled<QT, 4, STRICT>(p, groups, s);
    if (p.batch >= 2 && 2 * act_row <= 64u * 1024u) return launch_tiled<QT, 2, STRICT>(p, groups, s);
    return launch_tiled<QT, 1, STRICT>(p, groups, s);
}

template <int QT>
int set_attrs() {
    int rc = 0;
#define MB_ATTR(BT, ST)                                                                         \
    if (rc == 0)                                                                                \
        rc = (int)cudaFuncSetAttribute(k_gemv<QT, BT, ST, false>,                               \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); \
    if (rc == 0 && QT == MB_INT8)                                                               \
        rc = (int)cudaFuncSetAttribute(k_gemv<QT, BT, ST, QT == MB_INT8>,                       \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)
    MB_ATTR(1, false); MB_ATTR(2, false); MB_ATTR(4, false); MB_ATTR(8, false);
    MB_ATTR(1, true); MB_ATTR(2, true); MB_ATTR(4, true); MB_ATTR(8, true);
#undef MB_ATTR
    return rc;
}

}  // namespace

// Opt every instantiation into large dynamic shared memory on the current
// device.  Called once per device at backend open, outside any stream capture.
extern "C" int mb_gemv_init(void) {
    int rc = set_attrs<MB_INT8>();
    if (rc == 0) rc = set_attrs<MB_INT4>();
    if (rc == 0) rc = set_attrs<MB_F16>();
    if (rc == 0) rc = set_attrs<MB_F32>();
    return rc;
}

extern "C" int mb_gemv(const mb_gemv_args *a, mb_stream stream) {
    if (a == nullptr || a->n == 0 || a->k == 0 || a->batch == 0 || a->w == nullptr ||
        a->out == nullptr)
        return (int)cudaErrorInvalidValue;
    const bool quant = a->qtype == MB_INT8 || a->qtype == MB_INT4;
    const bool fused = a->fuse != MB_FUSE_NONE;
    if (fused && (a->qtype != MB_INT8 || a->batch != 1 || a->fx == nullptr || a->groups > 1 || (a->k % 4u) != 0 ||
                  (a->fuse == MB_FUSE_LN && a->fuse_gain == nullptr)))
        return (int)cudaErrorInvalidValue;
    if (quant && ((!fused && (a->qx == nullptr || a->sx == nullptr)) || a->scales == nullptr))
        return (int)cudaErrorInvalidValue;
    if (!quant && a->x == nullptr) return (int)cudaErrorInvalidValue;
    if (a->qtype == MB_INT4 && (a->k % 32u) != 0) return (int)cudaErrorInvalidValue;
    GemvP p;
    p.w = static_cast<const unsigned char *>(a->w);
    p.scales = a->scales;
    p.bias = a->bias;
    p.qx = a->qx;
    p.sx = a->sx;
    p.x = a->x;
    p.out = a->out;
    p.n_active = a->n_active;
    p.tanh_tab = a->tanh_tab;
    p.n = (long)a->n;
    p.k = (long)a->k;
    p.out_stride = (long)a->out_stride;
    p.batch = (int)a->batch;
    p.fuse = a->fuse; p.fx = a->fx; p.fuse_gain = a->fuse_gain; p.fuse_eps = a->fuse_eps;
    p.epilogue = a->epilogue;
    switch (a->qtype) {
        case MB_INT8: p.row_bytes = (long)a->k; break;
        case MB_INT4: p.row_bytes = (long)a->k / 2; break;
        case MB_F16: p.row_bytes = (long)a->k * 2; break;
        default: p.row_bytes = (long)a->k * 4; break;
    }
    const size_t groups = a->groups > 1 ? a->groups : 1;
    p.w_gs = (long)a->w_group_stride;
    p.scale_gs = (long)a->scale_group_stride;
    p.act_gs = (long)a->act_group_stride;
    p.out_gs = (long)a->out_group_stride;
    // activations are staged in 16-byte pieces: k must allow it, and the packed
    // row must be whole 16-byte chunks, else the scalar kernel takes the shape.
    const bool act_ok = quant ? (a->k % 16u) == 0 : (a->k % 4u) == 0;
    const bool tiled = act_ok && (p.row_bytes % 16) == 0;
    if (fused && !tiled) return (int)cudaErrorInvalidValue;
    if (tiled) {
        const long cpr = p.row_bytes / 16;
        int lpr = 32;
        while (cpr % lpr != 0) lpr >>= 1;
        p.lpr = lpr;
        p.cpl = (int)(cpr / lpr);
    } else {
        p.lpr = 1;
        p.cpl = 0;
    }
    p.iters = 1;
    {
    }
    cudaStream_t s = (cudaStream_t)stream;
    const bool strict = a->strict != 0;
#define MB_DISPATCH(QT)                                                         \
    return strict ? launch_qt<QT, true>(p, groups, tiled, s)                    \
                  : launch_qt<QT, false>(p, groups, tiled, s)
    switch (a->qtype) {
        case MB_INT8: MB_DISPATCH(MB_INT8);
        case MB_INT4: MB_DISPATCH(MB_INT4);
        case MB_F16: MB_DISPATCH(MB_F16);
        case MB_F32: MB_DISPATCH(MB_F32);
        default: return (int)cudaErrorInvalidValue;
    }
#undef MB_DISPATCH
}

// The fused f32 projection + constrained argmax (see k_gemv_f32_seq<true>).  Every output's
// sum runs in index order in both modes, so the pick is the reference's in strict mode and
// deterministic in fast mode.
extern "C" size_t mb_heads_argmax_candidates(size_t batch, size_t tables, size_t vocab) {
    return batch * tables * (vocab / SEQ_ROWS);
}

extern "C" int mb_heads_argmax_f32_supported(size_t vocab, size_t k) {
    return vocab != 0 && (vocab % SEQ_ROWS) == 0 && (k % 4u) == 0;
}

extern "C" int mb_heads_argmax_f32(const mb_heads_argmax_args *a, mb_stream stream) {
    if (a == nullptr || a->w == nullptr || a->x == nullptr || a->cand_v == nullptr || a->cand_i == nullptr ||
        a->counters == nullptr || a->tokens == nullptr || a->batch == 0 || a->tables == 0 ||
        !mb_heads_argmax_f32_supported(a->vocab, a->k) || a->codebook_size > a->vocab ||
        ((reinterpret_cast<uintptr_t>(a->w) | reinterpret_cast<uintptr_t>(a->x)) & 15u) != 0)
        return (int)cudaErrorInvalidValue;
    GemvP p;
    memset(&p, 0, sizeof(p));
    p.w = reinterpret_cast<const unsigned char *>(a->w); p.bias = a->bias; p.x = a->x;
    p.n = (long)(a->tables * a->vocab); p.k = (long)a->k;
    p.batch = (int)a->batch; p.n_active = a->n_active;
    SeqArgmaxP q;
    q.vocab = (int)a->vocab; q.codebook_size = (int)a->codebook_size; q.eos_id = (int)a->eos_id; q.tables = (int)a->tables;
    q.allow_eos = a->allow_eos; q.cand_v = a->cand_v; q.cand_i = a->cand_i; q.counters = a->counters;
    q.tokens = a->tokens; q.codes = a->codes; q.eos_flag = a->eos_flag;
    const dim3 grid((unsigned)(p.n / SEQ_ROWS), (unsigned)((a->batch + SEQ_LANES - 1) / SEQ_LANES));
    mb_launch(k_gemv_f32_seq<true>, grid, dim3(SEQ_ROWS * SEQ_LANES), 0, (cudaStream_t)stream, p, q);
    return mb_check_launch();
}
