// Single-query attention over a resident KV cache: causal self-attention with
// KV append (12 heads x 64 in Magpie) and cross-attention to the text states
// (1 head x xattn_width), for a batch of independent streams that each own a
// cache slot and a position.
//
// Reference arithmetic (src/graph.c:3180-3202, 3221-3244): per head
//   sc[s] = (sum_d q[d]*k[s][d]) * scale ; m = max sc ; e[s] = expf(sc[s]-m)
//   den = sum_s e[s] ; out[d] = sum_s (e[s]/den) * v[s][d]
// all in f32, every sum sequential in index order.
//
// STRICT kernel: one CTA per (head, stream); scores by one thread per position
// (sequential over d, product and sum rounded separately), the denominator by
// one sequential chain, outputs by one thread per d (sequential over s).  exp
// is evaluated in double and rounded once.  Same bits as the CPU loop except
// where libm's expf is not correctly rounded.
//
// FAST kernel: grid (splits, heads, streams).  Each CTA takes a contiguous
// range of positions, computes a partial (max, sum, weighted V) and, when the
// work is split or the output must be quantized across heads, publishes it to
// a scratch buffer; the last CTA of a stream to arrive (one atomic counter per
// stream) merges all partials in split order and optionally quantizes the
// merged row to int8 for the next projection.  Results do not depend on
// arrival order.
#include "common.cuh"
#include "launch.h"

#include <float.h>

namespace {

struct AttnP {
    const float *q, *k_new, *v_new;
    float *k_cache, *v_cache;
    const int *slots, *lens, *n_active;
    float *out;
    int8_t *qx;
    float *sx;
    float *partials;
    unsigned *counters;
    int *status;
    long q_stride, slot_stride, cache_stride, out_stride;
    long position, valid;
    int heads, hw, batch, splits, chunk_max;
    float scale;
};

__device__ __forceinline__ bool lane_setup(const AttnP &p, int b, long &pos, long &valid,
                                           float *&kc, float *&vc) {
    if (p.n_active != nullptr && b >= *p.n_active) return false;
    if (p.lens != nullptr) { pos = p.lens[b]; valid = pos + 1; }
    else { pos = p.position; valid = p.valid; }
    const long slot = p.slots != nullptr ? p.slots[b] : b;
    kc = p.k_cache + slot * p.slot_stride;
    vc = p.v_cache + slot * p.slot_stride;
    return true;
}

// ------------------------------------------------------------------ strict
__global__ void __launch_bounds__(256) k_attn_strict(AttnP p) {
    extern __shared__ float sm[];
    __shared__ float red[33];
    __shared__ float s_denom;
    const int h = blockIdx.x, b = blockIdx.y;
    long pos, valid;
    float *kc, *vc;
    if (!lane_setup(p, b, pos, valid, kc, vc)) return;
    const int hw = p.hw;
    float *qs = sm;            // [hw]
    float *sc = sm + hw;       // [valid]
    const float *q = p.q + (long)b * p.q_stride + (long)h * hw;
    for (int d = threadIdx.x; d < hw; d += blockDim.x) {
        qs[d] = q[d];
        if (p.k_new != nullptr) {
            kc[pos * p.cache_stride + (long)h * hw + d] = p.k_new[(long)b * p.q_stride + (long)h * hw + d];
            vc[pos * p.cache_stride + (long)h * hw + d] = p.v_new[(long)b * p.q_stride + (long)h * hw + d];
        }
    }
    __syncthreads();
    const float *kh = kc + (long)h * hw;
    const float *vh = vc + (long)h * hw;
    float lmax = -FLT_MAX;
    for (long s = threadIdx.x; s < valid; s += blockDim.x) {
        const float *k = kh + s * p.cache_stride;
        float a = 0.0f;
        for (int d = 0; d < hw; ++d) a = __fadd_rn(a, __fmul_rn(qs[d], k[d]));
        a = __fmul_rn(a, p.scale);
        sc[s] = a;
        if (a > lmax) lmax = a;
    }
    const float m = block_max(lmax, red);
    for (long s = threadIdx.x; s < valid; s += blockDim.x)
        sc[s] = exp_ref<true>(__fsub_rn(sc[s], m));
    __syncthreads();
    if (threadIdx.x == 0) {
        float den = 0.0f;
        for (long s = 0; s < valid; ++s) den = __fadd_rn(den, sc[s]);
        s_denom = den;
    }
    __syncthreads();
    const float den = s_denom;
    for (long s = threadIdx.x; s < valid; s += blockDim.x) sc[s] = __fdiv_rn(sc[s], den);
    __syncthreads();
    for (int d = threadIdx.x; d < hw; d += blockDim.x) {
        float a = 0.0f;
        for (long s = 0; s < valid; ++s)
            a = __fadd_rn(a, __fmul_rn(sc[s], vh[s * p.cache_stride + d]));
        p.out[(long)b * p.out_stride + (long)h * hw + d] = a;
    }
}

// -------------------------------------------------------------------- fast
constexpr int FAST_THREADS = 128;

template <int VEC>
__global__ void __launch_bounds__(FAST_THREADS) k_attn_fast(AttnP p) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[33];
    __shared__ unsigned s_last;
    const int sp = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    long pos, valid;
    float *kc, *vc;
    if (!lane_setup(p, b, pos, valid, kc, vc)) return;
    const int hw = p.hw, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long chunk = (valid + p.splits - 1) / p.splits;
    const long s0 = (long)sp * chunk;
    const long s1 = min(valid, s0 + chunk);
    const long cnt = s1 > s0 ? s1 - s0 : 0;
    float *qs = sm;                                 // [hw]
    float *sc = sm + hw;                            // [chunk_max]
    float *accs = sc + p.chunk_max;                 // [groups][hw]
    const long hoff = (long)h * hw;
    const float *knew = p.k_new == nullptr ? nullptr : p.k_new + (long)b * p.q_stride + hoff;
    const float *vnew = p.v_new == nullptr ? nullptr : p.v_new + (long)b * p.q_stride + hoff;
    for (int d = threadIdx.x; d < hw; d += blockDim.x) {
        qs[d] = p.q[(long)b * p.q_stride + hoff + d];
        if (knew != nullptr && sp == 0) {   // one CTA per (stream, head) appends
            kc[pos * p.cache_stride + hoff + d] = knew[d];
            vc[pos * p.cache_stride + hoff + d] = vnew[d];
        }
    }
    __syncthreads();
    // ---- scores ---------------------------------------------------------------
    float lmax = -FLT_MAX;
    if (VEC == 4) {
        const int lpp = hw / 4;            // lanes per position (power of two <= 32)
        const int ppw = 32 / lpp;          // positions per warp step
        const int sub = lane / lpp, li = lane % lpp;
        const float4 qv = reinterpret_cast<const float4 *>(qs)[li];
        const int step = (FAST_THREADS / 32) * ppw;
        // all lanes iterate the same number of times so the shuffles stay converged
        const long bound = (cnt + step - 1) / step * step;
        for (long i = warp * ppw + sub; i < bound; i += step) {
            float a = 0.0f;
            const bool ok = i < cnt;
            if (ok) {
                const long s = s0 + i;
                const float *src = (knew != nullptr && s == pos) ? knew : kc + s * p.cache_stride + hoff;
                const float4 kv = reinterpret_cast<const float4 *>(src)[li];
                a = fmaf(qv.x, kv.x, a); a = fmaf(qv.y, kv.y, a);
                a = fmaf(qv.z, kv.z, a); a = fmaf(qv.w, kv.w, a);
            }
            for (int o = lpp >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(MB_FULL, a, o);
            if (ok && li == 0) {
                a *= p.scale;
                sc[i] = a;
                lmax = fmaxf(lmax, a);
            }
        }
    } else {
        for (long i = warp; i < cnt; i += FAST_THREADS / 32) {
            const long s = s0 + i;
            const float *src = (knew != nullptr && s == pos) ? knew : kc + s * p.cache_stride + hoff;
            float a = 0.0f;
            for (int d = lane; d < hw; d += 32) a = fmaf(qs[d], src[d], a);
            a = warp_sum(a);
            if (lane == 0) {
                a *= p.scale;
                sc[i] = a;
                lmax = fmaxf(lmax, a);
            }
        }
    }
    const float m = block_max(lmax, red);   // includes the barrier that publishes sc[]
    float lsum = 0.0f;
    for (long i = threadIdx.x; i < cnt; i += blockDim.x) {
        const float e = exp_ref<false>(sc[i] - m);
        sc[i] = e;
        lsum += e;
    }
    const float l = block_sum(lsum, red);
    // ---- weighted V -------------------------------------------------------------
    const int tpp = hw / VEC;                       // threads per position
    const int groups = tpp >= FAST_THREADS ? 1 : FAST_THREADS / tpp;
    if (VEC == 4) {
        const int g = threadIdx.x / tpp, li = threadIdx.x % tpp;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < groups) {
            for (long i = g; i < cnt; i += groups) {
                const long s = s0 + i;
                const float *src = (vnew != nullptr && s == pos) ? vnew : vc + s * p.cache_stride + hoff;
                const float4 vv = reinterpret_cast<const float4 *>(src)[li];
                const float w = sc[i];
                acc.x = fmaf(w, vv.x, acc.x); acc.y = fmaf(w, vv.y, acc.y);
                acc.z = fmaf(w, vv.z, acc.z); acc.w = fmaf(w, vv.w, acc.w);
            }
            reinterpret_cast<float4 *>(accs)[g * tpp + li] = acc;
        }
    } else {
        // scalar layout: thread t covers d = t, t + blockDim, ...; single group
        for (int d = threadIdx.x; d < hw; d += blockDim.x) {
            float a = 0.0f;
            for (long i = 0; i < cnt; ++i) {
                const long s = s0 + i;
                const float *src = (vnew != nullptr && s == pos) ? vnew : vc + s * p.cache_stride + hoff;
                a = fmaf(sc[i], src[d], a);
            }
            accs[d] = a;
        }
    }
    __syncthreads();
    const int ngroups = VEC == 4 ? groups : 1;
    const bool publish = p.splits > 1 || (p.qx != nullptr && p.heads > 1);
    float *part = p.partials == nullptr
                      ? nullptr
                      : p.partials + (((long)b * p.heads + h) * p.splits + sp) * (hw + 2);
    for (int d = threadIdx.x; d < hw; d += blockDim.x) {
        float a = 0.0f;
        for (int g = 0; g < ngroups; ++g) a += accs[g * hw + d];
        if (publish) part[2 + d] = a;
        else {
            const float o = l > 0.0f ? a / l : 0.0f;
            if (p.out != nullptr) p.out[(long)b * p.out_stride + hoff + d] = o;
            accs[d] = o;   // kept for the single-CTA quantization below
        }
    }
    if (!publish) {
        if (p.qx == nullptr) return;
        // heads == 1 and one split: this CTA owns the whole row
        __syncthreads();
        float amax = 0.0f;
        for (int d = threadIdx.x; d < hw; d += blockDim.x) amax = fmaxf(amax, fabsf(accs[d]));
        amax = block_max(amax, red);
        int8_t *qrow = p.qx + (long)b * p.heads * hw;
        const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        for (int d = threadIdx.x; d < hw; d += blockDim.x) {
            int v = round_half_away(__fmul_rn(accs[d], inv));
            qrow[d] = (int8_t)min(127, max(-127, v));
        }
        if (threadIdx.x == 0) p.sx[b] = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
        return;
    }
    if (threadIdx.x == 0) {
        part[0] = cnt > 0 ? m : -FLT_MAX;
        part[1] = cnt > 0 ? l : 0.0f;
    }
    // ---- last CTA of this stream merges ------------------------------------------
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total = (unsigned)(p.heads * p.splits);
        const unsigned prev = atomicAdd(&p.counters[b], 1u);
        s_last = (prev == total - 1u) ? 1u : 0u;
        if (s_last) p.counters[b] = 0u;   // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int width = p.heads * hw;
    const float *base = p.partials + (long)b * p.heads * p.splits * (hw + 2);
    float amax = 0.0f;
    // merged outputs are parked in this stream's first partial slots (each thread
    // overwrites only what it alone reads) before the quantization pass.
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int hh = i / hw, d = i % hw;
        const float *ph = base + (long)hh * p.splits * (hw + 2);
        float M = -FLT_MAX;
        for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(ph + (long)s * (hw + 2)));
        float L = 0.0f, O = 0.0f;
        for (int s = 0; s < p.splits; ++s) {
            const float *ps = ph + (long)s * (hw + 2);
            const float ls = __ldcg(ps + 1);
            if (ls > 0.0f) {
                const float wgt = exp_ref<false>(__ldcg(ps) - M);
                L = fmaf(ls, wgt, L);
                O = fmaf(__ldcg(ps + 2 + d), wgt, O);
            }
        }
        const float o = L > 0.0f ? O / L : 0.0f;
        if (p.out != nullptr) p.out[(long)b * p.out_stride + i] = o;
        if (p.qx != nullptr) {
            sm[i] = o;   // the launcher sizes shared memory for heads*hw floats
            amax = fmaxf(amax, fabsf(o));
        }
    }
    if (p.qx == nullptr) return;
    amax = block_max(amax, red);
    int8_t *qrow = p.qx + (long)b * width;
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        int v = round_half_away(__fmul_rn(sm[i], inv));
        qrow[i] = (int8_t)min(127, max(-127, v));
    }
    if (threadIdx.x == 0) p.sx[b] = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
}

bool is_pow2(long v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

// Opt the kernels into large dynamic shared memory on the current device; once
// per device at backend open, outside any stream capture.
extern "C" int mb_attention_init(void) {
    int rc = (int)cudaFuncSetAttribute(k_attn_strict, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_fast<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_fast<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return rc;
}

extern "C" size_t mb_attention_partials_floats(size_t batch, size_t heads, size_t splits,
                                               size_t head_width) {
    return batch * heads * splits * (head_width + 2);
}

extern "C" int mb_attention(const mb_attn_args *a, mb_stream stream) {
    if (a == nullptr || a->q == nullptr || a->k_cache == nullptr || a->v_cache == nullptr ||
        a->batch == 0 || a->heads == 0 || a->head_width == 0)
        return (int)cudaErrorInvalidValue;
    if (a->out == nullptr && a->qx == nullptr) return (int)cudaErrorInvalidValue;
    if ((a->k_new == nullptr) != (a->v_new == nullptr)) return (int)cudaErrorInvalidValue;
    AttnP p;
    p.q = a->q; p.k_new = a->k_new; p.v_new = a->v_new;
    p.k_cache = a->k_cache; p.v_cache = a->v_cache;
    p.slots = a->slots; p.lens = a->lens; p.n_active = a->n_active;
    p.out = a->out; p.qx = a->qx; p.sx = a->sx;
    p.partials = a->partials; p.counters = a->counters; p.status = a->status;
    p.q_stride = (long)a->q_stride; p.slot_stride = (long)a->slot_stride;
    p.cache_stride = (long)a->cache_stride; p.out_stride = (long)a->out_stride;
    p.position = (long)a->position; p.valid = (long)a->valid;
    p.heads = (int)a->heads; p.hw = (int)a->head_width; p.batch = (int)a->batch;
    p.scale = a->scale;
    cudaStream_t s = (cudaStream_t)stream;
    // Longest row any lane can attend over: callers with per-lane positions pass
    // the cache capacity in `valid`.
    const long max_valid = (long)a->valid;
    if (max_valid <= 0) return (int)cudaErrorInvalidValue;
    if (a->strict) {
        if (a->out == nullptr) return (int)cudaErrorInvalidValue;
        p.splits = 1; p.chunk_max = (int)max_valid;
        const size_t smem = (size_t)(p.hw + max_valid) * sizeof(float);
        if (smem > 200u * 1024u) return (int)cudaErrorInvalidValue;
        k_attn_strict<<<dim3((unsigned)p.heads, (unsigned)p.batch), 256, smem, s>>>(p);
        int rc = mb_check_launch();
        if (rc == 0 && a->qx != nullptr)
            rc = mb_quant_rows(a->out, a->batch, a->heads * a->head_width, a->qx, a->sx,
                               a->n_active, stream);
        return rc;
    }
    p.splits = (int)(a->splits > 0 ? a->splits : 1);
    const bool publish = p.splits > 1 || (a->qx != nullptr && p.heads > 1);
    if (publish && (a->partials == nullptr || a->counters == nullptr))
        return (int)cudaErrorInvalidValue;
    p.chunk_max = (int)((max_valid + p.splits - 1) / p.splits);
    const bool vec4 = (p.hw % 4) == 0 && is_pow2(p.hw / 4) && p.hw / 4 <= 32 &&
                      (p.cache_stride % 4) == 0 && (p.q_stride % 4) == 0 &&
                      (p.slot_stride % 4) == 0 &&
                      (((uintptr_t)a->k_cache | (uintptr_t)a->v_cache | (uintptr_t)a->q |
                        (uintptr_t)a->k_new | (uintptr_t)a->v_new) & 15u) == 0;
    const int tpp = vec4 ? p.hw / 4 : p.hw;
    const int groups = vec4 ? (tpp >= FAST_THREADS ? 1 : FAST_THREADS / tpp) : 1;
    size_t floats = (size_t)p.hw + p.chunk_max + (size_t)groups * p.hw;
    // the merging CTA parks heads*hw merged outputs in the same shared buffer
    if (a->qx != nullptr && publish && floats < (size_t)p.heads * p.hw) {
        p.chunk_max += (int)((size_t)p.heads * p.hw - floats);
        floats = (size_t)p.heads * p.hw;
    }
    const size_t smem = floats * sizeof(float);
    if (smem > 200u * 1024u) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)p.splits, (unsigned)p.heads, (unsigned)p.batch);
    if (vec4) k_attn_fast<4><<<grid, FAST_THREADS, smem, s>>>(p);
    else k_attn_fast<1><<<grid, FAST_THREADS, smem, s>>>(p);
    return mb_check_launch();
}
