// The cross-attention block of a decoder layer as one launch, one CTA per stream
// (src/graph.c:3213-3256 in mynah-tts):
//
//   x      = residual row (already holds x + o_self(...))
//   h      = layer_norm(x, norm_xattn_query)          -> int8 row + scale
//   q      = W_q h                                     (int8 x int8, int32 sums)
//   ctx    = softmax(q K^T * scale) V                  over the stream's text states
//   x     += W_o quant(ctx)
//   h2     = layer_norm(x, norm_pos_ff)                -> int8 row + scale (feed-forward input)
//
// Everything here is per stream, so the five launches it replaces (norm, product,
// attention, product, norm) only ever exchanged one row through global memory; each
// dependent launch costs 4-7 us in the step and the block runs 12 times per step.  The
// stream's K and V rows (constant after the slot is loaded) are requested as TMA tiles
// before the wait on the preceding launch, so they land while the norm and the query
// product run.
//
// Same bits as the separate launches: the norm is mb_ln_block<1> on 256 threads, the
// products are exact int32 sums scaled as (float)s * ws * sx with each product rounded,
// the attention is the chunked single-head form of k_attn_short (32-row chunks, ordered
// merge), the quantizations round half away from zero.
// Phase timestamps of profiling builds (make TICKS=1), 16 per CTA: 0 entry, 1 after the
// dependency wait, 2 row loaded, 3 first norm, 4 query product, 5 attention, 6 context
// quantized, 7 output product, 8 second norm; 9 .. 14 the steps inside the second norm (mean
// chain, squares, variance chain, normalized, absmax, quantized: the first norm writes them
// too and is overwritten).
#ifdef MB_PHASE_TICKS
__device__ unsigned long long g_xb_ticks[16 * 1024];
__device__ __forceinline__ void xb_tick(int i) {
    if (threadIdx.x == 0 && blockIdx.x < 1024u) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_xb_ticks[blockIdx.x * 16 + i] = t;
    }
}
#define XB_TICK(i) xb_tick(i)
#define MB_LN_TICK(i) xb_tick(9 + (i))
#else
#define XB_TICK(i)
#endif

#include "attn_tiles.cuh"
#include "launch.h"

#include <string.h>

namespace {

constexpr int XB_THREADS = 256;
constexpr int XB_WARPS = XB_THREADS / 32;
constexpr int XB_MAX_CHUNKS = 8;

struct CrossP {
    float *x;
    const float *gain_query, *gain_ff;
    const int8_t *wq, *wo;
    const float *wq_scales, *wo_scales;
    const int *slots, *n_active, *rows_per_slot;
    int8_t *qx;
    float *sx;
    int *status;
    const uint32_t *exp_tab;
    long slot_rows;
    int width, xw, rows, chunks;
    float scale, eps;
};

// A read-only 16-byte load the compiler may not move: the constants fetched early must be
// requested where the source says (before the dependency wait, before the attention), not
// next to their first use.
__device__ __forceinline__ uint4 ldg_pinned(const uint4 *ptr) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

__device__ __forceinline__ int dot16(const uint4 &a, const uint4 &b, int acc) {
    acc = __dp4a((int)a.x, (int)b.x, acc);
    acc = __dp4a((int)a.y, (int)b.y, acc);
    acc = __dp4a((int)a.z, (int)b.z, acc);
    acc = __dp4a((int)a.w, (int)b.w, acc);
    return acc;
}

// RO = rows of the output weight one thread ends up owning (width <= RO * 256); a thread of
// the query product holds every other 16-byte piece of one weight row, 8 * RO of them.
// LPR = 16-byte pieces of an output-weight row (xw = 16 * LPR).
// STRICT: the reference's summation orders (mb_ln_block_strict; scores, denominator and
// context as sequential chains, as k_attn_exact forms them) and the host libm's expf; the
// K/V tiles then arrive as 128-byte-swizzled [32][32] boxes so that a warp whose threads
// each walk one row reads 32 different banks.  Same bits as the separate strict launches.

// One group of 32 int4 weights (16 packed bytes, even index in the low nibble, +8 offset) times
// 32 int8 activations (two 16-byte pieces in natural order): the exact int32 sum.
__device__ __forceinline__ int dot_q4_group(uint4 w, uint4 x0, uint4 x1) {
    const unsigned ww[4] = {w.x, w.y, w.z, w.w};
    const unsigned xe[4] = {__byte_perm(x0.x, x0.y, 0x6420), __byte_perm(x0.z, x0.w, 0x6420),
                            __byte_perm(x1.x, x1.y, 0x6420), __byte_perm(x1.z, x1.w, 0x6420)};
    const unsigned xo[4] = {__byte_perm(x0.x, x0.y, 0x7531), __byte_perm(x0.z, x0.w, 0x7531),
                            __byte_perm(x1.x, x1.y, 0x7531), __byte_perm(x1.z, x1.w, 0x7531)};
    int gi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        gi = __dp4a((int)__vsub4(ww[j] & 0x0f0f0f0fu, 0x08080808u), (int)xe[j], gi);
        gi = __dp4a((int)__vsub4((ww[j] >> 4) & 0x0f0f0f0fu, 0x08080808u), (int)xo[j], gi);
    }
    return gi;
}

// INT4: the two weights are int4 in groups of 32 with f32 group scales (src/qmat.c:154-185:
// per group an exact int32 sum times the group's scale, added in group order, then times the
// activation scale); otherwise int8 with one scale per row.
template <int RO, int LPR, bool STRICT, bool INT4>
__global__ void __launch_bounds__(XB_THREADS, 1)
k_cross_block(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, CrossP p) {
    extern __shared__ __align__(1024) float sm[];
    __shared__ float red[96];
    __shared__ float stat[2];
    __shared__ __align__(8) unsigned long long mbar[2 * XB_MAX_CHUNKS];   // K chunks, then V chunks
    __shared__ unsigned s_bad;
    XB_TICK(0);
    const int b = blockIdx.x;
    // lane state was written by the previous step's last launch: readable before the wait
    const int live = p.n_active != nullptr ? *p.n_active : 0x7fffffff;
    const long slot = p.slots != nullptr ? (long)p.slots[b] : (long)b;
    if (b >= live) return;
    // text states of this stream (the slot's request), and the 32-row chunks they fill
    const int rows = p.rows_per_slot != nullptr ? min(max(p.rows_per_slot[slot], 1), p.rows) : p.rows;
    const int W = p.width, XW = p.xw, ns = (rows + CHUNK - 1) / CHUNK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile_floats = CHUNK * XW;
    const int nsmax = p.chunks;                       // the layout is sized for the longest request
    float *Kt = sm;                                   // [nsmax] tiles of [32][XW]
    float *Vt = Kt + (long)nsmax * tile_floats;
    float *xres = Vt + (long)nsmax * tile_floats;     // [W] the residual row as it came in
    float *row = xres + W;                            // [W] work row of the norms
    float *qs = row + W;                              // [XW] query
    float *P = qs + XW;                               // [nsmax][XW + 2] chunk partials
    float *wts = P + (long)nsmax * (XW + 2);          // [32] merge scratch
    float *vals = wts + 32;                           // [XW] merged context
    float *gq = vals + XW;                            // [W] gain of the first norm
    float *gf = gq + W;                               // [W] gain of the second norm
    float *sq = gf + W;                               // [W] squares of the strict norms
    int8_t *qrow = reinterpret_cast<int8_t *>((reinterpret_cast<uintptr_t>(sq + W) + 15u) & ~(uintptr_t)15u);   // [W] quantized first norm
    int8_t *ctxq = qrow + W;                                 // [XW] quantized context
    const unsigned tile_bytes = (unsigned)tile_floats * 4u;
    if (threadIdx.x == 0) {
        s_bad = 0u;
        const unsigned long long stream_policy = mb_l2_evict_first();
        for (int i = 0; i < 2 * XB_MAX_CHUNKS; ++i) mbar_init(&mbar[i], 1u);
        for (int c = 0; c < ns; ++c) {
            const int y = (int)(slot * p.slot_rows + (long)c * CHUNK);
            mbar_expect_tx(&mbar[c], tile_bytes);
            mbar_expect_tx(&mbar[XB_MAX_CHUNKS + c], tile_bytes);
            if (STRICT) {
                for (int bx = 0; bx < XW / 32; ++bx) {
                    mb_tma_load_2d_hint(Kt + (long)c * tile_floats + bx * 1024, &kmap, bx * 32, y, &mbar[c], stream_policy);
                    mb_tma_load_2d_hint(Vt + (long)c * tile_floats + bx * 1024, &vmap, bx * 32, y, &mbar[XB_MAX_CHUNKS + c], stream_policy);
                }
            } else {
                mb_tma_load_2d_hint(Kt + (long)c * tile_floats, &kmap, 0, y, &mbar[c], stream_policy);
                mb_tma_load_2d_hint(Vt + (long)c * tile_floats, &vmap, 0, y, &mbar[XB_MAX_CHUNKS + c], stream_policy);
            }
        }
    }
    // Constants, fetched while the preceding launch is still running: the norms' gains into
    // shared memory, each thread's half of a query-weight row into registers, and the
    // output weights into L2 (each CTA asks for its share of the lines).
    for (int i = threadIdx.x; i < W; i += XB_THREADS) {
        gq[i] = __ldg(p.gain_query + i);
        gf[i] = __ldg(p.gain_ff + i);
    }
    const int npc = INT4 ? W / 32 : W / 16;           // 16-byte pieces of a query-weight row
    constexpr int PQ = INT4 ? 4 * RO : 8 * RO;
    const int oq = threadIdx.x >> 1, hq = threadIdx.x & 1;   // query row of this thread, and which pieces
    uint4 wq0[PQ];
    float wqg[INT4 ? PQ : 1];                         // int4: the group scale of each piece
#pragma unroll
    for (int j = 0; j < PQ; ++j) {
        const int pc = 2 * j + hq;
        wq0[j] = (oq < XW && pc < npc) ? ldg_pinned(reinterpret_cast<const uint4 *>(p.wq + (long)oq * (INT4 ? W / 2 : W)) + pc)
                                       : make_uint4(0u, 0u, 0u, 0u);
        if (INT4) wqg[j] = (oq < XW && pc < npc) ? __ldg(p.wq_scales + (long)oq * npc + pc) : 0.0f;
    }
    const float wqs0 = (!INT4 && oq < XW) ? __ldg(p.wq_scales + oq) : 0.0f;
    {
        const long lines = ((long)W * XW / (INT4 ? 2 : 1) + 127) / 128;
        for (long ln = (long)blockIdx.x * XB_THREADS + threadIdx.x; ln < lines; ln += (long)gridDim.x * XB_THREADS)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.wo + ln * 128));
    }
    mb_pdl_wait();
    mb_pdl_trigger();
    XB_TICK(1);

    // ---- first norm, quantized into shared memory
    float *xg = p.x + (long)b * W;
    for (int i = threadIdx.x; i < W; i += XB_THREADS) {
        const float v = xg[i];
        xres[i] = v;
        row[i] = v;
    }
    __syncthreads();
    XB_TICK(2);
    const float sxq = STRICT ? mb_ln_block_strict(row, W, gq, nullptr, p.eps, sq, stat, red, nullptr, true, qrow)
                             : mb_ln_block<1>(row, W, gq, nullptr, p.eps, red, nullptr, true, qrow);
    __syncthreads();

    XB_TICK(3);
    // ---- query product: two threads per output row, pieces of the row interleaved
    if (INT4) {
        // a piece is one group: its exact sum times its scale; the two threads of a row then
        // add the groups in order, each taking the other's from a shuffle
        float gp[PQ];
#pragma unroll
        for (int j = 0; j < PQ; ++j) {
            const int pc = 2 * j + hq;
            gp[j] = 0.0f;
            if (pc < npc) {
                const uint4 x0 = reinterpret_cast<const uint4 *>(qrow)[2 * pc];
                const uint4 x1 = reinterpret_cast<const uint4 *>(qrow)[2 * pc + 1];
                gp[j] = __fmul_rn((float)dot_q4_group(wq0[j], x0, x1), wqg[j]);
            }
        }
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < PQ; ++j) {
            const float mine = gp[j];
            const float even = __shfl_sync(MB_FULL, mine, lane & ~1);     // group 2j
            const float odd = __shfl_sync(MB_FULL, mine, lane | 1);       // group 2j + 1
            if (2 * j < npc) acc = __fadd_rn(acc, even);
            if (2 * j + 1 < npc) acc = __fadd_rn(acc, odd);
        }
        if (hq == 0 && oq < XW) qs[oq] = __fmul_rn(acc, sxq);
    } else {
        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;           // four chains instead of one of 4 * PQ steps
#pragma unroll
        for (int j = 0; j < PQ; ++j) {
            const int pc = 2 * j + hq;
            if (pc < npc) {
                const uint4 h = reinterpret_cast<const uint4 *>(qrow)[pc];
                a0 = __dp4a((int)wq0[j].x, (int)h.x, a0);
                a1 = __dp4a((int)wq0[j].y, (int)h.y, a1);
                a2 = __dp4a((int)wq0[j].z, (int)h.z, a2);
                a3 = __dp4a((int)wq0[j].w, (int)h.w, a3);
            }
        }
        int acc = (a0 + a1) + (a2 + a3);
        acc += __shfl_xor_sync(MB_FULL, acc, 1);
        if (hq == 0 && oq < XW) qs[oq] = __fmul_rn(__fmul_rn((float)acc, wqs0), sxq);
    }
    // The output weights are requested now and land during the attention.  A warp owns
    // 32 * RO consecutive weight rows and reads them LPR lanes to a row (whole 128-byte lines
    // per load: a thread per row would touch 32 lines per load instruction).
    constexpr int RPI = 32 / LPR;                     // rows per warp load
    constexpr int NI = RO * LPR;                      // loads per lane
    const int lr = lane / LPR, lp = lane % LPR;
    const int wrow0 = warp * RO * 32;
    uint4 wo0[INT4 ? 1 : NI];
    constexpr int OG = 4;                             // int4: groups of an output-weight row (xw = 128), or fewer
    uint4 wo4[INT4 ? RO * OG : 1];                    // int4: a thread owns rows threadIdx.x + 256 i
    float wog[INT4 ? RO * OG : 1];
    const int og = XW / 32;
    if (INT4) {
#pragma unroll
        for (int i = 0; i < RO; ++i) {
            const int r = (int)threadIdx.x + i * XB_THREADS;
#pragma unroll
            for (int g = 0; g < OG; ++g) {
                const bool ok = r < W && g < og;
                wo4[i * OG + g] = ok ? ldg_pinned(reinterpret_cast<const uint4 *>(p.wo + (long)r * (XW / 2)) + g) : make_uint4(0u, 0u, 0u, 0u);
                wog[i * OG + g] = ok ? __ldg(p.wo_scales + (long)r * og + g) : 0.0f;
            }
        }
    } else {
#pragma unroll
        for (int u = 0; u < NI; ++u) {
            const int r = wrow0 + u * RPI + lr;
            wo0[u] = r < W ? ldg_pinned(reinterpret_cast<const uint4 *>(p.wo + (long)r * XW) + lp) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // after the exchange below this lane holds the sums of loads ubase .. ubase + RO - 1
    int ubase = 0;
    {
        int n = NI;
#pragma unroll
        for (int m = LPR / 2; m >= 1; m >>= 1) {
            n >>= 1;
            if (lp & m) ubase += n;
        }
    }
    float wos0[RO];
#pragma unroll
    for (int i = 0; i < RO; ++i) {
        const int r = wrow0 + (ubase + i) * RPI + lr;
        wos0[i] = (!INT4 && r < W) ? __ldg(p.wo_scales + r) : 0.0f;
    }
    __syncthreads();

    XB_TICK(4);
    float ctx = 0.0f;
    // ---- attention over the text states: warp c makes the partial of chunk c
    const int tpp = XW / 4, rps = 32 / tpp, sub = lane / tpp, li = lane % tpp;
    if (STRICT) {
        // reference order (src/graph.c:3221-3244): thread s forms the score of text state s as
        // one chain over d; the denominator is one chain over s; thread d forms context
        // element d as one chain over s
        float *scs = P;                               // [ns * 32] scores, then weights
        const int s = threadIdx.x, c = s >> 5, r = s & 31;
        float a = -FLT_MAX;
        if (s < rows) {
            if (mbar_wait(&mbar[c], 0u, SPIN_LIMIT)) {
                const float *tile = Kt + (long)c * tile_floats + r * 32;
                float dot = 0.0f;
                // sixteen 16-byte pieces of the row at a time into registers, then their part of
                // the chain (loads inside the chain would each cost a shared-memory round trip)
                for (int d0 = 0; d0 < XW; d0 += 64) {
                    float4 kr[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int d4 = d0 + 4 * c;
                        kr[c] = d4 < XW ? *reinterpret_cast<const float4 *>(tile + (d4 >> 5) * 1024 + (((((d4 & 31) >> 2)) ^ (r & 7)) << 2))
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int d4 = d0 + 4 * c;
                        if (d4 < XW) {
                            const float4 qv = *reinterpret_cast<const float4 *>(qs + d4);
                            dot = __fadd_rn(dot, __fmul_rn(qv.x, kr[c].x));
                            dot = __fadd_rn(dot, __fmul_rn(qv.y, kr[c].y));
                            dot = __fadd_rn(dot, __fmul_rn(qv.z, kr[c].z));
                            dot = __fadd_rn(dot, __fmul_rn(qv.w, kr[c].w));
                        }
                    }
                }
                a = __fmul_rn(dot, p.scale);
            } else {
                s_bad = 1u;
                if (p.status != nullptr) atomicOr(p.status, 2);
            }
        }
        const float m = block_max1(a, red);
        if (s < rows) scs[s] = exp_ref<true>(__fsub_rn(a, m), p.exp_tab);
        __syncthreads();
        if (threadIdx.x == 0) stat[0] = mb_seq_sum(scs, rows);
        __syncthreads();
        if (s < rows) scs[s] = __fdiv_rn(scs[s], stat[0]);
        __syncthreads();
        if (threadIdx.x < XW && s_bad == 0u) {
            const int d = threadIdx.x;
            const float *col = Vt + (d >> 5) * 1024 + (d & 3);
            const int jc = (d & 31) >> 2;
            float acc = 0.0f;
            for (int cc = 0; cc < ns; ++cc) {
                if (!mbar_wait(&mbar[XB_MAX_CHUNKS + cc], 0u, SPIN_LIMIT)) {
                    s_bad = 1u;
                    if (p.status != nullptr) atomicOr(p.status, 2);
                    break;
                }
                const int cnt = min(CHUNK, rows - cc * CHUNK);
                const float *tile = col + (long)cc * tile_floats;
                const float *w = scs + cc * CHUNK;
                float vr[CHUNK], wr[CHUNK];
#pragma unroll
                for (int rr = 0; rr < CHUNK; ++rr) vr[rr] = tile[rr * 32 + ((jc ^ (rr & 7)) << 2)];
#pragma unroll
                for (int r4 = 0; r4 < CHUNK / 4; ++r4) {
                    const float4 w4 = *reinterpret_cast<const float4 *>(w + 4 * r4);
                    wr[4 * r4] = w4.x; wr[4 * r4 + 1] = w4.y; wr[4 * r4 + 2] = w4.z; wr[4 * r4 + 3] = w4.w;
                }
#pragma unroll
                for (int rr = 0; rr < CHUNK; ++rr)
                    if (rr < cnt) acc = __fadd_rn(acc, __fmul_rn(wr[rr], vr[rr]));
            }
            ctx = acc;
        }
    } else if (warp < ns) {
        const int c = warp;
        const float4 qv = reinterpret_cast<const float4 *>(qs)[li];
        const int cnt = min(CHUNK, rows - c * CHUNK);
        const bool k_ok = mbar_wait(&mbar[c], 0u, SPIN_LIMIT);
        const bool v_ok = k_ok && mbar_wait(&mbar[XB_MAX_CHUNKS + c], 0u, SPIN_LIMIT);
        if (k_ok && v_ok) {
            const float *Ks = Kt + (long)c * tile_floats;
            float dot;
            switch (tpp) {
            case 32: dot = chunk_scores<32>(Ks, XW, qv, sub, li); break;
            case 16: dot = chunk_scores<16>(Ks, XW, qv, sub, li); break;
            case 8: dot = chunk_scores<8>(Ks, XW, qv, sub, li); break;
            default: dot = chunk_scores<4>(Ks, XW, qv, sub, li); break;
            }
            const int my_row = li * rps + sub;
            const float mine = my_row < cnt ? dot * p.scale : -FLT_MAX;
            const float m = warp_max(mine);
            const float e = my_row < cnt ? exp_ref<false>(mine - m) : 0.0f;
            const float l = warp_sum(e);
            const float *Vs = Vt + (long)c * tile_floats;
            float4 acc;
            switch (tpp) {
            case 32: acc = chunk_values<32>(Vs, XW, e, sub, li); break;
            case 16: acc = chunk_values<16>(Vs, XW, e, sub, li); break;
            case 8: acc = chunk_values<8>(Vs, XW, e, sub, li); break;
            default: acc = chunk_values<4>(Vs, XW, e, sub, li); break;
            }
            float *part = P + (long)c * (XW + 2);
            if (sub == 0) {
                part[2 + 4 * li] = acc.x; part[3 + 4 * li] = acc.y;
                part[4 + 4 * li] = acc.z; part[5 + 4 * li] = acc.w;
            }
            if (lane == 0) { part[0] = m; part[1] = l; }
        } else if (lane == 0) {
            s_bad = 1u;
            if (p.status != nullptr) atomicOr(p.status, 2);
        }
    }
    __syncthreads();
    if (s_bad != 0u) {
        // a tile never landed: one more bounded wait per tile so that none is in flight when
        // this CTA's shared memory is released
        if (threadIdx.x == 0)
            for (int c = 0; c < ns; ++c) {
                mbar_wait(&mbar[c], 0u, SPIN_LIMIT);
                mbar_wait(&mbar[XB_MAX_CHUNKS + c], 0u, SPIN_LIMIT);
            }
        return;
    }
    // merge of the chunk partials, a thread per dimension, and the int8 quantization of the
    // merged row (one warp doing both in turn was a 4 us chain of dependent instructions)
    XB_TICK(5);
    if (!STRICT && threadIdx.x < XW) ctx = merge_dim(P, ns, XW, threadIdx.x);
    const float cmax = block_max1(fabsf(ctx), red);
    const float cinv = cmax > 0.0f ? __fdiv_rn(127.0f, cmax) : 0.0f;
    if (threadIdx.x < XW) ctxq[threadIdx.x] = (int8_t)min(127, max(-127, round_half_away(__fmul_rn(ctx, cinv))));
    const float sxc = cmax > 0.0f ? __fdiv_rn(cmax, 127.0f) : 0.0f;
    __syncthreads();

    XB_TICK(6);
    // ---- output product added to the residual row
    if (INT4) {
#pragma unroll
        for (int i = 0; i < RO; ++i) {
            const int r = (int)threadIdx.x + i * XB_THREADS;
            if (r < W) {
                float acc = 0.0f;
#pragma unroll
                for (int g = 0; g < OG; ++g) {
                    if (g < og) {
                        const uint4 x0 = reinterpret_cast<const uint4 *>(ctxq)[2 * g];
                        const uint4 x1 = reinterpret_cast<const uint4 *>(ctxq)[2 * g + 1];
                        acc = __fadd_rn(acc, __fmul_rn((float)dot_q4_group(wo4[i * OG + g], x0, x1), wog[i * OG + g]));
                    }
                }
                const float xn = __fadd_rn(xres[r], __fmul_rn(acc, sxc));
                row[r] = xn;
                xg[r] = xn;
            }
        }
    } else {
        const uint4 creg = reinterpret_cast<const uint4 *>(ctxq)[lp];
        int part[NI];
#pragma unroll
        for (int u = 0; u < NI; ++u) part[u] = dot16(wo0[u], creg, 0);
        // the LPR lanes of a row exchange halves of their lists: log2(LPR) rounds, after which
        // each lane holds RO complete sums (integers: the order does not matter)
        int n = NI;
#pragma unroll
        for (int m = LPR / 2; m >= 1; m >>= 1) {
            n >>= 1;
            const bool upper = (lp & m) != 0;
#pragma unroll
            for (int i = 0; i < NI / 2; ++i) {
                if (i < n) {
                    const int send = upper ? part[i] : part[i + n];
                    const int keep = upper ? part[i + n] : part[i];
                    part[i] = keep + __shfl_xor_sync(MB_FULL, send, m);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < RO; ++i) {
            const int r = wrow0 + (ubase + i) * RPI + lr;
            if (r < W) {
                const float y = __fmul_rn(__fmul_rn((float)part[i], wos0[i]), sxc);
                const float xn = __fadd_rn(xres[r], y);
                row[r] = xn;
                xg[r] = xn;
            }
        }
    }
    __syncthreads();

    XB_TICK(7);
    // ---- second norm, quantized for the feed-forward product
    const float sx2 = STRICT ? mb_ln_block_strict(row, W, gf, nullptr, p.eps, sq, stat, red, nullptr, true, p.qx + (long)b * W)
                             : mb_ln_block<1>(row, W, gf, nullptr, p.eps, red, nullptr, true, p.qx + (long)b * W);
    if (threadIdx.x == 0) p.sx[b] = sx2;
    XB_TICK(8);
}

size_t cross_block_smem(size_t width, size_t xw, size_t chunks) {
    const size_t floats = 2u * chunks * CHUNK * xw + 5u * width + xw + chunks * (xw + 2u) + 32u + xw;
    return floats * sizeof(float) + width + xw + 16u;
}

bool is_pow2(size_t v) { return v != 0 && (v & (v - 1u)) == 0; }

}  // namespace

extern "C" int mb_cross_block_supported(size_t width, size_t xw, size_t rows) {
    if (rows == 0 || width == 0 || xw == 0) return 0;
    const size_t chunks = (rows + CHUNK - 1) / CHUNK;
    // instantiated: xw = 128 with any width up to 1024, and xw = 32 with width up to 256
    const size_t ro = (width + XB_THREADS - 1) / XB_THREADS;
    if (!(xw == 128 || (xw == 32 && ro == 1))) return 0;
    return chunks <= (size_t)XB_MAX_CHUNKS && chunks <= (size_t)XB_WARPS && is_pow2(xw) && xw >= 16 && xw <= 128 &&
           (width % 16u) == 0 && width <= 1024u && cross_block_smem(width, xw, chunks) <= 225u * 1024u;
}

extern "C" int mb_cross_block(const mb_cross_block_args *a, mb_stream stream) {
    if (a == nullptr || a->x == nullptr || a->gain_query == nullptr || a->gain_ff == nullptr || a->wq == nullptr ||
        a->wo == nullptr || a->wq_scales == nullptr || a->wo_scales == nullptr || a->k_cache == nullptr ||
        a->v_cache == nullptr || a->qx == nullptr || a->sx == nullptr || a->batch == 0)
        return (int)cudaErrorInvalidValue;
    if (!mb_cross_block_supported(a->width, a->xw, a->rows)) return (int)cudaErrorInvalidValue;
    if (a->qtype != MB_INT8 && a->qtype != MB_INT4) return (int)cudaErrorInvalidValue;
    if (a->qtype == MB_INT4 && ((a->width % 32u) != 0 || (a->xw % 32u) != 0)) return (int)cudaErrorInvalidValue;
    if ((((uintptr_t)a->k_cache | (uintptr_t)a->v_cache | (uintptr_t)a->wq | (uintptr_t)a->wo | (uintptr_t)a->x |
          (uintptr_t)a->qx) & 15u) != 0 ||
        (a->slot_stride % a->xw) != 0 || (a->batch > 1 && a->cache_rows == 0))
        return (int)cudaErrorInvalidValue;
    CrossP p;
    memset(&p, 0, sizeof(p));
    p.x = a->x;
    p.gain_query = a->gain_query; p.gain_ff = a->gain_ff;
    p.wq = a->wq; p.wo = a->wo; p.wq_scales = a->wq_scales; p.wo_scales = a->wo_scales;
    p.slots = a->slots; p.n_active = a->n_active; p.rows_per_slot = a->rows_per_slot;
    p.qx = a->qx; p.sx = a->sx; p.status = a->status;
    p.slot_rows = (long)(a->slot_stride / a->xw);
    p.width = (int)a->width; p.xw = (int)a->xw; p.rows = (int)a->rows;
    p.chunks = (int)((a->rows + CHUNK - 1) / CHUNK);
    p.scale = a->scale; p.eps = a->eps;
    p.exp_tab = a->exp_tab;
    const size_t rows = a->cache_rows != 0 ? a->cache_rows : a->rows;
    const unsigned box_cols = a->strict ? 32u : (unsigned)a->xw;
    const CUtensorMapSwizzle swz = a->strict ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUtensorMap kmap, vmap;
    if (!mb_make_map_2d(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->k_cache, rows, a->xw, a->xw * 4u, box_cols, CHUNK, swz) ||
        !mb_make_map_2d(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->v_cache, rows, a->xw, a->xw * 4u, box_cols, CHUNK, swz))
        return (int)cudaErrorInvalidValue;
    const size_t smem = cross_block_smem(a->width, a->xw, (size_t)p.chunks);
    const int ro = (int)((a->width + XB_THREADS - 1) / XB_THREADS);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)a->batch), block(XB_THREADS);
    const int lpr = (int)(a->xw / 16u);
    const bool int4 = a->qtype == MB_INT4;
#define XB_CASE(RO_, LPR_) \
    if (ro == RO_ && lpr == LPR_) { \
        if (a->strict && int4) mb_launch(k_cross_block<RO_, LPR_, true, true>, grid, block, smem, s, kmap, vmap, p); \
        else if (a->strict) mb_launch(k_cross_block<RO_, LPR_, true, false>, grid, block, smem, s, kmap, vmap, p); \
        else if (int4) mb_launch(k_cross_block<RO_, LPR_, false, true>, grid, block, smem, s, kmap, vmap, p); \
        else mb_launch(k_cross_block<RO_, LPR_, false, false>, grid, block, smem, s, kmap, vmap, p); \
    }
    XB_CASE(1, 2); XB_CASE(1, 8); XB_CASE(2, 8); XB_CASE(3, 8); XB_CASE(4, 8);
#undef XB_CASE
    return mb_check_launch();
}

#ifdef MB_PHASE_TICKS
extern "C" __attribute__((visibility("default")))
int mynah_b200_debug_cross_block_ticks(unsigned long long *host, size_t n) {
    if (n > 16u * 1024u) n = 16u * 1024u;
    cudaDeviceSynchronize();
    return (int)cudaMemcpyFromSymbol(host, g_xb_ticks, n * sizeof(unsigned long long));
}
#endif

extern "C" int mb_cross_block_init(void) {
    int rc = 0;
    const int bytes = 225 * 1024;
#define XB_ATTR(RO_, LPR_) \
    rc |= (int)cudaFuncSetAttribute(k_cross_block<RO_, LPR_, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); \
    rc |= (int)cudaFuncSetAttribute(k_cross_block<RO_, LPR_, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); \
    rc |= (int)cudaFuncSetAttribute(k_cross_block<RO_, LPR_, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); \
    rc |= (int)cudaFuncSetAttribute(k_cross_block<RO_, LPR_, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    XB_ATTR(1, 2) XB_ATTR(1, 8) XB_ATTR(2, 8) XB_ATTR(3, 8) XB_ATTR(4, 8)
#undef XB_ATTR
    return rc;
}
