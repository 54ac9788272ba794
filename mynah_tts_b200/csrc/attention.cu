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
// FAST kernel: grid (CTAs per stream, streams), one warp per head.  Positions are cut
// into fixed chunks of 32 rows.  A CTA brings a chunk's K rows and V rows -- whole
// rows, all heads, contiguous in the cache -- into shared memory as TMA tiles
// (completion on an mbarrier, bounded wait) and each warp computes its head's
// partial (max, sum, weighted V) of that chunk without leaving the warp.  Partials
// go to a scratch buffer; the last CTA of a stream to finish (an atomic counter per
// stream; none when one CTA owns the stream) merges every head's chunks in index
// order and, when the next projection wants int8 input, quantizes the merged row.
// Results depend neither on arrival order nor on the batch a stream is stepped in.
#include "common.cuh"
#include "launch.h"
#include "tma.cuh"
#include "attn_tiles.cuh"

#include <float.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace {

struct AttnP {
    const float *q, *k_new, *v_new;
    float *k_cache, *v_cache;
    const int *slots, *lens, *n_active;
    const int *valids;   // lens == nullptr: rows attended by the lane in slot s, or nullptr (p.valid)
    float *out;
    int8_t *qx;
    float *sx;
    float *partials;
    unsigned *counters;
    int *status;
    const uint32_t *exp_tab;
    long q_stride, slot_stride, cache_stride, out_stride;
    long position, valid;
    int heads, hw, batch, max_chunks, splits;
    long slot_rows;      // cache rows between consecutive slots (slot_stride / cache_stride)
    int box_cols, nbox;  // a 32-row tile is nbox TMA boxes of box_cols columns
    int depth;           // ring slots per tile kind (K, V)
    int ps, map4d;       // k_attn_exact: 128-byte segments per tile row (odd), rank of its tensor maps
    int mchunks;         // k_attn_exact: 32-row chunks per copy
    int inv_norm;        // strict kernels: weights e * (1 / den) (the reference's multi-row softmax) instead of e / den
    int early;           // first tiles are requested before the dependency wait
    float scale;
};

__device__ __forceinline__ bool lane_setup(const AttnP &p, int b, long &pos, long &valid,
                                           float *&kc, float *&vc, long *slot_out = nullptr) {
    // the three lane-state words are fetched together: one memory round trip, not three
    const int live = p.n_active != nullptr ? *p.n_active : 0x7fffffff;
    const long len = p.lens != nullptr ? (long)p.lens[b] : 0L;
    const long slot = p.slots != nullptr ? (long)p.slots[b] : (long)b;
    if (b >= live) return false;
    if (slot_out != nullptr) *slot_out = slot;
    if (p.lens != nullptr) { pos = len; valid = pos + 1; }
    else {
        pos = p.position;
        valid = p.valid;
        if (p.valids != nullptr) valid = min((long)max(p.valids[slot], 1), p.valid);
    }
    kc = p.k_cache + slot * p.slot_stride;
    vc = p.v_cache + slot * p.slot_stride;
    return true;
}

// ------------------------------------------------------------------ strict
__global__ void __launch_bounds__(256) k_attn_strict(AttnP p) {
    mb_pdl_wait();
    mb_pdl_trigger();
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
        sc[s] = exp_ref<true>(__fsub_rn(sc[s], m), p.exp_tab);
    __syncthreads();
    if (threadIdx.x == 0) {
        float den = 0.0f;
        for (long s = 0; s < valid; ++s) den = __fadd_rn(den, sc[s]);
        s_denom = den;
    }
    __syncthreads();
    const float den = s_denom;
    if (p.inv_norm) {
        const float inv = den > 0.0f ? __fdiv_rn(1.0f, den) : 0.0f;
        for (long s = threadIdx.x; s < valid; s += blockDim.x) sc[s] = __fmul_rn(sc[s], inv);
    } else {
        for (long s = threadIdx.x; s < valid; s += blockDim.x) sc[s] = __fdiv_rn(sc[s], den);
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hw; d += blockDim.x) {
        float a = 0.0f;
        for (long s = 0; s < valid; ++s)
            a = __fadd_rn(a, __fmul_rn(sc[s], vh[s * p.cache_stride + d]));
        p.out[(long)b * p.out_stride + (long)h * hw + d] = a;
    }
}

// ------------------------------------------------------------------ short caches
// A cache of at most 32 rows (the local transformer's: one row per stacked stream of the
// frame): one CTA per stream, a thread per column.  Everything a thread needs from global
// memory -- its column of V, then the rows of K -- is requested up front, so the launch is a
// few memory round trips, not a ring of copies with its set-up and tail.  Every sum runs in
// the reference's order (scores as one chain over the head's width, the denominator and each
// context element as one chain over the rows), so strict mode gives the bits of the other
// strict kernels; fast mode only swaps expf.
constexpr int SMALL_ROWS = 32;
template <bool STRICT>
__global__ void __launch_bounds__(1024) k_attn_small(AttnP p) {
    extern __shared__ float sm_small[];
    __shared__ float red[33];
    mb_pdl_wait();
    mb_pdl_trigger();
    const int b = blockIdx.x;
    long pos, valid_l;
    float *kc, *vc;
    if (!lane_setup(p, b, pos, valid_l, kc, vc)) return;
    const int valid = (int)valid_l, hw = p.hw, W = p.heads * p.hw;
    float *qs = sm_small;                       // [W]
    float *sc = qs + W;                         // [heads][SMALL_ROWS]
    float *row = sc + p.heads * SMALL_ROWS;     // [W] the context row (for the quantization)
    const int c = threadIdx.x;                  // this thread's column
    float vr[SMALL_ROWS];
    if (c < W) {
        qs[c] = p.q[(long)b * p.q_stride + c];
        float vnew = 0.0f;
        if (p.k_new != nullptr) {
            kc[pos * p.cache_stride + c] = p.k_new[(long)b * p.q_stride + c];
            vnew = p.v_new[(long)b * p.q_stride + c];
            vc[pos * p.cache_stride + c] = vnew;
        }
#pragma unroll
        for (int s = 0; s < SMALL_ROWS; ++s)
            vr[s] = s < valid ? ((p.k_new != nullptr && s == (int)pos) ? vnew : vc[(long)s * p.cache_stride + c]) : 0.0f;
    }
    __syncthreads();
    // scores: a thread per (head, row), the row's hw values in registers sixteen at a time
    for (int idx = threadIdx.x; idx < p.heads * valid; idx += blockDim.x) {
        const int h = idx / valid, s = idx - h * valid;
        const float *k = kc + (long)s * p.cache_stride + h * hw;
        const float *qh = qs + h * hw;
        float dot = 0.0f;
        for (int d0 = 0; d0 < hw; d0 += 16) {
            float kr[16];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
                const float4 f = d0 + 4 * j4 < hw ? *reinterpret_cast<const float4 *>(k + d0 + 4 * j4) : make_float4(0.f, 0.f, 0.f, 0.f);
                kr[4 * j4] = f.x; kr[4 * j4 + 1] = f.y; kr[4 * j4 + 2] = f.z; kr[4 * j4 + 3] = f.w;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (d0 + j < hw) dot = __fadd_rn(dot, __fmul_rn(qh[d0 + j], kr[j]));
        }
        sc[h * SMALL_ROWS + s] = __fmul_rn(dot, p.scale);
    }
    __syncthreads();
    // softmax of a head by one warp: lane s holds row s
    for (int h = threadIdx.x >> 5; h < p.heads; h += blockDim.x >> 5) {
        const int lane = threadIdx.x & 31;
        const float a = lane < valid ? sc[h * SMALL_ROWS + lane] : -FLT_MAX;
        const float m = warp_max(a);
        const float e = lane < valid ? exp_ref<STRICT>(__fsub_rn(a, m), p.exp_tab) : 0.0f;
        float den = 0.0f;
        for (int s = 0; s < valid; ++s) den = __fadd_rn(den, __shfl_sync(MB_FULL, e, s));   // rows in order
        float w;
        if (p.inv_norm) w = __fmul_rn(e, den > 0.0f ? __fdiv_rn(1.0f, den) : 0.0f);
        else w = __fdiv_rn(e, den);
        if (lane < valid) sc[h * SMALL_ROWS + lane] = w;
    }
    __syncthreads();
    float acc = 0.0f;
    if (c < W) {
        const float *w = sc + (c / hw) * SMALL_ROWS;
#pragma unroll
        for (int s = 0; s < SMALL_ROWS; ++s)
            if (s < valid) acc = __fadd_rn(acc, __fmul_rn(w[s], vr[s]));
        if (p.out != nullptr) p.out[(long)b * p.out_stride + c] = acc;
    }
    if (p.qx != nullptr) {
        // per-row int8 quantization of the context (src/qmat.c:93-113), as mb_quant_rows
        const float amax = block_max(c < W ? fabsf(acc) : 0.0f, red);
        const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        if (c < W) p.qx[(long)b * W + c] = (int8_t)min(127, max(-127, round_half_away(__fmul_rn(acc, inv))));
        if (threadIdx.x == 0) p.sx[b] = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    }
    (void)row;
}


}  // namespace
#include "attn_exact.cuh"
namespace {

// -------------------------------------------------------------------- fast
// Positions are cut into fixed chunks of CHUNK rows: the partition depends only on
// the stream's own length, never on how many streams are stepped together, so a
// stream's result is bit-identical whatever batch it runs in.
// (CHUNK, the tile helpers and the merge live in attn_tiles.cuh)

// One CTA = one stream (lane), a group of its heads (warp w is head h0 + w) and a subset
// of its 32-row chunks.  A chunk's K rows (32 rows x the group's columns, whole rows when
// the group is all heads) come in as one tile, its V rows as another; wide row pieces
// keep DRAM pages open (head-sliced 256-byte reads were measured at 29% of HBM peak).
// K and V tiles each go through a ring of p.depth slots, so while the warps work on one
// tile the next 2 * depth - 1 are landing.
constexpr int RING_MAX = 4;
// MAXT: most threads of a launch (32 per head).  The 1024-thread bound caps the kernel at 64
// registers; an instantiation bounded at 384 threads (twelve heads) gets 160 and is faster
// where the launch is bound by bandwidth (64 streams: 882 against 889 us per step) but slower
// for a few streams (one stream: 497 against 486), so it is taken from 32 streams.
template <int MAXT>
__global__ void __launch_bounds__(MAXT, 1)
k_attn_rows(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, AttnP p) {
    // With p.early the dependency wait comes AFTER the first tiles are requested.  The caller
    // then vouches that what is read before it (lane state, cache rows below `pos`) was
    // written at least two launches back: every launch waits for its predecessor before it
    // lets its successor start, so all of that is complete, and only q and the new K/V rows
    // come from the immediate predecessor.
    if (!p.early) {
        mb_pdl_wait();
        mb_pdl_trigger();
    }
    // a name of its own: a redeclaration of another kernel's array would take that one's alignment,
    // and the TMA tiles need 128 bytes
    extern __shared__ __align__(128) float sm_rows[];
    float *sm = sm_rows;
    __shared__ float red[33];
    __shared__ unsigned s_last;
    __shared__ __align__(8) unsigned long long mbar[2 * RING_MAX];   // K slots, then V slots
    const int sp = blockIdx.x, b = blockIdx.y;
    long pos, valid;
    float *kc, *vc;
    long slot;
    if (!lane_setup(p, b, pos, valid, kc, vc, &slot)) return;
    const int ns = (int)((valid + CHUNK - 1) / CHUNK);      // chunks of this stream
    const int splits = p.splits;                             // CTAs that share a stream
    if (sp >= ns) return;
    const int hw = p.hw, heads = p.heads, width = heads * hw;
    const int hg = blockDim.x >> 5;                          // heads (= warps) of this CTA
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h0 = blockIdx.z * hg, h = h0 + warp;           // this warp's head
    const int cwidth = hg * hw;                              // columns this CTA covers
    const int tpp = hw / 4;                         // float4 lanes per row (power of two <= 32)
    const int rps = 32 / tpp;                       // rows a warp covers per step
    const int sub = lane / tpp, li = lane % tpp;
    const int tile_floats = CHUNK * cwidth;
    const int depth = p.depth;
    float *Kt = sm;                                 // [depth][nbox][CHUNK][box_cols]
    float *Vt = sm + (long)depth * tile_floats;
    float *qs = Vt + (long)depth * tile_floats;     // [cwidth]
    float *wts = qs + cwidth + warp * p.max_chunks; // this warp's merge weights
    const long hoff = (long)h * hw;
    const float *knew = p.k_new == nullptr ? nullptr : p.k_new + (long)b * p.q_stride;
    const float *vnew = p.v_new == nullptr ? nullptr : p.v_new + (long)b * p.q_stride;
    const unsigned tile_bytes = (unsigned)tile_floats * 4u;
    // this CTA's j-th tile (chunk sp + j * splits) goes to ring slot j % depth:
    // p.nbox boxes of box_cols columns x 32 rows each
    const int mine_chunks = sp < ns ? (ns - sp + splits - 1) / splits : 0;
    // cache rows are read once per launch: they must not push weights, activations and
    // code out of L2
    const unsigned long long stream_policy = mb_l2_evict_first();
    auto issue = [&](const CUtensorMap *map, float *ring, int j, int first_bar) {
        const int c = sp + j * splits, rs = j % depth;
        const int y = (int)(slot * p.slot_rows + (long)c * CHUNK);
        float *tile = ring + (long)rs * tile_floats;
        mbar_expect_tx(&mbar[first_bar + rs], tile_bytes);
        for (int bx = 0; bx < p.nbox; ++bx)
            mb_tma_load_2d_hint(tile + (long)bx * CHUNK * p.box_cols, map, h0 * hw + bx * p.box_cols, y,
                                &mbar[first_bar + rs], stream_policy);
    };
    // A wait ran out at this CTA's tile `it`: flag it, give every copy still in flight one
    // more bounded wait so none lands after this CTA's shared memory is released.
    auto drain = [&](int it, int k_issued, int v_issued) {
        if (threadIdx.x == 0) {
            if (p.status != nullptr) atomicOr(p.status, 2);
            for (int j = it; j < k_issued; ++j) mbar_wait(&mbar[j % depth], (unsigned)((j / depth) & 1), SPIN_LIMIT);
            for (int j = it; j < v_issued; ++j)
                mbar_wait(&mbar[depth + j % depth], (unsigned)((j / depth) & 1), SPIN_LIMIT);
        }
        __syncthreads();
    };
    // the first tiles start before anything else of the prologue: the copy engine works
    // while the threads fetch q and append the new row
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * depth; ++i) mbar_init(&mbar[i], 1u);
        for (int j = 0; j < depth && j < mine_chunks; ++j) {
            issue(&kmap, Kt, j, 0);
            issue(&vmap, Vt, j, depth);
        }
    }
    if (p.early) {
        mb_pdl_wait();
        mb_pdl_trigger();
    }
    // q into shared memory and the new K/V row into the cache: all loads of a batch are
    // issued before its stores, so they overlap instead of queueing behind one another.
    // One CTA per (stream, head group) appends; readers of row `pos` take it from the new
    // row, never from the cache.
    const bool append = knew != nullptr && sp == 0;
    for (int d0 = threadIdx.x; d0 < cwidth; d0 += 4 * blockDim.x) {
        float qq[4], kk[4], vv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int d = d0 + u * blockDim.x;
            const long col = (long)h0 * hw + d;
            if (d < cwidth) {
                qq[u] = p.q[(long)b * p.q_stride + col];
                if (append) { kk[u] = knew[col]; vv[u] = vnew[col]; }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int d = d0 + u * blockDim.x;
            const long col = (long)h0 * hw + d;
            if (d < cwidth) {
                qs[d] = qq[u];
                if (append) {
                    kc[pos * p.cache_stride + col] = kk[u];
                    vc[pos * p.cache_stride + col] = vv[u];
                }
            }
        }
    }
    __syncthreads();
    // this head's slice inside a tile: box, column offset, row pitch
    const long slice = (long)((warp * hw) / p.box_cols) * CHUNK * p.box_cols + (warp * hw) % p.box_cols;
    const int pitch = p.box_cols;
    const float4 qv = reinterpret_cast<const float4 *>(qs + warp * hw)[li];
    bool failed = false;                                     // a tile never landed (CTA-uniform)
    for (int it = 0; it < mine_chunks; ++it) {
        const int c = sp + it * splits, rs = it % depth;
        const unsigned parity = (unsigned)((it / depth) & 1);
        const int issued = min(mine_chunks, it + depth);     // tiles of each kind issued so far
        const long s0 = (long)c * CHUNK;
        const int cnt = (int)min((long)CHUNK, valid - s0);
        const bool fresh = knew != nullptr && pos >= s0 && pos < s0 + cnt;
        // ---- K tile ---------------------------------------------------------------------
        if (__syncthreads_or(mbar_wait(&mbar[rs], parity, SPIN_LIMIT) ? 0 : 1)) {
            drain(it, issued, issued);
            failed = true;
            break;
        }
        float *Ks = Kt + (long)rs * tile_floats + slice;
        if (fresh) {
            // the row being appended now may not have reached the cache when the tile was
            // read: take it from the new K row itself
            for (int d = lane; d < hw; d += 32) Ks[(pos - s0) * pitch + d] = knew[hoff + d];
            __syncwarp();
        }
        // scores: tpp lanes share a row, rps rows per step; lane (sub, li) keeps the score
        // of row li * rps + sub
        float dot;
        switch (tpp) {
        case 32: dot = chunk_scores<32>(Ks, pitch, qv, sub, li); break;
        case 16: dot = chunk_scores<16>(Ks, pitch, qv, sub, li); break;
        case 8: dot = chunk_scores<8>(Ks, pitch, qv, sub, li); break;
        case 4: dot = chunk_scores<4>(Ks, pitch, qv, sub, li); break;
        case 2: dot = chunk_scores<2>(Ks, pitch, qv, sub, li); break;
        default: dot = chunk_scores<1>(Ks, pitch, qv, sub, li); break;
        }
        const float mine = li * rps + sub < cnt ? dot * p.scale : -FLT_MAX;
        const float m = warp_max(mine);
        const int my_row = li * rps + sub;
        const float e = my_row < cnt ? exp_ref<false>(mine - m) : 0.0f;
        const float l = warp_sum(e);
        __syncthreads();                                     // every warp is done with the K tile
        const bool more = it + depth < mine_chunks;
        if (threadIdx.x == 0 && more) issue(&kmap, Kt, it + depth, 0);
        // ---- V tile ---------------------------------------------------------------------
        if (__syncthreads_or(mbar_wait(&mbar[depth + rs], parity, SPIN_LIMIT) ? 0 : 1)) {
            drain(it, more ? issued + 1 : issued, issued);
            failed = true;
            break;
        }
        float *Vs = Vt + (long)rs * tile_floats + slice;
        if (fresh) {
            for (int d = lane; d < hw; d += 32) Vs[(pos - s0) * pitch + d] = vnew[hoff + d];
            __syncwarp();
        }
        // weighted V: the sub-groups take interleaved rows, then add up
        float4 acc;
        switch (tpp) {
        case 32: acc = chunk_values<32>(Vs, pitch, e, sub, li); break;
        case 16: acc = chunk_values<16>(Vs, pitch, e, sub, li); break;
        case 8: acc = chunk_values<8>(Vs, pitch, e, sub, li); break;
        case 4: acc = chunk_values<4>(Vs, pitch, e, sub, li); break;
        case 2: acc = chunk_values<2>(Vs, pitch, e, sub, li); break;
        default: acc = chunk_values<1>(Vs, pitch, e, sub, li); break;
        }
        // this chunk's partial (max, sum, weighted V) of head h
        float *part = p.partials + (((long)b * heads + h) * p.max_chunks + c) * (hw + 2);
        if (sub == 0) {
            part[2 + 4 * li] = acc.x; part[3 + 4 * li] = acc.y;
            part[4 + 4 * li] = acc.z; part[5 + 4 * li] = acc.w;
        }
        if (lane == 0) { part[0] = m; part[1] = l; }
        __syncthreads();                                     // every warp is done with the V tile
        if (threadIdx.x == 0 && more) issue(&vmap, Vt, it + depth, depth);
    }
    const int groups = (int)gridDim.z;
    const bool quant = p.qx != nullptr;
    float *outrow = p.out == nullptr ? nullptr : p.out + (long)b * p.out_stride;
    // staging of the merged row when its head groups sit in different CTAs
    float *merged = p.partials == nullptr
                        ? nullptr
                        : p.partials + (long)p.batch * heads * p.max_chunks * (hw + 2) + (long)b * width;
    const int per_head = ns * (hw + 2);
    float *vals;                                             // merged row, for the quantization pass
    if (failed) return;
    {
        // ---- the head group's last CTA merges its heads ------------------------------------
        __threadfence();
        __syncthreads();
        if (min(ns, splits) > 1) {                           // several CTAs shared this head group
            if (threadIdx.x == 0) {
                unsigned *ctr = p.counters + (long)b * groups + blockIdx.z;
                const unsigned prev = atomicAdd(ctr, 1u);
                s_last = prev == (unsigned)min(ns, splits) - 1u;
                if (s_last) *ctr = 0u;
            }
            __syncthreads();
            if (!s_last) return;
            __threadfence();
        }
        // Every tile has been consumed, so the tile memory is free: bring this head group's
        // partials into it with one round of independent, coalesced loads (walking them from
        // global memory inside the ordered sums would pay one memory round trip per chunk),
        // then merge out of shared memory.  The merged row for the quantization pass sits
        // behind them.  Streams too long for that keep the partials in global memory.
        const long tile_room = 2L * depth * tile_floats;
        const bool staged = (long)hg * per_head + width <= tile_room;
        float *stage = Kt;
        vals = staged ? Kt + (long)hg * per_head : Kt;
        if (staged) {
            const float *src = p.partials + ((long)b * heads + h0) * p.max_chunks * (hw + 2);
            const long head_pitch = (long)p.max_chunks * (hw + 2);
            const int total = hg * per_head;
            for (int i0 = threadIdx.x; i0 < total; i0 += 8 * blockDim.x) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * blockDim.x;
                    const int w = i / per_head, o = i - w * per_head;
                    if (i < total) v[u] = __ldcg(src + w * head_pitch + o);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = i0 + u * blockDim.x;
                    if (i < total) stage[i] = v[u];
                }
            }
            __syncthreads();
        }
        auto emit = [&](int d, float o) {
            if (outrow != nullptr) outrow[hoff + d] = o;
            if (quant) {
                if (groups == 1) vals[hoff + d] = o;         // behind the staged partials
                else merged[hoff + d] = o;
            }
        };
        if (staged) merge_chunks<false>(stage + (long)warp * per_head, ns, hw, lane, wts, emit);
        else merge_chunks<true>(p.partials + ((long)b * heads + h) * p.max_chunks * (hw + 2), ns, hw, lane, wts, emit);
    }
    if (!quant) return;
    // ---- the stream's last head group quantizes the whole row ---------------------------
    if (groups > 1) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned *ctr = p.counters + (long)p.batch * groups + b;
            const unsigned prev = atomicAdd(ctr, 1u);
            s_last = prev == (unsigned)groups - 1u;
            if (s_last) *ctr = 0u;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        for (int i = threadIdx.x; i < width; i += blockDim.x) vals[i] = __ldcg(merged + i);
    }
    __syncthreads();
    quantize_shared_row(vals, width, p.qx + (long)b * width, p.sx + b, red);
}

// ------------------------------------------------------------- short caches
// A cache short enough that every (head, chunk) pair gets its own warp of one CTA (cross
// attention over the text memory: 1 head x 4 chunks): all K and V tiles are requested at
// once, each warp makes its chunk's partial, and the partials meet in shared memory -- no
// scratch in global memory, no arrival counter, no fence.  No row is appended (k_new is
// null).  Per (head, chunk) and in the merge the operations and their order are those of
// k_attn_rows: results are bit-identical.
constexpr int SHORT_MAX_CHUNKS = 8;
// MAXT: most threads of a launch; the cross attention's four warps get an instantiation
// bounded at 128 threads (the 1024-thread bound caps the registers at 64).
template <int MAXT>
__global__ void __launch_bounds__(MAXT, 1)
k_attn_short(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, AttnP p) {
    extern __shared__ __align__(128) float sm_short[];      // (own name: see k_attn_rows)
    float *sm = sm_short;
    __shared__ float red[33];
    __shared__ __align__(8) unsigned long long mbar[2 * SHORT_MAX_CHUNKS];   // K chunks, then V chunks
    __shared__ unsigned s_bad;
    if (!p.early) {
        mb_pdl_wait();
        mb_pdl_trigger();
    }
    const int b = blockIdx.x;
    long pos, valid, slot;
    float *kc, *vc;
    if (!lane_setup(p, b, pos, valid, kc, vc, &slot)) return;
    const int hw = p.hw, heads = p.heads, width = heads * hw;
    const int cmax = p.max_chunks;
    const int ns = (int)((valid + CHUNK - 1) / CHUNK);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = warp % heads, c = warp / heads;             // this warp's head and chunk
    const int tpp = hw / 4, rps = 32 / tpp, sub = lane / tpp, li = lane % tpp;
    const int tile_floats = CHUNK * width;
    float *Kt = sm;                                           // [cmax] tiles
    float *Vt = Kt + (long)cmax * tile_floats;
    float *qs = Vt + (long)cmax * tile_floats;                // [width]
    float *P = qs + width;                                    // [heads][cmax][hw + 2]
    float *wts = P + (long)heads * cmax * (hw + 2) + (long)h * 2 * cmax;   // merge scratch of head h
    float *vals = P + (long)heads * cmax * (hw + 2) + (long)heads * 2 * cmax;   // [width]
    const unsigned tile_bytes = (unsigned)tile_floats * 4u;
    if (threadIdx.x == 0) {
        s_bad = 0u;
        const unsigned long long stream_policy = mb_l2_evict_first();
        for (int i = 0; i < 2 * cmax; ++i) mbar_init(&mbar[i], 1u);
        for (int cc = 0; cc < ns; ++cc) {
            const int y = (int)(slot * p.slot_rows + (long)cc * CHUNK);
            mbar_expect_tx(&mbar[cc], tile_bytes);
            mbar_expect_tx(&mbar[cmax + cc], tile_bytes);
            for (int bx = 0; bx < p.nbox; ++bx) {
                mb_tma_load_2d_hint(Kt + (long)cc * tile_floats + (long)bx * CHUNK * p.box_cols, &kmap, bx * p.box_cols, y,
                                    &mbar[cc], stream_policy);
                mb_tma_load_2d_hint(Vt + (long)cc * tile_floats + (long)bx * CHUNK * p.box_cols, &vmap, bx * p.box_cols, y,
                                    &mbar[cmax + cc], stream_policy);
            }
        }
    }
    if (p.early) {
        mb_pdl_wait();
        mb_pdl_trigger();
    }
    for (int d = threadIdx.x; d < width; d += blockDim.x) qs[d] = p.q[(long)b * p.q_stride + d];
    __syncthreads();
    if (c < ns) {
        const long slice = (long)((h * hw) / p.box_cols) * CHUNK * p.box_cols + (h * hw) % p.box_cols;
        const int pitch = p.box_cols;
        const float4 qv = reinterpret_cast<const float4 *>(qs + h * hw)[li];
        const long s0 = (long)c * CHUNK;
        const int cnt = (int)min((long)CHUNK, valid - s0);
        const bool k_ok = mbar_wait(&mbar[c], 0u, SPIN_LIMIT);
        const bool v_ok = k_ok && mbar_wait(&mbar[cmax + c], 0u, SPIN_LIMIT);
        if (k_ok && v_ok) {
            const float *Ks = Kt + (long)c * tile_floats + slice;
            float dot;
            switch (tpp) {
            case 32: dot = chunk_scores<32>(Ks, pitch, qv, sub, li); break;
            case 16: dot = chunk_scores<16>(Ks, pitch, qv, sub, li); break;
            case 8: dot = chunk_scores<8>(Ks, pitch, qv, sub, li); break;
            case 4: dot = chunk_scores<4>(Ks, pitch, qv, sub, li); break;
            case 2: dot = chunk_scores<2>(Ks, pitch, qv, sub, li); break;
            default: dot = chunk_scores<1>(Ks, pitch, qv, sub, li); break;
            }
            const int my_row = li * rps + sub;
            const float mine = my_row < cnt ? dot * p.scale : -FLT_MAX;
            const float m = warp_max(mine);
            const float e = my_row < cnt ? exp_ref<false>(mine - m) : 0.0f;
            const float l = warp_sum(e);
            const float *Vs = Vt + (long)c * tile_floats + slice;
            float4 acc;
            switch (tpp) {
            case 32: acc = chunk_values<32>(Vs, pitch, e, sub, li); break;
            case 16: acc = chunk_values<16>(Vs, pitch, e, sub, li); break;
            case 8: acc = chunk_values<8>(Vs, pitch, e, sub, li); break;
            case 4: acc = chunk_values<4>(Vs, pitch, e, sub, li); break;
            case 2: acc = chunk_values<2>(Vs, pitch, e, sub, li); break;
            default: acc = chunk_values<1>(Vs, pitch, e, sub, li); break;
            }
            float *part = P + ((long)h * cmax + c) * (hw + 2);
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
            for (int cc = 0; cc < ns; ++cc) {
                mbar_wait(&mbar[cc], 0u, SPIN_LIMIT);
                mbar_wait(&mbar[cmax + cc], 0u, SPIN_LIMIT);
            }
        return;
    }
    const bool quant = p.qx != nullptr;
    float *outrow = p.out == nullptr ? nullptr : p.out + (long)b * p.out_stride;
    if (warp < heads) {
        const long hoff = (long)h * hw;
        merge_chunks<false>(P + (long)h * cmax * (hw + 2), ns, hw, lane, wts, [&](int d, float o) {
            if (outrow != nullptr) outrow[hoff + d] = o;
            if (quant) vals[hoff + d] = o;
        });
    }
    if (!quant) return;
    __syncthreads();
    quantize_shared_row(vals, width, p.qx + (long)b * width, p.sx + b, red);
}

// Shapes the chunked kernel cannot take (head width not a power-of-two multiple
// of 4, or unaligned rows): one CTA per (head, stream), plain loads, no split.
__global__ void __launch_bounds__(FAST_THREADS) k_attn_scalar(AttnP p) {
    mb_pdl_wait();
    mb_pdl_trigger();
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[33];
    const int h = blockIdx.x, b = blockIdx.y;
    long pos, valid;
    float *kc, *vc;
    if (!lane_setup(p, b, pos, valid, kc, vc)) return;
    const int hw = p.hw, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *qs = sm;
    float *sc = sm + hw;
    const long hoff = (long)h * hw;
    const float *knew = p.k_new == nullptr ? nullptr : p.k_new + (long)b * p.q_stride + hoff;
    const float *vnew = p.v_new == nullptr ? nullptr : p.v_new + (long)b * p.q_stride + hoff;
    for (int d = threadIdx.x; d < hw; d += blockDim.x) {
        qs[d] = p.q[(long)b * p.q_stride + hoff + d];
        if (knew != nullptr) {
            kc[pos * p.cache_stride + hoff + d] = knew[d];
            vc[pos * p.cache_stride + hoff + d] = vnew[d];
        }
    }
    __syncthreads();
    float lmax = -FLT_MAX;
    for (long s = warp; s < valid; s += FAST_THREADS / 32) {
        const float *src = (knew != nullptr && s == pos) ? knew : kc + s * p.cache_stride + hoff;
        float a = 0.0f;
        for (int d = lane; d < hw; d += 32) a = fmaf(qs[d], src[d], a);
        a = warp_sum(a);
        if (lane == 0) {
            a *= p.scale;
            sc[s] = a;
            lmax = fmaxf(lmax, a);
        }
    }
    const float m = block_max(lmax, red);
    float lsum = 0.0f;
    for (long s = threadIdx.x; s < valid; s += blockDim.x) {
        const float e = exp_ref<false>(sc[s] - m);
        sc[s] = e;
        lsum += e;
    }
    const float l = block_sum(lsum, red);
    for (int d = threadIdx.x; d < hw; d += blockDim.x) {
        float a = 0.0f;
        for (long s = 0; s < valid; ++s) {
            const float *src = (vnew != nullptr && s == pos) ? vnew : vc + s * p.cache_stride + hoff;
            a = fmaf(sc[s], src[d], a);
        }
        p.out[(long)b * p.out_stride + hoff + d] = l > 0.0f ? a / l : 0.0f;
    }
}

bool is_pow2(long v) { return v > 0 && (v & (v - 1)) == 0; }

size_t chunks_for(size_t max_valid) { return (max_valid + CHUNK - 1) / CHUNK; }


int env_int(const char *name) {
    const char *v = getenv(name);
    return v == nullptr ? 0 : atoi(v);
}

// The streaming reference-order kernel (attn_exact.cuh) where the shape allows it: heads are
// dealt to CTAs in groups whose columns fill whole 32-float boxes; about one CTA per SM.
// Returns false (nothing launched) when the shape needs the plain strict kernel.
bool launch_exact(const mb_attn_args *a, AttnP &p, cudaStream_t s) {
    static const int force_groups = env_int("MYNAH_B200_ATTN_GROUPS");
    static const int force_depth = env_int("MYNAH_B200_ATTN_DEPTH");
    static const int off = env_int("MYNAH_B200_NO_EXACT_ATTN");
    if (off || (p.hw % 4) != 0 || (p.cache_stride % 4) != 0 || (p.q_stride % 4) != 0 ||
        (p.slot_stride % 4) != 0 || (p.cache_stride != 0 && (p.slot_stride % p.cache_stride) != 0) ||
        !(a->batch == 1 || a->cache_rows != 0) ||
        (((uintptr_t)a->k_cache | (uintptr_t)a->v_cache) & 15u) != 0 ||
        (a->qx != nullptr && (a->counters == nullptr || a->sx == nullptr)))
        return false;
    const int sms = a->sm_count > 0 ? a->sm_count : 148;
    // Head groups per stream: enough CTAs to cover the SMs about one and a half times with
    // groups of three or more heads (cache rows are then read in runs of 768 bytes or more),
    // else the first count that covers them once, else as many groups as the shape allows.
    int best_g = 0, best_depth = 0, cover_g = 0, cover_depth = 0, many_g = 0, many_depth = 0;
    double many_fill = 0.0;
    long many_off = 0;
    int many_per_sm = 0;
    for (int g = 1; g <= p.heads; ++g) {
        if (p.heads % g != 0) continue;
        if (force_groups > 0 && g != force_groups) continue;
        const int hg = p.heads / g, cw = hg * p.hw;
        const int threads = cw > hg * 32 ? cw : hg * 32;
        if ((cw % EX_SEG) != 0 || threads > 1024) continue;
        const int mch = exact_chunks_per_copy(hg, p.hw, p.max_chunks);
        auto depth_for = [&](size_t room) {
            int depth = 0;
            for (int d = EX_RING_MAX; d >= 1 && depth == 0; --d)
                if (exact_smem(hg, p.hw, p.max_chunks, d, mch) + 1024u <= room) depth = d;
            return depth;
        };
        // more CTAs than SMs: two of them share an SM if each still gets a ring of two tiles
        int depth = (long)p.batch * g > sms ? depth_for((size_t)110 * 1024) : 0;
        const int per_sm = depth >= 2 ? 2 : 1;
        if (depth < 2) depth = depth_for((size_t)ROWS_SMEM_MAX);
        if (depth > 2 * ((p.max_chunks + mch - 1) / mch)) depth = 2 * ((p.max_chunks + mch - 1) / mch);
        if (force_depth > 0 && force_depth < depth) depth = force_depth;
        if (depth < 1) continue;
        // many streams (128 or more): among groups of three or more heads keep the split whose
        // CTAs fill whole waves best; of equally full ones the split closest to three waves, then
        // the one that puts two CTAs on an SM (measured at position 256: 256 streams 140 / 116 /
        // 100 / 109 us for 1 / 2 / 3 / 4 groups; 128 streams 63 / 67 / 60 us for 2 / 3 / 4 groups)
        if (p.batch >= 128 && hg >= 3 && force_groups <= 0) {
            const long ctas = (long)p.batch * g, slots = (long)sms * per_sm;
            const long waves = (ctas + slots - 1) / slots;
            const double fill = (double)ctas / (double)(waves * slots);
            const long off = waves > 3 ? waves - 3 : 3 - waves;
            if (many_g == 0 || fill > many_fill + 0.05 ||
                (fill > many_fill - 0.05 && (off < many_off || (off == many_off && per_sm > many_per_sm)))) {
                many_g = g; many_depth = depth; many_fill = fill > many_fill ? fill : many_fill; many_off = off;
                many_per_sm = per_sm;
            }
        }
        best_g = g;
        best_depth = depth;
        if (force_groups > 0) break;
        if (cover_g == 0 && (long)p.batch * g >= sms) { cover_g = g; cover_depth = depth; }
        if (2L * p.batch * g >= 3L * sms && hg >= 3) {
            cover_g = g;
            cover_depth = depth;
            if (p.batch < 128) break;          // many streams: every split of three or more heads is weighed above
        }
        if (hg < 3 && cover_g != 0) break;
    }
    if (cover_g != 0 && force_groups <= 0) { best_g = cover_g; best_depth = cover_depth; }
    if (many_g != 0 && force_groups <= 0) { best_g = many_g; best_depth = many_depth; }
    if (best_g == 0) return false;
    const int hg = p.heads / best_g, cw = hg * p.hw;
    const int threads = cw > hg * 32 ? cw : hg * 32;
    p.depth = best_depth;
    p.splits = 1;
    p.early = a->early_prefetch ? 1 : 0;
    p.slot_rows = p.cache_stride != 0 ? p.slot_stride / p.cache_stride : 0;
    p.box_cols = EX_SEG;
    p.nbox = 1;
    p.ps = exact_pitch_segments(hg, p.hw);
    p.mchunks = exact_chunks_per_copy(hg, p.hw, p.max_chunks);
    size_t rows = a->cache_rows;
    if (rows == 0) rows = (size_t)(p.valid > p.position + 1 ? p.valid : p.position + 1);
    const size_t nseg = (size_t)cw / EX_SEG, row_bytes = (size_t)p.cache_stride * 4u;
    CUtensorMap kmap, vmap;
    // (float of a segment, segment of the group, group, cache row): a box of ps segments is
    // one wider than the group's when that count is even; the extra one is never fetched
    const size_t dims4[4] = {EX_SEG, nseg, (size_t)best_g, rows};
    const size_t strides4[3] = {EX_SEG * 4u, (size_t)cw * 4u, row_bytes};
    const unsigned box4[4] = {EX_SEG, (unsigned)p.ps, 1u, (unsigned)(CHUNK * p.mchunks)};
    p.map4d = 1;
    if (!mb_make_map_nd(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->k_cache, 4, dims4, strides4, box4, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !mb_make_map_nd(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->v_cache, 4, dims4, strides4, box4, CU_TENSOR_MAP_SWIZZLE_128B)) {
        // (float, segment of the row, cache row): the extra segment of an even group is then
        // the next group's first one (fetched and ignored) or lies outside the row
        const size_t dims3[3] = {EX_SEG, (size_t)p.cache_stride / EX_SEG, rows};
        const size_t strides3[2] = {EX_SEG * 4u, row_bytes};
        const unsigned box3[3] = {EX_SEG, (unsigned)p.ps, (unsigned)(CHUNK * p.mchunks)};
        p.map4d = 0;
        if ((size_t)p.heads * p.hw > dims3[1] * EX_SEG ||
            !mb_make_map_nd(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->k_cache, 3, dims3, strides3, box3, CU_TENSOR_MAP_SWIZZLE_128B) ||
            !mb_make_map_nd(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->v_cache, 3, dims3, strides3, box3, CU_TENSOR_MAP_SWIZZLE_128B))
            return false;
    }
    const size_t smem = exact_smem(hg, p.hw, p.max_chunks, best_depth, p.mchunks);
    const dim3 grid((unsigned)best_g, (unsigned)p.batch), block((unsigned)threads);
    if (threads <= 384) mb_launch(k_attn_exact<384>, grid, block, smem, s, kmap, vmap, p);
    else mb_launch(k_attn_exact<1024>, grid, block, smem, s, kmap, vmap, p);
    return true;
}

}  // namespace

// Opt the kernels into large dynamic shared memory on the current device; once
// per device at backend open, outside any stream capture.
extern "C" int mb_attention_init(void) {
    int rc = (int)cudaFuncSetAttribute(k_attn_strict, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_rows<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_SMEM_MAX);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_rows<384>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_SMEM_MAX);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_short<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_SMEM_MAX - 1024);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_short<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_SMEM_MAX - 1024);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_scalar, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_exact<384>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_SMEM_MAX);
    if (rc == 0) rc = (int)cudaFuncSetAttribute(k_attn_exact<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_SMEM_MAX);
    return rc;
}

// Scratch the chunked kernel needs for `batch` lanes that attend at most
// `max_valid` rows: per-chunk partials, then one merged row per lane.
extern "C" size_t mb_attention_scratch_floats(size_t batch, size_t heads, size_t max_valid,
                                              size_t head_width) {
    return batch * heads * chunks_for(max_valid) * (head_width + 2) + batch * heads * head_width;
}
// Arrival counters: one per (lane, head), then one per lane.
extern "C" size_t mb_attention_counters(size_t batch, size_t heads) { return batch * (heads + 1); }

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
    p.valids = a->lens == nullptr ? a->valid_per_slot : nullptr;
    p.out = a->out; p.qx = a->qx; p.sx = a->sx;
    p.partials = a->partials; p.counters = a->counters; p.status = a->status;
    p.exp_tab = a->exp_tab;
    p.q_stride = (long)a->q_stride; p.slot_stride = (long)a->slot_stride;
    p.cache_stride = (long)a->cache_stride; p.out_stride = (long)a->out_stride;
    p.position = (long)a->position; p.valid = (long)a->valid;
    p.heads = (int)a->heads; p.hw = (int)a->head_width; p.batch = (int)a->batch;
    p.scale = a->scale;
    p.inv_norm = a->softmax_inverse ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    // Longest row any lane can attend over: callers with per-lane positions pass
    // the cache capacity in `valid`.
    const long max_valid = (long)a->valid;
    if (max_valid <= 0) return (int)cudaErrorInvalidValue;
    {
        // at most 32 rows per stream: one CTA per stream, a thread per column
        static const int no_small = env_int("MYNAH_B200_NO_SMALL_ATTN");
        const size_t w = a->heads * a->head_width;
        if (!no_small && a->short_cache && max_valid <= SMALL_ROWS && w <= 1024u && (a->head_width % 4u) == 0 && (p.cache_stride % 4) == 0 &&
            (((uintptr_t)a->k_cache) & 15u) == 0 && (p.slot_stride % 4) == 0 && (a->qx == nullptr || a->sx != nullptr)) {
            const unsigned threads = (unsigned)((w + 31u) / 32u * 32u);
            const size_t smem = (2u * w + a->heads * SMALL_ROWS) * sizeof(float);
            if (a->strict) mb_launch(k_attn_small<true>, dim3((unsigned)p.batch), dim3(threads), smem, s, p);
            else mb_launch(k_attn_small<false>, dim3((unsigned)p.batch), dim3(threads), smem, s, p);
            if (a->launched != nullptr) *a->launched += 1u;
            return mb_check_launch();
        }
    }
    p.max_chunks = (int)chunks_for((size_t)max_valid);
    const size_t width = a->heads * a->head_width;
    // heads per CTA (one warp each): all of them.  Whole cache rows per tile keep DRAM pages
    // open, and one CTA per (stream, chunk subset) needs a single arrival counter per stream;
    // head groups of 1 or 4 with more CTAs were measured slower at every batch size
    // (one stream at position 256: 560 / 512 / 501 us per step for 1 / 4 / 12 heads per CTA).
    int hg = p.heads;
    int hpb = 0;   // heads per TMA box: a box holds whole heads and at most 256 columns
    for (int c = p.hw > 0 ? 256 / p.hw : 0; c >= 1 && hpb == 0; --c)
        if (c <= hg && hg % c == 0) hpb = c;
    const size_t cwidth = (size_t)hg * p.hw;
    const size_t tile_bytes = (size_t)CHUNK * cwidth * sizeof(float);
    // CTAs per stream: about one CTA per SM in all; with many streams one CTA walks
    // all chunks of its stream
    const long groups = p.heads / hg;
    long splits = a->sm_count > 0 ? a->sm_count / ((long)p.batch * groups) : p.max_chunks;
    if (hg < 4) splits = p.max_chunks;        // few warps per CTA: one chunk each, many CTAs
    if (splits > p.max_chunks) splits = p.max_chunks;
    if (splits < 1) splits = 1;
    const long per_cta = (p.max_chunks + splits - 1) / splits;   // most tiles of a kind one CTA walks
    const size_t fixed_bytes = (cwidth + (size_t)hg * p.max_chunks) * sizeof(float);
    long depth = ((long)ROWS_SMEM_MAX - (long)fixed_bytes) / (long)(2u * tile_bytes);
    if (depth > per_cta) depth = per_cta;
    if (depth > RING_MAX) depth = RING_MAX;
    const size_t rows_bytes = 2u * (size_t)(depth < 1 ? 1 : depth) * tile_bytes + fixed_bytes;
    const bool chunked = !a->strict && hpb > 0 && (p.hw % 4) == 0 && is_pow2(p.hw / 4) && p.hw / 4 <= 32 &&
                         p.heads <= 32 && p.max_chunks <= MERGE_MAX &&
                         depth >= 1 && rows_bytes <= (size_t)ROWS_SMEM_MAX && 64u * cwidth >= width &&
                         (p.cache_stride % 4) == 0 && (p.q_stride % 4) == 0 && (p.slot_stride % 4) == 0 &&
                         (a->batch == 1 || a->cache_rows != 0) && (p.slot_stride % p.cache_stride) == 0 &&
                         (((uintptr_t)a->k_cache | (uintptr_t)a->v_cache | (uintptr_t)a->q |
                           (uintptr_t)a->k_new | (uintptr_t)a->v_new) & 15u) == 0;
    // a cache of a few chunks that nothing is appended to: one CTA per stream, one warp per
    // (head, chunk), partials merged in shared memory
    {
        int hpb_all = 0;
        for (int c = p.hw > 0 ? 256 / p.hw : 0; c >= 1 && hpb_all == 0; --c)
            if (c <= p.heads && p.heads % c == 0) hpb_all = c;
        const size_t short_bytes =
            (2u * (size_t)p.max_chunks * CHUNK * width + 2u * width + (size_t)p.heads * p.max_chunks * (p.hw + 2) +
             2u * (size_t)p.heads * p.max_chunks) * sizeof(float);
        if (chunked && a->k_new == nullptr && hpb_all > 0 && p.max_chunks <= SHORT_MAX_CHUNKS &&
            p.heads * p.max_chunks <= 32 && short_bytes <= (size_t)ROWS_SMEM_MAX - 1024u &&
            (a->batch == 1 || a->cache_rows != 0)) {
            p.box_cols = hpb_all * p.hw;
            p.nbox = p.heads / hpb_all;
            p.slot_rows = p.slot_stride / p.cache_stride;
            p.splits = 1;
            p.depth = 1;
            p.early = a->early_prefetch ? 1 : 0;
            size_t rows = a->cache_rows;
            if (rows == 0) rows = (size_t)p.valid;
            CUtensorMap kmap, vmap;
            if (!mb_make_map_2d(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->k_cache, rows, (size_t)p.cache_stride,
                                (size_t)p.cache_stride * 4u, (unsigned)p.box_cols, CHUNK, CU_TENSOR_MAP_SWIZZLE_NONE) ||
                !mb_make_map_2d(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->v_cache, rows, (size_t)p.cache_stride,
                                (size_t)p.cache_stride * 4u, (unsigned)p.box_cols, CHUNK, CU_TENSOR_MAP_SWIZZLE_NONE))
                return (int)cudaErrorInvalidValue;
            if (p.heads * p.max_chunks * 32 <= 128)
                mb_launch(k_attn_short<128>, dim3((unsigned)p.batch), dim3((unsigned)(p.heads * p.max_chunks) * 32u), short_bytes, s,
                          kmap, vmap, p);
            else
                mb_launch(k_attn_short<1024>, dim3((unsigned)p.batch), dim3((unsigned)(p.heads * p.max_chunks) * 32u), short_bytes, s,
                          kmap, vmap, p);
            if (a->launched != nullptr) *a->launched += 1u;
            return mb_check_launch();
        }
    }
    if (chunked) {
        if (a->partials == nullptr || a->counters == nullptr) return (int)cudaErrorInvalidValue;
        p.splits = (int)splits;
        p.depth = (int)depth;
        p.early = a->early_prefetch ? 1 : 0;
        p.box_cols = hpb * p.hw;
        p.nbox = hg / hpb;
        p.slot_rows = p.slot_stride / p.cache_stride;
        size_t rows = a->cache_rows;
        if (rows == 0) rows = (size_t)(p.valid > p.position + 1 ? p.valid : p.position + 1);
        CUtensorMap kmap, vmap;
        if (!mb_make_map_2d(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->k_cache, rows, (size_t)p.cache_stride,
                            (size_t)p.cache_stride * 4u, (unsigned)p.box_cols, CHUNK, CU_TENSOR_MAP_SWIZZLE_NONE) ||
            !mb_make_map_2d(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->v_cache, rows, (size_t)p.cache_stride,
                            (size_t)p.cache_stride * 4u, (unsigned)p.box_cols, CHUNK, CU_TENSOR_MAP_SWIZZLE_NONE))
            return (int)cudaErrorInvalidValue;
        if (hg * 32 <= 384 && p.batch >= 32)
            mb_launch(k_attn_rows<384>, dim3((unsigned)splits, (unsigned)p.batch, (unsigned)groups),
                      dim3((unsigned)hg * 32u), rows_bytes, s, kmap, vmap, p);
        else
            mb_launch(k_attn_rows<1024>, dim3((unsigned)splits, (unsigned)p.batch, (unsigned)groups),
                      dim3((unsigned)hg * 32u), rows_bytes, s, kmap, vmap, p);
        if (a->launched != nullptr) *a->launched += 1u;
        return mb_check_launch();
    }
    if (a->out == nullptr) return (int)cudaErrorInvalidValue;
    if (a->strict && launch_exact(a, p, s)) {
        if (a->launched != nullptr) *a->launched += 1u;
        return mb_check_launch();
    }
    const size_t smem = (size_t)(p.hw + max_valid) * sizeof(float);
    if (smem > 200u * 1024u) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)p.heads, (unsigned)p.batch);
    if (a->strict) mb_launch(k_attn_strict, dim3(grid), dim3(256), smem, s, p);
    else mb_launch(k_attn_scalar, dim3(grid), dim3(FAST_THREADS), smem, s, p);
    int rc = mb_check_launch();
    if (a->launched != nullptr) *a->launched += 1u;
    if (rc == 0 && a->qx != nullptr) {
        rc = mb_quant_rows(a->out, a->batch, width, a->qx, a->sx, a->n_active, stream);
        if (a->launched != nullptr) *a->launched += 1u;
    }
    return rc;
}

#ifdef MB_PHASE_TICKS
// Profiling builds only (make TICKS=1): the phase timestamps of the last k_attn_exact launch,
// eight per CTA (see attn_exact.cuh), copied to `host` (n values).
extern "C" __attribute__((visibility("default")))
int mynah_b200_debug_attention_ticks(unsigned long long *host, size_t n) {
    if (n > 8u * 8192u) n = 8u * 8192u;
    cudaDeviceSynchronize();
    return (int)cudaMemcpyFromSymbol(host, g_exact_ticks, n * sizeof(unsigned long long));
}
#endif

// ---------------------------------------------------------------------------
// Allocation-free self-attention for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off the table: a
// real-time audio thread that may not block in the allocator, a plugin loaded
// into a process whose memory pool is owned by someone else, or code that runs
// under a CUDA context it is not allowed to grow.  For them the split-position
// kernel's scratch (per-chunk partial results, one merged row, arrival
// counters) lives in the fixed array below instead of in memory obtained with
// cudaMalloc.  Every GPU that loads this library holds the array until the
// process exits.
//
// Limits: one stream per call, at most MB_STATIC_MAX_VALID attended rows and
// heads * head_width <= MB_STATIC_MAX_WIDTH; head_width a power-of-two multiple
// of 4 up to 128 and 16-byte aligned buffers (the chunked kernel's shapes).
// Every call uses the same array, so two calls that overlap on the GPU (two
// streams, two threads) race; serialize them.  The array keeps the previous
// call's partial results, which are always rewritten before they are read; the
// counters must start at zero and are cleared at the start of each call.
#define MB_STATIC_MAX_VALID 4096u
#define MB_STATIC_MAX_WIDTH 768u
#define MB_STATIC_MAX_HEADS 32u
#define MB_STATIC_MAX_DEVICES 16
// chunks * (width + 2 * heads) partial floats + one merged row, then the counters
#define MB_STATIC_FLOATS ((MB_STATIC_MAX_VALID / 32u) * (MB_STATIC_MAX_WIDTH + 2u * MB_STATIC_MAX_HEADS) + MB_STATIC_MAX_WIDTH)
#define MB_STATIC_COUNTERS (MB_STATIC_MAX_HEADS + 1u)
#define MB_STATIC_BYTES (MB_STATIC_FLOATS * 4u + MB_STATIC_COUNTERS * 4u)

static __device__ __align__(256) unsigned char g_attention_static_scratch[MB_STATIC_BYTES];

// Device address of the array on each device, resolved on first use there.  In
// host code the array's name is only a handle; a kernel must be given the
// address cudaGetSymbolAddress returns for the current device.
static void *g_static_scratch_addr[MB_STATIC_MAX_DEVICES];

static void static_error(char *error, size_t cap, const char *message) {
    if (error != nullptr && cap > 0) snprintf(error, cap, "%s", message);
}

// Same contract as mynah_cuda_self_attention_dev (append K/V of dev_qkv at
// `position`, attend rows below `valid`, `heads` heads of `head_width`), but
// state-free and allocation-free: no cudaMalloc, cudaFree or allocating library
// call is made, here or on any later call.  The first call on a device
// resolves the scratch array's device address and opts the kernel into its
// shared-memory size; make that first call outside stream capture.  Work is enqueued on `cuda_stream` (a cudaStream_t, may be
// 0) and is not synchronized.  Returns 0, or -1 with a message.
extern "C" __attribute__((visibility("default")))
int mynah_b200_self_attention_static(const float *dev_qkv, float *dev_k_cache, float *dev_v_cache,
                                     size_t position, size_t cache_stride, size_t valid,
                                     size_t heads, size_t head_width, float scale, float *dev_out,
                                     void *cuda_stream, char *error, size_t cap) {
    if (dev_qkv == nullptr || dev_k_cache == nullptr || dev_v_cache == nullptr || dev_out == nullptr ||
        heads == 0 || head_width == 0 || valid == 0 || cache_stride < heads * head_width) {
        static_error(error, cap, "invalid attention request");
        return -1;
    }
    const size_t width = heads * head_width;
    if (valid > MB_STATIC_MAX_VALID || width > MB_STATIC_MAX_WIDTH || heads > MB_STATIC_MAX_HEADS) {
        if (error != nullptr && cap > 0)
            snprintf(error, cap,
                     "request exceeds the static scratch: at most %u rows, width %u, %u heads",
                     MB_STATIC_MAX_VALID, MB_STATIC_MAX_WIDTH, MB_STATIC_MAX_HEADS);
        return -1;
    }
    const bool shape_ok = (head_width % 4) == 0 && is_pow2((long)head_width / 4) && head_width <= 128 &&
                          (cache_stride % 4) == 0 && (width % 4) == 0 &&
                          (((uintptr_t)dev_k_cache | (uintptr_t)dev_v_cache | (uintptr_t)dev_qkv) & 15u) == 0;
    if (!shape_ok) {
        static_error(error, cap, "head width must be a power-of-two multiple of 4 up to 128 and buffers 16-byte aligned");
        return -1;
    }
    int device = -1;
    cudaError_t rc = cudaGetDevice(&device);
    if (rc != cudaSuccess || device < 0 || device >= MB_STATIC_MAX_DEVICES) {
        static_error(error, cap, rc != cudaSuccess ? cudaGetErrorString(rc) : "device ordinal out of range");
        return -1;
    }
    if (g_static_scratch_addr[device] == nullptr) {
        void *addr = nullptr;
        rc = cudaGetSymbolAddress(&addr, g_attention_static_scratch);
        if (rc != cudaSuccess || addr == nullptr) {
            static_error(error, cap, rc != cudaSuccess ? cudaGetErrorString(rc) : "no address for the static scratch");
            return -1;
        }
        // the chunk kernel stages two chunks of K and V: above 48 KB of dynamic shared
        // memory for wide heads, which a kernel must opt into once per device
        rc = cudaFuncSetAttribute(k_attn_rows<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_SMEM_MAX);
        if (rc != cudaSuccess) {
            static_error(error, cap, cudaGetErrorString(rc));
            return -1;
        }
        g_static_scratch_addr[device] = addr;
    }
    float *scratch = static_cast<float *>(g_static_scratch_addr[device]);
    unsigned *counters = reinterpret_cast<unsigned *>(scratch + MB_STATIC_FLOATS);
    cudaStream_t s = (cudaStream_t)cuda_stream;
    rc = cudaMemsetAsync(counters, 0, MB_STATIC_COUNTERS * sizeof(unsigned), s);
    if (rc != cudaSuccess) {
        static_error(error, cap, cudaGetErrorString(rc));
        return -1;
    }
    AttnP p;
    memset(&p, 0, sizeof(p));
    p.q = dev_qkv;
    p.k_new = dev_qkv + width;
    p.v_new = dev_qkv + 2 * width;
    p.k_cache = dev_k_cache;
    p.v_cache = dev_v_cache;
    p.out = dev_out;
    p.partials = scratch;
    p.counters = counters;
    p.q_stride = (long)(3 * width);
    p.cache_stride = (long)cache_stride;
    p.out_stride = (long)width;
    p.position = (long)position;
    p.valid = (long)valid;
    p.heads = (int)heads;
    p.hw = (int)head_width;
    p.batch = 1;
    p.max_chunks = (int)chunks_for(valid);
    p.splits = p.max_chunks;           // one chunk per CTA: partials go through the static scratch
    p.depth = 1;
    p.early = 0;
    p.scale = scale;
    int hpb = 0;
    for (int c = 256 / p.hw; c >= 1 && hpb == 0; --c)
        if (c <= p.heads && p.heads % c == 0) hpb = c;
    const size_t floats = 2u * CHUNK * width + width + (size_t)p.heads * MERGE_MAX;
    if (hpb == 0 || floats * sizeof(float) > (size_t)ROWS_SMEM_MAX || p.max_chunks > MERGE_MAX) {
        static_error(error, cap, "shape needs more shared memory than the allocation-free path uses");
        return -1;
    }
    p.box_cols = hpb * p.hw;
    p.nbox = p.heads / hpb;
    p.slot_rows = 0;
    const size_t rows = valid > position + 1 ? valid : position + 1;
    CUtensorMap kmap, vmap;   // encoded on the host: no device memory involved
    if (!mb_make_map_2d(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, dev_k_cache, rows, cache_stride,
                        cache_stride * 4u, (unsigned)p.box_cols, CHUNK, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !mb_make_map_2d(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, dev_v_cache, rows, cache_stride,
                        cache_stride * 4u, (unsigned)p.box_cols, CHUNK, CU_TENSOR_MAP_SWIZZLE_NONE)) {
        static_error(error, cap, "could not describe the KV cache to the copy engine");
        return -1;
    }
    k_attn_rows<1024><<<dim3((unsigned)p.splits, 1u), (unsigned)p.heads * 32u, floats * sizeof(float), s>>>(kmap, vmap, p);
    rc = cudaGetLastError();
    if (rc != cudaSuccess) {
        static_error(error, cap, cudaGetErrorString(rc));
        return -1;
    }
    if (error != nullptr && cap > 0) error[0] = '\0';
    return 0;
}
