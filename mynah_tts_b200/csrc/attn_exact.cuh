// Reference-order ("strict") single-query attention at streaming speed.  Included by
// attention.cu after AttnP and lane_setup.
//
// The reference's loops (src/graph.c:3182-3202 self, 3221-3244 cross) fix the ORDER of
// three kinds of sums -- a score's 64 products over d, the denominator over s, an output's
// products over s -- but nothing else: scores of different rows, outputs of different
// dimensions, heads and streams are independent.  k_attn_exact keeps every such sum one
// sequential chain of separately rounded products and adds, in index order, and runs the
// chains side by side while the cache streams through shared memory:
//
//   CTA = one stream (lane) and a group of its heads.  K rows, then V rows, of the group's
//   columns arrive as 32-row TMA tiles through one ring of mbarrier-guarded slots (every
//   wait bounded, status bit 2), one copy per tile.  The copy reads each cache row's piece
//   as one contiguous run (segments of 128 bytes, innermost), and lays the tile out as
//   [32 rows][ps segments][32 floats] with the 128-byte swizzle, where ps is the group's
//   segment count made odd: when it is even the box is one segment wider than the array's
//   segment dimension, and that segment is zero-filled without being fetched.  With ps odd
//   the swizzle key (row * ps + segment) mod 8 differs between any 8 consecutive rows, so
//   the threads of a warp, which read the same column piece of 32 different rows in the
//   score pass, hit 32 different banks; the value pass reads along a row and is conflict
//   free anyway.  A copy brings p.mchunks chunks of 32 rows at once (one when a chunk is tens
//   of KB, several for narrow head groups): copies of one CTA complete about one per memory
//   round trip, so a copy should carry 30 KB or more.
//   pass 1 (K tiles): thread (head, row) forms its row's score, d = 0 .. hw-1 in order.
//   middle: max per head (exact in any order), e = expf(score - max) with the host libm's
//           bits, the denominator by one thread per head in row order, weights e / den.
//   pass 2 (V tiles): thread (head, d) adds weight[s] * v[s][d] for s = 0 .. valid-1 in order.
//   tail: the stream's last CTA (arrival counter; none when one CTA owns the stream)
//         quantizes the row to int8 when the next product wants that.
//
// Same bits as k_attn_strict and as the CPU loop, whatever the batch or the head grouping.
#pragma once

namespace {

constexpr int EX_RING_MAX = 8;
constexpr int EX_SEG = 32;                     // floats of a 128-byte segment

// float offset of element (row r, column col) of a tile with ps segments per row
__device__ __forceinline__ int ex_offset(int r, int col, int ps) {
    const int line = r * ps + (col >> 5), j = col & 31;
    return line * EX_SEG + ((((j >> 2) ^ (line & 7)) << 2) | (j & 3));
}

// Phase timestamps for profiling, compiled in with -DMB_PHASE_TICKS (make TICKS=1): thread 0
// of every CTA records the global nanosecond timer at its phase boundaries -- 0 entry, 1
// prologue done, 2 score pass done, 3 weights ready, 4 value pass done, 5 exit -- into a
// device array that mynah_b200_debug_attention_ticks copies out.  Absent from normal builds.
#ifdef MB_PHASE_TICKS
__device__ unsigned long long g_exact_ticks[8 * 8192];
__device__ __forceinline__ void mb_tick(int i) {
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const unsigned cta = blockIdx.y * gridDim.x + blockIdx.x;
        if (cta < 8192u) g_exact_ticks[cta * 8 + i] = t;
    }
}
#define MB_TICK(i) mb_tick(i)
#else
#define MB_TICK(i)
#endif

template <int MAXT>
__global__ void __launch_bounds__(MAXT, 1)
k_attn_exact(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, AttnP p) {
    MB_TICK(0);
    if (!p.early) {
        mb_pdl_wait();
        mb_pdl_trigger();
    }
    extern __shared__ __align__(1024) float sm_exact[];
    __shared__ float red[33];
    __shared__ unsigned s_last, s_fail;
    __shared__ __align__(8) unsigned long long mbar[EX_RING_MAX];
    const int b = blockIdx.y;
    long pos, valid, slot;
    float *kc, *vc;
    if (!lane_setup(p, b, pos, valid, kc, vc, &slot)) return;
    const int hw = p.hw, heads = p.heads, width = heads * hw;
    const int groups = (int)gridDim.x, hg = heads / groups;
    const int h0 = blockIdx.x * hg, cw = hg * hw, c0 = h0 * hw;     // this CTA's heads and columns
    const int ps = p.ps, chunk_floats = CHUNK * ps * EX_SEG, mch = p.mchunks, tile_floats = mch * chunk_floats;
    const int ns = (int)((valid + CHUNK - 1) / CHUNK);      // chunks of this stream
    const int nk = (ns + mch - 1) / mch, ntiles = 2 * nk;   // copies per pass, and in all
    const int depth = p.depth, scap = p.max_chunks * CHUNK;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float *tiles = sm_exact;                                  // [depth][mch * 32 rows][ps][32], swizzled
    float *qs = tiles + (long)depth * tile_floats;            // [cw]
    float *kn = qs + cw;                                      // [cw] the row appended now
    float *vn = kn + cw;
    float *sc = vn + cw;                                      // [hg][scap] scores, then weights
    float *stat = sc + (long)hg * scap;                       // [hg] max, [hg] denominator
    const unsigned tile_bytes = (unsigned)tile_floats * 4u;
    const unsigned long long stream_policy = mb_l2_evict_first();
    // copy t of this CTA: K chunks [t * mch, (t + 1) * mch) for t < nk, then the V chunks
    // likewise; ring slot t % depth
    auto issue = [&](int t) {
        const int c = (t < nk ? t : t - nk) * mch, rs = t % depth;
        const CUtensorMap *map = t < nk ? &kmap : &vmap;
        const int y = (int)(slot * p.slot_rows + (long)c * CHUNK);
        float *tile = tiles + (long)rs * tile_floats;
        mbar_expect_tx(&mbar[rs], tile_bytes);
        // 4-D map: (float, segment of the group, group, row); 3-D: (float, segment of the row, row)
        if (p.map4d) mb_tma_load_4d_hint(tile, map, 0, 0, (int)blockIdx.x, y, &mbar[rs], stream_policy);
        else mb_tma_load_3d_hint(tile, map, 0, c0 / EX_SEG, y, &mbar[rs], stream_policy);
    };
    if (tid == 0) {
        s_fail = 0u;
        for (int i = 0; i < depth; ++i) mbar_init(&mbar[i], 1u);
        for (int t = 0; t < depth && t < ntiles; ++t) issue(t);
    }
    if (p.early) {
        mb_pdl_wait();
        mb_pdl_trigger();
    }
    const bool append = p.k_new != nullptr;
    for (int d = tid; d < cw; d += blockDim.x) {
        qs[d] = p.q[(long)b * p.q_stride + c0 + d];
        if (append) {
            const float kk = p.k_new[(long)b * p.q_stride + c0 + d], vv = p.v_new[(long)b * p.q_stride + c0 + d];
            kn[d] = kk;
            vn[d] = vv;
            kc[pos * p.cache_stride + c0 + d] = kk;
            vc[pos * p.cache_stride + c0 + d] = vv;
        }
    }
    __syncthreads();
    MB_TICK(1);
    const bool p1 = warp < hg;                                // pass-1 thread: head h0 + warp, row `lane` of a chunk
    const int col = tid;                                      // pass-2 thread: column c0 + col
    const bool p2 = col < cw;
    const int h2 = p2 ? col / hw : 0;
    const int seg2 = col >> 5, j2c = (col & 31) >> 2, j2e = col & 3;
    float lmax = -FLT_MAX, acc = 0.0f;
    int done = 0;                                             // tiles consumed
    for (int t = 0; t < ntiles; ++t) {
        const int rs = t % depth;
        const unsigned parity = (unsigned)((t / depth) & 1);
        if (t == nk) {
            MB_TICK(2);
            // ---- all scores are in: max, exp, denominator, weights -------------------------
            if (p1) {
                const float m = warp_max(lmax);
                if (lane == 0) stat[warp] = m;
            }
            __syncthreads();
            // e = expf(score - max) with the host libm's bits, over the (head, row) pairs of the
            // group six at a time per thread: the table words of a batch are requested
            // together, so a batch costs one memory round trip, not six
            {
                constexpr int EXB = 6;
                const int total = hg * (int)valid;
                for (int i0 = tid; i0 < total; i0 += EXB * blockDim.x) {
                    float arg[EXB];
                    uint32_t word[EXB];
                    int at[EXB];
#pragma unroll
                    for (int j = 0; j < EXB; ++j) {
                        const int i = i0 + j * blockDim.x;
                        at[j] = -1;
                        if (i < total) {
                            const int h = i / (int)valid, s = i - h * (int)valid;
                            at[j] = h * scap + s;
                            arg[j] = __fsub_rn(sc[at[j]], stat[h]);
                            word[j] = mb_exp_fetch(arg[j], p.exp_tab);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < EXB; ++j)
                        if (at[j] >= 0) sc[at[j]] = mb_expf_host_with(arg[j], word[j], p.exp_tab != nullptr);
                }
            }
            __syncthreads();
            if (p1 && lane == 0) {
                stat[hg + warp] = mb_seq_sum(sc + (long)warp * scap, (int)valid);
            }
            __syncthreads();
            for (int h = 0; h < hg; ++h) {
                const float den = stat[hg + h];
                if (p.inv_norm) {     // softmax_row_inplace of the multi-row path: values *= 1 / total
                    const float inv = den > 0.0f ? __fdiv_rn(1.0f, den) : 0.0f;
                    for (long s = tid; s < valid; s += blockDim.x)
                        sc[(long)h * scap + s] = __fmul_rn(sc[(long)h * scap + s], inv);
                } else {
                    for (long s = tid; s < valid; s += blockDim.x)
                        sc[(long)h * scap + s] = __fdiv_rn(sc[(long)h * scap + s], den);
                }
            }
            __syncthreads();
            MB_TICK(3);
        }
        if (!mbar_wait(&mbar[rs], parity, SPIN_LIMIT)) s_fail = 1u;
        else if (t < nk) {
          for (int sub = 0; sub < mch; ++sub) {
            // ---- pass 1: this thread's row of chunk t * mch + sub ----------------------------
            const long s = ((long)t * mch + sub) * CHUNK + lane;
            if (p1 && s < valid) {
                const float *tile = tiles + (long)rs * tile_floats + (long)sub * chunk_floats;
                const float *qh = qs + warp * hw;
                float a = 0.0f;
                if (append && s == pos) {
                    const float *kr = kn + warp * hw;
                    for (int d = 0; d < hw; ++d) a = __fadd_rn(a, __fmul_rn(qh[d], kr[d]));
                } else if (hw == 64) {
                    // the row's 64 floats first (sixteen independent 16-byte loads), then the chain:
                    // a loop that loads inside the chain pays a shared-memory round trip per step
                    // when few warps share a scheduler (measured 117 cycles per four elements)
                    float4 kr[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int line = lane * ps + 2 * warp + (c >> 3);
                        kr[c] = *reinterpret_cast<const float4 *>(tile + line * EX_SEG + (((c & 7) ^ (line & 7)) << 2));
                    }
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const float4 qv = *reinterpret_cast<const float4 *>(qh + 4 * c);
                        a = __fadd_rn(a, __fmul_rn(qv.x, kr[c].x));
                        a = __fadd_rn(a, __fmul_rn(qv.y, kr[c].y));
                        a = __fadd_rn(a, __fmul_rn(qv.z, kr[c].z));
                        a = __fadd_rn(a, __fmul_rn(qv.w, kr[c].w));
                    }
                } else {
#pragma unroll 4
                    for (int d4 = 0; d4 < hw; d4 += 4) {
                        const float4 kv = *reinterpret_cast<const float4 *>(tile + ex_offset(lane, warp * hw + d4, ps));
                        const float4 qv = *reinterpret_cast<const float4 *>(qh + d4);
                        a = __fadd_rn(a, __fmul_rn(qv.x, kv.x));
                        a = __fadd_rn(a, __fmul_rn(qv.y, kv.y));
                        a = __fadd_rn(a, __fmul_rn(qv.z, kv.z));
                        a = __fadd_rn(a, __fmul_rn(qv.w, kv.w));
                    }
                }
                a = __fmul_rn(a, p.scale);
                sc[(long)warp * scap + s] = a;
                if (a > lmax) lmax = a;
            }
          }
        } else if (p2) {
          for (int sub = 0; sub < mch; ++sub) {
            // ---- pass 2: this thread's column over the rows of chunk (t - nk) * mch + sub ------
            const int c = (t - nk) * mch + sub;
            if (c >= ns) break;
            const long s0 = (long)c * CHUNK;
            const int cnt = (int)min((long)CHUNK, valid - s0);
            const float *tile = tiles + (long)rs * tile_floats + (long)sub * chunk_floats;
            const float *w = sc + (long)h2 * scap + s0;
            const int fresh = (append && pos >= s0 && pos < s0 + cnt) ? (int)(pos - s0) : -1;
            // the chunk's 32 values of this column and its 32 weights first, then the chain
            float vr[CHUNK], wr[CHUNK];
#pragma unroll
            for (int r = 0; r < CHUNK; ++r) {
                const int line = r * ps + seg2;
                vr[r] = tile[line * EX_SEG + (((j2c ^ (line & 7)) << 2) | j2e)];
            }
#pragma unroll
            for (int r4 = 0; r4 < CHUNK / 4; ++r4) {
                const float4 w4 = *reinterpret_cast<const float4 *>(w + 4 * r4);
                wr[4 * r4] = w4.x; wr[4 * r4 + 1] = w4.y; wr[4 * r4 + 2] = w4.z; wr[4 * r4 + 3] = w4.w;
            }
            if (fresh >= 0) {
                const float vf = vn[col];
#pragma unroll
                for (int r = 0; r < CHUNK; ++r) vr[r] = r == fresh ? vf : vr[r];
            }
#pragma unroll
            for (int r = 0; r < CHUNK; ++r)
                if (r < cnt) acc = __fadd_rn(acc, __fmul_rn(wr[r], vr[r]));
          }
        }
        __syncthreads();                                     // every thread is done with the slot
        done = t + 1;
        if (s_fail != 0u) break;
        if (tid == 0 && t + depth < ntiles) issue(t + depth);
    }
    if (s_fail != 0u) {
        // a tile never landed: flag it and give every copy still in flight one more bounded wait,
        // so that none lands after this CTA's shared memory is released
        if (tid == 0) {
            if (p.status != nullptr) atomicOr(p.status, 2);
            const int issued = min(ntiles, done - 1 + depth);
            for (int t = done - 1; t < issued; ++t) mbar_wait(&mbar[t % depth], (unsigned)((t / depth) & 1), SPIN_LIMIT);
        }
        return;
    }
    MB_TICK(4);
    float *outrow = p.out + (long)b * p.out_stride;
    if (p2) outrow[c0 + col] = acc;
    if (p.qx == nullptr) return;
    // ---- the stream's last CTA quantizes the whole row ------------------------------------
    float *vals = tiles;                                      // every tile has been consumed
    if (groups > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            unsigned *ctr = p.counters + b;
            const unsigned prev = atomicAdd(ctr, 1u);
            s_last = prev == (unsigned)groups - 1u;
            if (s_last) *ctr = 0u;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        for (int i = tid; i < width; i += blockDim.x) vals[i] = __ldcg(outrow + i);
    } else if (p2) {
        vals[col] = acc;
    }
    __syncthreads();
    quantize_shared_row(vals, width, p.qx + (long)b * width, p.sx + b, red);
    MB_TICK(5);
}

// Segments per tile row: the group's column count in 128-byte segments, made odd.
inline int exact_pitch_segments(int hg, int hw) { return ((hg * hw) / EX_SEG) | 1; }

// Shared memory of one CTA of k_attn_exact: `depth` tiles, q and the appended K/V row, the
// scores of the group's heads, two statistics per head.
inline size_t exact_smem(int hg, int hw, int max_chunks, int depth, int mchunks) {
    const size_t cw = (size_t)hg * hw;
    return ((size_t)depth * mchunks * CHUNK * exact_pitch_segments(hg, hw) * EX_SEG + 3u * cw + (size_t)hg * max_chunks * CHUNK +
            2u * hg) * sizeof(float);
}
// Chunks per copy: as many as fit in 40 KB, at least one, at most four (and no more than the
// longest stream has).
inline int exact_chunks_per_copy(int hg, int hw, int max_chunks) {
    const size_t chunk_bytes = (size_t)CHUNK * exact_pitch_segments(hg, hw) * EX_SEG * sizeof(float);
    int m = (int)((40u * 1024u) / chunk_bytes);
    if (m > 4) m = 4;
    if (m > max_chunks) m = max_chunks;
    return m < 1 ? 1 : m;
}

}  // namespace
