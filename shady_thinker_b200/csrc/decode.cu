// Split-KV GQA decode attention for sm_100a.
//
// What it computes is gqa_attention_head.wgsl:30-124 (one query token per sequence attends
// to rows [0, L) of that sequence's cache with an online softmax) followed by
// gqa_reduce.wgsl:20-65 (log-sum-exp merge of the splits) — but the work is laid out for
// HBM bandwidth instead of one workgroup per (q_head, split):
//   * one CTA owns (sequence, kv_head, position range) and serves ALL query heads of the
//     KV group from one pass over the K/V rows, so each cache byte leaves HBM once;
//   * 16-bit caches: every warp runs a private multi-stage cp.async (16-byte, L2-only)
//     pipeline over 16-position blocks into XOR-swizzled shared memory, feeds
//     mma.sync.m16n8k16 through ldmatrix (query heads on the M axis), keeps the softmax
//     statistics in fp32 with quad shuffles; no block-wide barrier in the main loop;
//   * fp32 caches (the reference's native format): lanes span head_dim with 128-bit
//     loads, warp-shuffle dot products, fp32 FMA;
//   * ranges come either from an explicit num_splits (ceil(L/ns) ranges, wgsl:46-48) or
//     from a balanced partition: all sequences laid end to end are cut into as many equal
//     spans as there are resident CTAs (one wave, no tail); every CTA re-derives its span
//     from the device-side lengths with a warp scan, so no plan has to be uploaded;
//   * the splits of a sequence are merged inside the same launch by the CTA that arrives
//     last (self-resetting arrival counters), not by a second kernel.
#include <stdlib.h>

#include "p2p.cuh"

namespace shady {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr uint32_t kMaxSlots = 148u * 8u;  // bound on resident CTAs (spans); sizes the workspace and the merge tables
constexpr uint32_t kBlkPos = 16;  // positions per row-block: unit of the work line and of the MMA pipeline

struct DecodeArgs {
    const void *q;
    void *out;
    float *lse;
    const float *gate;
    KvAddr kv;
    const uint32_t *seq_lens;
    float *partials;     // workspace: split records of (hd+2) floats
    uint32_t *counters;  // workspace: arrivals per (sequence, kv head, head group); zero between calls
    uint32_t gz;         // head groups per kv head (folded into blockIdx.x)
    uint32_t num_seqs, nkv, nh, G, hd;
    uint32_t num_splits; // >0: every sequence is cut into ceil(L/ns) ranges (wgsl:46-48); 0: balanced spans
    uint32_t line_blocks; // balanced mode: length of the work line, sum_i (max(1, ceil(L_i/16)) + pad)
    uint32_t pad;         // balanced mode: line units appended to every sequence (see the comment on span_begin)
    uint32_t spans;       // balanced mode: number of equal spans the line is cut into
    uint32_t span_math32; // (spans + 1) * line_blocks + spans < 2^32: span arithmetic in 32 bits
    uint32_t q_dtype, out_dtype;
    uint32_t force_partials;  // 1: always write the partial record (shady_attn_decode_partials)
    uint32_t defer_merge;     // 1: CTAs only write records; balanced_merge_kernel merges them (sequences cut into many spans)
    uint32_t grid_merge;      // 1 (with defer_merge, cooperative launch): the decode grid meets at a barrier and merges the records itself
    uint32_t interleave;      // 1 (with grid_merge, one sequence): the warps of all CTAs take the sequence's 16-row blocks in turn
    uint32_t *grid_sync;      // workspace: {arrivals, departures} of that barrier; zero between calls
    uint32_t out_row_stride;  // elements between consecutive head rows of `out` (hd, or hd+2 when out is a record buffer)
    uint32_t lse_stride;      // elements between consecutive entries of `lse` (1, or hd+2 inside a record buffer)
    float scale_log2;         // 1/sqrt(hd) * log2(e)
    // fused append (16-bit caches): Q comes raw from the projection and is normed/rotated while it is staged, and
    // the CTA that owns the tail of a sequence norms/rotates the new K row and writes it and the V row to the cache
    // (fused_split_qknorm_kvstore.wgsl:106-230) before it streams them — one launch per layer instead of three.
    uint32_t fuse_append;
    const void *ap_q, *ap_k, *ap_v;   // q_proj_full [seq][nh][(1+gate)*hd], k_proj / v_proj [seq][nkv][hd]
    const uint16_t *ap_norm_w;        // bf16 bits q[hd] then k[hd], or NULL
    uint32_t ap_in_dtype, ap_has_gate, ap_rd;
    float ap_eps;
    float ap_inv_freq[128];
    // row-sharded sequence (one process per GPU): the launch that merges this rank's records also exchanges the
    // result with the peers over NVLink and merges across ranks (shard_merge_p2p_kernel); px_world == 0: off
    char *const *px_peer_bases;   // device array [world] of every rank's exchange buffer as mapped into this process
    StatusRef status;             // where a bounded wait that ran out is reported (grid barrier, peer flags)
    uint32_t wait_grid, wait_peer;   // poll limits of the two waits
    void *px_out;                 // final rows [nh][hd]
    const float *px_gate;         // optional [nh][hd] f32
    uint32_t px_world, px_rank, px_epoch, px_out_dtype;
    // the lengths by value (small batches whose caller gave them on the host): a kernel-parameter read instead of a
    // global load at the head of every dependent chain (span search, piece set-up, record merge); lens_n == 0: off
    uint32_t lens_n;
    uint32_t lens_v[32];
};
__device__ __forceinline__ uint32_t seq_len_at(const DecodeArgs &a, uint32_t i) {
    return i < a.lens_n ? a.lens_v[i] : a.seq_lens[i];
}

// 8 consecutive elements (16-byte aligned for 16-bit types, 32-byte for f32) of a buffer of run-time dtype
__device__ __forceinline__ void load8_as_f32(const void *p, size_t i, uint32_t dt, float (&v)[8]) {
    if (dt == SHADY_F32) {
        const float4 x = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + i);
        const float4 y = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + i + 4);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
    } else {
        const uint4 u = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p) + i);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (dt == SHADY_F16) {
                const __half2 h = *reinterpret_cast<const __half2 *>(&w[k]);
                v[2 * k] = __low2float(h); v[2 * k + 1] = __high2float(h);
            } else {
                v[2 * k] = __uint_as_float(w[k] << 16); v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
            }
        }
    }
}

// The same access in two halves: the request (raw 16 or 32 bytes, nothing depends on them yet) and the conversion.
// A thread stalls at the first use of loaded data, so requests that should overlap other work must stay raw.
__device__ __forceinline__ void load8_raw(const void *p, size_t i, uint32_t dt, uint4 (&r)[2]) {
    if (dt == SHADY_F32) {
        r[0] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(p) + i);
        r[1] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(p) + i + 4);
    } else {
        r[0] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p) + i);
        r[1] = make_uint4(0, 0, 0, 0);
    }
}
__device__ __forceinline__ void cvt8_raw(const uint4 (&r)[2], uint32_t dt, float (&v)[8]) {
    if (dt == SHADY_F32) {
        v[0] = __uint_as_float(r[0].x); v[1] = __uint_as_float(r[0].y); v[2] = __uint_as_float(r[0].z); v[3] = __uint_as_float(r[0].w);
        v[4] = __uint_as_float(r[1].x); v[5] = __uint_as_float(r[1].y); v[6] = __uint_as_float(r[1].z); v[7] = __uint_as_float(r[1].w);
    } else {
        const uint32_t w[4] = {r[0].x, r[0].y, r[0].z, r[0].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (dt == SHADY_F16) {
                const __half2 h = *reinterpret_cast<const __half2 *>(&w[k]);
                v[2 * k] = __low2float(h); v[2 * k + 1] = __high2float(h);
            } else {
                v[2 * k] = __uint_as_float(w[k] << 16); v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
            }
        }
    }
}

__device__ __forceinline__ float gate_value(const DecodeArgs &a, uint32_t seq, uint32_t head, uint32_t d) {
    if (a.fuse_append)   // the gate is the second half of the token's q_proj_full row (wgsl:122-135)
        return load_as_f32(a.ap_q, ((size_t)seq * a.nh + head) * 2 * a.hd + a.hd + d, a.ap_in_dtype);
    return a.gate[((size_t)seq * a.nh + head) * a.hd + d];
}
__device__ __forceinline__ bool has_gate(const DecodeArgs &a) { return a.fuse_append ? a.ap_has_gate != 0 : a.gate != nullptr; }

// ---- balanced ("stream-K") partition of the batch -------------------------------------------
// All sequences are laid end to end on a line of 16-position row-blocks; span c owns units
// [ceil(c*T/C), ceil((c+1)*T/C)) of it.  A span may end one sequence, hold several whole ones and start
// another; each intersection is a "piece".  There is one full wave and no tail.
// Every sequence is followed by a.pad units that stand for no rows: starting a second piece costs a CTA about
// 8 us (its pipeline drains 0.8, the warps' states are merged, a record written, fenced and counted 3.6, the next
// sequence's pointers, Q rows and first tiles are requested 2.7, and data has to arrive) — in the cfg2 batch the CTAs
// whose span held a sequence boundary ended at 78-89 us and the others at 69-73 us.  A span that contains a boundary
// also contains the pad and so gets that many fewer row-blocks: spans are equal in time, not in rows (after: both
// kinds end at 77-79 us on average; what is left of the spread, 64-90 us, is between CTAs of equal work).  A span that
// begins inside a pad starts at the next sequence's first block.
// (products that fit 32 bits — every batch short of some 50 million rows — take the 32-bit divider: the 64-bit one
//  is a long dependent instruction sequence, and these sit at the head of every piece)
__device__ __forceinline__ uint32_t span_begin(const DecodeArgs &a, uint32_t c) {
    if (a.span_math32) return (c * a.line_blocks + a.spans - 1) / a.spans;
    return (uint32_t)(((unsigned long long)c * a.line_blocks + a.spans - 1) / a.spans);
}
__device__ __forceinline__ uint32_t span_of(const DecodeArgs &a, uint32_t u) {
    if (a.span_math32) return (u * a.spans) / a.line_blocks;
    return (uint32_t)(((unsigned long long)u * a.spans) / a.line_blocks);
}
__device__ __forceinline__ uint32_t blocks_of(uint32_t L) { return L == 0 ? 1u : (L + kBlkPos - 1) / kBlkPos; }

struct Piece {
    uint32_t seq, L, start, end;  // positions [start, end) of sequence seq
    uint32_t nrec;                // records this sequence is split into (1 => written directly)
    uint32_t my_rec;              // which of them this piece is
    uint32_t c0;                  // balanced: first span of the sequence; explicit: seq * ns
    uint32_t B;                   // balanced: first row-block of the sequence on the line
};
struct Cursor {
    uint32_t seq, B, u, u1, span, done;
};

// Record r of `head` for the sequence a piece belongs to.
__device__ __forceinline__ float *rec_ptr(const DecodeArgs &a, const Piece &p, uint32_t head, uint32_t r) {
    if (a.num_splits || a.force_partials)  // reference layout [nh][ns][hd+2] per sequence (wgsl:112-123)
        return a.partials + ((size_t)p.c0 * a.nh + (size_t)head * p.nrec + r) * (a.hd + 2);
    // balanced: two slots per span — slot 0 if the piece starts at the span's first block, else slot 1
    const uint32_t c = p.c0 + r;
    const uint32_t slot = span_begin(a, c) >= p.B ? 0u : 1u;
    return a.partials + (((size_t)c * 2 + slot) * a.nh + head) * (a.hd + 2);
}

// Position the cursor at this CTA's first piece.  Warp 0 scans the lengths; res is shared memory.
__device__ __forceinline__ void cursor_init(const DecodeArgs &a, uint32_t work, uint32_t lane, uint32_t *res) {
    if (a.num_splits) {
        if (lane == 0) { res[0] = work / a.num_splits; res[1] = 0; res[2] = work % a.num_splits; res[3] = 0; res[4] = 0; }
        return;
    }
    const uint32_t u0 = span_begin(a, work), u1 = span_begin(a, work + 1);
    uint32_t pref = 0;
    bool found = false;
    for (uint32_t base = 0; base < a.num_seqs && !found; base += 32) {
        const uint32_t j = base + lane;
        const uint32_t nb = j < a.num_seqs ? blocks_of(seq_len_at(a, j)) + a.pad : 0u;   // the sequence's extent on the line
        uint32_t incl = nb;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= (uint32_t)o) incl += n;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        if (u0 < pref + total) {
            const uint32_t mask = __ballot_sync(0xffffffffu, pref + incl > u0);
            const uint32_t f = __ffs(mask) - 1;
            const uint32_t ext = __shfl_sync(0xffffffffu, nb, f);
            const uint32_t excl = __shfl_sync(0xffffffffu, incl, f) - ext;
            if (lane == 0) {
                uint32_t seq = base + f, B = pref + excl, u = u0;
                if (u0 >= B + ext - a.pad) { ++seq; B += ext; u = B; }   // the span begins in the pad: on to the next sequence
                res[0] = seq; res[1] = B; res[2] = u; res[3] = u1; res[4] = 0;
            }
            found = true;
        }
        pref += total;
    }
    if (!found && lane == 0) { res[0] = a.num_seqs; res[1] = 0; res[2] = 0; res[3] = 0; res[4] = 1; }
}

__device__ __forceinline__ bool next_piece(const DecodeArgs &a, Cursor &cur, Piece &p) {
    if (cur.done) return false;
    if (a.num_splits) {
        cur.done = 1;
        const uint32_t ns = a.num_splits, split = cur.u;
        p.seq = cur.seq; p.L = seq_len_at(a, cur.seq);
        const uint32_t pps = (p.L + ns - 1u) / ns;  // wgsl:46
        p.start = min(split * pps, p.L); p.end = min(p.start + pps, p.L);
        p.nrec = ns; p.my_rec = split; p.c0 = cur.seq * ns; p.B = 0;
        return true;
    }
    if (cur.u >= cur.u1 || cur.seq >= a.num_seqs) return false;
    const uint32_t L = seq_len_at(a, cur.seq), nb = blocks_of(L);
    const uint32_t ub1 = min(cur.u1, cur.B + nb);
    p.seq = cur.seq; p.L = L;
    p.start = min((cur.u - cur.B) * kBlkPos, L);
    p.end = min((ub1 - cur.B) * kBlkPos, L);
    p.B = cur.B; p.c0 = span_of(a, cur.B);
    p.nrec = span_of(a, cur.B + nb - 1) - p.c0 + 1;
    p.my_rec = cur.span - p.c0;
    cur.u = ub1;
    if (ub1 == cur.B + nb) { cur.B += nb + a.pad; cur.seq++; cur.u = cur.B; }   // over the pad (possibly past the span's end)
    return true;
}

// Merge the per-warp (m, l, O) states of one CTA for one piece and write either the final rows or
// the piece's record ([hd] = lse, [hd+1] = running max as in wgsl:112-123).  When the sequence has
// several records, the CTA that arrives last for its (sequence, kv head, head group) merges all of
// them (gqa_reduce.wgsl:20-65) — no second launch.
// Warp w's O tile starts at sm_o + w*WSTRIDE floats, rows of HD floats.
// The CTA serves KPC kv heads (kvh_base + k); warps k, k+KPC, k+2*KPC, ... share kv head k.
// OSTRIDE: floats between consecutive head rows of a warp's O tile (padded by the 16-bit kernel against bank conflicts)
template <int R, int HD, int NW, int WSTRIDE, int KPC, int OSTRIDE = HD>
__device__ __forceinline__ void finish_piece(const DecodeArgs &a, const Piece &p, float *sm_m, float *sm_l,
                                             const float *sm_o, uint32_t *sm_flag, uint32_t *scratch,
                                             uint32_t scratch_words, uint32_t kvh_base, uint32_t row0,
                                             uint32_t rows_valid, uint32_t counter_idx) {
    const bool direct = (p.nrec == 1u) && !a.force_partials;
    // ---- per head row, once: the warps' weights e_w = 2^(m_w - M), the row's sum L, the normalised weights e_w / L
    //      (left in sm_m in place of m_w) and the row's log-sum-exp.  Which record slot the piece writes is one
    //      64-bit division (rec_ptr) for the whole piece: it is resolved here, not per element ----
    const bool ref_layout = a.num_splits || a.force_partials;
    uint32_t rec_row0 = 0;
    if (!direct && !ref_layout) {
        const uint32_t c = p.c0 + p.my_rec;
        rec_row0 = (c * 2 + (span_begin(a, c) >= p.B ? 0u : 1u)) * a.nh;
    }
    auto rec_of = [&](uint32_t head) {
        return ref_layout ? a.partials + ((size_t)p.c0 * a.nh + (size_t)head * p.nrec + p.my_rec) * (a.hd + 2)
                          : a.partials + ((size_t)rec_row0 + head) * (a.hd + 2);
    };
    if (threadIdx.x < KPC * rows_valid) {
        const uint32_t r = threadIdx.x % rows_valid, kvl = threadIdx.x / rows_valid;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w)
            if (w % KPC == (int)kvl) M = fmaxf(M, sm_m[w * R + r]);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            if (w % KPC != (int)kvl) continue;
            const float mw = sm_m[w * R + r];
            const float e = mw > -INFINITY ? exp2f(mw - M) : 0.f;
            if (mw > -INFINITY) L += sm_l[w * R + r] * e;
            sm_m[w * R + r] = e;
        }
        // the element loop below multiplies by e_w / L: one division per head row here instead of one per element there
        const float inv_l = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w)
            if (w % KPC == (int)kvl) sm_m[w * R + r] *= inv_l;
        const float lse = L > 0.f ? logf(L) + M * kLn2 : -INFINITY;
        const uint32_t head = (kvh_base + kvl) * a.G + row0 + r;
        if (direct) {
            if (a.lse) a.lse[((size_t)p.seq * a.nh + head) * a.lse_stride] = lse;
        } else {
            float *rec = rec_of(head);
            rec[HD] = lse;
            rec[HD + 1] = L > 0.f ? M * kLn2 : -INFINITY;
        }
    }
    __syncthreads();
    // rows outside, head dims across the threads: no index arithmetic with run-time divisors per element
    if constexpr (KPC == 1) {
        // four head rows per round: all their shared-memory reads first, then the stores (a store to global memory
        // in between keeps the compiler from moving the next row's reads above it, and the rows ran one after another)
        for (uint32_t d = threadIdx.x; d < HD; d += NW * 32) {
            for (uint32_t r0 = 0; r0 < rows_valid; r0 += 4) {
                float val[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t r = min(r0 + j, rows_valid - 1);   // past the last row: a valid read, never stored
                    val[j] = 0.f;
#pragma unroll
                    for (int w = 0; w < NW; ++w) val[j] += sm_o[(size_t)w * WSTRIDE + r * OSTRIDE + d] * sm_m[w * R + r];   // empty warps and rows: 0 * 0
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (r0 + j >= rows_valid) break;
                    const uint32_t head = kvh_base * a.G + row0 + r0 + j;
                    if (direct) {
                        float v = val[j];
                        if (has_gate(a)) v *= sigmoidf_ref(gate_value(a, p.seq, head, d));
                        store_from_f32(a.out, ((size_t)p.seq * a.nh + head) * a.out_row_stride + d, a.out_dtype, v);
                    } else {
                        rec_of(head)[d] = val[j];
                    }
                }
            }
        }
    } else {
        uint32_t r = 0, kvl = 0;
#pragma unroll 4
        for (uint32_t hr = 0; hr < KPC * rows_valid; ++hr) {
            const uint32_t head = (kvh_base + kvl) * a.G + row0 + r;
            float *rec = direct ? nullptr : rec_of(head);
            for (uint32_t d = threadIdx.x; d < HD; d += NW * 32) {
                float val = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w)
                    if (w % KPC == (int)kvl) val += sm_o[(size_t)w * WSTRIDE + r * OSTRIDE + d] * sm_m[w * R + r];   // empty warps and rows: 0 * 0
                if (direct) {
                    if (has_gate(a)) val *= sigmoidf_ref(gate_value(a, p.seq, head, d));
                    store_from_f32(a.out, ((size_t)p.seq * a.nh + head) * a.out_row_stride + d, a.out_dtype, val);
                } else {
                    rec[d] = val;
                }
            }
            if (++r == rows_valid) { r = 0; ++kvl; }
        }
    }
    if (direct || a.force_partials || a.defer_merge) return;
    // ---- last-arriving CTA merges the records ----
    __syncthreads();   // every thread's record stores are issued ...
    if (threadIdx.x == 0) {
        __threadfence();   // ... and this fence, being cumulative over what the barrier ordered before it, publishes them all
        // atomicInc wraps to 0 when the old value is nrec-1, so the counter is zero again for the next call
        const uint32_t old = atomicInc(&a.counters[counter_idx], p.nrec - 1u);
        *sm_flag = (old == p.nrec - 1u);
    }
    __syncthreads();
    if (!*sm_flag) return;
    __threadfence();
    // scratch: [nrec] record bases | [rows] gmax | [rows] wsum | [RG][nrec] weights
    const uint32_t nrec = p.nrec, rows_total = KPC * rows_valid;
    uint32_t *sm_rec = scratch;
    float *sm_gmax = reinterpret_cast<float *>(scratch + nrec);
    float *sm_wsum = sm_gmax + rows_total;
    float *sm_w = sm_wsum + rows_total;
    const uint32_t RG = min(rows_total, (scratch_words - nrec - 2 * rows_total) / nrec);  // >= 1 by construction
    // record s of head h lives at partials + (sm_rec[s] + h*hmul) * (HD+2)
    const uint32_t hmul = (a.num_splits || a.force_partials) ? nrec : 1u;
    for (uint32_t s = threadIdx.x; s < nrec; s += NW * 32) {
        if (a.num_splits) sm_rec[s] = p.c0 * a.nh + s;
        else {
            const uint32_t c = p.c0 + s;
            sm_rec[s] = (c * 2 + (span_begin(a, c) >= p.B ? 0u : 1u)) * a.nh;
        }
    }
    __syncthreads();
    if (nrec <= 4) {
        // Few records (the usual case of a batch: a sequence cut by one or two span boundaries): every thread requests
        // the log-sum-exps and the values of its elements in one go — one L2 round trip instead of three with two
        // CTA barriers in between.
        // four head rows at a time, all their loads requested before the first is used
        for (uint32_t d = threadIdx.x; d < HD; d += NW * 32) {
            for (uint32_t hr0 = 0; hr0 < rows_total; hr0 += 4) {
                float l[4][4], v[4][4];
                uint32_t heads[4];
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) {
                    const uint32_t hr = min(hr0 + k, rows_total - 1);           // clamped rows recompute a valid row
                    heads[k] = (kvh_base + hr / rows_valid) * a.G + row0 + hr % rows_valid;
#pragma unroll
                    for (uint32_t s2 = 0; s2 < 4; ++s2) {
                        const float *rp = a.partials + ((size_t)sm_rec[min(s2, nrec - 1)] + (size_t)heads[k] * hmul) * (HD + 2);
                        l[k][s2] = s2 < nrec ? __ldcg(rp + HD) : -INFINITY;
                        v[k][s2] = s2 < nrec ? __ldcg(rp + d) : 0.f;
                    }
                }
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) {
                    if (hr0 + k >= rows_total) break;
                    float gmax = -INFINITY;
#pragma unroll
                    for (uint32_t s2 = 0; s2 < 4; ++s2)
                        if (l[k][s2] > -INFINITY) gmax = fmaxf(gmax, l[k][s2]);
                    float acc = 0.f, wsum = 0.f;
#pragma unroll
                    for (uint32_t s2 = 0; s2 < 4; ++s2) {
                        const float w = l[k][s2] > -INFINITY ? expf(l[k][s2] - gmax) : 0.f;   // gqa_reduce.wgsl:56; empty ranges weigh nothing
                        acc += w > 0.f ? w * v[k][s2] : 0.f;
                        wsum += w;
                    }
                    float val = wsum > 0.f ? acc / wsum : 0.f;
                    const uint32_t head = heads[k];
                    if (has_gate(a)) val *= sigmoidf_ref(gate_value(a, p.seq, head, d));
                    store_from_f32(a.out, ((size_t)p.seq * a.nh + head) * a.out_row_stride + d, a.out_dtype, val);
                    if (d == 0 && a.lse) a.lse[((size_t)p.seq * a.nh + head) * a.lse_stride] = wsum > 0.f ? gmax + logf(wsum) : -INFINITY;
                }
            }
        }
        return;
    }
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t rg0 = 0; rg0 < rows_total; rg0 += RG) {
        const uint32_t nrows = min(RG, rows_total - rg0);
        // weights of every record for each head row: w_s = exp(lse_s - max lse)  (gqa_reduce.wgsl:33-56)
        for (uint32_t row = warp; row < nrows; row += NW) {
            const uint32_t hr = rg0 + row, r = hr % rows_valid, kvl = hr / rows_valid;
            const uint32_t head = (kvh_base + kvl) * a.G + row0 + r;
            float gmax = -INFINITY;
            for (uint32_t s = lane; s < nrec; s += 32) {
                const float l = __ldcg(a.partials + ((size_t)sm_rec[s] + (size_t)head * hmul) * (HD + 2) + HD);
                sm_w[row * nrec + s] = l;
                if (l > -INFINITY) gmax = fmaxf(gmax, l);  // false for -inf and NaN: empty ranges
            }
            gmax = warp_max(gmax);
            float wsum = 0.f;
            for (uint32_t s = lane; s < nrec; s += 32) {
                const float l = sm_w[row * nrec + s];
                const float w = l > -INFINITY ? expf(l - gmax) : 0.f;
                sm_w[row * nrec + s] = w;
                wsum += w;
            }
            wsum = warp_sum(wsum);
            if (lane == 0) { sm_gmax[hr] = gmax; sm_wsum[hr] = wsum; }
        }
        __syncthreads();
        // EU independent elements per thread keep EU record loads in flight: the merge is L2-latency bound
        constexpr uint32_t EU = 4, NT = NW * 32;
        const uint32_t nelem = nrows * HD;
        for (uint32_t idx0 = threadIdx.x; idx0 < nelem; idx0 += NT * EU) {
            float acc[EU];
            const float *src[EU];
            const float *wrow[EU];
#pragma unroll
            for (uint32_t k = 0; k < EU; ++k) {
                const uint32_t idx = min(idx0 + k * NT, nelem - 1);   // clamped lanes recompute a valid element
                const uint32_t d = idx % HD, row = idx / HD;
                const uint32_t hr = rg0 + row, r = hr % rows_valid, kvl = hr / rows_valid;
                const uint32_t head = (kvh_base + kvl) * a.G + row0 + r;
                src[k] = a.partials + (size_t)head * hmul * (HD + 2) + d;
                wrow[k] = sm_w + row * nrec;
                acc[k] = 0.f;
            }
#pragma unroll 2
            for (uint32_t s = 0; s < nrec; ++s) {
                const size_t off = (size_t)sm_rec[s] * (HD + 2);
                float v[EU];
#pragma unroll
                for (uint32_t k = 0; k < EU; ++k) v[k] = __ldcg(src[k] + off);
#pragma unroll
                for (uint32_t k = 0; k < EU; ++k) {
                    const float w = wrow[k][s];
                    acc[k] += w > 0.f ? w * v[k] : 0.f;   // weight 0 also hides NaN payloads of empty ranges
                }
            }
#pragma unroll
            for (uint32_t k = 0; k < EU; ++k) {
                const uint32_t idx = idx0 + k * NT;
                if (idx >= nelem) break;
                const uint32_t d = idx % HD, row = idx / HD;
                const uint32_t hr = rg0 + row, r = hr % rows_valid, kvl = hr / rows_valid;
                const uint32_t head = (kvh_base + kvl) * a.G + row0 + r;
                const float wsum = sm_wsum[hr];
                float val = wsum > 0.f ? acc[k] / wsum : 0.f;
                    const size_t oi = ((size_t)p.seq * a.nh + head) * a.out_row_stride + d;
                if (has_gate(a)) val *= sigmoidf_ref(gate_value(a, p.seq, head, d));
                store_from_f32(a.out, oi, a.out_dtype, val);
                if (d == 0 && a.lse) a.lse[((size_t)p.seq * a.nh + head) * a.lse_stride] = wsum > 0.f ? sm_gmax[hr] + logf(wsum) : -INFINITY;
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// 16-bit cache path
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t smem, const void *gptr, bool valid) {
    const int sz = valid ? 16 : 0;  // src-size 0 => 16 bytes of zeros, nothing read
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gptr), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// transposes an 8x8 matrix of 16-bit elements held one row per eight threads (the mma C layout -> its B layout)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// Two 8-bit floats -> f16x2.  `SEL` picks the bytes of x: the low half of the result comes from byte (SEL & 0xf),
// the high half from byte (SEL >> 4).  FMT 1 = e4m3, 2 = e5m2.
//  * e5m2 is the top byte of the f16 with the same value: one byte permute.
//  * An e4m3 byte s.eeee.mmm, shifted left by 7 inside its 16-bit half, has its magnitude where the f16
//    0eeee.mmm0000000 wants it — 2^(e-15) (1 + m/8) for e > 0, the f16 subnormal m 2^-17 for e = 0: in both cases the
//    e4m3 value times 2^-8, so one factor 256 on the score scale (K) and on the output (V) puts it right — and its
//    sign one bit too low; adding the sign bit to itself moves it up (the carry never leaves the half).  The shift
//    and the add are written as multiply-adds so that they can go to the FMA pipe: widening the bytes is integer
//    work, and it is the integer pipe, not memory, that bounds this kernel (cvt.rn.f16x2.e4m3x2 measured no faster).
__host__ __device__ constexpr float f8_unscale(int fmt) { return fmt == 1 ? 256.0f : 1.0f; }
// One value into the cache's 8-bit format (1: e4m3, 2: e5m2), rounded and saturated as the stand-alone append does it.
template <int FMT> __device__ __forceinline__ unsigned char f32_to_f8(float v) {
    if constexpr (FMT == 2) return __nv_fp8_e5m2(v).__x;
    else return __nv_fp8_e4m3(v).__x;
}
template <int FMT, uint32_t SEL> __device__ __forceinline__ uint32_t f8x2_to_f16x2(uint32_t x) {
    if constexpr (FMT == 2) {
        // result byte 1 <- x byte (SEL & 0xf), result byte 3 <- x byte (SEL >> 4), bytes 0 and 2 <- 0
        return __byte_perm(x, 0u, 0x0404u | ((SEL & 0xfu) << 4) | ((SEL >> 4) << 12));
    } else {
        // result byte 0 <- x byte (SEL & 0xf), result byte 2 <- x byte (SEL >> 4), bytes 1 and 3 <- 0
        const uint32_t z = __byte_perm(x, 0u, 0x4040u | (SEL & 0xfu) | ((SEL >> 4) << 8));
        uint32_t t, out;
        asm("mad.lo.u32 %0, %1, 128, 0;" : "=r"(t) : "r"(z));                  // bytes at bits 14..7 and 30..23
        asm("mad.lo.u32 %0, %1, 1, %2;" : "=r"(out) : "r"(t & 0x40004000u), "r"(t));   // sign: bit 14 -> bit 15
        return out;
    }
}

constexpr int kBlk = (int)kBlkPos;  // positions per warp block (one MMA k-step of P·V)

template <int HD, int NW, int STAGES, int KPC, int F8 = 0> struct Decode16Smem {
    static constexpr int kRowBytes = HD * (F8 ? 1 : 2);          // one kv head's part of a cache row
    static constexpr int kTileBytes = kBlk * kRowBytes;          // one K or V block
    static constexpr int kWarpBytes = STAGES * kTileBytes;       // ring of STAGES tile slots; K and V tiles alternate in it
    static constexpr int kQRowBytes = HD * 2;                    // Q is staged as 16-bit whatever the cache holds
    static constexpr int kQTile = 16 * kQRowBytes;               // Q rows of one kv head
    static constexpr int kQBytes = KPC * kQTile;
    static constexpr int kStatBytes = (2 * NW * 16 * 4 > HD * 4) ? 2 * NW * 16 * 4 : HD * 4;   // merge m and l; cos/sin table of the fused append
    static constexpr int kTotal = kQBytes + NW * kWarpBytes + kStatBytes + 32;
    // floats per head row of a warp's O tile: 8 pad floats put the eight rows a store instruction touches on different
    // banks (where the warp's pipeline memory has room for them)
    static constexpr int kORow = kWarpBytes >= 16 * (HD + 8) * 4 ? HD + 8 : HD;
    static_assert(kWarpBytes >= 16 * kORow * 4, "merge tile must fit in the warp's pipeline memory");
};

// ---------------------------------------------------------------------------------------
// Record merge by the decode grid itself (cooperative launch, a.grid_merge).  A sequence that is cut into many
// spans would leave its merge to a second launch; ~10 us behind a 50 us kernel, most of it launch gap and
// ramp-up.  Here every CTA, after its last record, arrives at a grid barrier (the launch is cooperative, so all
// CTAs are resident; the wait is bounded all the same and raises the status word if it runs out), and the grid
// then merges the records: a work item is 32 dims of one head, warp g of the CTA takes the records g, g + NW, ...
// with a running maximum of its own (values and log-sum-exps of a batch requested together: one L2 round trip),
// and the warps are rescaled to a common maximum and summed through shared memory.  The last CTA
// to leave zeroes the barrier for the next launch.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr int kTailBatch = 20;   // records whose value and log-sum-exp one thread requests together (148 records over 8 warps: one round trip; over the 4 warps of a half in the exchange tail: two)

// What the tail reads in its dependent chains, by value: the function is not inlined (inlined, it cost the
// streaming loop registers), and through the reference every field of the kernel's parameter block is a
// generic-address load, several of them in a row ahead of the first record request.
struct TailArgs {
    const float *partials;
    void *out;
    float *lse;
    uint32_t *grid_sync;
    StatusRef status;
    uint32_t wait_grid, wait_peer;
    uint32_t nh, hd, num_seqs, out_row_stride, lse_stride, out_dtype, spans, line_blocks, span_math32, gated;
    uint32_t len0;   // length of sequence 0 (the others are read through the reference)
    uint32_t pad;
};
__device__ __forceinline__ TailArgs tail_args(const DecodeArgs &a) {
    return TailArgs{a.partials, a.out, a.lse, a.grid_sync, a.status, a.wait_grid, a.wait_peer, a.nh, a.hd, a.num_seqs, a.out_row_stride,
                    a.lse_stride, a.out_dtype, a.spans, a.line_blocks, a.span_math32, has_gate(a) ? 1u : 0u,
                    seq_len_at(a, 0), a.pad};
}

// The two halves of the grid barrier, both called by thread 0 of every CTA after its arrival (atomicAdd on
// grid_sync[0]).  The wait is bounded (ta.wait_grid polls) and is skipped when an earlier wait of this context has
// already run out; a CTA that does not get through skips the merge but still leaves, so the barrier words are
// clean again when the kernel ends, whatever happened.
__device__ __forceinline__ uint32_t grid_barrier_wait(const TailArgs &ta) {
    uint32_t ok = 0;
    if (!gave_up(ta.status))
        for (uint32_t i = 0; i < ta.wait_grid; ++i)
            if (ld_acquire_gpu(ta.grid_sync) >= gridDim.x) { ok = 1; break; }
    if (!ok) report_timeout(ta.status, 90);
    return ok;
}
__device__ __forceinline__ void grid_barrier_leave(const TailArgs &ta) {
    if (atomicInc(ta.grid_sync + 1, gridDim.x - 1) == gridDim.x - 1) *ta.grid_sync = 0;   // every CTA is past the wait
}

template <int NW>
__device__ __noinline__ void grid_merge_tail(const DecodeArgs &a, const TailArgs ta, uint32_t *scratch) {
    const uint32_t tid = threadIdx.x, g = tid >> 5, t = tid & 31u;
    float *sm_acc = reinterpret_cast<float *>(scratch);                // [NW][32] weighted sums of each warp's records
    float *sm_ws = sm_acc + NW * 32;                                   // [NW] sums of weights
    float *sm_mx = sm_ws + NW;                                         // [NW] the maximum each warp's weights refer to
    uint32_t *sm_misc = reinterpret_cast<uint32_t *>(sm_mx + NW);      // {barrier passed, first row-block of the sequence}
    if (tid == 0) {
        __threadfence();   // cumulative over the record stores the CTA barrier before this call ordered
        atomicAdd(ta.grid_sync, 1u);
    }
    auto first_block_of_span = [&](uint32_t c) {   // span_begin / span_of on the by-value fields
        return ta.span_math32 ? (c * ta.line_blocks + ta.spans - 1) / ta.spans
                              : (uint32_t)(((unsigned long long)c * ta.line_blocks + ta.spans - 1) / ta.spans);
    };
    auto span_of_block = [&](uint32_t u) {
        return ta.span_math32 ? (u * ta.spans) / ta.line_blocks : (uint32_t)(((unsigned long long)u * ta.spans) / ta.line_blocks);
    };
    const uint32_t chunks = ta.hd / 32, items = ta.num_seqs * ta.nh * chunks, rs = ta.hd + 2;
    // Where an item's records are: three integer divisions and, past the first sequence, a sum over the lengths.
    // A long dependent chain, so the first item's is worked out before the wait below, not after it.
    struct Item { uint32_t seq, head, d, nrec; const float *row0; uint32_t skip0; };
    auto locate = [&](uint32_t it) {
        Item x;
        const uint32_t chunk = it % chunks;
        x.head = (it / chunks) % ta.nh; x.seq = it / (chunks * ta.nh); x.d = chunk * 32 + t;
        uint32_t B = 0;
        if (x.seq) {   // first row-block of this sequence on the line
            __syncthreads();
            if (tid < 32) {
                uint32_t acc = 0;
                for (uint32_t j = tid; j < x.seq; j += 32) acc += blocks_of(seq_len_at(a, j)) + ta.pad;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (tid == 0) sm_misc[1] = acc;
            }
            __syncthreads();
            B = sm_misc[1];
        }
        const uint32_t nb = blocks_of(x.seq ? seq_len_at(a, x.seq) : ta.len0);
        const uint32_t c0 = span_of_block(B);
        x.nrec = span_of_block(B + nb - 1) - c0 + 1;
        // only the sequence's first span can have begun before the sequence: its record is in slot 1 then
        x.skip0 = first_block_of_span(c0) >= B ? 0u : 1u;
        x.row0 = ta.partials + ((size_t)(c0 * 2) * ta.nh + x.head) * rs;     // slot 0 of the sequence's first span
        return x;
    };
    Item cur{};
    if (blockIdx.x < items) cur = locate(blockIdx.x);
    if (tid == 0) sm_misc[0] = grid_barrier_wait(ta);
    __syncthreads();
    for (uint32_t it = blockIdx.x; it < items && sm_misc[0]; it += gridDim.x) {
        const uint32_t seq = cur.seq, head = cur.head, d = cur.d, nrec = cur.nrec;
        if (nrec > 1) {       // a single record went straight to the output
            const size_t span_stride = (size_t)2 * ta.nh * rs;               // floats between the slot-0 records of two spans
            const float *row_first = cur.row0 + (cur.skip0 ? (size_t)ta.nh * rs : 0);
            float m = -INFINITY, acc = 0.f, wsum = 0.f;
            for (uint32_t base = g; base < nrec; base += kTailBatch * NW) {
                float v[kTailBatch], l[kTailBatch];
#pragma unroll
                for (int i = 0; i < kTailBatch; ++i) {   // one round trip for the whole batch, values and weights together
                    const uint32_t s = base + i * NW;
                    v[i] = 0.f; l[i] = -INFINITY;
                    if (s < nrec) {
                        const float *row = s == 0 ? row_first : cur.row0 + s * span_stride;
                        v[i] = __ldcg(row + d);
                        l[i] = __ldcg(row + ta.hd);
                    }
                }
                float bm = m;
#pragma unroll
                for (int i = 0; i < kTailBatch; ++i) bm = fmaxf(bm, l[i]);
                if (bm > -INFINITY) {
                    const float sc = expf(m - bm);           // 0 while nothing has been accumulated (m = -inf)
                    acc *= sc; wsum *= sc;
#pragma unroll
                    for (int i = 0; i < kTailBatch; ++i)
                        if (l[i] > -INFINITY) {              // gqa_reduce.wgsl:56; empty ranges weigh nothing
                            const float w = expf(l[i] - bm);
                            acc += w * v[i];
                            wsum += w;
                        }
                    m = bm;
                }
            }
            sm_acc[g * 32 + t] = acc;
            if (t == 0) { sm_ws[g] = wsum; sm_mx[g] = m; }
            __syncthreads();
            if (g == 0) {
                float gmax = -INFINITY;
#pragma unroll
                for (int k = 0; k < NW; ++k) gmax = fmaxf(gmax, sm_mx[k]);
                acc = 0.f; wsum = 0.f;
#pragma unroll
                for (int k = 0; k < NW; ++k)
                    if (sm_mx[k] > -INFINITY) {
                        const float sc = expf(sm_mx[k] - gmax);
                        acc += sc * sm_acc[k * 32 + t];
                        wsum += sc * sm_ws[k];
                    }
                float val = wsum > 0.f ? acc / wsum : 0.f;
                if (ta.gated) val *= sigmoidf_ref(gate_value(a, seq, head, d));
                store_from_f32(ta.out, ((size_t)seq * ta.nh + head) * ta.out_row_stride + d, ta.out_dtype, val);
                if (d == 0 && ta.lse) ta.lse[((size_t)seq * ta.nh + head) * ta.lse_stride] = wsum > 0.f ? gmax + logf(wsum) : -INFINITY;
            }
        }
        if (it + gridDim.x < items) {
            __syncthreads();   // the scratch words are rewritten for the next item
            cur = locate(it + gridDim.x);
        }
    }
    if (tid == 0) grid_barrier_leave(ta);
}

// The same tail for a row-sharded sequence (one process per GPU): after the grid barrier a CTA merges 64 dims of one
// head from this rank's records (two groups of NW/2 warps, 32 dims each) and the two finishing warps then do what
// shard_merge_p2p_kernel does — slice and log-sum-exp into every rank's exchange buffer with plain peer stores, a
// system-scope release flag per (rank, head, chunk), a bounded wait for the peers' flags, the merge across ranks.
// One launch per step instead of two.
template <int NW>
__device__ __noinline__ void grid_exchange_tail(const DecodeArgs &a, const TailArgs ta, uint32_t *scratch) {
    constexpr int HW = NW / 2;   // warps per 32-dim half
    static_assert(NW >= 2 && NW % 2 == 0, "two groups of warps");
    const uint32_t tid = threadIdx.x, g = tid >> 5, t = tid & 31u, half = g / HW, gw = g % HW;
    float *sm_acc = reinterpret_cast<float *>(scratch);                // [NW][32]
    float *sm_ws = sm_acc + NW * 32;                                   // [NW]
    float *sm_mx = sm_ws + NW;                                         // [NW]
    float *sm_lse = sm_mx + NW;                                        // [kP2PMaxWorld]
    uint32_t *sm_misc = reinterpret_cast<uint32_t *>(sm_lse + kP2PMaxWorld);   // {barrier passed, a flag wait ran out}
    if (tid == 0) {
        __threadfence();
        atomicAdd(ta.grid_sync, 1u);
        sm_misc[1] = 0;
    }
    // everything the exchange needs from the parameter block and the peer table, read while the barrier fills
    const uint32_t world = a.px_world, rank = a.px_rank, epoch = a.px_epoch, par = epoch & 1u, out_dt = a.px_out_dtype;
    char *const *bases = a.px_peer_bases;
    void *const final_out = a.px_out;
    const float *const final_gate = a.px_gate;
    const uint32_t xt = half * 32 + t;                                 // 0..63 within the two finishing warps
    char *const my_base = bases[rank];
    char *const peer_base = xt < world ? bases[xt] : nullptr;
    const uint32_t nb = blocks_of(ta.len0);
    const uint32_t nrec = (ta.span_math32 ? ((nb - 1) * ta.spans) / ta.line_blocks
                                          : (uint32_t)(((unsigned long long)(nb - 1) * ta.spans) / ta.line_blocks)) + 1;
    const uint32_t chunks = p2p_chunks(ta.hd), items = ta.nh * chunks, rs = ta.hd + 2;
    const unsigned long long flags_bytes = p2p_chunk_flags_bytes(world, ta.nh, ta.hd);
    if (tid == 0) sm_misc[0] = grid_barrier_wait(ta);
    __syncthreads();
    auto bar64 = [] { asm volatile("bar.sync 1, 64;" ::: "memory"); };
    for (uint32_t it = blockIdx.x; it < items && sm_misc[0]; it += gridDim.x) {
        const uint32_t head = it / chunks, chunk = it % chunks;
        const uint32_t d = chunk * kP2PChunk + xt, dd = min(d, ta.hd - 1);
        float val, lse;
        if (nrec == 1) {   // the only record went straight to the rank's record buffer (ta.out / ta.lse)
            val = __ldcg(reinterpret_cast<const float *>(ta.out) + (size_t)head * ta.out_row_stride + dd);
            lse = ta.lse ? __ldcg(ta.lse + (size_t)head * ta.lse_stride) : 0.f;
        } else {
            const float *row0 = ta.partials + (size_t)head * rs;      // slot 0 of span 0 (the sequence starts the line)
            const size_t span_stride = (size_t)2 * ta.nh * rs;
            float m = -INFINITY, acc = 0.f, wsum = 0.f;
            for (uint32_t base = gw; base < nrec; base += kTailBatch * HW) {
                float v[kTailBatch], l[kTailBatch];
#pragma unroll
                for (int i = 0; i < kTailBatch; ++i) {
                    const uint32_t s = base + i * HW;
                    v[i] = 0.f; l[i] = -INFINITY;
                    if (s < nrec) {
                        const float *row = row0 + s * span_stride;
                        v[i] = __ldcg(row + dd);
                        l[i] = __ldcg(row + ta.hd);
                    }
                }
                float bm = m;
#pragma unroll
                for (int i = 0; i < kTailBatch; ++i) bm = fmaxf(bm, l[i]);
                if (bm > -INFINITY) {
                    const float sc = expf(m - bm);
                    acc *= sc; wsum *= sc;
#pragma unroll
                    for (int i = 0; i < kTailBatch; ++i)
                        if (l[i] > -INFINITY) {              // gqa_reduce.wgsl:56; empty ranges weigh nothing
                            const float w = expf(l[i] - bm);
                            acc += w * v[i];
                            wsum += w;
                        }
                    m = bm;
                }
            }
            sm_acc[g * 32 + t] = acc;
            if (t == 0) { sm_ws[g] = wsum; sm_mx[g] = m; }
            __syncthreads();
            float gmax = -INFINITY;
#pragma unroll
            for (int k = 0; k < HW; ++k) gmax = fmaxf(gmax, sm_mx[half * HW + k]);
            acc = 0.f; wsum = 0.f;
#pragma unroll
            for (int k = 0; k < HW; ++k) {
                const float mk = sm_mx[half * HW + k];
                if (mk > -INFINITY) {
                    const float sc = expf(mk - gmax);
                    acc += sc * sm_acc[(half * HW + k) * 32 + t];
                    wsum += sc * sm_ws[half * HW + k];
                }
            }
            val = wsum > 0.f ? acc / wsum : 0.f;
            lse = wsum > 0.f ? gmax + logf(wsum) : -INFINITY;
        }
        if (gw == 0) {   // the first warp of each half: 64 threads, meeting at a named barrier of their own
            const size_t my_slot = (((size_t)par * world + rank) * ta.nh + head) * chunks + chunk;
            for (uint32_t r = 0; r < world; ++r) {
                float *dst = reinterpret_cast<float *>(bases[r] + flags_bytes) + my_slot * kP2PSlotFloats;
                dst[xt] = val;
                if (xt == 0) dst[kP2PChunk] = lse;
            }
            // the barrier orders the 64 threads' slot stores before the flag stores of threads 0..world-1, and a release
            // at system scope is cumulative over what happened before it
            bar64();
            if (xt < world) {
                st_release_sys(reinterpret_cast<uint32_t *>(peer_base) + my_slot, epoch);
                const uint32_t *flag = reinterpret_cast<const uint32_t *>(my_base) +
                                       (((size_t)par * world + xt) * ta.nh + head) * chunks + chunk;
                bool ok = false;
                for (uint32_t i = 0; i < ta.wait_peer; ++i) {
                    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) { ok = true; break; }
                    if ((i & 4095u) == 4095u && gave_up(ta.status)) break;   // somebody already gave up
                }
                if (!ok) {
                    sm_misc[1] = 1;
                    report_timeout(ta.status, 100 + (int)xt);
                }
            }
            bar64();
            if (!sm_misc[1]) {
                const float *mine = reinterpret_cast<const float *>(my_base + flags_bytes);
                auto slot_of = [&](uint32_t r) { return mine + ((((size_t)par * world + r) * ta.nh + head) * chunks + chunk) * kP2PSlotFloats; };
                // every rank's value is requested before any is used, and before the log-sum-exps are staged: the slots
                // were written by the peers over NVLink, so each first read goes out to memory, and one after the other
                // they took 3 us for 8 ranks
                float pv[kP2PMaxWorld];
#pragma unroll
                for (uint32_t r = 0; r < kP2PMaxWorld; ++r) pv[r] = (r < world && d < ta.hd) ? __ldcg(slot_of(r) + xt) : 0.f;
                if (xt < world) sm_lse[xt] = __ldcg(slot_of(xt) + kP2PChunk);
                bar64();
                if (d < ta.hd) {
                    float gmax = -INFINITY;
                    for (uint32_t r = 0; r < world; ++r)
                        if (sm_lse[r] > -INFINITY) gmax = fmaxf(gmax, sm_lse[r]);
                    float acc = 0.f, wsum = 0.f;
#pragma unroll
                    for (uint32_t r = 0; r < kP2PMaxWorld; ++r) {
                        const float l = r < world ? sm_lse[r] : -INFINITY;
                        if (!(l > -INFINITY)) continue;
                        const float w = expf(l - gmax);
                        acc += w * pv[r];
                        wsum += w;
                    }
                    float out = wsum > 0.f ? acc / wsum : 0.f;
                    const size_t oi = (size_t)head * ta.hd + d;
                    if (final_gate) out *= sigmoidf_ref(final_gate[oi]);
                    store_from_f32(final_out, oi, out_dt, out);
                }
            }
        }
        __syncthreads();   // scratch and sm_lse are rewritten by the next item
        if (sm_misc[1]) break;
    }
    if (tid == 0) grid_barrier_leave(ta);
}

// Resident CTAs per SM each configuration is built for (bounds the registers per thread).
constexpr int decode16_min_blocks(int HD, int NW, int STAGES) {
    return HD > 128 ? 1 : (NW == 4 ? (STAGES <= 6 ? 2 : 1) : 1);
}

// KPC kv heads per CTA: warp w streams kv head (w % KPC) of the CTA's rows, and the WPK = NW/KPC warps
// that share a kv head take alternate 16-position blocks.  With KPC == nkv a CTA reads whole cache rows.
// ILV (one sequence, merged by the grid): instead of walking a span of its own, warp g of the W warps that serve a
// kv head takes the sequence's 16-row blocks g, g + W, g + 2W, ...  Equal spans do not finish together — CTAs whose
// span lies in memory that is far from their SM stream several microseconds longer over a 40 us launch, and the grid
// barrier waits for the slowest — whereas interleaved every warp sees the same mix of memory and they end within a
// block of each other (long-context step 53.8 -> 51.7 us).  Taking the blocks from a shared atomic counter instead
// measured slower (59.9 us: the counter's answer is one more dependent memory round trip per block, and under load
// a round trip is a whole iteration).  Which rows a warp saw does not matter to the result: its (m, l, O) state is
// merged by log-sum-exp like any other.
// F8: the cache holds e4m3 bytes (T is __half: Q, P and the MMAs are f16).  Tiles are half as large, a 16-byte
// chunk is 16 head dims, and every byte has to be widened on its way to the tensor core — integer work that, not
// memory, bounds this path.  So the MMAs are turned round to waste as little as possible: the 16 positions of a
// block are the M rows and (up to) 8 query heads the N columns, S^T = K Q^T and O^T = V^T P^T; half the MMAs, half
// the accumulator registers and half the exponentials of the heads-on-M form when a KV group has 8 heads or fewer.
//   * ldmatrix moves 16-bit units, so a thread receives four consecutive dims of a K row where the f16 A fragment
//     has two: the Q columns are staged in the matching order (a dot product does not care in which order its
//     terms are added);
//   * P^T comes out of the softmax in the accumulator layout (position g, heads 2t, 2t+1) and goes into the next
//     MMA as a B fragment (positions 2t, 2t+1, head g): one movmatrix per eight positions;
//   * for V^T, ldmatrix.trans hands a thread the bytes (pos 2t, dims 2g, 2g+1) and (pos 2t+1, dims 2g, 2g+1): its
//     even bytes are the A fragment of dim 2g, its odd bytes that of dim 2g+1, so the M rows of an accumulator tile
//     are the even dims of a 16-dim chunk followed by its odd dims.
template <typename T, int HD, int NW, int STAGES, int KPC, bool ILV = false, int F8 = 0>
__global__ void __launch_bounds__(NW * 32, (F8 && HD <= 128) ? 3 : decode16_min_blocks(HD, NW, STAGES)) decode16_kernel(const __grid_constant__ DecodeArgs a) {
    using S = Decode16Smem<HD, NW, STAGES, KPC, F8>;
    constexpr int WPK = NW / KPC;
    static_assert(!F8 || (KPC == 1 && sizeof(T) == 2), "8-bit caches: one kv head per CTA, f16 arithmetic");
    static_assert(!ILV || KPC == 1, "the interleaved mode serves one kv head per CTA");
    // a tile is requested STAGES-1 tiles ahead of its use: the K-phase of iteration i requests a tile of block
    // i + kOffK, the V-phase one of block i + kOffV
    constexpr int kOffK = (STAGES - 1) / 2, kOffV = STAGES / 2;
    static_assert(NW % KPC == 0, "warps must divide evenly over the kv heads of a CTA");
    constexpr int CH = HD / 8;            // 16-byte chunks per 16-bit row (Q, and the projections of the fused append)
    constexpr int CHK = S::kRowBytes / 16;   // 16-byte chunks per K/V tile row
    constexpr bool QREG = HD <= 128;      // keep the Q fragments in registers (else re-read them from shared memory)
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *sm_q = smem;
    unsigned char *sm_pipe = smem + S::kQBytes;
    float *sm_m = reinterpret_cast<float *>(smem + S::kQBytes + NW * S::kWarpBytes);
    float *sm_l = sm_m + NW * 16;
    uint32_t *sm_item = reinterpret_cast<uint32_t *>(smem + S::kQBytes + NW * S::kWarpBytes + S::kStatBytes);  // 8 words

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // A launch in programmatic stream order (the host launcher) starts while the kernel before it drains: let the
    // next launch do the same with this one, and read nothing that kernel may have written before it has completed.
    // Both are no-ops in a plain launch.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // blockIdx.x = (work * KG + kg) * gz + z, KG = nkv / KPC groups of kv heads
    const uint32_t KG = a.nkv / KPC;
    const uint32_t zi = blockIdx.x % a.gz, kg = (blockIdx.x / a.gz) % KG;
    const uint32_t work = blockIdx.x / (a.gz * KG);
    Cursor cur{};
    if constexpr (!ILV) {
        if (warp == 0) cursor_init(a, work, lane, sm_item);
        __syncthreads();
        cur = Cursor{sm_item[0], sm_item[1], sm_item[2], sm_item[3], work, sm_item[4]};
        __syncthreads();  // sm_item[7] is reused as the merge flag below
    }
    const uint32_t kvl = warp % KPC, sub = warp / KPC;             // kv head within the CTA, block phase
    const uint32_t kvh = kg * KPC + kvl;
    constexpr uint32_t kRows = F8 ? 8u : 16u;                      // query heads a CTA serves (8-bit cache: the MMA's N columns)
    const uint32_t row0 = zi * kRows;                              // first head of the group handled here
    const uint32_t rows_valid = min(kRows, a.G - row0);

    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t mat = lane >> 3, rin = lane & 7;
    const uint32_t sm_q_addr = (uint32_t)__cvta_generic_to_shared(sm_q) + kvl * S::kQTile;
    const uint32_t warp_smem = (uint32_t)__cvta_generic_to_shared(sm_pipe + warp * S::kWarpBytes);
    const size_t pos_stride = (size_t)a.nkv * S::kRowBytes;
    // per-lane load geometry: a warp instruction copies 512 bytes = 512/kRowBytes rows
    constexpr int RPI = 512 / S::kRowBytes;          // rows per instruction (2 for hd128, 1 for hd256)
    constexpr int NI = kBlk / RPI;                   // instructions per tile
    const uint32_t l_row = lane / CHK * (RPI > 1), l_chunk = lane % CHK;

    Piece p;
    uint32_t pf_seq = 0xffffffffu;            // sequence whose cache pointers were requested ahead (pointer-array caches)
    const char *pf_k = nullptr, *pf_v = nullptr;
    bool ilv_todo = ILV;
    if constexpr (ILV) {   // the whole sequence is this CTA's piece; its record is number `work` of a.spans
        p.seq = 0; p.L = seq_len_at(a, 0); p.start = 0; p.end = p.L; p.nrec = a.spans; p.my_rec = work; p.c0 = 0; p.B = 0;
    }
    while (ILV ? ilv_todo : next_piece(a, cur, p)) {
        ilv_todo = false;
        const uint32_t start = p.start, end = p.end;
        // paged cache: kbase/vbase are the pools and every 16-row block takes its page number from the table; the
        // number of the warp's next block is fetched one block ahead so that its latency never meets a cp.async
        const uint32_t *ptab = a.kv.page_table ? a.kv.page_table + (size_t)p.seq * a.kv.max_pages : nullptr;
        // pointer-array caches: the sequence's two base pointers are a dependent load at the head of the piece; the next
        // sequence's are requested now, a whole piece ahead of their use
        const char *kseq, *vseq;
        if (!ptab && a.kv.k_ptrs && p.seq == pf_seq) { kseq = pf_k; vseq = pf_v; }
        else {
            kseq = ptab ? a.kv.k_base : kv_seq_ptr(a.kv.k_base, a.kv.k_ptrs, a.kv.seq_stride_bytes, p.seq);
            vseq = ptab ? a.kv.v_base : kv_seq_ptr(a.kv.v_base, a.kv.v_ptrs, a.kv.seq_stride_bytes, p.seq);
        }
        if (!ILV && !ptab && a.kv.k_ptrs && p.seq + 1 < a.num_seqs) {
            pf_seq = p.seq + 1;
            pf_k = reinterpret_cast<const char *>(__ldg(reinterpret_cast<const unsigned long long *>(a.kv.k_ptrs) + pf_seq));
            pf_v = reinterpret_cast<const char *>(__ldg(reinterpret_cast<const unsigned long long *>(a.kv.v_ptrs) + pf_seq));
        }
        const char *kbase = kseq + (size_t)kvh * S::kRowBytes;
        const char *vbase = vseq + (size_t)kvh * S::kRowBytes;
        const uint32_t nblk = (end - start + kBlk - 1) / kBlk;
        const uint32_t my_n = nblk > sub ? (nblk - sub + WPK - 1) / WPK : 0;
        // The pipeline moves single tiles: item 2i is the K tile of the warp's i-th block, item 2i+1 its V tile,
        // item t lives in slot t % STAGES, and STAGES-1 items are in flight while one is being consumed.
        constexpr int NIT = (2 * CH + 31) / 32;   // K and V chunks per lane
        const bool tail = !ILV && a.fuse_append && p.L > 0 && p.end == p.L;
        const bool owner = tail && ((nblk - 1) % WPK == sub) && KPC == 1;
        // interleaved mode: the warp's i-th block is block ilv_g + i * ilv_w of the sequence
        const uint32_t ilv_w = a.spans * NW, ilv_g = work * NW + warp;
        const uint32_t ilv_n = nblk > ilv_g ? (nblk - ilv_g + ilv_w - 1) / ilv_w : 0;
        uint4 newrow[NIT];
        // put the kept row into the tile that was just fetched (the copy in flight may predate the store above)
        auto patch_tile = [&](uint32_t tile_addr, uint32_t pos0, uint32_t want_v) {
            const uint32_t r = p.L - 1 - pos0;
#pragma unroll
            for (int it = 0; it < NIT; ++it) {
                const uint32_t tt = lane + 32 * it;
                if (tt < 2 * CH && tt / CH == want_v) {
                    const uint32_t c = tt % CH;
                    if constexpr (F8)   // eight bytes: half (c & 1) of the row's 16-byte chunk c / 2
                        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(tile_addr + r * S::kRowBytes + (((c >> 1) ^ (r & 7)) << 4) + (c & 1) * 8),
                                     "r"(newrow[it].x), "r"(newrow[it].y) : "memory");
                    else
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_addr + r * S::kRowBytes + ((c ^ (r & 7)) << 4)),
                                     "r"(newrow[it].x), "r"(newrow[it].y), "r"(newrow[it].z), "r"(newrow[it].w) : "memory");
                }
            }
            __syncwarp();
        };
        uint32_t pg_cur = 0, pg_nxt = 0;
        auto page_of_block = [&](uint32_t bi) {
            const uint32_t pos0 = start + (sub + bi * WPK) * kBlk;
            return pos0 < end ? ptab[pos0 / a.kv.page_rows] : 0u;
        };
        if (ptab) pg_nxt = page_of_block(0);
        // called with t = 0, 1, 2, ... in order: the K tile of a block, then its V tile; blk = the block's number in the piece
        auto issue = [&](uint32_t t, uint32_t blk) {
            const uint32_t pos0 = start + blk * kBlk;
            const uint32_t st = warp_smem + (t % STAGES) * S::kTileBytes;
            const char *src = (t & 1) ? vbase : kbase;
            uint32_t row0_src = pos0;     // row of the block's first position relative to src
            if (ptab) {
                if (!(t & 1)) { pg_cur = pg_nxt; pg_nxt = page_of_block((t >> 1) + 1); }
                src += (size_t)pg_cur * a.kv.page_bytes;
                row0_src = pos0 % a.kv.page_rows;
            }
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const uint32_t r = i * RPI + l_row;
                const bool ok = pos0 + r < end;
                const size_t goff = (size_t)(row0_src + r) * pos_stride + l_chunk * 16;
                const uint32_t soff = r * S::kRowBytes + ((l_chunk ^ (r & 7)) << 4);
                cp_async16(st + soff, src + (ok ? goff : 0), ok);
            }
        };
        // ---- fused append: the projected rows of this piece are requested before the K/V stream.  Behind the burst of
        //      tile copies they waited two microseconds in the memory queues, and nothing can be computed without Q ----
        constexpr int QIT = (KPC * 16 * CH + NW * 32 - 1) / (NW * 32);
        uint4 q_req[QIT][2], own_req[NIT][2];
        if (a.fuse_append) {
#pragma unroll
            for (int qi = 0; qi < QIT; ++qi) {
                const uint32_t idx = tid + qi * NW * 32;
                const uint32_t c = idx % CH, r = (idx / CH) % 16, k = idx / (CH * 16);
                q_req[qi][0] = q_req[qi][1] = make_uint4(0, 0, 0, 0);
                if (idx < KPC * 16 * CH && r < rows_valid) {
                    const size_t e0 = ((size_t)p.seq * a.nh + (kg * KPC + k) * a.G + row0 + r) * (a.ap_has_gate ? 2 * HD : HD) + c * 8;
                    load8_raw(a.ap_q, e0, a.ap_in_dtype, q_req[qi]);
                }
            }
            if (owner) {
#pragma unroll
                for (int it = 0; it < NIT; ++it) {
                    const uint32_t tt = lane + 32 * it;
                    const uint32_t is_v = tt < 2 * CH ? tt / CH : 1u, c = tt % CH;
                    load8_raw(is_v ? a.ap_v : a.ap_k, ((size_t)p.seq * a.nkv + kvh) * HD + c * 8, a.ap_in_dtype, own_req[it]);
                }
            }
        }
        // ---- start the K/V stream, the rest of the prologue runs underneath it ----
        // block number (within the piece) of the warp's i-th block, and how many it has
        auto block_of = [&](uint32_t i) { return ILV ? ilv_g + i * ilv_w : sub + i * WPK; };
        const uint32_t w_n = ILV ? ilv_n : my_n, w_items = 2 * w_n;
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if ((uint32_t)s < w_items) issue(s, block_of(s >> 1));
            cp_async_commit();
        }
        // ---- fused append: the warp that will process the block holding row L-1 builds that row of K (norm + RoPE)
        //      and of V, stores both in the cache for later steps and keeps them to patch its shared-memory tiles.
        //      Here it only requests the projected rows; the arithmetic follows once Q is staged, so the latency of
        //      these loads passes under the staging and the cos/sin table built for Q serves K as well ----
        float own_raw[NIT][8];
        if (owner) {
#pragma unroll
            for (int it = 0; it < NIT; ++it) {
                const uint32_t tt = lane + 32 * it;
                const uint32_t is_v = tt < 2 * CH ? tt / CH : 1u, c = tt % CH;
                (void)is_v; (void)c;
                cvt8_raw(own_req[it], a.ap_in_dtype, own_raw[it]);
            }
        }
        // stage Q of the CTA's kv heads (rows >= rows_valid are zero) as T, swizzled
        auto store_q_chunk = [&](uint32_t k, uint32_t r, uint32_t c, const uint4 &v) {
            if constexpr (F8) {
                // dims 8c .. 8c+7 of the 16-dim group c/2: the pair (4u, 4u+1) goes to column 2u, the pair (4u+2, 4u+3)
                // to column 8 + 2u of the group (u = 2*(c&1), 2*(c&1)+1): two 8-byte halves in the group's two chunks
                const uint32_t u2 = (c & 1) * 2, grp = c >> 1;
                unsigned char *rowp = sm_q + k * S::kQTile + r * S::kQRowBytes;
                *reinterpret_cast<uint2 *>(rowp + (((2 * grp) ^ (r & 7)) << 4) + u2 * 4) = make_uint2(v.x, v.z);
                *reinterpret_cast<uint2 *>(rowp + (((2 * grp + 1) ^ (r & 7)) << 4) + u2 * 4) = make_uint2(v.y, v.w);
            } else {
                *reinterpret_cast<uint4 *>(sm_q + k * S::kQTile + r * S::kQRowBytes + ((c ^ (r & 7)) << 4)) = v;
            }
        };
        if (a.fuse_append) {
            // raw Q row -> RMSNorm(1+w) -> RoPE at position L-1 (wgsl:126-166); CH consecutive threads share a row.
            // cos/sin of the rotary pairs are the same for all rows: one table per piece in the merge-statistics area
            float qraw[QIT][8];
#pragma unroll
            for (int qi = 0; qi < QIT; ++qi) cvt8_raw(q_req[qi], a.ap_in_dtype, qraw[qi]);
            const uint32_t pos = p.L ? p.L - 1 : 0;
            float2 *sm_cs = reinterpret_cast<float2 *>(sm_m);   // HD/2 pairs; sm_m/sm_l are free until the piece ends
            for (uint32_t i2 = tid; i2 < HD / 2; i2 += NW * 32) {
                float sn = 0.f, cs = 1.f;
                if (i2 < a.ap_rd / 2) sincosf((float)pos * a.ap_inv_freq[i2], &sn, &cs);
                sm_cs[i2] = make_float2(cs, sn);
            }
            __syncthreads();
#pragma unroll
            for (int qi = 0; qi < QIT; ++qi) {
                const uint32_t idx = tid + qi * NW * 32;
                if (idx >= KPC * 16 * CH) break;
                const uint32_t c = idx % CH, r = (idx / CH) % 16, k = idx / (CH * 16);
                float (&v8)[8] = qraw[qi];
                if (a.ap_norm_w) {
                    float ssq = 0.f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) ssq += v8[e] * v8[e];
#pragma unroll
                    for (int o = CH / 2; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o, CH);
                    const float rms = 1.0f / sqrtf(ssq / (float)HD + a.ap_eps);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v8[e] = v8[e] * rms * (1.0f + __uint_as_float(((uint32_t)a.ap_norm_w[c * 8 + e]) << 16));
                }
#pragma unroll
                for (int k2 = 0; k2 < 4; ++k2) {
                    const float2 t2 = sm_cs[c * 4 + k2];   // (1, 0) beyond the rotary dims
                    const float x = v8[2 * k2], y = v8[2 * k2 + 1];
                    v8[2 * k2] = x * t2.x - y * t2.y;
                    v8[2 * k2 + 1] = y * t2.x + x * t2.y;
                }
                uint4 v;
                v.x = pack2<T>(v8[0], v8[1]); v.y = pack2<T>(v8[2], v8[3]); v.z = pack2<T>(v8[4], v8[5]); v.w = pack2<T>(v8[6], v8[7]);
                store_q_chunk(k, r, c, v);
            }
        } else
        for (uint32_t idx = tid; idx < KPC * 16 * CH; idx += NW * 32) {
            const uint32_t c = idx % CH, r = (idx / CH) % 16, k = idx / (CH * 16);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < rows_valid) {
                const size_t e0 = ((size_t)p.seq * a.nh + (kg * KPC + k) * a.G + row0 + r) * HD + c * 8;
                if (a.q_dtype == SHADY_F32) {
                    const float4 f0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(a.q) + e0);
                    const float4 f1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(a.q) + e0 + 4);
                    v.x = pack2<T>(f0.x, f0.y); v.y = pack2<T>(f0.z, f0.w);
                    v.z = pack2<T>(f1.x, f1.y); v.w = pack2<T>(f1.z, f1.w);
                } else {
                    v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.q) + e0);
                }
            }
            store_q_chunk(k, r, c, v);
        }
        __syncthreads();
        if (owner) {   // (fused append, second half) norm + RoPE of the new K row, V as it is; cache stores; kept for the patch
            const uint32_t pos = p.L - 1;
            const float2 *sm_cs = reinterpret_cast<const float2 *>(sm_m);   // this piece's table: (cos, sin) per pair, (1, 0) past rd
#pragma unroll
            for (int it = 0; it < NIT; ++it) {
                const uint32_t tt = lane + 32 * it;
                const bool act = tt < 2 * CH;
                const uint32_t is_v = act ? tt / CH : 1u, c = tt % CH;
                float (&v8)[8] = own_raw[it];
                if (a.ap_norm_w && it == 0) {   // K chunks sit in item set 0 (all lanes, or the first CH of them)
                    float ssq = 0.f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) ssq += v8[e] * v8[e];
#pragma unroll
                    for (int o = CH / 2; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o, CH);
                    if (!is_v) {
                        const float rms = 1.0f / sqrtf(ssq / (float)HD + a.ap_eps);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            v8[e] = v8[e] * rms * (1.0f + __uint_as_float(((uint32_t)a.ap_norm_w[HD + c * 8 + e]) << 16));
                    }
                }
                if (!is_v) {
#pragma unroll
                    for (int k2 = 0; k2 < 4; ++k2) {
                        const float2 t2 = sm_cs[c * 4 + k2];
                        const float x = v8[2 * k2], y = v8[2 * k2 + 1];
                        v8[2 * k2] = x * t2.x - y * t2.y;
                        v8[2 * k2 + 1] = y * t2.x + x * t2.y;
                    }
                }
                char *dst = act ? const_cast<char *>(kv_row_ptr(a.kv, is_v != 0, p.seq, pos, pos_stride)) + (size_t)kvh * S::kRowBytes : nullptr;
                if constexpr (F8) {   // stored = value / scale, rounded as the stand-alone append rounds it
                    const float inv = 1.0f / (is_v ? a.kv.v_scale : a.kv.k_scale);
                    uint32_t lo = 0, hi = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        lo |= (uint32_t)f32_to_f8<F8>(v8[e] * inv) << (8 * e);
                        hi |= (uint32_t)f32_to_f8<F8>(v8[4 + e] * inv) << (8 * e);
                    }
                    newrow[it] = make_uint4(lo, hi, 0u, 0u);
                    if (act) *reinterpret_cast<uint2 *>(dst + c * 8) = make_uint2(newrow[it].x, newrow[it].y);
                } else {
                    newrow[it].x = pack2<T>(v8[0], v8[1]); newrow[it].y = pack2<T>(v8[2], v8[3]);
                    newrow[it].z = pack2<T>(v8[4], v8[5]); newrow[it].w = pack2<T>(v8[6], v8[7]);
                    if (act) *reinterpret_cast<uint4 *>(dst + c * 16) = newrow[it];
                }
            }
        }
        float *sm_o = reinterpret_cast<float *>(sm_pipe);  // warp w's [16][HD] tile at w*kWarpBytes
        if constexpr (F8) {
            // ---- 8-bit cache: positions on the M rows, heads on the N columns (S^T = K Q^T, O^T = V^T P^T) ----
            // Q^T fragments (B operand): per 16-dim k-step the (permuted) columns 0-7 and 8-15 of heads 0-7
            uint32_t qb[HD / 16][2];
#pragma unroll
            for (int c = 0; c < HD / 16; c += 2) {
                uint32_t r4[4];   // (heads 0-7, chunk 2c), (.., 2c+1), (.., 2c+2), (.., 2c+3) of the 16-bit Q rows
                ldsm_x4(r4, sm_q_addr + rin * S::kQRowBytes + (((2 * c + mat) ^ rin) << 4));
                qb[c][0] = r4[0]; qb[c][1] = r4[1]; qb[c + 1][0] = r4[2]; qb[c + 1][1] = r4[3];
            }
            float oT[HD / 16][4];   // tile c: (dim 16c+2g, heads 2t, 2t+1), (dim 16c+2g+1, heads 2t, 2t+1)
#pragma unroll
            for (int c = 0; c < HD / 16; ++c) oT[c][0] = oT[c][1] = oT[c][2] = oT[c][3] = 0.f;
            float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // heads 2t, 2t+1 (l: this lane's positions only)

            for (uint32_t i = 0; i < w_n; ++i) {
                cp_async_wait<STAGES - 2>();   // this block's K tile has landed
                __syncwarp();
                if (2 * i + STAGES - 1 < w_items) issue(2 * i + STAGES - 1, block_of(i + kOffK));
                cp_async_commit();
                const uint32_t st = warp_smem + ((2 * i) % STAGES) * S::kTileBytes;
                const uint32_t pos0 = start + block_of(i) * kBlk;
                if (owner && i == w_n - 1) patch_tile(st, pos0, 0u);
                // ---- S^T = K Q^T : 16 positions x 8 heads ----
                float sT[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < HD / 16; c += 2) {
                    uint32_t kb[4];   // (pos 0-7, chunk c), (pos 8-15, chunk c), (pos 0-7, chunk c+1), (pos 8-15, chunk c+1)
                    ldsm_x4(kb, st + ((mat & 1) * 8 + rin) * S::kRowBytes + (((c + (mat >> 1)) ^ rin) << 4));
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // a register holds dims 4t..4t+3 of its row: the low pair is k = 2t, 2t+1, the high pair k = 2t+8, 2t+9
                        const uint32_t ka[4] = {f8x2_to_f16x2<F8, 0x10>(kb[2 * h]), f8x2_to_f16x2<F8, 0x10>(kb[2 * h + 1]),
                                                f8x2_to_f16x2<F8, 0x32>(kb[2 * h]), f8x2_to_f16x2<F8, 0x32>(kb[2 * h + 1])};
                        mma16816<T>(sT, ka, qb[c + h][0], qb[c + h][1]);
                    }
                }
                // ---- online softmax (log2 domain): this lane holds positions g, g+8 of heads 2t, 2t+1 ----
                const bool v0 = pos0 + g < end, v1 = pos0 + g + 8 < end;
                float x[4];
                x[0] = v0 ? sT[0] * a.scale_log2 : -INFINITY; x[1] = v0 ? sT[1] * a.scale_log2 : -INFINITY;
                x[2] = v1 ? sT[2] * a.scale_log2 : -INFINITY; x[3] = v1 ? sT[3] * a.scale_log2 : -INFINITY;
                float mx[2] = {fmaxf(x[0], x[2]), fmaxf(x[1], x[3])}, corr[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 4));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 8));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
                    const float m_new = fmaxf(m_run[r], mx[r]);   // finite: every block holds >= 1 valid position
                    corr[r] = exp2f(m_run[r] - m_new);
                    m_run[r] = m_new;
                }
                const float p0 = exp2f(x[0] - m_run[0]), p1 = exp2f(x[1] - m_run[1]);
                const float p2 = exp2f(x[2] - m_run[0]), p3 = exp2f(x[3] - m_run[1]);
                l_run[0] = l_run[0] * corr[0] + (p0 + p2);
                l_run[1] = l_run[1] * corr[1] + (p1 + p3);
                // P^T as the B operand: (pos g; heads 2t, 2t+1) -> (pos 2t, 2t+1; head g), positions 0-7 and 8-15
                const uint32_t pb0 = movmatrix_trans(pack2<T>(p0, p1)), pb1 = movmatrix_trans(pack2<T>(p2, p3));
                const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f);
                // ---- O^T = O^T * corr + V^T P^T ----
                cp_async_wait<STAGES - 2>();   // this block's V tile has landed
                __syncwarp();
                if (2 * i + STAGES < w_items) issue(2 * i + STAGES, block_of(i + kOffV));   // into the slot of the K tile just consumed
                cp_async_commit();
                const uint32_t stv = warp_smem + ((2 * i + 1) % STAGES) * S::kTileBytes;
                if (owner && i == w_n - 1) patch_tile(stv, pos0, 1u);
#pragma unroll
                for (int c = 0; c < HD / 16; c += 2) {
                    uint32_t vb[4];   // (pos 0-7, chunk c), (pos 8-15, chunk c), (pos 0-7, chunk c+1), (pos 8-15, chunk c+1)
                    ldsm_x4_t(vb, stv + ((mat & 1) * 8 + rin) * S::kRowBytes + (((c + (mat >> 1)) ^ rin) << 4));
                    if (rescale) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            oT[c + h][0] *= corr[0]; oT[c + h][1] *= corr[1];
                            oT[c + h][2] *= corr[0]; oT[c + h][3] *= corr[1];
                        }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // a register holds (pos 2t, dim 2g), (pos 2t, dim 2g+1), (pos 2t+1, dim 2g), (pos 2t+1, dim 2g+1):
                        // rows 0-7 of the tile are the even dims, rows 8-15 the odd dims
                        const uint32_t va[4] = {f8x2_to_f16x2<F8, 0x20>(vb[2 * h]), f8x2_to_f16x2<F8, 0x31>(vb[2 * h]),
                                                f8x2_to_f16x2<F8, 0x20>(vb[2 * h + 1]), f8x2_to_f16x2<F8, 0x31>(vb[2 * h + 1])};
                        mma16816<T>(oT[c + h], va, pb0, pb1);
                    }
                }
            }
            cp_async_wait<0>();
            __syncthreads();  // every warp is done with its pipeline memory: reuse it for the merge

            // ---- per-warp state -> shared: rows are heads, as the 16-bit path writes them ----
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 4);
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 8);
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 16);
            }
            float *my_o = reinterpret_cast<float *>(sm_pipe + warp * S::kWarpBytes);
            if (g == 0) {
                sm_m[warp * 16 + 2 * t] = m_run[0]; sm_m[warp * 16 + 2 * t + 1] = m_run[1];
                sm_l[warp * 16 + 2 * t] = l_run[0]; sm_l[warp * 16 + 2 * t + 1] = l_run[1];
            }
            // the cache scale of V and the 2^8 the byte-to-f16 conversion leaves out are applied here, once per element of O
            const float vs = a.kv.v_scale * f8_unscale(F8);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const uint32_t head = 2 * t + hh;
                if (head < rows_valid) {
#pragma unroll
                    for (int c = 0; c < HD / 16; ++c)
                        *reinterpret_cast<float2 *>(my_o + head * S::kORow + c * 16 + 2 * g) = make_float2(oT[c][hh] * vs, oT[c][2 + hh] * vs);
                }
            }
        } else {
            // Q fragments (A operand), one ldmatrix.x4 per k-step: mats = (rows0-7,c), (rows8-15,c), (rows0-7,c+1), (rows8-15,c+1)
            uint32_t qa[QREG ? HD / 16 : 1][4];
            if constexpr (QREG) {
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t row = (mat & 1) * 8 + rin, chunk = 2 * ks + (mat >> 1);
                    ldsm_x4(qa[ks], sm_q_addr + row * S::kQRowBytes + ((chunk ^ rin) << 4));
                }
            }

            float o[HD / 8][4];
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
            float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

            for (uint32_t i = 0; i < w_n; ++i) {
                cp_async_wait<STAGES - 2>();   // this block's K tile has landed
                __syncwarp();
                if (2 * i + STAGES - 1 < w_items) issue(2 * i + STAGES - 1, block_of(i + kOffK));
                cp_async_commit();

                const uint32_t st = warp_smem + ((2 * i) % STAGES) * S::kTileBytes;
                const uint32_t pos0 = start + block_of(i) * kBlk;
                if (owner && i == w_n - 1) patch_tile(st, pos0, 0u);
                // ---- S = Q K^T : heads x 16 positions ----
                float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                #pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    uint32_t kb[4];
                    const uint32_t row = (mat >> 1) * 8 + rin, chunk = 2 * ks + (mat & 1);
                    ldsm_x4(kb, st + row * S::kRowBytes + ((chunk ^ rin) << 4));
                    if constexpr (QREG) {
                        mma16816<T>(s[0], qa[ks], kb[0], kb[1]);
                        mma16816<T>(s[1], qa[ks], kb[2], kb[3]);
                    } else {
                        const uint32_t qrow = (mat & 1) * 8 + rin, qchunk = 2 * ks + (mat >> 1);
                        ldsm_x4(qa[0], sm_q_addr + qrow * S::kQRowBytes + ((qchunk ^ rin) << 4));
                        mma16816<T>(s[0], qa[0], kb[0], kb[1]);
                        mma16816<T>(s[1], qa[0], kb[2], kb[3]);
                    }
                }
            
                // ---- online softmax (log2 domain), rows g and g+8 ----
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t pos = pos0 + 8 * j + 2 * t + (c & 1);
                        s[j][c] = pos < end ? s[j][c] * a.scale_log2 : -INFINITY;
                        mx[c >> 1] = fmaxf(mx[c >> 1], s[j][c]);
                    }
                float corr[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    const float m_new = fmaxf(m_run[r], mx[r]);   // finite: every block holds >= 1 valid position
                    corr[r] = exp2f(m_run[r] - m_new);
                    m_run[r] = m_new;
                }
                float psum[2] = {0.f, 0.f};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        s[j][c] = exp2f(s[j][c] - m_run[c >> 1]);
                        psum[c >> 1] += s[j][c];
                    }
                l_run[0] = l_run[0] * corr[0] + psum[0];
                l_run[1] = l_run[1] * corr[1] + psum[1];
                // O is rescaled only when some row's maximum grew in this block (after the first few blocks of a piece that
                // is rare): HD/2 multiplies per lane saved in the common case
                const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f);
                uint32_t pa[4];
                pa[0] = pack2<T>(s[0][0], s[0][1]);
                pa[1] = pack2<T>(s[0][2], s[0][3]);
                pa[2] = pack2<T>(s[1][0], s[1][1]);
                pa[3] = pack2<T>(s[1][2], s[1][3]);
                // ---- O = O*corr + P V ----
                cp_async_wait<STAGES - 2>();   // this block's V tile has landed
                __syncwarp();
                if (2 * i + STAGES < w_items) issue(2 * i + STAGES, block_of(i + kOffV));   // into the slot of the K tile just consumed
                cp_async_commit();
                const uint32_t stv = warp_smem + ((2 * i + 1) % STAGES) * S::kTileBytes;
                if (owner && i == w_n - 1) patch_tile(stv, pos0, 1u);
                #pragma unroll
                for (int jn = 0; jn < HD / 8; jn += 2) {
                    uint32_t vb[4];
                    const uint32_t row = (mat & 1) * 8 + rin, chunk = jn + (mat >> 1);
                    ldsm_x4_t(vb, stv + row * S::kRowBytes + ((chunk ^ rin) << 4));
                    if (rescale) {
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            o[jn + u][0] *= corr[0]; o[jn + u][1] *= corr[0];
                            o[jn + u][2] *= corr[1]; o[jn + u][3] *= corr[1];
                        }
                    }
                    mma16816<T>(o[jn], pa, vb[0], vb[1]);
                    mma16816<T>(o[jn + 1], pa, vb[2], vb[3]);
                }
            
            }
            cp_async_wait<0>();
            __syncthreads();  // every warp is done with its pipeline memory: reuse it for the merge

            // ---- per-warp state -> shared ----
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
            }
            float *my_o = reinterpret_cast<float *>(sm_pipe + warp * S::kWarpBytes);
            if (t == 0) {
                sm_m[warp * 16 + g] = m_run[0];
                sm_m[warp * 16 + g + 8] = m_run[1];
                sm_l[warp * 16 + g] = l_run[0];
                sm_l[warp * 16 + g + 8] = l_run[1];
            }
                    if (g < rows_valid) {          // only the head rows that exist go to shared memory
#pragma unroll
                for (int jn = 0; jn < HD / 8; ++jn)
                    *reinterpret_cast<float2 *>(my_o + g * S::kORow + jn * 8 + 2 * t) = make_float2(o[jn][0], o[jn][1]);
            }
            if (g + 8 < rows_valid) {
#pragma unroll
                for (int jn = 0; jn < HD / 8; ++jn)
                    *reinterpret_cast<float2 *>(my_o + (g + 8) * S::kORow + jn * 8 + 2 * t) = make_float2(o[jn][2], o[jn][3]);
            }
        
        }
        __syncthreads();
        // after its first loop finish_piece no longer reads the O tiles: the pipeline memory doubles as merge scratch
        finish_piece<16, HD, NW, S::kWarpBytes / 4, KPC, S::kORow>(a, p, sm_m, sm_l, sm_o, sm_item + 7,
                                                         reinterpret_cast<uint32_t *>(sm_pipe), NW * S::kWarpBytes / 4,
                                                         kg * KPC, row0, rows_valid, (p.seq * KG + kg) * a.gz + zi);
        __syncthreads();  // the next piece overwrites Q and the pipeline memory
    }
    if (a.grid_merge) {
        if (a.px_world) grid_exchange_tail<NW>(a, tail_args(a), reinterpret_cast<uint32_t *>(sm_pipe));
        else grid_merge_tail<NW>(a, tail_args(a), reinterpret_cast<uint32_t *>(sm_pipe));
    }
}

// ---------------------------------------------------------------------------------------
// fp32 cache path (the reference's own cache format)
// ---------------------------------------------------------------------------------------
template <int HD, int GT, int NW>
__global__ void __launch_bounds__(NW * 32) decode32_kernel(const DecodeArgs a) {
    constexpr int EPL = HD / 32;                 // elements per lane
    constexpr int VEC = EPL >= 4 ? 4 : EPL;      // floats per vector load
    constexpr int NV = EPL / VEC;
    constexpr int U = 4;                         // positions in flight per warp
    __shared__ float sm_m[NW * GT], sm_l[NW * GT];
    __shared__ float sm_o[NW * GT * HD];
    __shared__ uint32_t sm_item[8];
    constexpr uint32_t kScratchWords = 3072;   // merge scratch: >= 2*spans + 2*GT for any balanced launch
    __shared__ __align__(16) uint32_t sm_scratch[kScratchWords];   // finish_piece keeps 64-bit row addresses at its head

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t zi = blockIdx.x % a.gz, kvh = (blockIdx.x / a.gz) % a.nkv;
    const uint32_t work = blockIdx.x / (a.gz * a.nkv);
    if (warp == 0) cursor_init(a, work, lane, sm_item);
    __syncthreads();
    Cursor cur{sm_item[0], sm_item[1], sm_item[2], sm_item[3], work, sm_item[4]};
    __syncthreads();
    const uint32_t row0 = zi * GT;
    const uint32_t rows_valid = min((uint32_t)GT, a.G - row0);
    const uint32_t head0 = kvh * a.G + row0;
    const size_t pos_stride = (size_t)a.nkv * HD;

    Piece p;
    while (next_piece(a, cur, p)) {
        const uint32_t start = p.start, end = p.end;
        // lane owns dims (i*32 + lane)*VEC + e
        float q[GT][EPL];
#pragma unroll
        for (int h = 0; h < GT; ++h)
#pragma unroll
            for (int i = 0; i < NV; ++i)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const uint32_t d = (i * 32 + lane) * VEC + e;
                    q[h][i * VEC + e] = (uint32_t)h < rows_valid
                                            ? load_as_f32(a.q, ((size_t)p.seq * a.nh + head0 + h) * HD + d, a.q_dtype) * a.scale_log2
                                            : 0.f;
                }
        float acc[GT][EPL];
        float m_run[GT], l_run[GT];
#pragma unroll
        for (int h = 0; h < GT; ++h) {
            m_run[h] = -INFINITY;
            l_run[h] = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[h][e] = 0.f;
        }
        const float *kbase = reinterpret_cast<const float *>(kv_seq_ptr(a.kv.k_base, a.kv.k_ptrs, a.kv.seq_stride_bytes, p.seq)) + (size_t)kvh * HD;
        const float *vbase = reinterpret_cast<const float *>(kv_seq_ptr(a.kv.v_base, a.kv.v_ptrs, a.kv.seq_stride_bytes, p.seq)) + (size_t)kvh * HD;

        for (uint32_t p0 = start + warp * U; p0 < end; p0 += NW * U) {
            float kr[U][EPL], vr[U][EPL];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t pos = min(p0 + u, end - 1);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const size_t off = (size_t)pos * pos_stride + (i * 32 + lane) * VEC;
                    if constexpr (VEC == 4) {
                        const float4 kk = __ldcs(reinterpret_cast<const float4 *>(kbase + off));
                        const float4 vv = __ldcs(reinterpret_cast<const float4 *>(vbase + off));
                        kr[u][i * 4 + 0] = kk.x; kr[u][i * 4 + 1] = kk.y; kr[u][i * 4 + 2] = kk.z; kr[u][i * 4 + 3] = kk.w;
                        vr[u][i * 4 + 0] = vv.x; vr[u][i * 4 + 1] = vv.y; vr[u][i * 4 + 2] = vv.z; vr[u][i * 4 + 3] = vv.w;
                    } else {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            kr[u][i * VEC + e] = __ldcs(kbase + off + e);
                            vr[u][i * VEC + e] = __ldcs(vbase + off + e);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (p0 + u >= end) break;
#pragma unroll
                for (int h = 0; h < GT; ++h) {
                    float dot = 0.f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) dot = fmaf(q[h][e], kr[u][e], dot);
                    dot = warp_sum(dot);  // already in log2 units (q carries scale*log2e)
                    const float m_new = fmaxf(m_run[h], dot);
                    const float corr = exp2f(m_run[h] - m_new);
                    const float pr = exp2f(dot - m_new);
                    l_run[h] = l_run[h] * corr + pr;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) acc[h][e] = fmaf(pr, vr[u][e], acc[h][e] * corr);
                    m_run[h] = m_new;
                }
            }
        }
        // ---- merge the warps ----
#pragma unroll
        for (int h = 0; h < GT; ++h) {
            if (lane == 0) {
                sm_m[warp * GT + h] = m_run[h];
                sm_l[warp * GT + h] = l_run[h];
            }
#pragma unroll
            for (int i = 0; i < NV; ++i)
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                    sm_o[((size_t)warp * GT + h) * HD + (i * 32 + lane) * VEC + e] = acc[h][i * VEC + e];
        }
        __syncthreads();
        finish_piece<GT, HD, NW, GT * HD, 1>(a, p, sm_m, sm_l, sm_o, sm_item + 7, sm_scratch, kScratchWords, kvh, row0,
                                             rows_valid, (p.seq * a.nkv + kvh) * a.gz + zi);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// Merge of balanced-mode records as its own launch.  A sequence that is cut into many spans (one long
// context spread over every SM) would leave its whole merge to the single CTA that arrives last — a
// serial tail of L2 round trips; here every (sequence, head, 64-dim chunk) gets its own CTA instead.
// ---------------------------------------------------------------------------------------
constexpr uint32_t kMergeGroups = 4;                       // record subsets merged side by side by one CTA
constexpr uint32_t kMergeThreads = kMergeGroups * 64;

// Merged value of element d (= 64*chunk + threadIdx.x % 64) of `head` of sequence seq and the head's log-sum-exp, from
// the balanced-mode records.  Called by all kMergeThreads threads of a CTA: group g = threadIdx.x / 64 accumulates the
// records s = g, g + 4, ... (the loop is a chain of L2 round trips, so four short chains beat one long one) and the
// groups are summed through shared memory; every thread returns the result.  `single` tells that the sequence has one
// record only, which its CTA wrote directly to a.out / a.lse.
__device__ __forceinline__ void merge_balanced_records(const DecodeArgs &a, uint32_t seq, uint32_t head, uint32_t d,
                                                       float &val, float &lse, bool &single) {
    __shared__ uint32_t sm_b;
    const uint32_t tid = threadIdx.x, g = tid >> 6, t = tid & 63u;
    if (tid < 32) {   // first row-block of this sequence on the line
        uint32_t acc = 0;
        for (uint32_t j = tid; j < seq; j += 32) acc += blocks_of(seq_len_at(a, j)) + a.pad;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (tid == 0) sm_b = acc;
    }
    __syncthreads();
    const uint32_t B = sm_b, nb = blocks_of(seq_len_at(a, seq));
    const uint32_t c0 = span_of(a, B), nrec = span_of(a, B + nb - 1) - c0 + 1;
    const uint32_t dd = min(d, a.hd - 1);
    single = nrec == 1;       // uniform for the CTA
    if (single) {
        const float *row = reinterpret_cast<const float *>(a.out) + ((size_t)seq * a.nh + head) * a.out_row_stride;
        val = __ldcg(row + dd);
        lse = a.lse ? __ldcg(a.lse + ((size_t)seq * a.nh + head) * a.lse_stride) : 0.f;
        return;
    }
    const uint32_t rs = a.hd + 2;
    // record rows of this sequence, resolved once per CTA (span_begin is a 64-bit division)
    __shared__ uint32_t sm_row[kMaxSlots];
    __shared__ float sm_w[kMaxSlots];
    __shared__ float sm_acc[kMergeGroups][64];
    __shared__ float sm_ws[kMergeGroups];
    for (uint32_t s = tid; s < nrec; s += kMergeThreads) {
        const uint32_t c = c0 + s;
        sm_row[s] = (c * 2 + (span_begin(a, c) >= B ? 0u : 1u)) * a.nh + head;
        sm_w[s] = __ldcg(a.partials + (size_t)sm_row[s] * rs + a.hd);   // lse of record s
    }
    __syncthreads();
    float gmax = -INFINITY;
    for (uint32_t s = 0; s < nrec; ++s)
        if (sm_w[s] > -INFINITY) gmax = fmaxf(gmax, sm_w[s]);
    float acc = 0.f, wsum = 0.f;
#pragma unroll 8
    for (uint32_t s = g; s < nrec; s += kMergeGroups) {
        const float v = __ldcg(a.partials + (size_t)sm_row[s] * rs + dd);
        const float l = sm_w[s];
        const float w = l > -INFINITY ? expf(l - gmax) : 0.f;   // gqa_reduce.wgsl:56; empty ranges weigh nothing
        acc += w > 0.f ? w * v : 0.f;
        wsum += w;
    }
    sm_acc[g][t] = acc;
    if (t == 0) sm_ws[g] = wsum;
    __syncthreads();
    acc = 0.f; wsum = 0.f;
#pragma unroll
    for (uint32_t k = 0; k < kMergeGroups; ++k) { acc += sm_acc[k][t]; wsum += sm_ws[k]; }
    val = wsum > 0.f ? acc / wsum : 0.f;
    lse = wsum > 0.f ? gmax + logf(wsum) : -INFINITY;
}

__global__ void __launch_bounds__(kMergeThreads) balanced_merge_kernel(const DecodeArgs a) {
    const uint32_t seq = blockIdx.x, head = blockIdx.y, d = blockIdx.z * 64 + (threadIdx.x & 63u);
    float val, lse;
    bool single;
    merge_balanced_records(a, seq, head, d, val, lse, single);
    if (single || threadIdx.x >= 64 || d >= a.hd) return;   // a single record is already in place
    if (has_gate(a)) val *= sigmoidf_ref(gate_value(a, seq, head, d));
    store_from_f32(a.out, ((size_t)seq * a.nh + head) * a.out_row_stride + d, a.out_dtype, val);
    if (d == 0 && a.lse) a.lse[((size_t)seq * a.nh + head) * a.lse_stride] = lse;
}

// Merge of this rank's records, exchange with the peers and merge across ranks in ONE launch: one CTA per
// (query head, 64-dim chunk) of the single row-sharded sequence.  The CTA
//   1. merges its slice of the rank's records (as balanced_merge_kernel does),
//   2. stores the slice and the head's log-sum-exp into its slot of every rank's exchange buffer with plain peer
//      stores (no TMA, no multicast), fences at system scope and raises its flag on every rank,
//   3. waits — bounded — for the same flag of every rank in its own buffer,
//   4. merges the `world` slices (gqa_reduce.wgsl:33-64; empty shards weigh nothing) and writes the final values.
// Slots and flags are double-buffered by the parity of the epoch, as in p2p_combine_kernel.
__global__ void __launch_bounds__(kMergeThreads) shard_merge_p2p_kernel(const DecodeArgs a) {
    const uint32_t head = blockIdx.y, chunk = blockIdx.z, chunks = gridDim.z, tid = threadIdx.x;
    const uint32_t d = chunk * kP2PChunk + (tid & 63u);
    float val, lse;
    bool single;
    merge_balanced_records(a, 0, head, d, val, lse, single);
    if (tid >= 64) return;    // the exchange is the first 64 threads' job: from here on they meet at a 64-thread named barrier
    auto bar64 = [] { asm volatile("bar.sync 1, 64;" ::: "memory"); };
    __shared__ float sm_lse[kP2PMaxWorld];
    __shared__ int sm_fail;
    if (tid == 0) sm_fail = 0;
    const uint32_t world = a.px_world, par = a.px_epoch & 1u;
    const unsigned long long flags_bytes = p2p_chunk_flags_bytes(world, a.nh, a.hd);
    const size_t my_slot = (((size_t)par * world + a.px_rank) * a.nh + head) * chunks + chunk;
    for (uint32_t r = 0; r < world; ++r) {
        float *dst = reinterpret_cast<float *>(a.px_peer_bases[r] + flags_bytes) + my_slot * kP2PSlotFloats;
        dst[tid] = val;
        if (tid == 0) dst[kP2PChunk] = lse;
    }
    // the barrier orders the 64 threads' slot stores before the flag stores of threads 0..world-1, and a release at
    // system scope is cumulative over what happened before it: no separate system fence by every thread
    bar64();
    if (tid < world) st_release_sys(reinterpret_cast<uint32_t *>(a.px_peer_bases[tid]) + my_slot, a.px_epoch);
    if (tid < world) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(a.px_peer_bases[a.px_rank]) +
                               (((size_t)par * world + tid) * a.nh + head) * chunks + chunk;
        bool ok = false;
        for (uint32_t i = 0; i < a.wait_peer; ++i) {
            if ((int32_t)(ld_acquire_sys(flag) - a.px_epoch) >= 0) { ok = true; break; }
            if ((i & 4095u) == 4095u && gave_up(a.status)) break;   // somebody already gave up
        }
        if (!ok) {
            sm_fail = 1;
            report_timeout(a.status, 100 + (int)tid);
        }
    }
    bar64();
    if (sm_fail) return;
    const float *mine = reinterpret_cast<const float *>(a.px_peer_bases[a.px_rank] + flags_bytes);
    auto slot_of = [&](uint32_t r) { return mine + ((((size_t)par * world + r) * a.nh + head) * chunks + chunk) * kP2PSlotFloats; };
    if (tid < world) sm_lse[tid] = __ldcg(slot_of(tid) + kP2PChunk);
    bar64();
    if (d >= a.hd) return;
    float gmax = -INFINITY;
    for (uint32_t r = 0; r < world; ++r)
        if (sm_lse[r] > -INFINITY) gmax = fmaxf(gmax, sm_lse[r]);
    float acc = 0.f, wsum = 0.f;
    for (uint32_t r = 0; r < world; ++r) {
        const float l = sm_lse[r];
        if (!(l > -INFINITY)) continue;
        const float w = expf(l - gmax);
        acc += w * __ldcg(slot_of(r) + tid);
        wsum += w;
    }
    float out = wsum > 0.f ? acc / wsum : 0.f;
    const size_t oi = (size_t)head * a.hd + d;
    if (a.px_gate) out *= sigmoidf_ref(a.px_gate[oi]);
    store_from_f32(a.px_out, oi, a.px_out_dtype, out);
}

// ---------------------------------------------------------------------------------------
// Stand-alone merge of split records (gqa_reduce.wgsl:20-65), stride-generalised
// ---------------------------------------------------------------------------------------
struct ReduceArgs {
    const float *partials;
    void *out;
    const float *gate;
    uint32_t ns, nh, hd;
    unsigned long long split_stride, head_stride;  // floats
    uint32_t out_dtype;
};

__global__ void __launch_bounds__(128) reduce_kernel(const ReduceArgs a) {
    const uint32_t head = blockIdx.x;
    const float *hb = a.partials + (size_t)head * a.head_stride;
    // wgsl:33-43 (a thread-0 loop there; every thread repeats it here, it is ns loads)
    float gmax = -INFINITY;
    for (uint32_t s = 0; s < a.ns; ++s) {
        const float l = hb[(size_t)s * a.split_stride + a.hd];
        if (l > -INFINITY) gmax = fmaxf(gmax, l);  // false for -inf and NaN: empty splits
    }
    for (uint32_t d = threadIdx.x; d < a.hd; d += blockDim.x) {
        float acc = 0.f, wsum = 0.f;
        for (uint32_t s = 0; s < a.ns; ++s) {
            const float *rec = hb + (size_t)s * a.split_stride;
            const float l = rec[a.hd];
            if (!(l > -INFINITY)) continue;
            const float w = expf(l - gmax);  // wgsl:56
            acc += w * rec[d];
            wsum += w;
        }
        float val = wsum > 0.f ? acc / wsum : 0.f;
        const size_t oi = (size_t)head * a.hd + d;
        if (a.gate) val *= sigmoidf_ref(a.gate[oi]);
        store_from_f32(a.out, oi, a.out_dtype, val);
    }
}

__global__ void sigmoid_mul_kernel(float *x, const float *gate, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = x[i] * sigmoidf_ref(gate[i]);  // sigmoid_mul.wgsl:20-22
}

// ---------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------
template <typename T, int HD, int NW, int STAGES, int KPC, bool ILV = false, int F8 = 0>
static int launch16(shady_ctx *ctx, const DecodeArgs &a, uint32_t blocks) {
    using S = Decode16Smem<HD, NW, STAGES, KPC, F8>;
    static_assert(S::kTotal <= 232448, "shared memory of this configuration exceeds 227 KB");
    auto kern = decode16_kernel<T, HD, NW, STAGES, KPC, ILV, F8>;
    static thread_local int configured_dev = -1;
    if (configured_dev != ctx->device) {
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured_dev = ctx->device;
    }
    // Programmatic stream order: the CTAs of this launch may become resident while the kernel before it in the
    // stream drains (a decode launch ends with a few CTAs merging records while the other SMs idle) and wait at the
    // kernel's first instructions until that kernel has completed and its writes are visible.
    // The grid barrier needs every CTA resident: a cooperative launch, refused if they would not fit.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks); cfg.blockDim = dim3(NW * 32); cfg.dynamicSmemBytes = S::kTotal; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2]{};
    unsigned n = 0;
    if (a.grid_merge) { attr[n].id = cudaLaunchAttributeCooperative; attr[n].val.cooperative = 1; ++n; }
    if (ctx->knobs.early_launch && !a.grid_merge) {   // (measured on cooperative launches too: no gain)
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr; cfg.numAttrs = n;
    SHADY_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, kern, a));
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

// Dispatch on dtype and on the kv heads per CTA (a power of two that divides nkv, at most NW).
template <int HD, int NW, int STAGES>
static int launch16_kpc(shady_ctx *ctx, const DecodeArgs &a, uint32_t kpc, bool half, uint32_t blocks) {
#define SHADY_L16(K_) \
    (half ? launch16<__half, HD, NW, STAGES, K_>(ctx, a, blocks) : launch16<__nv_bfloat16, HD, NW, STAGES, K_>(ctx, a, blocks))
    if constexpr (NW >= 8 && HD <= 128) {   // eight Q tiles of head_dim 256 would not fit next to the pipeline
        if (kpc == 8) return SHADY_L16(8);
    }
    if (kpc == 4) return SHADY_L16(4);
    if (kpc == 2) return SHADY_L16(2);
    return SHADY_L16(1);
#undef SHADY_L16
}
// The interleaved mode exists for the default configuration of each head_dim only.
template <int HD, int NW, int STAGES>
static int launch16_ilv(shady_ctx *ctx, const DecodeArgs &a, bool half, uint32_t blocks) {
    return half ? launch16<__half, HD, NW, STAGES, 1, true>(ctx, a, blocks)
                : launch16<__nv_bfloat16, HD, NW, STAGES, 1, true>(ctx, a, blocks);
}

struct Variant16 {
    uint32_t nw, stages, ctas_per_sm;
};
// {warps, tile slots per warp, CTAs per SM}.  head_dim 128: 4 warps x 6 slots at two CTAs per SM measured best on the
// ragged fp16 batch (8 warps and 128 KB of K/V in flight per SM).  head_dim 256: tiles are twice as large and a block
// costs twice the math, so one CTA of 8 warps x 3 slots keeps the same number of warps and bytes in flight per SM.
static Variant16 variant16(uint32_t hd, uint32_t v) {
    if (hd > 128) return v == 1 ? Variant16{4, 6, 1} : (v == 2 ? Variant16{8, 2, 1} : Variant16{8, 3, 1});
    switch (v) {
        case 1: return Variant16{8, 4, 1};
        case 2: return Variant16{8, 6, 1};
        default: return Variant16{4, 6, 2};
    }
}
static uint32_t kv_heads_per_cta(uint32_t nkv, uint32_t nw) {
    uint32_t k = 1;
    while (k * 2 <= nw && k * 2 <= nkv && nkv % (k * 2) == 0) k *= 2;
    return k;
}

template <int HD, int NW>
static int launch32(shady_ctx *ctx, const DecodeArgs &a, uint32_t blocks, uint32_t GT) {
    switch (GT) {
        case 8: decode32_kernel<HD, 8, NW><<<blocks, NW * 32, 0, ctx->stream>>>(a); break;
        case 4: decode32_kernel<HD, 4, NW><<<blocks, NW * 32, 0, ctx->stream>>>(a); break;
        case 2: decode32_kernel<HD, 2, NW><<<blocks, NW * 32, 0, ctx->stream>>>(a); break;
        default: decode32_kernel<HD, 1, NW><<<blocks, NW * 32, 0, ctx->stream>>>(a); break;
    }
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

static uint32_t group_rows_f32(uint32_t G) { return G >= 8 ? 8u : (G >= 4 ? 4u : (G >= 2 ? 2u : 1u)); }
static uint32_t head_groups(uint32_t kv_dtype, uint32_t G) {
    if (kv_dtype == SHADY_F32) {
        const uint32_t gt = group_rows_f32(G);
        return (G + gt - 1) / gt;
    }
    if (kv_dtype == SHADY_F8E4M3 || kv_dtype == SHADY_F8E5M2) return (G + 7) / 8;   // heads sit on the MMA's eight N columns
    return (G + 15) / 16;
}

constexpr uint32_t kDeferMergeRecords = 12;  // more records than this per sequence: merged by the whole grid, not by its last CTA

// Workspace layout: [arrival counters: num_seqs*nkv*gz u32][grid barrier: 2 u32], padded to 256 B, [partial records].
static size_t counter_words(const shady_decode_params *p) {
    return (size_t)p->num_seqs * p->num_kv_heads * ((p->heads_per_kv + 15) / 16 + p->heads_per_kv);
}
static size_t counters_bytes(const shady_decode_params *p) {
    return ((counter_words(p) + 2) * sizeof(uint32_t) + 255) / 256 * 256;   // + the two words of the grid barrier
}
size_t decode_workspace_bytes(const shady_decode_params *p) {
    if (p->num_splits == 1) return 0;
    const size_t rec = (size_t)p->num_q_heads * (p->head_dim + 2) * sizeof(float);
    size_t recs;
    if (p->num_splits > 1) recs = (size_t)p->num_seqs * p->num_splits;
    // balanced: two record slots per span; spans <= resident CTAs (one CTA may serve all kv heads)
    else recs = 2 * ((size_t)kMaxSlots + 1);
    return counters_bytes(p) + recs * rec;
}

// Inputs of the fused append (NULL = plain decode).
struct FusedAppendIn {
    const shady_append_params *ap;
    const void *q_full, *k_proj, *v_proj;
    const uint16_t *norm_w;
};

// Cross-GPU tail of a row-sharded decode (NULL = none): merge + exchange + merge across ranks in the same launch.
struct ShardExchangeIn {
    uint32_t world, rank, epoch, out_dtype;
    void *const *d_peer_table;
    void *d_out;
    const float *d_gate;
};

// Everything a decode launch needs except the scratch memory: checked arguments, the span plan, which kernel
// variant runs and how much scratch this particular launch touches.  Both entry points that launch a decode (with
// the caller's workspace, with the built-in array) go through plan_decode and run_decode, so they cannot drift.
struct DecodePlan {
    DecodeArgs a;
    Variant16 var;
    uint32_t kpc, blocks;
    bool f32, half, need_ws, second_launch;
    int f8;                  // 0: not an 8-bit cache, 1: e4m3, 2: e5m2
    size_t counters_bytes;   // arrival counters + barrier words at the head of the scratch
    size_t scratch_bytes;    // counters + the records this launch writes (<= decode_workspace_bytes)
    dim3 merge_grid;         // second launch (no grid merge): balanced_merge_kernel / shard_merge_p2p_kernel
    bool exchange;
};

static int plan_decode(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                       const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, void *d_out, float *d_lse,
                       const float *d_gate, float *d_force_partials, float *d_shard_records, const FusedAppendIn *fa,
                       const ShardExchangeIn *px, DecodePlan *plan) {
    SHADY_REQUIRE(ctx, p && (d_q || fa) && cache && d_seq_lens, SHADY_ERR_BAD_ARG, "decode: null argument");
    SHADY_REQUIRE(ctx, d_out || d_force_partials || d_shard_records, SHADY_ERR_BAD_ARG, "decode: null output");
    SHADY_REQUIRE(ctx, p->num_seqs > 0 && p->num_kv_heads > 0 && p->heads_per_kv > 0, SHADY_ERR_BAD_ARG,
                  "decode: zero-sized problem");
    SHADY_REQUIRE(ctx, p->num_q_heads == p->num_kv_heads * p->heads_per_kv, SHADY_ERR_BAD_ARG,
                  "decode: num_q_heads != num_kv_heads * heads_per_kv");
    SHADY_REQUIRE(ctx, cache->dtype <= SHADY_F8E5M2, SHADY_ERR_BAD_ARG, "decode: bad cache dtype");
    SHADY_REQUIRE(ctx, (cache->d_k_ptrs && cache->d_v_ptrs) || (cache->d_k_base && cache->d_v_base),
                  SHADY_ERR_BAD_ARG, "decode: cache has neither base pointers nor pointer arrays");
    const int f8 = cache->dtype == SHADY_F8E4M3 ? 1 : (cache->dtype == SHADY_F8E5M2 ? 2 : 0);   // 8-bit format of the cache
    const uint32_t act_dtype = f8 ? (uint32_t)SHADY_F16 : cache->dtype;   // what Q and the output may be besides f32
    SHADY_REQUIRE(ctx, p->q_dtype == SHADY_F32 || p->q_dtype == act_dtype, SHADY_ERR_UNSUPPORTED,
                  "decode: q_dtype must be f32 or the cache dtype (f16 for an 8-bit cache)");
    SHADY_REQUIRE(ctx, p->out_dtype == SHADY_F32 || p->out_dtype == act_dtype, SHADY_ERR_UNSUPPORTED,
                  "decode: out_dtype must be f32 or the cache dtype (f16 for an 8-bit cache)");
    SHADY_REQUIRE(ctx, !f8 || !d_force_partials, SHADY_ERR_UNSUPPORTED,
                  "decode: an 8-bit cache is read by shady_attn_decode / _static / _shard / _append");
    if (const int st = pending_timeout(ctx, "decode")) return st;
    const uint32_t hd = p->head_dim;
    SHADY_REQUIRE(ctx, hd <= 256, SHADY_ERR_UNSUPPORTED, "decode: head_dim > 256 (the reference shader's limit)");
    const bool f32 = cache->dtype == SHADY_F32;
    if (f32) SHADY_REQUIRE(ctx, hd == 64 || hd == 128 || hd == 256, SHADY_ERR_UNSUPPORTED, "decode: f32 cache needs head_dim 64/128/256");
    else SHADY_REQUIRE(ctx, hd == 128 || hd == 256, SHADY_ERR_UNSUPPORTED, "decode: 16-bit cache needs head_dim 128/256");

    DecodeArgs &a = plan->a;
    a = DecodeArgs{};
    a.q = d_q; a.out = d_out; a.lse = d_lse; a.gate = d_gate;
    if (const int st = fill_kv_addr(ctx, cache, p->num_kv_heads, hd, "decode", &a.kv)) return st;
    SHADY_REQUIRE(ctx, !a.kv.page_table || p->num_splits <= 1, SHADY_ERR_UNSUPPORTED,
                  "decode: a paged cache needs num_splits 0 or 1 (16-row blocks must not straddle pages)");
    a.seq_lens = d_seq_lens;
    if (seq_lens_host && p->num_seqs <= 32) {
        a.lens_n = p->num_seqs;
        for (uint32_t i = 0; i < p->num_seqs; ++i) a.lens_v[i] = seq_lens_host[i];
    }
    a.num_seqs = p->num_seqs; a.nkv = p->num_kv_heads; a.nh = p->num_q_heads; a.G = p->heads_per_kv; a.hd = hd;
    a.q_dtype = p->q_dtype; a.out_dtype = p->out_dtype;
    // 8-bit cache: K's scale, and the 2^8 the byte-to-f16 conversion leaves out, ride on the score scale
    a.scale_log2 = (1.0f / sqrtf((float)hd)) * kLog2e * a.kv.k_scale * f8_unscale(f8);
    a.num_splits = p->num_splits;
    a.out_row_stride = hd; a.lse_stride = 1;
    a.status = status_ref(ctx); a.wait_grid = ctx->wait_grid; a.wait_peer = ctx->wait_peer;
    if (d_shard_records) {   // rank-local result of one shard as records [seq][nh][hd+2]: out, lse, (unused)
        a.out = d_shard_records; a.out_dtype = SHADY_F32; a.out_row_stride = hd + 2;
        a.lse = d_shard_records + hd; a.lse_stride = hd + 2; a.gate = nullptr;
    }
    a.gz = head_groups(cache->dtype, p->heads_per_kv);
    plan->exchange = px != nullptr;
    if (px) {
        SHADY_REQUIRE(ctx, d_shard_records && px->d_peer_table && px->d_out && !fa, SHADY_ERR_BAD_ARG, "decode_shard_p2p: null argument");
        SHADY_REQUIRE(ctx, p->num_seqs == 1 && p->num_splits == 0, SHADY_ERR_UNSUPPORTED,
                      "decode_shard_p2p: one sequence, balanced spans (num_splits 0)");
        SHADY_REQUIRE(ctx, px->world >= 1 && px->world <= kP2PMaxWorld && px->rank < px->world, SHADY_ERR_BAD_ARG,
                      "decode_shard_p2p: bad world/rank");
        SHADY_REQUIRE(ctx, px->epoch != 0, SHADY_ERR_BAD_ARG, "decode_shard_p2p: epoch must start at 1 (flags start at 0)");
        SHADY_REQUIRE(ctx, px->out_dtype <= SHADY_BF16, SHADY_ERR_BAD_ARG, "decode_shard_p2p: bad out dtype");
        a.px_peer_bases = reinterpret_cast<char *const *>(px->d_peer_table);
        a.px_out = px->d_out; a.px_gate = px->d_gate; a.px_out_dtype = px->out_dtype;
        a.px_world = px->world; a.px_rank = px->rank; a.px_epoch = px->epoch;
        a.defer_merge = 1;   // the decode CTAs only write records; the tail (or the second launch) merges and exchanges
    }
    if (fa) {
        const shady_append_params *ap = fa->ap;
        SHADY_REQUIRE(ctx, ap && fa->q_full && fa->k_proj && fa->v_proj, SHADY_ERR_BAD_ARG, "decode_append: null argument");
        SHADY_REQUIRE(ctx, !f32, SHADY_ERR_UNSUPPORTED, "decode_append: needs a 16-bit cache (use the two calls for fp32)");
        SHADY_REQUIRE(ctx, ap->num_heads == p->num_q_heads && ap->num_kv_heads == p->num_kv_heads && ap->head_dim == hd &&
                               ap->num_seqs == p->num_seqs && ap->tokens_per_seq == 1,
                      SHADY_ERR_BAD_ARG, "decode_append: append and decode parameters disagree");
        SHADY_REQUIRE(ctx, ap->interleaved && ap->rotary_dim <= hd && (ap->rotary_dim % 2) == 0 &&
                               ap->s1_limit == ap->rotary_dim / 2 && ap->s2_limit == ap->rotary_dim / 2,
                      SHADY_ERR_UNSUPPORTED, "decode_append: interleaved RoPE with one position per token only");
        SHADY_REQUIRE(ctx, ap->in_dtype <= SHADY_BF16, SHADY_ERR_BAD_ARG, "decode_append: bad input dtype");
        a.fuse_append = 1;
        a.ap_q = fa->q_full; a.ap_k = fa->k_proj; a.ap_v = fa->v_proj; a.ap_norm_w = fa->norm_w;
        a.ap_in_dtype = ap->in_dtype; a.ap_has_gate = ap->has_gate; a.ap_rd = ap->rotary_dim; a.ap_eps = ap->eps;
        for (uint32_t i = 0; i < ap->rotary_dim / 2; ++i)   // same libm call as the stand-alone append and the oracle
            a.ap_inv_freq[i] = 1.0f / powf(ap->rope_theta, 2.0f * (float)i / (float)ap->rotary_dim);
        a.gate = nullptr;
    }
    const DecodeKnobs &kn = ctx->knobs;
    // 8-bit tiles are half as large: twice the slots keep the same bytes in flight per warp
    const Variant16 var = f8 ? (hd > 128 ? Variant16{8, 6, 1} : Variant16{4, 8, 3}) : variant16(hd, kn.variant);
    // One kv head per CTA measured fastest (sibling CTAs of the other kv heads run next to each other in
    // the grid and fetch the rest of each cache row); the kpc knob packs more kv heads into a CTA.
    uint32_t kpc = 1u;
    if (!f32 && !f8 && !fa && kn.kpc && kn.kpc <= kv_heads_per_cta(p->num_kv_heads, hd > 128 ? 4u : var.nw) && (kn.kpc & (kn.kpc - 1)) == 0)
        kpc = kn.kpc;
    const uint32_t kv_groups = p->num_kv_heads / kpc;
    uint32_t ctas_per_sm = kn.ctas_per_sm ? kn.ctas_per_sm : (f32 ? 4u : var.ctas_per_sm);
    if (ctas_per_sm > 8) ctas_per_sm = 8;
    uint32_t min_span = kn.min_span ? kn.min_span : (f32 ? 2u : 4u * (var.nw / kpc));
    // one sequence: nothing else fills the SMs, so spans go down to one 16-row block per warp (a 16384-row shard of a
    // row-sharded context then streams on all SMs instead of 64: 22.6 -> 21.3 us per step)
    if (!kn.min_span && !f32 && p->num_seqs == 1) min_span = var.nw / kpc;

    const size_t rec_bytes = (size_t)p->num_q_heads * (hd + 2) * sizeof(float);
    unsigned long long items, recs = 0;
    plan->need_ws = false;
    if (d_force_partials) {
        SHADY_REQUIRE(ctx, p->num_seqs == 1 && p->num_splits >= 2, SHADY_ERR_BAD_ARG,
                      "decode_partials: needs num_seqs == 1 and num_splits >= 2");
        a.force_partials = 1; a.partials = d_force_partials;
        items = p->num_splits;
    } else if (p->num_splits >= 1) {
        items = (unsigned long long)p->num_seqs * p->num_splits;
        plan->need_ws = p->num_splits > 1;
        recs = items;
    } else {
        SHADY_REQUIRE(ctx, seq_lens_host, SHADY_ERR_BAD_ARG, "decode: num_splits == 0 needs seq_lens_host");
        // what a second piece costs a CTA, in row-blocks: a least-squares fit of the spans' end times on the cfg2 batch
        // gives 0.265 us per block and 7.7 us per piece, i.e. 29 blocks of 8 KB (head_dim 128, 16 bits) — about 256 KB
        // of K and V at a CTA's share of the memory bandwidth (steps measured with 0/12/20/25/32/40/56 blocks lie within
        // 2 % of each other, the best between 32 and 40); the SHADY_DECODE_PAD knob overrides (0 = none)
        if (p->num_seqs > 1 && !f32) {
            // (8-bit caches: three CTAs share an SM and a boundary idles a third of its streams; half the 16-bit figure
            //  measured best for both formats on the cfg2 batch: e4m3 70.9 / 70.7 / 70.1 / 72.3 / 78.8 us with
            //  0 / 8 / 16 / 32 / 64 blocks, e5m2 56.6 / 55.4 / 54.9 / 55.3 / 59.7)
            const unsigned long long block_bytes = 2ull * kBlkPos * hd * 2 * kpc;
            unsigned long long pad = kn.pad != ~0u ? kn.pad : (256ull << 10) / block_bytes / (f8 ? 2 : 1);
            a.pad = (uint32_t)(pad > 64 ? 64 : pad);
        }
        unsigned long long line = 0;
        for (uint32_t i = 0; i < p->num_seqs; ++i) line += (seq_lens_host[i] == 0 ? 1 : (seq_lens_host[i] + kBlkPos - 1) / kBlkPos) + a.pad;
        SHADY_REQUIRE(ctx, line <= 0xffffffffull, SHADY_ERR_UNSUPPORTED, "decode: batch too long for one launch");
        unsigned long long slots = (unsigned long long)ctx->num_sms * ctas_per_sm;
        if (slots > kMaxSlots) slots = kMaxSlots;
        unsigned long long spans = slots / ((unsigned long long)kv_groups * a.gz);
        const unsigned long long by_size = (line + min_span - 1) / min_span;
        if (spans > by_size) spans = by_size;
        if (spans < 1) spans = 1;
        a.line_blocks = (uint32_t)line;
        a.spans = (uint32_t)spans;
        a.span_math32 = (spans + 1) * line + spans < 0xffffffffull ? 1u : 0u;
        items = spans;
        plan->need_ws = spans > 1;  // a sequence may straddle spans whenever there is more than one
        recs = 2 * spans;           // two record slots per span
        // a sequence cut into many spans is merged by the grid (or a wide second launch) instead of by its last CTA
        unsigned long long u = 0;
        for (uint32_t i = 0; i < p->num_seqs && !a.defer_merge; ++i) {
            const unsigned long long nb = seq_lens_host[i] == 0 ? 1 : (seq_lens_host[i] + kBlkPos - 1) / kBlkPos;
            const unsigned long long nrec = ((u + nb - 1) * spans) / line - (u * spans) / line + 1;
            if (nrec > kDeferMergeRecords) a.defer_merge = 1;
            u += nb + a.pad;
        }
    }
    plan->counters_bytes = counters_bytes(p);
    plan->scratch_bytes = plan->need_ws ? plan->counters_bytes + (size_t)recs * rec_bytes : 0;
    const unsigned long long blocks64 = items * kv_groups * a.gz;
    SHADY_REQUIRE(ctx, blocks64 <= 0x7fffffffull, SHADY_ERR_UNSUPPORTED, "decode: too many work items for one launch");
    plan->blocks = (uint32_t)blocks64;
    // one launch instead of two: the grid is one resident wave (it is sized from the SM count above), so it can meet
    // at a barrier and merge (and, row-sharded, exchange) itself; the grid_merge knob set to 0 keeps the second
    // launch, and so does an experimental CTAs-per-SM override, which may ask for more CTAs than can be resident
    if (a.defer_merge && plan->need_ws && !f32 && kn.grid_merge && !kn.ctas_per_sm) {   // (a single span has no workspace)
        a.grid_merge = 1;
        // one sequence of many spans in the default configuration: its blocks are interleaved over all warps
        if (kn.interleave && p->num_seqs == 1 && !fa && !f8 && !a.kv.page_table && kpc == 1 && kn.variant == 0) a.interleave = 1;
    }
    plan->var = var; plan->kpc = kpc; plan->f32 = f32; plan->half = cache->dtype == SHADY_F16; plan->f8 = f8;
    plan->second_launch = a.defer_merge && !a.grid_merge;
    plan->merge_grid = px ? dim3(1, p->num_q_heads, p2p_chunks(hd)) : dim3(p->num_seqs, p->num_q_heads, (hd + 63) / 64);
    return SHADY_OK;
}

// Launches a planned decode on `scratch` (counters zeroed, at least plan.scratch_bytes; NULL when the plan needs none).
static int run_decode(shady_ctx *ctx, const shady_decode_params *p, DecodePlan &plan, void *scratch) {
    DecodeArgs &a = plan.a;
    const uint32_t hd = p->head_dim, blocks = plan.blocks;
    if (plan.need_ws) {
        a.counters = reinterpret_cast<uint32_t *>(scratch);
        a.partials = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + plan.counters_bytes);
        a.grid_sync = a.counters + counter_words(p);
    }
    int rc;
    if (plan.f32) {
        const uint32_t gt = group_rows_f32(p->heads_per_kv);
        if (hd == 64) rc = launch32<64, 8>(ctx, a, blocks, gt);
        else if (hd == 128) rc = launch32<128, 8>(ctx, a, blocks, gt);
        else rc = launch32<256, 4>(ctx, a, blocks, gt);
    } else {
        const bool h = plan.half;
        const Variant16 &var = plan.var;
        if (plan.f8 == 1) rc = hd == 128 ? launch16<__half, 128, 4, 8, 1, false, 1>(ctx, a, blocks)
                                         : launch16<__half, 256, 8, 6, 1, false, 1>(ctx, a, blocks);
        else if (plan.f8 == 2) rc = hd == 128 ? launch16<__half, 128, 4, 8, 1, false, 2>(ctx, a, blocks)
                                              : launch16<__half, 256, 8, 6, 1, false, 2>(ctx, a, blocks);
        else if (a.interleave) rc = hd == 128 ? launch16_ilv<128, 4, 6>(ctx, a, h, blocks) : launch16_ilv<256, 8, 3>(ctx, a, h, blocks);
        else if (hd == 128) {
            if (var.nw == 8 && var.stages == 6) rc = launch16_kpc<128, 8, 6>(ctx, a, plan.kpc, h, blocks);
            else if (var.nw == 8) rc = launch16_kpc<128, 8, 4>(ctx, a, plan.kpc, h, blocks);
            else rc = launch16_kpc<128, 4, 6>(ctx, a, plan.kpc, h, blocks);
        } else if (var.nw == 4) rc = launch16_kpc<256, 4, 6>(ctx, a, plan.kpc, h, blocks);
        else if (var.stages == 2) rc = launch16_kpc<256, 8, 2>(ctx, a, plan.kpc, h, blocks);
        else rc = launch16_kpc<256, 8, 3>(ctx, a, plan.kpc, h, blocks);
    }
    if (rc != SHADY_OK || !plan.second_launch) return rc;
    // (launching the merge as a programmatic dependent of the decode grid measured slower: 72.7 vs 67.4 us per step)
    if (plan.exchange) shard_merge_p2p_kernel<<<plan.merge_grid, kMergeThreads, 0, ctx->stream>>>(a);
    else balanced_merge_kernel<<<plan.merge_grid, kMergeThreads, 0, ctx->stream>>>(a);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

int launch_decode(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                  const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, void *d_out, float *d_lse,
                  const float *d_gate, void *d_ws, size_t ws_bytes, float *d_force_partials, float *d_shard_records,
                  const FusedAppendIn *fa, const ShardExchangeIn *px) {
    DecodePlan plan;
    if (const int st = plan_decode(ctx, p, d_q, cache, d_seq_lens, seq_lens_host, d_out, d_lse, d_gate, d_force_partials,
                                   d_shard_records, fa, px, &plan))
        return st;
    if (plan.need_ws)   // the documented size is the bound over any lengths, so that one allocation serves every step
        SHADY_REQUIRE(ctx, d_ws && ws_bytes >= decode_workspace_bytes(p), SHADY_ERR_WORKSPACE, "decode: workspace missing or too small");
    return run_decode(ctx, p, plan, d_ws);
}

// The workspace must hold zeros in its counter area before the first call; the kernels
// leave it zeroed again.
int init_decode_workspace(shady_ctx *ctx, const shady_decode_params *p, void *d_ws, size_t ws_bytes) {
    SHADY_REQUIRE(ctx, p, SHADY_ERR_BAD_ARG, "decode_workspace_init: null params");
    const size_t need = decode_workspace_bytes(p);
    if (need == 0) return SHADY_OK;
    SHADY_REQUIRE(ctx, d_ws && ws_bytes >= need, SHADY_ERR_WORKSPACE, "decode_workspace_init: workspace missing or too small");
    SHADY_CUDA_OK(ctx, cudaMemsetAsync(d_ws, 0, counters_bytes(p), ctx->stream));
    return SHADY_OK;
}

// ---------------------------------------------------------------------------------------
// Decode with built-in scratch (no counterpart in the reference)
// ---------------------------------------------------------------------------------------
// Some hosts cannot give this library a workspace allocated at call time: an inference server that
// hands all device memory to its KV-cache arena at start-up has nothing left for cudaMalloc, and a
// decode loop that must not stall cannot afford cudaMalloc's implicit device synchronisation.  For them
// the arrival counters and split records live in this fixed array, which every GPU that loads the
// library holds until the process exits.  Launches that need more than kStaticScratchBytes are refused.
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
static unsigned char *g_static_scratch_addr[kMaxDevices] = {};  // device address of the array, per device

// `g_static_scratch` in host code is only a handle; the device address comes from the runtime, once per
// device, with that device current.
static int static_scratch_ptr(shady_ctx *ctx, unsigned char **out) {
    SHADY_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kMaxDevices, SHADY_ERR_UNSUPPORTED,
                  "decode_static: device ordinal out of range");
    if (!g_static_scratch_addr[ctx->device]) {
        unsigned char *ptr = nullptr;
        SHADY_CUDA_OK(ctx, cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch));
        SHADY_REQUIRE(ctx, ptr != nullptr, SHADY_ERR_CUDA, "decode_static: cudaGetSymbolAddress returned a null address");
        g_static_scratch_addr[ctx->device] = ptr;
    }
    *out = g_static_scratch_addr[ctx->device];
    return SHADY_OK;
}

// Same checks, same span plan and same kernels as launch_decode (plan_decode / run_decode); only the scratch differs:
// what this particular launch touches must fit the array, and the counters are cleared on the stream first because
// every call on the device shares it.
int launch_decode_static(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                         const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, void *d_out, float *d_lse,
                         const float *d_gate) {
    SHADY_REQUIRE(ctx, d_q && d_out, SHADY_ERR_BAD_ARG, "decode_static: null argument");
    DecodePlan plan;
    if (const int st = plan_decode(ctx, p, d_q, cache, d_seq_lens, seq_lens_host, d_out, d_lse, d_gate, nullptr, nullptr,
                                   nullptr, nullptr, &plan))
        return st;
    unsigned char *scratch = nullptr;
    if (plan.need_ws) {
        if (plan.scratch_bytes > kStaticScratchBytes)
            return fail(ctx, SHADY_ERR_WORKSPACE,
                        "decode_static: this launch needs " + std::to_string(plan.scratch_bytes) + " bytes of scratch but the built-in array holds " +
                            std::to_string(kStaticScratchBytes) + "; use shady_attn_decode with a caller-provided workspace");
        if (const int rc = static_scratch_ptr(ctx, &scratch)) return rc;
        // the array keeps whatever the previous call left: the arrival counters and barrier words must start at zero
        SHADY_CUDA_OK(ctx, cudaMemsetAsync(scratch, 0, plan.counters_bytes, ctx->stream));
    }
    return run_decode(ctx, p, plan, scratch);
}

int launch_reduce(shady_ctx *ctx, uint32_t hd, uint32_t ns, uint32_t nh, uint64_t split_stride, uint64_t head_stride,
                  const float *d_partials, void *d_out, uint32_t out_dtype, const float *d_gate) {
    SHADY_REQUIRE(ctx, d_partials && d_out && hd && ns && nh, SHADY_ERR_BAD_ARG, "reduce: null or zero argument");
    SHADY_REQUIRE(ctx, out_dtype <= SHADY_BF16, SHADY_ERR_BAD_ARG, "reduce: bad out dtype");
    ReduceArgs r{};
    r.partials = d_partials; r.out = d_out; r.gate = d_gate; r.ns = ns; r.nh = nh; r.hd = hd;
    r.split_stride = split_stride; r.head_stride = head_stride; r.out_dtype = out_dtype;
    reduce_kernel<<<nh, 128, 0, ctx->stream>>>(r);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

int launch_sigmoid_mul(shady_ctx *ctx, float *d_x, const float *d_gate, uint32_t n) {
    SHADY_REQUIRE(ctx, d_x && d_gate, SHADY_ERR_BAD_ARG, "sigmoid_mul: null argument");
    if (n == 0) return SHADY_OK;
    sigmoid_mul_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(d_x, d_gate, n);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

}  // namespace shady
