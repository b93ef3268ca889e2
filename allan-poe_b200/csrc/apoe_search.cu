// Batched greedy beam search over the hybrid graph (one CTA per query, persistent grid).
//
// Behaviour follows the reference search kernels (src/query.cu:277-1268 for the seven weight subsets,
// :1271-1483 keyword, :1541-1779 knowledge graph): same pool / staging arrays, the same visited-set reset every
// 4th iteration, the same 32-element bitonic network and the same tie rules in the pool merge, and the same
// dense arithmetic (fp16 multiply-adds in the reference's lane/chunk association), so the pool contents match
// it element for element.  What differs is how the work is mapped to the machine:
//   * every document is one contiguous, 16-byte aligned record (dense halves + interleaved sparse and BM25
//     pairs); an expansion fetches the records of all unvisited neighbours with cp.async.bulk copies into a ring
//     of shared-memory slots, each with a "filled" and a "free" mbarrier, fed by one warp and drained by the others;
//   * graph rows carry each neighbour's record locator, so an expansion is two dependent memory round trips
//     (row, records) instead of four (row, CSR offsets, CSR rows / dense row);
//   * the query's sparse and BM25 rows are hashed into shared memory and probed with the document's terms;
//   * selection, visited filtering, the 32-wide sort and the copy planning run in one warp on registers and
//     shuffles; scoring runs in the consumer warps and the pool merge in the whole CTA.
#include <algorithm>
#include <cstdio>

#include "apoe_common.cuh"

namespace apoe {

#ifndef AP_SEARCH_THREADS
#define AP_SEARCH_THREADS 96    // threads of one CTA = one query in flight (a multiple of 32, at least 32)
#endif
#ifndef AP_SEARCH_CTAS
#define AP_SEARCH_CTAS 6        // CTAs the kernel is compiled to fit on one SM (registers) and the arena is sized for (shared memory)
#endif
constexpr int kSearchThreads = AP_SEARCH_THREADS;   // the throughput shape: batches that fill the GPU
constexpr int kSearchWarps = kSearchThreads / 32;
constexpr int kSearchCtas = AP_SEARCH_CTAS;
// The latency shape, for batches too small to fill the SMs (a single query is the extreme): more warps score the
// records of one expansion, fewer CTAs share an SM.  Same code, same results; only the mapping of work to warps differs.
constexpr int kLatencyThreads = 256;
constexpr int kLatencyCtas = 2;
constexpr int ctas_for_shape(int threads) { return threads == kSearchThreads ? kSearchCtas : kLatencyCtas; }
constexpr uint32_t kFull = 0xFFFFFFFFu;
constexpr int kMaxIter = 1000;    // ref: MAX_ITER, src/query.cu:7
constexpr int kHashReset = 4;     // ref: HASH_RESET, src/query.cu:16
constexpr int kKeywordRing = 32;  // ref: KEYWORD, src/query.cu:18
constexpr int kMaxSlots = 16;     // ring slots of the staging arena (a "filled" and a "free" mbarrier each)
constexpr uint32_t kHeaderBytes = 16u * kMaxSlots + 64u;   // the mbarriers, then 16 control words

enum : int { PF_DENSE = 1, PF_SPARSE = 2, PF_BM25 = 4, PF_KEYWORD = 8, PF_KG = 16, PF_UNFUSED = 32 };
enum : int { CTL_QUERY = 0, CTL_SEL = 1, CTL_NPAIRS = 2, CTL_NEXT = 3, CTL_MERGE = 4, CTL_SLOT = 5, CTL_KWNUM = 6, CTL_M = 7, CTL_MULT_S = 8, CTL_MULT_B = 9 };

struct SearchArgs {
    const FatEdge *fat;
    const FatEdge *ep_fat;
    const uint8_t *rec;
    const uint64_t *meta;
    uint32_t n;
    const float *qdense;
    const uint32_t *qs_off, *qs_idx;
    const float *qs_val;
    const uint32_t *qb_off, *qb_idx;
    const float *qb_val;
    const uint32_t *e2e_off, *e2e_idx, *e2d_off, *e2d_idx, *qe_off, *qe_idx;
    uint32_t nq;
    float w_sparse, w_bm25, w_dense, kg_weight;
    uint32_t cands;
    uint32_t *out_ids;
    float *out_dis;
    unsigned long long *out_keys;  // corpus-sharded search: nq x key_top_k packed (ordered distance, global id), or null
    uint32_t key_top_k, id_base;   // global id = local id + id_base
    uint32_t *ctl;            // [0] next query, [1] error word
    unsigned long long *cnt;  // [0] expansions, [1] evaluations, [2] gathered bytes
    uint32_t arena_bytes;
    uint32_t slot_bytes, slots;    // the arena as a ring of slots, each holding the records one warp scores side by side
    uint32_t single;               // 1: a slot holds one record (records too large for two per slot)
    uint32_t vis_mask;           // visited table size - 1
    uint32_t ts_slots, ts_shift; // collision-free table of the query's sparse row (0 slots: not allocated)
    uint32_t tb_slots, tb_shift; // same for the BM25 row
    // shared-memory byte offsets
    uint32_t o_pool_id, o_pool_dis, o_pool_ent, o_pool_hop, o_vis, o_info, o_sq, o_bq, o_ts, o_tb, o_kw, o_arena;
};

// A query row as the scoring code sees it: the terms as given (ascending ids; BM25 ids may carry the keyword flag
// in bit 31) and, when the row is short, a collision-free hash table: slot = (id * mult) >> shift, every slot holds
// at most one term, so a lookup is one shared-memory load and one compare.  mult == 0: no table, use the terms.
struct QRow {
    const uint2 *terms; uint32_t n;
    const uint2 *tab; uint32_t shift, mult;
};

struct Ctx {  // per-thread view of the CTA's shared state
    uint64_t *mbar;
    volatile uint32_t *ctl;
    uint32_t *pool_id;
    float *pool_dis;
    uint32_t *pool_ent, *pool_hop;
    uint32_t *vis;
    uint2 *info;
    uint2 *sq, *bq;     // the query's sparse / BM25 terms (id, weighted value), as given
    uint2 *ts, *tb;     // their collision-free tables
    QRow qs, qb;
    uint32_t *kw_id;
    float *kw_dis;
    uint8_t *arena;
    uint32_t gpair;     // slots filled so far by this CTA: slot = gpair % slots, barrier phase = gpair / slots
    unsigned long long c_exp, c_eval, c_bytes;
    long long t_wait, t_score, t_ctl, t_sort, t_merge, t_mark;   // clock64 phase totals (thread 0)
    int tid, lane, warp;
};

// ---------------------------------------------------------------------------------------------------------
// small device pieces
// ---------------------------------------------------------------------------------------------------------
// Visited set (ref: hash_insert, include/utils.cuh:282-297).  1 = newly inserted, 0 = already present / full.
__device__ __forceinline__ uint32_t vis_insert(uint32_t *tab, uint32_t mask, uint32_t key) {
    uint32_t idx = (key ^ (key >> 10)) & mask;
    for (uint32_t i = 0; i <= mask; ++i) {
        const uint32_t old = atomicCAS(&tab[idx], kEmpty, key);
        if (old == kEmpty) return 1;
        if (old == key) return 0;
        idx = (idx + 1) & mask;
    }
    return 0;
}

// order-preserving map of a float onto unsigned integers (ascending floats -> ascending words)
__device__ __forceinline__ uint32_t f2ord_s(float f) { const uint32_t b = __float_as_uint(f); return (b & 0x80000000u) ? ~b : (b | 0x80000000u); }
__device__ __forceinline__ float ord2f_s(uint32_t o) { return __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o); }
// One result of a shard as the exchange step ships it: (ordered distance, global id) in one word, so that keys of
// different shards compare like (distance, id); an empty pool slot becomes the all-ones word.
__device__ __forceinline__ unsigned long long shard_key(uint32_t local_id, float dis, uint32_t n, uint32_t id_base) {
    return local_id < n ? (((unsigned long long)f2ord_s(dis) << 32) | (unsigned long long)(local_id + id_base)) : ~0ull;
}

#ifndef AP_SCORE_BATCH
#define AP_SCORE_BATCH 2
#endif
constexpr int kScoreBatch = AP_SCORE_BATCH;  // records a warp scores side by side (independent instruction streams)
constexpr int kPerfectMax = 32; // query rows up to this many terms get a collision-free hash table
#ifndef AP_SLOTS_PER_TERM
#define AP_SLOTS_PER_TERM 8
#endif
constexpr uint32_t kSlotsPerTerm = AP_SLOTS_PER_TERM;  // table slots per query term: fewer slots leave more of the CTA's shared memory to the arena

// One section of R staged records against the query row's collision-free table: every lane takes the pairs
// j = lane, lane + 32, ... in ascending order, NS per pass with all loads of a pass in flight together; a miss adds a
// zero product, which leaves the lane's sum as the reference's per-term loop has it.
template <int NS, int R, bool BM>
__device__ __forceinline__ void table_pass(const uint2 *const (&pr)[R], const uint32_t (&cnt)[R], uint32_t nmax, const QRow &q,
                                           uint32_t keymask, int lane, float (&part)[R], uint32_t (&hit)[R]) {
    for (uint32_t j0 = 0; j0 < nmax; j0 += 32 * NS) {
        uint2 pv[R][NS], e[R][NS];
#pragma unroll
        for (int t = 0; t < NS; ++t)
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t j = j0 + 32 * t + lane;
                pv[r][t] = j < cnt[r] ? pr[r][j] : make_uint2(kEmpty, 0u);  // padding never adds to the sum
            }
#pragma unroll
        for (int t = 0; t < NS; ++t)
#pragma unroll
            for (int r = 0; r < R; ++r) e[r][t] = q.tab[(pv[r][t].x * q.mult) >> q.shift];
#pragma unroll
        for (int t = 0; t < NS; ++t)
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const bool match = (e[r][t].x & keymask) == pv[r][t].x;
                part[r] = __fmaf_rn(match ? __uint_as_float(e[r][t].y) : 0.0f, __uint_as_float(pv[r][t].y), part[r]);
                if (BM) hit[r] |= match ? (e[r][t].x >> 31) : 0u;
            }
    }
}

// Fused distances of R records staged in shared memory, computed by a full warp.  Valid in lane 0.
//   dense : HFMA2 in the reference's lane / chunk association (src/query.cu:538-554);
//   sparse: each lane walks the document's pairs j = lane, lane + 32, ... in ascending order, looks the id up in the
//           query row and multiply-adds matches in fp32 -- the per-lane sums of cal_sparse_dist / cal_bm25_dist
//           (include/utils.cuh:299-340).  The lookup is the collision-free table when the row has one (all loads of
//           a 128-term chunk in flight together, misses contribute a zero product, which leaves the sum unchanged),
//           else the reference's own binary search over the query row;
//   then the reference's shfl_down trees and its double-precision `1.0 - dense - sparse`.
template <int F, int R>
__device__ __forceinline__ void score_records(const uint8_t *const (&rec)[R], const uint32_t (&ns)[R], const uint32_t (&nb)[R],
                                              const uint32_t (&qreg)[16], const QRow &qs, const QRow &qb, int lane,
                                              float (&out)[R], uint32_t (&hit)[R]) {
    constexpr bool D = (F & PF_DENSE) != 0, S = (F & PF_SPARSE) != 0, B = (F & PF_BM25) != 0, UNF = (F & PF_UNFUSED) != 0;
    uint32_t acc[R];
    const uint8_t *p[R];
    float tot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) { acc[r] = 0; p[r] = rec[r]; tot[r] = 0.0f; hit[r] = 0; }
    if (D) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint2 v = reinterpret_cast<const uint2 *>(p[r])[lane + 32 * k];
                if (UNF) {
                    acc[r] = hadd2_rn(acc[r], hmul2_rn(qreg[2 * k], v.x));
                    acc[r] = hadd2_rn(acc[r], hmul2_rn(qreg[2 * k + 1], v.y));
                } else {
                    acc[r] = hfma2_rn(qreg[2 * k], v.x, acc[r]);
                    acc[r] = hfma2_rn(qreg[2 * k + 1], v.y, acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) p[r] += kDenseBytes;
    }
#pragma unroll
    for (int sec = 0; sec < 2; ++sec) {
        if ((sec == 0 && !S) || (sec == 1 && !B)) continue;
        const QRow &q = sec == 0 ? qs : qb;
        const uint32_t keymask = sec == 0 ? 0xFFFFFFFFu : 0x7FFFFFFFu;
        const uint2 *pr[R];
        uint32_t cnt[R], nmax = 0;
        float part[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            pr[r] = reinterpret_cast<const uint2 *>(p[r]);
            cnt[r] = sec == 0 ? ns[r] : nb[r];
            nmax = max(nmax, cnt[r]);
            part[r] = 0.0f;
        }
        if (q.mult != 0) {
            // sparse rows average ~120 terms (four per lane and pass), BM25 rows ~60 (two per lane and pass)
            if (sec == 0) table_pass<4, R, false>(pr, cnt, nmax, q, keymask, lane, part, hit);
            else table_pass<2, R, true>(pr, cnt, nmax, q, keymask, lane, part, hit);
        } else if (q.n != 0) {
            // ref: cal_sparse_dist / cal_bm25_dist -- lower bound of the document's id in the query row
            for (uint32_t j = lane; j < nmax; j += 32) {
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (j < cnt[r]) {
                        const uint2 pv = pr[r][j];
                        uint32_t base = 0, n = q.n;
                        while (n > 1) {
                            const uint32_t half = n >> 1;
                            base += ((q.terms[base + half].x & keymask) < pv.x) ? half : 0u;
                            n -= half;
                        }
                        base += ((q.terms[base].x & keymask) < pv.x) ? 1u : 0u;
                        if (base < q.n && (q.terms[base].x & keymask) == pv.x) {
                            part[r] = __fmaf_rn(__uint_as_float(q.terms[base].y), __uint_as_float(pv.y), part[r]);
                            if (sec == 1) hit[r] |= q.terms[base].x >> 31;
                        }
                    }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            tot[r] = (sec == 1 && S) ? __fadd_rn(tot[r], part[r]) : part[r];
            p[r] += 8u * pad2(cnt[r]);
        }
    }
#pragma unroll
    for (int mm = 16; mm > 0; mm >>= 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (D) acc[r] = hadd2_rn(acc[r], __shfl_down_sync(kFull, acc[r], mm));
            if (S || B) tot[r] = __fadd_rn(tot[r], __shfl_down_sync(kFull, tot[r], mm));
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        // the reference writes `1.0 - dense - sparse` with a double literal: the subtraction chain runs in double
        double v = 1.0;
        if (D) v -= (double)half_sum_to_float(acc[r]);
        if (S || B) v -= (double)tot[r];
        out[r] = (float)v;
    }
}

// Collision-free multiplier for a query row of up to 32 terms (one per lane of the calling warp): the first of a
// fixed sequence of odd constants under which all slots differ.  0 when none of 128 candidates works (or the row is
// longer, or holds a repeated id): the caller then scores through the terms.  Fills the (pre-cleared) table.
__device__ __forceinline__ uint32_t build_perfect_table(const uint2 *terms, uint32_t n, uint2 *tab, uint32_t shift, int lane) {
    if (n == 0 || n > (uint32_t)kPerfectMax || shift == 0) return 0;
    const bool on = (uint32_t)lane < n;
    const uint2 t = on ? terms[lane] : make_uint2(0u, 0u);
    const uint32_t key = t.x & 0x7FFFFFFFu;
    uint32_t found = 0, slot = 0;
    for (uint32_t trial = 0; trial < 128 && !found; ++trial) {
        const uint32_t mult = (0x9E3779B1u + trial * 0x3C6EF372u) | 1u;
        slot = on ? ((key * mult) >> shift) : (0x80000000u | (uint32_t)lane);
        const uint32_t grp = __match_any_sync(kFull, slot);
        if (__all_sync(kFull, __popc(grp) == 1)) found = mult;
    }
    if (found && on) tab[slot] = t;
    return found;
}

// The reference's bitonic network on 32 elements held one per lane (include/utils.cuh:147-165 with len = 32):
// the first step of each stage pairs p with its mirror inside the 2*step block, later steps pair p with
// p ^ step; the lower position keeps the smaller key and equal keys never swap.
template <bool EXTRA>
__device__ __forceinline__ void warp_sort32(float &dis, uint32_t &id, uint32_t &e0, uint32_t &e1, int lane) {
#pragma unroll
    for (int stride = 1; stride < 32; stride <<= 1) {
#pragma unroll
        for (int step = stride; step > 0; step >>= 1) {
            const int partner = (step == stride) ? (lane ^ (2 * step - 1)) : (lane ^ step);
            const float od = __shfl_sync(kFull, dis, partner);
            const uint32_t oi = __shfl_sync(kFull, id, partner);
            uint32_t o0 = 0, o1 = 0;
            if (EXTRA) { o0 = __shfl_sync(kFull, e0, partner); o1 = __shfl_sync(kFull, e1, partner); }
            const bool lower = lane < partner;
            const bool take = lower ? (dis > od) : (od > dis);
            if (take) { dis = od; id = oi; if (EXTRA) { e0 = o0; e1 = o1; } }
        }
    }
}

__device__ __forceinline__ uint32_t count_le(const float *arr, uint32_t n, float v) {  // #{arr[i] <= v}, ascending arr
    uint32_t lo = 0, hi = n;
    while (lo < hi) { const uint32_t mid = (lo + hi) >> 1; if (arr[mid] <= v) lo = mid + 1; else hi = mid; }
    return lo;
}
__device__ __forceinline__ uint32_t count_lt(const float *arr, uint32_t n, float v) {  // #{arr[i] < v}
    uint32_t lo = 0, hi = n;
    while (lo < hi) { const uint32_t mid = (lo + hi) >> 1; if (arr[mid] < v) lo = mid + 1; else hi = mid; }
    return lo;
}

// Score the pool slots [base, base + 32) flagged by `need` (lane j of warp 0 owns slot base + j and that
// document's locator word).  The arena is a ring of slots, each holding the records one warp scores side by side
// (kScoreBatch of them, one when the records are too large).  Warp 0 is the producer: for every group of needed
// records, in lane order, it waits until the slot's previous content has been scored ("free" mbarrier), writes the
// group's entry, arms the slot's "filled" mbarrier with the byte count and issues one bulk copy per record (the
// groups that find a free slot at once are issued by all their lanes together).  A consumer warp waits for its
// group's slot to be filled, scores the records out of shared memory and releases the slot.  No CTA-wide barrier
// inside an expansion: slots are refilled one by one as they are released, so all but the slots being scored are in
// flight.
// pool_dis[base + j] receives the distance; keyword hits set bit 30 of pool_id[base + j].
// Called by all threads of the CTA; ends with the CTA synchronised.
template <int F, int NT>
__device__ __forceinline__ void score_slots(const SearchArgs &a, Ctx &c, const uint32_t (&qreg)[16], uint32_t base,
                                            uint64_t my_meta, bool my_need) {
    constexpr bool D = (F & PF_DENSE) != 0, S = (F & PF_SPARSE) != 0, B = (F & PF_BM25) != 0, KW = (F & PF_KEYWORD) != 0;
    static_assert(NT >= 64, "the search CTA needs the producer warp and at least one more warp");
    static_assert(kScoreBatch == 2, "a ring slot holds the two records a warp scores side by side");
    const int lane = c.lane;
    uint32_t need_mask = 0, sz = 0, ns = 0, nb = 0;
    if (c.warp == 0) {
        ns = meta_ns(my_meta); nb = meta_nb(my_meta);
        sz = my_need ? (D ? kDenseBytes : 0u) + (S ? 8u * pad2(ns) : 0u) + (B ? 8u * pad2(nb) : 0u) : 0u;
        need_mask = __ballot_sync(kFull, my_need);
        const uint32_t cnt = __popc(need_mask);
        if (lane == 0) { c.ctl[CTL_NPAIRS] = a.single ? cnt : (cnt + 1u) / 2u; c.ctl[CTL_NEXT] = 0; c.c_eval += cnt; }
    }
    __syncthreads();
    const uint32_t n_groups = c.ctl[CTL_NPAIRS];
    const uint32_t g0 = c.gpair;
    c.gpair = g0 + n_groups;   // the same in every thread
    uint64_t *filled = c.mbar, *freed = c.mbar + kMaxSlots;
    if (c.warp == 0) {
        long long tw = 0;
        if (c.tid == 0) tw = clock64();
        // First wave: the groups that get a slot each without waiting -- whatever those slots held belongs to an
        // earlier expansion, which ended with every group scored -- are armed and issued by all their lanes at once.
        const uint32_t wave = min(n_groups, a.slots);
        const uint32_t below = need_mask & ((1u << lane) - 1u), above = need_mask & ~((2u << lane) - 1u);
        const uint32_t rank = __popc(below);
        const uint32_t grp = a.single ? rank : rank >> 1, second = a.single ? 0u : (rank & 1u);
        const int prev_lane = below ? 31 - __clz(below) : lane, next_lane = above ? __ffs(above) - 1 : lane;
        const uint32_t sz_prev = __shfl_sync(kFull, sz, prev_lane), sz_next = __shfl_sync(kFull, sz, next_lane);
        const bool in_wave = my_need && grp < wave;
        const bool has_partner = !a.single && !second && above != 0u;
        fence_proxy_async();   // the slots were last read by ordinary loads; the copies below write them through the async proxy
        uint32_t w_slot = 0, w_aoff = 0;
        if (in_wave) {
            w_slot = (g0 + grp) % a.slots;
            w_aoff = w_slot * a.slot_bytes + (second ? sz_prev : 0u);
            c.info[2u * w_slot + second] = make_uint2(w_aoff | ((uint32_t)lane << 24), ns | (nb << 16));
            if (!second && !has_partner) c.info[2u * w_slot + 1u] = make_uint2(0xFF000000u, 0u);   // no second record
        }
        __syncwarp();
        if (in_wave && !second) mbar_arrive_expect_tx(c.mbar + w_slot, sz + (has_partner ? sz_next : 0u));
        const uint32_t wave_bytes = __reduce_add_sync(kFull, in_wave ? sz : 0u);
        if (lane == 0) c.c_bytes += wave_bytes;
        __syncwarp();
        if (in_wave && sz) {
            const uint8_t *src = a.rec + meta_off16(my_meta) * 16ull;
            uint8_t *dst = c.arena + w_aoff;
            uint64_t *bar = c.mbar + w_slot;
            const uint32_t ps = 8u * pad2(ns), pb = 8u * pad2(nb);
            if (D && S && B) bulk_g2s(dst, src, kDenseBytes + ps + pb, bar);
            else if (D && S) bulk_g2s(dst, src, kDenseBytes + ps, bar);
            else if (D && B) { bulk_g2s(dst, src, kDenseBytes, bar); if (pb) bulk_g2s(dst + kDenseBytes, src + kDenseBytes + ps, pb, bar); }
            else if (D) bulk_g2s(dst, src, kDenseBytes, bar);
            else if (S && B) { if (ps + pb) bulk_g2s(dst, src + kDenseBytes, ps + pb, bar); }
            else if (S) { if (ps) bulk_g2s(dst, src + kDenseBytes, ps, bar); }
            else { if (pb) bulk_g2s(dst, src + kDenseBytes + ps, pb, bar); }
        }
        // the rest goes slot by slot, as slots are released
        uint32_t rem = need_mask & ~__ballot_sync(kFull, in_wave);
        for (uint32_t p = wave; p < n_groups; ++p) {
            const uint32_t g = g0 + p, slot = g % a.slots, round = g / a.slots;
            const int l0 = __ffs(rem) - 1;
            rem &= rem - 1u;
            int l1 = -1;
            if (!a.single && rem) { l1 = __ffs(rem) - 1; rem &= rem - 1u; }
            const uint32_t sz0 = __shfl_sync(kFull, sz, l0);
            const uint32_t sz1 = __shfl_sync(kFull, sz, l1 < 0 ? l0 : l1);
            const uint32_t total = sz0 + (l1 < 0 ? 0u : sz1);
            if (round != 0) {   // the slot's previous records have been scored
                if (lane == 0) mbar_wait_bounded(freed + slot, (round - 1u) & 1u, a.ctl + 1, 1u);
                __syncwarp();
            }
            fence_proxy_async();   // the slot was last read by ordinary loads; the copies below write it through the async proxy
            const bool mine = lane == l0 || lane == l1;
            const uint32_t aoff = slot * a.slot_bytes + (lane == l1 ? sz0 : 0u);
            if (mine) c.info[2u * slot + (lane == l1 ? 1u : 0u)] = make_uint2(aoff | ((uint32_t)lane << 24), ns | (nb << 16));
            if (l1 < 0 && lane == l0) c.info[2u * slot + 1u] = make_uint2(0xFF000000u, 0u);   // no second record
            __syncwarp();
            if (lane == 0) { mbar_arrive_expect_tx(filled + slot, total); c.c_bytes += total; }
            __syncwarp();
            if (mine && total) {
                const uint8_t *src = a.rec + meta_off16(my_meta) * 16ull;
                uint8_t *dst = c.arena + aoff;
                uint64_t *bar = filled + slot;
                const uint32_t ps = 8u * pad2(ns), pb = 8u * pad2(nb);
                if (D && S && B) bulk_g2s(dst, src, kDenseBytes + ps + pb, bar);
                else if (D && S) bulk_g2s(dst, src, kDenseBytes + ps, bar);
                else if (D && B) { bulk_g2s(dst, src, kDenseBytes, bar); if (pb) bulk_g2s(dst + kDenseBytes, src + kDenseBytes + ps, pb, bar); }
                else if (D) bulk_g2s(dst, src, kDenseBytes, bar);
                else if (S && B) { if (ps + pb) bulk_g2s(dst, src + kDenseBytes, ps + pb, bar); }
                else if (S) { if (ps) bulk_g2s(dst, src + kDenseBytes, ps, bar); }
                else { if (pb) bulk_g2s(dst, src + kDenseBytes + ps, pb, bar); }
            }
        }
        if (c.tid == 0) c.t_wait += clock64() - tw;
    }
    // Consumers.  Latency shape (many warps, an expansion mostly fits the ring): every warp takes the next group that
    // nobody has taken yet -- warp 0 too, once it has issued the last copy.  Throughput shape: warp 0 stays the
    // producer and the groups are dealt round robin to the other warps.
    constexpr bool kDynamic = NT / 32 > 4;
    constexpr uint32_t kConsumers = NT / 32 - 1;
    if (kDynamic || c.warp != 0) {
        for (uint32_t turn = 0;; ++turn) {
            uint32_t p = ((uint32_t)c.warp - 1u) + turn * kConsumers;
            if (kDynamic) {
                if (lane == 0) p = atomicAdd(const_cast<uint32_t *>(&c.ctl[CTL_NEXT]), 1u);
                p = __shfl_sync(kFull, p, 0);
            }
            if (p >= n_groups) break;
            const uint32_t g = g0 + p, slot = g % a.slots, round = g / a.slots;
            if (lane == 0) {
                // the slot's previous round is over (a consumer that runs ahead must not take an earlier phase of the
                // "filled" barrier for its own), then this round's records have landed
                if (round != 0) mbar_wait_bounded(freed + slot, (round - 1u) & 1u, a.ctl + 1, 1u);
                mbar_wait_bounded(filled + slot, round & 1u, a.ctl + 1, 1u);
            }
            __syncwarp();
            const uint8_t *rec[kScoreBatch];
            uint32_t rns[kScoreBatch], rnb[kScoreBatch], hit[kScoreBatch];
            int pslot[kScoreBatch];
            float d[kScoreBatch];
#pragma unroll
            for (int r = 0; r < kScoreBatch; ++r) {
                const uint2 inf = c.info[2u * slot + r];
                const bool valid = (inf.x >> 24) < 32u;
                pslot[r] = valid ? (int)(inf.x >> 24) : -1;
                rec[r] = c.arena + (valid ? (inf.x & 0xFFFFFFu) : slot * a.slot_bytes);
                rns[r] = valid ? (inf.y & 0xFFFFu) : 0u; rnb[r] = valid ? (inf.y >> 16) : 0u;
            }
            score_records<F, kScoreBatch>(rec, rns, rnb, qreg, c.qs, c.qb, lane, d, hit);
#pragma unroll
            for (int r = 0; r < kScoreBatch; ++r) {
                const uint32_t h = KW ? __ballot_sync(kFull, hit[r] != 0) : 0u;
                if (lane == 0 && pslot[r] >= 0) {
                    c.pool_dis[base + pslot[r]] = d[r];
                    if (KW && h) c.pool_id[base + pslot[r]] |= 0x40000000u;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(freed + slot);
        }
    }
    __syncthreads();
}

// Block-wide restatement of the reference's shared-memory bitonic network for an arbitrary length
// (include/utils.cuh:261-280), used once per query by the KG variant to order the seeded pool prefix.
template <int NT>
__device__ __forceinline__ void block_sort_kg(float *dis, uint32_t *id, uint32_t *ent, uint32_t *hop, uint32_t len, int tid) {
    for (uint32_t stride = 1; stride < len; stride <<= 1) {
        for (uint32_t step = stride; step > 0; step >>= 1) {
            for (uint32_t k = tid; k < len / 2; k += NT) {
                const uint32_t aa = 2 * step * (k / step), bb = k % step;
                const uint32_t u = (step == stride) ? (aa + step - 1 - bb) : (aa + bb), d = aa + bb + step;
                if (d < len && dis[u] > dis[d]) {
                    const float td = dis[u]; dis[u] = dis[d]; dis[d] = td;
                    uint32_t t = id[u]; id[u] = id[d]; id[d] = t;
                    t = ent[u]; ent[u] = ent[d]; ent[d] = t;
                    t = hop[u]; hop[u] = hop[d]; hop[d] = t;
                }
            }
            __syncthreads();
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// the search kernel
// ---------------------------------------------------------------------------------------------------------
template <int F, int NT>
__global__ void __launch_bounds__(NT, ctas_for_shape(NT)) search_kernel(const SearchArgs a) {
    constexpr int kMergeMax = (AP_MAX_CANDS + 32 + NT - 1) / NT;
    constexpr bool D = (F & PF_DENSE) != 0, S = (F & PF_SPARSE) != 0, B = (F & PF_BM25) != 0;
    constexpr bool KW = (F & PF_KEYWORD) != 0, KG = (F & PF_KG) != 0;
    constexpr uint32_t IDMASK = KW ? 0x3FFFFFFFu : 0x7FFFFFFFu;

    extern __shared__ __align__(128) uint8_t smem[];
    Ctx c;
    c.mbar = reinterpret_cast<uint64_t *>(smem);
    c.ctl = reinterpret_cast<volatile uint32_t *>(smem + 16 * kMaxSlots);
    c.pool_id = reinterpret_cast<uint32_t *>(smem + a.o_pool_id);
    c.pool_dis = reinterpret_cast<float *>(smem + a.o_pool_dis);
    c.pool_ent = reinterpret_cast<uint32_t *>(smem + a.o_pool_ent);
    c.pool_hop = reinterpret_cast<uint32_t *>(smem + a.o_pool_hop);
    c.vis = reinterpret_cast<uint32_t *>(smem + a.o_vis);
    c.info = reinterpret_cast<uint2 *>(smem + a.o_info);
    c.sq = reinterpret_cast<uint2 *>(smem + a.o_sq);
    c.bq = reinterpret_cast<uint2 *>(smem + a.o_bq);
    c.ts = reinterpret_cast<uint2 *>(smem + a.o_ts);
    c.tb = reinterpret_cast<uint2 *>(smem + a.o_tb);
    c.qs = QRow{c.sq, 0u, c.ts, a.ts_shift, 0u};
    c.qb = QRow{c.bq, 0u, c.tb, a.tb_shift, 0u};
    c.kw_id = reinterpret_cast<uint32_t *>(smem + a.o_kw);
    c.kw_dis = reinterpret_cast<float *>(smem + a.o_kw + 4 * kKeywordRing);
    c.arena = smem + a.o_arena;
    c.tid = threadIdx.x; c.lane = c.tid & 31; c.warp = c.tid >> 5;
    c.gpair = 0; c.c_exp = 0; c.c_eval = 0; c.c_bytes = 0;
    c.t_wait = c.t_score = c.t_ctl = c.t_sort = c.t_merge = c.t_mark = 0;
    const int tid = c.tid, lane = c.lane, warp = c.warp;
    const uint32_t topm = a.cands;
    uint32_t *pool_id = c.pool_id;
    float *pool_dis = c.pool_dis;
    uint32_t *stg_id = pool_id + topm;
    float *stg_dis = pool_dis + topm;

    if (tid == 0) { for (int i = 0; i < 2 * kMaxSlots; ++i) mbar_init(c.mbar + i, 1); mbar_fence_init(); }
    __syncthreads();

    for (;;) {
        if (tid == 0) c.ctl[CTL_QUERY] = atomicAdd(a.ctl, 1u);
        __syncthreads();
        const uint32_t qi = c.ctl[CTL_QUERY];
        if (qi >= a.nq) break;

        // ---- per-query state -----------------------------------------------------------------------------
        for (uint32_t i = tid; i <= a.vis_mask; i += NT) c.vis[i] = kEmpty;
        for (uint32_t i = tid; i < topm + 32; i += NT) {
            pool_id[i] = kEmpty; pool_dis[i] = kInfDis;
            if (KG) { c.pool_ent[i] = kEmpty; c.pool_hop[i] = 0; }
        }
        if (KW && tid < kKeywordRing) { c.kw_id[tid] = 0x3FFFFFFFu; c.kw_dis[tid] = kInfDis; }
        if (tid == 0) c.ctl[CTL_KWNUM] = 0;
        // query: weight folded in fp32, then rounded to half (ref: src/query.cu:1871-1875, 2002)
        uint32_t qreg[16];
        if (D) {
            const float4 *qp = reinterpret_cast<const float4 *>(a.qdense + (size_t)qi * kDim);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float4 f = __ldg(qp + lane + 32 * k);
                qreg[2 * k] = pack_half2(__fmul_rn(f.x, a.w_dense), __fmul_rn(f.y, a.w_dense));
                qreg[2 * k + 1] = pack_half2(__fmul_rn(f.z, a.w_dense), __fmul_rn(f.w, a.w_dense));
            }
        } else {
#pragma unroll
            for (int k = 0; k < 16; ++k) qreg[k] = 0;
        }
        __syncthreads();
        if (S) {
            const uint32_t o = a.qs_off[qi];
            c.qs.n = a.qs_off[qi + 1] - o;
            for (uint32_t j = tid; j < c.qs.n; j += NT)
                c.sq[j] = make_uint2(a.qs_idx[o + j], __float_as_uint(__fmul_rn(a.qs_val[o + j], a.w_sparse)));
            for (uint32_t j = tid; j < a.ts_slots; j += NT) c.ts[j] = make_uint2(kEmpty, 0u);
        }
        if (B) {
            const uint32_t o = a.qb_off[qi];
            c.qb.n = a.qb_off[qi + 1] - o;
            for (uint32_t j = tid; j < c.qb.n; j += NT)
                c.bq[j] = make_uint2(a.qb_idx[o + j], __float_as_uint(__fmul_rn(a.qb_val[o + j], a.w_bm25)));
            for (uint32_t j = tid; j < a.tb_slots; j += NT) c.tb[j] = make_uint2(kEmpty, 0u);
        }
        __syncthreads();
        if (warp == 0) {
            const uint32_t ms = (S && a.ts_slots) ? build_perfect_table(c.sq, c.qs.n, c.ts, a.ts_shift, lane) : 0u;
            const uint32_t mb = (B && a.tb_slots) ? build_perfect_table(c.bq, c.qb.n, c.tb, a.tb_shift, lane) : 0u;
            if (lane == 0) { c.ctl[CTL_MULT_S] = ms; c.ctl[CTL_MULT_B] = mb; }
        }
        __syncthreads();
        c.qs.mult = c.ctl[CTL_MULT_S];
        c.qb.mult = c.ctl[CTL_MULT_B];

        // ---- seeding -------------------------------------------------------------------------------------
        if (!KG) {
            // entry points: all 32 are scored (ref: src/query.cu:440-485)
            uint64_t meta = 0;
            if (warp == 0) {
                const FatEdge e = a.ep_fat[lane];
                vis_insert(c.vis, a.vis_mask, e.id);
                stg_id[lane] = e.id;
                meta = (uint64_t)e.meta_lo | ((uint64_t)e.meta_hi << 32);
            }
            score_slots<F, NT>(a, c, qreg, topm, meta, true);
            if (warp == 0) {
                float d = stg_dis[lane];
                uint32_t id = stg_id[lane], e0 = 0, e1 = 0;
                warp_sort32<false>(d, id, e0, e1, lane);
                stg_id[lane] = id; stg_dis[lane] = d;
                pool_id[lane] = id; pool_dis[lane] = d;
            }
            __syncthreads();
        } else {
            // docs of the query's entities, then entry points, scored and sorted (ref: src/query.cu:1577-1643)
            if (warp == 0) {
                uint32_t nfill = 0;
                if (lane == 0) {
                    for (uint32_t i = a.qe_off[qi]; i < a.qe_off[qi + 1]; ++i) {
                        const uint32_t e = a.qe_idx[i];
                        for (uint32_t j = a.e2d_off[e]; j < a.e2d_off[e + 1]; ++j) {
                            const uint32_t d = a.e2d_idx[j];
                            if (vis_insert(c.vis, a.vis_mask, d) != 0 && nfill < topm + 32) {
                                pool_id[nfill] = d; c.pool_ent[nfill] = e; c.pool_hop[nfill] = 0; ++nfill;
                            }
                        }
                    }
                }
                nfill = __shfl_sync(kFull, nfill, 0);
                if (nfill < topm) {
                    const uint32_t id = a.ep_fat[lane].id;
                    const uint32_t grp = __match_any_sync(kFull, id);
                    const bool leader = (__ffs(grp) - 1) == lane;
                    const bool isnew = leader && vis_insert(c.vis, a.vis_mask, id) != 0;
                    const uint32_t bal = __ballot_sync(kFull, isnew);
                    const uint32_t t = nfill + __popc(bal & ((1u << lane) - 1u));
                    if (isnew && t < topm + 32) { pool_id[t] = id; c.pool_ent[t] = kEmpty; c.pool_hop[t] = 0; }
                    nfill += __popc(bal);
                }
                if (lane == 0) c.ctl[CTL_M] = min(nfill, topm + 32);
            }
            __syncthreads();
            const uint32_t m = c.ctl[CTL_M];
            for (uint32_t cb = 0; cb < m; cb += 32) {
                uint64_t meta = 0; bool need = false;
                if (warp == 0) {
                    need = cb + lane < m;
                    if (need) meta = a.meta[pool_id[cb + lane]];
                }
                score_slots<F, NT>(a, c, qreg, cb, meta, need);
            }
            for (uint32_t i = tid; i < m; i += NT)
                if (c.pool_ent[i] != kEmpty) pool_dis[i] = __fsub_rn(pool_dis[i], a.kg_weight);
            __syncthreads();
            block_sort_kg<NT>(pool_dis, pool_id, c.pool_ent, c.pool_hop, m, tid);
            __syncthreads();
        }

        // ---- greedy iterations (ref: src/query.cu:488-563) ---------------------------------------------------
        for (int it = 0; it < kMaxIter; ++it) {
            if (tid == 0) c.t_mark = clock64();
            if ((it + 1) % kHashReset == 0) {
                for (uint32_t i = tid; i <= a.vis_mask; i += NT) c.vis[i] = kEmpty;
                __syncthreads();
                for (uint32_t i = tid; i < topm + 32; i += NT) vis_insert(c.vis, a.vis_mask, pool_id[i] & IDMASK);
                __syncthreads();
            }
            // first pool entry whose explored bit is clear
            if (warp == 0) {
                uint32_t sel = kEmpty, slot = 0;
                for (uint32_t b0 = 0; b0 < topm; b0 += 32) {
                    const uint32_t id = pool_id[b0 + lane];
                    const uint32_t bal = __ballot_sync(kFull, (id & 0x80000000u) == 0);
                    if (bal) {
                        const int f = __ffs(bal) - 1;
                        sel = __shfl_sync(kFull, id, f);
                        slot = b0 + f;
                        if (lane == f) pool_id[b0 + lane] = id | 0x80000000u;
                        break;
                    }
                }
                if (lane == 0) { c.ctl[CTL_SEL] = sel; c.ctl[CTL_SLOT] = slot; }
            }
            __syncthreads();
            const uint32_t sel = c.ctl[CTL_SEL];
            if (sel == kEmpty) break;
            const uint32_t node = sel & IDMASK;

            // stage the row: ids, visited filter, (keyword refill | KG tagging and augmentation)
            uint64_t my_meta = 0;
            bool my_need = false;
            uint32_t my_ent = kEmpty, my_hop = 0;
            bool my_tag = false;
            if (warp == 0) {
                if (lane == 0) { c.c_exp += 1; c.c_bytes += 32 * sizeof(FatEdge); }
                const FatEdge *row = a.fat + (size_t)node * AP_ROW;
                const uint4 raw_e = __ldg(reinterpret_cast<const uint4 *>(row) + lane);
                uint32_t my_id = raw_e.x;
                my_meta = (uint64_t)raw_e.y | ((uint64_t)raw_e.z << 32);
                {   // duplicates inside a row: the lowest slot is the one that counts as new
                    const uint32_t grp = __match_any_sync(kFull, my_id);
                    const bool leader = (__ffs(grp) - 1) == lane;
                    my_need = leader && vis_insert(c.vis, a.vis_mask, my_id) != 0;
                }
                if (KW) {
                    // visited slots are refilled from the row's keyword edges (ref: src/query.cu:1413-1425)
                    const uint32_t visited = __ballot_sync(kFull, !my_need);
                    const uint32_t t = __popc(visited & ((1u << lane) - 1u));
                    const uint32_t cnt = __ldg(&row[AP_DEGREE].id);
                    const bool part = !my_need && t < cnt;
                    const uint32_t act = __ballot_sync(kFull, part);
                    if (part) {
                        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(row) + AP_DEGREE + 1 + t);
                        const uint32_t grp = __match_any_sync(act, raw.x);
                        const bool leader = (__ffs(grp) - 1) == lane;
                        if (leader && vis_insert(c.vis, a.vis_mask, raw.x) != 0) {
                            my_id = raw.x; my_meta = (uint64_t)raw.y | ((uint64_t)raw.z << 32); my_need = true;
                        }
                    }
                }
                stg_id[lane] = my_id;
                stg_dis[lane] = my_need ? 0.0f : kInfDis;
                if (KG) {
                    const uint32_t slot = c.ctl[CTL_SLOT];
                    const uint32_t hop_cur = c.pool_hop[slot], ent_cur = c.pool_ent[slot];
                    my_hop = hop_cur + 1;
                    c.pool_ent[topm + lane] = kEmpty;
                    c.pool_hop[topm + lane] = my_hop;
                    __syncwarp();
                    if (hop_cur < 3 && ent_cur != kEmpty) {
                        // Logical-edge augmentation (ref: src/query.cu:1697-1735), restated sequentially: docs of
                        // the KG neighbours of the entity that brought this node are tagged when staged, and
                        // already-visited slots are replaced by such docs.
                        if (lane == 0) {
                            const uint32_t e0 = a.e2e_off[ent_cur], e1 = a.e2e_off[ent_cur + 1];
                            for (uint32_t j = e0; j < e1; ++j) {
                                const uint32_t ne = a.e2e_idx[j];
                                for (uint32_t k = a.e2d_off[ne]; k < a.e2d_off[ne + 1]; ++k) {
                                    const uint32_t val = a.e2d_idx[k];
                                    uint32_t tmp = 32, res = 0;
                                    while (tmp > 1) {  // the reference's halving probe over the (unsorted) staged ids
                                        const uint32_t half = tmp / 2;
                                        res += ((stg_id[res + half] & 0x3FFFFFFFu) < val) ? half : 0;
                                        tmp -= half;
                                    }
                                    res += ((stg_id[res] & 0x3FFFFFFFu) < val);
                                    if (res <= 31 && (stg_id[res] & 0x3FFFFFFFu) == val && stg_dis[res] < 1.0f) {
                                        stg_dis[res] = 2.0f;
                                        c.pool_ent[topm + res] = ne;
                                    }
                                }
                            }
                            uint32_t claimed = 0;
                            for (int j = 0; j < 32; ++j) {
                                if (stg_dis[j] > 3.0f) {
                                    const uint32_t t = claimed++;
                                    if (t < e1 - e0) {
                                        const uint32_t ne = a.e2e_idx[e0 + t];
                                        for (uint32_t k = a.e2d_off[ne]; k < a.e2d_off[ne + 1]; ++k) {
                                            const uint32_t cand = a.e2d_idx[k];
                                            if ((sel & 0x3FFFFFFFu) == cand) continue;
                                            if (vis_insert(c.vis, a.vis_mask, cand) != 0) {
                                                stg_id[j] = cand; stg_dis[j] = 2.0f;
                                                c.pool_ent[topm + j] = ne; c.pool_hop[topm + j] = hop_cur + 1;
                                                break;
                                            }
                                        }
                                    }
                                }
                            }
                        }
                        __syncwarp();
                        const uint32_t nid = stg_id[lane];
                        if (nid != my_id) { my_id = nid; my_meta = a.meta[nid]; }
                        const float sd = stg_dis[lane];
                        my_need = sd < 3.0f;
                        my_tag = sd > 1.0f && my_need;
                        my_ent = c.pool_ent[topm + lane];
                    }
                }
            }
            if (tid == 0) { const long long t = clock64(); c.t_ctl += t - c.t_mark; }
            score_slots<F, NT>(a, c, qreg, topm, my_meta, my_need);
            if (tid == 0) c.t_mark = clock64();

            // Order the staged entries for the merge.  Only entries that can enter the pool (distance <= the pool's
            // last) are observable afterwards: the rest is dropped by the merge and overwritten by the next expansion
            // (the visited-set reset uses the staged ids as a set).  No such entry: nothing to do.  Otherwise, when
            // their distances are all different, the reference's bitonic network leaves them in ascending order at the
            // front, which a rank count reproduces; with ties its exact compare-exchange sequence is replayed.
            if (warp == 0) {
                float d = stg_dis[lane];
                uint32_t id = stg_id[lane];
                if (KG && my_tag) d = __fsub_rn(d, __fdiv_rn(a.kg_weight, (float)my_hop));
                const bool q = d <= pool_dis[topm - 1];
                const uint32_t qm = __ballot_sync(kFull, q);
                if (qm != 0) {
                    uint32_t less = 0, eq = 0;
                    for (uint32_t m = qm; m; m &= m - 1) {
                        const float dk = __shfl_sync(kFull, d, __ffs(m) - 1);
                        less += dk < d; eq += dk == d;
                    }
                    if (__any_sync(kFull, q && eq > 1)) {
                        warp_sort32<KG>(d, id, my_ent, my_hop, lane);
                        stg_id[lane] = id; stg_dis[lane] = d;
                        if (KG) { c.pool_ent[topm + lane] = my_ent; c.pool_hop[topm + lane] = my_hop; }
                    } else {
                        const uint32_t pos = q ? less : __popc(qm) + __popc(~qm & ((1u << lane) - 1u));
                        __syncwarp();
                        stg_id[pos] = id; stg_dis[pos] = q ? d : 3.0e38f;
                        if (KG) { c.pool_ent[topm + pos] = my_ent; c.pool_hop[topm + pos] = my_hop; }
                    }
                }
                if (lane == 0) c.ctl[CTL_MERGE] = qm != 0 ? 1u : 0u;
            }
            __syncthreads();
            if (tid == 0) { const long long t = clock64(); c.t_sort += t - c.t_mark; c.t_mark = t; }
            if (c.ctl[CTL_MERGE]) {
                // rank merge (ref: merge_top, src/query.cu:181-224): a pool element moves right by the number of
                // staged elements <= it, a staged element lands at its index plus the number of pool elements < it
                uint32_t r_id[kMergeMax], r_pos[kMergeMax], r_e[kMergeMax], r_h[kMergeMax];
                float r_dis[kMergeMax];
#pragma unroll
                for (int e = 0; e < kMergeMax; ++e) {
                    const uint32_t idx = tid + e * NT;
                    r_pos[e] = kEmpty;
                    if (idx < topm + 32) {
                        r_dis[e] = pool_dis[idx]; r_id[e] = pool_id[idx];
                        if (KG) { r_e[e] = c.pool_ent[idx]; r_h[e] = c.pool_hop[idx]; }
                        r_pos[e] = idx < topm ? idx + count_le(stg_dis, 32, r_dis[e])
                                              : (idx - topm) + count_lt(pool_dis, topm, r_dis[e]);
                    }
                }
                if (KW && warp == 0) {
                    // pool elements pushed out whose id word has bit 0 set go to the side ring, in ascending pool
                    // index (ref: merge_top_keyword, src/query.cu:244-248, `id & 0x40000000 != 0` parses as `id & 1`)
                    const uint32_t idx = topm - 32 + lane;
                    const float v = pool_dis[idx];
                    const uint32_t id = pool_id[idx];
                    const bool ev = (idx + count_le(stg_dis, 32, v) >= topm) && (id & 1u);
                    const uint32_t bal = __ballot_sync(kFull, ev);
                    const uint32_t kn = c.ctl[CTL_KWNUM];
                    if (ev) {
                        const uint32_t s = (kn + __popc(bal & ((1u << lane) - 1u))) % kKeywordRing;
                        c.kw_id[s] = id & 0x3FFFFFFFu; c.kw_dis[s] = v;
                    }
                    __syncwarp();
                    if (lane == 0) c.ctl[CTL_KWNUM] = kn + __popc(bal);
                }
                __syncthreads();
#pragma unroll
                for (int e = 0; e < kMergeMax; ++e)
                    if (r_pos[e] < topm) {
                        pool_id[r_pos[e]] = r_id[e]; pool_dis[r_pos[e]] = r_dis[e];
                        if (KG) { c.pool_ent[r_pos[e]] = r_e[e]; c.pool_hop[r_pos[e]] = r_h[e]; }
                    }
                __syncthreads();
                if (tid == 0) c.t_merge += clock64() - c.t_mark;
            }
        }

        // ---- results (ref: src/query.cu:566-569; keyword ordering :1465-1481) ---------------------------------
        if (!KW) {
            for (uint32_t i = tid; i < topm; i += NT) {
                const uint32_t id = pool_id[i] & 0x7FFFFFFFu;
                const float d = pool_dis[i];
                if (a.out_ids) { a.out_ids[(size_t)qi * topm + i] = id; a.out_dis[(size_t)qi * topm + i] = d; }
                if (a.out_keys && i < a.key_top_k) a.out_keys[(size_t)qi * a.key_top_k + i] = shard_key(id, d, a.n, a.id_base);
            }
        } else {
            if (warp == 0) {
                float d = c.kw_dis[lane];
                uint32_t id = c.kw_id[lane], e0 = 0, e1 = 0;
                warp_sort32<false>(d, id, e0, e1, lane);
                c.kw_id[lane] = id; c.kw_dis[lane] = d;
                uint32_t nout = 0;  // keyword hits first, in pool order
                for (uint32_t b0 = 0; b0 < topm; b0 += 32) {
                    const uint32_t pid = pool_id[b0 + lane];
                    const bool h = (pid & 0x40000000u) != 0;
                    const uint32_t bal = __ballot_sync(kFull, h);
                    if (h) {
                        const uint32_t o = nout + __popc(bal & ((1u << lane) - 1u));
                        if (a.out_ids) { a.out_ids[(size_t)qi * topm + o] = pid & 0x3FFFFFFFu; a.out_dis[(size_t)qi * topm + o] = pool_dis[b0 + lane]; }
                        if (a.out_keys && o < a.key_top_k) a.out_keys[(size_t)qi * a.key_top_k + o] = shard_key(pid & 0x3FFFFFFFu, pool_dis[b0 + lane], a.n, a.id_base);
                    }
                    nout += __popc(bal);
                }
                __syncwarp();
                for (uint32_t i = nout + lane; i < topm; i += 32) {
                    const uint32_t s = i - nout;
                    const uint32_t id = s < kKeywordRing ? (c.kw_id[s] & 0x3FFFFFFFu) : 0x3FFFFFFFu;
                    const float d = s < kKeywordRing ? c.kw_dis[s] : kInfDis;
                    if (a.out_ids) { a.out_ids[(size_t)qi * topm + i] = id; a.out_dis[(size_t)qi * topm + i] = d; }
                    if (a.out_keys && i < a.key_top_k) a.out_keys[(size_t)qi * a.key_top_k + i] = shard_key(id, d, a.n, a.id_base);
                }
            }
        }
        __syncthreads();
    }
    if (tid == 0) {
        atomicAdd(a.cnt + 0, c.c_exp);
        atomicAdd(a.cnt + 1, c.c_eval);
        atomicAdd(a.cnt + 2, c.c_bytes);
        atomicAdd(a.cnt + 3, (unsigned long long)c.t_ctl);
        atomicAdd(a.cnt + 4, (unsigned long long)c.t_wait);
        atomicAdd(a.cnt + 5, (unsigned long long)c.t_score);
        atomicAdd(a.cnt + 6, (unsigned long long)c.t_sort);
        atomicAdd(a.cnt + 7, (unsigned long long)c.t_merge);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Distances of explicit (query, doc) pairs with the same scoring code (test hook): one warp per pair.
// ---------------------------------------------------------------------------------------------------------
template <int F>
__global__ void __launch_bounds__(32) distances_kernel(const SearchArgs a, size_t n_pairs, const uint32_t *pair_q,
                                                       const uint32_t *pair_d, float *out) {
    constexpr bool D = (F & PF_DENSE) != 0, S = (F & PF_SPARSE) != 0, B = (F & PF_BM25) != 0;
    extern __shared__ __align__(128) uint8_t smem[];
    uint2 *sq = reinterpret_cast<uint2 *>(smem + a.o_sq);
    uint2 *bq = reinterpret_cast<uint2 *>(smem + a.o_bq);
    uint2 *ts = reinterpret_cast<uint2 *>(smem + a.o_ts);
    uint2 *tb = reinterpret_cast<uint2 *>(smem + a.o_tb);
    uint8_t *arena = smem + a.o_arena;
    const int lane = threadIdx.x;
    for (size_t p = blockIdx.x; p < n_pairs; p += gridDim.x) {
        const uint32_t qi = pair_q[p], x = pair_d[p];
        uint32_t qreg[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) qreg[k] = 0;
        if (D) {
            const float4 *qp = reinterpret_cast<const float4 *>(a.qdense + (size_t)qi * kDim);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float4 f = __ldg(qp + lane + 32 * k);
                qreg[2 * k] = pack_half2(__fmul_rn(f.x, a.w_dense), __fmul_rn(f.y, a.w_dense));
                qreg[2 * k + 1] = pack_half2(__fmul_rn(f.z, a.w_dense), __fmul_rn(f.w, a.w_dense));
            }
        }
        __syncwarp();
        QRow qs{sq, 0u, ts, a.ts_shift, 0u}, qb{bq, 0u, tb, a.tb_shift, 0u};
        if (S) {
            const uint32_t o = a.qs_off[qi];
            qs.n = a.qs_off[qi + 1] - o;
            for (uint32_t j = lane; j < qs.n; j += 32) sq[j] = make_uint2(a.qs_idx[o + j], __float_as_uint(__fmul_rn(a.qs_val[o + j], a.w_sparse)));
            for (uint32_t j = lane; j < a.ts_slots; j += 32) ts[j] = make_uint2(kEmpty, 0u);
        }
        if (B) {
            const uint32_t o = a.qb_off[qi];
            qb.n = a.qb_off[qi + 1] - o;
            for (uint32_t j = lane; j < qb.n; j += 32) bq[j] = make_uint2(a.qb_idx[o + j], __float_as_uint(__fmul_rn(a.qb_val[o + j], a.w_bm25)));
            for (uint32_t j = lane; j < a.tb_slots; j += 32) tb[j] = make_uint2(kEmpty, 0u);
        }
        __syncwarp();
        // odd pairs go through the table, even pairs through the terms, so both lookups are exercised
        if (S && a.ts_slots && (p & 1)) qs.mult = build_perfect_table(sq, qs.n, ts, a.ts_shift, lane);
        if (B && a.tb_slots && (p & 1)) qb.mult = build_perfect_table(bq, qb.n, tb, a.tb_shift, lane);
        __syncwarp();
        const uint64_t m = a.meta[x];
        const uint32_t ns = meta_ns(m), nb = meta_nb(m);
        const uint4 *src = reinterpret_cast<const uint4 *>(a.rec + meta_off16(m) * 16ull);
        uint4 *dst = reinterpret_cast<uint4 *>(arena);
        uint32_t o = 0;
        if (D) { for (uint32_t i = lane; i < kDenseBytes / 16; i += 32) dst[i] = src[i]; o += kDenseBytes / 16; }
        if (S) { const uint32_t w = pad2(ns) / 2; for (uint32_t i = lane; i < w; i += 32) dst[o + i] = src[kDenseBytes / 16 + i]; o += w; }
        if (B) { const uint32_t w = pad2(nb) / 2; for (uint32_t i = lane; i < w; i += 32) dst[o + i] = src[kDenseBytes / 16 + pad2(ns) / 2 + i]; }
        __syncwarp();
        const uint8_t *rec[1] = {arena};
        const uint32_t rns[1] = {ns}, rnb[1] = {nb};
        uint32_t hit[1];
        float d[1];
        score_records<F, 1>(rec, rns, rnb, qreg, qs, qb, lane, d, hit);
        if (lane == 0) out[p] = d[0];
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
static uint32_t pow2_at_least(uint32_t v) { uint32_t p = 32; while (p < v) p <<= 1; return p; }
static uint32_t log2u(uint32_t p) { uint32_t l = 0; while ((1u << l) < p) ++l; return l; }

static uint32_t layout(SearchArgs &a, const ap_index *ix, uint32_t warps, uint32_t cands, uint32_t flags, uint32_t max_qs, uint32_t max_qb) {
    (void)ix; (void)warps;
    uint32_t o = kHeaderBytes;
    auto take = [&](uint32_t bytes, uint32_t align) { o = (o + align - 1) / align * align; uint32_t r = o; o += bytes; return r; };
    a.o_pool_id = take(4 * (cands + 32), 16);
    a.o_pool_dis = take(4 * (cands + 32), 16);
    a.o_pool_ent = a.o_pool_hop = 0;
    if (flags & PF_KG) { a.o_pool_ent = take(4 * (cands + 32), 16); a.o_pool_hop = take(4 * (cands + 32), 16); }
    const uint32_t vis = (cands + 32 + 3 * 32) * 2 <= 1024 ? 1024u : 2048u;
    a.vis_mask = vis - 1;
    a.o_vis = take(4 * vis, 16);
    a.o_info = take(8 * 2 * kMaxSlots, 16);   // two record entries per ring slot
    a.o_sq = take((flags & PF_SPARSE) ? 8 * std::max(1u, max_qs) : 0, 16);
    a.o_bq = take((flags & PF_BM25) ? 8 * std::max(1u, max_qb) : 0, 16);
    // collision-free tables for short query rows: kSlotsPerTerm slots per term (a multiplier is found within a few
    // trials: 30 terms in 256 slots are collision-free under one random multiplier in six)
    a.ts_slots = ((flags & PF_SPARSE) && max_qs <= (uint32_t)kPerfectMax) ? pow2_at_least(kSlotsPerTerm * std::max(1u, max_qs)) : 0u;
    a.tb_slots = ((flags & PF_BM25) && max_qb <= (uint32_t)kPerfectMax) ? pow2_at_least(kSlotsPerTerm * std::max(1u, max_qb)) : 0u;
    a.ts_shift = a.ts_slots ? 32 - log2u(a.ts_slots) : 0u;
    a.tb_shift = a.tb_slots ? 32 - log2u(a.tb_slots) : 0u;
    a.o_ts = take(8 * a.ts_slots, 16);
    a.o_tb = take(8 * a.tb_slots, 16);
    a.o_kw = take((flags & PF_KEYWORD) ? 8 * kKeywordRing : 0, 16);
    a.o_arena = take(0, 128);
    return a.o_arena;  // fixed bytes before the arena
}

template <int F, int NT>
static int launch_shape(ap_index *ix, SearchArgs &a, uint32_t fixed, uint32_t want_ctas, uint32_t arena_req,
                        uint32_t need_bytes, cudaStream_t stream) {
    // arena: as large as lets `want_ctas` CTAs share one SM, never smaller than the largest record
    uint32_t ctas = want_ctas ? want_ctas : (uint32_t)(NT == kSearchThreads ? kSearchCtas : kLatencyCtas);
    uint32_t arena = 0;
    for (;; --ctas) {
        const size_t per = std::min(ix->smem_per_sm / ctas - 1024, ix->smem_per_block);
        if (per > fixed + need_bytes) { arena = (uint32_t)((per - fixed) / 128 * 128); if (arena >= need_bytes) break; }
        if (ctas == 1) return fail(AP_ERR_LIMIT, "a document record of %u bytes does not fit the shared-memory arena", need_bytes);
    }
    if (arena_req) {
        arena = std::max(need_bytes, arena_req) / 128 * 128 + ((std::max(need_bytes, arena_req) % 128) ? 128 : 0);
        if (fixed + arena > ix->smem_per_block) return fail(AP_ERR_LIMIT, "arena of %u bytes exceeds the per-block shared memory", arena);
    }
    arena = std::min(arena, 512u * 1024u);  // the mbarrier transaction count is 20 bits wide
    a.arena_bytes = arena;
    // ring slots: two records (the largest two fit) per slot when the arena holds at least two such slots, else one
    // record per slot
    {
        const uint32_t pair = (2u * need_bytes + 127u) / 128u * 128u, one = (need_bytes + 127u) / 128u * 128u;
        a.single = arena / pair >= 2u ? 0u : 1u;
        a.slot_bytes = a.single ? one : pair;
        a.slots = std::max(1u, std::min<uint32_t>((uint32_t)kMaxSlots, arena / a.slot_bytes));
    }
    const size_t smem = fixed + arena;
    AP_CUDA(cudaFuncSetAttribute(search_kernel<F, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int occ = 0;
    AP_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, search_kernel<F, NT>, NT, smem));
    if (occ < 1) return fail(AP_ERR_LIMIT, "search kernel does not fit on an SM (%zu bytes of shared memory)", smem);
    const uint32_t grid = (uint32_t)std::min<uint64_t>(a.nq, (uint64_t)occ * ix->num_sms);
    search_kernel<F, NT><<<grid, NT, smem, stream>>>(a);
    AP_CUDA(cudaGetLastError());
    return AP_OK;
}

// Batches that leave SMs empty with one query per CTA take the latency shape (unless the caller fixes the CTA count).
template <int F>
static int launch_one(ap_index *ix, SearchArgs &a, uint32_t fixed, uint32_t want_ctas, uint32_t arena_req,
                      uint32_t need_bytes, cudaStream_t stream) {
    if (kLatencyThreads != kSearchThreads && want_ctas == 0 && a.nq <= (uint32_t)ix->num_sms * kLatencyCtas)
        return launch_shape<F, kLatencyThreads>(ix, a, fixed, 0, arena_req, need_bytes, stream);
    return launch_shape<F, kSearchThreads>(ix, a, fixed, want_ctas, arena_req, need_bytes, stream);
}

static void fill_args(ap_index *ix, const SearchLaunch &L, SearchArgs &a) {
    a.fat = ix->fat; a.ep_fat = ix->ep_fat; a.rec = ix->rec; a.meta = ix->meta; a.n = ix->n;
    a.qdense = L.qdense; a.qs_off = L.qs_off; a.qs_idx = L.qs_idx; a.qs_val = L.qs_val;
    a.qb_off = L.qb_off; a.qb_idx = L.qb_idx; a.qb_val = L.qb_val;
    a.e2e_off = ix->e2e_off; a.e2e_idx = ix->e2e_idx; a.e2d_off = ix->e2d_off; a.e2d_idx = ix->e2d_idx;
    a.qe_off = L.qe_off; a.qe_idx = L.qe_idx;
    a.nq = L.nq; a.w_sparse = L.w_sparse; a.w_bm25 = L.w_bm25; a.w_dense = L.w_dense; a.kg_weight = L.kg_weight;
    a.cands = L.cands; a.out_ids = L.out_ids; a.out_dis = L.out_dis;
    a.out_keys = L.out_keys; a.key_top_k = L.key_top_k; a.id_base = L.id_base;
    a.ctl = L.ctl ? L.ctl : ix->d_ctl; a.cnt = L.cnt ? L.cnt : ix->d_cnt;
}

static int kernel_flags(const SearchLaunch &L) {
    int f = (int)L.path;
    if (L.flags & AP_SEARCH_KEYWORD) f |= PF_KEYWORD;
    if (L.flags & AP_SEARCH_KG) f |= PF_KG;
    if (L.flags & AP_SEARCH_UNFUSED_DENSE) f |= PF_UNFUSED;
    return f;
}

static uint32_t need_bytes_for(const ap_index *ix, int f) {
    // upper bound of one record's staged size for the active paths
    return ((f & PF_DENSE) ? kDenseBytes : 0u) + ((f & PF_SPARSE) ? 8u * pad2(ix->max_ns) : 0u) +
           ((f & PF_BM25) ? 8u * pad2(ix->max_nb) : 0u);
}

#define AP_SEARCH_CASES(X) \
    X(1) X(2) X(3) X(4) X(5) X(6) X(7) X(7 | PF_KEYWORD) X(7 | PF_KG) \
    X(1 | PF_UNFUSED) X(3 | PF_UNFUSED) X(5 | PF_UNFUSED) X(7 | PF_UNFUSED) X(7 | PF_KEYWORD | PF_UNFUSED) X(7 | PF_KG | PF_UNFUSED)

int search_launch(ap_index *ix, const SearchLaunch &L, uint32_t *launches) {
    SearchArgs a{};
    fill_args(ix, L, a);
    int f = kernel_flags(L);
    if (!(f & PF_DENSE)) f &= ~PF_UNFUSED;
    const uint32_t fixed = layout(a, ix, kSearchWarps, L.cands, (uint32_t)f, L.max_qs, L.max_qb);
    const uint32_t need = std::max(16u, need_bytes_for(ix, f));
    AP_CUDA(cudaMemsetAsync(a.ctl, 0, 4, L.stream));  // next-query counter; the error word is sticky
    int rc = AP_ERR_ARG;
    switch (f) {
#define X(FL) case (FL): rc = launch_one<(FL)>(ix, a, fixed, L.ctas_per_sm, L.arena_bytes, need, L.stream); break;
        AP_SEARCH_CASES(X)
#undef X
        default: return fail(AP_ERR_ARG, "unsupported search mode 0x%x (keyword and KG search use all three paths)", f);
    }
    if (rc == AP_OK && launches) *launches += 1;
    return rc;
}

int distances_launch(ap_index *ix, const SearchLaunch &L, size_t n_pairs, const uint32_t *pair_q, const uint32_t *pair_d,
                     float *out) {
    SearchArgs a{};
    fill_args(ix, L, a);
    int f = kernel_flags(L) & (PF_DENSE | PF_SPARSE | PF_BM25 | PF_UNFUSED);
    if (!(f & PF_DENSE)) f &= ~PF_UNFUSED;
    const uint32_t fixed = layout(a, ix, 1, 32, (uint32_t)f, L.max_qs, L.max_qb);
    const size_t smem = fixed + record_bytes(ix->max_ns, ix->max_nb);
    const uint32_t grid = (uint32_t)std::min<size_t>(n_pairs, (size_t)ix->num_sms * 16);
    if (grid == 0) return AP_OK;
    switch (f) {
#define X(FL)                                                                                                        \
    case (FL):                                                                                                       \
        AP_CUDA(cudaFuncSetAttribute(distances_kernel<(FL)>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        distances_kernel<(FL)><<<grid, 32, smem, L.stream>>>(a, n_pairs, pair_q, pair_d, out);                       \
        break;
        X(1) X(2) X(3) X(4) X(5) X(6) X(7) X(1 | PF_UNFUSED) X(3 | PF_UNFUSED) X(5 | PF_UNFUSED) X(7 | PF_UNFUSED)
#undef X
        default: return fail(AP_ERR_ARG, "unsupported distance mode 0x%x", f);
    }
    AP_CUDA(cudaGetLastError());
    return AP_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Gather probe: what the memory system gives this access pattern when nothing else is done with the data.  Same CTA
// count and the same shared-memory budget as the search kernel; warp 0 of every CTA keeps both arena halves filled with
// bulk copies of whole records of pseudo-random documents (the other warps, which would be scoring, idle), for a fixed
// number of batches, refilling a half the moment it has landed.  The bytes moved / the kernel time is the ceiling a
// search over this index can reach in gathered bytes with this footprint; the search itself holds a half while it
// scores it, so it keeps fewer bytes in flight than the probe does.
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kSearchThreads, kSearchCtas) gather_probe_kernel(const uint8_t *__restrict__ rec, const uint64_t *__restrict__ meta,
                                                                                  uint32_t n, uint32_t batches, uint32_t per_batch, uint32_t half_bytes,
                                                                                  uint32_t halves, unsigned long long *bytes_out, uint32_t *err) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *mbar = reinterpret_cast<uint64_t *>(smem);
    uint8_t *arena = smem + 128;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { mbar_init(mbar, 1); mbar_init(mbar + 1, 1); mbar_fence_init(); }
    __syncthreads();
    if (warp != 0) return;
    unsigned long long moved = 0;
    uint32_t phase = 0, counter = blockIdx.x * 0x9E3779B1u;
    // the locator of a lane's next document is read one batch ahead (the search gets it with the graph row), so the
    // probe times the record copies and not a dependent lookup in front of each of them
    auto locator = [&]() -> uint64_t {
        uint32_t x = (counter + (uint32_t)lane) * 0x85EBCA6Bu; x ^= x >> 15; x *= 0x2C1B3C6Du; x ^= x >> 13;
        return meta[x % n];
    };
    uint64_t m_next = (uint32_t)lane < per_batch ? locator() : 0ull;
    auto issue = [&](int h) {
        uint32_t sz = 0;
        const uint8_t *src = nullptr;
        const uint64_t m = m_next;
        counter += per_batch;
        m_next = (uint32_t)lane < per_batch ? locator() : 0ull;
        if ((uint32_t)lane < per_batch) {
            sz = kDenseBytes + 8u * (pad2(meta_ns(m)) + pad2(meta_nb(m)));
            src = rec + meta_off16(m) * 16ull;
        }
        uint32_t incl = sz;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
        const bool fits = sz != 0 && incl <= half_bytes;     // records past the half's capacity are left out of this batch
        const uint32_t bm = __ballot_sync(kFull, fits);
        const uint32_t total = bm ? __shfl_sync(kFull, incl, 31 - __clz(bm)) : 0u;
        if (lane == 0 && total) { mbar_arrive_expect_tx(mbar + h, total); moved += total; }
        __syncwarp();
        if (fits) bulk_g2s(arena + (size_t)h * half_bytes + (incl - sz), src, sz, mbar + h);
        return total != 0;
    };
    bool live[2] = {false, false};
    live[0] = issue(0);
    if (halves == 2) live[1] = issue(1);
    for (uint32_t b = 0; b < batches; ++b) {
        const int h = halves == 2 ? (int)(b & 1u) : 0;
        if (live[h]) {
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(mbar + h, (phase >> h) & 1u, err, 1u);
            ok = __shfl_sync(kFull, ok ? 1 : 0, 0) != 0;
            if (!ok) return;
            phase ^= 1u << h;
        }
        fence_proxy_async();
        live[h] = (b + halves < batches) ? issue(h) : false;
    }
    if (lane == 0) atomicAdd(bytes_out, moved);
}

// ---------------------------------------------------------------------------------------------------------
// Corpus-sharded search: merge the per-shard result lists of every query into a global top-k.  One warp per
// query; the k smallest (distance, id) keys are extracted in ascending order, each round taking the smallest key
// above the previous one (document ids are unique across shards, so keys are distinct).
// ---------------------------------------------------------------------------------------------------------
__global__ void merge_shards_kernel(uint32_t shards, uint32_t nq, uint32_t per, const uint32_t *__restrict__ in_ids,
                                    const float *__restrict__ in_dis, uint32_t top_k, uint32_t *__restrict__ out_ids,
                                    float *__restrict__ out_dis) {
    const uint32_t q = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (q >= nq) return;
    const uint32_t total = shards * per;
    unsigned long long prev = 0;
    bool have_prev = false;
    for (uint32_t r = 0; r < top_k; ++r) {
        unsigned long long best = ~0ull;
        float bd = kInfDis;
        for (uint32_t e = lane; e < total; e += 32) {
            const uint32_t s = e / per, j = e % per;
            const size_t at = ((size_t)s * nq + q) * per + j;
            const float d = in_dis[at];
            const unsigned long long key = ((unsigned long long)f2ord_s(d) << 32) | in_ids[at];
            if ((!have_prev || key > prev) && key < best) { best = key; bd = d; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long ob = __shfl_xor_sync(kFull, best, o);
            const float od = __shfl_xor_sync(kFull, bd, o);
            if (ob < best) { best = ob; bd = od; }
        }
        if (lane == 0) {
            out_ids[(size_t)q * top_k + r] = best == ~0ull ? kEmpty : (uint32_t)best;
            out_dis[(size_t)q * top_k + r] = best == ~0ull ? kInfDis : bd;
        }
        prev = best; have_prev = true;
    }
}

// The same merge on packed keys, as the sharded search ships them (one all-gather of shards x nq x per words): one
// thread per key counts the keys that precede it -- smaller, or equal with a lower position, which only empty slots
// are -- and writes itself to that rank when it is below top_k.  A single pass over shards x per keys per query,
// independent of any order inside the lists.
__global__ void merge_shard_keys_kernel(uint32_t shards, uint32_t nq, uint32_t per, const unsigned long long *__restrict__ keys,
                                        uint32_t top_k, uint32_t *__restrict__ out_ids, float *__restrict__ out_dis) {
    const uint32_t total = shards * per;
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (size_t)nq * total) return;
    const uint32_t q = (uint32_t)(t / total), e = (uint32_t)(t % total);
    const uint32_t s = e / per, j = e % per;
    const unsigned long long mine = keys[((size_t)s * nq + q) * per + j];
    uint32_t rank = 0;
    for (uint32_t s2 = 0; s2 < shards; ++s2) {
        const unsigned long long *row = keys + ((size_t)s2 * nq + q) * per;
        for (uint32_t j2 = 0; j2 < per; ++j2) {
            const unsigned long long other = __ldg(row + j2);
            rank += (other < mine) || (other == mine && s2 * per + j2 < e);
        }
    }
    if (rank < top_k) {
        out_ids[(size_t)q * top_k + rank] = mine == ~0ull ? kEmpty : (uint32_t)mine;
        out_dis[(size_t)q * top_k + rank] = mine == ~0ull ? kInfDis : ord2f_s((uint32_t)(mine >> 32));
    }
}

}  // namespace apoe

extern "C" int ap_merge_shard_keys(int device, uint32_t shards, uint32_t nq, uint32_t per_shard, const unsigned long long *keys,
                                   uint32_t top_k, uint32_t *out_ids, float *out_dis, void *stream) {
    using namespace apoe;
    if (!keys || !out_ids || !out_dis) return fail(AP_ERR_ARG, "null pointer");
    if (shards == 0 || nq == 0 || per_shard == 0 || top_k == 0 || top_k > shards * per_shard) return fail(AP_ERR_ARG, "empty merge or top_k beyond the gathered entries");
    AP_CUDA(cudaSetDevice(device));
    const size_t threads = (size_t)nq * shards * per_shard;
    merge_shard_keys_kernel<<<(uint32_t)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(shards, nq, per_shard, keys, top_k, out_ids, out_dis);
    AP_CUDA(cudaGetLastError());
    return AP_OK;
}

extern "C" int ap_debug_gather_probe(ap_index *ix, uint32_t batches, double *gb_per_s, double *ms_out, unsigned long long *bytes_out) {
    using namespace apoe;
    if (!ix || !gb_per_s) return fail(AP_ERR_ARG, "null argument");
    AP_CUDA(cudaSetDevice(ix->device));
    // the search kernel's shared-memory budget for the three-path search with short query rows
    SearchArgs a{};
    const uint32_t fixed = layout(a, ix, kSearchWarps, 128, 7, 32, 8);
    const uint32_t need = record_bytes(ix->max_ns, ix->max_nb);
    const size_t per = std::min(ix->smem_per_sm / kSearchCtas - 1024, ix->smem_per_block);
    if (per <= fixed + need) return fail(AP_ERR_LIMIT, "records of %u bytes leave no room for the probe's arena", need);
    const uint32_t arena = (uint32_t)std::min<size_t>((per - fixed) / 128 * 128, 512u * 1024u);
    const uint32_t halves = (arena / 2) / 128 * 128 >= need ? 2u : 1u;
    const uint32_t half_bytes = halves == 2 ? (arena / 2) / 128 * 128 : arena;
    const size_t smem = 128 + (size_t)halves * half_bytes;
    AP_CUDA(cudaFuncSetAttribute(gather_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, (size_t)fixed + arena)));
    unsigned long long *d_bytes = ix->d_cnt + 7;
    AP_CUDA(cudaMemset(d_bytes, 0, 8));
    const uint32_t grid = (uint32_t)kSearchCtas * (uint32_t)ix->num_sms;
    AP_CUDA(cudaEventRecord(ix->ev0, 0));
    // Lanes that look a locator up per batch: two more than records of average size fit a half.  Every lookup is a
    // random 8-byte read, which costs the memory system far more than its size, and the search does not make them
    // (a graph row brings the locators of its 32 neighbours in one 512-byte read).
    const uint32_t per_batch = std::min<uint32_t>(32u, (uint32_t)(half_bytes / std::max<size_t>(ix->rec_total / ix->n, 1)) + 2u);
    // the launch asks for the search kernel's full footprint, so the same number of CTAs shares an SM
    gather_probe_kernel<<<grid, kSearchThreads, std::max(smem, (size_t)fixed + arena)>>>(ix->rec, ix->meta, ix->n, batches ? batches : 2000u, per_batch, half_bytes, halves,
                                                                                         d_bytes, ix->d_ctl + 1);
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaEventRecord(ix->ev1, 0));
    AP_CUDA(cudaEventSynchronize(ix->ev1));
    float ms = 0.f;
    AP_CUDA(cudaEventElapsedTime(&ms, ix->ev0, ix->ev1));
    unsigned long long moved = 0;
    AP_CUDA(cudaMemcpy(&moved, d_bytes, 8, cudaMemcpyDeviceToHost));
    uint32_t ew = 0;
    AP_CUDA(cudaMemcpy(&ew, ix->d_ctl + 1, 4, cudaMemcpyDeviceToHost));
    if (ew) { cudaMemset(ix->d_ctl + 1, 0, 4); return fail(AP_ERR_DEVICE, "the gather probe raised error word %u (a bounded wait ran out)", ew); }
    *gb_per_s = (double)moved / (ms * 1e-3) / 1e9;
    if (ms_out) *ms_out = ms;
    if (bytes_out) *bytes_out = moved;
    return AP_OK;
}

extern "C" int ap_merge_shard_results(int device, uint32_t shards, uint32_t nq, uint32_t per_shard, const uint32_t *in_ids,
                                      const float *in_dis, uint32_t top_k, uint32_t *out_ids, float *out_dis, void *stream) {
    using namespace apoe;
    if (!in_ids || !in_dis || !out_ids || !out_dis) return fail(AP_ERR_ARG, "null pointer");
    if (shards == 0 || nq == 0 || per_shard == 0 || top_k == 0) return fail(AP_ERR_ARG, "empty merge");
    AP_CUDA(cudaSetDevice(device));
    merge_shards_kernel<<<(nq + 3) / 4, 128, 0, (cudaStream_t)stream>>>(shards, nq, per_shard, in_ids, in_dis, top_k, out_ids, out_dis);
    AP_CUDA(cudaGetLastError());
    return AP_OK;
}
