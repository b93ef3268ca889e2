// Index construction on the device: hybrid norms, NN-Descent with a local join, RNG-IP pruning with
// keyword-aware neighbour recycling, reverse-edge collection, 40-wide row assembly and entry points.
//
// What is kept from the reference (src/index.cu): the k-NN list width 64, the hybrid distance
// 1 - <x, y> with the dense part scaled by 7 and rounded to half, cal_power's arithmetic (:483-534), and the
// exact semantics of allan_poe (:539-714) and allan_poe_final_graph (:717-807), whose outputs are compared bit
// for bit with the CPU restatement.  What is new is the k-NN construction: instead of 25 rounds of a
// 1 x 512 gather-dot per node (:156-376) every round samples new / old neighbours and their reverses, joins
// the sampled set all-pairs (dense inner products as one 128 x 64 x 1024 tensor-core tile per two nodes, sparse
// and BM25 inner products by hashing one row and probing with the other), proposes the best partners to every
// participant and merges proposals into the sorted lists with a warp bitonic sort.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "apoe_common.cuh"

namespace apoe {

constexpr uint32_t kFull = 0xFFFFFFFFu;
constexpr int kK = AP_KNN;          // 64
constexpr int kSample = 16;         // forward / reverse samples per class (new, old)
constexpr int kPart = 64;           // participants of one local join (the node itself, new, old)
constexpr int kNewMax = 32;         // "new" rows of a join = columns of its distance tile
constexpr int kPropCap = 192;       // proposals a node can receive per round (64 + 192 = one 256-wide merge sort)
constexpr int kPropPerMax = 8;      // upper bound of the partners proposed to each participant of a join
constexpr uint32_t kNewFlag = 0x80000000u;

// ---------------------------------------------------------------------------------------------------------
// norms: ref cal_power, src/index.cu:483-534 -- half squares and half tree sums per 32-chunk of the dense row,
// float squares / tree sums for the sparse and BM25 values (all added onto chunk slot 0), then a left-to-right
// float sum of the 32 slots.
// ---------------------------------------------------------------------------------------------------------
__global__ void norms_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec, float *__restrict__ power) {
    const uint32_t d = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (d >= n) return;
    const uint64_t m = meta[d];
    const uint8_t *r = rec + meta_off16(m) * 16ull;
    const __half *dense = reinterpret_cast<const __half *>(r);
    float slot = 0.0f;  // lane c keeps chunk c's sum
    for (int c = 0; c < 32; ++c) {
        const __half x = dense[c * 32 + lane];
        __half v = __hmul_rn(x, x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = __hadd_rn(v, __shfl_down_sync(kFull, v, o));
        const float s = __half2float(__shfl_sync(kFull, v, 0));
        if ((int)lane == c) slot = s;
    }
    const uint2 *pairs = reinterpret_cast<const uint2 *>(r + kDenseBytes);
    const uint32_t ns = meta_ns(m), nb = meta_nb(m);
    float s0 = __shfl_sync(kFull, slot, 0);
    for (int w = 0; w < 2; ++w) {
        const uint2 *p = w == 0 ? pairs : pairs + pad2(ns);
        const uint32_t cnt = w == 0 ? ns : nb;
        for (uint32_t base = 0; base < cnt; base += 32) {
            const float x = base + lane < cnt ? __uint_as_float(p[base + lane].y) : 0.0f;
            float t = __fmul_rn(x, x);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_down_sync(kFull, t, o));
            s0 = __fadd_rn(s0, __shfl_sync(kFull, t, 0));
        }
    }
    float acc = s0;
    for (int i = 1; i < 32; ++i) acc = __fadd_rn(acc, __shfl_sync(kFull, slot, i));
    if (lane == 0) power[d] = acc;
}

// Largest sparse / BM25 term id of the corpus (warp per document): decides whether the join and pruning tables can
// carry a generation number in the spare high bits of their keys.
__global__ void max_term_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec, uint32_t *__restrict__ out) {
    const uint32_t d = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (d >= n) return;
    const uint64_t m = meta[d];
    const uint2 *pairs = reinterpret_cast<const uint2 *>(rec + meta_off16(m) * 16ull + kDenseBytes);
    const uint32_t ns = meta_ns(m), nb = meta_nb(m), pns = pad2(ns);
    uint32_t mx = 0;
    for (uint32_t j = lane; j < ns; j += 32) mx = max(mx, pairs[j].x);
    for (uint32_t j = lane; j < nb; j += 32) mx = max(mx, pairs[pns + j].x);
    mx = __reduce_max_sync(kFull, mx);
    if (lane == 0 && mx) atomicMax(out, mx);
}

// ---------------------------------------------------------------------------------------------------------
// NN-Descent state
// ---------------------------------------------------------------------------------------------------------
struct Knn {
    uint32_t n;
    uint32_t *ids;   // n x 64, bit 31 = not yet sampled ("new")
    float *dis;      // n x 64 ascending
    uint32_t *samp;  // n x 64: [new fwd 16 | new rev 16 | old fwd 16 | old rev 16]
    uint32_t *scnt;  // n x 4 counts of the above (reverse counts may exceed the capacity)
    uint32_t *plist; // n x 64 participants of the node's join (the node first, then new, then old)
    uint32_t *pcnt;  // n x 2: rows that are new, rows in total
    uint2 *prop;     // n x kPropCap (distance bits, id)
    uint32_t *propn; // n
    unsigned long long *stats;  // [0] distance evaluations, [1] list updates, [2] proposal overflows, [3] records gathered by the joins
    uint32_t det;    // deterministic mode: reverse samples and proposals are kept by key, not by arrival (see offer_proposal)
};

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}
// mix32 is a bijection of the 32-bit words; this is its inverse (the multipliers' inverses modulo 2^32)
__device__ __forceinline__ uint32_t unmix32(uint32_t x) {
    x ^= x >> 16; x *= 0x43021123u; x = x ^ (x >> 15) ^ (x >> 30); x *= 0x1d69e2a5u; x ^= x >> 16;
    return x;
}
__device__ __forceinline__ uint32_t f2ord(float f);

// A proposal (distance d to document `other`) for `target`'s list.
//   default: appended to the target's inbox in arrival order; the inbox holds kPropCap entries per round, later ones
//            are dropped (counted in stats[2]) -- which ones depends on the order the CTAs happen to run in;
//   deterministic: the inbox is a table of kPropCap slots, a proposal goes to the slot its source id hashes to and the
//            smallest (distance, id) word per slot survives (64-bit atomicMin).  The outcome is a function of the set
//            of proposals alone; repeated proposals of one pair collapse, different sources that share a slot
//            compete and the closer one stays.  Entry layout in this mode: x = id, y = ordered distance bits.
__device__ __forceinline__ void offer_proposal(uint32_t det, uint2 *prop, uint32_t *propn, unsigned long long *stats,
                                               uint32_t target, float d, uint32_t other) {
    if (det) {
        const unsigned long long key = ((unsigned long long)f2ord(d) << 32) | other;
        atomicMin(reinterpret_cast<unsigned long long *>(prop + (size_t)target * kPropCap + mix32(other ^ 0x2545F491u) % (uint32_t)kPropCap), key);
        atomicAdd(&propn[target], 1u);
        return;
    }
    const uint32_t t = atomicAdd(&propn[target], 1u);
    if (t < (uint32_t)kPropCap) prop[(size_t)target * kPropCap + t] = make_uint2(__float_as_uint(d), other);
    else if (stats) atomicAdd(stats + 2, 1ull);
}

// Pair ownership: an evaluated pair is offered to exactly one of its ends, chosen by a hash of the two ids, unless
// `shared` asks for both.  A document's list then holds its nearest among the pairs it owns, the other pairs reach it
// as reverse edges of the final rows.
__device__ __forceinline__ bool pair_owned(uint32_t shared, uint32_t me, uint32_t other) {
    if (shared) return true;
    const uint32_t lo = min(me, other), hi = max(me, other), h = mix32(lo * 0x9e3779b1u + hi);
    return (h & 1u) ? me < other : me > other;
}

// Random initial lists: 64 distinct ids != v with distance 1e6 and the "new" flag (ref: initialize_graph,
// src/index.cu:99-106, seeded there from clock(); here from `seed` so a build is repeatable).
__global__ void knn_init_kernel(Knn k, uint32_t seed) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k.n * (uint32_t)kK) return;
    const uint32_t v = i / kK, s = i % kK, n = k.n;
    uint32_t id;
    if (n <= (uint32_t)kK + 1) id = (v + 1 + s % (n - 1)) % n;  // tiny corpora: duplicates are unavoidable
    else {
        const uint32_t span = n - 1, step_max = span / kK;
        const uint32_t a = 1 + mix32(seed ^ (v * 2654435761u)) % step_max, b = mix32(seed + 0x9e3779b9u + v) % span;
        id = (v + 1 + (uint32_t)(((uint64_t)b + (uint64_t)s * a) % span)) % n;
    }
    k.ids[i] = id | kNewFlag;
    k.dis[i] = kInfDis;
}

__device__ __forceinline__ void jtab_insert(uint2 *tab, uint32_t mask, uint32_t shift, uint32_t key, uint32_t valbits);
__device__ __forceinline__ uint32_t f2ord(float f);
__device__ __forceinline__ float ord2f(uint32_t o);

// ---------------------------------------------------------------------------------------------------------
// Term-seeded start.  The hybrid distance of two documents is dominated by the BM25 weights of the rare terms
// they share, so before the first round every document meets the documents next to it in the posting lists of
// its rarest BM25 terms: the (term, document) pairs of the corpus are radix-sorted into postings, each document
// takes up to `take` followers from its rarest postings until it has 64 candidates, their distances are
// evaluated directly and offered to both sides, and a merge turns the offers into the first sorted lists.
// (The reference starts from random lists only, src/index.cu:99-106; random entries stay behind the seeds.)
// ---------------------------------------------------------------------------------------------------------
__global__ void inv_count_kernel(uint32_t n, const uint64_t *__restrict__ meta, uint32_t *__restrict__ cnt, unsigned long long *__restrict__ total) {
    __shared__ unsigned long long part;
    if (threadIdx.x == 0) part = 0;
    __syncthreads();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t c = i < n ? meta_nb(meta[i]) : 0u;
    if (i <= n) cnt[i] = c;
    if (c) atomicAdd(&part, (unsigned long long)c);
    __syncthreads();
    if (threadIdx.x == 0 && part) atomicAdd(total, part);   // 64-bit count of all postings
}
__global__ void inv_keys_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec,
                                const uint32_t *__restrict__ off, unsigned long long *__restrict__ keys) {
    const uint32_t d = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (d >= n) return;
    const uint64_t m = meta[d];
    const uint2 *pr = reinterpret_cast<const uint2 *>(rec + meta_off16(m) * 16ull + kDenseBytes) + pad2(meta_ns(m));
    unsigned long long *out = keys + off[d];
    for (uint32_t j = lane; j < meta_nb(m); j += 32) out[j] = ((unsigned long long)pr[j].x << 32) | d;
}
__device__ __forceinline__ uint32_t lower_bound_u64(const unsigned long long *__restrict__ a, uint32_t lo, uint32_t hi, unsigned long long key) {
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (__ldg(a + mid) < key) lo = mid + 1; else hi = mid;
    }
    return lo;
}
constexpr int kSeedTermsPerLane = 4;   // the first 128 BM25 terms of a document are considered
__global__ void seed_cand_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec,
                                 const unsigned long long *__restrict__ keys, uint32_t total, uint32_t take,
                                 uint32_t *__restrict__ cand) {
    const uint32_t v = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (v >= n) return;
    const uint64_t m = meta[v];
    const uint32_t nb = meta_nb(m);
    const uint2 *pr = reinterpret_cast<const uint2 *>(rec + meta_off16(m) * 16ull + kDenseBytes) + pad2(meta_ns(m));
    uint32_t lo[kSeedTermsPerLane], df[kSeedTermsPerLane], term[kSeedTermsPerLane];
#pragma unroll
    for (int t = 0; t < kSeedTermsPerLane; ++t) {
        const uint32_t j = lane + 32 * t;
        lo[t] = 0; df[t] = kEmpty; term[t] = 0;
        if (j < nb) {
            term[t] = pr[j].x;
            lo[t] = lower_bound_u64(keys, 0, total, (unsigned long long)term[t] << 32);
            const uint32_t hi = lower_bound_u64(keys, lo[t], total, ((unsigned long long)term[t] + 1ull) << 32);
            df[t] = hi - lo[t] >= 2 ? hi - lo[t] : kEmpty;   // a posting of one document (this one) seeds nothing
        }
    }
    uint32_t cnt = 0;
    while (cnt < (uint32_t)kK) {
        unsigned long long best = ~0ull;   // (df, slot, lane), smallest first
#pragma unroll
        for (int t = 0; t < kSeedTermsPerLane; ++t) {
            const unsigned long long c = ((unsigned long long)df[t] << 8) | ((unsigned long long)t << 5) | lane;
            best = c < best ? c : best;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(kFull, best, o);
            best = other < best ? other : best;
        }
        const uint32_t DF = (uint32_t)(best >> 8);
        if (DF == kEmpty) break;
        const uint32_t owner = (uint32_t)best & 31u, slot = ((uint32_t)best >> 5) & 3u;
        uint32_t my_lo = lo[0], my_term = term[0];
#pragma unroll
        for (int t = 1; t < kSeedTermsPerLane; ++t) if (slot == (uint32_t)t) { my_lo = lo[t]; my_term = term[t]; }
        const uint32_t L = __shfl_sync(kFull, my_lo, owner), T = __shfl_sync(kFull, my_term, owner);
        if (lane == owner) {
#pragma unroll
            for (int t = 0; t < kSeedTermsPerLane; ++t) if (slot == (uint32_t)t) df[t] = kEmpty;
        }
        const uint32_t p = lower_bound_u64(keys, L, L + DF, ((unsigned long long)T << 32) | v) - L;
        const uint32_t tk = min(min(DF - 1u, take), (uint32_t)kK - cnt);
        if (lane < tk) cand[(size_t)v * kK + cnt + lane] = (uint32_t)__ldg(keys + L + (p + 1u + lane) % DF);
        cnt += tk;
    }
    for (uint32_t j = cnt + lane; j < (uint32_t)kK; j += 32) cand[(size_t)v * kK + j] = kEmpty;
}

// Distances of every document to its seed candidates, one warp per document: the document's sparse and BM25
// terms go into a per-warp hash table, its dense row into registers, each candidate's record is read once.
constexpr int kSeedWarps = 4;
__global__ void __launch_bounds__(kSeedWarps * 32) seed_dist_kernel(Knn k, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec,
                                                                   const uint32_t *__restrict__ cand, uint32_t tab_mask, uint32_t tab_shift, uint32_t shared_pairs) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t v = blockIdx.x * kSeedWarps + warp;
    if (v >= k.n) return;
    uint2 *tab = reinterpret_cast<uint2 *>(smem) + (size_t)warp * (tab_mask + 1);
    for (uint32_t i = lane; i <= tab_mask; i += 32) tab[i] = make_uint2(kEmpty, 0u);
    __syncwarp();
    const uint64_t m = meta[v];
    const uint8_t *r = rec + meta_off16(m) * 16ull;
    {
        const uint2 *pr = reinterpret_cast<const uint2 *>(r + kDenseBytes);
        const uint32_t ns = meta_ns(m), nb = meta_nb(m), pns = pad2(ns);
        for (uint32_t j = lane; j < ns + nb; j += 32) {
            const uint2 p = j < ns ? pr[j] : pr[pns + (j - ns)];
            jtab_insert(tab, tab_mask, tab_shift, j < ns ? p.x : (p.x | 0x80000000u), p.y);
        }
    }
    uint4 a[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) a[q] = __ldg(reinterpret_cast<const uint4 *>(r) + lane + 32 * q);
    __syncwarp();
    unsigned long long evals = 0;
    for (int j = 0; j < kK; ++j) {
        const uint32_t c = cand[(size_t)v * kK + j];
        if (c >= k.n || c == v) continue;
        const uint64_t cm = meta[c];
        const uint8_t *cr = rec + meta_off16(cm) * 16ull;
        float acc = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 b = __ldg(reinterpret_cast<const uint4 *>(cr) + lane + 32 * q);
            const uint32_t aw[4] = {a[q].x, a[q].y, a[q].z, a[q].w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&aw[w]));
                const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&bw[w]));
                acc = fmaf(fa.x, fb.x, acc); acc = fmaf(fa.y, fb.y, acc);
            }
        }
        const uint2 *pr = reinterpret_cast<const uint2 *>(cr + kDenseBytes);
        const uint32_t ns = meta_ns(cm), nb = meta_nb(cm), pns = pad2(ns);
        for (uint32_t q = lane; q < ns + nb; q += 32) {
            const uint2 p = q < ns ? __ldg(pr + q) : __ldg(pr + pns + (q - ns));
            const uint32_t key = q < ns ? p.x : (p.x | 0x80000000u);
            uint32_t h = (key * 2654435761u) >> tab_shift;
            for (uint32_t s = 0; s <= tab_mask; ++s) {
                const uint2 e = tab[h];
                if (e.x == kEmpty) break;
                if (e.x == key) { acc = fmaf(__uint_as_float(e.y), __uint_as_float(p.y), acc); break; }
                h = (h + 1) & tab_mask;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
        if (lane == 0) {
            const float d = 1.0f - acc;
            if (pair_owned(shared_pairs, v, c)) offer_proposal(k.det, k.prop, k.propn, nullptr, v, d, c);
            if (pair_owned(shared_pairs, c, v)) offer_proposal(k.det, k.prop, k.propn, nullptr, c, d, v);
        }
        ++evals;
    }
    if (lane == 0 && evals) atomicAdd(k.stats + 0, evals);
}

// Sampling: the closest 16 unsampled ("new") entries and a random 16 of the sampled ("old") entries of every list,
// plus the reverse of those choices.  Sampled new entries lose their flag.  Old entries are drawn at random so
// that over the rounds every old neighbour meets the new ones.
__global__ void knn_sample_kernel(Knn k, uint32_t round) {
    const uint32_t v = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (v >= k.n) return;
    uint32_t raw[2];
    raw[0] = k.ids[(size_t)v * kK + lane];
    raw[1] = k.ids[(size_t)v * kK + 32 + lane];
    const uint32_t bn0 = __ballot_sync(kFull, (raw[0] & kNewFlag) != 0), bn1 = __ballot_sync(kFull, (raw[1] & kNewFlag) != 0);
    const uint32_t n_old = 64 - __popc(bn0) - __popc(bn1);
    // keep an old entry with probability 16 / n_old (hash of node, round and slot)
    const uint32_t thresh = n_old <= (uint32_t)kSample ? 0xFFFFFFFFu : (uint32_t)(((unsigned long long)kSample << 32) / n_old);
    uint32_t nn = 0, no = 0;
    for (int h = 0; h < 2; ++h) {
        const uint32_t slot = h * 32 + lane;
        const bool isnew = (raw[h] & kNewFlag) != 0;
        const uint32_t id = raw[h] & ~kNewFlag;
        const bool oldpick = !isnew && mix32((v * 64u + slot) ^ (round * 0x9e3779b9u) ^ 0x5bd1e995u) <= thresh;
        const uint32_t bn = h == 0 ? bn0 : bn1, bo = __ballot_sync(kFull, oldpick);
        const uint32_t rn = nn + __popc(bn & ((1u << lane) - 1u)), ro = no + __popc(bo & ((1u << lane) - 1u));
        if (isnew && rn < kSample && id < k.n) {
            k.samp[(size_t)v * 64 + rn] = id;
            k.ids[(size_t)v * kK + slot] = id;  // now "old"
            if (k.det) {   // the slot this source hashes to keeps the smallest scrambled source id (decoded by knn_rev_decode_kernel)
                const uint32_t scr = mix32(v ^ (round * 0x9e3779b9u));
                if (scr != kEmpty) atomicMin(&k.samp[(size_t)id * 64 + 16 + (mix32(v + 0x632BE5ABu) & 15u)], scr);
            } else {
                const uint32_t t = atomicAdd(&k.scnt[(size_t)id * 4 + 1], 1u);
                if (t < kSample) k.samp[(size_t)id * 64 + 16 + t] = v;
                else { const uint32_t r = mix32(v ^ (round * 0x9e3779b9u) ^ t) % (t + 1); if (r < kSample) k.samp[(size_t)id * 64 + 16 + r] = v; }
            }
        }
        if (oldpick && ro < kSample && id < k.n) {
            k.samp[(size_t)v * 64 + 32 + ro] = id;
            if (k.det) {
                const uint32_t scr = mix32(v ^ (round * 0x9e3779b9u));
                if (scr != kEmpty) atomicMin(&k.samp[(size_t)id * 64 + 48 + (mix32(v + 0x632BE5ABu) & 15u)], scr);
            } else {
                const uint32_t t = atomicAdd(&k.scnt[(size_t)id * 4 + 3], 1u);
                if (t < kSample) k.samp[(size_t)id * 64 + 48 + t] = v;
                else { const uint32_t r = mix32(v ^ (round * 0x85ebca6bu) ^ t) % (t + 1); if (r < kSample) k.samp[(size_t)id * 64 + 48 + r] = v; }
            }
        }
        nn += __popc(bn); no += __popc(bo);
    }
    if (lane == 0) { k.scnt[(size_t)v * 4 + 0] = min(nn, (uint32_t)kSample); k.scnt[(size_t)v * 4 + 2] = min(no, (uint32_t)kSample); }
}

// Deterministic mode: the reverse-sample slots hold scrambled source ids (or 0xFFFFFFFF); turn them back into ids and
// set the reverse counts to the slot count (empty slots are skipped by knn_plist_kernel's id check).
__global__ void knn_rev_decode_kernel(Knn k, uint32_t round) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k.n * 32u) return;
    const uint32_t v = i >> 5, s = i & 31u, slot = s < 16 ? 16 + s : 32 + s;   // [16, 32) and [48, 64)
    const uint32_t x = k.samp[(size_t)v * 64 + slot];
    if (x != kEmpty) k.samp[(size_t)v * 64 + slot] = unmix32(x) ^ (round * 0x9e3779b9u);
    if (s == 0) { k.scnt[(size_t)v * 4 + 1] = kSample; k.scnt[(size_t)v * 4 + 3] = kSample; }
}

// Participants of v's join: v itself, then the distinct new samples, then the distinct old samples not already
// present; at most 32 new rows and 64 rows in total.  One warp per node.
__global__ void knn_plist_kernel(Knn k, const uint64_t *__restrict__ meta, uint32_t arena_bytes) {
    const uint32_t v = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (v >= k.n) return;
    __shared__ uint32_t sh[8][kPart];
    uint32_t *pl = sh[(threadIdx.x >> 5)];
    const uint32_t *sm = k.samp + (size_t)v * 64;
    const uint32_t c0 = k.scnt[(size_t)v * 4 + 0], c1 = min(k.scnt[(size_t)v * 4 + 1], (uint32_t)kSample);
    const uint32_t c2 = k.scnt[(size_t)v * 4 + 2], c3 = min(k.scnt[(size_t)v * 4 + 3], (uint32_t)kSample);
    if (lane == 0) pl[0] = v;
    __syncwarp();
    uint32_t cnt = 1, n_new = 1;
    for (int cls = 0; cls < 2; ++cls) {
        const uint32_t na = cls == 0 ? c0 : c2, nb = cls == 0 ? c1 : c3, base = cls * 32;
        const uint32_t cap = cls == 0 ? (uint32_t)kNewMax : (uint32_t)kPart;
        // lane l < 16: forward sample l, lane l >= 16: reverse sample l - 16
        const bool have = lane < 16 ? lane < na : (lane - 16) < nb;
        const uint32_t id = have ? sm[base + lane] : kEmpty;
        bool ok = have && id < k.n;
        for (uint32_t j = 0; ok && j < cnt; ++j) ok = pl[j] != id;         // not yet a participant
        const uint32_t grp = __match_any_sync(kFull, id);
        ok = ok && (__ffs(grp) - 1) == (int)lane;                          // first of equal ids in this batch
        const uint32_t bal = __ballot_sync(kFull, ok);
        const uint32_t pos = cnt + __popc(bal & ((1u << lane) - 1u));
        if (ok && pos < cap) pl[pos] = id;
        cnt = min(cnt + __popc(bal), cap);
        if (cls == 0) n_new = cnt;
        __syncwarp();
    }
    // Participants whose sparse sections would not fit the join's staging area are cut off here already (from the
    // end, as the join kernel itself would do), so that their dense rows are not gathered for nothing.
    {
        uint32_t fit = cnt, run = 0;
        for (uint32_t b0 = 0; b0 < cnt; b0 += 32) {
            const uint32_t j = b0 + lane;
            uint32_t sz = 0;
            if (j < cnt) { const uint64_t m = meta[pl[j]]; sz = 8u * (pad2(meta_ns(m)) + pad2(meta_nb(m))); }
            uint32_t incl = sz;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if ((int)lane >= o) incl += t; }
            const uint32_t over = __ballot_sync(kFull, j < cnt && run + incl > arena_bytes);
            if (over) { fit = b0 + (uint32_t)__ffs(over) - 1u; break; }
            run += __shfl_sync(kFull, incl, 31);
        }
        cnt = fit; n_new = min(n_new, cnt);
    }
    for (uint32_t j = lane; j < kPart; j += 32) k.plist[(size_t)v * kPart + j] = j < cnt ? pl[j] : kEmpty;
    if (lane == 0) { k.pcnt[(size_t)v * 2] = n_new; k.pcnt[(size_t)v * 2 + 1] = cnt; }
}

// ---------------------------------------------------------------------------------------------------------
// Join, dense part on CUDA cores: D[v][j][i] = <dense(plist[j]), dense(plist[i])>, j < rows, i < n_new, fp32
// accumulation of half products.  The tensor-core kernel in apoe_join_tc.cu fills the same scratch layout.
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256, 2) join_dense_simt_kernel(uint32_t node0, uint32_t nodes, const uint32_t *__restrict__ plist,
                                                              const uint32_t *__restrict__ pcnt, const uint64_t *__restrict__ meta,
                                                              const uint8_t *__restrict__ rec, float *__restrict__ D) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint4 *newrows = reinterpret_cast<uint4 *>(smem);  // 32 rows x 128 uint4
    const uint32_t local = blockIdx.x;
    if (local >= nodes) return;
    const uint32_t v = node0 + local;
    const uint32_t n_new = pcnt[(size_t)v * 2], rows = pcnt[(size_t)v * 2 + 1];
    if (n_new <= 1 && rows <= 1) return;
    const uint32_t *pl = plist + (size_t)v * kPart;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t idx = tid; idx < n_new * 128; idx += 256) {
        const uint32_t i = idx >> 7, c = idx & 127;
        const uint4 *src = reinterpret_cast<const uint4 *>(rec + meta_off16(meta[pl[i]]) * 16ull);
        newrows[idx] = __ldg(src + c);
    }
    __syncthreads();
    float *out = D + (size_t)local * kPart * kNewMax;
    for (uint32_t j = warp; j < rows; j += 8) {
        const uint4 *src = reinterpret_cast<const uint4 *>(rec + meta_off16(meta[pl[j]]) * 16ull);
        uint4 a[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] = __ldg(src + lane + 32 * k);
        float vals[kNewMax];
#pragma unroll
        for (int i = 0; i < kNewMax; ++i) {
            float acc = 0.0f;
            if ((uint32_t)i < n_new) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint4 b = newrows[i * 128 + lane + 32 * k];
                    const uint32_t aw[4] = {a[k].x, a[k].y, a[k].z, a[k].w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&aw[q]));
                        const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&bw[q]));
                        acc = fmaf(fa.x, fb.x, acc); acc = fmaf(fa.y, fb.y, acc);
                    }
                }
            }
            vals[i] = acc;
        }
        // 32 warp sums in 31 shuffles: lane l ends up with the total of vals[l]
#pragma unroll
        for (int o = 16, len = 32; o >= 1; o >>= 1, len >>= 1) {
#pragma unroll
            for (int q = 0; q < len / 2; ++q) {
                const bool up = (lane & o) != 0;
                const float keep = up ? vals[q + len / 2] : vals[q];
                const float send = up ? vals[q] : vals[q + len / 2];
                vals[q] = keep + __shfl_xor_sync(kFull, send, o);
            }
        }
        out[(size_t)j * kNewMax + lane] = vals[0];
    }
}

// ---------------------------------------------------------------------------------------------------------
// Two-choice (cuckoo) term tables in shared memory, G tables side by side.  Every key of a hashed row sits in one of
// its two hashed slots, so a lookup is two loads and two compares with no branch -- this matters because a warp
// probes 100+ keys per step and a rarely taken chain walk would be taken by some lane every time.  The G tables of
// a group share the hash functions and are interleaved: slot h is one line of G keys (K[h * G + g]) and one line of
// G value words (V[h * G + g]); a probe fetches the key line of all G tables in one vector load and touches V only
// on a match, which halves the shared-memory wavefronts against G separate (key, value) tables.  Empty: key
// 0xFFFFFFFF, value 0.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ck_h1(uint32_t key, uint32_t shift) { return (key * 2654435761u) >> shift; }
__device__ __forceinline__ uint32_t ck_h2(uint32_t key, uint32_t shift) { return ((key ^ 0x5bd1e995u) * 0x85ebca6bu + 0x1b873593u) >> shift; }
// Lock-free key insertion by eviction into table g; false when the kick budget runs out (the caller gives the row up).
// Generations: when the ids leave their high bits free, the keys of one pass carry the pass number there (gen_mask
// selects those bits, the key holds the current number).  A slot whose key carries another number is left over
// from an earlier pass: an insertion takes it as if it were empty and no probe can match it, so the tables are
// never emptied between passes.  gen_mask = 0: plain keys, tables wiped by the caller.
template <int G>
__device__ __forceinline__ bool ck_insert_key(uint32_t *K, uint32_t g, uint32_t shift, uint32_t key, uint32_t gen_mask = 0u) {
    const uint32_t gen = key & gen_mask;
    uint32_t h = ck_h1(key, shift);
    for (int kick = 0; kick < 48; ++kick) {
        const uint32_t old = atomicExch(K + h * G + g, key);
        if (old == kEmpty || (old & gen_mask) != gen) return true;
        key = old;
        const uint32_t a1 = ck_h1(key, shift), a2 = ck_h2(key, shift);
        h = h == a1 ? a2 : a1;
    }
    return false;
}
// After all keys of table g are placed: the value goes where its key ended up.
template <int G>
__device__ __forceinline__ uint32_t ck_store_value(const uint32_t *K, uint32_t *V, uint32_t g, uint32_t shift, uint32_t key, uint32_t valbits) {
    const uint32_t h1 = ck_h1(key, shift), h2 = ck_h2(key, shift);
    const uint32_t h = K[h1 * G + g] == key ? h1 : (K[h2 * G + g] == key ? h2 : kEmpty);
    if (h != kEmpty) V[h * G + g] = valbits;
    return h;   // the slot, 0xFFFFFFFF when the key was given up
}
template <int G> struct KeyLine;
template <> struct KeyLine<4> { static __device__ __forceinline__ void load(const uint32_t *K, uint32_t h, uint32_t (&k)[4]) { const uint4 v = *reinterpret_cast<const uint4 *>(K + h * 4); k[0] = v.x; k[1] = v.y; k[2] = v.z; k[3] = v.w; } };
template <> struct KeyLine<2> { static __device__ __forceinline__ void load(const uint32_t *K, uint32_t h, uint32_t (&k)[2]) { const uint2 v = *reinterpret_cast<const uint2 *>(K + h * 2); k[0] = v.x; k[1] = v.y; } };
template <> struct KeyLine<1> { static __device__ __forceinline__ void load(const uint32_t *K, uint32_t h, uint32_t (&k)[1]) { k[0] = K[h]; } };
// value x matched value of table g for one probed key (0 when the table lacks the key); *found tells which
template <int G>
__device__ __forceinline__ uint32_t ck_match(const uint32_t *V, const uint32_t (&k1)[G], const uint32_t (&k2)[G], int g, uint32_t h1, uint32_t h2,
                                             uint32_t key, bool *found) {
    const bool hit1 = k1[g] == key, hit2 = k2[g] == key;
    uint32_t vb = 0;
    if (hit1 || hit2) vb = V[(hit1 ? h1 : h2) * G + g];
    *found = hit1 || hit2;
    return vb;
}

// ---------------------------------------------------------------------------------------------------------
// Join, sparse + BM25 part, distance assembly, partner selection and proposals.  One CTA per node.
// ---------------------------------------------------------------------------------------------------------
struct JoinArgs {
    uint32_t node0, nodes;
    const uint32_t *plist, *pcnt;
    const uint64_t *meta;
    const uint8_t *rec;
    const float *D;          // nodes x 64 x 32 dense inner products
    const float *knn_dis;    // n x 64 (kth distance filter)
    uint2 *prop; uint32_t *propn;
    unsigned long long *stats;
    uint32_t *err;
    uint32_t arena_bytes;    // shared-memory budget for the sparse sections of all participants
    uint32_t tab_mask, tab_shift, groups;  // hash table of one new row's terms; rows hashed per round
    uint32_t prop_per;                     // partners proposed to each participant (<= kPropPerMax)
    uint32_t shared_pairs;                 // see pair_owned
    uint32_t det;                          // see offer_proposal
    uint32_t gen_shift;                    // pass number goes to key bits gen_shift .. 30 (see ck_insert_key); 0 = tables are wiped
    uint32_t o_tab, o_dm, o_arena;
};
constexpr int kJoinThreads = 512;
constexpr int kJoinSlots = 2;     // terms per lane and pass of the probing loop (a pass covers 32 x this many terms)

__device__ __forceinline__ void jtab_insert(uint2 *tab, uint32_t mask, uint32_t shift, uint32_t key, uint32_t valbits) {
    uint32_t h = (key * 2654435761u) >> shift;
    for (uint32_t i = 0; i <= mask; ++i) {
        const uint32_t old = atomicCAS(&tab[h].x, kEmpty, key);
        if (old == kEmpty) { tab[h].y = valbits; return; }
        if (old == key) return;
        h = (h + 1) & mask;
    }
}

template <int G>
__global__ void __launch_bounds__(kJoinThreads, 2) join_sparse_kernel(const JoinArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t mbar;
    __shared__ uint32_t s_off[kPart + 1], s_id[kPart], s_ns[kPart], s_nb[kPart];
    __shared__ float s_kth[kPart];
    __shared__ uint32_t s_rows, s_new, s_bad[2];   // s_bad: one word per pass parity, reset a pass ahead
    const uint32_t tabn = a.tab_mask + 1;
    uint32_t *K = reinterpret_cast<uint32_t *>(smem + a.o_tab);   // [slot][G] keys, then [slot][G] value words
    uint32_t *V = K + (size_t)tabn * G;
    float *dm = reinterpret_cast<float *>(smem + a.o_dm);  // [32][64] distances: new row i x participant j
    uint8_t *arena = smem + a.o_arena;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t local = blockIdx.x;
    if (local >= a.nodes) return;
    const uint32_t v = a.node0 + local;
    uint32_t n_new = a.pcnt[(size_t)v * 2], rows = a.pcnt[(size_t)v * 2 + 1];
    if (rows <= 1) return;
    if (tid == 0) { mbar_init(&mbar, 1); mbar_fence_init(); s_bad[0] = 0; s_bad[1] = 0; }
    if (tid < kPart) {
        const uint32_t id = tid < (int)rows ? a.plist[(size_t)v * kPart + tid] : kEmpty;
        s_id[tid] = id;
        uint64_t m = 0;
        if (id != kEmpty) { m = a.meta[id]; s_kth[tid] = a.knn_dis[(size_t)id * kK + kK - 1]; }
        s_ns[tid] = meta_ns(m); s_nb[tid] = meta_nb(m);
    }
    __syncthreads();
    if (tid == 0) {
        // participants are dropped from the end when their sparse sections overflow the arena
        uint32_t o = 0, r = 0;
        for (; r < rows; ++r) {
            const uint32_t sz = 8u * (pad2(s_ns[r]) + pad2(s_nb[r]));
            if (o + sz > a.arena_bytes) break;
            s_off[r] = o; o += sz;
        }
        s_off[r] = o;
        s_rows = r; s_new = min(n_new, r);
        mbar_arrive_expect_tx(&mbar, o);
    }
    __syncthreads();
    rows = s_rows; n_new = s_new;
    if (tid < (int)rows) {
        const uint32_t sz = s_off[tid + 1] - s_off[tid];
        if (sz) bulk_g2s(arena + s_off[tid], a.rec + meta_off16(a.meta[s_id[tid]]) * 16ull + kDenseBytes, sz, &mbar);
    }
    for (uint32_t i = tid; i < tabn * G; i += kJoinThreads) { K[i] = kEmpty; V[i] = 0u; }
    mbar_wait_bounded(&mbar, 0, a.err, 3u);
    __syncthreads();

    // the dense tile of this join, staged once (coalesced) instead of one global read per pair
    __shared__ __align__(16) float s_D[kPart * kNewMax];
    {
        const float4 *src = reinterpret_cast<const float4 *>(a.D + (size_t)local * kPart * kNewMax);
        float4 *dst = reinterpret_cast<float4 *>(s_D);
        for (uint32_t q = tid; q < rows * kNewMax / 4; q += kJoinThreads) dst[q] = __ldg(src + q);
    }
    __syncthreads();
    const float *D = s_D;
    unsigned long long evals = 0;
    const uint32_t gen_mask = a.gen_shift ? (0x7FFFFFFFu >> a.gen_shift) << a.gen_shift : 0u;
    for (uint32_t i0 = 0; i0 < n_new; i0 += G) {
        const uint32_t g_cnt = min((uint32_t)G, n_new - i0);
        const uint32_t gen = a.gen_shift ? (i0 / G) << a.gen_shift : 0u;   // this pass's number, in the keys' spare bits
        // hash the terms of rows i0 .. i0+g_cnt-1 (BM25 ids get bit 31 so both vocabularies share one table), a
        // quarter of the CTA per row: keys first, then every value to the slot its key settled in
        constexpr uint32_t kSlice = kJoinThreads / 4;
        for (uint32_t g = tid / kSlice; g < g_cnt; g += 4) {
            const uint32_t i = i0 + g;
            const uint2 *pr = reinterpret_cast<const uint2 *>(arena + s_off[i]);
            const uint32_t ns = s_ns[i], nb = s_nb[i], pns = pad2(ns);
            for (uint32_t j = tid % kSlice; j < ns + nb; j += kSlice) {
                const uint32_t id = (j < ns ? pr[j].x : (pr[pns + (j - ns)].x | 0x80000000u)) | gen;
                if (!ck_insert_key<G>(K, g, a.tab_shift, id, gen_mask)) atomicOr(&s_bad[(i0 / G) & 1u], 1u << g);
            }
        }
        __syncthreads();
        const uint32_t bad = s_bad[(i0 / G) & 1u];   // rows whose table could not be built sit this join out
        if (tid == 0) s_bad[((i0 / G) & 1u) ^ 1u] = 0;   // the next pass's word: nobody touches it before the barrier after the probing
        for (uint32_t g = tid / kSlice; g < g_cnt; g += 4) {
            const uint32_t i = i0 + g;
            const uint2 *pr = reinterpret_cast<const uint2 *>(arena + s_off[i]);
            const uint32_t ns = s_ns[i], nb = s_nb[i], pns = pad2(ns);
            for (uint32_t j = tid % kSlice; j < ns + nb; j += kSlice) {
                const uint2 p = j < ns ? pr[j] : pr[pns + (j - ns)];
                ck_store_value<G>(K, V, g, a.tab_shift, (j < ns ? p.x : (p.x | 0x80000000u)) | gen, p.y);
            }
        }
        __syncthreads();
        // One warp per participant j: its terms pass through registers 64 at a time (the two slot indices of each
        // computed once -- every table uses the same hashes) and are probed against the key lines of the group.
        for (uint32_t j = warp; j < rows; j += kJoinThreads / 32) {
            if (j <= i0) continue;
            const uint2 *pr = reinterpret_cast<const uint2 *>(arena + s_off[j]);
            const uint32_t ns = s_ns[j], nb = s_nb[j], pns = pad2(ns), nt = ns + nb;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (uint32_t base = 0; base < nt; base += 32 * kJoinSlots) {
                uint32_t key[kJoinSlots], h1[kJoinSlots], h2[kJoinSlots]; float val[kJoinSlots];
#pragma unroll
                for (int t = 0; t < kJoinSlots; ++t) {
                    const uint32_t q = base + t * 32 + lane;
                    uint2 p = make_uint2(kEmpty, 0u);   // padding: matches only an empty slot, and its own value is 0
                    if (q < nt) { p = q < ns ? pr[q] : pr[pns + (q - ns)]; if (q >= ns) p.x |= 0x80000000u; p.x |= gen; }
                    key[t] = p.x; val[t] = __uint_as_float(p.y);
                    h1[t] = ck_h1(p.x, a.tab_shift); h2[t] = ck_h2(p.x, a.tab_shift);
                }
#pragma unroll
                for (int t = 0; t < kJoinSlots; ++t) {
                    uint32_t k1[G], k2[G];
                    KeyLine<G>::load(K, h1[t], k1); KeyLine<G>::load(K, h2[t], k2);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        bool found;
                        const uint32_t vb = ck_match<G>(V, k1, k2, g, h1[t], h2[t], key[t], &found);
                        acc[g] = fmaf(__uint_as_float(vb), val[t], acc[g]);
                    }
                }
            }
            // four warp sums in 2 + 1 + 3 shuffles: after two halving exchanges lane l holds the partial of row
            // g = (l >> 3) & 3 over its 8-lane class, the remaining three butterflies finish it
            {
                const bool up4 = (lane & 16) != 0;
                const float k0 = up4 ? acc[2] : acc[0], k1 = up4 ? acc[3] : acc[1];
                const float s0 = up4 ? acc[0] : acc[2], s1 = up4 ? acc[1] : acc[3];
                const float a0 = k0 + __shfl_xor_sync(kFull, s0, 16), a1 = k1 + __shfl_xor_sync(kFull, s1, 16);
                const bool up3 = (lane & 8) != 0;
                float r = (up3 ? a1 : a0) + __shfl_xor_sync(kFull, up3 ? a0 : a1, 8);
                r += __shfl_xor_sync(kFull, r, 4);
                r += __shfl_xor_sync(kFull, r, 2);
                r += __shfl_xor_sync(kFull, r, 1);
                const uint32_t g = (lane >> 3) & 3u, i = i0 + g;
                if ((lane & 7) == 0 && g < g_cnt && i < j) { dm[i * kPart + j] = ((bad >> g) & 1u) ? kInfDis : 1.0f - D[(size_t)j * kNewMax + i] - r; ++evals; }
            }
        }
        __syncthreads();   // every warp is done with this pass's tables
        if (gen_mask && !bad) continue;   // the next pass's keys carry another number: nothing to empty
        // empty the tables again: every term wipes the slots that hold its key
        if (bad) { for (uint32_t q = tid; q < tabn * G; q += kJoinThreads) { K[q] = kEmpty; V[q] = 0u; } }
        else {
            for (uint32_t g = tid / kSlice; g < g_cnt; g += 4) {
                const uint32_t i = i0 + g;
                const uint2 *pr = reinterpret_cast<const uint2 *>(arena + s_off[i]);
                const uint32_t ns = s_ns[i], nb = s_nb[i], pns = pad2(ns);
                for (uint32_t j = tid % kSlice; j < ns + nb; j += kSlice) {
                    const uint32_t id = j < ns ? pr[j].x : (pr[pns + (j - ns)].x | 0x80000000u);
                    const uint32_t h1 = ck_h1(id, a.tab_shift), h2 = ck_h2(id, a.tab_shift);
                    if (K[h1 * G + g] == id) { K[h1 * G + g] = kEmpty; V[h1 * G + g] = 0u; }
                    if (K[h2 * G + g] == id) { K[h2 * G + g] = kEmpty; V[h2 * G + g] = 0u; }
                }
            }
        }
        __syncthreads();
    }

    // partner selection: every participant proposes to itself its prop_per closest partners of this join that beat
    // its current 64th distance.  One warp per participant: each lane holds the distances to partners lane and
    // lane + 32, the best ones are peeled off by warp-wide minima.
    for (uint32_t p = warp; p < rows; p += kJoinThreads / 32) {
        const uint32_t lim = p < n_new ? rows : n_new, me = s_id[p];
        const float kth = s_kth[p];
        unsigned long long c[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t j = lane + 32 * h;
            c[h] = ~0ull;
            if (j < lim && j != p && pair_owned(a.shared_pairs, me, s_id[j])) {
                const float d = dm[min(p, j) * kPart + max(p, j)];
                if (d < kth) c[h] = ((unsigned long long)f2ord(d) << 32) | j;
            }
        }
        unsigned long long mine = ~0ull;   // lane q ends up with the q-th best
        for (uint32_t q = 0; q < a.prop_per; ++q) {
            unsigned long long best = c[0] < c[1] ? c[0] : c[1];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(kFull, best, o);
                best = other < best ? other : best;
            }
            if (best == ~0ull) break;
            if (c[0] == best) c[0] = ~0ull;
            if (c[1] == best) c[1] = ~0ull;
            if (lane == q) mine = best;
        }
        if (mine != ~0ull) offer_proposal(a.det, a.prop, a.propn, a.stats, me, ord2f((uint32_t)(mine >> 32)), s_id[(uint32_t)mine & 63u]);
    }
    if (evals) atomicAdd(a.stats + 0, evals);
    if (tid == 0) atomicAdd(a.stats + 3, (unsigned long long)rows);   // records this join gathered
}

// ---------------------------------------------------------------------------------------------------------
// Merge proposals into the sorted lists: one warp per node, bitonic sorts over 64 + proposals elements held in
// shared memory (first by id to drop duplicates, then by distance), best 64 written back.
// ---------------------------------------------------------------------------------------------------------
constexpr int kMergeLen = 256;  // = 64 + kPropCap
__device__ __forceinline__ void warp_bitonic_u64(unsigned long long *key, int lane) {
    for (int size = 2; size <= kMergeLen; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = lane; t < kMergeLen / 2; t += 32) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool asc = (lo & size) == 0;
                const unsigned long long x = key[lo], y = key[hi];
                if ((x > y) == asc) { key[lo] = y; key[hi] = x; }
            }
            __syncwarp();
        }
}
__device__ __forceinline__ uint32_t f2ord(float f) { const uint32_t b = __float_as_uint(f); return (b & 0x80000000u) ? ~b : (b | 0x80000000u); }
__device__ __forceinline__ float ord2f(uint32_t o) { return __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o); }

__global__ void __launch_bounds__(128, 8) knn_merge_kernel(Knn k) {
    __shared__ unsigned long long keys[4][kMergeLen];
    const uint32_t v = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (v >= k.n) return;
    if (k.propn[v] == 0) return;
    const uint32_t np = k.det ? (uint32_t)kPropCap : min(k.propn[v], (uint32_t)kPropCap);   // deterministic: every slot of the table
    unsigned long long *key = keys[threadIdx.x >> 5];
    // pass 1 key: id (30 bits) | origin (0 = sampled list entry, 1 = unsampled list entry, 2 = proposal) | distance
    // order bits -> equal ids become adjacent with the existing entry first
    for (int t = lane; t < kMergeLen; t += 32) {
        unsigned long long kk = ~0ull;
        if (t < kK) {
            const uint32_t raw = k.ids[(size_t)v * kK + t];
            kk = ((unsigned long long)(raw & 0x3FFFFFFFu) << 34) | ((unsigned long long)(raw >> 31) << 32) | f2ord(k.dis[(size_t)v * kK + t]);
        } else if (t - kK < (int)np) {
            const uint2 p = k.prop[(size_t)v * kPropCap + (t - kK)];
            if (k.det) { if ((p.x & p.y) != kEmpty && p.x != v) kk = ((unsigned long long)(p.x & 0x3FFFFFFFu) << 34) | (2ull << 32) | p.y; }
            else if (p.y != v) kk = ((unsigned long long)(p.y & 0x3FFFFFFFu) << 34) | (2ull << 32) | f2ord(__uint_as_float(p.x));
        }
        key[t] = kk;
    }
    __syncwarp();
    warp_bitonic_u64(key, lane);
    // pass 2 key: distance order bits | id | origin, duplicates of an id (all but the first) dropped
    unsigned long long nk[kMergeLen / 32];
#pragma unroll
    for (int q = 0; q < kMergeLen / 32; ++q) {
        const int t = lane + 32 * q;
        const unsigned long long kk = key[t];
        unsigned long long out = ~0ull;
        if (kk != ~0ull) {
            const uint32_t id = (uint32_t)(kk >> 34);
            const bool dup = t > 0 && key[t - 1] != ~0ull && (uint32_t)(key[t - 1] >> 34) == id;
            if (!dup) out = ((unsigned long long)(uint32_t)kk << 32) | ((unsigned long long)id << 2) | ((kk >> 32) & 3ull);
        }
        nk[q] = out;
    }
    __syncwarp();
#pragma unroll
    for (int q = 0; q < kMergeLen / 32; ++q) key[lane + 32 * q] = nk[q];
    __syncwarp();
    warp_bitonic_u64(key, lane);
    uint32_t changed = 0;
    for (int t = lane; t < kK; t += 32) {
        const unsigned long long kk = key[t];
        uint32_t id = kEmpty & 0x7FFFFFFFu, fl = 0; float d = kInfDis;
        if (kk != ~0ull) { id = (uint32_t)(kk >> 2) & 0x3FFFFFFFu; fl = ((uint32_t)kk & 3u) != 0; d = ord2f((uint32_t)(kk >> 32)); }
        const uint32_t raw = id | (fl << 31);
        if ((k.ids[(size_t)v * kK + t] & 0x7FFFFFFFu) != id) ++changed;
        k.ids[(size_t)v * kK + t] = raw;
        k.dis[(size_t)v * kK + t] = d;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) changed += __shfl_xor_sync(kFull, changed, o);
    if (lane == 0 && changed) atomicAdd(k.stats + 1, (unsigned long long)changed);
}

// Reverse pass (ref: merge_reverse_plus, src/index.cu:386-478): every list entry (v -> u, d) is offered to u as
// (u -> v, d); the following merge keeps u's best 64.  Offers beyond the proposal capacity keep the closer ones.
__global__ void knn_reverse_kernel(Knn k) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k.n * (uint32_t)kK) return;
    const uint32_t v = i / kK, u = k.ids[i] & 0x7FFFFFFFu;
    const float d = k.dis[i];
    if (u >= k.n || u == v || !(d < kInfDis)) return;
    if (!(d < k.dis[(size_t)u * kK + kK - 1])) return;           // cannot enter u's list
    offer_proposal(k.det, k.prop, k.propn, nullptr, u, d, v);
}

__global__ void knn_finish_kernel(Knn k, uint32_t *out_ids) {  // strip flags; unfilled slots point at a valid id
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k.n * (uint32_t)kK) return;
    uint32_t id = k.ids[i] & 0x7FFFFFFFu;
    if (id >= k.n) id = (i / kK + 1) % k.n;
    out_ids[i] = id;
}

// ---------------------------------------------------------------------------------------------------------
// Pruning: ref allan_poe, src/index.cu:539-714.  One CTA (8 warps) per node.
// ---------------------------------------------------------------------------------------------------------
constexpr int kPruneThreads = 256;
constexpr int kPruneWarps = 8;

struct PruneArgs {
    uint32_t n;
    const uint32_t *knn; const float *knn_dis; const float *power;
    const uint64_t *meta; const uint8_t *rec;
    uint32_t *new_list;   // n x 32
    uint32_t *detour;     // n x 32 (detour count riding with slot i, as the reference scatters it)
    uint32_t *kw_edge;    // n x 33
    uint32_t tab_mask, tab_shift;   // candidate's term table (sparse ids, BM25 ids | bit 31)
    uint32_t own_mask, own_shift;   // the node's own BM25 term set
    uint32_t o_tab, o_own, o_lists;
    int unfused;
    const uint32_t *node_list;      // when set, block i prunes node node_list[i]
};

// the reference's shared-memory bitonic network on (key, value) pairs, run by the whole CTA
__device__ __forceinline__ void block_bitonic_kv(uint32_t *key, uint32_t *val, uint32_t len, int tid, int nthreads) {
    for (uint32_t stride = 1; stride < len; stride <<= 1)
        for (uint32_t step = stride; step > 0; step >>= 1) {
            for (uint32_t k = tid; k < len / 2; k += nthreads) {
                const uint32_t aa = 2 * step * (k / step), bb = k % step;
                const uint32_t u = (step == stride) ? (aa + step - 1 - bb) : (aa + bb), d = aa + bb + step;
                if (d < len && key[u] > key[d]) {
                    uint32_t t = key[u]; key[u] = key[d]; key[d] = t;
                    t = val[u]; val[u] = val[d]; val[d] = t;
                }
            }
            __syncthreads();
        }
}

__device__ __forceinline__ bool set_contains(const uint32_t *tab, uint32_t mask, uint32_t shift, uint32_t key) {
    uint32_t h = (key * 2654435761u) >> shift;
    for (uint32_t i = 0; i <= mask; ++i) {
        const uint32_t e = tab[h];
        if (e == kEmpty) return false;
        if (e == key) return true;
        h = (h + 1) & mask;
    }
    return false;
}

__global__ void __launch_bounds__(kPruneThreads, 2) prune_kernel(const PruneArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ uint32_t nei0[kK], nei1[kK], nei2[kK + 1], det[kK];
    __shared__ uint64_t meta0[kK], sel_meta[kK];   // locator words of the detour-ordered candidates / of the selected ones
    __shared__ float pow0[kK], sel_pow[kK];
    __shared__ uint32_t s_tmp_id, s_ipn, s_cur_nei, s_cur_nei2;
    __shared__ uint32_t vflag[16];
    uint2 *tab = reinterpret_cast<uint2 *>(smem + a.o_tab);
    uint32_t *own = reinterpret_cast<uint32_t *>(smem + a.o_own);
    uint32_t *lists = reinterpret_cast<uint32_t *>(smem + a.o_lists);   // 64 x 64 neighbour ids
    float *ldis = reinterpret_cast<float *>(lists + kK * kK);          // 64 x 64 neighbour distances
    const uint32_t bid = a.node_list ? a.node_list[blockIdx.x] : blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (bid >= a.n) return;
    const uint32_t *g = a.knn + (size_t)bid * kK;

    if (tid < kK) { nei0[tid] = g[tid]; det[tid] = 0; nei2[tid] = 0; }
    if (tid == 0) nei2[kK] = 0;
    if (tid < 16) vflag[tid] = 0;
    for (uint32_t i = tid; i <= a.own_mask; i += kPruneThreads) own[i] = kEmpty;
    for (uint32_t i = tid; i <= a.tab_mask; i += kPruneThreads) tab[i] = make_uint2(kEmpty, 0u);
    __syncthreads();
    {   // the node's own BM25 terms (ref :559-565)
        const uint64_t m = a.meta[bid];
        const uint2 *pr = reinterpret_cast<const uint2 *>(a.rec + meta_off16(m) * 16ull + kDenseBytes) + pad2(meta_ns(m));
        for (uint32_t j = tid; j < meta_nb(m); j += kPruneThreads) {
            const uint32_t key = pr[j].x;
            uint32_t h = (key * 2654435761u) >> a.own_shift;
            for (uint32_t s = 0; s <= a.own_mask; ++s) {
                const uint32_t old = atomicCAS(&own[h], kEmpty, key);
                if (old == kEmpty || old == key) break;
                h = (h + 1) & a.own_mask;
            }
        }
    }
    // neighbours' lists for the detour count (ref :572-597)
    for (uint32_t idx = tid; idx < kK * kK; idx += kPruneThreads) {
        const uint32_t p = idx >> 6, j = idx & 63;
        lists[idx] = a.knn[(size_t)nei0[p] * kK + j];
        ldis[idx] = a.knn_dis[(size_t)nei0[p] * kK + j];
    }
    __syncthreads();
    for (uint32_t pair = tid; pair < kK * kK; pair += kPruneThreads) {
        const uint32_t p = pair >> 6, t = pair & 63;
        if (t <= p) continue;
        const uint32_t key = nei0[t];
        int r = -1;
        for (int j = 0; j < kK; ++j) if (lists[p * kK + j] == key) { r = j; break; }
        if (r >= 0 && ldis[p * kK + r] < a.knn_dis[(size_t)bid * kK + t]) atomicAdd(&det[t], 1u);
    }
    __syncthreads();
    block_bitonic_kv(det, nei0, kK, tid, kPruneThreads);
    if (tid < kK) { meta0[tid] = a.meta[nei0[tid]]; pow0[tid] = a.power[nei0[tid]]; }
    __syncthreads();
    if (tid == 0) { nei1[0] = nei0[0]; sel_meta[0] = meta0[0]; sel_pow[0] = pow0[0]; s_tmp_id = 1; s_ipn = 1; s_cur_nei = 0; s_cur_nei2 = 0; }
    __syncthreads();

    // RNG-IP joint pruning (ref :613-676)
    while (s_ipn < kK) {
        const uint32_t cn = nei0[s_tmp_id], ipn = s_ipn;
        const uint64_t cm = meta0[s_tmp_id];
        const uint8_t *crec = a.rec + meta_off16(cm) * 16ull;
        {   // candidate's terms into the table
            const uint2 *pr = reinterpret_cast<const uint2 *>(crec + kDenseBytes);
            const uint32_t ns = meta_ns(cm), nb = meta_nb(cm), pns = pad2(ns);
            for (uint32_t j = tid; j < ns + nb; j += kPruneThreads) {
                const uint2 p = j < ns ? pr[j] : pr[pns + (j - ns)];
                jtab_insert(tab, a.tab_mask, a.tab_shift, j < ns ? p.x : (p.x | 0x80000000u), p.y);
            }
        }
        uint32_t creg[16];  // candidate's dense row in the reference's lane / chunk association
        {
            const uint2 *d = reinterpret_cast<const uint2 *>(crec);
#pragma unroll
            for (int k = 0; k < 8; ++k) { const uint2 x = __ldg(d + lane + 32 * k); creg[2 * k] = x.x; creg[2 * k + 1] = x.y; }
        }
        const float cpow = pow0[s_tmp_id];
        __syncthreads();
        for (uint32_t i = warp; i < ipn; i += kPruneWarps) {
            const uint32_t sn = nei1[i];
            if (sn == kEmpty) continue;
            const uint64_t sm = sel_meta[i];
            const uint8_t *srec = a.rec + meta_off16(sm) * 16ull;
            uint32_t acc = 0;
            const uint2 *d = reinterpret_cast<const uint2 *>(srec);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint2 x = __ldg(d + lane + 32 * k);
                if (a.unfused) { acc = hadd2_rn(acc, hmul2_rn(creg[2 * k], x.x)); acc = hadd2_rn(acc, hmul2_rn(creg[2 * k + 1], x.y)); }
                else { acc = hfma2_rn(creg[2 * k], x.x, acc); acc = hfma2_rn(creg[2 * k + 1], x.y, acc); }
            }
            const uint2 *pr = reinterpret_cast<const uint2 *>(srec + kDenseBytes);
            const uint32_t ns = meta_ns(sm), nb = meta_nb(sm), pns = pad2(ns);
            float sp = 0.0f, bm = 0.0f;
            uint32_t kw = 0;
            // Four terms per lane in flight: all first slots are read together, colliding ones take the next slot
            // together, longer chains are walked one by one; the multiply-adds then run in ascending term order
            // with the matched value or zero (a zero product leaves the sum as it is), so each lane's partial is
            // the one the reference's per-term loop produces.
#pragma unroll
            for (int sec = 0; sec < 2; ++sec) {
                const uint2 *row = sec == 0 ? pr : pr + pns;
                const uint32_t cnt = sec == 0 ? ns : nb;
                float part = 0.0f;
                for (uint32_t j0 = 0; j0 < cnt; j0 += 128) {
                    uint2 pv[4], e[4];
                    uint32_t key[4], hs[4], chain = 0;
                    float qv[4];
                    bool fnd[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const uint32_t j = j0 + 32 * t + lane;
                        pv[t] = j < cnt ? __ldg(row + j) : make_uint2(kEmpty, 0u);
                        key[t] = (sec == 1 && j < cnt) ? (pv[t].x | 0x80000000u) : pv[t].x;
                        hs[t] = (key[t] * 2654435761u) >> a.tab_shift;
                    }
#pragma unroll
                    for (int t = 0; t < 4; ++t) e[t] = tab[hs[t]];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        fnd[t] = e[t].x == key[t];
                        qv[t] = fnd[t] ? __uint_as_float(e[t].y) : 0.0f;
                        chain |= (!fnd[t] && e[t].x != kEmpty) ? (1u << t) : 0u;
                    }
                    if (__any_sync(kFull, chain != 0)) {
#pragma unroll
                        for (int t = 0; t < 4; ++t) e[t] = tab[(hs[t] + 1) & a.tab_mask];
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            if ((chain >> t) & 1u) {
                                if (e[t].x == key[t]) { fnd[t] = true; qv[t] = __uint_as_float(e[t].y); }
                                else if (e[t].x != kEmpty) {
                                    uint32_t h = (hs[t] + 2) & a.tab_mask;
                                    for (uint32_t s2 = 0; s2 < a.tab_mask; ++s2) {
                                        const uint2 e2 = tab[h];
                                        if (e2.x == kEmpty) break;
                                        if (e2.x == key[t]) { fnd[t] = true; qv[t] = __uint_as_float(e2.y); break; }
                                        h = (h + 1) & a.tab_mask;
                                    }
                                }
                            }
                    }
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        part = __fmaf_rn(qv[t], __uint_as_float(pv[t].y), part);
                        // a BM25 term of s that the candidate lacks but the node owns (ref :144-149)
                        if (sec == 1 && j0 + 32 * t + lane < cnt && !fnd[t] && set_contains(own, a.own_mask, a.own_shift, pv[t].x)) kw = 1;
                    }
                }
                if (sec == 0) sp = part; else bm = part;
            }
            float tot = __fadd_rn(sp, bm);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                acc = hadd2_rn(acc, __shfl_down_sync(kFull, acc, o));
                tot = __fadd_rn(tot, __shfl_down_sync(kFull, tot, o));
            }
            kw = __any_sync(kFull, kw != 0);
            if (lane == 0) {
                // the reference runs slot i on warp i % 16 and leaves that warp's flag set until the end of the step
                if (kw) vflag[i & 15] = 1;
                const float ip = __fadd_rn(half_sum_to_float(acc), tot);
                if (cpow < ip) s_cur_nei = 1;
                if (sel_pow[i] < ip) nei1[i] = kEmpty;
                if (vflag[i & 15] != 1) s_cur_nei2 = 1;
            }
            __syncwarp();
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t n2 = ipn;
            if (s_cur_nei == 0) { nei1[n2] = cn; sel_meta[n2] = cm; sel_pow[n2] = cpow; ++n2; }
            if (s_cur_nei2 == 0) nei2[n2] = 1;  // written after the increment, as in the reference
            s_ipn = n2; s_cur_nei = 0; s_cur_nei2 = 0; s_tmp_id = s_tmp_id + 1;
        }
        if (tid < 16) vflag[tid] = 0;
        for (uint32_t i = tid; i <= a.tab_mask; i += kPruneThreads) tab[i] = make_uint2(kEmpty, 0u);
        __syncthreads();
        if (s_tmp_id >= kK) break;
    }
    __syncthreads();
    if (tid == 0) {
        const uint32_t ipn = s_ipn;
        uint32_t count = 0, i_neis;
        for (i_neis = 0; i_neis < ipn && count < AP_DEGREE; ++i_neis)
            if (nei1[i_neis] != kEmpty) nei0[count++] = nei1[i_neis];
        uint32_t *ke = a.kw_edge + (size_t)bid * 33;
        uint32_t kc = 0;
        for (uint32_t i = i_neis; i < ipn; ++i)
            if (nei2[i] == 1 && nei1[i] != kEmpty && kc < 32) { ke[kc + 1] = nei1[i]; ++kc; }
        ke[0] = kc;
        for (uint32_t i = kc + 1; i < 33; ++i) ke[i] = 0;
    }
    __syncthreads();
    if (tid < AP_DEGREE) {
        a.new_list[(size_t)bid * AP_DEGREE + tid] = nei0[tid];
        a.detour[(size_t)bid * AP_DEGREE + tid] = det[tid];
    }
}

// ---------------------------------------------------------------------------------------------------------
// Pruning, all-pairs form.  The step-wise kernel above walks the 63 selection steps one after the other and
// evaluates the inner products of a step only when the step is reached, so most of its time is load latency on
// a chain of dependent steps.  Every inner product a step can ask for is known in advance, though: step b
// compares candidate b (hashed / held in registers) with an earlier candidate a < b (streamed), in that
// orientation.  This kernel therefore evaluates all 2016 ordered pairs of a node's 64 neighbours first, with the
// rows staged in shared memory and the reference's lane / chunk association and rounding kept per pair, and
// then replays the selection steps on the finished 64 x 64 tables with one warp.  Nodes whose neighbours'
// sparse sections do not fit the staging area are listed for the step-wise kernel.
// ---------------------------------------------------------------------------------------------------------
constexpr int kP2Threads = 1024;
constexpr int kP2Warps = kP2Threads / 32;
constexpr int kP2Groups = 4;   // candidate rows hashed per pass

struct Prune2Args {
    PruneArgs p;
    uint32_t groups;                       // <= kP2Groups
    uint32_t gen_shift;                    // pass number in key bits gen_shift .. 30 (see ck_insert_key); 0 = tables are wiped
    uint32_t o_ip, o_kw, o_region, region_bytes;
    uint32_t *ovf_list, *ovf_cnt, *err;
};

// One section (sparse or BM25) of streamed row `row` against the hashed candidate rows of a group: every lane walks
// its terms j = lane, lane + 32, ... in ascending order, NS terms per pass, and adds value x matched value (zero
// when the candidate lacks the term, which leaves the running sum as it is) -- the reference's per-lane order.
template <int NS, bool BM, int G>
__device__ __forceinline__ void p2_section(const uint2 *__restrict__ row, uint32_t cnt, const uint32_t *__restrict__ K, const uint32_t *__restrict__ V,
                                           uint32_t shift, uint32_t gen, int lane, float (&part)[kP2Groups], uint32_t &kwm) {
    for (uint32_t j0 = 0; j0 < cnt; j0 += 32 * NS) {
        uint32_t key[NS], h1[NS], h2[NS], ownbit = 0;
        float val[NS];
#pragma unroll
        for (int t = 0; t < NS; ++t) {
            const uint32_t j = j0 + 32 * t + lane;
            uint2 pv = make_uint2(kEmpty, 0u);   // padding meets an empty slot or nothing: a zero product either way
            if (j < cnt) {
                pv = row[j];
                if (BM) { ownbit |= (pv.x >> 31) << t; pv.x |= 0x80000000u; }
                pv.x |= gen;
            }
            key[t] = pv.x; val[t] = __uint_as_float(pv.y);
            h1[t] = ck_h1(pv.x, shift); h2[t] = ck_h2(pv.x, shift);
        }
#pragma unroll
        for (int t = 0; t < NS; ++t) {
            uint32_t k1[G], k2[G];
            KeyLine<G>::load(K, h1[t], k1); KeyLine<G>::load(K, h2[t], k2);
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                bool found;
                const uint32_t vb = ck_match<G>(V, k1, k2, gi, h1[t], h2[t], key[t], &found);
                part[gi] = __fmaf_rn(__uint_as_float(vb), val[t], part[gi]);
                if (BM && ((ownbit >> t) & 1u) && !found) kwm |= 1u << gi;
            }
        }
    }
}

template <int G>
__global__ void __launch_bounds__(kP2Threads, 1) prune_pairs_kernel(const Prune2Args q) {
    const PruneArgs &a = q.p;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t mbar;
    __shared__ uint32_t nei0[kK], nei1[kK], nei2[kK + 1], det[kK], s_off[kK + 1];
    __shared__ uint64_t meta0[kK];
    __shared__ float pow0[kK];
    __shared__ uint32_t s_task, s_fit, s_dup;
    float *IP = reinterpret_cast<float *>(smem + q.o_ip);      // [b][a], a < b
    uint8_t *KW = smem + q.o_kw;                               // [b][a] keyword flag of the pair
    const uint32_t tabn = a.tab_mask + 1;
    uint32_t *K = reinterpret_cast<uint32_t *>(smem + a.o_tab);   // [slot][G] keys, then [slot][G] value words
    uint32_t *V = K + (size_t)tabn * G;
    uint32_t *own = reinterpret_cast<uint32_t *>(smem + a.o_own);
    uint8_t *region = smem + q.o_region;
    uint32_t *lists = reinterpret_cast<uint32_t *>(region);
    float *ldis = reinterpret_cast<float *>(lists + kK * kK);
    const uint32_t bid = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (bid >= a.n) return;
    const uint32_t *g = a.knn + (size_t)bid * kK;

    if (tid == 0) { mbar_init(&mbar, 1); mbar_fence_init(); s_task = 0; nei2[kK] = 0; }
    if (tid < kK) { nei0[tid] = g[tid]; det[tid] = 0; nei2[tid] = 0; }
    for (uint32_t i = tid; i <= a.own_mask; i += kP2Threads) own[i] = kEmpty;
    for (uint32_t i = tid; i < kK * kK; i += kP2Threads) KW[i] = 0;
    __syncthreads();
    {   // the node's own BM25 terms (ref :559-565)
        const uint64_t m = a.meta[bid];
        const uint2 *pr = reinterpret_cast<const uint2 *>(a.rec + meta_off16(m) * 16ull + kDenseBytes) + pad2(meta_ns(m));
        for (uint32_t j = tid; j < meta_nb(m); j += kP2Threads) {
            const uint32_t key = pr[j].x;
            uint32_t h = (key * 2654435761u) >> a.own_shift;
            for (uint32_t s = 0; s <= a.own_mask; ++s) {
                const uint32_t old = atomicCAS(&own[h], kEmpty, key);
                if (old == kEmpty || old == key) break;
                h = (h + 1) & a.own_mask;
            }
        }
    }
    // detour counts (ref :572-597) and the detour order
    for (uint32_t idx = tid; idx < kK * kK; idx += kP2Threads) {
        const uint32_t p = idx >> 6, j = idx & 63;
        lists[idx] = a.knn[(size_t)nei0[p] * kK + j];
        ldis[idx] = a.knn_dis[(size_t)nei0[p] * kK + j];
    }
    // position table: R[p][t] = first place of neighbour t's id in neighbour p's list (the reference scans the list
    // for it); filled by looking every list entry up in a small hash of the node's own 64 neighbour ids
    uint32_t *R = reinterpret_cast<uint32_t *>(ldis + kK * kK);          // 64 x 64
    uint32_t *hk = R + kK * kK, *hv = hk + 256;                          // 256-slot hash: id -> a place t in nei0
    for (uint32_t i = tid; i < kK * kK; i += kP2Threads) R[i] = kEmpty;
    if (tid < 256) hk[tid] = kEmpty;
    if (tid == 0) s_dup = 0;
    __syncthreads();
    if (tid < kK) {
        const uint32_t id = nei0[tid];
        uint32_t h = (id * 2654435761u) >> 24;
        for (int s = 0; s < 256; ++s) {
            const uint32_t old = atomicCAS(&hk[h], kEmpty, id);
            if (old == kEmpty) { hv[h] = tid; break; }
            if (old == id) { s_dup = 1; break; }      // the same id twice among the neighbours: slow path below
            h = (h + 1) & 255u;
        }
    }
    __syncthreads();
    const bool dup = s_dup != 0;
    for (uint32_t idx = tid; idx < kK * kK; idx += kP2Threads) {
        const uint32_t pl = idx >> 6, j = idx & 63, id = lists[idx];
        uint32_t h = (id * 2654435761u) >> 24, t = kEmpty;
        for (int s = 0; s < 256; ++s) {
            const uint32_t e = hk[h];
            if (e == kEmpty) break;
            if (e == id) { t = hv[h]; break; }
            h = (h + 1) & 255u;
        }
        if (t != kEmpty) {
            if (!dup) atomicMin(&R[pl * kK + t], j);
            else for (uint32_t t2 = 0; t2 < (uint32_t)kK; ++t2) if (nei0[t2] == id) atomicMin(&R[pl * kK + t2], j);
        }
    }
    __syncthreads();
    for (uint32_t pair = tid; pair < kK * kK; pair += kP2Threads) {
        const uint32_t pl = pair >> 6, t = pair & 63;
        if (t <= pl) continue;
        const uint32_t r = R[pair];
        if (r != kEmpty && ldis[pl * kK + r] < a.knn_dis[(size_t)bid * kK + t]) atomicAdd(&det[t], 1u);
    }
    __syncthreads();
    block_bitonic_kv(det, nei0, kK, tid, kP2Threads);
    if (tid < kK) { meta0[tid] = a.meta[nei0[tid]]; pow0[tid] = a.power[nei0[tid]]; }
    __syncthreads();
    if (tid == 0) {
        uint32_t o = 0;
        for (int r = 0; r < kK; ++r) { s_off[r] = o; o += 8u * (pad2(meta_ns(meta0[r])) + pad2(meta_nb(meta0[r]))); }
        s_off[kK] = o;
        s_fit = o <= q.region_bytes;
        if (!s_fit) q.ovf_list[atomicAdd(q.ovf_cnt, 1u)] = bid;
    }
    __syncthreads();
    if (!s_fit) return;

    // ---- dense inner products: rows a of one half staged, candidate rows b in registers ----------------------
    uint32_t parity = 0;
    for (int ch = 0; ch < 2; ++ch) {
        if (tid == 0) { s_task = 0; mbar_arrive_expect_tx(&mbar, 32u * kDenseBytes); }
        fence_proxy_async();   // the region was last touched by ordinary loads / stores
        __syncthreads();
        if (tid < 32) bulk_g2s(region + (size_t)tid * kDenseBytes, a.rec + meta_off16(meta0[32 * ch + tid]) * 16ull, kDenseBytes, &mbar);
        mbar_wait_bounded(&mbar, parity, q.err, 5u);
        parity ^= 1u;
        const uint2 *srow = reinterpret_cast<const uint2 *>(region);
        const uint32_t ntasks = ch == 0 ? 63u : 31u;
        for (;;) {
            uint32_t t = 0;
            if (lane == 0) t = atomicAdd(&s_task, 1u);
            t = __shfl_sync(kFull, t, 0);
            if (t >= ntasks) break;
            const uint32_t b = 63u - t;
            const uint32_t n_a = min(32u, b - 32u * ch);    // rows a = 32 ch .. 32 ch + n_a - 1 are earlier than b
            uint32_t creg[16];
            {
                const uint2 *d = reinterpret_cast<const uint2 *>(a.rec + meta_off16(meta0[b]) * 16ull);
#pragma unroll
                for (int k = 0; k < 8; ++k) { const uint2 x = __ldg(d + lane + 32 * k); creg[2 * k] = x.x; creg[2 * k + 1] = x.y; }
            }
            uint32_t acc[32];
#pragma unroll
            for (int al = 0; al < 32; ++al) {
                uint32_t s = 0;
                if ((uint32_t)al < n_a) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const uint2 x = srow[al * 256 + lane + 32 * k];
                        s = hfma2_rn(creg[2 * k], x.x, s); s = hfma2_rn(creg[2 * k + 1], x.y, s);
                    }
                }
                acc[al] = s;
            }
            // 32 tree sums at once; the pairing (l, l ^ 16), (l, l ^ 8), ... is the reference's shuffle-down tree as seen
            // from lane 0, and half addition commutes, so lane l ends with exactly the sum lane 0 would hold for row l
#pragma unroll
            for (int o = 16, len = 32; o >= 1; o >>= 1, len >>= 1) {
#pragma unroll
                for (int w = 0; w < len / 2; ++w) {
                    const bool up = (lane & o) != 0;
                    const uint32_t keep = up ? acc[w + len / 2] : acc[w];
                    const uint32_t send = up ? acc[w] : acc[w + len / 2];
                    acc[w] = hadd2_rn(keep, __shfl_xor_sync(kFull, send, o));
                }
            }
            if ((uint32_t)lane < n_a) IP[b * kK + 32 * ch + lane] = half_sum_to_float(acc[0]);
        }
        __syncthreads();
    }

    // ---- sparse and BM25 sections of all 64 rows into the region ------------------------------------------
    if (tid == 0) mbar_arrive_expect_tx(&mbar, s_off[kK]);
    fence_proxy_async();
    __syncthreads();
    if (tid < kK) {
        const uint32_t sz = s_off[tid + 1] - s_off[tid];
        if (sz) bulk_g2s(region + s_off[tid], a.rec + meta_off16(meta0[tid]) * 16ull + kDenseBytes, sz, &mbar);
    }
    for (uint32_t i = tid; i < tabn * G; i += kP2Threads) { K[i] = kEmpty; V[i] = 0u; }
    if (s_off[kK]) mbar_wait_bounded(&mbar, parity, q.err, 6u);
    __syncthreads();
    // bit 31 of a staged BM25 id: the node itself owns the term (ref :144-149 asks this per pair)
    for (int r = warp; r < kK; r += kP2Warps) {
        uint2 *pr = reinterpret_cast<uint2 *>(region + s_off[r]) + pad2(meta_ns(meta0[r]));
        for (uint32_t j = lane; j < meta_nb(meta0[r]); j += 32)
            if (set_contains(own, a.own_mask, a.own_shift, pr[j].x)) pr[j].x |= 0x80000000u;
    }
    __syncthreads();

    const uint32_t gen_mask = q.gen_shift ? (0x7FFFFFFFu >> q.gen_shift) << q.gen_shift : 0u;
    for (uint32_t b0 = 0; b0 < (uint32_t)kK; b0 += G) {
        const uint32_t g_cnt = min((uint32_t)G, (uint32_t)kK - b0);
        const uint32_t gen = q.gen_shift ? (b0 / G) << q.gen_shift : 0u;   // this pass's number, in the keys' spare bits
        // the G candidate rows are hashed side by side: a quarter of the CTA per row
        constexpr uint32_t kSlice = kP2Threads / 4;
        for (uint32_t gi = tid / kSlice; gi < g_cnt; gi += 4) {
            const uint32_t b = b0 + gi;
            if (b == 0) continue;
            const uint2 *pr = reinterpret_cast<const uint2 *>(region + s_off[b]);
            const uint32_t ns = meta_ns(meta0[b]), nb = meta_nb(meta0[b]), pns = pad2(ns);
            for (uint32_t j = tid % kSlice; j < ns + nb; j += kSlice) {
                const uint32_t id = (j < ns ? pr[j].x : (pr[pns + (j - ns)].x | 0x80000000u)) | gen;
                if (!ck_insert_key<G>(K, gi, a.tab_shift, id, gen_mask)) s_fit = 0;
            }
        }
        __syncthreads();
        if (!s_fit) {   // a table could not be built: the step-wise kernel takes the node
            if (tid == 0) q.ovf_list[atomicAdd(q.ovf_cnt, 1u)] = bid;
            return;
        }
        for (uint32_t gi = tid / kSlice; gi < g_cnt; gi += 4) {
            const uint32_t b = b0 + gi;
            if (b == 0) continue;
            const uint2 *pr = reinterpret_cast<const uint2 *>(region + s_off[b]);
            const uint32_t ns = meta_ns(meta0[b]), nb = meta_nb(meta0[b]), pns = pad2(ns);
            for (uint32_t j = tid % kSlice; j < ns + nb; j += kSlice) {
                const uint2 p = j < ns ? pr[j] : pr[pns + (j - ns)];
                ck_store_value<G>(K, V, gi, a.tab_shift, (j < ns ? p.x : (p.x | 0x80000000u)) | gen, p.y);
            }
        }
        __syncthreads();
        const uint32_t a_end = min(b0 + g_cnt - 1u, (uint32_t)kK - 1u);   // rows a < the group's last candidate
        for (uint32_t ar = warp; ar < a_end; ar += kP2Warps) {
            const uint2 *pr = reinterpret_cast<const uint2 *>(region + s_off[ar]);
            const uint32_t ns = meta_ns(meta0[ar]), nb = meta_nb(meta0[ar]), pns = pad2(ns);
            float sp[kP2Groups] = {0.f, 0.f, 0.f, 0.f}, bm[kP2Groups] = {0.f, 0.f, 0.f, 0.f};
            uint32_t kwm = 0;   // bit g: a BM25 term of row a that the node owns and candidate g lacks
            p2_section<4, false, G>(pr, ns, K, V, a.tab_shift, gen, lane, sp, kwm);
            p2_section<2, true, G>(pr + pns, nb, K, V, a.tab_shift, gen, lane, bm, kwm);
            float tot[kP2Groups];
#pragma unroll
            for (int gi = 0; gi < kP2Groups; ++gi) tot[gi] = __fadd_rn(sp[gi], bm[gi]);
            // four tree sums in 2 + 1 + 3 shuffles, same pairing order (16, 8, 4, 2, 1) as the reference's tree
            const bool up4 = (lane & 16) != 0;
            const float k0 = up4 ? tot[2] : tot[0], k1 = up4 ? tot[3] : tot[1];
            const float s0 = up4 ? tot[0] : tot[2], s1 = up4 ? tot[1] : tot[3];
            const float a0 = __fadd_rn(k0, __shfl_xor_sync(kFull, s0, 16)), a1 = __fadd_rn(k1, __shfl_xor_sync(kFull, s1, 16));
            const bool up3 = (lane & 8) != 0;
            float r = __fadd_rn(up3 ? a1 : a0, __shfl_xor_sync(kFull, up3 ? a0 : a1, 8));
            r = __fadd_rn(r, __shfl_xor_sync(kFull, r, 4));
            r = __fadd_rn(r, __shfl_xor_sync(kFull, r, 2));
            r = __fadd_rn(r, __shfl_xor_sync(kFull, r, 1));
            uint32_t kw_any = 0;
#pragma unroll
            for (int gi = 0; gi < kP2Groups; ++gi) kw_any |= __any_sync(kFull, (kwm >> gi) & 1u) ? (1u << gi) : 0u;
            const uint32_t gi = (lane >> 3) & 3u, b = b0 + gi;
            if ((lane & 7) == 0 && gi < g_cnt && b > ar) {
                IP[b * kK + ar] = __fadd_rn(IP[b * kK + ar], r);
                KW[b * kK + ar] = (kw_any >> gi) & 1u;
            }
        }
        __syncthreads();   // every warp is done with this pass's tables
        if (gen_mask) continue;   // the next pass's keys carry another number: nothing to empty
        // empty the tables again: every term wipes the slots that hold its key
        for (uint32_t gi = tid / kSlice; gi < g_cnt; gi += 4) {
            const uint32_t b = b0 + gi;
            if (b == 0) continue;
            const uint2 *pr = reinterpret_cast<const uint2 *>(region + s_off[b]);
            const uint32_t ns = meta_ns(meta0[b]), nb = meta_nb(meta0[b]), pns = pad2(ns);
            for (uint32_t j = tid % kSlice; j < ns + nb; j += kSlice) {
                const uint32_t id = j < ns ? pr[j].x : (pr[pns + (j - ns)].x | 0x80000000u);
                const uint32_t h1 = ck_h1(id, a.tab_shift), h2 = ck_h2(id, a.tab_shift);
                if (K[h1 * G + gi] == id) { K[h1 * G + gi] = kEmpty; V[h1 * G + gi] = 0u; }
                if (K[h2 * G + gi] == id) { K[h2 * G + gi] = kEmpty; V[h2 * G + gi] = 0u; }
            }
        }
        __syncthreads();
    }

    // ---- the selection steps (ref :613-676) replayed on the tables by one warp -----------------------------
    if (warp == 0) {
        // lane l keeps selected slots l and l + 32: the candidate's place in detour order, its norm, whether it is
        // still alive (not tombstoned)
        uint32_t pos[2] = {0u, 0u};
        float spow[2] = {pow0[0], 0.f};
        bool alive[2] = {lane == 0, false};
        uint32_t ipn = 1;
        unsigned long long kwmask = 0;   // bit n - 1: nei2[n] set
        for (uint32_t b = 1; b < (uint32_t)kK && ipn < (uint32_t)kK; ++b) {
            const float cpow = pow0[b];
            bool rej = false, tomb[2], kw[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const bool valid = lane + 32u * h < ipn && alive[h];
                const float ip = valid ? IP[b * kK + pos[h]] : 0.0f;
                rej = rej || (valid && cpow < ip);
                tomb[h] = valid && spow[h] < ip;
                kw[h] = valid && KW[b * kK + pos[h]] != 0;
            }
            const uint32_t am0 = __ballot_sync(kFull, lane < ipn && alive[0]), am1 = __ballot_sync(kFull, lane + 32u < ipn && alive[1]);
            const uint32_t km0 = __ballot_sync(kFull, kw[0]), km1 = __ballot_sync(kFull, kw[1]);
            // The reference runs slot i on warp i % 16 and that warp's flag, once a slot set it, stays set for the rest of
            // the step: within a class (i mod 16, ascending i) the step stays "open" exactly when the first live slot of
            // the class has no keyword flag.
            const uint32_t r = lane & 15u;
            const uint32_t e = ((am0 >> r) & 1u) | (((am0 >> (r + 16)) & 1u) << 1) | (((am1 >> r) & 1u) << 2) | (((am1 >> (r + 16)) & 1u) << 3);
            const uint32_t kk = ((km0 >> r) & 1u) | (((km0 >> (r + 16)) & 1u) << 1) | (((km1 >> r) & 1u) << 2) | (((km1 >> (r + 16)) & 1u) << 3);
            const bool open = e != 0 && ((kk >> (__ffs(e) - 1)) & 1u) == 0;
            const bool rej_any = __any_sync(kFull, rej), open_any = __any_sync(kFull, open);
            alive[0] = alive[0] && !tomb[0]; alive[1] = alive[1] && !tomb[1];
            uint32_t n2 = ipn;
            if (!rej_any) {
                if (lane == (n2 & 31u)) {
                    if (n2 < 32u) { pos[0] = b; spow[0] = cpow; alive[0] = true; }
                    else { pos[1] = b; spow[1] = cpow; alive[1] = true; }
                }
                ++n2;
            }
            if (!open_any) kwmask |= 1ull << (n2 - 1u);   // nei2[n2], indexed after the increment as in the reference
            ipn = n2;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t i = lane + 32u * h;
            if (i < ipn) nei1[i] = alive[h] ? nei0[pos[h]] : kEmpty;
            if (i < (uint32_t)kK) nei2[i + 1] = (uint32_t)((kwmask >> i) & 1ull);
        }
        __syncwarp();
        if (lane == 0) {
            uint32_t count = 0, i_neis;
            for (i_neis = 0; i_neis < ipn && count < AP_DEGREE; ++i_neis)
                if (nei1[i_neis] != kEmpty) nei0[count++] = nei1[i_neis];
            uint32_t *ke = a.kw_edge + (size_t)bid * 33;
            uint32_t kc = 0;
            for (uint32_t i = i_neis; i < ipn; ++i)
                if (nei2[i] == 1 && nei1[i] != kEmpty && kc < 32) { ke[kc + 1] = nei1[i]; ++kc; }
            ke[0] = kc;
            for (uint32_t i = kc + 1; i < 33; ++i) ke[i] = 0;
        }
    }
    __syncthreads();
    if (tid < AP_DEGREE) {
        a.new_list[(size_t)bid * AP_DEGREE + tid] = nei0[tid];
        a.detour[(size_t)bid * AP_DEGREE + tid] = det[tid];
    }
}

// ---------------------------------------------------------------------------------------------------------
// Reverse edges and final rows: ref src/index.cu:699-711 (scatter) and :717-807 (allan_poe_final_graph).
// The reference scatters with atomics from racing blocks; here every edge gets the key
// (target, source, slot), the keys are radix-sorted, and each target replays its edges in ascending
// (source, slot) order with the reference's "first 32 fill, later ones replace slot k % 32 when their detour
// count is smaller" rule.
// ---------------------------------------------------------------------------------------------------------
__global__ void rev_keys_kernel(uint32_t n, const uint32_t *__restrict__ new_list, const uint32_t *__restrict__ detour,
                                unsigned long long *__restrict__ keys, uint32_t *__restrict__ vals, uint32_t *__restrict__ indeg) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * (uint32_t)AP_DEGREE) return;
    const uint32_t bid = i / AP_DEGREE, s = i % AP_DEGREE, t = new_list[i];
    keys[i] = ((unsigned long long)t << 37) | ((unsigned long long)bid << 5) | s;
    vals[i] = detour[i];
    atomicAdd(&indeg[t], 1u);
}
__global__ void seg_start_kernel(uint32_t total, const unsigned long long *__restrict__ keys, uint32_t *__restrict__ start) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const uint32_t t = (uint32_t)(keys[i] >> 37);
    if (i == 0 || (uint32_t)(keys[i - 1] >> 37) != t) start[t] = i;
}

// the reference's bitonic network on up to 32 (key, value) pairs in thread-local arrays
__device__ __forceinline__ void local_bitonic_kv(uint32_t *key, uint32_t *val, uint32_t len) {
    for (uint32_t stride = 1; stride < len; stride <<= 1)
        for (uint32_t step = stride; step > 0; step >>= 1)
            for (uint32_t k = 0; k < len / 2; ++k) {
                const uint32_t aa = 2 * step * (k / step), bb = k % step;
                const uint32_t u = (step == stride) ? (aa + step - 1 - bb) : (aa + bb), d = aa + bb + step;
                if (d < len && key[u] > key[d]) {
                    uint32_t t = key[u]; key[u] = key[d]; key[d] = t;
                    t = val[u]; val[u] = val[d]; val[d] = t;
                }
            }
}

__global__ void final_rows_kernel(uint32_t n, const uint32_t *__restrict__ new_list, const uint32_t *__restrict__ kw_edge,
                                  const unsigned long long *__restrict__ keys, const uint32_t *__restrict__ vals,
                                  const uint32_t *__restrict__ start, const uint32_t *__restrict__ indeg,
                                  uint32_t *__restrict__ graph) {
    const uint32_t bid = blockIdx.x * blockDim.x + threadIdx.x;
    if (bid >= n) return;
    constexpr uint32_t d = AP_DEGREE;
    uint32_t rid[d], rdt[d];
    const uint32_t deg = indeg[bid], s0 = deg ? start[bid] : 0;
    for (uint32_t k = 0; k < deg; ++k) {
        const uint32_t src = (uint32_t)(keys[s0 + k] >> 5) & 0xFFFFFFFFu, dt = vals[s0 + k], slot = k % d;
        if (k < d || rdt[slot] > dt) { rid[slot] = src; rdt[slot] = dt; }
    }
    const uint32_t rv = min(deg, d);
    const uint32_t *nl = new_list + (size_t)bid * d;
    uint32_t *row = graph + (size_t)bid * AP_ROW;
    for (uint32_t i = 0; i < AP_ROW; ++i) row[i] = 0;
    local_bitonic_kv(rid, rdt, rv);  // by id
    uint32_t key2[d];
    for (uint32_t i = 0; i < rv; ++i) key2[i] = (i > 0 && rid[i] == rid[i - 1]) ? kEmpty : rdt[i];
    for (uint32_t i = 0; i < d / 2; ++i) row[i] = nl[i];
    local_bitonic_kv(key2, rid, rv);  // by detour count, repeated ids last
    uint32_t cur = 0;
    const uint32_t lim = rv < d / 2 ? d - rv : d / 2;
    for (uint32_t i = 0; i < rv; ++i) {
        bool found = false;
        for (uint32_t j = 0; j < lim; ++j) if (rid[i] == nl[j]) { found = true; break; }
        if (!found) { const uint32_t t = cur++; if (t < d / 2) row[d / 2 + t] = rid[i]; }
    }
    const uint32_t placed = min(cur, d / 2);
    for (uint32_t i = 0; i < d / 2 - placed; ++i) row[d / 2 + placed + i] = nl[i + d / 2];
    const uint32_t *ke = kw_edge + (size_t)bid * 33;
    cur = 0;
    for (uint32_t i = 0; i < ke[0]; ++i) {
        bool found = false;
        for (uint32_t j = d / 2; j < d; ++j) if (row[j] == ke[1 + i]) { found = true; break; }
        if (!found) { const uint32_t t = cur++; if (t < 7) row[d + t + 1] = ke[1 + i]; }
    }
    row[d] = min(cur, 7u);
}

__global__ void ep_keys_kernel(uint32_t n, const float *__restrict__ power, unsigned long long *__restrict__ keys) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) keys[i] = ((unsigned long long)f2ord(power[i]) << 32) | i;
}
__global__ void ep_take_kernel(uint32_t n, const unsigned long long *__restrict__ keys, uint32_t *__restrict__ ep) {
    const uint32_t i = threadIdx.x;
    if (i < AP_ENTRY_POINTS) ep[i] = (uint32_t)keys[i < n ? i : n - 1];
}

// ---------------------------------------------------------------------------------------------------------
// host drivers
// ---------------------------------------------------------------------------------------------------------
static uint32_t pow2_at_least(uint32_t v, uint32_t lo) { uint32_t p = lo; while (p < v) p <<= 1; return p; }
static uint32_t log2u(uint32_t p) { uint32_t l = 0; while ((1u << l) < p) ++l; return l; }

// Device scratch of one build step.  Memory handed over with donate() (buffers of an earlier phase that are dead by
// now) is carved up first, so a later phase does not go back to cudaMalloc, whose cost on a busy allocator varies
// from microseconds to hundreds of milliseconds; what does not fit is allocated and freed with the object.
struct DevBuf {
    std::vector<void *> ptrs;
    struct Slab { uint8_t *p; size_t left; };
    std::vector<Slab> slabs;
    ~DevBuf() { for (void *p : ptrs) cudaFree(p); }
    void donate(void *p, size_t bytes) { if (p && bytes) slabs.push_back(Slab{(uint8_t *)p, bytes}); }
    template <class T> int alloc(T **out, size_t count) {
        const size_t bytes = (std::max<size_t>(count * sizeof(T), 16) + 255) / 256 * 256;
        for (Slab &sl : slabs)
            if (sl.left >= bytes) { *out = (T *)sl.p; sl.p += bytes; sl.left -= bytes; return AP_OK; }
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess) return fail(AP_ERR_CUDA, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        ptrs.push_back(p); *out = (T *)p; return AP_OK;
    }
};

static int sort_u64_pairs(DevBuf &db, unsigned long long *keys, uint32_t *vals, size_t count, int end_bit,
                          unsigned long long **keys_out, uint32_t **vals_out) {
    unsigned long long *k2; uint32_t *v2 = nullptr;
    AP_TRY(db.alloc(&k2, count));
    if (vals) AP_TRY(db.alloc(&v2, count));
    size_t tmp_bytes = 0;
    if (vals) AP_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, keys, k2, vals, v2, (int)count, 0, end_bit));
    else AP_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, tmp_bytes, keys, k2, (int)count, 0, end_bit));
    uint8_t *tmp; AP_TRY(db.alloc(&tmp, tmp_bytes));
    if (vals) AP_CUDA(cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, keys, k2, vals, v2, (int)count, 0, end_bit));
    else AP_CUDA(cub::DeviceRadixSort::SortKeys(tmp, tmp_bytes, keys, k2, (int)count, 0, end_bit));
    *keys_out = k2; if (vals_out) *vals_out = v2;
    return AP_OK;
}

// Largest term id of the corpus, computed once per index.
static int max_term_run(ap_index *ix, uint32_t *out) {
    if (!ix->max_term_known) {
        if (!ix->rec_build) return fail(AP_ERR_STATE, "the index was created without AP_CREATE_FOR_BUILD");
        uint32_t *d = ix->d_ctl + 3;   // spare control word
        AP_CUDA(cudaMemsetAsync(d, 0, 4));
        max_term_kernel<<<(ix->n + 7) / 8, 256>>>(ix->n, ix->meta, ix->rec_build, d);
        AP_CUDA(cudaGetLastError());
        AP_CUDA(cudaMemcpy(&ix->max_term, d, 4, cudaMemcpyDeviceToHost));
        ix->max_term_known = true;
    }
    *out = ix->max_term;
    return AP_OK;
}
// Key bit from which the pass number of a table is stored (see ck_insert_key), or 0 when the ids leave no room for
// `passes` numbers below bit 31.
static uint32_t gen_shift_for(uint32_t max_term, uint32_t passes) {
    uint32_t bits = 0;
    while ((1u << bits) < passes) ++bits;
    const uint32_t shift = 31u - bits;
    return (bits > 0 && max_term < (1u << shift) - 1u) ? shift : 0u;
}

int norms_run(ap_index *ix, float *d_power) {
    if (!ix->rec_build) return fail(AP_ERR_STATE, "the index was created without AP_CREATE_FOR_BUILD");
    norms_kernel<<<(ix->n + 7) / 8, 256>>>(ix->n, ix->meta, ix->rec_build, d_power);
    AP_CUDA(cudaGetLastError());
    return AP_OK;
}

// prune + reverse edges + final rows + entry points, on device k-NN lists; installs the graph.
static int prune_run_in(DevBuf &db, ap_index *ix, const uint32_t *d_knn, const float *d_knn_dis, const float *d_power, uint32_t *d_new_list,
                        uint32_t *d_kw, uint32_t *launches, uint32_t flags) {
    const uint32_t n = ix->n;
    if (n >= (1u << 27)) return fail(AP_ERR_LIMIT, "pruning supports up to 2^27 documents per index");
    const bool trace = (flags & AP_BUILD_TRACE) != 0;
    const auto tr0 = std::chrono::high_resolution_clock::now();
    auto mark = [&](const char *what) {
        if (!trace) return;
        cudaDeviceSynchronize();
        fprintf(stderr, "prune: %.1f ms after %s\n", std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - tr0).count(), what);
    };
    uint32_t *detour, *nl = d_new_list, *kw = d_kw;
    AP_TRY(db.alloc(&detour, (size_t)n * AP_DEGREE));
    if (!nl) AP_TRY(db.alloc(&nl, (size_t)n * AP_DEGREE));
    if (!kw) AP_TRY(db.alloc(&kw, (size_t)n * 33));
    PruneArgs a{};
    a.n = n; a.knn = d_knn; a.knn_dis = d_knn_dis; a.power = d_power; a.meta = ix->meta; a.rec = ix->rec_build;
    a.new_list = nl; a.detour = detour; a.kw_edge = kw; a.unfused = 0; a.node_list = nullptr;
    const uint32_t tabn = pow2_at_least(2 * (ix->max_ns + ix->max_nb), 64), ownn = pow2_at_least(2 * ix->max_nb, 64);
    a.tab_mask = tabn - 1; a.tab_shift = 32 - log2u(tabn); a.own_mask = ownn - 1; a.own_shift = 32 - log2u(ownn);
    a.o_tab = 0; a.o_own = 8 * tabn; a.o_lists = a.o_own + 4 * ownn;
    const size_t smem = a.o_lists + (size_t)kK * kK * 8;
    if (smem > ix->smem_per_block) return fail(AP_ERR_LIMIT, "pruning needs %zu bytes of shared memory per block", smem);
    AP_CUDA(cudaFuncSetAttribute(prune_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

    // all-pairs kernel first; the step-wise kernel takes the nodes it lists (or all of them when the tables alone
    // leave no room for a staging area, or when AP_BUILD_PRUNE_STEPWISE asks for it)
    Prune2Args q{};
    q.p = a;
    q.o_ip = 0; q.o_kw = kK * kK * 4; q.p.o_own = q.o_kw + kK * kK;
    q.p.o_tab = (q.p.o_own + 4 * ownn + 15) / 16 * 16;
    const size_t fixed = 4096;   // static shared memory of the kernel, rounded up
    const size_t avail = ix->smem_per_block > fixed ? ix->smem_per_block - fixed : 0;
    uint32_t groups = kP2Groups;
    while (groups > 1 && q.p.o_tab + (size_t)groups * tabn * 8 + 96 * 1024 > avail) groups >>= 1;   // key lines are 1, 2 or 4 wide
    q.groups = groups;
    {
        uint32_t max_term = 0;
        AP_TRY(max_term_run(ix, &max_term));
        q.gen_shift = (flags & AP_BUILD_WIPE_TABLES) ? 0u : gen_shift_for(max_term, (kK + groups - 1) / groups);
    }
    q.o_region = (uint32_t)((q.p.o_tab + (size_t)groups * tabn * 8 + 127) / 128 * 128);
    const bool pairs_ok = avail >= (size_t)q.o_region + 64 * 1024 && !(flags & AP_BUILD_PRUNE_STEPWISE);
    uint32_t n_step = n;
    uint32_t *ovf_list = nullptr, *ovf_cnt = nullptr;
    if (pairs_ok) {
        q.region_bytes = (uint32_t)((avail - q.o_region) / 128 * 128);
        AP_TRY(db.alloc(&ovf_list, n)); AP_TRY(db.alloc(&ovf_cnt, 1));
        AP_CUDA(cudaMemsetAsync(ovf_cnt, 0, 4));
        q.ovf_list = ovf_list; q.ovf_cnt = ovf_cnt; q.err = ix->d_ctl + 1;
        const size_t smem2 = (size_t)q.o_region + q.region_bytes;
        auto pairs_kernel = groups == 4 ? prune_pairs_kernel<4> : (groups == 2 ? prune_pairs_kernel<2> : prune_pairs_kernel<1>);
        AP_CUDA(cudaFuncSetAttribute(pairs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
        pairs_kernel<<<n, kP2Threads, smem2>>>(q);
        AP_CUDA(cudaGetLastError());
        AP_CUDA(cudaMemcpy(&n_step, ovf_cnt, 4, cudaMemcpyDeviceToHost));
        mark("the all-pairs kernel");
        if (trace) fprintf(stderr, "prune: %u nodes left to the step-wise kernel\n", n_step);
        a.node_list = ovf_list;
        if (launches) ++*launches;
    }
    if (n_step) {
        prune_kernel<<<n_step, kPruneThreads, smem>>>(a);
        AP_CUDA(cudaGetLastError());
    }
    {
        uint32_t ew = 0;
        AP_CUDA(cudaMemcpy(&ew, ix->d_ctl + 1, 4, cudaMemcpyDeviceToHost));
        if (ew) { cudaMemset(ix->d_ctl + 1, 0, 4); return fail(AP_ERR_DEVICE, "a pruning kernel raised error word %u (a bounded wait ran out)", ew); }
    }

    mark("the step-wise kernel");
    const size_t total = (size_t)n * AP_DEGREE;
    unsigned long long *keys, *keys_s; uint32_t *vals, *vals_s, *indeg, *start;
    AP_TRY(db.alloc(&keys, total)); AP_TRY(db.alloc(&vals, total));
    AP_TRY(db.alloc(&indeg, n)); AP_TRY(db.alloc(&start, n));
    AP_CUDA(cudaMemsetAsync(indeg, 0, (size_t)n * 4));
    AP_CUDA(cudaMemsetAsync(start, 0, (size_t)n * 4));
    mark("allocations");
    rev_keys_kernel<<<(uint32_t)((total + 255) / 256), 256>>>(n, nl, detour, keys, vals, indeg);
    mark("edge keys");
    AP_TRY(sort_u64_pairs(db, keys, vals, total, 64, &keys_s, &vals_s));
    mark("edge sort");
    seg_start_kernel<<<(uint32_t)((total + 255) / 256), 256>>>((uint32_t)total, keys_s, start);
    if (!ix->graph) AP_CUDA(cudaMalloc(&ix->graph, (size_t)n * AP_ROW * 4));
    if (!ix->ep) AP_CUDA(cudaMalloc(&ix->ep, AP_ENTRY_POINTS * 4));
    final_rows_kernel<<<(n + 127) / 128, 128>>>(n, nl, kw, keys_s, vals_s, start, indeg, ix->graph);
    // entry points: the 32 smallest norms, ties by id (ref src/index.cu:916-925)
    unsigned long long *ek, *ek_s;
    AP_TRY(db.alloc(&ek, n));
    ep_keys_kernel<<<(n + 255) / 256, 256>>>(n, d_power, ek);
    AP_TRY(sort_u64_pairs(db, ek, nullptr, n, 64, &ek_s, nullptr));
    ep_take_kernel<<<1, 32>>>(n, ek_s, ix->ep);
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaDeviceSynchronize());
    mark("reverse edges, rows and entry points");
    if (launches) *launches += 8;
    const int rc_install = index_install_graph(ix);
    mark("the fat rows");
    return rc_install;
}

int prune_run(ap_index *ix, const uint32_t *d_knn, const float *d_knn_dis, const float *d_power, uint32_t *d_new_list,
              uint32_t *d_kw, uint32_t *launches, uint32_t flags) {
    DevBuf db;
    return prune_run_in(db, ix, d_knn, d_knn_dis, d_power, d_new_list, d_kw, launches, flags);
}

int join_dense_tc_launch(ap_index *ix, uint32_t node0, uint32_t nodes, const uint32_t *plist, const uint32_t *pcnt, float *D,
                         cudaStream_t stream);  // apoe_join_tc.cu

// Term-seeded first lists (see seed_cand_kernel).  Skipped when the corpus has no BM25 postings or 2^31 and more
// (about 35 M documents of the benchmark's shape): the build then starts from the random lists alone.
static int seed_run(ap_index *ix, const Knn &k, uint32_t take, uint32_t shared_pairs, uint32_t *launches, void *scratch, size_t scratch_bytes) {
    const uint32_t n = ix->n;
    DevBuf db;
    db.donate(scratch, scratch_bytes);   // memory the rounds use later
    uint32_t *cnt, *off, *cand;
    unsigned long long *total64;
    AP_TRY(db.alloc(&cnt, (size_t)n + 1)); AP_TRY(db.alloc(&off, (size_t)n + 1)); AP_TRY(db.alloc(&total64, 1));
    AP_CUDA(cudaMemset(total64, 0, 8));
    inv_count_kernel<<<n / 256 + 1, 256>>>(n, ix->meta, cnt, total64);
    unsigned long long all = 0;
    AP_CUDA(cudaMemcpy(&all, total64, 8, cudaMemcpyDeviceToHost));
    if (all == 0 || all >= (1ull << 31)) return AP_OK;   // nothing to seed from, or more postings than one sort call takes
    size_t tmp_bytes = 0;
    AP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, cnt, off, (int)(n + 1)));
    uint8_t *tmp; AP_TRY(db.alloc(&tmp, tmp_bytes));
    AP_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, cnt, off, (int)(n + 1)));
    const uint32_t total = (uint32_t)all;
    unsigned long long *keys, *keys_s;
    AP_TRY(db.alloc(&keys, total));
    inv_keys_kernel<<<(n + 7) / 8, 256>>>(n, ix->meta, ix->rec_build, off, keys);
    AP_TRY(sort_u64_pairs(db, keys, nullptr, total, 64, &keys_s, nullptr));
    AP_TRY(db.alloc(&cand, (size_t)n * kK));
    seed_cand_kernel<<<(n + 7) / 8, 256>>>(n, ix->meta, ix->rec_build, keys_s, total, take, cand);
    const uint32_t tabn = pow2_at_least(2 * (ix->max_ns + ix->max_nb), 64);
    const size_t smem = (size_t)kSeedWarps * tabn * 8;
    if (smem > ix->smem_per_block) return AP_OK;   // rows too long for per-warp tables: random start only
    AP_CUDA(cudaFuncSetAttribute(seed_dist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    AP_CUDA(cudaMemsetAsync(k.propn, 0, (size_t)n * 4));
    if (k.det) AP_CUDA(cudaMemsetAsync(k.prop, 0xFF, (size_t)n * kPropCap * sizeof(uint2)));
    seed_dist_kernel<<<(n + kSeedWarps - 1) / kSeedWarps, kSeedWarps * 32, smem>>>(k, ix->meta, ix->rec_build, cand, tabn - 1, 32 - log2u(tabn), shared_pairs);
    knn_merge_kernel<<<(n + 3) / 4, 128>>>(k);
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaDeviceSynchronize());
    *launches += 7;
    return AP_OK;
}

int build_run(ap_index *ix, const ap_build_opts *opts_in, ap_build_stats *stats) {
    ap_build_opts o{};
    if (opts_in) o = *opts_in;
    const uint32_t iters = o.iterations ? o.iterations : 6;
    const float scale = o.dense_scale != 0.f ? o.dense_scale : 7.0f;
    const uint32_t n = ix->n;
    if (n < 2) return fail(AP_ERR_ARG, "a graph needs at least 2 documents");
    AP_CUDA(cudaSetDevice(ix->device));
    AP_TRY(ensure_build_copy(ix, scale));
    const auto t0 = std::chrono::high_resolution_clock::now();
    DevBuf db;
    Knn k{};
    k.n = n;
    // one allocation for the whole k-NN phase (lists, samples, participant lists, inboxes, dense tiles)
    const uint32_t batch = std::min<uint32_t>(n, 1u << 18);   // nodes per batch of dense tiles
    {
        auto r256 = [](size_t b) { return (std::max<size_t>(b, 16) + 255) / 256 * 256; };
        const size_t total = 2 * r256((size_t)n * kK * 4) + r256((size_t)n * 64 * 4) + r256((size_t)n * 16) + r256((size_t)n * kPart * 4) +
                             r256((size_t)n * 8) + r256((size_t)n * kPropCap * sizeof(uint2)) + r256((size_t)n * 4) + r256(32) +
                             r256((size_t)batch * kPart * kNewMax * 4);
        uint8_t *slab;
        AP_TRY(db.alloc(&slab, total));
        db.donate(slab, total);
    }
    AP_TRY(db.alloc(&k.ids, (size_t)n * kK)); AP_TRY(db.alloc(&k.dis, (size_t)n * kK));
    AP_TRY(db.alloc(&k.samp, (size_t)n * 64)); AP_TRY(db.alloc(&k.scnt, (size_t)n * 4));
    AP_TRY(db.alloc(&k.plist, (size_t)n * kPart)); AP_TRY(db.alloc(&k.pcnt, (size_t)n * 2));
    AP_TRY(db.alloc(&k.prop, (size_t)n * kPropCap)); AP_TRY(db.alloc(&k.propn, n));
    AP_TRY(db.alloc(&k.stats, 4));
    AP_CUDA(cudaMemset(k.stats, 0, 32));
    k.det = (o.flags & AP_BUILD_DETERMINISTIC) ? 1u : 0u;
    float *power = ix->power;
    if (!power) { AP_CUDA(cudaMalloc(&ix->power, (size_t)n * 4)); power = ix->power; }
    uint32_t launches = 0;
    AP_TRY(norms_run(ix, power)); ++launches;
    knn_init_kernel<<<(uint32_t)(((size_t)n * kK + 255) / 256), 256>>>(k, o.seed ? o.seed : 20261125u); ++launches;
    const uint32_t shared_pairs = (o.flags & AP_BUILD_SHARED_PAIRS) ? 1u : 0u;
    float *D;   // dense tiles of a node batch; the seeded start borrows the memory for its posting lists
    AP_TRY(db.alloc(&D, (size_t)batch * kPart * kNewMax));
    if (!(o.flags & AP_BUILD_RANDOM_START))
        AP_TRY(seed_run(ix, k, o.seed_take ? std::min<uint32_t>(o.seed_take, 32u) : 4u, shared_pairs, &launches, D, (size_t)batch * kPart * kNewMax * sizeof(float)));

    uint32_t *err = ix->d_ctl + 1;

    JoinArgs ja{};
    ja.plist = k.plist; ja.pcnt = k.pcnt; ja.meta = ix->meta; ja.rec = ix->rec_build; ja.D = D; ja.knn_dis = k.dis;
    ja.prop = k.prop; ja.propn = k.propn; ja.stats = k.stats; ja.err = err;
    ja.prop_per = std::min<uint32_t>(kPropPerMax, o.proposals ? o.proposals : 4);
    ja.shared_pairs = shared_pairs; ja.det = k.det;
    const uint32_t tabn = pow2_at_least(2 * (ix->max_ns + ix->max_nb), 64);
    ja.tab_mask = tabn - 1; ja.tab_shift = 32 - log2u(tabn);
    // two CTAs per SM: tables for up to 4 hashed rows, the 32 x 64 distance tile, the rest is arena
    const size_t per_cta = ix->smem_per_sm / 2 - 1024 - 10240 /* static: dense tile + bookkeeping */;
    // key lines of a group are 1, 2 or 4 wide; four tables may take up to 40 % of the CTA's shared memory
    ja.groups = 8 * (size_t)tabn * 4 <= per_cta * 2 / 5 ? 4u : (8 * (size_t)tabn * 2 <= per_cta / 3 ? 2u : 1u);
    {
        uint32_t max_term = 0;
        AP_TRY(max_term_run(ix, &max_term));
        ja.gen_shift = (o.flags & AP_BUILD_WIPE_TABLES) ? 0u : gen_shift_for(max_term, (kNewMax + ja.groups - 1) / ja.groups);
    }
    ja.o_tab = 0; ja.o_dm = 8 * tabn * ja.groups; ja.o_arena = (ja.o_dm + 4 * kNewMax * kPart + 127) / 128 * 128;
    if (per_cta <= ja.o_arena + 8u * (pad2(ix->max_ns) + pad2(ix->max_nb)) * 2)
        return fail(AP_ERR_LIMIT, "rows of %u + %u terms leave no room for a local join in shared memory", ix->max_ns, ix->max_nb);
    ja.arena_bytes = (uint32_t)std::min<size_t>((per_cta - ja.o_arena) / 128 * 128, 512u * 1024u);
    const size_t join_smem = ja.o_arena + ja.arena_bytes;
    auto join_kernel = ja.groups == 4 ? join_sparse_kernel<4> : (ja.groups == 2 ? join_sparse_kernel<2> : join_sparse_kernel<1>);
    AP_CUDA(cudaFuncSetAttribute(join_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)join_smem));
    const size_t simt_smem = (size_t)kNewMax * kDenseBytes;
    AP_CUDA(cudaFuncSetAttribute(join_dense_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)simt_smem));

    const uint32_t wblocks = (n + 7) / 8;  // warp-per-node kernels, 256 threads
    struct Events {   // released on every return path
        cudaEvent_t e[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
        ~Events() { for (auto x : e) if (x) cudaEventDestroy(x); }
    } evs;
    cudaEvent_t *ev = evs.e;
    for (int i = 0; i < 5; ++i) AP_CUDA(cudaEventCreate(&ev[i]));
    float phase_ms[4] = {0, 0, 0, 0};  // sample + lists, dense tiles, sparse + proposals, merge
    uint32_t it = 0;
    unsigned long long prev_updates = 0;
    const bool trace = (o.flags & AP_BUILD_TRACE) != 0;   // per-round progress on stderr
    for (; it < iters; ++it) {
        AP_CUDA(cudaMemsetAsync(k.scnt, 0, (size_t)n * 16));
        AP_CUDA(cudaMemsetAsync(k.propn, 0, (size_t)n * 4));
        if (k.det) {
            AP_CUDA(cudaMemsetAsync(k.prop, 0xFF, (size_t)n * kPropCap * sizeof(uint2)));
            AP_CUDA(cudaMemsetAsync(k.samp, 0xFF, (size_t)n * 64 * 4));
        }
        AP_CUDA(cudaEventRecord(ev[0]));
        knn_sample_kernel<<<wblocks, 256>>>(k, it);
        if (k.det) { knn_rev_decode_kernel<<<(uint32_t)(((size_t)n * 32 + 255) / 256), 256>>>(k, it); ++launches; }
        knn_plist_kernel<<<wblocks, 256>>>(k, ix->meta, ja.arena_bytes);
        launches += 2;
        AP_CUDA(cudaEventRecord(ev[1]));
        for (uint32_t node0 = 0; node0 < n; node0 += batch) {
            const uint32_t nodes = std::min(batch, n - node0);
            if (o.flags & AP_BUILD_SIMT_JOIN) join_dense_simt_kernel<<<nodes, 256, simt_smem>>>(node0, nodes, k.plist, k.pcnt, ix->meta, ix->rec_build, D);
            else AP_TRY(join_dense_tc_launch(ix, node0, nodes, k.plist, k.pcnt, D, 0));
            if (node0 == 0) AP_CUDA(cudaEventRecord(ev[2]));
            ja.node0 = node0; ja.nodes = nodes;
            join_kernel<<<nodes, kJoinThreads, join_smem>>>(ja);
            launches += 2;
        }
        AP_CUDA(cudaEventRecord(ev[3]));
        knn_merge_kernel<<<(n + 3) / 4, 128>>>(k); ++launches;
        AP_CUDA(cudaEventRecord(ev[4]));
        AP_CUDA(cudaGetLastError());
        unsigned long long st[4];
        AP_CUDA(cudaMemcpy(st, k.stats, 32, cudaMemcpyDeviceToHost));
        for (int ph = 0; ph < 4; ++ph) { float ms = 0.f; cudaEventElapsedTime(&ms, ev[ph], ev[ph + 1]); phase_ms[ph] += ms; }
        const unsigned long long upd = st[1] - prev_updates;
        prev_updates = st[1];
        if (trace) fprintf(stderr, "round %u: %.2f %% of the list entries replaced, %llu distances so far, %llu proposals dropped\n", it,
                           100.0 * (double)upd / ((double)n * kK), st[0], st[2]);
        if (it >= 3 && upd < (unsigned long long)n * kK / 1000) { ++it; break; }  // < 0.1 % of the entries changed
    }
    if (shared_pairs && (o.flags & AP_BUILD_REVERSE_PASS)) {
        AP_CUDA(cudaMemsetAsync(k.propn, 0, (size_t)n * 4));
        if (k.det) AP_CUDA(cudaMemsetAsync(k.prop, 0xFF, (size_t)n * kPropCap * sizeof(uint2)));
        knn_reverse_kernel<<<(uint32_t)(((size_t)n * kK + 255) / 256), 256>>>(k);
        knn_merge_kernel<<<(n + 3) / 4, 128>>>(k);
        launches += 2;
    }
    AP_CUDA(cudaDeviceSynchronize());
    const auto t1 = std::chrono::high_resolution_clock::now();

    // The lists go to the pruning step where they lie unless the caller wants them kept; its scratch is carved out of
    // the k-NN phase's dead buffers (the sample lists take the cleaned ids, the inboxes and the dense tiles the rest).
    const bool keep = (o.flags & AP_BUILD_KEEP_KNN) != 0;
    uint32_t *knn_ids = k.samp;
    const float *knn_dis = k.dis;
    if (keep) {
        if (!ix->knn_ids) AP_CUDA(cudaMalloc(&ix->knn_ids, (size_t)n * kK * 4));
        if (!ix->knn_dis) AP_CUDA(cudaMalloc(&ix->knn_dis, (size_t)n * kK * 4));
        knn_ids = ix->knn_ids; knn_dis = ix->knn_dis;
        AP_CUDA(cudaMemcpyAsync(ix->knn_dis, k.dis, (size_t)n * kK * 4, cudaMemcpyDeviceToDevice));
    }
    knn_finish_kernel<<<(uint32_t)(((size_t)n * kK + 255) / 256), 256>>>(k, knn_ids); ++launches;
    {
        DevBuf pdb;
        pdb.donate(k.prop, (size_t)n * kPropCap * sizeof(uint2));
        pdb.donate(D, (size_t)batch * kPart * kNewMax * sizeof(float));
        pdb.donate(k.plist, (size_t)n * kPart * 4);
        AP_TRY(prune_run_in(pdb, ix, knn_ids, knn_dis, power, nullptr, nullptr, &launches, o.flags));
    }
    const auto t2 = std::chrono::high_resolution_clock::now();

    uint32_t ew = 0;
    AP_CUDA(cudaMemcpy(&ew, err, 4, cudaMemcpyDeviceToHost));
    if (ew) { cudaMemset(err, 0, 4); return fail(AP_ERR_DEVICE, "a build kernel raised error word %u (a bounded wait ran out)", ew); }
    if (stats) {
        unsigned long long st[4];
        AP_CUDA(cudaMemcpy(st, k.stats, 32, cudaMemcpyDeviceToHost));
        stats->seconds_knn = std::chrono::duration<double>(t1 - t0).count();
        stats->seconds_prune = std::chrono::duration<double>(t2 - t1).count();
        stats->seconds_total = std::chrono::duration<double>(t2 - t0).count();
        stats->distance_evals = st[0]; stats->list_updates = st[1]; stats->iterations_run = it; stats->launches = launches;
        stats->proposal_overflows = (uint32_t)st[2];
        stats->rows_gathered = st[3];
        // phase times in 10 us units: sample + lists, dense tiles (first batch), sparse + proposals, merge
        for (int ph = 0; ph < 3; ++ph) stats->phase_10us[ph] = (uint32_t)(phase_ms[ph + 1] * 100.f);
    }
    if (!keep) { cudaFree(ix->knn_ids); cudaFree(ix->knn_dis); ix->knn_ids = nullptr; ix->knn_dis = nullptr; }   // lists of an earlier build
    // the build-time copy is no longer needed once the graph exists
    if (!(o.flags & AP_BUILD_KEEP_KNN)) { cudaFree(ix->rec_build); ix->rec_build = nullptr; ix->build_scale = 0.f; ix->dense_src = nullptr; }
    return AP_OK;
}

}  // namespace apoe

using namespace apoe;

extern "C" {

int ap_index_build(ap_index *ix, const ap_build_opts *opts, ap_build_stats *stats) {
    if (!ix) return fail(AP_ERR_ARG, "null index");
    return build_run(ix, opts, stats);
}

int ap_index_get_knn(const ap_index *ix, uint32_t *ids, float *dis, float *power) {
    if (!ix) return fail(AP_ERR_ARG, "null index");
    if (!ix->knn_ids || !ix->knn_dis || !ix->power) return fail(AP_ERR_STATE, "no k-NN lists kept: build with AP_BUILD_KEEP_KNN");
    AP_CUDA(cudaSetDevice(ix->device));
    if (ids) AP_CUDA(cudaMemcpy(ids, ix->knn_ids, (size_t)ix->n * kK * 4, cudaMemcpyDeviceToHost));
    if (dis) AP_CUDA(cudaMemcpy(dis, ix->knn_dis, (size_t)ix->n * kK * 4, cudaMemcpyDeviceToHost));
    if (power) AP_CUDA(cudaMemcpy(power, ix->power, (size_t)ix->n * 4, cudaMemcpyDeviceToHost));
    return AP_OK;
}

int ap_index_norms(ap_index *ix, float *out) {
    if (!ix || !out) return fail(AP_ERR_ARG, "null argument");
    AP_CUDA(cudaSetDevice(ix->device));
    AP_TRY(ensure_build_copy(ix, ix->build_scale != 0.f ? ix->build_scale : 7.0f));
    if (!ix->power) AP_CUDA(cudaMalloc(&ix->power, (size_t)ix->n * 4));
    AP_TRY(norms_run(ix, ix->power));
    AP_CUDA(cudaMemcpy(out, ix->power, (size_t)ix->n * 4, cudaMemcpyDeviceToHost));
    return AP_OK;
}

int ap_index_prune(ap_index *ix, const uint32_t *knn_ids, const float *knn_dis, const float *power, uint32_t flags,
                   uint32_t *new_list, uint32_t *keyword_edges, uint32_t *rows) {
    if (!ix || !knn_ids || !knn_dis || !power) return fail(AP_ERR_ARG, "null argument");
    const uint32_t n = ix->n;
    for (size_t i = 0; i < (size_t)n * kK; ++i)
        if (knn_ids[i] >= n) return fail(AP_ERR_ARG, "k-NN entry %zu = %u is not a document id", i, knn_ids[i]);
    AP_CUDA(cudaSetDevice(ix->device));
    if (!ix->rec_build) return fail(AP_ERR_STATE, "the index was created without AP_CREATE_FOR_BUILD");
    DevBuf db;
    uint32_t *d_knn, *d_nl, *d_kw; float *d_dis, *d_pow;
    AP_TRY(db.alloc(&d_knn, (size_t)n * kK)); AP_TRY(db.alloc(&d_dis, (size_t)n * kK)); AP_TRY(db.alloc(&d_pow, n));
    AP_TRY(db.alloc(&d_nl, (size_t)n * AP_DEGREE)); AP_TRY(db.alloc(&d_kw, (size_t)n * 33));
    AP_CUDA(cudaMemcpy(d_knn, knn_ids, (size_t)n * kK * 4, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMemcpy(d_dis, knn_dis, (size_t)n * kK * 4, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMemcpy(d_pow, power, (size_t)n * 4, cudaMemcpyHostToDevice));
    uint32_t launches = 0;
    AP_TRY(prune_run(ix, d_knn, d_dis, d_pow, d_nl, d_kw, &launches, flags));
    if (new_list) AP_CUDA(cudaMemcpy(new_list, d_nl, (size_t)n * AP_DEGREE * 4, cudaMemcpyDeviceToHost));
    if (keyword_edges) AP_CUDA(cudaMemcpy(keyword_edges, d_kw, (size_t)n * 33 * 4, cudaMemcpyDeviceToHost));
    if (rows) AP_CUDA(cudaMemcpy(rows, ix->graph, (size_t)n * AP_ROW * 4, cudaMemcpyDeviceToHost));
    return AP_OK;
}

// Test hook: dense join tiles of the given participant lists, by the tensor-core kernel (use_tc != 0) or the
// CUDA-core kernel.  plist: nodes x 64 ids, pcnt: nodes x 2 (new rows, rows), both host; out: nodes x 64 x 32 floats
// (entries outside the lists' extents are left at zero).
int ap_debug_join_dense(ap_index *ix, uint32_t nodes, const uint32_t *plist, const uint32_t *pcnt, int use_tc, float *out) {
    if (!ix || !plist || !pcnt || !out || nodes == 0) return fail(AP_ERR_ARG, "null argument");
    if (!ix->rec_build) return fail(AP_ERR_STATE, "the index was created without AP_CREATE_FOR_BUILD");
    for (uint32_t v = 0; v < nodes; ++v) {
        const uint32_t nn = pcnt[2 * v], rows = pcnt[2 * v + 1];
        if (nn > (uint32_t)kNewMax || rows > (uint32_t)kPart || nn > rows || rows - nn > 32) return fail(AP_ERR_ARG, "bad extents for node %u", v);
        for (uint32_t j = 0; j < rows; ++j) if (plist[(size_t)v * kPart + j] >= ix->n) return fail(AP_ERR_ARG, "participant out of range");
    }
    AP_CUDA(cudaSetDevice(ix->device));
    DevBuf db;
    uint32_t *d_pl, *d_pc; float *d_D;
    AP_TRY(db.alloc(&d_pl, (size_t)nodes * kPart)); AP_TRY(db.alloc(&d_pc, (size_t)nodes * 2));
    AP_TRY(db.alloc(&d_D, (size_t)nodes * kPart * kNewMax));
    AP_CUDA(cudaMemcpy(d_pl, plist, (size_t)nodes * kPart * 4, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMemcpy(d_pc, pcnt, (size_t)nodes * 8, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMemset(d_D, 0, (size_t)nodes * kPart * kNewMax * 4));
    // the kernels index plist / pcnt by absolute node id: node0 = 0 here
    if (use_tc) AP_TRY(join_dense_tc_launch(ix, 0, nodes, d_pl, d_pc, d_D, 0));
    else {
        const size_t simt_smem = (size_t)kNewMax * kDenseBytes;
        AP_CUDA(cudaFuncSetAttribute(join_dense_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)simt_smem));
        join_dense_simt_kernel<<<nodes, 256, simt_smem>>>(0, nodes, d_pl, d_pc, ix->meta, ix->rec_build, d_D);
    }
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaDeviceSynchronize());
    uint32_t ew = 0;
    AP_CUDA(cudaMemcpy(&ew, ix->d_ctl + 1, 4, cudaMemcpyDeviceToHost));
    if (ew) { cudaMemset(ix->d_ctl + 1, 0, 4); return fail(AP_ERR_DEVICE, "join kernel raised error word %u (a bounded wait ran out)", ew); }
    AP_CUDA(cudaMemcpy(out, d_D, (size_t)nodes * kPart * kNewMax * 4, cudaMemcpyDeviceToHost));
    return AP_OK;
}

}  // extern "C"
