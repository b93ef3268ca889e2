/*
 * apoe_oracle.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C, CPU restatement of the Allan-Poe reference algorithms for the
 * hybrid graph index: fp16 conversion, the fused dense + sparse + BM25 score
 * (with the reference's fp16 accumulation order), weight auto-normalisation,
 * the greedy beam search (all weight subsets, keyword and KG variants), the
 * hybrid norm, RNG-IP pruning with keyword-aware neighbour recycling, the
 * final 40-wide row assembly, entry-point selection, and an exact OpenMP
 * brute-force hybrid top-k.
 *
 * It is the checker for the CUDA library, never the thing shipped: only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg may load
 * it.  Every function cites the reference file:line it follows (paths are
 * relative to the reference project's root).
 *
 * Parity status: the reference ships no tests and no golden vectors; this
 * file is pinned against outputs of the reference's own CUDA kernels captured
 * on a B200 (tests/golden/).  Where the reference has a data race or reads
 * uninitialised memory the order used here is stated at the spot.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define DIM 1024
#define INF_DIS 1000000.0f
#define EMPTY 0xFFFFFFFFu
#define HASHLEN 1024
#define ROW 40        /* index.poe row width: 32 graph slots + count + 7 keyword edges */
#define DEG 32
#define KNN 64
#define MAX_ITER 1000 /* query.cu:7 */
#define HASH_RESET 4  /* query.cu:16 */
#define KEYWORD 32    /* query.cu:18 */

/* ------------------------------------------------------------------ */
/* IEEE binary16 helpers (bit patterns in uint16_t)                    */
/* ------------------------------------------------------------------ */
static float g_h2f[65536];
static int g_h2f_ready = 0;

static float h2f_slow(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ff, o;
    if (e == 0) {
        if (m == 0) o = s;
        else {
            int sh = 0;
            while (!(m & 0x400)) { m <<= 1; sh++; }
            m &= 0x3ff;
            o = s | ((uint32_t)(113 - sh) << 23) | (m << 13);
        }
    } else if (e == 31) o = s | 0x7f800000u | (m << 13);
    else o = s | ((e + 112) << 23) | (m << 13);
    float f; memcpy(&f, &o, 4); return f;
}
static void h2f_init(void) {
    if (g_h2f_ready) return;
    for (uint32_t i = 0; i < 65536; i++) g_h2f[i] = h2f_slow((uint16_t)i);
    g_h2f_ready = 1;
}
static inline float h2f(uint16_t h) { return g_h2f[h]; }

/* double -> half, round-to-nearest-even, one rounding */
static inline uint16_t d2h(double d) {
    uint64_t b; memcpy(&b, &d, 8);
    uint16_t sign = (uint16_t)((b >> 48) & 0x8000u);
    uint32_t be = (uint32_t)((b >> 52) & 0x7ff);
    uint64_t m = b & 0xFFFFFFFFFFFFFull;
    if (be == 0x7ff) return (uint16_t)(sign | 0x7c00u | (m ? 0x200u : 0));
    if (be == 0) return sign;
    int e = (int)be - 1023;
    if (e > 15) return (uint16_t)(sign | 0x7c00u);
    if (e >= -14) {
        uint64_t keep = m >> 42, rem = m & ((1ull << 42) - 1), half = 1ull << 41;
        uint32_t h = ((uint32_t)(e + 15) << 10) | (uint32_t)keep;
        if (rem > half || (rem == half && (keep & 1))) h++;
        return (uint16_t)(sign | h);
    }
    if (e < -25) return sign;
    uint64_t full = m | (1ull << 52);
    int shift = 28 - e; /* 43..53 */
    uint64_t keep = full >> shift, rem = full & ((1ull << shift) - 1), half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (keep & 1))) keep++;
    return (uint16_t)(sign | (uint16_t)keep);
}
static inline uint16_t h_mul(uint16_t a, uint16_t b) { return d2h((double)h2f(a) * (double)h2f(b)); }
static inline uint16_t h_add(uint16_t a, uint16_t b) { return d2h((double)h2f(a) + (double)h2f(b)); }
static inline uint16_t h_fma(uint16_t a, uint16_t b, uint16_t c) {
    return d2h((double)h2f(a) * (double)h2f(b) + (double)h2f(c));
}

/* include/utils.cuh:78-83 (f2h: __float2half, round to nearest even) */
void orc_f2h(const float *in, uint16_t *out, size_t n) {
    h2f_init();
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = d2h((double)in[i]);
}
void orc_h2f(const uint16_t *in, float *out, size_t n) {
    h2f_init();
    for (size_t i = 0; i < n; i++) out[i] = h2f(in[i]);
}

/* ------------------------------------------------------------------ */
/* Score pieces                                                        */
/* ------------------------------------------------------------------ */

/*
 * Dense inner product exactly as the reference's warp computes it
 * (src/query.cu:538-554, src/index.cu:250-266,629-644): lane l owns the
 * 4-half chunks j = l, l+32, ..., l+224; per chunk two half2 multiply-adds;
 * then a 16-8-4-2-1 shfl_down tree in half2 and a final hadd(x, y).
 * fused != 0: the multiply-add pairs are single-rounding HFMA2;
 * fused == 0: separately rounded HMUL2 then HADD2.
 */
static uint16_t dense_ip_half(const uint16_t *q, const uint16_t *v, int fused) {
    uint16_t ax[32], ay[32];
    for (int l = 0; l < 32; l++) {
        uint16_t x = 0, y = 0;
        for (int k = 0; k < 8; k++) {
            const uint16_t *qq = q + 4 * (l + 32 * k), *vv = v + 4 * (l + 32 * k);
            if (fused) {
                x = h_fma(qq[0], vv[0], x); y = h_fma(qq[1], vv[1], y);
                x = h_fma(qq[2], vv[2], x); y = h_fma(qq[3], vv[3], y);
            } else {
                x = h_add(x, h_mul(qq[0], vv[0])); y = h_add(y, h_mul(qq[1], vv[1]));
                x = h_add(x, h_mul(qq[2], vv[2])); y = h_add(y, h_mul(qq[3], vv[3]));
            }
        }
        ax[l] = x; ay[l] = y;
    }
    for (int mask = 16; mask > 0; mask >>= 1)
        for (int l = 0; l < mask; l++) { ax[l] = h_add(ax[l], ax[l + mask]); ay[l] = h_add(ay[l], ay[l + mask]); }
    return h_add(ax[0], ay[0]);
}

/*
 * Per-lane partial of a sparse inner product (include/utils.cuh:299-340):
 * lane l walks row 1 at j = l, l+32, ...; each term is looked up in row 2
 * (strictly ascending, bit 31 of a row-2 id is the keyword flag and is masked
 * for the comparison).  *hit is raised when a matched row-2 id carries the
 * flag.  fma != 0: res = fmaf(v2, v1, res); else res += v2 * v1.
 */
static float sparse_lane(const uint32_t *idx1, const float *val1, uint32_t n1, const uint32_t *idx2,
                         const float *val2, uint32_t n2, int lane, int fma, int *hit) {
    float res = 0.0f;
    for (uint32_t j = (uint32_t)lane; j < n1; j += 32) {
        uint32_t t = idx1[j];
        uint32_t lo = 0, hi = n2;
        while (lo < hi) {
            uint32_t mid = (lo + hi) >> 1;
            if ((idx2[mid] & 0x7FFFFFFFu) < t) lo = mid + 1; else hi = mid;
        }
        if (lo < n2 && (idx2[lo] & 0x7FFFFFFFu) == t) {
            if (fma) res = fmaf(val2[lo], val1[j], res);
            else { volatile float p = val2[lo] * val1[j]; res += p; }
            if (hit && (idx2[lo] & 0x80000000u)) *hit = 1;
        }
    }
    return res;
}

static float tree32(float *s) {
    for (int mask = 16; mask > 0; mask >>= 1)
        for (int l = 0; l < mask; l++) s[l] = s[l] + s[l + mask];
    return s[0];
}

typedef struct {
    uint32_t n;
    const uint16_t *dense; /* n x DIM half bits */
    const uint32_t *s_off, *s_idx; const float *s_val;
    const uint32_t *b_off, *b_idx; const float *b_val;
} csr_set;

/* flags */
#define F_DENSE 1
#define F_SPARSE 2
#define F_BM25 4
#define F_KEYWORD 8
#define F_KG 16
#define F_UNFUSED_DENSE 32 /* HMUL2+HADD2 instead of HFMA2 */
#define F_NOFMA_SPARSE 64  /* mul then add instead of FFMA */

/*
 * Fused distance of query row qi against document x
 * (src/query.cu:538-555 and its seven siblings): the dense half result and
 * the tree-reduced sparse+BM25 partials are combined in double because the
 * reference writes `1.0 - ...` with a double literal.
 */
static float fused_dis(const csr_set *c, const csr_set *q, uint32_t qi, uint32_t x, int flags, int *key_hit) {
    double r = 1.0;
    if (flags & F_DENSE) {
        uint16_t h = dense_ip_half(q->dense + (size_t)qi * DIM, c->dense + (size_t)x * DIM, !(flags & F_UNFUSED_DENSE));
        r -= (double)h2f(h);
    }
    if (flags & (F_SPARSE | F_BM25)) {
        float lanes[32];
        int fma = !(flags & F_NOFMA_SPARSE);
        for (int l = 0; l < 32; l++) {
            float s = 0.0f, b = 0.0f;
            if (flags & F_SPARSE)
                s = sparse_lane(c->s_idx + c->s_off[x], c->s_val + c->s_off[x], c->s_off[x + 1] - c->s_off[x],
                                q->s_idx + q->s_off[qi], q->s_val + q->s_off[qi], q->s_off[qi + 1] - q->s_off[qi], l, fma, NULL);
            if (flags & F_BM25)
                b = sparse_lane(c->b_idx + c->b_off[x], c->b_val + c->b_off[x], c->b_off[x + 1] - c->b_off[x],
                                q->b_idx + q->b_off[qi], q->b_val + q->b_off[qi], q->b_off[qi + 1] - q->b_off[qi], l, fma, key_hit);
            lanes[l] = ((flags & F_SPARSE) && (flags & F_BM25)) ? (s + b) : ((flags & F_SPARSE) ? s : b);
        }
        r -= (double)tree32(lanes);
    }
    return (float)r;
}

/* ------------------------------------------------------------------ */
/* Visited set: include/utils.cuh:282-297                              */
/* ------------------------------------------------------------------ */
static uint32_t hash_insert(uint32_t *tab, uint32_t key) {
    uint32_t idx = (key ^ (key >> 10)) & (HASHLEN - 1);
    for (int i = 0; i < HASHLEN; i++) {
        if (tab[idx] == EMPTY) { tab[idx] = key; return 1; }
        if (tab[idx] == key) return 0;
        idx = (idx + 1) & (HASHLEN - 1);
    }
    return 0;
}

/*
 * The reference's shared-memory bitonic network (include/utils.cuh:147-165
 * and siblings): for each (stride, step) every k < len/2 compares positions
 * u and d and swaps when key[u] > key[d]; pairs with d >= len are skipped.
 * Ties never swap, so the outcome on equal keys is fixed by the network.
 */
typedef struct { float dis; uint32_t id, a, b; } ent_f;
static void bitonic_f(ent_f *e, uint32_t len) {
    for (uint32_t stride = 1; stride < len; stride <<= 1)
        for (uint32_t step = stride; step > 0; step >>= 1)
            for (uint32_t k = 0; k < len / 2; k++) {
                uint32_t a = 2 * step * (k / step), b = k % step;
                uint32_t u = (step == stride) ? (a + step - 1 - b) : (a + b), d = a + b + step;
                if (d < len && e[u].dis > e[d].dis) { ent_f t = e[u]; e[u] = e[d]; e[d] = t; }
            }
}
typedef struct { uint32_t key, val; } ent_u;
static void bitonic_u(ent_u *e, uint32_t len) {
    for (uint32_t stride = 1; stride < len; stride <<= 1)
        for (uint32_t step = stride; step > 0; step >>= 1)
            for (uint32_t k = 0; k < len / 2; k++) {
                uint32_t a = 2 * step * (k / step), b = k % step;
                uint32_t u = (step == stride) ? (a + step - 1 - b) : (a + b), d = a + b + step;
                if (d < len && e[u].key > e[d].key) { ent_u t = e[u]; e[u] = e[d]; e[d] = t; }
            }
}

/* ------------------------------------------------------------------ */
/* Greedy beam search: src/query.cu:414-570 (+ 277-1268 subsets,       */
/* 1271-1483 keyword, 1541-1779 KG)                                    */
/* ------------------------------------------------------------------ */
typedef struct {
    const uint32_t *e2e_off, *e2e_idx;     /* entity -> entity CSR */
    const uint32_t *e2d_off, *e2d_idx;     /* entity -> doc CSR    */
    const uint32_t *qe_off, *qe_idx;       /* query  -> entity CSR */
    float kg_weight;
} kg_set;

/*
 * merge_top / merge_top_keyword / merge_top_kg (src/query.cu:181-275,1485-1538).
 * pool[0..topm) and stg[0..32) are both ascending.  Pool element i moves to
 * i + #{stg <= it}; staged element j moves to j + #{pool < it}; ranks >= topm
 * are dropped.  Keyword variant: a pool element pushed out whose id word has
 * bit 0 set is appended to the 32-slot ring `kw` (the reference tests
 * `id & 0x40000000 != 0`, which C parses as `id & 1`; kept as is).  The
 * reference appends with an atomic counter from racing threads; the order used
 * here is ascending pool index.
 */
static void merge_top(ent_f *pool, ent_f *stg, uint32_t topm, ent_f *kw, uint32_t *kw_num, ent_f *scratch) {
    for (uint32_t i = 0; i < topm; i++) scratch[i].id = EMPTY, scratch[i].dis = -1.0f;
    for (uint32_t i = 0; i < topm; i++) {
        uint32_t r = 0;
        while (r < 32 && stg[r].dis <= pool[i].dis) r++;
        uint32_t pos = i + r;
        if (pos < topm) scratch[pos] = pool[i];
        else if (kw && (pool[i].id & 1u)) {
            uint32_t t = (*kw_num)++;
            kw[t % KEYWORD].id = pool[i].id & 0x3FFFFFFFu;
            kw[t % KEYWORD].dis = pool[i].dis;
        }
    }
    for (uint32_t j = 0; j < 32; j++) {
        uint32_t lo = 0, hi = topm;
        while (lo < hi) { uint32_t mid = (lo + hi) >> 1; if (pool[mid].dis < stg[j].dis) lo = mid + 1; else hi = mid; }
        uint32_t pos = j + lo;
        if (pos < topm) scratch[pos] = stg[j];
    }
    memcpy(pool, scratch, sizeof(ent_f) * topm);
}

typedef struct {
    uint64_t expansions, evaluations;
} search_counts;

static void search_one(const csr_set *c, const csr_set *q, uint32_t qi, const uint32_t *graph, const uint32_t *ep,
                       uint32_t topm, int flags, const kg_set *kg, uint32_t *out_id, float *out_dis,
                       search_counts *cnt) {
    uint32_t hash[HASHLEN];
    ent_f *pool = (ent_f *)malloc(sizeof(ent_f) * (topm + 32) * 2);
    ent_f *stg = pool + topm, *scratch = pool + topm + 32;
    ent_f kw[KEYWORD];
    uint32_t kw_num = 0;
    const int keyword = (flags & F_KEYWORD) != 0, kgm = (flags & F_KG) != 0;
    const uint32_t idmask = keyword ? 0x3FFFFFFFu : 0x7FFFFFFFu;
    /* the reference leaves the keyword side list uninitialised; defined here as empty */
    for (int i = 0; i < KEYWORD; i++) { kw[i].id = 0x3FFFFFFFu; kw[i].dis = INF_DIS; }
    memset(hash, 0xFF, sizeof(hash));
    for (uint32_t i = 0; i < topm; i++) { pool[i].id = EMPTY; pool[i].dis = INF_DIS; pool[i].a = EMPTY; pool[i].b = 0; }
    uint64_t evals = 0, expans = 0;

    if (!kgm) {
        /* query.cu:440-485 */
        for (int j = 0; j < 32; j++) { stg[j].id = ep[j]; stg[j].a = EMPTY; stg[j].b = 0; hash_insert(hash, ep[j]); }
        for (int j = 0; j < 32; j++) {
            int hit = 0;
            stg[j].dis = fused_dis(c, q, qi, stg[j].id, flags, keyword ? &hit : NULL);
            if (hit) stg[j].id |= 0x40000000u;
            evals++;
        }
        bitonic_f(stg, 32);
        for (uint32_t i = 0; i < (topm < 32 ? topm : 32); i++) pool[i] = stg[i];
    } else {
        /* query.cu:1577-1643: docs of the query's entities first (thread 0, in
         * CSR order), then entry points (the reference claims slots with an
         * atomic counter from 32 racing threads; ascending j here), scored,
         * entity-seeded docs get -kg_weight, then one sort of the filled prefix.
         * Slots beyond topm+32 are dropped as in the reference. */
        uint32_t n = 0;
        for (uint32_t i = kg->qe_off[qi]; i < kg->qe_off[qi + 1]; i++) {
            uint32_t e = kg->qe_idx[i];
            for (uint32_t j = kg->e2d_off[e]; j < kg->e2d_off[e + 1]; j++) {
                uint32_t d = kg->e2d_idx[j];
                if (hash_insert(hash, d) != 0 && n < topm + 32) { pool[n].id = d; pool[n].a = e; pool[n].b = 0; n++; }
            }
        }
        if (n < topm) {
            for (int j = 0; j < 32; j++)
                if (hash_insert(hash, ep[j]) != 0) {
                    uint32_t t = n++;
                    if (t < topm + 32) { pool[t].id = ep[j]; pool[t].a = EMPTY; pool[t].b = 0; }
                }
        }
        uint32_t m = n < topm + 32 ? n : topm + 32;
        for (uint32_t i = 0; i < m; i++) {
            pool[i].dis = fused_dis(c, q, qi, pool[i].id, flags, NULL);
            if (pool[i].a != EMPTY) pool[i].dis -= kg->kg_weight;
            evals++;
        }
        bitonic_f(pool, m);
        /* staging slots the seeding did not fill hold no defined value in the
         * reference (uninitialised shared memory); defined here as empty */
        for (uint32_t i = (m > topm ? m : topm); i < topm + 32; i++) { pool[i].id = EMPTY; pool[i].dis = INF_DIS; pool[i].a = EMPTY; pool[i].b = 0; }
    }

    for (int it = 0; it < MAX_ITER; it++) {
        if ((it + 1) % HASH_RESET == 0) {
            memset(hash, 0xFF, sizeof(hash));
            for (uint32_t j = 0; j < topm + 32; j++) hash_insert(hash, pool[j].id & idmask);
        }
        uint32_t sel = EMPTY, slot = 0;
        for (uint32_t j = 0; j < topm; j++)
            if ((pool[j].id & 0x80000000u) == 0) { sel = pool[j].id; pool[j].id |= 0x80000000u; slot = j; break; }
        if (sel == EMPTY) break;
        expans++;
        const uint32_t node = sel & idmask;
        const uint32_t *row = graph + (size_t)node * ROW;
        /* duplicates inside one row: the lowest slot is the one that counts as new */
        for (int j = 0; j < 32; j++) {
            stg[j].id = row[j];
            stg[j].dis = hash_insert(hash, row[j]) == 0 ? INF_DIS : 0.0f;
            stg[j].a = EMPTY;
            stg[j].b = kgm ? pool[slot].b + 1 : 0;
        }
        if (keyword) {
            /* query.cu:1413-1425: already-visited slots are refilled from the
             * explored node's keyword edges (claimed in ascending slot order) */
            uint32_t claimed = 0;
            for (int j = 0; j < 32; j++)
                if (stg[j].dis > 1.0f) {
                    uint32_t t = claimed++;
                    if (t < row[DEG]) {
                        uint32_t cand = row[DEG + 1 + t];
                        if (hash_insert(hash, cand) != 0) { stg[j].id = cand; stg[j].dis = 0.0f; }
                    }
                }
        }
        if (kgm && pool[slot].b < 3 && pool[slot].a != EMPTY) {
            /* query.cu:1697-1735.  kg_cur_id is never assigned in the reference;
             * here it is the pool slot of the node being expanded.  The staged
             * ids are not sorted at this point, so the reference's binary search
             * over them is restated as what it can actually find: a probe that
             * follows the same halving steps. */
            const uint32_t ent = pool[slot].a;
            for (uint32_t j = kg->e2e_off[ent]; j < kg->e2e_off[ent + 1]; j++) {
                uint32_t ne = kg->e2e_idx[j];
                for (uint32_t k = kg->e2d_off[ne]; k < kg->e2d_off[ne + 1]; k++) {
                    uint32_t val = kg->e2d_idx[k], tmp = 32, res = 0;
                    while (tmp > 1) {
                        uint32_t half = tmp / 2;
                        uint32_t cand = stg[res + half].id & 0x3FFFFFFFu;
                        res += (cand < val) ? half : 0;
                        tmp -= half;
                    }
                    res += ((stg[res].id & 0x3FFFFFFFu) < val);
                    if (res <= 31 && (stg[res].id & 0x3FFFFFFFu) == val && stg[res].dis < 1.0f) {
                        stg[res].dis = 2.0f;
                        stg[res].a = ne;
                    }
                }
            }
            uint32_t claimed = 0;
            const uint32_t deg = kg->e2e_off[ent + 1] - kg->e2e_off[ent];
            for (int j = 0; j < 32; j++)
                if (stg[j].dis > 3.0f) {
                    uint32_t t = claimed++;
                    if (t < deg) {
                        uint32_t ne = kg->e2e_idx[kg->e2e_off[ent] + t];
                        for (uint32_t k = kg->e2d_off[ne]; k < kg->e2d_off[ne + 1]; k++) {
                            uint32_t cand = kg->e2d_idx[k];
                            if ((sel & 0x3FFFFFFFu) == cand) continue;
                            if (hash_insert(hash, cand) != 0) {
                                stg[j].id = cand; stg[j].dis = 2.0f; stg[j].a = ne; stg[j].b = pool[slot].b + 1;
                                break;
                            }
                        }
                    }
                }
        }
        for (int j = 0; j < 32; j++) {
            if (stg[j].dis < (kgm ? 3.0f : 1.0f)) {
                int hit = 0;
                float d = fused_dis(c, q, qi, stg[j].id, flags, keyword ? &hit : NULL);
                if (kgm && stg[j].dis > 1.0f) d = d - (kg->kg_weight / (float)stg[j].b);
                stg[j].dis = d;
                if (hit) stg[j].id |= 0x40000000u;
                evals++;
            }
        }
        bitonic_f(stg, 32);
        merge_top(pool, stg, topm, keyword ? kw : NULL, &kw_num, scratch);
    }

    if (!keyword) {
        for (uint32_t i = 0; i < topm; i++) { out_id[i] = pool[i].id & 0x7FFFFFFFu; out_dis[i] = pool[i].dis; }
    } else {
        /* query.cu:1465-1481: keyword hits first (pool order), then the side
         * list sorted by distance; slots past the 32-entry side list are
         * out-of-bounds reads in the reference and are emitted as empty here */
        bitonic_f(kw, KEYWORD);
        uint32_t n = 0;
        for (uint32_t i = 0; i < topm; i++)
            if (pool[i].id & 0x40000000u) { out_id[n] = pool[i].id & 0x3FFFFFFFu; out_dis[n] = pool[i].dis; n++; }
        for (uint32_t i = n; i < topm; i++) {
            uint32_t s = i - n;
            if (s < KEYWORD) { out_id[i] = kw[s].id & 0x3FFFFFFFu; out_dis[i] = kw[s].dis; }
            else { out_id[i] = 0x3FFFFFFFu; out_dis[i] = INF_DIS; }
        }
    }
    if (cnt) { cnt->expansions = expans; cnt->evaluations = evals; }
    free(pool);
}

/*
 * Batched search.  graph: n x 40 u32 (index.poe rows), ep: 32 entry points.
 * Queries arrive already scaled by the effective weights and converted to
 * half (src/query.cu:1871-1881, 2001-2002); bit 31 of a query BM25 id marks a
 * required keyword (src/query.cu:1828-1843).
 * counts (may be NULL): per query {expansions, evaluations}.
 */
int orc_search(uint32_t n, const uint16_t *dense, const uint32_t *s_off, const uint32_t *s_idx, const float *s_val,
               const uint32_t *b_off, const uint32_t *b_idx, const float *b_val, uint32_t nq, const uint16_t *qdense,
               const uint32_t *qs_off, const uint32_t *qs_idx, const float *qs_val, const uint32_t *qb_off,
               const uint32_t *qb_idx, const float *qb_val, const uint32_t *graph, const uint32_t *ep, uint32_t cands,
               int flags, const uint32_t *e2e_off, const uint32_t *e2e_idx, const uint32_t *e2d_off,
               const uint32_t *e2d_idx, const uint32_t *qe_off, const uint32_t *qe_idx, float kg_weight,
               uint32_t *out_ids, float *out_dis, uint64_t *counts) {
    h2f_init();
    csr_set c = {n, dense, s_off, s_idx, s_val, b_off, b_idx, b_val};
    csr_set q = {nq, qdense, qs_off, qs_idx, qs_val, qb_off, qb_idx, qb_val};
    kg_set kg = {e2e_off, e2e_idx, e2d_off, e2d_idx, qe_off, qe_idx, kg_weight};
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t qi = 0; qi < nq; qi++) {
        search_counts sc;
        search_one(&c, &q, qi, graph, ep, cands, flags, (flags & F_KG) ? &kg : NULL, out_ids + (size_t)qi * cands,
                   out_dis + (size_t)qi * cands, &sc);
        if (counts) { counts[2 * (size_t)qi] = sc.expansions; counts[2 * (size_t)qi + 1] = sc.evaluations; }
    }
    return 0;
}

/* Distances of explicit (query, doc) pairs with the reference's arithmetic. */
int orc_fused_distances(uint32_t n, const uint16_t *dense, const uint32_t *s_off, const uint32_t *s_idx,
                        const float *s_val, const uint32_t *b_off, const uint32_t *b_idx, const float *b_val,
                        uint32_t nq, const uint16_t *qdense, const uint32_t *qs_off, const uint32_t *qs_idx,
                        const float *qs_val, const uint32_t *qb_off, const uint32_t *qb_idx, const float *qb_val,
                        size_t npairs, const uint32_t *pair_q, const uint32_t *pair_d, int flags, float *out) {
    h2f_init();
    csr_set c = {n, dense, s_off, s_idx, s_val, b_off, b_idx, b_val};
    csr_set q = {nq, qdense, qs_off, qs_idx, qs_val, qb_off, qb_idx, qb_val};
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < npairs; i++) out[i] = fused_dis(&c, &q, pair_q[i], pair_d[i], flags, NULL);
    return 0;
}

/* ------------------------------------------------------------------ */
/* Exact fp32 pieces: src/query.cu:148-178, 1847-1869                  */
/* ------------------------------------------------------------------ */
static float dot_f32_seq(const float *a, const float *b, uint32_t dim) {
    float r = 0.0f;
    for (uint32_t i = 0; i < dim; i++) r += a[i] * b[i];
    return r;
}
static float sparse_merge_f32(const uint32_t *i1, const float *v1, uint32_t n1, const uint32_t *i2, const float *v2,
                              uint32_t n2) {
    float r = 0.0f;
    uint32_t p1 = 0, p2 = 0;
    while (p1 < n1 && p2 < n2) {
        uint32_t a = i1[p1], b = i2[p2] & 0x7FFFFFFFu;
        if (a < b) p1++;
        else if (a > b) p2++;
        else { r += v1[p1] * v2[p2]; p1++; p2++; }
    }
    return r;
}

/*
 * Weight auto-normalisation (src/query.cu:1847-1869): per-path maxima of the
 * exact inner products over the first min(100, n) docs x first min(100, nq)
 * queries; the two weaker paths are scaled up to the strongest path's maximum.
 * w = {sparse, bm25, dense} in, rescaled out.
 */
int orc_effective_weights(uint32_t n, const float *dense, const uint32_t *s_off, const uint32_t *s_idx,
                          const float *s_val, const uint32_t *b_off, const uint32_t *b_idx, const float *b_val,
                          uint32_t nq, const float *qdense, const uint32_t *qs_off, const uint32_t *qs_idx,
                          const float *qs_val, const uint32_t *qb_off, const uint32_t *qb_idx, const float *qb_val,
                          float *w_sparse, float *w_bm25, float *w_dense) {
    /* the reference indexes docs by the query-bounded loop variable and queries
     * by the doc-bounded one; both bounds are 100 whenever n, nq >= 100 */
    uint32_t nd = nq < 100 ? nq : 100, nqq = n < 100 ? n : 100;
    if (nd > n) nd = n;
    if (nqq > nq) nqq = nq;
    float r1 = 0, r2 = 0, r3 = 0; /* minima of the negated inner products */
    int first = 1;
    for (uint32_t bb = 0; bb < nqq; bb++)
        for (uint32_t aa = 0; aa < nd; aa++) {
            float d = -dot_f32_seq(dense + (size_t)aa * DIM, qdense + (size_t)bb * DIM, DIM);
            float s = -sparse_merge_f32(s_idx + s_off[aa], s_val + s_off[aa], s_off[aa + 1] - s_off[aa],
                                        qs_idx + qs_off[bb], qs_val + qs_off[bb], qs_off[bb + 1] - qs_off[bb]);
            float b = -sparse_merge_f32(b_idx + b_off[aa], b_val + b_off[aa], b_off[aa + 1] - b_off[aa],
                                        qb_idx + qb_off[bb], qb_val + qb_off[bb], qb_off[bb + 1] - qb_off[bb]);
            if (first || d < r1) r1 = d;
            if (first || s < r2) r2 = s;
            if (first || b < r3) r3 = b;
            first = 0;
        }
    if ((-r2) > (-r3) && (-r2) > (-r1)) { *w_bm25 *= (r2 / r3); *w_dense *= (r2 / r1); }
    else if ((-r3) > (-r2) && (-r3) > (-r1)) { *w_sparse *= (r3 / r2); *w_dense *= (r3 / r1); }
    else if ((-r1) > (-r2) && (-r1) > (-r3)) { *w_sparse *= (r1 / r2); *w_bm25 *= (r1 / r3); }
    return 0;
}

/*
 * Exact brute-force hybrid top-k on fp32 data (score of src/query.cu:148-178,
 * `1 - sum` of src/index.cu:50-79), OpenMP over document blocks.  Queries are
 * already weight-scaled.  Sparse parts go through a transposed (term-major)
 * copy of the corpus rows so each query only touches the postings of its own
 * terms.  Ties are broken by ascending doc id.  Returns 0.
 */
typedef struct { float d; uint32_t id; } hit_t;
static inline int hit_less(hit_t a, hit_t b) { return a.d < b.d || (a.d == b.d && a.id < b.id); }
static void heap_push(hit_t *h, uint32_t k, uint32_t *sz, hit_t x) { /* max-heap of the k best */
    if (*sz < k) {
        uint32_t i = (*sz)++;
        h[i] = x;
        while (i > 0) { uint32_t p = (i - 1) / 2; if (hit_less(h[p], h[i])) { hit_t t = h[p]; h[p] = h[i]; h[i] = t; i = p; } else break; }
    } else if (hit_less(x, h[0])) {
        h[0] = x;
        uint32_t i = 0;
        for (;;) {
            uint32_t l = 2 * i + 1, r = l + 1, m = i;
            if (l < k && hit_less(h[m], h[l])) m = l;
            if (r < k && hit_less(h[m], h[r])) m = r;
            if (m == i) break;
            hit_t t = h[m]; h[m] = h[i]; h[i] = t; i = m;
        }
    }
}
static int hit_cmp(const void *a, const void *b) {
    hit_t x = *(const hit_t *)a, y = *(const hit_t *)b;
    return hit_less(x, y) ? -1 : (hit_less(y, x) ? 1 : 0);
}

static void transpose_csr(uint32_t n, const uint32_t *off, const uint32_t *idx, const float *val, uint32_t vocab,
                          uint32_t **t_off, uint32_t **t_doc, float **t_val) {
    size_t nnz = off[n];
    uint32_t *to = (uint32_t *)calloc((size_t)vocab + 2, 4);
    for (size_t i = 0; i < nnz; i++) to[idx[i] + 2]++;
    for (uint32_t t = 0; t < vocab; t++) to[t + 2] += to[t + 1];
    uint32_t *td = (uint32_t *)malloc(4 * (nnz ? nnz : 1));
    float *tv = (float *)malloc(4 * (nnz ? nnz : 1));
    for (uint32_t d = 0; d < n; d++)
        for (uint32_t j = off[d]; j < off[d + 1]; j++) { uint32_t p = to[idx[j] + 1]++; td[p] = d; tv[p] = val[j]; }
    *t_off = to; *t_doc = td; *t_val = tv;
}

int orc_bruteforce(uint32_t n, const float *dense, const uint32_t *s_off, const uint32_t *s_idx, const float *s_val,
                   const uint32_t *b_off, const uint32_t *b_idx, const float *b_val, uint32_t nq, const float *qdense,
                   const uint32_t *qs_off, const uint32_t *qs_idx, const float *qs_val, const uint32_t *qb_off,
                   const uint32_t *qb_idx, const float *qb_val, int flags, uint32_t topk, uint32_t *out_ids,
                   float *out_dis, int *threads_used) {
    uint32_t vs = 0, vb = 0;
    for (size_t i = 0; i < s_off[n]; i++) if (s_idx[i] >= vs) vs = s_idx[i] + 1;
    for (size_t i = 0; i < b_off[n]; i++) if (b_idx[i] >= vb) vb = b_idx[i] + 1;
    uint32_t *ts_off = NULL, *ts_doc = NULL, *tb_off = NULL, *tb_doc = NULL;
    float *ts_val = NULL, *tb_val = NULL;
    if (flags & F_SPARSE) transpose_csr(n, s_off, s_idx, s_val, vs, &ts_off, &ts_doc, &ts_val);
    if (flags & F_BM25) transpose_csr(n, b_off, b_idx, b_val, vb, &tb_off, &tb_doc, &tb_val);
    const uint32_t QB = 16;
    int nthreads = omp_get_max_threads();
    if (threads_used) *threads_used = nthreads;
    float *score = (float *)malloc(sizeof(float) * (size_t)QB * n);
    for (uint32_t q0 = 0; q0 < nq; q0 += QB) {
        uint32_t qn = nq - q0 < QB ? nq - q0 : QB;
#pragma omp parallel for schedule(static)
        for (uint32_t d = 0; d < n; d++) {
            const float *x = dense + (size_t)d * DIM;
            for (uint32_t qq = 0; qq < qn; qq++) {
                float acc = 0.0f;
                if (flags & F_DENSE) {
                    const float *y = qdense + (size_t)(q0 + qq) * DIM;
                    float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    for (uint32_t i = 0; i < DIM; i += 8)
                        for (int u = 0; u < 8; u++) a8[u] += x[i + u] * y[i + u];
                    acc = ((a8[0] + a8[1]) + (a8[2] + a8[3])) + ((a8[4] + a8[5]) + (a8[6] + a8[7]));
                }
                score[(size_t)qq * n + d] = acc;
            }
        }
#pragma omp parallel for schedule(dynamic, 1)
        for (uint32_t qq = 0; qq < qn; qq++) {
            uint32_t qi = q0 + qq;
            float *sc = score + (size_t)qq * n;
            if (flags & F_SPARSE)
                for (uint32_t j = qs_off[qi]; j < qs_off[qi + 1]; j++) {
                    uint32_t t = qs_idx[j];
                    if (t >= vs) continue;
                    float w = qs_val[j];
                    for (uint32_t p = ts_off[t]; p < ts_off[t + 1]; p++) sc[ts_doc[p]] += w * ts_val[p];
                }
            if (flags & F_BM25)
                for (uint32_t j = qb_off[qi]; j < qb_off[qi + 1]; j++) {
                    uint32_t t = qb_idx[j] & 0x7FFFFFFFu;
                    if (t >= vb) continue;
                    float w = qb_val[j];
                    for (uint32_t p = tb_off[t]; p < tb_off[t + 1]; p++) sc[tb_doc[p]] += w * tb_val[p];
                }
            hit_t *heap = (hit_t *)malloc(sizeof(hit_t) * topk);
            uint32_t sz = 0;
            for (uint32_t d = 0; d < n; d++) { hit_t h = {1.0f - sc[d], d}; heap_push(heap, topk, &sz, h); }
            qsort(heap, sz, sizeof(hit_t), hit_cmp);
            for (uint32_t i = 0; i < topk; i++) {
                out_ids[(size_t)qi * topk + i] = i < sz ? heap[i].id : EMPTY;
                out_dis[(size_t)qi * topk + i] = i < sz ? heap[i].d : INF_DIS;
            }
            free(heap);
        }
    }
    free(score);
    free(ts_off); free(ts_doc); free(ts_val); free(tb_off); free(tb_doc); free(tb_val);
    return 0;
}

/* ------------------------------------------------------------------ */
/* Build side                                                          */
/* ------------------------------------------------------------------ */

/*
 * Squared norm of the hybrid vector (src/index.cu:483-534): per 32-element
 * chunk of the dense row the squares are formed and tree-summed in half, the
 * 32 chunk sums are kept as floats; sparse and BM25 squares are tree-summed in
 * float per 32-chunk and all added onto chunk slot 0; the 32 slots are then
 * summed left to right.
 */
int orc_cal_power(uint32_t n, const uint16_t *dense, const uint32_t *s_off, const float *s_val, const uint32_t *b_off,
                  const float *b_val, float *power) {
    h2f_init();
#pragma omp parallel for schedule(static)
    for (uint32_t d = 0; d < n; d++) {
        float slot[32];
        for (int ch = 0; ch < 32; ch++) {
            uint16_t v[32];
            for (int l = 0; l < 32; l++) { uint16_t x = dense[(size_t)d * DIM + ch * 32 + l]; v[l] = h_mul(x, x); }
            for (int mask = 16; mask > 0; mask >>= 1)
                for (int l = 0; l < mask; l++) v[l] = h_add(v[l], v[l + mask]);
            slot[ch] = h2f(v[0]);
        }
        const uint32_t *offs[2] = {s_off, b_off};
        const float *vals[2] = {s_val, b_val};
        for (int w = 0; w < 2; w++) {
            uint32_t a = offs[w][d], e = offs[w][d + 1];
            for (uint32_t base = a; base < e; base += 32) {
                float t[32];
                for (uint32_t l = 0; l < 32; l++) { float x = base + l < e ? vals[w][base + l] : 0.0f; t[l] = x * x; }
                slot[0] += tree32(t);
            }
        }
        float r = 0.0f;
        for (int i = 0; i < 32; i++) r += slot[i];
        power[d] = r;
    }
    return 0;
}

/* Entry points: the 32 smallest norms, ties by id (src/index.cu:916-925). */
typedef struct { float p; uint32_t id; } pw_t;
static int pw_cmp(const void *a, const void *b) {
    pw_t x = *(const pw_t *)a, y = *(const pw_t *)b;
    if (x.p < y.p) return -1;
    if (x.p > y.p) return 1;
    return x.id < y.id ? -1 : (x.id > y.id ? 1 : 0);
}
int orc_entry_points(uint32_t n, const float *power, uint32_t *ep) {
    pw_t *a = (pw_t *)malloc(sizeof(pw_t) * n);
    for (uint32_t i = 0; i < n; i++) { a[i].p = power[i]; a[i].id = i; }
    qsort(a, n, sizeof(pw_t), pw_cmp);
    for (uint32_t i = 0; i < 32; i++) ep[i] = a[i < n ? i : n - 1].id;
    free(a);
    return 0;
}

/* build-side BM25 partial with the keyword probe (src/index.cu:128-153) */
static int in_sorted(const uint32_t *idx, uint32_t n, uint32_t t) {
    uint32_t lo = 0, hi = n;
    while (lo < hi) { uint32_t mid = (lo + hi) >> 1; if (idx[mid] < t) lo = mid + 1; else hi = mid; }
    return lo < n && idx[lo] == t;
}

/*
 * Inner product of two corpus rows as the pruning kernel forms it
 * (src/index.cu:629-644): half dense part (staged row = c, streamed row = s),
 * float sparse + BM25 lanes over s's terms looked up in c's rows; *kwflag is
 * raised when s owns a BM25 term that c lacks but `self` owns
 * (src/index.cu:144-149).
 */
static float prune_ip(const csr_set *c, uint32_t cnode, uint32_t snode, uint32_t self, int flags, int *kwflag) {
    uint16_t h = dense_ip_half(c->dense + (size_t)cnode * DIM, c->dense + (size_t)snode * DIM, !(flags & F_UNFUSED_DENSE));
    float lanes[32];
    int fma = !(flags & F_NOFMA_SPARSE);
    const uint32_t *ci = c->b_idx + c->b_off[cnode]; uint32_t cn = c->b_off[cnode + 1] - c->b_off[cnode];
    const uint32_t *bi = c->b_idx + c->b_off[self]; uint32_t bn = c->b_off[self + 1] - c->b_off[self];
    for (int l = 0; l < 32; l++) {
        float s = sparse_lane(c->s_idx + c->s_off[snode], c->s_val + c->s_off[snode], c->s_off[snode + 1] - c->s_off[snode],
                              c->s_idx + c->s_off[cnode], c->s_val + c->s_off[cnode], c->s_off[cnode + 1] - c->s_off[cnode], l, fma, NULL);
        float b = sparse_lane(c->b_idx + c->b_off[snode], c->b_val + c->b_off[snode], c->b_off[snode + 1] - c->b_off[snode],
                              ci, c->b_val + c->b_off[cnode], cn, l, fma, NULL);
        lanes[l] = s + b;
    }
    for (uint32_t j = c->b_off[snode]; j < c->b_off[snode + 1]; j++) {
        uint32_t t = c->b_idx[j];
        if (!in_sorted(ci, cn, t) && in_sorted(bi, bn, t)) { *kwflag = 1; break; }
    }
    return h2f(h) + tree32(lanes);
}

/*
 * RNG-IP joint pruning with keyword-aware neighbour recycling
 * (src/index.cu:539-714) followed by the reverse-edge scatter and the
 * 40-wide row assembly (src/index.cu:717-807).
 *
 * In:  knn[n][64] ids ascending by knn_dis[n][64]; power[n]; corpus rows with
 *      the dense part already scaled by 7 and converted to half
 *      (src/index.cu:836-840, 891).
 * Out: new_list[n][32] forward ids, kw_edge[n][33] (count + 32 ids),
 *      graph[n][40] final rows, detour[n][32] (scatter payload, for tests).
 * The reference scatters reverse edges with atomics from racing blocks; the
 * order used here is ascending source node, then ascending slot.
 * Row slots the reference never writes (33+count..39) are zero here.
 */
int orc_prune(uint32_t n, const uint16_t *dense, const uint32_t *s_off, const uint32_t *s_idx, const float *s_val,
              const uint32_t *b_off, const uint32_t *b_idx, const float *b_val, const uint32_t *knn,
              const float *knn_dis, const float *power, int flags, uint32_t *new_list, uint32_t *kw_edge,
              uint32_t *graph, uint32_t *detour_out) {
    h2f_init();
    csr_set c = {n, dense, s_off, s_idx, s_val, b_off, b_idx, b_val};
    uint32_t *detour_all = (uint32_t *)malloc(4 * (size_t)n * DEG);
#pragma omp parallel for schedule(dynamic, 8)
    for (uint32_t bid = 0; bid < n; bid++) {
        uint32_t nei0[KNN], nei1[KNN], nei2[KNN + 1];
        ent_u det[KNN];
        const uint32_t *g = knn + (size_t)bid * KNN;
        for (int j = 0; j < KNN; j++) { nei0[j] = g[j]; det[j].key = 0; det[j].val = g[j]; }
        /* detour counting, src/index.cu:572-597: pivot p < target t; t found at
         * slot r of p's list with a shorter p->t edge than bid->t */
        for (int p = 0; p < KNN; p++) {
            const uint32_t *pl = knn + (size_t)g[p] * KNN;
            for (int t = p + 1; t < KNN; t++) {
                int r = -1;
                for (int j = 0; j < KNN; j++) if (pl[j] == g[t]) { r = j; break; }
                if (r >= 0 && knn_dis[(size_t)g[p] * KNN + r] < knn_dis[(size_t)bid * KNN + t]) det[t].key++;
            }
        }
        bitonic_u(det, KNN);
        for (int j = 0; j < KNN; j++) nei0[j] = det[j].val;
        memset(nei2, 0, sizeof(nei2));
        nei1[0] = nei0[0];
        uint32_t tmp_id = 1, ipn = 1;
        while (ipn < KNN) {
            uint32_t cn = nei0[tmp_id];
            int cur_nei = 0, cur_nei2 = 0;
            int warp_flag[16];
            memset(warp_flag, 0, sizeof(warp_flag));
            for (uint32_t i = 0; i < ipn; i++) {
                /* the reference runs i on warp i % 16, in ascending order per warp */
                if (nei1[i] == EMPTY) continue;
                uint32_t sn = nei1[i];
                int kw = 0;
                float ip = prune_ip(&c, cn, sn, bid, flags, &kw);
                if (kw) warp_flag[i % 16] = 1;
                if (power[cn] < ip) cur_nei = 1;
                if (power[sn] < ip) nei1[i] = EMPTY;
                if (warp_flag[i % 16] != 1) cur_nei2 = 1;
            }
            if (cur_nei == 0) { nei1[ipn] = cn; ipn++; }
            if (cur_nei2 == 0) nei2[ipn] = 1; /* written after the increment, as in the reference */
            tmp_id++;
            if (tmp_id >= KNN) break;
        }
        uint32_t count = 0, i_neis;
        for (i_neis = 0; i_neis < ipn && count < DEG; i_neis++)
            if (nei1[i_neis] != EMPTY) nei0[count++] = nei1[i_neis];
        uint32_t *ke = kw_edge + (size_t)bid * 33;
        memset(ke, 0, 33 * 4);
        for (uint32_t i = i_neis; i < ipn; i++)
            if (nei2[i] == 1 && nei1[i] != EMPTY && ke[0] < 32) { ke[ke[0] + 1] = nei1[i]; ke[0]++; }
        for (int i = 0; i < DEG; i++) {
            new_list[(size_t)bid * DEG + i] = nei0[i];
            detour_all[(size_t)bid * DEG + i] = det[i].key;
        }
    }
    if (detour_out) memcpy(detour_out, detour_all, 4 * (size_t)n * DEG);

    /* reverse scatter, src/index.cu:699-711 */
    uint32_t *rnum = (uint32_t *)calloc(n, 4);
    uint32_t *rg = (uint32_t *)calloc((size_t)n * DEG * 2, 4);
    for (uint32_t bid = 0; bid < n; bid++)
        for (int i = 0; i < DEG; i++) {
            uint32_t t = new_list[(size_t)bid * DEG + i], dt = detour_all[(size_t)bid * DEG + i];
            uint32_t k = rnum[t]++;
            uint32_t *slot = rg + (size_t)t * DEG * 2 + (size_t)(k % DEG) * 2;
            if (k < DEG || slot[1] > dt) { slot[0] = bid; slot[1] = dt; }
        }

    /* final rows, src/index.cu:717-807 */
#pragma omp parallel for schedule(static)
    for (uint32_t bid = 0; bid < n; bid++) {
        uint32_t rv = rnum[bid] < DEG ? rnum[bid] : DEG;
        ent_u r[DEG];
        const uint32_t *nl = new_list + (size_t)bid * DEG;
        uint32_t *row = graph + (size_t)bid * ROW;
        memset(row, 0, ROW * 4);
        for (uint32_t i = 0; i < rv; i++) { r[i].key = rg[(size_t)bid * DEG * 2 + 2 * i]; r[i].val = rg[(size_t)bid * DEG * 2 + 2 * i + 1]; }
        bitonic_u(r, rv); /* by id */
        uint32_t dup[DEG];
        for (uint32_t i = 0; i < rv; i++) dup[i] = (i > 0 && r[i].key == r[i - 1].key);
        for (uint32_t i = 0; i < rv; i++) { uint32_t id = r[i].key; r[i].key = dup[i] ? EMPTY : r[i].val; r[i].val = id; }
        for (int i = 0; i < DEG / 2; i++) row[i] = nl[i];
        bitonic_u(r, rv); /* by detour, duplicates last */
        uint32_t cur = 0;
        uint32_t lim = rv < DEG / 2 ? DEG - rv : DEG / 2;
        for (uint32_t i = 0; i < rv; i++) {
            int found = 0;
            for (uint32_t j = 0; j < lim; j++) if (r[i].val == nl[j]) { found = 1; break; }
            if (!found) { uint32_t t = cur++; if (t < DEG / 2) row[DEG / 2 + t] = r[i].val; }
        }
        uint32_t placed = cur < DEG / 2 ? cur : DEG / 2;
        for (uint32_t i = 0; i < DEG / 2 - placed; i++) row[DEG / 2 + placed + i] = nl[i + DEG / 2];
        const uint32_t *ke = kw_edge + (size_t)bid * 33;
        cur = 0;
        for (uint32_t i = 0; i < ke[0]; i++) {
            int found = 0;
            for (int j = DEG / 2; j < DEG; j++) if (row[j] == ke[1 + i]) { found = 1; break; }
            if (!found) { uint32_t t = cur++; if (t < 7) row[DEG + t + 1] = ke[1 + i]; }
        }
        row[DEG] = cur < 7 ? cur : 7;
    }
    free(rnum); free(rg); free(detour_all);
    return 0;
}


/* ------------------------------------------------------------------ */
/* nDCG@k as the reference prints it: cal_precision, src/query.cu:111-145.
 * results: nq x stride ids (the first top_k of a row are used, as the host
 * copies them at src/query.cu:2070-2075); qrels as a CSR of relevant ids.
 * Everything accumulates in float, `1 / log2(float(j + 2))` per position,
 * DCG over the intersection of the sorted result ids and the sorted
 * relevant ids (multiset semantics of std::set_intersection), each common id
 * credited at its first position in the result row; a query without relevant
 * ids divides 0 by 0 exactly as the reference does (the figure becomes NaN). */
static int u32_cmp(const void *a, const void *b) {
    const uint32_t x = *(const uint32_t *)a, y = *(const uint32_t *)b;
    return x < y ? -1 : (x > y ? 1 : 0);
}
float orc_cal_precision(uint32_t nq, const uint32_t *results, uint32_t stride, uint32_t top_k, const uint32_t *qrel_off,
                        const uint32_t *qrel_ids) {
    float ndcg = 0.0f;
    uint32_t *tmp = (uint32_t *)malloc(sizeof(uint32_t) * (top_k ? top_k : 1));
    for (uint32_t i = 0; i < nq; ++i) {
        const uint32_t nrel = qrel_off[i + 1] - qrel_off[i];
        uint32_t *rel = (uint32_t *)malloc(sizeof(uint32_t) * (nrel ? nrel : 1));
        float idcg = 0.0f;
        for (uint32_t j = 0; j < nrel; ++j) idcg += (1 / log2f((float)(j + 2)));
        const uint32_t *row = results + (size_t)i * stride;
        memcpy(tmp, row, sizeof(uint32_t) * top_k);
        memcpy(rel, qrel_ids + qrel_off[i], sizeof(uint32_t) * nrel);
        qsort(tmp, top_k, sizeof(uint32_t), u32_cmp);
        qsort(rel, nrel, sizeof(uint32_t), u32_cmp);
        float dcg = 0.0f;
        uint32_t a = 0, b = 0;
        while (a < top_k && b < nrel) {           /* std::set_intersection */
            if (tmp[a] < rel[b]) ++a;
            else if (rel[b] < tmp[a]) ++b;
            else {
                const uint32_t x = tmp[a];
                for (uint32_t it = 0; it < top_k; ++it)
                    if (row[it] == x) { dcg += (1 / log2f((float)(it + 2))); break; }
                ++a; ++b;
            }
        }
        ndcg += (dcg / idcg);
        free(rel);
    }
    free(tmp);
    return ndcg / (float)nq;
}

int orc_num_threads(void) { return omp_get_max_threads(); }
int orc_version(void) { return 1; }
