// Exact hybrid top-k on the device: the ground truth that recall is measured against.
//
// The score is the reference's fused score (compute_hybrid_dis, src/query.cu:148-178: dense inner product + sparse
// inner product + BM25 inner product, distance = 1 - sum) over the documents as the index stores them (dense values
// rounded to half, sparse values in fp32) and the queries as the search sees them (weights folded in, dense rounded
// to half), accumulated in fp32.  Every (query, document) pair is scored; nothing is approximate.
//
//   1. exact_sparse_kernel  -- sparse + BM25 part through an inverted index of the corpus (term -> postings sorted by
//      document, built once per index with a radix sort): one CTA per (query, window of 8192 documents) adds the
//      postings of the query's terms into a shared-memory window, term after term (a fixed order, no atomics), and
//      stores the window to the scratch matrix S[query][document].
//   2. exact_dense_topk_kernel -- dense part as a Q x N x 1024 contraction on the 5th-generation tensor cores:
//      128 x 256 tiles, operands staged by tiled TMA loads (128-byte swizzle, four stages) from the fp16 query batch
//      and a contiguous fp16 copy of the corpus' dense rows, tcgen05.mma kind::f16 accumulating fp32 in tensor memory
//      (two 256-column accumulators, so the epilogue of one tile overlaps the MMAs of the next); the epilogue reads
//      the accumulator with tcgen05.ld, adds the tile of S, and keeps a running top-k per query row in registers.
//      A CTA owns one block of 128 queries and one slice of the documents; the per-slice lists are merged afterwards
//      by the key merge of the sharded search.
//
// Every load is issued by one CTA for itself alone; the tensor maps cover this GPU's own memory only.  Every wait is bounded and raises
// the index's error word instead of spinning.
#include <cuda.h>

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <mutex>

#include "apoe_common.cuh"

extern "C" int ap_merge_shard_keys(int device, uint32_t shards, uint32_t nq, uint32_t per_shard, const unsigned long long *keys,
                                   uint32_t top_k, uint32_t *out_ids, float *out_dis, void *stream);

namespace apoe {

constexpr int kBM = 128, kBN = 256, kBK = 64;            // tile: queries x documents x halves of K per stage
constexpr int kExStages = 4;
constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = kBN * kBK * 2, kExStageBytes = kABytes + kBBytes;   // 16 + 32 KB
constexpr int kKBlocks = AP_DIM / kBK;                   // 16
constexpr int kExThreads = 192;                          // warps 0-3 epilogue, warp 4 TMA producer, warp 5 MMA issue + tensor memory
constexpr int kTopMax = 16;                              // running list per query row (top_k <= 16)
constexpr uint32_t kExTmemCols = 512;
constexpr uint32_t kExWaitLimit = 1u << 22;
constexpr uint32_t kWindow = 8192;                       // documents per CTA of the sparse pass
constexpr uint32_t kFullMask = 0xFFFFFFFFu;

// ---------------------------------------------------------------------------------------------------------
// inverted index of the corpus
// ---------------------------------------------------------------------------------------------------------
struct Inverted {
    uint32_t vocab_s = 0, vocab = 0;     // sparse vocabulary, sparse + BM25 vocabulary (BM25 term t is term vocab_s + t)
    uint32_t *toff = nullptr;            // vocab + 1 posting offsets
    uint2 *post = nullptr;               // (document, value bits), ascending document inside a term
    size_t total = 0;
    __half *dense = nullptr;             // n x 1024 contiguous copy of the dense rows
    uint32_t n = 0;
};

__global__ void ex_count_kernel(uint32_t n, const uint64_t *__restrict__ meta, uint32_t *__restrict__ cnt) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= n) cnt[i] = i < n ? meta_ns(meta[i]) + meta_nb(meta[i]) : 0u;
}
__global__ void ex_maxid_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec, uint32_t *__restrict__ mx) {
    const uint32_t d = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (d >= n) return;
    const uint64_t m = meta[d];
    const uint2 *pr = reinterpret_cast<const uint2 *>(rec + meta_off16(m) * 16ull + kDenseBytes);
    const uint32_t ns = meta_ns(m), nb = meta_nb(m), pns = pad2(ns);
    uint32_t a = 0, b = 0;
    for (uint32_t j = lane; j < ns; j += 32) a = max(a, pr[j].x);
    for (uint32_t j = lane; j < nb; j += 32) b = max(b, pr[pns + j].x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { a = max(a, __shfl_xor_sync(kFullMask, a, o)); b = max(b, __shfl_xor_sync(kFullMask, b, o)); }
    if (lane == 0) { if (ns) atomicMax(mx + 0, a); if (nb) atomicMax(mx + 1, b); }
}
__global__ void ex_keys_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec, const uint32_t *__restrict__ off,
                               uint32_t vocab_s, unsigned long long *__restrict__ keys, uint32_t *__restrict__ vals, uint32_t *__restrict__ hist) {
    const uint32_t d = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (d >= n) return;
    const uint64_t m = meta[d];
    const uint2 *pr = reinterpret_cast<const uint2 *>(rec + meta_off16(m) * 16ull + kDenseBytes);
    const uint32_t ns = meta_ns(m), nb = meta_nb(m), pns = pad2(ns);
    const size_t o = off[d];
    for (uint32_t j = lane; j < ns + nb; j += 32) {
        const uint2 p = j < ns ? pr[j] : pr[pns + (j - ns)];
        const uint32_t term = j < ns ? p.x : vocab_s + p.x;
        keys[o + j] = ((unsigned long long)term << 32) | d;
        vals[o + j] = p.y;
        atomicAdd(hist + term, 1u);
    }
}
__global__ void ex_post_kernel(size_t total, const unsigned long long *__restrict__ keys, const uint32_t *__restrict__ vals, uint2 *__restrict__ post) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) post[i] = make_uint2((uint32_t)keys[i], vals[i]);
}
__global__ void ex_dense_copy_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ rec, uint4 *__restrict__ out) {
    const uint32_t d = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (d >= n) return;
    const uint4 *src = reinterpret_cast<const uint4 *>(rec + meta_off16(meta[d]) * 16ull);
#pragma unroll
    for (int k = 0; k < 4; ++k) out[(size_t)d * 128 + lane + 32 * k] = __ldg(src + lane + 32 * k);
}

struct ExBuf {   // device allocations released on every return path unless handed over
    std::vector<void *> ptrs;
    ~ExBuf() { for (void *p : ptrs) if (p) cudaFree(p); }
    template <class T> int alloc(T **out, size_t count) {
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, std::max<size_t>(count * sizeof(T), 16));
        if (e != cudaSuccess) return fail(AP_ERR_CUDA, "cudaMalloc of %zu bytes failed: %s", count * sizeof(T), cudaGetErrorString(e));
        ptrs.push_back(p); *out = (T *)p; return AP_OK;
    }
    void keep(void *p) { for (auto &q : ptrs) if (q == p) q = nullptr; }
};

static int build_inverted(ap_index *ix, Inverted **out) {
    if (ix->exact) { *out = static_cast<Inverted *>(ix->exact); return AP_OK; }
    const uint32_t n = ix->n;
    ExBuf db;
    uint32_t *cnt, *off, *mx;
    AP_TRY(db.alloc(&cnt, (size_t)n + 1)); AP_TRY(db.alloc(&off, (size_t)n + 1)); AP_TRY(db.alloc(&mx, 2));
    AP_CUDA(cudaMemset(mx, 0, 8));
    ex_count_kernel<<<n / 256 + 1, 256>>>(n, ix->meta, cnt);
    ex_maxid_kernel<<<(n + 7) / 8, 256>>>(n, ix->meta, ix->rec, mx);
    size_t tmp_bytes = 0;
    AP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, cnt, off, (int)(n + 1)));
    uint8_t *tmp; AP_TRY(db.alloc(&tmp, tmp_bytes));
    AP_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, cnt, off, (int)(n + 1)));
    uint32_t h_mx[2], total32 = 0;
    AP_CUDA(cudaMemcpy(h_mx, mx, 8, cudaMemcpyDeviceToHost));
    AP_CUDA(cudaMemcpy(&total32, off + n, 4, cudaMemcpyDeviceToHost));
    if (total32 >= (1u << 31)) return fail(AP_ERR_LIMIT, "%u postings: the exact scorer sorts up to 2^31 per index (shard the corpus)", total32);
    if (h_mx[0] >= (1u << 26) || h_mx[1] >= (1u << 26)) return fail(AP_ERR_LIMIT, "term ids up to %u / %u: the exact scorer indexes vocabularies below 2^26", h_mx[0], h_mx[1]);
    Inverted *inv = new Inverted();
    inv->n = n; inv->vocab_s = h_mx[0] + 1; inv->vocab = inv->vocab_s + h_mx[1] + 1; inv->total = total32;
    struct Holder { Inverted *p; ~Holder() { if (p) { cudaFree(p->toff); cudaFree(p->post); cudaFree(p->dense); delete p; } } } hold{inv};
    const size_t total = inv->total;
    uint32_t *hist;
    AP_TRY(db.alloc(&hist, (size_t)inv->vocab + 1));
    AP_CUDA(cudaMemset(hist, 0, ((size_t)inv->vocab + 1) * 4));
    unsigned long long *keys, *keys_s; uint32_t *vals, *vals_s;
    AP_TRY(db.alloc(&keys, total)); AP_TRY(db.alloc(&keys_s, total)); AP_TRY(db.alloc(&vals, total)); AP_TRY(db.alloc(&vals_s, total));
    ex_keys_kernel<<<(n + 7) / 8, 256>>>(n, ix->meta, ix->rec, off, inv->vocab_s, keys, vals, hist);
    AP_CUDA(cudaGetLastError());
    int end_bit = 33;
    while (end_bit < 64 && (1ull << (end_bit - 32)) < inv->vocab) ++end_bit;
    if (total) {
        size_t sort_bytes = 0;
        AP_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, keys, keys_s, vals, vals_s, (int)total, 0, end_bit));
        uint8_t *stmp; AP_TRY(db.alloc(&stmp, sort_bytes));
        AP_CUDA(cub::DeviceRadixSort::SortPairs(stmp, sort_bytes, keys, keys_s, vals, vals_s, (int)total, 0, end_bit));
    }
    AP_CUDA(cudaMalloc(&inv->toff, ((size_t)inv->vocab + 1) * 4));
    size_t scan_bytes = 0;
    AP_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, hist, inv->toff, (int)(inv->vocab + 1)));
    uint8_t *stmp2; AP_TRY(db.alloc(&stmp2, scan_bytes));
    AP_CUDA(cub::DeviceScan::ExclusiveSum(stmp2, scan_bytes, hist, inv->toff, (int)(inv->vocab + 1)));
    AP_CUDA(cudaMalloc(&inv->post, std::max<size_t>(total, 1) * sizeof(uint2)));
    if (total) ex_post_kernel<<<(uint32_t)((total + 255) / 256), 256>>>(total, keys_s, vals_s, inv->post);
    AP_CUDA(cudaMalloc(&inv->dense, (size_t)n * kDenseBytes));
    ex_dense_copy_kernel<<<(n + 7) / 8, 256>>>(n, ix->meta, ix->rec, reinterpret_cast<uint4 *>(inv->dense));
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaDeviceSynchronize());
    hold.p = nullptr;
    ix->exact = inv;
    *out = inv;
    return AP_OK;
}

void exact_release(ap_index *ix) {
    Inverted *inv = static_cast<Inverted *>(ix->exact);
    if (!inv) return;
    cudaFree(inv->toff); cudaFree(inv->post); cudaFree(inv->dense);
    delete inv;
    ix->exact = nullptr;
}

// ---------------------------------------------------------------------------------------------------------
// query batch: weights folded in (fp32 multiply, as src/query.cu:1871-1875), dense rounded to half
// ---------------------------------------------------------------------------------------------------------
__global__ void ex_query_kernel(uint32_t rows, uint32_t valid, const float *__restrict__ qdense, float w, uint2 *__restrict__ out) {
    const uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= rows) return;
    for (uint32_t i = lane; i < kDim / 4; i += 32) {
        uint2 v = make_uint2(0u, 0u);
        if (r < valid) {
            const float4 f = __ldg(reinterpret_cast<const float4 *>(qdense + (size_t)r * kDim) + i);
            v = make_uint2(pack_half2(__fmul_rn(f.x, w), __fmul_rn(f.y, w)), pack_half2(__fmul_rn(f.z, w), __fmul_rn(f.w, w)));
        }
        out[(size_t)r * (kDim / 4) + i] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------
// sparse + BM25 part
// ---------------------------------------------------------------------------------------------------------
struct SparseArgs {
    uint32_t n, ld;                // documents, row stride of S (a multiple of 256)
    uint32_t q0;                   // first query of the batch
    const uint32_t *qs_off, *qs_idx; const float *qs_val;
    const uint32_t *qb_off, *qb_idx; const float *qb_val;
    float w_sparse, w_bm25;
    uint32_t vocab_s, vocab;
    const uint32_t *toff; const uint2 *post;
    float *S;                      // [batch rows][ld]
    uint32_t keyword;              // only documents holding a flagged (bit 31) BM25 term of the query stay eligible
};
constexpr float kIneligible = -3.0e38f;   // S entry of a document the keyword filter excludes
constexpr int kSpThreads = 256, kSpTerms = 64;

__device__ __forceinline__ uint32_t lower_bound_doc(const uint2 *__restrict__ post, uint32_t lo, uint32_t hi, uint32_t doc) {
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (__ldg(&post[mid].x) < doc) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(kSpThreads) exact_sparse_kernel(const SparseArgs a) {
    __shared__ float win[kWindow];
    __shared__ uint8_t hit[kWindow];
    __shared__ uint32_t s_lo[kSpTerms], s_hi[kSpTerms], s_flag[kSpTerms];
    __shared__ float s_w[kSpTerms];
    const int tid = threadIdx.x;
    const uint32_t row = blockIdx.y, q = a.q0 + row;
    const uint32_t x0 = blockIdx.x * kWindow, x1 = min(x0 + kWindow, a.n);
    for (uint32_t i = tid; i < kWindow; i += kSpThreads) { win[i] = 0.0f; hit[i] = 0; }
    for (int sec = 0; sec < 2; ++sec) {
        const uint32_t *qoff = sec == 0 ? a.qs_off : a.qb_off, *qidx = sec == 0 ? a.qs_idx : a.qb_idx;
        const float *qval = sec == 0 ? a.qs_val : a.qb_val;
        const float w = sec == 0 ? a.w_sparse : a.w_bm25;
        if (w == 0.0f && !(sec == 1 && a.keyword)) continue;
        const uint32_t o = qoff[q], nt = qoff[q + 1] - o;
        for (uint32_t t0 = 0; t0 < nt; t0 += kSpTerms) {
            const uint32_t m = min((uint32_t)kSpTerms, nt - t0);
            __syncthreads();
            if (tid < (int)m) {
                const uint32_t raw = qidx[o + t0 + tid] & 0x7FFFFFFFu;    // bit 31 of a BM25 id is the keyword flag
                const uint32_t term = sec == 0 ? raw : a.vocab_s + raw;
                const bool known = sec == 0 ? raw < a.vocab_s : term < a.vocab;
                uint32_t lo = 0, hi = 0;
                if (known) {
                    const uint32_t b = a.toff[term], e = a.toff[term + 1];
                    lo = lower_bound_doc(a.post, b, e, x0);
                    hi = lower_bound_doc(a.post, lo, e, x1);
                }
                s_lo[tid] = lo; s_hi[tid] = hi;
                s_flag[tid] = (sec == 1 && a.keyword) ? (qidx[o + t0 + tid] >> 31) : 0u;
                s_w[tid] = __fmul_rn(qval[o + t0 + tid], w);
            }
            __syncthreads();
            for (uint32_t i = 0; i < m; ++i) {          // one term at a time: its postings name distinct documents
                const float wq = s_w[i];
                const bool flagged = s_flag[i] != 0;
                for (uint32_t p = s_lo[i] + tid; p < s_hi[i]; p += kSpThreads) {
                    const uint2 e = __ldg(a.post + p);
                    win[e.x - x0] = __fmaf_rn(wq, __uint_as_float(e.y), win[e.x - x0]);
                    if (flagged) hit[e.x - x0] = 1;
                }
                __syncthreads();
            }
        }
    }
    __syncthreads();
    float *dst = a.S + (size_t)row * a.ld + x0;
    for (uint32_t i = tid; i < kWindow && x0 + i < a.ld; i += kSpThreads) dst[i] = (a.keyword && !hit[i]) ? kIneligible : win[i];
}

// ---------------------------------------------------------------------------------------------------------
// dense part + top-k
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ex_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ex_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ex_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ex_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart; descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t ex_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16: D fp32 (bit 4), A and B fp16 K-major, N = 256 (bits 17-22 = N >> 3), M = 128 (bits 24-28 = M >> 4)
constexpr uint32_t kExIdesc = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

// Tiled TMA load of one box (inner coordinate x in elements: a multiple of 64 halves = 128 bytes, so always 16-byte
// aligned; y = row) into shared memory, completing on an mbarrier; one CTA, one destination.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst_smem)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool ex_wait(uint64_t *bar, uint32_t parity, uint32_t *err, uint32_t code) {
    for (uint32_t i = 0; i < kExWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, code);
    return false;
}
__device__ __forceinline__ uint32_t ex_f2ord(float f) { const uint32_t b = __float_as_uint(f); return (b & 0x80000000u) ? ~b : (b | 0x80000000u); }

struct DenseArgs {
    uint32_t n;                    // documents
    uint32_t tiles_n;              // ceil(n / 256)
    uint32_t splits;               // document slices (CTAs per block of 128 queries)
    uint32_t rows_valid;           // queries in this batch
    uint32_t q0, nq_total;         // first query of the batch, queries overall (layout of `part`)
    uint32_t top_k;
    uint32_t ld;                   // row stride of S
    const float *S;
    unsigned long long *part;      // [splits][nq_total][top_k] keys
    uint32_t *err;
};

__global__ void __launch_bounds__(kExThreads, 1) exact_dense_topk_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                         const __grid_constant__ CUtensorMap map_x, const DenseArgs a) {
    extern __shared__ __align__(1024) uint8_t ex_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(ex_smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[kExStages], empty_bar[kExStages], tfull_bar[2], tempty_bar[2];
    __shared__ uint32_t tmem_base_s;
    float *scratch = reinterpret_cast<float *>(smem + (size_t)kExStages * kExStageBytes);   // 32 x 128 distances of the epilogue
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t m_tile = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const uint32_t t0 = (uint32_t)((uint64_t)a.tiles_n * split / a.splits), t1 = (uint32_t)((uint64_t)a.tiles_n * (split + 1) / a.splits);

    if (tid == 0) {
        for (int s = 0; s < kExStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 4); }
        mbar_fence_init();
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kExTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    ex_fence_before();
    __syncthreads();
    ex_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 4) {
        // ---------------- TMA producer ---------------------------------------------------------------------
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t t = t0; t < t1 && ok; ++t) {
                for (int kb = 0; kb < kKBlocks && ok; ++kb, ++g) {
                    const uint32_t s = g % kExStages;
                    ok = ex_wait(&empty_bar[s], ((g / kExStages) & 1u) ^ 1u, a.err, 20u);
                    if (!ok) break;
                    uint8_t *stage = smem + (size_t)s * kExStageBytes;
                    mbar_arrive_expect_tx(&full_bar[s], kExStageBytes);
                    tma_load_2d(stage, &map_q, kb * kBK, (int)(m_tile * kBM), &full_bar[s]);
                    tma_load_2d(stage + kABytes, &map_x, kb * kBK, (int)(t * kBN), &full_bar[s]);
                }
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issue -------------------------------------------------------------------------
        if (lane == 0) {
            uint32_t g = 0, it = 0;
            bool ok = true;
            for (uint32_t t = t0; t < t1 && ok; ++t, ++it) {
                const uint32_t acc = it & 1u;
                ok = ex_wait(&tempty_bar[acc], ((it >> 1) & 1u) ^ 1u, a.err, 21u);
                if (!ok) break;
                ex_fence_after();
                for (int kb = 0; kb < kKBlocks && ok; ++kb, ++g) {
                    const uint32_t s = g % kExStages;
                    ok = ex_wait(&full_bar[s], (g / kExStages) & 1u, a.err, 22u);
                    if (!ok) break;
                    ex_fence_after();
                    const uint32_t a_base = smem_u32(smem + (size_t)s * kExStageBytes), b_base = a_base + kABytes;
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk)
                        ex_mma_f16(tmem_base + acc * 256, ex_desc_sw128(a_base + kk * 32), ex_desc_sw128(b_base + kk * 32), kExIdesc, (kb | kk) != 0 ? 1u : 0u);
                    ex_commit(&empty_bar[s]);     // the stage is free once these MMAs have read it
                }
                if (ok) ex_commit(&tfull_bar[acc]);
            }
        }
    } else {
        // ---------------- epilogue: warp w owns tensor-memory lanes 32w .. 32w+31 = query rows ----------------------
        const uint32_t row = m_tile * kBM + warp * 32 + lane;       // row of the batch
        const bool valid_row = row < a.rows_valid;
        unsigned long long best[kTopMax];
#pragma unroll
        for (int i = 0; i < kTopMax; ++i) best[i] = ~0ull;
        constexpr float kOpen = 2.9e38f;                             // below the 3.0e38 that marks an ineligible column
        float thr = kOpen;                                          // distance of the last kept entry
        const float *srow = a.S + (size_t)row * a.ld;
        uint32_t it = 0;
        bool ok = true;
        // The tile of S a row needs is read 32 columns (one 128-byte line) ahead of its use: the loads of the next chunk
        // are in flight while the current one is scored, the first chunk of the next tile while the last one is.
        float4 sbuf[2][8];
        auto fetch = [&](float4 (&dst)[8], uint32_t x0) {
            const float4 *sp = reinterpret_cast<const float4 *>(srow + x0);
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) dst[j4] = valid_row ? __ldg(sp + j4) : make_float4(0.f, 0.f, 0.f, 0.f);
        };
        if (t0 < t1) fetch(sbuf[0], t0 * kBN);
        for (uint32_t t = t0; t < t1 && ok; ++t, ++it) {
            const uint32_t acc = it & 1u;
            ok = ex_wait(&tfull_bar[acc], (it >> 1) & 1u, a.err, 23u);
            if (!ok) break;
            ex_fence_after();
#pragma unroll
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * warp) << 16) + acc * 256 + c * 32;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                    "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                if (c + 1 < kBN / 32) fetch(sbuf[(c + 1) & 1], t * kBN + (c + 1) * 32);
                else if (t + 1 < t1) fetch(sbuf[0], (t + 1) * kBN);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const uint32_t x0 = t * kBN + c * 32;
                if (valid_row) {
                    // pass 1, branch-free: distances of the 32 columns to this thread's scratch column, a mask of the
                    // ones that beat the current threshold; pass 2 (rare): insert those -- one copy of the insertion
                    // code per chunk instead of one per column keeps the loop inside the instruction cache
                    const uint32_t lim = a.n - min(a.n, x0);      // columns of this chunk that are documents
                    uint32_t mask = 0;
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        const float4 s4 = sbuf[c & 1][j4];
                        const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int j = j4 * 4 + u;
                            const float d = sv[u] > -1.0e38f ? 1.0f - (__uint_as_float(r[j]) + sv[u]) : 3.0e38f;
                            scratch[j * 128 + warp * 32 + lane] = d;
                            mask |= (d <= thr && (uint32_t)j < lim) ? (1u << j) : 0u;
                        }
                    }
                    while (mask) {
                        const int j = __ffs(mask) - 1;
                        mask &= mask - 1;
                        const float d = scratch[j * 128 + warp * 32 + lane];
                        if (d <= thr) {
                            unsigned long long key = ((unsigned long long)ex_f2ord(d) << 32) | (x0 + j);
                            if (key < best[kTopMax - 1]) {
#pragma unroll
                                for (int i = 0; i < kTopMax; ++i)
                                    if (key < best[i]) { const unsigned long long tmp = best[i]; best[i] = key; key = tmp; }
                                const uint32_t o = (uint32_t)(best[kTopMax - 1] >> 32);
                                thr = best[kTopMax - 1] == ~0ull ? kOpen : __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o);
                            }
                        }
                    }
                }
            }
            ex_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        }
        if (valid_row) {
            unsigned long long *out = a.part + ((size_t)split * a.nq_total + a.q0 + row) * a.top_k;
#pragma unroll
            for (int i = 0; i < kTopMax; ++i) if ((uint32_t)i < a.top_k) out[i] = best[i];
        }
    }
    ex_fence_before();
    __syncthreads();
    if (warp == 5) {
        ex_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kExTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_fn(EncodeTiledFn *out) {
    static std::mutex mu;
    static EncodeTiledFn cached = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        AP_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (!p || qres != cudaDriverEntryPointSuccess) return fail(AP_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled");
        cached = reinterpret_cast<EncodeTiledFn>(p);
    }
    *out = cached;
    return AP_OK;
}

// rows x 1024 halves, row-major; box = 64 halves (128 bytes, one swizzle span) x box_rows rows
static int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint32_t box_rows) {
    EncodeTiledFn fn;
    AP_TRY(encode_fn(&fn));
    const cuuint64_t dims[2] = {kDim, rows};
    const cuuint64_t strides[1] = {kDenseBytes};
    const cuuint32_t box[2] = {kBK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AP_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return AP_OK;
}

}  // namespace apoe

using namespace apoe;

extern "C" int ap_exact_topk_device(ap_index *ix, const ap_queries *q, float sparse_weight, float bm25_weight, float dense_weight,
                                    uint32_t flags, uint32_t top_k, uint32_t *out_ids, float *out_dis, void *stream_, ap_exact_stats *stats) {
    if (!ix || !q || !out_ids || !out_dis) return fail(AP_ERR_ARG, "null argument");
    if (q->nq == 0 || !q->dense || !q->sparse.off || !q->bm25.off) return fail(AP_ERR_ARG, "no queries");
    if (top_k == 0 || top_k > (uint32_t)kTopMax) return fail(AP_ERR_ARG, "top_k = %u: the exact scorer keeps up to %d results per query", top_k, kTopMax);
    AP_CUDA(cudaSetDevice(ix->device));
    cudaStream_t st = (cudaStream_t)stream_;
    const auto t_begin = std::chrono::high_resolution_clock::now();
    Inverted *inv = nullptr;
    AP_TRY(build_inverted(ix, &inv));
    const auto t_index = std::chrono::high_resolution_clock::now();
    const uint32_t n = ix->n, nq = q->nq;
    const uint32_t tiles_n = (n + kBN - 1) / kBN, ld = tiles_n * kBN;
    // batch of queries: up to 1024 rows, the scratch matrix S (rows x ld floats) kept below 4 GiB
    uint32_t qb = (uint32_t)std::min<uint64_t>(1024, ((4ull << 30) / ((uint64_t)ld * 4)) / kBM * kBM);
    qb = std::max<uint32_t>(kBM, std::min<uint32_t>(qb, (nq + kBM - 1) / kBM * kBM));
    const uint32_t m_tiles_max = qb / kBM;
    uint32_t splits = std::max<uint32_t>(1, std::min<uint32_t>((uint32_t)ix->num_sms / m_tiles_max, tiles_n));
    ExBuf db;
    float *S; __half *qh; unsigned long long *part;
    AP_TRY(db.alloc(&S, (size_t)qb * ld));
    AP_TRY(db.alloc(&qh, (size_t)qb * kDim));
    // the last batch may use more slices per block of queries: size the partial lists for the largest count
    const uint32_t splits_cap = std::max<uint32_t>(splits, std::min<uint32_t>((uint32_t)ix->num_sms, tiles_n));
    AP_TRY(db.alloc(&part, (size_t)splits_cap * nq * top_k));
    CUtensorMap map_q, map_x;
    AP_TRY(make_map(&map_q, qh, qb, kBM));
    AP_TRY(make_map(&map_x, inv->dense, n, kBN));
    const size_t smem = (size_t)kExStages * kExStageBytes + 32 * 128 * sizeof(float) + 1024;
    AP_CUDA(cudaFuncSetAttribute(exact_dense_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t ev[3];
    for (auto &e : ev) AP_CUDA(cudaEventCreate(&e));
    struct EvGuard { cudaEvent_t *e; ~EvGuard() { for (int i = 0; i < 3; ++i) cudaEventDestroy(e[i]); } } evg{ev};
    float sparse_ms = 0.f, dense_ms = 0.f;
    const bool keyword = (flags & AP_EXACT_KEYWORD) != 0;
    const bool any_sparse = sparse_weight != 0.0f || bm25_weight != 0.0f || keyword;
    // every batch uses the slice count of the first one, so that `part` is one [splits][nq][top_k] array for the merge
    for (uint32_t q0 = 0; q0 < nq; q0 += qb) {
        const uint32_t rows = std::min(qb, nq - q0), m_tiles = (rows + kBM - 1) / kBM;
        ex_query_kernel<<<(qb + 7) / 8, 256, 0, st>>>(qb, rows, q->dense + (size_t)q0 * kDim, dense_weight, reinterpret_cast<uint2 *>(qh));
        AP_CUDA(cudaEventRecord(ev[0], st));
        if (any_sparse) {
            SparseArgs sa{};
            sa.n = n; sa.ld = ld; sa.q0 = q0;
            sa.qs_off = q->sparse.off; sa.qs_idx = q->sparse.idx; sa.qs_val = q->sparse.val;
            sa.qb_off = q->bm25.off; sa.qb_idx = q->bm25.idx; sa.qb_val = q->bm25.val;
            sa.w_sparse = sparse_weight; sa.w_bm25 = bm25_weight;
            sa.vocab_s = inv->vocab_s; sa.vocab = inv->vocab; sa.toff = inv->toff; sa.post = inv->post; sa.S = S;
            sa.keyword = keyword ? 1u : 0u;
            const dim3 grid((ld + kWindow - 1) / kWindow, rows);
            exact_sparse_kernel<<<grid, kSpThreads, 0, st>>>(sa);
        } else {
            AP_CUDA(cudaMemsetAsync(S, 0, (size_t)rows * ld * 4, st));
        }
        AP_CUDA(cudaEventRecord(ev[1], st));
        DenseArgs da{};
        da.n = n; da.tiles_n = tiles_n; da.splits = splits; da.rows_valid = rows; da.q0 = q0; da.nq_total = nq; da.top_k = top_k;
        da.ld = ld; da.S = S; da.part = part; da.err = ix->d_ctl + 1;
        exact_dense_topk_kernel<<<m_tiles * splits, kExThreads, smem, st>>>(map_q, map_x, da);
        AP_CUDA(cudaGetLastError());
        AP_CUDA(cudaEventRecord(ev[2], st));
        AP_CUDA(cudaEventSynchronize(ev[2]));
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev[0], ev[1]); sparse_ms += ms;
        cudaEventElapsedTime(&ms, ev[1], ev[2]); dense_ms += ms;
    }
    AP_TRY(ap_merge_shard_keys(ix->device, splits, nq, top_k, part, top_k, out_ids, out_dis, st));
    AP_CUDA(cudaStreamSynchronize(st));
    uint32_t ew = 0;
    AP_CUDA(cudaMemcpy(&ew, ix->d_ctl + 1, 4, cudaMemcpyDeviceToHost));
    if (ew) { cudaMemset(ix->d_ctl + 1, 0, 4); return fail(AP_ERR_DEVICE, "the exact scorer raised error word %u (a bounded wait ran out)", ew); }
    if (stats) {
        const auto t_end = std::chrono::high_resolution_clock::now();
        stats->seconds_index = std::chrono::duration<double>(t_index - t_begin).count();
        stats->seconds_total = std::chrono::duration<double>(t_end - t_begin).count();
        stats->sparse_ms = sparse_ms; stats->dense_ms = dense_ms;
        stats->dense_flops = 2ull * (uint64_t)nq * n * kDim;
        stats->postings = inv->total;
        stats->batch_queries = qb; stats->slices = splits;
    }
    return AP_OK;
}

extern "C" int ap_exact_release(ap_index *ix) {
    if (!ix) return fail(AP_ERR_ARG, "null index");
    AP_CUDA(cudaSetDevice(ix->device));
    exact_release(ix);
    return AP_OK;
}
