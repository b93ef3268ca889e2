// Input preparation next to the index path: BM25 weights from raw term frequencies, document frequencies and
// idf, optional renumbering of the vocabulary by descending document frequency, and rows sorted by term id.
// The reference has no code for this step: it expects pre-weighted rows with ascending ids (README.md:73-77) and its
// searches binary-search those rows (include/utils.cuh:299-340).  The arithmetic is the published Okapi BM25:
//   idf(t)  = ln(1 + (N - df(t) + 0.5) / (df(t) + 0.5))
//   w(t, d) = idf(t) * tf * (k1 + 1) / (tf + k1 * (1 - b + b * len(d) / avglen)),   len(d) = sum of the row's tf
// and for queries w(t, q) = idf(t) * tf.  Everything is float (fp32) on the device.
#include <cub/device/device_radix_sort.cuh>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <vector>

#include "apoe_common.cuh"

namespace apoe {

constexpr uint32_t kFullMask = 0xFFFFFFFFu;

// Document frequencies: one posting per (row, term).  A few head terms occur in most rows, and a global atomic per
// posting would serialise on their counters, so every block first counts in a direct-mapped shared-memory cache
// (4096 slots, first term to claim a slot keeps it) and adds each cached count to the global counter once.
constexpr uint32_t kDfSlots = 4096;
__global__ void __launch_bounds__(256) prep_df_kernel(size_t nnz, const uint32_t *__restrict__ idx, uint32_t vocab, uint32_t *__restrict__ df, uint32_t *__restrict__ bad) {
    __shared__ uint32_t tag[kDfSlots], cnt[kDfSlots];
    for (uint32_t i = threadIdx.x; i < kDfSlots; i += blockDim.x) { tag[i] = kEmpty; cnt[i] = 0; }
    __syncthreads();
    const size_t per = (nnz + gridDim.x - 1) / gridDim.x, lo = per * blockIdx.x, hi = lo + per < nnz ? lo + per : nnz;
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const uint32_t t = idx[i];
        if (t >= vocab) { atomicMin(bad, i < 0xFFFFFFFEull ? (uint32_t)i : 0xFFFFFFFEu); continue; }
        const uint32_t slot = (t * 2654435761u) >> 20;
        const uint32_t old = atomicCAS(&tag[slot], kEmpty, t);
        if (old == kEmpty || old == t) atomicAdd(&cnt[slot], 1u);
        else atomicAdd(&df[t], 1u);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < kDfSlots; i += blockDim.x)
        if (cnt[i]) atomicAdd(&df[tag[i]], cnt[i]);
}

// row lengths (sum of tf) and their total
__global__ void prep_len_kernel(uint32_t rows, const uint32_t *__restrict__ off, const float *__restrict__ tf, float *__restrict__ len, double *__restrict__ total) {
    __shared__ double part[8];
    const uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float s = 0.f;
    if (r < rows) {
        for (uint32_t j = off[r] + lane; j < off[r + 1]; j += 32) s += tf[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(kFullMask, s, o);
        if (lane == 0) len[r] = s;
    }
    if (lane == 0) part[warp] = r < rows ? (double)s : 0.0;
    __syncthreads();
    if (threadIdx.x == 0) {   // one atomic per block: a counter shared by every row would serialise
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += part[w];
        atomicAdd(total, t);
    }
}

__global__ void prep_idf_kernel(uint32_t vocab, float n_docs, const uint32_t *__restrict__ df, float *__restrict__ idf, unsigned long long *__restrict__ keys) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= vocab) return;
    const float d = (float)df[t];
    idf[t] = logf(1.0f + (n_docs - d + 0.5f) / (d + 0.5f));
    if (keys) keys[t] = ((unsigned long long)(0xFFFFFFFFu - df[t]) << 32) | t;   // descending df, ties by id
}
__global__ void prep_rank_kernel(uint32_t vocab, const unsigned long long *__restrict__ sorted, uint32_t *__restrict__ relabel) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < vocab) relabel[(uint32_t)sorted[i]] = i;
}

// One CTA per row: weight every posting, renumber its id, sort the row by the new id when it is not ascending.
struct PrepRowArgs {
    uint32_t rows;
    const uint32_t *off;
    uint32_t *idx;          // in / out
    const float *tf;        // in (null: keep `weight` as it is, only renumber and sort)
    float *weight;          // out (in as well when tf is null)
    const float *len;       // null for queries
    const float *idf;       // null: weights are not touched
    const uint32_t *relabel;
    float k1, b;
    const double *total;    // sum of all row lengths (device); average length = *total / rows
    uint32_t vocab;
    uint32_t *sorted_rows;  // counter of rows that needed the sort
    uint32_t *bad;          // first posting with a term id outside the vocabulary
    uint32_t *long_rows;    // rows of more than 128 postings, left to the CTA-per-row kernel
    uint32_t *n_long;
};

// weight and new id of one posting, packed as (new id << 32) | weight bits
__device__ __forceinline__ unsigned long long prep_key(const PrepRowArgs &a, uint32_t p, float norm) {
    uint32_t t = a.idx[p];
    float w = a.weight[p];
    if (t >= a.vocab) { atomicMin(a.bad, p); t = 0; }
    if (a.tf && a.idf) {
        const float f = a.tf[p];
        w = a.len ? a.idf[t] * f * (a.k1 + 1.0f) / (f + norm) : a.idf[t] * f;
    }
    return ((unsigned long long)(a.relabel ? a.relabel[t] : t) << 32) | __float_as_uint(w);
}
__device__ __forceinline__ float prep_norm(const PrepRowArgs &a, uint32_t r) {
    if (!a.len) return 0.0f;
    const float avglen = (float)(*a.total / (double)a.rows);
    return a.k1 * (1.0f - a.b + a.b * a.len[r] / avglen);
}

// Rows of up to 128 postings: one warp per row, two or four postings per lane, bitonic network through shuffles.
// H postings per lane (element e = lane + 32 h): exchanges at strides below 32 go through shuffles, the others stay
// inside the lane.
template <int H>
__device__ __forceinline__ void prep_row_warp_n(const PrepRowArgs &a, uint32_t r, uint32_t j0, uint32_t cnt, uint32_t lane, uint32_t &sorted_in_block) {
    const float norm = prep_norm(a, r);
    unsigned long long k[H];
#pragma unroll
    for (int h = 0; h < H; ++h) k[h] = lane + 32u * h < cnt ? prep_key(a, j0 + lane + 32u * h, norm) : ~0ull;
    // ascending already?  compare every element with its successor (the successor of lane 31 is lane 0 of the next h)
    bool inv = false;
#pragma unroll
    for (int h = 0; h < H; ++h) {
        const unsigned long long nxt = __shfl_down_sync(kFullMask, k[h], 1);
        const unsigned long long wrap = h + 1 < H ? __shfl_sync(kFullMask, k[h + 1 < H ? h + 1 : h], 0) : ~0ull;
        const unsigned long long s = lane == 31 ? wrap : nxt;
        inv = inv || (uint32_t)(k[h] >> 32) > (uint32_t)(s >> 32);
    }
    if (__any_sync(kFullMask, inv)) {
#pragma unroll
        for (uint32_t size = 2; size <= 32u * H; size <<= 1)
#pragma unroll
            for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
                if (stride >= 32) {   // partner sits in the same lane, at h ^ (stride / 32)
                    const int dh = (int)(stride >> 5);
#pragma unroll
                    for (int h = 0; h < H; ++h)
                        if ((h & dh) == 0) {
                            const bool asc = ((32u * h) & size) == 0;
                            const unsigned long long x = k[h], y = k[h | dh];
                            if ((x > y) == asc) { k[h] = y; k[h | dh] = x; }
                        }
                } else {
#pragma unroll
                    for (int h = 0; h < H; ++h) {
                        const uint32_t e = lane + 32u * h;
                        const unsigned long long o = __shfl_xor_sync(kFullMask, k[h], stride);
                        const bool asc = (e & size) == 0, low = (lane & stride) == 0;
                        const bool take_min = asc == low;
                        k[h] = take_min ? (o < k[h] ? o : k[h]) : (o > k[h] ? o : k[h]);
                    }
                }
            }
        if (lane == 0) atomicAdd(&sorted_in_block, 1u);
    }
#pragma unroll
    for (int h = 0; h < H; ++h)
        if (lane + 32u * h < cnt) { a.idx[j0 + lane + 32u * h] = (uint32_t)(k[h] >> 32); a.weight[j0 + lane + 32u * h] = __uint_as_float((uint32_t)k[h]); }
}

__device__ __forceinline__ void prep_row_warp(const PrepRowArgs &a, uint32_t &sorted_in_block) {
    const uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= a.rows) return;
    const uint32_t j0 = a.off[r], cnt = a.off[r + 1] - j0;
    if (cnt == 0) return;
    if (cnt <= 64) prep_row_warp_n<2>(a, r, j0, cnt, lane, sorted_in_block);
    else if (cnt <= 128) prep_row_warp_n<4>(a, r, j0, cnt, lane, sorted_in_block);
    else if (lane == 0) a.long_rows[atomicAdd(a.n_long, 1u)] = r;
}

__global__ void __launch_bounds__(256) prep_rows_warp_kernel(const PrepRowArgs a) {
    __shared__ uint32_t s_sorted;
    if (threadIdx.x == 0) s_sorted = 0;
    __syncthreads();
    prep_row_warp(a, s_sorted);
    __syncthreads();
    if (threadIdx.x == 0 && s_sorted) atomicAdd(a.sorted_rows, s_sorted);
}
// Longer rows: one CTA per row, bitonic network in shared memory.
__global__ void __launch_bounds__(128) prep_rows_kernel(const PrepRowArgs a) {
    extern __shared__ __align__(16) unsigned long long keys[];   // (new id << 32) | weight bits
    __shared__ uint32_t s_unsorted;
    const uint32_t tid = threadIdx.x, n_long = *a.n_long;
    for (uint32_t li = blockIdx.x; li < n_long; li += gridDim.x) {
        const uint32_t r = a.long_rows[li];
        const uint32_t j0 = a.off[r], cnt = a.off[r + 1] - j0;
        uint32_t p2 = 1;
        while (p2 < cnt) p2 <<= 1;
        if (tid == 0) s_unsorted = 0;
        __syncthreads();
        const float norm = prep_norm(a, r);
        for (uint32_t j = tid; j < p2; j += blockDim.x) keys[j] = j < cnt ? prep_key(a, j0 + j, norm) : ~0ull;
        __syncthreads();
        for (uint32_t j = tid + 1; j < cnt; j += blockDim.x)
            if ((uint32_t)(keys[j - 1] >> 32) > (uint32_t)(keys[j] >> 32)) s_unsorted = 1;
        __syncthreads();
        if (s_unsorted) {
            for (uint32_t size = 2; size <= p2; size <<= 1)
                for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
                    for (uint32_t t = tid; t < p2 / 2; t += blockDim.x) {
                        const uint32_t lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
                        const bool asc = (lo & size) == 0;
                        const unsigned long long x = keys[lo], y = keys[hi];
                        if ((x > y) == asc) { keys[lo] = y; keys[hi] = x; }
                    }
                    __syncthreads();
                }
            if (tid == 0) atomicAdd(a.sorted_rows, 1u);
        }
        for (uint32_t j = tid; j < cnt; j += blockDim.x) {
            a.idx[j0 + j] = (uint32_t)(keys[j] >> 32);
            a.weight[j0 + j] = __uint_as_float((uint32_t)keys[j]);
        }
        __syncthreads();
    }
}

struct PrepBuf {
    std::vector<void *> ptrs;
    ~PrepBuf() { for (void *p : ptrs) cudaFree(p); }
    template <class T> int alloc(T **out, size_t count) {
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, std::max<size_t>(count * sizeof(T), 16));
        if (e != cudaSuccess) return fail(AP_ERR_CUDA, "cudaMalloc of %zu bytes failed: %s", count * sizeof(T), cudaGetErrorString(e));
        ptrs.push_back(p); *out = (T *)p; return AP_OK;
    }
};

static int rows_launch(const PrepRowArgs &a, uint32_t max_row, cudaStream_t st, uint32_t *launches) {
    prep_rows_warp_kernel<<<(a.rows + 7) / 8, 256, 0, st>>>(a);
    AP_CUDA(cudaGetLastError());
    ++*launches;
    if (max_row > 128) {
        uint32_t p2 = 1;
        while (p2 < max_row) p2 <<= 1;
        const size_t smem = (size_t)p2 * 8;
        prep_rows_kernel<<<std::min<uint32_t>(a.rows, 148u * 8u), 128, smem, st>>>(a);
        AP_CUDA(cudaGetLastError());
        ++*launches;
    }
    return AP_OK;
}

// all pointers in device memory; off_host is the host copy of the offsets (for the row maximum)
static int bm25_device(bool corpus, uint32_t rows, uint32_t vocab, const uint32_t *off, uint32_t max_row, size_t nnz, uint32_t *idx,
                       const float *tf, float *weight, uint32_t *df, float *idf, uint32_t *relabel, const ap_bm25_opts *opts,
                       cudaStream_t st, ap_prep_stats *stats) {
    const float k1 = opts ? opts->k1 : 1.2f, b = opts ? opts->b : 0.75f;
    const bool want_relabel = opts && (opts->flags & AP_PREP_RELABEL_BY_DF);
    PrepBuf pb;
    uint32_t *scratch;   // [0] first bad posting, [1] rows sorted, [2] long rows
    uint32_t *long_rows;
    double *total;
    float *len = nullptr;
    AP_TRY(pb.alloc(&scratch, 4)); AP_TRY(pb.alloc(&total, 1)); AP_TRY(pb.alloc(&long_rows, rows));
    // every allocation before the timed region: cudaMalloc stalls the host while the stream runs dry
    unsigned long long *keys = nullptr, *keys_s = nullptr;
    uint8_t *sort_tmp = nullptr;
    size_t sort_bytes = 0;
    if (corpus) {
        AP_TRY(pb.alloc(&len, rows));
        if (want_relabel) {
            AP_TRY(pb.alloc(&keys, vocab)); AP_TRY(pb.alloc(&keys_s, vocab));
            AP_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, sort_bytes, keys, keys_s, (int)vocab, 0, 64, st));
            AP_TRY(pb.alloc(&sort_tmp, sort_bytes));
        }
    }
    if (max_row > 128) {
        uint32_t p2 = 1;
        while (p2 < max_row) p2 <<= 1;
        if ((size_t)p2 * 8 > 200 * 1024) return fail(AP_ERR_LIMIT, "a row of %u entries does not fit the sorting buffer", max_row);
        AP_CUDA(cudaFuncSetAttribute(prep_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)p2 * 8)));
    }
    AP_CUDA(cudaMemsetAsync(scratch, 0xFF, 4, st));
    AP_CUDA(cudaMemsetAsync(scratch + 1, 0, 8, st));
    AP_CUDA(cudaMemsetAsync(total, 0, 8, st));
    struct Events {   // released on every return path
        cudaEvent_t a = nullptr, b = nullptr;
        ~Events() { if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b); }
    } ev;
    AP_CUDA(cudaEventCreate(&ev.a)); AP_CUDA(cudaEventCreate(&ev.b));
    cudaEvent_t e0 = ev.a, e1 = ev.b;
    AP_CUDA(cudaEventRecord(e0, st));
    uint32_t launches = 0;
    if (corpus) {
        AP_CUDA(cudaMemsetAsync(df, 0, (size_t)vocab * 4, st));
        if (nnz) { prep_df_kernel<<<(uint32_t)std::min<size_t>((nnz + 4095) / 4096, 148 * 6), 256, 0, st>>>(nnz, idx, vocab, df, scratch); ++launches; }
        prep_len_kernel<<<(rows + 7) / 8, 256, 0, st>>>(rows, off, tf, len, total); ++launches;
        prep_idf_kernel<<<(vocab + 255) / 256, 256, 0, st>>>(vocab, (float)rows, df, idf, keys); ++launches;
        if (want_relabel) {
            AP_CUDA(cub::DeviceRadixSort::SortKeys(sort_tmp, sort_bytes, keys, keys_s, (int)vocab, 0, 64, st));
            prep_rank_kernel<<<(vocab + 255) / 256, 256, 0, st>>>(vocab, keys_s, relabel); ++launches;
        }
    }
    PrepRowArgs a{};
    a.rows = rows; a.off = off; a.idx = idx; a.tf = tf; a.weight = weight; a.len = corpus ? len : nullptr; a.idf = idf;
    a.relabel = (corpus ? want_relabel : relabel != nullptr) ? relabel : nullptr;
    a.k1 = k1; a.b = b; a.total = total; a.sorted_rows = scratch + 1; a.vocab = vocab; a.bad = scratch;
    a.long_rows = long_rows; a.n_long = scratch + 2;
    if (rows && max_row) AP_TRY(rows_launch(a, max_row, st, &launches));
    AP_CUDA(cudaEventRecord(e1, st));
    uint32_t back[3] = {0, 0, 0};
    double tot = 0.0;
    AP_CUDA(cudaMemcpyAsync(back, scratch, 12, cudaMemcpyDeviceToHost, st));
    AP_CUDA(cudaMemcpyAsync(&tot, total, 8, cudaMemcpyDeviceToHost, st));
    AP_CUDA(cudaStreamSynchronize(st));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (back[0] != 0xFFFFFFFFu) return fail(AP_ERR_ARG, "posting %u holds a term id outside the vocabulary of %u terms", back[0], vocab);
    const float avglen = corpus && rows ? (float)(tot / rows) : 0.f;
    if (corpus && !(avglen > 0.f)) return fail(AP_ERR_ARG, "the corpus has no term frequencies (average length %g)", avglen);
    const uint32_t sorted = back[1];
    if (stats) { stats->kernel_ms = ms; stats->avg_len = avglen; stats->rows_sorted = sorted; stats->nnz = nnz; stats->launches = launches; }
    return AP_OK;
}

static int offsets_info(const uint32_t *off_host, uint32_t rows, uint32_t *max_row, size_t *nnz) {
    uint32_t mx = 0;
    if (off_host[0] != 0) return fail(AP_ERR_ARG, "first offset is %u, expected 0", off_host[0]);
    for (uint32_t i = 0; i < rows; ++i) {
        if (off_host[i + 1] < off_host[i]) return fail(AP_ERR_ARG, "offsets decrease at row %u", i);
        mx = std::max(mx, off_host[i + 1] - off_host[i]);
    }
    *max_row = mx; *nnz = off_host[rows];
    return AP_OK;
}

}  // namespace apoe

using namespace apoe;

extern "C" {

int ap_bm25_corpus_device(int device, uint32_t rows, uint32_t vocab, const uint32_t *off_host, const uint32_t *off, uint32_t *idx,
                          const float *tf, float *weight, uint32_t *df, float *idf, uint32_t *relabel, const ap_bm25_opts *opts,
                          void *stream, ap_prep_stats *stats) {
    if (!off_host || !off || !idx || !tf || !weight || !df || !idf) return fail(AP_ERR_ARG, "null argument");
    if (opts && (opts->flags & AP_PREP_RELABEL_BY_DF) && !relabel) return fail(AP_ERR_ARG, "AP_PREP_RELABEL_BY_DF needs the relabel table");
    if (rows == 0 || vocab == 0) return fail(AP_ERR_ARG, "empty corpus or vocabulary");
    AP_CUDA(cudaSetDevice(device));
    uint32_t max_row; size_t nnz;
    AP_TRY(offsets_info(off_host, rows, &max_row, &nnz));
    const auto t0 = std::chrono::high_resolution_clock::now();
    if (stats) memset(stats, 0, sizeof *stats);
    AP_TRY(bm25_device(true, rows, vocab, off, max_row, nnz, idx, tf, weight, df, idf, relabel, opts, (cudaStream_t)stream, stats));
    if (stats) stats->seconds = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
    return AP_OK;
}

int ap_bm25_queries_device(int device, uint32_t rows, uint32_t vocab, const uint32_t *off_host, const uint32_t *off, uint32_t *idx,
                           const float *tf, float *weight, const float *idf, const uint32_t *relabel, void *stream, ap_prep_stats *stats) {
    if (!off_host || !off || !idx || !tf || !weight || !idf) return fail(AP_ERR_ARG, "null argument");
    if (rows == 0 || vocab == 0) return fail(AP_ERR_ARG, "empty query set or vocabulary");
    AP_CUDA(cudaSetDevice(device));
    uint32_t max_row; size_t nnz;
    AP_TRY(offsets_info(off_host, rows, &max_row, &nnz));
    const auto t0 = std::chrono::high_resolution_clock::now();
    if (stats) memset(stats, 0, sizeof *stats);
    AP_TRY(bm25_device(false, rows, vocab, off, max_row, nnz, idx, tf, weight, nullptr, const_cast<float *>(idf), const_cast<uint32_t *>(relabel),
                       nullptr, (cudaStream_t)stream, stats));
    if (stats) stats->seconds = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
    return AP_OK;
}

// Host-pointer forms: upload, run, download.
static int bm25_host(bool corpus, int device, uint32_t rows, uint32_t vocab, const uint32_t *off, uint32_t *idx, const float *tf, float *weight,
                     uint32_t *df, float *idf, uint32_t *relabel, const ap_bm25_opts *opts, ap_prep_stats *stats) {
    if (!off || !idx || !tf || !weight || !idf || (corpus && !df)) return fail(AP_ERR_ARG, "null argument");
    AP_CUDA(cudaSetDevice(device));
    const auto t0 = std::chrono::high_resolution_clock::now();
    const size_t nnz = off[rows];
    const bool rl = corpus ? (opts && (opts->flags & AP_PREP_RELABEL_BY_DF)) : relabel != nullptr;
    if (corpus && rl && !relabel) return fail(AP_ERR_ARG, "AP_PREP_RELABEL_BY_DF needs the relabel table");
    PrepBuf pb;
    uint32_t *d_off, *d_idx, *d_df = nullptr, *d_rl = nullptr; float *d_tf, *d_w, *d_idf;
    AP_TRY(pb.alloc(&d_off, (size_t)rows + 1)); AP_TRY(pb.alloc(&d_idx, nnz)); AP_TRY(pb.alloc(&d_tf, nnz)); AP_TRY(pb.alloc(&d_w, nnz));
    AP_TRY(pb.alloc(&d_idf, vocab));
    if (corpus) AP_TRY(pb.alloc(&d_df, vocab));
    if (rl) AP_TRY(pb.alloc(&d_rl, vocab));
    AP_CUDA(cudaMemcpy(d_off, off, ((size_t)rows + 1) * 4, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMemcpy(d_idx, idx, nnz * 4, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMemcpy(d_tf, tf, nnz * 4, cudaMemcpyHostToDevice));
    if (!corpus) {
        AP_CUDA(cudaMemcpy(d_idf, idf, (size_t)vocab * 4, cudaMemcpyHostToDevice));
        if (rl) AP_CUDA(cudaMemcpy(d_rl, relabel, (size_t)vocab * 4, cudaMemcpyHostToDevice));
    }
    int rc = corpus ? ap_bm25_corpus_device(device, rows, vocab, off, d_off, d_idx, d_tf, d_w, d_df, d_idf, d_rl, opts, nullptr, stats)
                    : ap_bm25_queries_device(device, rows, vocab, off, d_off, d_idx, d_tf, d_w, d_idf, d_rl, nullptr, stats);
    if (rc != AP_OK) return rc;
    AP_CUDA(cudaMemcpy(idx, d_idx, nnz * 4, cudaMemcpyDeviceToHost));
    AP_CUDA(cudaMemcpy(weight, d_w, nnz * 4, cudaMemcpyDeviceToHost));
    if (corpus) {
        AP_CUDA(cudaMemcpy(df, d_df, (size_t)vocab * 4, cudaMemcpyDeviceToHost));
        AP_CUDA(cudaMemcpy(idf, d_idf, (size_t)vocab * 4, cudaMemcpyDeviceToHost));
        if (rl) AP_CUDA(cudaMemcpy(relabel, d_rl, (size_t)vocab * 4, cudaMemcpyDeviceToHost));
    }
    if (stats) stats->seconds = std::chrono::duration<double>(std::chrono::high_resolution_clock::now() - t0).count();
    return AP_OK;
}

int ap_bm25_corpus_host(int device, uint32_t rows, uint32_t vocab, const uint32_t *off, uint32_t *idx, const float *tf, float *weight,
                        uint32_t *df, float *idf, uint32_t *relabel, const ap_bm25_opts *opts, ap_prep_stats *stats) {
    if (rows == 0 || vocab == 0) return fail(AP_ERR_ARG, "empty corpus or vocabulary");
    return bm25_host(true, device, rows, vocab, off, idx, tf, weight, df, idf, relabel, opts, stats);
}

int ap_bm25_queries_host(int device, uint32_t rows, uint32_t vocab, const uint32_t *off, uint32_t *idx, const float *tf, float *weight,
                         const float *idf, const uint32_t *relabel, ap_prep_stats *stats) {
    if (rows == 0 || vocab == 0) return fail(AP_ERR_ARG, "empty query set or vocabulary");
    return bm25_host(false, device, rows, vocab, off, idx, tf, weight, nullptr, const_cast<float *>(idf), const_cast<uint32_t *>(relabel), nullptr, stats);
}

}  // extern "C"
