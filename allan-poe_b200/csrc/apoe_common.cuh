// Shared declarations of the Allan-Poe B200 library: error plumbing, the resident index
// object, the packed device layout of a document, and small sm_100a device helpers
// (mbarrier, bulk async copy, explicitly rounded half arithmetic).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <functional>
#include <string>
#include <vector>

#include "../../include/allan_poe.h"

namespace apoe {

// ---------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define AP_CUDA(expr)                                                                                   \
    do {                                                                                                \
        cudaError_t _e = (expr);                                                                        \
        if (_e != cudaSuccess)                                                                          \
            return ::apoe::fail(AP_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                                __FILE__, __LINE__);                                                    \
    } while (0)

#define AP_TRY(expr)                 \
    do {                             \
        int _r = (expr);             \
        if (_r != AP_OK) return _r;  \
    } while (0)

// ---------------------------------------------------------------------------------------
// Device layout of one document ("record"), 16-byte aligned, in one pool per index:
//   [ dense: 1024 halves = 2048 B ][ sparse: pad2(nnz_s) x (u32 id, f32 val) ][ bm25: pad2(nnz_b) x (u32 id, f32 val) ]
// Padding pairs hold id 0xFFFFFFFF, value 0.  One 64-bit word per document locates it:
//   bits  0..35  record start in 16-byte units
//   bits 36..49  nnz_s      bits 50..63  nnz_b
// A single bulk copy therefore fetches everything one fused distance needs.
// ---------------------------------------------------------------------------------------
constexpr uint32_t kDim = AP_DIM;
constexpr uint32_t kDenseBytes = kDim * 2;
constexpr uint32_t kMaxRowNnz = 16383;  // 14-bit fields
constexpr uint32_t kEmpty = 0xFFFFFFFFu;
constexpr float kInfDis = 1000000.0f;  // ref: INF_DIS, src/query.cu:11

__host__ __device__ inline uint64_t meta_pack(uint64_t off16, uint32_t ns, uint32_t nb) {
    return off16 | ((uint64_t)ns << 36) | ((uint64_t)nb << 50);
}
__host__ __device__ inline uint64_t meta_off16(uint64_t m) { return m & ((1ull << 36) - 1); }
__host__ __device__ inline uint32_t meta_ns(uint64_t m) { return (uint32_t)(m >> 36) & 0x3FFF; }
__host__ __device__ inline uint32_t meta_nb(uint64_t m) { return (uint32_t)(m >> 50) & 0x3FFF; }
__host__ __device__ inline uint32_t pad2(uint32_t n) { return (n + 1u) & ~1u; }
__host__ __device__ inline uint32_t record_bytes(uint32_t ns, uint32_t nb) {
    return kDenseBytes + 8u * (pad2(ns) + pad2(nb));
}

// Graph edge as the search kernel reads it: neighbour id plus that neighbour's locator word, so that an
// expansion needs one dependent load (the row) before the record copies can be issued.
//   x = id, y = meta low 32, z = meta high 32, w = unused.  Slot 32 of a row carries the keyword-edge count in x.
struct __align__(16) FatEdge {
    uint32_t id, meta_lo, meta_hi, pad;
};

struct HostSample {  // first rows of the corpus, kept on the host for weight auto-normalisation
    uint32_t n = 0;
    std::vector<float> dense;
    std::vector<uint32_t> s_off, s_idx, b_off, b_idx;
    std::vector<float> s_val, b_val;
};

struct Workspace {  // grow-only device buffers of the host-pointer search path
    void *buf[16] = {nullptr};
    size_t cap[16] = {0};
};

}  // namespace apoe

struct ap_index {
    int device = 0;
    uint32_t n = 0;
    int num_sms = 0;
    size_t smem_per_sm = 0, smem_per_block = 0;

    uint8_t *rec = nullptr;        // search-time records (dense as given)
    uint8_t *rec_build = nullptr;  // build-time records (dense x dense_scale), same offsets
    float build_scale = 0.f;       // scale the build copy currently holds (0 = none)
    const float *dense_src = nullptr;  // caller's fp32 dense (device) kept only while rec_build may be re-made
    size_t rec_total = 0;          // bytes of one pool
    uint64_t *meta = nullptr;      // n locator words
    uint32_t max_rec_bytes = 0, max_ns = 0, max_nb = 0;
    uint32_t max_term = 0;         // largest sparse / BM25 term id, found by the first build or pruning call
    bool max_term_known = false;

    uint32_t *graph = nullptr;     // n x 40, index.poe rows
    apoe::FatEdge *fat = nullptr;  // n x 40
    uint32_t *ep = nullptr;        // 32 entry points
    apoe::FatEdge *ep_fat = nullptr;
    bool has_graph = false;

    uint32_t *knn_ids = nullptr;   // n x 64 (kept on request)
    float *knn_dis = nullptr;
    float *power = nullptr;        // n norms of the build-time copy

    uint32_t n_ent = 0;            // knowledge graph
    uint32_t *e2e_off = nullptr, *e2e_idx = nullptr, *e2d_off = nullptr, *e2d_idx = nullptr;

    uint32_t *d_ctl = nullptr;     // [0] next query, [1] error word
    unsigned long long *d_cnt = nullptr;  // [0] expansions [1] evaluations [2] bytes

    void *exact = nullptr;         // inverted index + contiguous dense copy of the exact scorer (made on first use)

    apoe::HostSample sample;
    apoe::Workspace ws;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
};

namespace apoe {

// ---- internal entry points shared between translation units ------------------------------------
int index_alloc(ap_index **out, int device, uint32_t n);
// Source of the corpus arrays for index_pack when they are not in memory yet.  read(dst, which, offset, bytes) writes
// bytes [offset, offset + bytes) of array `which` to dst (pinned or ordinary host memory) and may use threads of its
// own.  which: 0 dense rows in .fvecs layout (u32 1024, then 1024 floats per row; offset counted from the first row),
// 1 sparse ids, 2 sparse values, 3 BM25 ids, 4 BM25 values.
struct CorpusFeed {
    std::function<int(void *dst, int which, size_t offset, size_t bytes)> read;
};
int index_pack(ap_index *ix, const float *dense, const uint32_t *s_off, const uint32_t *s_idx, const float *s_val,
               const uint32_t *b_off, const uint32_t *b_idx, const float *b_val, bool on_device, uint32_t flags,
               const CorpusFeed *feed = nullptr);
int index_install_graph(ap_index *ix);  // graph + ep on device -> fat rows
int ws_reserve(ap_index *ix, int slot, size_t bytes, void **out);

struct SearchLaunch {
    const float *qdense;
    const uint32_t *qs_off, *qs_idx;
    const float *qs_val;
    const uint32_t *qb_off, *qb_idx;
    const float *qb_val;
    const uint32_t *qe_off, *qe_idx;
    uint32_t nq, max_qs, max_qb;
    float w_sparse, w_bm25, w_dense, kg_weight;
    uint32_t cands, flags, path;
    uint32_t arena_bytes, ctas_per_sm;
    uint32_t *out_ids;
    float *out_dis;
    cudaStream_t stream;
    unsigned long long *out_keys = nullptr;   // sharded search: nq x key_top_k packed (ordered distance, global id) words
    uint32_t key_top_k = 0, id_base = 0;
    uint32_t *ctl = nullptr;            // control words of the kernel (next query, error word); null = the index's own
    unsigned long long *cnt = nullptr;  // counters; null = the index's own
};
int search_launch(ap_index *ix, const SearchLaunch &L, uint32_t *launches);
int distances_launch(ap_index *ix, const SearchLaunch &L, size_t n_pairs, const uint32_t *pair_q,
                     const uint32_t *pair_d, float *out);

int build_run(ap_index *ix, const ap_build_opts *opts, ap_build_stats *stats);
int prune_run(ap_index *ix, const uint32_t *d_knn, const float *d_knn_dis, const float *d_power, uint32_t *d_new_list,
              uint32_t *d_kw, uint32_t *launches, uint32_t flags);
int norms_run(ap_index *ix, float *d_power);
int ensure_build_copy(ap_index *ix, float scale);
void exact_release(ap_index *ix);   // frees what the exact scorer keeps on the index

// ---------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls, raises the error word and returns false.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t *err_word, uint32_t code,
                                                  uint32_t limit = (1u << 24)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err_word, code);
    return false;
}
// Linear global -> shared bulk copy completing on an mbarrier.  Both addresses 16-byte aligned, bytes a
// positive multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Orders earlier ordinary (generic-proxy) accesses of shared memory before later bulk async copies into it.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// half2 arithmetic on packed bit patterns with the rounding spelled out, so the compiler can neither fuse nor split.
__device__ __forceinline__ uint32_t hfma2_rn(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_rn(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hadd2_rn(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ float half_sum_to_float(uint32_t packed) {  // float(hadd(x, y))
    __half lo = __ushort_as_half((unsigned short)(packed & 0xFFFFu));
    __half hi = __ushort_as_half((unsigned short)(packed >> 16));
    return __half2float(__hadd_rn(lo, hi));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    return (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
}
#endif

}  // namespace apoe
