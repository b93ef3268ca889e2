/*
 * allan_poe.h -- C ABI of the B200-native Allan-Poe hybrid graph index.
 *
 * Plain C: opaque handle, pointers and sizes only.  Every entry point returns
 * AP_OK or an AP_ERR_* code; ap_last_error() gives the message of the calling
 * thread's last failure.  Nothing here calls exit(): the reference ends the
 * process on a missing file or a CUDA error (include/utils.cuh:344,363,382,
 * src/index.cu:19-28, src/query.cu:23-32), this library reports it.
 *
 * "ref:" comments name the reference interface an entry point stands in for
 * (paths relative to the reference project's root).
 */
#ifndef ALLAN_POE_H
#define ALLAN_POE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AP_OK 0
#define AP_ERR_ARG 1    /* bad argument (null pointer, cands not a multiple of 32, ...) */
#define AP_ERR_IO 2     /* file missing, truncated or malformed */
#define AP_ERR_CUDA 3   /* CUDA runtime error */
#define AP_ERR_LIMIT 4  /* a row or a pool exceeds a kernel capacity */
#define AP_ERR_STATE 5  /* call out of order (search before a graph is set, ...) */
#define AP_ERR_DEVICE 6 /* a kernel gave up on a bounded wait and raised its error word */

#define AP_DIM 1024          /* dense dimension, ref: include/utils.cuh:31 */
#define AP_ROW 40            /* index.poe row width, ref: src/index.cu:888,903 */
#define AP_DEGREE 32         /* graph slots searched per row, ref: src/query.cu:6 */
#define AP_KNN 64            /* k-NN list width before pruning, ref: src/index.cu:6 */
#define AP_ENTRY_POINTS 32   /* ref: src/index.cu:923, src/query.cu:440-444 */
#define AP_MAX_CANDS 512     /* ref: src/query.cu:9 */
#define AP_STATIC_SCRATCH_BYTES (8u << 20) /* staging area of ap_search_host_static, held by every GPU that loads the library */

typedef struct ap_index ap_index;

/* CSR triple; rows + 1 offsets.  Term ids of a row strictly ascending. */
typedef struct {
    const uint32_t *off;
    const uint32_t *idx;
    const float *val;
} ap_csr;

/* flags of ap_index_create_* */
#define AP_CREATE_FOR_BUILD 1u /* also keep the build-time copy (dense x dense_scale) until the graph is built */

/* ---- build ---------------------------------------------------------- */
#define AP_BUILD_SIMT_JOIN 1u     /* local join on CUDA cores instead of tcgen05 (debug / cross-check) */
#define AP_BUILD_KEEP_KNN 2u      /* keep the pre-pruning k-NN lists readable through ap_index_get_knn */
#define AP_BUILD_RANDOM_START 4u  /* random initial lists only, as the reference (src/index.cu:99-106); default: the lists
                                     are first seeded from the posting lists of each document's rarest BM25 terms */
#define AP_BUILD_SHARED_PAIRS 8u  /* offer every evaluated pair to both of its ends (classic NN-Descent).  Default: each
                                     pair belongs to one end (hash of the two ids), so the forward half of a final row
                                     and its reverse-edge half (src/index.cu:699-711) carry different neighbours */
#define AP_BUILD_REVERSE_PASS 16u /* with AP_BUILD_SHARED_PAIRS: closing reverse merge as merge_reverse_plus
                                     (src/index.cu:386-478) */
#define AP_BUILD_PRUNE_STEPWISE 32u /* prune every node with the step-wise kernel (the form of src/index.cu:613-676) instead
                                     of the all-pairs kernel; same result, used to cross-check the two */
#define AP_BUILD_TRACE 64u        /* per-round and per-phase progress lines on stderr */
#define AP_BUILD_DETERMINISTIC 128u /* one seed, one graph: reverse samples and proposals are kept by an order-independent
                                     rule (smallest key per hashed slot) instead of first come, first served */
#define AP_BUILD_WIPE_TABLES 256u /* empty the shared-memory term tables of the joins and of the pruning between passes.
                                     Default: where the term ids leave high bits free the keys carry the pass number
                                     instead and nothing is emptied; same results either way (debug / cross-check) */

typedef struct {
    uint32_t iterations;   /* NN-Descent rounds; 0 = library default (6) */
    uint32_t seed;         /* random initial graph; the reference seeds from clock() (src/index.cu:102) */
    uint32_t flags;        /* AP_BUILD_* */
    float dense_scale;     /* build-time dense weight; 0 = 7.0 as in src/index.cu:836-840 */
    uint32_t proposals;    /* closest partners each participant of a local join keeps; 0 = 4, at most 8 */
    uint32_t seed_take;    /* followers taken from each posting list by the seeded start; 0 = 4, at most 32 */
    uint32_t reserved[2];
} ap_build_opts;

typedef struct {
    double seconds_total;      /* same span as the reference's "Indexing time" (src/index.cu:889-910) */
    double seconds_knn;        /* seeded start + NN-Descent part */
    double seconds_prune;      /* detour count + RNG-IP prune + row assembly */
    uint64_t distance_evals;   /* hybrid distances evaluated by the seeded start and the local joins */
    uint64_t list_updates;     /* k-NN list entries replaced */
    uint32_t iterations_run;
    uint32_t launches;         /* kernels launched */
    uint32_t proposal_overflows; /* proposals dropped because a document's inbox (192 per round) was full */
    uint32_t phase_10us[3];    /* summed over rounds, in 10 us: dense tiles of the first node batch, the remaining
                                  join work (sparse / BM25 parts, proposals), list merge */
    uint32_t reserved0;
    uint64_t rows_gathered;    /* participant records the local joins staged (each once for the dense tile, once for the
                                  sparse part); a join of r rows evaluates up to 32 x r distances from them */
} ap_build_stats;

/* ---- search --------------------------------------------------------- */
#define AP_SEARCH_KEYWORD 1u       /* bit 31 of query BM25 ids marks required terms (ref: src/query.cu:1828-1843,2005-2007) */
#define AP_SEARCH_KG 2u            /* entity-seeded search with logical-edge augmentation (ref: src/query.cu:2042-2046) */
#define AP_SEARCH_RAW_WEIGHTS 4u   /* use the weights as given, skip the auto-normalisation of src/query.cu:1847-1869 */
#define AP_SEARCH_UNFUSED_DENSE 8u /* dense products and sums rounded separately (HMUL2 + HADD2) instead of HFMA2 */

typedef struct {
    uint32_t cands;        /* pool size, multiple of 32, 32..512 */
    uint32_t flags;        /* AP_SEARCH_* */
    float sparse_weight;
    float bm25_weight;
    float dense_weight;
    float kg_weight;
    uint32_t arena_bytes;  /* per-CTA staging arena for gathered rows; 0 = default */
    uint32_t ctas_per_sm;  /* 0 = as many as fit */
    uint32_t reserved[4];
} ap_search_opts;

typedef struct {
    uint32_t nq;
    const float *dense; /* nq x 1024, unscaled */
    ap_csr sparse;
    ap_csr bm25;
    const uint32_t *ent_off; /* query -> entity CSR (KG search only, else NULL) */
    const uint32_t *ent_idx;
    uint32_t max_sparse_nnz; /* device-pointer calls: longest query row (0 = let the library read the offsets back) */
    uint32_t max_bm25_nnz;
} ap_queries;

typedef struct {
    float eff_sparse, eff_bm25, eff_dense; /* weights after auto-normalisation */
    uint32_t path;             /* AP_PATH_* bit set actually searched */
    double kernel_ms;          /* search kernel, CUDA events on the launch stream */
    double total_ms;           /* host wall time of the call */
    uint64_t expansions;       /* graph rows expanded, all queries */
    uint64_t evaluations;      /* fused distances computed, all queries */
    uint64_t gathered_bytes;   /* bytes of corpus rows + graph rows the kernel asked for */
    uint32_t launches;         /* kernels launched by the call */
    uint32_t h2d_bytes_lo, h2d_bytes_hi, d2h_bytes_lo, d2h_bytes_hi;
    uint32_t reserved[3];
} ap_search_stats;

#define AP_PATH_DENSE 1u
#define AP_PATH_SPARSE 2u
#define AP_PATH_BM25 4u

/* ---- errors ---------------------------------------------------------- */
const char *ap_last_error(void);
int ap_version(void);

/* ---- file-level drop-ins --------------------------------------------- */
/* ref: build_index_impl, include/hybrid_search.cuh:6-11, src/index.cu:810-941.
 * Reads the three corpus files, builds the graph on `device`, writes index.poe
 * (byte layout of src/index.cu:928-939) and prints "Indexing time: <s>s". */
int ap_build_index(const char *dense_data_path, const char *sparse_data_path, const char *bm25_data_path,
                   const char *output_graph_path, int device, const ap_build_opts *opts, ap_build_stats *stats);

/* ref: search_index_impl, include/hybrid_search.cuh:14-33, src/query.cu:1781-2080.
 * Empty string = feature off for keyword_id_path / knowledge_path.  Prints
 * "Query time: <s>s" and "nDCG@10: <v>".  max_queries = 0 searches every query
 * in the files (the reference hard-codes 100, src/query.cu:1825).  out_ids /
 * out_dis (nullable) receive nq x cands results; *out_nq the query count. */
int ap_search_index(const char *dense_data_path, const char *dense_query_path, const char *sparse_data_path,
                    const char *sparse_query_path, const char *bm25_data_path, const char *bm25_query_path,
                    const char *keyword_id_path, const char *knowledge_path, const char *entity2doc_path,
                    const char *query_entity_path, const char *graph_path, const char *ground_truth_path, int top_k,
                    int cands, float sparse_weight, float bm25_weight, float dense_weight, float kg_weight, int device,
                    uint32_t max_queries, uint32_t *out_ids, float *out_dis, uint32_t *out_nq, double *out_ndcg,
                    ap_search_stats *stats);

/* ---- input preparation ------------------------------------------------ */
/* BM25 weights from raw term frequencies, on the device.  No counterpart in the reference, which expects pre-weighted
 * rows with ascending term ids (README.md:73-77; its searches binary-search the rows, include/utils.cuh:299-340):
 *   idf(t) = ln(1 + (N - df(t) + 0.5) / (df(t) + 0.5)),  w = idf * tf * (k1 + 1) / (tf + k1 * (1 - b + b * len / avglen)),
 * len = sum of the row's tf; queries get w = idf * tf.  Rows come back sorted by term id; with AP_PREP_RELABEL_BY_DF the
 * vocabulary is first renumbered by descending document frequency (ties by old id) and `relabel[old] = new` is
 * returned, to be applied to the queries and to any other file that uses the same term ids. */
#define AP_PREP_RELABEL_BY_DF 1u
typedef struct {
    float k1, b;        /* Okapi parameters; pass NULL options for 1.2 / 0.75 */
    uint32_t flags;     /* AP_PREP_* */
    uint32_t reserved[5];
} ap_bm25_opts;
typedef struct {
    double seconds;       /* whole call, with the transfers of the host-pointer forms */
    float kernel_ms;      /* device time of the kernels (CUDA events) */
    float avg_len;
    uint64_t nnz;
    uint32_t rows_sorted; /* rows that were not ascending after the renumbering and went through the sort */
    uint32_t launches;
    uint32_t reserved[2];
} ap_prep_stats;
/* corpus, host pointers: idx is renumbered / reordered in place, weight[nnz], df[vocab], idf[vocab], relabel[vocab] out */
int ap_bm25_corpus_host(int device, uint32_t rows, uint32_t vocab, const uint32_t *off, uint32_t *idx, const float *tf,
                        float *weight, uint32_t *df, float *idf, uint32_t *relabel, const ap_bm25_opts *opts,
                        ap_prep_stats *stats);
/* queries, host pointers: idf (and relabel, may be NULL) as the corpus call returned them */
int ap_bm25_queries_host(int device, uint32_t rows, uint32_t vocab, const uint32_t *off, uint32_t *idx, const float *tf,
                         float *weight, const float *idf, const uint32_t *relabel, ap_prep_stats *stats);
/* the same with every array in device memory (off_host: host copy of the offsets); `stream` is a cudaStream_t */
int ap_bm25_corpus_device(int device, uint32_t rows, uint32_t vocab, const uint32_t *off_host, const uint32_t *off,
                          uint32_t *idx, const float *tf, float *weight, uint32_t *df, float *idf, uint32_t *relabel,
                          const ap_bm25_opts *opts, void *stream, ap_prep_stats *stats);
int ap_bm25_queries_device(int device, uint32_t rows, uint32_t vocab, const uint32_t *off_host, const uint32_t *off,
                           uint32_t *idx, const float *tf, float *weight, const float *idf, const uint32_t *relabel,
                           void *stream, ap_prep_stats *stats);

/* ---- resident index --------------------------------------------------- */
/* Corpus in host memory (ref: the uploads of src/query.cu:1901-1934). */
int ap_index_create_host(ap_index **out, int device, uint32_t n, const float *dense, ap_csr sparse, ap_csr bm25,
                         uint32_t flags);
/* Corpus straight from the reference's files (dense .fvecs, two CSR .bin): reader threads pread() byte ranges into
 * pinned staging buffers while the previous buffer is uploaded and packed.  Replaces load_data + load_sparse_data
 * (include/utils.cuh:361-398) followed by the uploads of src/index.cu:845-887 / src/query.cu:1901-1934.
 * threads = 0 picks min(16, hardware threads). */
typedef struct {
    double seconds_total;   /* open + headers + offsets + streaming + packing, until the records are resident */
    double seconds_open;    /* open, headers and row offsets */
    uint64_t bytes_read;
    uint32_t rows, threads;
    uint32_t nnz_sparse, nnz_bm25;
    uint32_t reserved[2];
} ap_ingest_stats;
int ap_index_create_files(ap_index **out, int device, const char *dense_path, const char *sparse_path,
                          const char *bm25_path, uint32_t flags, uint32_t threads, ap_ingest_stats *stats);
/* The same for documents [row_start, row_start + row_count) of the files only (a corpus shard; ids inside the index
 * are local: document row_start becomes id 0).  row_count = 0 reads everything. */
int ap_index_create_files_range(ap_index **out, int device, const char *dense_path, const char *sparse_path,
                                const char *bm25_path, uint32_t row_start, uint32_t row_count, uint32_t flags,
                                uint32_t threads, ap_ingest_stats *stats);
/* Corpus already in device memory of `device` (same layouts). */
int ap_index_create_device(ap_index **out, int device, uint32_t n, const float *dense, ap_csr sparse, ap_csr bm25,
                           uint32_t flags);
int ap_index_destroy(ap_index *ix);
uint32_t ap_index_size(const ap_index *ix);

/* Graph in, out, to and from index.poe (ref: src/index.cu:928-939, load_graph src/query.cu:35-62). */
int ap_index_set_graph(ap_index *ix, const uint32_t *rows /* n x 40, host */, const uint32_t *entry_points /* 32 */);
int ap_index_get_graph(const ap_index *ix, uint32_t *rows, uint32_t *entry_points);
int ap_index_load_graph(ap_index *ix, const char *path);
int ap_index_save_graph(const ap_index *ix, const char *path);

/* ref: the kernel sequence of src/index.cu:890-903 (NN-Descent, reverse merge, allan_poe, allan_poe_final_graph)
 * plus entry-point selection (src/index.cu:916-925).  Needs AP_CREATE_FOR_BUILD. */
int ap_index_build(ap_index *ix, const ap_build_opts *opts, ap_build_stats *stats);

/* Pre-pruning k-NN lists of the last build (AP_BUILD_KEEP_KNN): n x 64 ids, distances, n norms. */
int ap_index_get_knn(const ap_index *ix, uint32_t *ids, float *dis, float *power);

/* ref: cal_power, src/index.cu:483-534 (on the build-time copy).  out: n floats, host. */
int ap_index_norms(ap_index *ix, float *out);

/* ref: allan_poe + allan_poe_final_graph, src/index.cu:539-807, on caller-supplied k-NN lists (host, n x 64 ids
 * ascending by distance, n x 64 distances, n norms).  Writes the forward lists (n x 32), keyword-edge lists
 * (n x 33: count + 32 ids) and final rows (n x 40) to host memory; any output may be NULL.  Also installs the rows
 * and the entry points derived from `power` as the index's graph. */
int ap_index_prune(ap_index *ix, const uint32_t *knn_ids, const float *knn_dis, const float *power,
                   uint32_t flags /* AP_BUILD_PRUNE_STEPWISE | AP_BUILD_TRACE | AP_BUILD_WIPE_TABLES */, uint32_t *new_list,
                   uint32_t *keyword_edges, uint32_t *rows);

/* Knowledge graph for AP_SEARCH_KG (ref: load_kg_graph src/query.cu:89-108 and the uploads of :1963-1980).
 * Host pointers; entity->entity and entity->doc CSRs over n_entities rows. */
int ap_index_set_kg(ap_index *ix, uint32_t n_entities, const uint32_t *e2e_off, const uint32_t *e2e_idx,
                    const uint32_t *e2d_off, const uint32_t *e2d_idx);

/* ref: the weight auto-normalisation of src/query.cu:1847-1869.  Host query buffers.  In/out weights. */
int ap_effective_weights(const ap_index *ix, const ap_queries *q, float *sparse_weight, float *bm25_weight,
                         float *dense_weight);

/* ref: one search_index call's kernel phase, src/query.cu:1999-2054, with results returned.
 * Host query buffers in, host results out (nq x cands ids and fused distances, best first). */
int ap_search_host(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids, float *out_dis,
                   ap_search_stats *stats);
/* Same with every query and result pointer in device memory; `stream` is a cudaStream_t (NULL = default stream).
 * The weights are used as given (the auto-normalisation needs host copies of the first 100 queries: run
 * ap_effective_weights on those and pass its result).  With stats == NULL the call only enqueues the kernel and
 * returns: a device-side error (AP_ERR_DEVICE) of such a call is reported by the next call that passes stats, or by
 * ap_index_check_status. */
int ap_search_device(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids, float *out_dis,
                     void *stream, ap_search_stats *stats);

/* Waits for the work queued on the default stream and reports (and clears) the kernels' error word: AP_ERR_DEVICE when
 * a bounded wait of an earlier asynchronous call gave up or a record did not fit its staging area, else AP_OK. */
int ap_index_check_status(ap_index *ix);

/* No counterpart in the reference.  ap_search_host for callers that cannot allocate device memory while they serve:
 * a process whose GPU memory is entirely owned by another pool (cudaMalloc would fail), or a query loop that cannot
 * tolerate the device-wide synchronisation cudaMalloc / cudaFree may cause.  Same arguments, same results, but the
 * device staging of the batch (queries, control words, results) lives in a fixed array inside the library image
 * (AP_STATIC_SCRATCH_BYTES per GPU, held until the process exits) and the call performs no cudaMalloc, cudaFree or
 * other allocating call.  A batch whose staging does not fit returns AP_ERR_LIMIT and says how much it needs.
 * The first call on a device looks up the array's device address (once per device); make that first call before
 * any stream capture starts.  All calls on a device share the array, whatever index they use: it keeps the previous
 * call's contents (the call clears what must start at zero), and two calls that overlap on the GPU race. */
int ap_search_host_static(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids,
                          float *out_dis, ap_search_stats *stats);

/* Fused distances of explicit (query, doc) pairs with the search kernel's arithmetic (test hook).
 * Host buffers; weights are applied as given (no normalisation). */
int ap_fused_distances(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, size_t n_pairs,
                       const uint32_t *pair_query, const uint32_t *pair_doc, float *out);

/* ref: cal_precision, src/query.cu:111-145, with its float arithmetic (the printed figure has the reference's digits).
 * results: nq x stride ids (first top_k used); qrels: CSR of relevant ids.  A query without relevant ids adds nothing
 * (the reference divides 0 by 0 there). */
double ap_ndcg(uint32_t nq, const uint32_t *results, uint32_t stride, uint32_t top_k, const uint32_t *qrel_off,
               const uint32_t *qrel_ids);

/* ---- the reference's file formats, parsed into host memory (no device needed) ------------------------- */
/* Each call may be made with null arrays first to learn the sizes.
 * ref: load_data, include/utils.cuh:361-378 (.fvecs: per row an int32 dimension word and 1024 floats). */
int ap_file_read_fvecs(const char *path, uint32_t *rows, float *out /* rows x 1024 */, size_t cap_rows);
/* ref: load_sparse_data, include/utils.cuh:380-398 (u32 nnz | u32 off[rows+1] | u32 idx[nnz] | f32 val[nnz]).  The file
 * does not store its row count (the reference takes it from the dense file): pass it in *rows, or 0 to have it derived
 * from the file size. */
int ap_file_read_csr(const char *path, uint32_t *rows, uint32_t *nnz, uint32_t *off, uint32_t *idx, float *val);
/* ref: load_kg_graph, src/query.cu:89-108 (u32 n_off | u32 nnz | u32 off[n_off] | u32 idx[nnz]; n_off = entities + 1). */
int ap_file_read_kg(const char *path, uint32_t *n_off, uint32_t *nnz, uint32_t *off, uint32_t *idx);
/* ref: load_txt, src/query.cu:65-86 (text, line r = the ids of row r: required keywords or relevant documents).
 * off: rows + 1 entries; ids (capacity cap, may be NULL): the ids of all rows back to back; *total their number. */
int ap_file_read_id_lines(const char *path, uint32_t rows, uint32_t *off, uint32_t *ids, size_t cap, size_t *total);

/* ---- exact scoring (ground truth) ---------------------------------------------------------------------- */
/* Exact top-k of the fused score over every document of the index, on the device: the brute force that the score
 * definition of compute_hybrid_dis (src/query.cu:148-178) implies, over the documents as stored (dense halves, fp32
 * sparse values) and the queries as the search sees them (weights folded in, dense rounded to half), accumulated in
 * fp32.  Used as the ground truth of recall; the reference has no such call (it prints nDCG against a file).
 * Query pointers are device memory; the weights are used as given (pass the effective ones).  top_k <= 16.
 * out_ids / out_dis: nq x top_k, device, ascending (distance, id).  The first call on an index builds an inverted
 * index of its sparse and BM25 rows and a contiguous copy of its dense rows (kept until ap_exact_release or destroy). */
typedef struct {
    double seconds_total;   /* the call, including the one-time index below on the first call */
    double seconds_index;   /* inverted index + dense copy (0 when they were cached) */
    float sparse_ms;        /* sparse + BM25 accumulation kernels (CUDA events) */
    float dense_ms;         /* tensor-core contraction with the top-k epilogue */
    uint64_t dense_flops;   /* 2 x queries x documents x 1024 */
    uint64_t postings;
    uint32_t batch_queries, slices;
    uint32_t reserved[2];
} ap_exact_stats;
#define AP_EXACT_KEYWORD 1u /* keyword-constrained ground truth: only documents that hold at least one of the query's required
                               BM25 terms (bit 31 set, as for AP_SEARCH_KEYWORD) are eligible; queries with fewer than top_k
                               such documents get 0xFFFFFFFF / 1e6 in the remaining slots */
int ap_exact_topk_device(ap_index *ix, const ap_queries *q, float sparse_weight, float bm25_weight, float dense_weight,
                         uint32_t flags, uint32_t top_k, uint32_t *out_ids, float *out_dis, void *stream, ap_exact_stats *stats);
int ap_exact_release(ap_index *ix);

/* ---- corpus-sharded search ------------------------------------------------------------------------------ */
/* No counterpart in the reference (one GPU, one index).  Documents [start, start + count) of an n-document corpus belong to
 * shard `shard` of `shards`: contiguous ranges whose sizes differ by at most one. */
void ap_shard_range(uint32_t n, uint32_t shard, uint32_t shards, uint32_t *start, uint32_t *count);
/* ap_search_device on one shard, with the exchange format written by the search kernel itself: for every query the
 * best top_k pool entries as 64-bit keys (order-preserving bits of the fused distance << 32 | local id + id_base; an
 * empty slot is the all-ones word), out_keys: nq x top_k, device.  out_ids / out_dis (nq x cands) may be NULL.  The
 * effective weights must be the same on every shard (ap_effective_weights on global documents 0..99). */
int ap_search_shard_device(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t id_base, uint32_t top_k,
                           unsigned long long *out_keys, uint32_t *out_ids, float *out_dis, void *stream, ap_search_stats *stats);
/* The same with host buffers (queries in, keys out: nq x top_k), through the staging of ap_search_host. */
int ap_search_shard_host(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t id_base, uint32_t top_k,
                         unsigned long long *out_keys, uint32_t *out_ids, float *out_dis, ap_search_stats *stats);
/* Shards on disk: one index.poe per shard (local ids, the byte layout of src/index.cu:928-939) named
 * <graph_prefix>.<shard>.poe, and the text manifest <graph_prefix>.manifest (written by shard 0) that lists the
 * document range and the file of every shard.  ap_build_index_shard reads only its own rows of the corpus files. */
#define AP_SHARD_NAME_BYTES 256
int ap_build_index_shard(const char *dense_data_path, const char *sparse_data_path, const char *bm25_data_path,
                         const char *graph_prefix, uint32_t shard, uint32_t shards, int device, const ap_build_opts *opts,
                         ap_build_stats *stats);
int ap_shard_manifest_write(const char *manifest_path, uint32_t n_docs, uint32_t shards, const char *graph_prefix);
/* starts / counts: cap_shards entries, names: cap_shards x AP_SHARD_NAME_BYTES characters; all three may be NULL to
 * learn *n_docs and *shards first.  Rejects manifests whose ranges leave gaps or overlap. */
int ap_shard_manifest_read(const char *manifest_path, uint32_t *n_docs, uint32_t *shards, uint32_t *starts, uint32_t *counts,
                           char *names, uint32_t cap_shards);
/* One shard's part of a sharded search_index call: loads the shard's documents and its graph file (looked up in the
 * manifest), normalises the weights on global documents 0..99 (so every shard scores alike), searches every query
 * and returns the exchange keys (host, nq x top_k) that ap_merge_shard_keys turns into the global top-k. */
int ap_search_index_shard(const char *dense_data_path, const char *dense_query_path, const char *sparse_data_path,
                          const char *sparse_query_path, const char *bm25_data_path, const char *bm25_query_path,
                          const char *manifest_path, uint32_t shard, int top_k, int cands, float sparse_weight, float bm25_weight,
                          float dense_weight, int device, uint32_t max_queries, unsigned long long *out_keys, uint32_t *out_nq,
                          ap_search_stats *stats);
/* Global top-k of the gathered keys (keys: shards x nq x per_shard, device, e.g. the receive buffer of one
 * all-gather): ascending (distance, id); out: nq x top_k ids (0xFFFFFFFF when fewer results exist) and distances. */
int ap_merge_shard_keys(int device, uint32_t shards, uint32_t nq, uint32_t per_shard, const unsigned long long *keys,
                        uint32_t top_k, uint32_t *out_ids, float *out_dis, void *stream);

/* Merge per-shard result lists into a global top-k on the device (corpus-sharded search).
 * in_ids/in_dis: shards x nq x per_shard (ids already global), device; out: nq x top_k, device. */
int ap_merge_shard_results(int device, uint32_t shards, uint32_t nq, uint32_t per_shard, const uint32_t *in_ids,
                           const float *in_dis, uint32_t top_k, uint32_t *out_ids, float *out_dis, void *stream);

/* Test hook for the dense half of the NN-Descent local join: inner products of the dense rows of the given
 * participant lists (host: nodes x 64 ids; nodes x 2 counts = new rows, rows), computed by the tcgen05 kernel
 * (use_tc != 0) or by the CUDA-core kernel.  out: nodes x 64 x 32 floats, host.  Needs AP_CREATE_FOR_BUILD. */
int ap_debug_join_dense(ap_index *ix, uint32_t nodes, const uint32_t *plist, const uint32_t *pcnt, int use_tc, float *out);

/* Test hook for the error path of the bounded waits: runs a one-thread kernel that waits at most `polls` (<= 4096)
 * polls on a barrier nothing completes, so the wait gives up and raises the index's error word; the kernel returns
 * normally and the context stays usable.  ap_index_check_status then returns AP_ERR_DEVICE once. */
int ap_debug_wait_timeout(ap_index *ix, uint32_t polls);

/* Profiling hook: the bandwidth the memory system gives the search's access pattern when the data is only fetched --
 * whole records of pseudo-random documents brought into shared memory by bulk copies, with the search kernel's CTA
 * count and shared-memory budget, `batches` batches per CTA (0 = 2000).  The ceiling, in gathered bytes per second, of
 * a search over this index; random ~3.5 KB reads stay below the streaming-copy bandwidth. */
int ap_debug_gather_probe(ap_index *ix, uint32_t batches, double *gb_per_s, double *ms, unsigned long long *bytes);

/* Profiling hook: counters of the last search on this index -- expansions, evaluations, gathered bytes, then clock
 * cycles (thread 0 of every CTA, summed) spent in control, waiting for copies, scoring, sorting, merging. */
int ap_debug_counters(ap_index *ix, uint64_t *out8);

#ifdef __cplusplus
}
#endif
#endif /* ALLAN_POE_H */
