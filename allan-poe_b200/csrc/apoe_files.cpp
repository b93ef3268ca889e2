// File-level drop-ins: the loaders and writers of the reference's on-disk formats and the two calls behind
// hybrid_search.build_index / hybrid_search.search_index, implemented over the resident-index C ABI.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "apoe_common.cuh"

using apoe::fail;

namespace {

struct CsrHost {
    std::vector<uint32_t> off, idx;
    std::vector<float> val;
    ap_csr view() const { return ap_csr{off.data(), idx.data(), val.data()}; }
};

bool file_size(const char *path, size_t *out) {
    std::ifstream in(path, std::ios::binary | std::ios::ate);
    if (!in.is_open()) return false;
    *out = (size_t)in.tellg();
    return true;
}

// ref: load_data, include/utils.cuh:361-378 -- int32 dim, then per row (int32 dim, dim floats)
int load_fvecs(const char *path, std::vector<float> &data, uint32_t *num) {
    size_t fsize;
    if (!file_size(path, &fsize)) return fail(AP_ERR_IO, "cannot open %s", path);
    std::ifstream in(path, std::ios::binary);
    uint32_t dim = 0;
    in.read((char *)&dim, 4);
    if (!in || dim != AP_DIM) return fail(AP_ERR_IO, "%s: dimension %u, this index is built for %d", path, dim, AP_DIM);
    const size_t n = fsize / ((size_t)(dim + 1) * 4);
    if (n == 0 || n > 0x7FFFFFFFull) return fail(AP_ERR_IO, "%s: %zu rows", path, n);
    data.resize(n * dim);
    in.seekg(0, std::ios::beg);
    std::vector<float> rowbuf((size_t)(dim + 1) * 1024);
    for (size_t r0 = 0; r0 < n; r0 += 1024) {
        const size_t rows = std::min<size_t>(1024, n - r0);
        in.read((char *)rowbuf.data(), rows * (dim + 1) * 4);
        if (!in) return fail(AP_ERR_IO, "%s: truncated at row %zu", path, r0);
        for (size_t r = 0; r < rows; ++r) memcpy(&data[(r0 + r) * dim], &rowbuf[r * (dim + 1) + 1], (size_t)dim * 4);
    }
    *num = (uint32_t)n;
    return AP_OK;
}

// ref: load_sparse_data, include/utils.cuh:380-398 -- u32 nnz | u32 off[rows+1] | u32 idx[nnz] | f32 val[nnz]
int load_csr(const char *path, uint32_t rows, CsrHost &c) {
    size_t fsize;
    if (!file_size(path, &fsize)) return fail(AP_ERR_IO, "cannot open %s", path);
    std::ifstream in(path, std::ios::binary);
    uint32_t nnz = 0;
    in.read((char *)&nnz, 4);
    const size_t need = 4 + (size_t)(rows + 1) * 4 + (size_t)nnz * 8;
    if (!in || fsize < need) return fail(AP_ERR_IO, "%s: %zu bytes, %zu needed for %u rows and %u entries", path, fsize, need, rows, nnz);
    c.off.resize(rows + 1); c.idx.resize(nnz); c.val.resize(nnz);
    in.read((char *)c.off.data(), (size_t)(rows + 1) * 4);
    in.read((char *)c.idx.data(), (size_t)nnz * 4);
    in.read((char *)c.val.data(), (size_t)nnz * 4);
    if (!in) return fail(AP_ERR_IO, "%s: truncated", path);
    if (c.off[rows] != nnz) return fail(AP_ERR_IO, "%s: last offset %u differs from the entry count %u", path, c.off[rows], nnz);
    std::cout << "Non zero num: " << nnz << std::endl;
    return AP_OK;
}

// ref: load_kg_graph, src/query.cu:89-108 -- u32 n_off | u32 nnz | u32 off[n_off] | u32 idx[nnz]
int load_kg(const char *path, std::vector<uint32_t> &off, std::vector<uint32_t> &idx) {
    size_t fsize;
    if (!file_size(path, &fsize)) return fail(AP_ERR_IO, "cannot open %s", path);
    std::ifstream in(path, std::ios::binary);
    uint32_t n_off = 0, nnz = 0;
    in.read((char *)&n_off, 4); in.read((char *)&nnz, 4);
    if (!in || n_off == 0 || fsize < 8 + (size_t)n_off * 4 + (size_t)nnz * 4) return fail(AP_ERR_IO, "%s: malformed CSR header", path);
    off.resize(n_off); idx.resize(nnz);
    in.read((char *)off.data(), (size_t)n_off * 4);
    in.read((char *)idx.data(), (size_t)nnz * 4);
    if (!in) return fail(AP_ERR_IO, "%s: truncated", path);
    std::cout << "Entity num: " << n_off << ", Non zero num: " << nnz << std::endl;
    return AP_OK;
}

// ref: load_txt, src/query.cu:65-86 -- one line of unsigned ids per query
int load_id_lines(const char *path, uint32_t rows, std::vector<std::vector<uint32_t>> &out) {
    std::ifstream in(path);
    if (!in.is_open()) return fail(AP_ERR_IO, "cannot open %s", path);
    out.assign(rows, {});
    std::string line;
    uint32_t r = 0;
    while (r < rows && std::getline(in, line)) {
        std::istringstream iss(line);
        uint32_t v;
        while (iss >> v) out[r].push_back(v);
        ++r;
    }
    return AP_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Streamed ingest.  The reference reads the corpus with one thread, one small read per row, into pageable
// memory (include/utils.cuh:361-398) and uploads afterwards (src/index.cu:845-887).  Here the three files stay
// open, byte ranges are fetched by several threads with pread() straight into pinned staging buffers, and the
// upload and packing of one buffer run while the next one is being filled.
// ---------------------------------------------------------------------------------------------------------
struct CorpusFiles {
    int fd[3] = {-1, -1, -1};          // dense, sparse, bm25
    std::string path[3];
    size_t size[3] = {0, 0, 0};
    uint32_t n = 0, nnz[3] = {0, 0, 0};    // rows and entries of the window that is read
    uint32_t n_file = 0, row0 = 0;         // rows in the files, first row of the window
    uint32_t nnz_file[3] = {0, 0, 0}, first[3] = {0, 0, 0};   // entries in the files, first entry of the window
    std::vector<uint32_t> off[3];      // [1], [2]: row offsets of the two CSR files, rebased to the window
    uint32_t threads = 8;
    std::atomic<unsigned long long> bytes_read{0};
    ~CorpusFiles() { for (int f : fd) if (f >= 0) close(f); }

    // bytes [offset, offset + bytes) of file f into dst, split over the reader threads
    int read_range(int f, void *dst, size_t offset, size_t bytes) {
        if (offset + bytes > size[f]) return fail(AP_ERR_IO, "%s: read of %zu bytes at %zu runs past the end (%zu bytes)", path[f].c_str(), bytes, offset, size[f]);
        const size_t min_slice = (size_t)4 << 20;
        const uint32_t parts = (uint32_t)std::max<size_t>(1, std::min<size_t>(threads, (bytes + min_slice - 1) / min_slice));
        std::atomic<int> err{0};
        auto work = [&](uint32_t p) {
            size_t a = bytes * p / parts, b = bytes * (p + 1) / parts;
            while (a < b) {
                const ssize_t got = pread(fd[f], (char *)dst + a, b - a, (off_t)(offset + a));
                if (got <= 0) { err = 1; return; }
                a += (size_t)got;
            }
        };
        if (parts == 1) work(0);
        else {
            std::vector<std::thread> pool;
            for (uint32_t p = 1; p < parts; ++p) pool.emplace_back(work, p);
            work(0);
            for (auto &t : pool) t.join();
        }
        if (err) return fail(AP_ERR_IO, "%s: read failed or file truncated", path[f].c_str());
        bytes_read += bytes;
        return AP_OK;
    }

    // row_count = 0: the whole corpus; else the window [row_start, row_start + row_count)
    int open_all(const char *dense_path, const char *sparse_path, const char *bm25_path, uint32_t row_start = 0, uint32_t row_count = 0) {
        const char *p[3] = {dense_path, sparse_path, bm25_path};
        for (int f = 0; f < 3; ++f) {
            path[f] = p[f];
            fd[f] = open(p[f], O_RDONLY);
            struct stat sb;
            if (fd[f] < 0 || fstat(fd[f], &sb) != 0) return fail(AP_ERR_IO, "cannot open %s", p[f]);
            size[f] = (size_t)sb.st_size;
        }
        // ref: load_data, include/utils.cuh:361-378 -- every row is (int32 dim, dim floats); the row count is the file size
        uint32_t dim = 0;
        if (size[0] < 4 || pread(fd[0], &dim, 4, 0) != 4 || dim != AP_DIM) return fail(AP_ERR_IO, "%s: dimension %u, this index is built for %d", p[0], dim, AP_DIM);
        const size_t rows = size[0] / ((size_t)(AP_DIM + 1) * 4);
        if (rows == 0 || rows > 0x7FFFFFFFull) return fail(AP_ERR_IO, "%s: %zu rows", p[0], rows);
        n_file = (uint32_t)rows;
        if (row_count == 0) { row_start = 0; row_count = n_file; }
        if ((uint64_t)row_start + row_count > n_file) return fail(AP_ERR_ARG, "rows [%u, %u) requested, %s holds %u", row_start, row_start + row_count, p[0], n_file);
        row0 = row_start; n = row_count;
        // ref: load_sparse_data, include/utils.cuh:380-398 -- u32 nnz | u32 off[rows+1] | u32 idx[nnz] | f32 val[nnz]
        for (int f = 1; f < 3; ++f) {
            if (size[f] < 4 || pread(fd[f], &nnz_file[f], 4, 0) != 4) return fail(AP_ERR_IO, "%s: no header", p[f]);
            const size_t need = 4 + (size_t)(n_file + 1) * 4 + (size_t)nnz_file[f] * 8;
            if (size[f] < need) return fail(AP_ERR_IO, "%s: %zu bytes, %zu needed for %u rows and %u entries", p[f], size[f], need, n_file, nnz_file[f]);
            off[f].resize((size_t)n + 1);
            int rc = read_range(f, off[f].data(), 4 + (size_t)row0 * 4, (size_t)(n + 1) * 4);
            if (rc != AP_OK) return rc;
            uint32_t last = 0;
            if (pread(fd[f], &last, 4, (off_t)(4 + (size_t)n_file * 4)) != 4 || last != nnz_file[f])
                return fail(AP_ERR_IO, "%s: last offset %u differs from the entry count %u", p[f], last, nnz_file[f]);
            first[f] = off[f][0];
            if (off[f][n] < first[f] || off[f][n] > nnz_file[f]) return fail(AP_ERR_IO, "%s: offsets of rows [%u, %u] are out of range", p[f], row0, row0 + n);
            for (auto &o : off[f]) o -= first[f];
            nnz[f] = off[f][n];
        }
        return AP_OK;
    }

    // the reader index_pack asks for its arrays (see apoe::CorpusFeed)
    int feed_read(void *dst, int which, size_t offset, size_t bytes) {
        if (which == 0) return read_range(0, dst, (size_t)row0 * (AP_DIM + 1) * 4 + offset, bytes);
        const int f = which <= 2 ? 1 : 2;
        const size_t base = 4 + (size_t)(n_file + 1) * 4 + ((which == 2 || which == 4) ? (size_t)nnz_file[f] * 4 : 0) + (size_t)first[f] * 4;
        return read_range(f, dst, base + offset, bytes);
    }
};

}  // namespace

extern "C" {

void ap_shard_range(uint32_t n, uint32_t shard, uint32_t shards, uint32_t *start, uint32_t *count) {
    if (shards == 0 || shard >= shards) { if (start) *start = 0; if (count) *count = 0; return; }
    const uint32_t base = n / shards, rem = n % shards;
    if (start) *start = shard * base + std::min(shard, rem);
    if (count) *count = base + (shard < rem ? 1u : 0u);
}

int ap_index_create_files(ap_index **out, int device, const char *dense_path, const char *sparse_path, const char *bm25_path,
                          uint32_t flags, uint32_t threads, ap_ingest_stats *stats) {
    return ap_index_create_files_range(out, device, dense_path, sparse_path, bm25_path, 0, 0, flags, threads, stats);
}

int ap_index_create_files_range(ap_index **out, int device, const char *dense_path, const char *sparse_path, const char *bm25_path,
                                uint32_t row_start, uint32_t row_count, uint32_t flags, uint32_t threads, ap_ingest_stats *stats) {
    if (!out || !dense_path || !sparse_path || !bm25_path) return fail(AP_ERR_ARG, "null argument");
    const auto t0 = std::chrono::high_resolution_clock::now();
    CorpusFiles cf;
    cf.threads = threads ? std::min(threads, 64u) : std::min(16u, std::max(1u, std::thread::hardware_concurrency()));
    int rc = cf.open_all(dense_path, sparse_path, bm25_path, row_start, row_count);
    if (rc != AP_OK) return rc;
    const auto t1 = std::chrono::high_resolution_clock::now();
    rc = apoe::index_alloc(out, device, cf.n);
    if (rc == AP_OK) {
        apoe::CorpusFeed feed{[&cf](void *dst, int which, size_t offset, size_t bytes) { return cf.feed_read(dst, which, offset, bytes); }};
        rc = apoe::index_pack(*out, nullptr, cf.off[1].data(), nullptr, nullptr, cf.off[2].data(), nullptr, nullptr, false, flags, &feed);
    }
    if (rc != AP_OK) { if (*out) ap_index_destroy(*out); *out = nullptr; return rc; }
    const auto t2 = std::chrono::high_resolution_clock::now();
    if (stats) {
        memset(stats, 0, sizeof *stats);
        stats->seconds_open = std::chrono::duration<double>(t1 - t0).count();
        stats->seconds_total = std::chrono::duration<double>(t2 - t0).count();
        stats->bytes_read = cf.bytes_read.load();
        stats->rows = cf.n; stats->threads = cf.threads;
        stats->nnz_sparse = cf.nnz[1]; stats->nnz_bm25 = cf.nnz[2];
    }
    return AP_OK;
}


// ref: cal_precision, src/query.cu:111-145.  Accumulates in float exactly as the reference does (per-position gains
// 1 / log2(float(j + 2)), DCG / IDCG per query, the sum divided by the query count in float), so the printed figure
// has the reference's digits.  One deliberate difference: a query without relevant ids adds nothing, where the
// reference divides 0 by 0 and prints nan for the whole run.
double ap_ndcg(uint32_t nq, const uint32_t *results, uint32_t stride, uint32_t top_k, const uint32_t *qrel_off,
               const uint32_t *qrel_ids) {
    float total = 0.f;
    for (uint32_t q = 0; q < nq; ++q) {
        const uint32_t *rel = qrel_ids + qrel_off[q];
        const uint32_t nrel = qrel_off[q + 1] - qrel_off[q];
        float idcg = 0.f;
        for (uint32_t j = 0; j < nrel; ++j) idcg += (1 / std::log2((float)(j + 2)));
        float dcg = 0.f;
        std::vector<uint32_t> a(results + (size_t)q * stride, results + (size_t)q * stride + top_k), b(rel, rel + nrel), common;
        std::sort(a.begin(), a.end()); std::sort(b.begin(), b.end());
        std::set_intersection(a.begin(), a.end(), b.begin(), b.end(), std::back_inserter(common));
        for (uint32_t x : common)
            for (uint32_t it = 0; it < top_k; ++it)
                if (results[(size_t)q * stride + it] == x) { dcg += (1 / std::log2((float)(it + 2))); break; }
        if (nrel) total += (dcg / idcg);
    }
    return nq ? (double)(total / (float)nq) : 0.0;
}

// ---------------------------------------------------------------------------------------------------------
// The loaders above behind the C ABI (host memory only, no device needed).  Every call can be made twice: first
// with null arrays to learn the sizes, then with buffers of at least that size.
// ---------------------------------------------------------------------------------------------------------
int ap_file_read_fvecs(const char *path, uint32_t *rows, float *out, size_t cap_rows) {
    if (!path || !rows) return fail(AP_ERR_ARG, "null argument");
    size_t fsize;
    if (!file_size(path, &fsize)) return fail(AP_ERR_IO, "cannot open %s", path);
    if (!out) {   // size query: the row count follows from the file size (include/utils.cuh:368-370)
        std::ifstream in(path, std::ios::binary);
        uint32_t dim = 0;
        in.read((char *)&dim, 4);
        if (!in || dim != AP_DIM) return fail(AP_ERR_IO, "%s: dimension %u, this index is built for %d", path, dim, AP_DIM);
        *rows = (uint32_t)(fsize / ((size_t)(dim + 1) * 4));
        return AP_OK;
    }
    std::vector<float> data;
    uint32_t n = 0;
    int rc = load_fvecs(path, data, &n);
    if (rc != AP_OK) return rc;
    *rows = n;
    if (n > cap_rows) return fail(AP_ERR_LIMIT, "%s holds %u rows, the buffer %zu", path, n, cap_rows);
    memcpy(out, data.data(), data.size() * 4);
    return AP_OK;
}

int ap_file_read_csr(const char *path, uint32_t *rows, uint32_t *nnz, uint32_t *off, uint32_t *idx, float *val) {
    if (!path || !rows || !nnz) return fail(AP_ERR_ARG, "null argument");
    size_t fsize;
    if (!file_size(path, &fsize)) return fail(AP_ERR_IO, "cannot open %s", path);
    std::ifstream in(path, std::ios::binary);
    uint32_t nz = 0;
    in.read((char *)&nz, 4);
    if (!in) return fail(AP_ERR_IO, "%s: no header", path);
    if (*rows == 0) {   // the file does not store its row count: u32 nnz | u32 off[rows + 1] | u32 idx[nnz] | f32 val[nnz]
        const size_t fixed = 4 + (size_t)nz * 8;
        if (fsize < fixed + 8 || (fsize - fixed) % 4 != 0) return fail(AP_ERR_IO, "%s: %zu bytes do not hold %u entries plus offsets", path, fsize, nz);
        *rows = (uint32_t)((fsize - fixed) / 4 - 1);
    }
    *nnz = nz;
    if (!off && !idx && !val) return AP_OK;
    if (!off || !idx || !val) return fail(AP_ERR_ARG, "pass all three arrays or none");
    CsrHost c;
    in.close();
    int rc = load_csr(path, *rows, c);
    if (rc != AP_OK) return rc;
    memcpy(off, c.off.data(), c.off.size() * 4);
    memcpy(idx, c.idx.data(), c.idx.size() * 4);
    memcpy(val, c.val.data(), c.val.size() * 4);
    return AP_OK;
}

int ap_file_read_kg(const char *path, uint32_t *n_off, uint32_t *nnz, uint32_t *off, uint32_t *idx) {
    if (!path || !n_off || !nnz) return fail(AP_ERR_ARG, "null argument");
    std::vector<uint32_t> o, i;
    int rc = load_kg(path, o, i);
    if (rc != AP_OK) return rc;
    *n_off = (uint32_t)o.size(); *nnz = (uint32_t)i.size();
    if (off) memcpy(off, o.data(), o.size() * 4);
    if (idx) memcpy(idx, i.data(), i.size() * 4);
    return AP_OK;
}

int ap_file_read_id_lines(const char *path, uint32_t rows, uint32_t *off, uint32_t *ids, size_t cap, size_t *total) {
    if (!path || !off || !total) return fail(AP_ERR_ARG, "null argument");
    std::vector<std::vector<uint32_t>> lines;
    int rc = load_id_lines(path, rows, lines);
    if (rc != AP_OK) return rc;
    size_t n = 0;
    for (uint32_t r = 0; r < rows; ++r) { off[r] = (uint32_t)n; n += lines[r].size(); }
    off[rows] = (uint32_t)n;
    *total = n;
    if (!ids) return AP_OK;
    if (n > cap) return fail(AP_ERR_LIMIT, "%s holds %zu ids, the buffer %zu", path, n, cap);
    size_t o = 0;
    for (uint32_t r = 0; r < rows; ++r) for (uint32_t x : lines[r]) ids[o++] = x;
    return AP_OK;
}

int ap_index_load_graph(ap_index *ix, const char *path) {
    if (!ix || !path) return fail(AP_ERR_ARG, "null argument");
    size_t fsize;
    if (!file_size(path, &fsize)) return fail(AP_ERR_IO, "cannot open %s", path);
    std::ifstream in(path, std::ios::binary);
    uint32_t k = 0, n_ep = 0;
    in.read((char *)&k, 4); in.read((char *)&n_ep, 4);
    if (!in || k != AP_ROW || n_ep != AP_ENTRY_POINTS) return fail(AP_ERR_IO, "%s: row width %u / %u entry points, expected %d / %d", path, k, n_ep, AP_ROW, AP_ENTRY_POINTS);
    const size_t num = (fsize - ((size_t)n_ep + 1) * 4) / ((size_t)k + 1) / 4;  // ref: src/query.cu:46
    std::cout << "Degree: " << k << "," << "num: " << num << std::endl;
    if (num != ap_index_size(ix)) return fail(AP_ERR_IO, "%s holds %zu rows, the corpus has %u documents", path, num, ap_index_size(ix));
    std::vector<uint32_t> ep(n_ep), rows(num * k), buf((size_t)(k + 1) * 4096);
    in.read((char *)ep.data(), (size_t)n_ep * 4);
    for (size_t r0 = 0; r0 < num; r0 += 4096) {
        const size_t cnt = std::min<size_t>(4096, num - r0);
        in.read((char *)buf.data(), cnt * (k + 1) * 4);
        if (!in) return fail(AP_ERR_IO, "%s: truncated at row %zu", path, r0);
        for (size_t r = 0; r < cnt; ++r) memcpy(&rows[(r0 + r) * k], &buf[r * (k + 1) + 1], (size_t)k * 4);
    }
    return ap_index_set_graph(ix, rows.data(), ep.data());
}

// ref: the writer of src/index.cu:928-939 -- u32 40 | u32 32 | u32 ep[32] | n x (u32 40 | u32 row[40])
int ap_index_save_graph(const ap_index *ix, const char *path) {
    if (!ix || !path) return fail(AP_ERR_ARG, "null argument");
    const uint32_t n = ap_index_size(ix);
    std::vector<uint32_t> rows((size_t)n * AP_ROW), ep(AP_ENTRY_POINTS);
    int rc = ap_index_get_graph(ix, rows.data(), ep.data());
    if (rc != AP_OK) return rc;
    std::ofstream out(path, std::ios::binary | std::ios::out);
    if (!out.is_open()) return fail(AP_ERR_IO, "cannot create %s", path);
    const uint32_t w = AP_ROW, ne = AP_ENTRY_POINTS;
    out.write((const char *)&w, 4); out.write((const char *)&ne, 4);
    out.write((const char *)ep.data(), (size_t)ne * 4);
    std::vector<uint32_t> buf((size_t)(w + 1) * 4096);
    for (size_t r0 = 0; r0 < n; r0 += 4096) {
        const size_t cnt = std::min<size_t>(4096, n - r0);
        for (size_t r = 0; r < cnt; ++r) { buf[r * (w + 1)] = w; memcpy(&buf[r * (w + 1) + 1], &rows[(r0 + r) * w], (size_t)w * 4); }
        out.write((const char *)buf.data(), cnt * (w + 1) * 4);
    }
    out.close();
    if (!out) return fail(AP_ERR_IO, "write to %s failed", path);
    return AP_OK;
}

int ap_build_index(const char *dense_data_path, const char *sparse_data_path, const char *bm25_data_path,
                   const char *output_graph_path, int device, const ap_build_opts *opts, ap_build_stats *stats) {
    if (!dense_data_path || !sparse_data_path || !bm25_data_path || !output_graph_path) return fail(AP_ERR_ARG, "null path");
    std::cout << "Loading dense data from " << dense_data_path << std::endl;
    ap_index *ix = nullptr;
    ap_ingest_stats ing{};
    int rc = ap_index_create_files(&ix, device, dense_data_path, sparse_data_path, bm25_data_path, AP_CREATE_FOR_BUILD, 0, &ing);
    if (rc != AP_OK) return rc;
    std::cout << "Non zero num: " << ing.nnz_sparse << std::endl << "Non zero num: " << ing.nnz_bm25 << std::endl;
    std::cout << "Points: " << ix->n << ", Dim: " << AP_DIM << std::endl;
    std::cout << "Max sparse dim: " << ix->max_ns << ", Max bm25 dim: " << ix->max_nb << std::endl;
    ap_build_stats st{};
    rc = ap_index_build(ix, opts, &st);
    if (rc == AP_OK) {
        std::cout << "Indexing time: " << (float)st.seconds_total << "s" << std::endl;
        rc = ap_index_save_graph(ix, output_graph_path);
    }
    if (stats) *stats = st;
    ap_index_destroy(ix);
    return rc;
}


// ---------------------------------------------------------------------------------------------------------
// Corpus shards on disk.  A sharded index is one index.poe per shard (rows hold shard-local ids, the byte layout
// of src/index.cu:928-939 unchanged) plus a small text manifest that says which documents each file covers:
//     allan-poe-shards 1
//     docs <n> shards <G>
//     <g> <first document> <documents> <file name, relative to the manifest's folder>     (G lines)
// ---------------------------------------------------------------------------------------------------------
static std::string dir_of(const std::string &path) {
    const size_t k = path.find_last_of('/');
    return k == std::string::npos ? std::string() : path.substr(0, k + 1);
}
static std::string base_of(const std::string &path) {
    const size_t k = path.find_last_of('/');
    return k == std::string::npos ? path : path.substr(k + 1);
}
static int dense_rows_of(const char *dense_path, uint32_t *n) {
    size_t fsize;
    if (!file_size(dense_path, &fsize)) return fail(AP_ERR_IO, "cannot open %s", dense_path);
    const size_t rows = fsize / ((size_t)(AP_DIM + 1) * 4);
    if (rows == 0 || rows > 0x7FFFFFFFull) return fail(AP_ERR_IO, "%s: %zu rows", dense_path, rows);
    *n = (uint32_t)rows;
    return AP_OK;
}

int ap_shard_manifest_write(const char *manifest_path, uint32_t n_docs, uint32_t shards, const char *graph_prefix) {
    if (!manifest_path || !graph_prefix || shards == 0 || n_docs < shards) return fail(AP_ERR_ARG, "bad manifest arguments");
    std::ofstream out(manifest_path);
    if (!out.is_open()) return fail(AP_ERR_IO, "cannot create %s", manifest_path);
    out << "allan-poe-shards 1\n" << "docs " << n_docs << " shards " << shards << "\n";
    const std::string stem = base_of(graph_prefix);
    for (uint32_t g = 0; g < shards; ++g) {
        uint32_t a, c;
        ap_shard_range(n_docs, g, shards, &a, &c);
        out << g << " " << a << " " << c << " " << stem << "." << g << ".poe\n";
    }
    out.close();
    if (!out) return fail(AP_ERR_IO, "write to %s failed", manifest_path);
    return AP_OK;
}

int ap_shard_manifest_read(const char *manifest_path, uint32_t *n_docs, uint32_t *shards, uint32_t *starts, uint32_t *counts,
                           char *names, uint32_t cap_shards) {
    if (!manifest_path || !n_docs || !shards) return fail(AP_ERR_ARG, "null argument");
    std::ifstream in(manifest_path);
    if (!in.is_open()) return fail(AP_ERR_IO, "cannot open %s", manifest_path);
    std::string magic, w1, w2;
    uint32_t version = 0, n = 0, G = 0;
    in >> magic >> version >> w1 >> n >> w2 >> G;
    if (!in || magic != "allan-poe-shards" || version != 1 || w1 != "docs" || w2 != "shards" || G == 0 || n < G)
        return fail(AP_ERR_IO, "%s is not a shard manifest", manifest_path);
    *n_docs = n; *shards = G;
    if (!starts && !counts && !names) return AP_OK;
    if (G > cap_shards) return fail(AP_ERR_LIMIT, "%s lists %u shards, the buffers hold %u", manifest_path, G, cap_shards);
    uint32_t next = 0;
    for (uint32_t g = 0; g < G; ++g) {
        uint32_t id = 0, a = 0, c = 0; std::string name;
        in >> id >> a >> c >> name;
        if (!in || id != g || a != next || c == 0 || name.empty() || name.size() >= AP_SHARD_NAME_BYTES)
            return fail(AP_ERR_IO, "%s: shard line %u is malformed or leaves a gap (first document %u, expected %u)", manifest_path, g, a, next);
        next = a + c;
        if (starts) starts[g] = a;
        if (counts) counts[g] = c;
        if (names) { memset(names + (size_t)g * AP_SHARD_NAME_BYTES, 0, AP_SHARD_NAME_BYTES); memcpy(names + (size_t)g * AP_SHARD_NAME_BYTES, name.data(), name.size()); }
    }
    if (next != n) return fail(AP_ERR_IO, "%s: the shards cover %u of %u documents", manifest_path, next, n);
    return AP_OK;
}

int ap_build_index_shard(const char *dense_data_path, const char *sparse_data_path, const char *bm25_data_path,
                         const char *graph_prefix, uint32_t shard, uint32_t shards, int device, const ap_build_opts *opts,
                         ap_build_stats *stats) {
    if (!dense_data_path || !sparse_data_path || !bm25_data_path || !graph_prefix) return fail(AP_ERR_ARG, "null path");
    if (shards == 0 || shard >= shards) return fail(AP_ERR_ARG, "shard %u of %u", shard, shards);
    uint32_t n = 0, a = 0, c = 0;
    int rc = dense_rows_of(dense_data_path, &n);
    if (rc != AP_OK) return rc;
    if (n < shards * 2) return fail(AP_ERR_ARG, "%u documents cannot be split into %u shards", n, shards);
    ap_shard_range(n, shard, shards, &a, &c);
    ap_index *ix = nullptr;
    rc = ap_index_create_files_range(&ix, device, dense_data_path, sparse_data_path, bm25_data_path, a, c, AP_CREATE_FOR_BUILD, 0, nullptr);
    if (rc != AP_OK) return rc;
    std::cout << "Shard " << shard << "/" << shards << ": documents [" << a << ", " << a + c << ")" << std::endl;
    ap_build_stats st{};
    rc = ap_index_build(ix, opts, &st);
    if (rc == AP_OK) {
        std::cout << "Indexing time: " << (float)st.seconds_total << "s" << std::endl;
        const std::string file = std::string(graph_prefix) + "." + std::to_string(shard) + ".poe";
        rc = ap_index_save_graph(ix, file.c_str());
    }
    if (rc == AP_OK && shard == 0) rc = ap_shard_manifest_write((std::string(graph_prefix) + ".manifest").c_str(), n, shards, graph_prefix);
    if (stats) *stats = st;
    ap_index_destroy(ix);
    return rc;
}

int ap_search_index_shard(const char *dense_data_path, const char *dense_query_path, const char *sparse_data_path,
                          const char *sparse_query_path, const char *bm25_data_path, const char *bm25_query_path,
                          const char *manifest_path, uint32_t shard, int top_k, int cands, float sparse_weight, float bm25_weight,
                          float dense_weight, int device, uint32_t max_queries, unsigned long long *out_keys, uint32_t *out_nq,
                          ap_search_stats *stats) {
    if (!dense_data_path || !dense_query_path || !sparse_data_path || !sparse_query_path || !bm25_data_path || !bm25_query_path || !manifest_path)
        return fail(AP_ERR_ARG, "null path");
    if (top_k <= 0 || top_k > cands) return fail(AP_ERR_ARG, "top_k = %d must lie in [1, cands = %d]", top_k, cands);
    uint32_t n = 0, G = 0, n_file = 0;
    int rc = ap_shard_manifest_read(manifest_path, &n, &G, nullptr, nullptr, nullptr, 0);
    if (rc != AP_OK) return rc;
    if (shard >= G) return fail(AP_ERR_ARG, "shard %u of %u", shard, G);
    std::vector<uint32_t> starts(G), counts(G);
    std::vector<char> names((size_t)G * AP_SHARD_NAME_BYTES);
    rc = ap_shard_manifest_read(manifest_path, &n, &G, starts.data(), counts.data(), names.data(), G);
    if (rc == AP_OK) rc = dense_rows_of(dense_data_path, &n_file);
    if (rc != AP_OK) return rc;
    if (n_file != n) return fail(AP_ERR_IO, "%s describes %u documents, %s holds %u", manifest_path, n, dense_data_path, n_file);
    std::vector<float> qdense;
    uint32_t nq_file = 0;
    CsrHost qsp, qbm;
    rc = load_fvecs(dense_query_path, qdense, &nq_file);
    if (rc == AP_OK) rc = load_csr(sparse_query_path, nq_file, qsp);
    if (rc == AP_OK) rc = load_csr(bm25_query_path, nq_file, qbm);
    if (rc != AP_OK) return rc;
    uint32_t nq = nq_file;
    if (max_queries && max_queries < nq) nq = max_queries;
    ap_queries q{};
    q.nq = nq; q.dense = qdense.data(); q.sparse = qsp.view(); q.bm25 = qbm.view();
    // the weights every shard must share: normalised on global documents 0..99 (ref: src/query.cu:1847-1869)
    float ws = sparse_weight, wb = bm25_weight, wd = dense_weight;
    {
        ap_index *head = nullptr;
        rc = ap_index_create_files_range(&head, device, dense_data_path, sparse_data_path, bm25_data_path, 0, std::min(n, 100u), 0, 1, nullptr);
        if (rc == AP_OK) rc = ap_effective_weights(head, &q, &ws, &wb, &wd);
        if (head) ap_index_destroy(head);
        if (rc != AP_OK) return rc;
    }
    ap_index *ix = nullptr;
    rc = ap_index_create_files_range(&ix, device, dense_data_path, sparse_data_path, bm25_data_path, starts[shard], counts[shard], 0, 0, nullptr);
    if (rc != AP_OK) return rc;
    struct Guard { ap_index *&p; ~Guard() { if (p) { ap_index_destroy(p); p = nullptr; } } } guard{ix};
    const std::string graph = dir_of(manifest_path) + std::string(names.data() + (size_t)shard * AP_SHARD_NAME_BYTES);
    rc = ap_index_load_graph(ix, graph.c_str());
    if (rc != AP_OK) return rc;
    ap_search_opts o{};
    o.cands = (uint32_t)cands; o.flags = AP_SEARCH_RAW_WEIGHTS;
    o.sparse_weight = ws; o.bm25_weight = wb; o.dense_weight = wd;
    ap_search_stats st{};
    rc = ap_search_shard_host(ix, &q, &o, starts[shard], (uint32_t)top_k, out_keys, nullptr, nullptr, &st);
    if (rc != AP_OK) return rc;
    if (out_nq) *out_nq = nq;
    if (stats) *stats = st;
    return AP_OK;
}

int ap_search_index(const char *dense_data_path, const char *dense_query_path, const char *sparse_data_path,
                    const char *sparse_query_path, const char *bm25_data_path, const char *bm25_query_path,
                    const char *keyword_id_path, const char *knowledge_path, const char *entity2doc_path,
                    const char *query_entity_path, const char *graph_path, const char *ground_truth_path, int top_k,
                    int cands, float sparse_weight, float bm25_weight, float dense_weight, float kg_weight, int device,
                    uint32_t max_queries, uint32_t *out_ids, float *out_dis, uint32_t *out_nq, double *out_ndcg,
                    ap_search_stats *stats) {
    if (!dense_data_path || !dense_query_path || !sparse_data_path || !sparse_query_path || !bm25_data_path ||
        !bm25_query_path || !graph_path)
        return fail(AP_ERR_ARG, "null path");
    if (top_k <= 0 || top_k > cands) return fail(AP_ERR_ARG, "top_k = %d must lie in [1, cands = %d]", top_k, cands);
    std::vector<float> qdense;
    uint32_t n = 0, nq_file = 0;
    CsrHost qsp, qbm;
    ap_index *ix = nullptr;
    int rc = ap_index_create_files(&ix, device, dense_data_path, sparse_data_path, bm25_data_path, 0, 0, nullptr);
    if (rc != AP_OK) return rc;
    struct Guard { ap_index *&p; ~Guard() { if (p) { ap_index_destroy(p); p = nullptr; } } } guard{ix};
    n = ix->n;
    rc = load_fvecs(dense_query_path, qdense, &nq_file);
    if (rc == AP_OK) rc = load_csr(sparse_query_path, nq_file, qsp);
    if (rc == AP_OK) rc = load_csr(bm25_query_path, nq_file, qbm);
    if (rc != AP_OK) return rc;
    const bool use_kg = knowledge_path && knowledge_path[0];
    const bool use_kw = keyword_id_path && keyword_id_path[0];
    std::vector<uint32_t> e2e_off, e2e_idx, e2d_off, e2d_idx, qe_off, qe_idx;
    if (use_kg) {
        if (!entity2doc_path || !query_entity_path) return fail(AP_ERR_ARG, "knowledge_path set without entity2doc_path / query_entity_path");
        rc = load_kg(knowledge_path, e2e_off, e2e_idx);
        if (rc == AP_OK) rc = load_kg(entity2doc_path, e2d_off, e2d_idx);
        if (rc == AP_OK) rc = load_kg(query_entity_path, qe_off, qe_idx);
        if (rc != AP_OK) return rc;
        if (e2e_off.size() != e2d_off.size()) return fail(AP_ERR_IO, "entity graph has %zu offsets, entity->doc map %zu", e2e_off.size(), e2d_off.size());
    }
    uint32_t nq = nq_file;
    if (max_queries && max_queries < nq) nq = max_queries;
    if (use_kg && qe_off.size() < (size_t)nq + 1) nq = (uint32_t)qe_off.size() - 1;
    std::cout << "query num: " << nq << std::endl;
    if (use_kw) {  // ref: src/query.cu:1828-1843
        std::vector<std::vector<uint32_t>> kw;
        rc = load_id_lines(keyword_id_path, nq, kw);
        if (rc != AP_OK) return rc;
        uint32_t cnt = 0;
        for (uint32_t i = 0; i < nq; ++i)
            for (uint32_t j = qbm.off[i]; j < qbm.off[i + 1]; ++j)
                for (uint32_t t : kw[i])
                    if (t == qbm.idx[j]) { qbm.idx[j] |= 0x80000000u; ++cnt; }
        std::cout << "keywords: " << cnt << std::endl;
    }
    std::cout << "Dense weight: " << dense_weight << ", Sparse weight: " << sparse_weight << ", BM25 weight: " << bm25_weight
              << ", KG weight: " << kg_weight << std::endl;
    rc = ap_index_load_graph(ix, graph_path);
    if (rc == AP_OK && use_kg) rc = ap_index_set_kg(ix, (uint32_t)e2e_off.size() - 1, e2e_off.data(), e2e_idx.data(), e2d_off.data(), e2d_idx.data());
    std::vector<uint32_t> ids((size_t)nq * cands);
    std::vector<float> dis((size_t)nq * cands);
    ap_search_stats st{};
    if (rc == AP_OK) {
        std::cout << "Points: " << n << ", Dim: " << AP_DIM << std::endl;
        std::cout << "Query: " << nq << ", Dim: " << AP_DIM << std::endl;
        ap_queries q{};
        q.nq = nq; q.dense = qdense.data(); q.sparse = qsp.view(); q.bm25 = qbm.view();
        if (use_kg) { q.ent_off = qe_off.data(); q.ent_idx = qe_idx.data(); }
        ap_search_opts o{};
        o.cands = (uint32_t)cands; o.flags = use_kw ? AP_SEARCH_KEYWORD : 0;
        o.sparse_weight = sparse_weight; o.bm25_weight = bm25_weight; o.dense_weight = dense_weight;
        o.kg_weight = use_kg ? kg_weight : 0.f;
        if (!use_kg && !(kg_weight < 1e-5f)) {  // the reference launches nothing in this case (src/query.cu:2042-2047)
            rc = fail(AP_ERR_ARG, "kg_weight = %g without a knowledge graph", kg_weight);
        } else {
            std::cout << "Begin search" << std::endl;
            const auto t0 = std::chrono::high_resolution_clock::now();
            rc = ap_search_host(ix, &q, &o, ids.data(), dis.data(), &st);
            const auto t1 = std::chrono::high_resolution_clock::now();
            if (rc == AP_OK) std::cout << "Query time: " << std::chrono::duration<float>(t1 - t0).count() << "s" << std::endl;
        }
    }
    if (rc == AP_OK) {
        if (out_ids) memcpy(out_ids, ids.data(), ids.size() * 4);
        if (out_dis) memcpy(out_dis, dis.data(), dis.size() * 4);
        if (out_nq) *out_nq = nq;
        if (stats) *stats = st;
        if (ground_truth_path && ground_truth_path[0]) {
            std::vector<std::vector<uint32_t>> rel;
            rc = load_id_lines(ground_truth_path, nq, rel);
            if (rc == AP_OK) {
                std::vector<uint32_t> off(nq + 1, 0), flat;
                for (uint32_t i = 0; i < nq; ++i) { flat.insert(flat.end(), rel[i].begin(), rel[i].end()); off[i + 1] = (uint32_t)flat.size(); }
                const double v = ap_ndcg(nq, ids.data(), (uint32_t)cands, (uint32_t)top_k, off.data(), flat.data());
                std::cout << "nDCG@10: " << (float)v << std::endl;
                if (out_ndcg) *out_ndcg = v;
            }
        }
    }
    return rc;
}

}  // extern "C"
