// Resident index: packing of the corpus into device records, graph installation, and the C ABI of the
// create / graph / search calls.
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "apoe_common.cuh"

namespace apoe {

// ---------------------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------------------
static thread_local char g_err[1024] = "";
void set_error(const char *fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof(g_err), fmt, ap); va_end(ap);
}
int fail(int code, const char *fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof(g_err), fmt, ap); va_end(ap);
    return code;
}

// ---------------------------------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------------------------------
// One warp per document: dense fp32 -> (x scale) -> half, CSR rows -> interleaved (id, value) pairs.
// ref for the conversions: src/index.cu:836-840 (x7 on fp32), include/utils.cuh:78-83 (__float2half).
__global__ void pack_records_kernel(uint32_t row0, uint32_t rows, const float *__restrict__ dense /* rows x stride */,
                                    float scale, const uint32_t *__restrict__ s_off, const uint32_t *__restrict__ s_idx,
                                    const float *__restrict__ s_val, const uint32_t *__restrict__ b_off,
                                    const uint32_t *__restrict__ b_idx, const float *__restrict__ b_val,
                                    const uint64_t *__restrict__ meta, uint8_t *__restrict__ rec, int write_sparse,
                                    uint32_t stride = kDim, uint32_t *__restrict__ bad_header = nullptr) {
    const uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= rows) return;
    const uint32_t d = row0 + w;
    const uint64_t m = meta[d];
    uint8_t *dst = rec + meta_off16(m) * 16ull;
    uint2 *dd = reinterpret_cast<uint2 *>(dst);
    if (stride == kDim) {
        const float4 *src = reinterpret_cast<const float4 *>(dense + (size_t)w * kDim);
        for (uint32_t i = lane; i < kDim / 4; i += 32) {
            const float4 f = __ldg(src + i);
            dd[i] = make_uint2(pack_half2(__fmul_rn(f.x, scale), __fmul_rn(f.y, scale)),
                               pack_half2(__fmul_rn(f.z, scale), __fmul_rn(f.w, scale)));
        }
    } else {
        // rows as they lie in an .fvecs file: one int32 dimension word, then the values (4-byte aligned only)
        const float *src = dense + (size_t)w * stride;
        if (lane == 0 && bad_header && __float_as_uint(src[0]) != kDim) atomicMin(bad_header, d);
        __half *dh = reinterpret_cast<__half *>(dst);
        for (uint32_t i = lane; i < kDim; i += 32) dh[i] = __float2half_rn(__fmul_rn(__ldg(src + 1 + i), scale));
    }
    if (!write_sparse) return;
    const uint32_t ns = meta_ns(m), nb = meta_nb(m);
    uint2 *sp = reinterpret_cast<uint2 *>(dst + kDenseBytes);
    const uint32_t s0 = s_off[d];
    for (uint32_t j = lane; j < pad2(ns); j += 32)
        sp[j] = j < ns ? make_uint2(s_idx[s0 + j], __float_as_uint(s_val[s0 + j])) : make_uint2(kEmpty, 0u);
    uint2 *bp = sp + pad2(ns);
    const uint32_t b0 = b_off[d];
    for (uint32_t j = lane; j < pad2(nb); j += 32)
        bp[j] = j < nb ? make_uint2(b_idx[b0 + j], __float_as_uint(b_val[b0 + j])) : make_uint2(kEmpty, 0u);
}

// Copies the sparse and BM25 sections of every record from one pool to another (same offsets).
__global__ void copy_sparse_sections_kernel(uint32_t n, const uint64_t *__restrict__ meta, const uint8_t *__restrict__ src,
                                            uint8_t *__restrict__ dst) {
    const uint32_t w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= n) return;
    const uint64_t m = meta[w];
    const size_t o = meta_off16(m) * 16ull + kDenseBytes;
    const uint32_t words = (pad2(meta_ns(m)) + pad2(meta_nb(m))) / 2;  // 16-byte units
    const uint4 *s = reinterpret_cast<const uint4 *>(src + o);
    uint4 *d = reinterpret_cast<uint4 *>(dst + o);
    for (uint32_t i = lane; i < words; i += 32) d[i] = s[i];
}

__global__ void fat_graph_kernel(uint32_t n, const uint32_t *__restrict__ graph, const uint64_t *__restrict__ meta,
                                 FatEdge *__restrict__ fat, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const uint32_t slot = (uint32_t)(i % AP_ROW);
    const uint32_t v = graph[i];
    FatEdge e{v, 0u, 0u, 0u};
    if (slot != AP_DEGREE && v < n) { const uint64_t m = meta[v]; e.meta_lo = (uint32_t)m; e.meta_hi = (uint32_t)(m >> 32); }
    fat[i] = e;
}

// Test hook for the bounded waits: one thread waits on an mbarrier that nothing ever completes.  After `limit`
// polls the wait gives up, raises the error word and the kernel returns normally -- the path every copy wait of
// the search and build kernels takes when its data does not arrive.
__global__ void wait_timeout_kernel(uint32_t *err_word, uint32_t limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_bounded(&bar, 0, err_word, 1u, limit);
}

// ---------------------------------------------------------------------------------------------------------
// creation
// ---------------------------------------------------------------------------------------------------------
int index_alloc(ap_index **out, int device, uint32_t n) {
    if (!out) return fail(AP_ERR_ARG, "null output handle");
    if (n == 0) return fail(AP_ERR_ARG, "empty corpus");
    int count = 0;
    AP_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return fail(AP_ERR_ARG, "device %d out of range (%d visible)", device, count);
    AP_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    AP_CUDA(cudaGetDeviceProperties(&prop, device));
    ap_index *ix = new ap_index();
    ix->device = device; ix->n = n; ix->num_sms = prop.multiProcessorCount;
    ix->smem_per_sm = prop.sharedMemPerMultiprocessor; ix->smem_per_block = prop.sharedMemPerBlockOptin;
    *out = ix;
    AP_CUDA(cudaMalloc(&ix->d_ctl, 16 * sizeof(uint32_t)));
    AP_CUDA(cudaMemset(ix->d_ctl, 0, 16 * sizeof(uint32_t)));
    AP_CUDA(cudaMalloc(&ix->d_cnt, 8 * sizeof(unsigned long long)));
    AP_CUDA(cudaMemset(ix->d_cnt, 0, 8 * sizeof(unsigned long long)));
    AP_CUDA(cudaEventCreate(&ix->ev0));
    AP_CUDA(cudaEventCreate(&ix->ev1));
    return AP_OK;
}

static int validate_offsets(const uint32_t *off, uint32_t rows, const char *what, uint32_t *max_nnz) {
    uint32_t mx = 0;
    if (off[0] != 0) return fail(AP_ERR_ARG, "%s: first offset is %u, expected 0", what, off[0]);
    for (uint32_t i = 0; i < rows; ++i) {
        if (off[i + 1] < off[i]) return fail(AP_ERR_ARG, "%s: offsets decrease at row %u", what, i);
        const uint32_t c = off[i + 1] - off[i];
        if (c > mx) mx = c;
    }
    if (mx > kMaxRowNnz) return fail(AP_ERR_LIMIT, "%s: a row holds %u entries, the limit is %u", what, mx, kMaxRowNnz);
    *max_nnz = mx;
    return AP_OK;
}

int ws_reserve(ap_index *ix, int slot, size_t bytes, void **out) {
    if (bytes == 0) bytes = 16;
    if (ix->ws.cap[slot] < bytes) {
        if (ix->ws.buf[slot]) AP_CUDA(cudaFree(ix->ws.buf[slot]));
        ix->ws.buf[slot] = nullptr; ix->ws.cap[slot] = 0;
        const size_t cap = bytes + bytes / 4 + 256;
        AP_CUDA(cudaMalloc(&ix->ws.buf[slot], cap));
        ix->ws.cap[slot] = cap;
    }
    *out = ix->ws.buf[slot];
    return AP_OK;
}

// Two pinned host buffers (and, on request, two device buffers) used alternately, so that filling buffer c + 1 on
// the host overlaps the upload (and packing) of buffer c on the stream.
struct Staging {
    void *pin[2] = {nullptr, nullptr}, *dev[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaStream_t st = nullptr;
    size_t bytes = 0;
    uint32_t uses = 0;
    int init(size_t b, bool with_dev) {
        bytes = b;
        AP_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            AP_CUDA(cudaMallocHost(&pin[i], bytes));
            if (with_dev) AP_CUDA(cudaMalloc(&dev[i], bytes));
            AP_CUDA(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
        return AP_OK;
    }
    int acquire(int *b) {   // the buffer whose previous use (two turns ago) has left the stream
        *b = (int)(uses & 1u);
        if (uses >= 2) AP_CUDA(cudaEventSynchronize(done[*b]));
        ++uses;
        return AP_OK;
    }
    int release(int b) { AP_CUDA(cudaEventRecord(done[b], st)); return AP_OK; }
    ~Staging() {
        if (st) cudaStreamSynchronize(st);
        for (int i = 0; i < 2; ++i) { if (pin[i]) cudaFreeHost(pin[i]); if (dev[i]) cudaFree(dev[i]); if (done[i]) cudaEventDestroy(done[i]); }
        if (st) cudaStreamDestroy(st);
    }
};

// One corpus array from the feed to device memory, through the staging buffers.
static int stream_array(const CorpusFeed &feed, int which, size_t bytes, void *d_dst, Staging &sg) {
    for (size_t o = 0; o < bytes; o += sg.bytes) {
        const size_t len = std::min(sg.bytes, bytes - o);
        int b;
        AP_TRY(sg.acquire(&b));
        AP_TRY(feed.read(sg.pin[b], which, o, len));
        AP_CUDA(cudaMemcpyAsync((uint8_t *)d_dst + o, sg.pin[b], len, cudaMemcpyHostToDevice, sg.st));
        AP_TRY(sg.release(b));
    }
    return AP_OK;
}

// Dense rows from the feed, in .fvecs layout (one dimension word, then 1024 floats per row), packed chunk by chunk.
static int pack_from_feed(ap_index *ix, const CorpusFeed &feed, Staging &sg, bool for_build, const uint32_t *d_soff, const uint32_t *d_sidx,
                          const float *d_sval, const uint32_t *d_boff, const uint32_t *d_bidx, const float *d_bval) {
    const uint32_t n = ix->n, stride = kDim + 1;
    const uint32_t chunk = (uint32_t)std::min<size_t>(n, sg.bytes / ((size_t)stride * 4));
    uint32_t *bad = reinterpret_cast<uint32_t *>(ix->d_ctl + 2);
    AP_CUDA(cudaMemsetAsync(bad, 0xFF, 4, sg.st));
    for (uint32_t r0 = 0; r0 < n; r0 += chunk) {
        const uint32_t rows = std::min(chunk, n - r0);
        int b;
        AP_TRY(sg.acquire(&b));
        AP_TRY(feed.read(sg.pin[b], 0, (size_t)r0 * stride * 4, (size_t)rows * stride * 4));
        AP_CUDA(cudaMemcpyAsync(sg.dev[b], sg.pin[b], (size_t)rows * stride * 4, cudaMemcpyHostToDevice, sg.st));
        const uint32_t blocks = (rows + 7) / 8;
        const float *src = (const float *)sg.dev[b];
        pack_records_kernel<<<blocks, 256, 0, sg.st>>>(r0, rows, src, 1.0f, d_soff, d_sidx, d_sval, d_boff, d_bidx, d_bval, ix->meta, ix->rec, 1, stride, bad);
        if (for_build)
            pack_records_kernel<<<blocks, 256, 0, sg.st>>>(r0, rows, src, 7.0f, d_soff, d_sidx, d_sval, d_boff, d_bidx, d_bval, ix->meta, ix->rec_build, 1, stride, nullptr);
        AP_CUDA(cudaGetLastError());
        AP_TRY(sg.release(b));
    }
    AP_CUDA(cudaStreamSynchronize(sg.st));
    uint32_t first_bad = 0xFFFFFFFFu;
    AP_CUDA(cudaMemcpy(&first_bad, bad, 4, cudaMemcpyDeviceToHost));
    AP_CUDA(cudaMemset(bad, 0, 4));
    if (first_bad != 0xFFFFFFFFu) return fail(AP_ERR_IO, "dense row %u does not start with the dimension word %u", first_bad, kDim);
    return AP_OK;
}

int index_pack(ap_index *ix, const float *dense, const uint32_t *s_off, const uint32_t *s_idx, const float *s_val,
               const uint32_t *b_off, const uint32_t *b_idx, const float *b_val, bool on_device, uint32_t flags,
               const CorpusFeed *feed) {
    const uint32_t n = ix->n;
    if ((!dense && !feed) || !s_off || !b_off) return fail(AP_ERR_ARG, "null corpus pointer");
    std::vector<uint32_t> hs(n + 1), hb(n + 1);
    if (on_device) {
        AP_CUDA(cudaMemcpy(hs.data(), s_off, (size_t)(n + 1) * 4, cudaMemcpyDeviceToHost));
        AP_CUDA(cudaMemcpy(hb.data(), b_off, (size_t)(n + 1) * 4, cudaMemcpyDeviceToHost));
    } else {
        memcpy(hs.data(), s_off, (size_t)(n + 1) * 4);
        memcpy(hb.data(), b_off, (size_t)(n + 1) * 4);
    }
    AP_TRY(validate_offsets(hs.data(), n, "sparse corpus", &ix->max_ns));
    AP_TRY(validate_offsets(hb.data(), n, "bm25 corpus", &ix->max_nb));
    if (!feed && ((hs[n] && (!s_idx || !s_val)) || (hb[n] && (!b_idx || !b_val)))) return fail(AP_ERR_ARG, "null CSR pointer");

    std::vector<uint64_t> meta(n);
    uint64_t off16 = 0;
    ix->max_rec_bytes = 0;
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t ns = hs[i + 1] - hs[i], nb = hb[i + 1] - hb[i];
        meta[i] = meta_pack(off16, ns, nb);
        const uint32_t rb = record_bytes(ns, nb);
        ix->max_rec_bytes = std::max(ix->max_rec_bytes, rb);
        off16 += rb / 16;
    }
    ix->rec_total = (size_t)off16 * 16;
    AP_CUDA(cudaMalloc(&ix->meta, (size_t)n * 8));
    AP_CUDA(cudaMemcpy(ix->meta, meta.data(), (size_t)n * 8, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMalloc(&ix->rec, ix->rec_total + 16));
    const bool for_build = (flags & AP_CREATE_FOR_BUILD) != 0;
    if (for_build) { AP_CUDA(cudaMalloc(&ix->rec_build, ix->rec_total + 16)); ix->build_scale = 7.0f; }

    // host sample for the weight auto-normalisation (first 100 documents)
    HostSample &sm = ix->sample;
    sm.n = std::min(n, 100u);
    sm.dense.resize((size_t)sm.n * kDim);
    sm.s_off.assign(hs.begin(), hs.begin() + sm.n + 1);
    sm.b_off.assign(hb.begin(), hb.begin() + sm.n + 1);
    sm.s_idx.resize(sm.s_off[sm.n]); sm.s_val.resize(sm.s_off[sm.n]);
    sm.b_idx.resize(sm.b_off[sm.n]); sm.b_val.resize(sm.b_off[sm.n]);
    const cudaMemcpyKind k = on_device ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost;
    if (feed) {
        std::vector<float> rows((size_t)sm.n * (kDim + 1));
        AP_TRY(feed->read(rows.data(), 0, 0, rows.size() * 4));
        for (uint32_t i = 0; i < sm.n; ++i) memcpy(&sm.dense[(size_t)i * kDim], &rows[(size_t)i * (kDim + 1) + 1], (size_t)kDim * 4);
        if (!sm.s_idx.empty()) { AP_TRY(feed->read(sm.s_idx.data(), 1, 0, sm.s_idx.size() * 4)); AP_TRY(feed->read(sm.s_val.data(), 2, 0, sm.s_val.size() * 4)); }
        if (!sm.b_idx.empty()) { AP_TRY(feed->read(sm.b_idx.data(), 3, 0, sm.b_idx.size() * 4)); AP_TRY(feed->read(sm.b_val.data(), 4, 0, sm.b_val.size() * 4)); }
    } else {
        AP_CUDA(cudaMemcpy(sm.dense.data(), dense, sm.dense.size() * 4, k));
        if (!sm.s_idx.empty()) { AP_CUDA(cudaMemcpy(sm.s_idx.data(), s_idx, sm.s_idx.size() * 4, k)); AP_CUDA(cudaMemcpy(sm.s_val.data(), s_val, sm.s_val.size() * 4, k)); }
        if (!sm.b_idx.empty()) { AP_CUDA(cudaMemcpy(sm.b_idx.data(), b_idx, sm.b_idx.size() * 4, k)); AP_CUDA(cudaMemcpy(sm.b_val.data(), b_val, sm.b_val.size() * 4, k)); }
    }

    // CSR arrays on the device
    const uint32_t *d_soff = s_off, *d_sidx = s_idx, *d_boff = b_off, *d_bidx = b_idx;
    const float *d_sval = s_val, *d_bval = b_val;
    void *tmp[6] = {nullptr};
    auto up = [&](int slot, const void *src, size_t bytes, const void **dst) -> int {
        AP_CUDA(cudaMalloc(&tmp[slot], std::max<size_t>(bytes, 16)));
        if (src) AP_CUDA(cudaMemcpy(tmp[slot], src, bytes, cudaMemcpyHostToDevice));
        *dst = tmp[slot];
        return AP_OK;
    };
    int rc = AP_OK;
    Staging sg;
    if (!on_device) {
        rc = up(0, s_off, (size_t)(n + 1) * 4, (const void **)&d_soff);
        if (rc == AP_OK) rc = up(1, s_idx, (size_t)hs[n] * 4, (const void **)&d_sidx);
        if (rc == AP_OK) rc = up(2, s_val, (size_t)hs[n] * 4, (const void **)&d_sval);
        if (rc == AP_OK) rc = up(3, b_off, (size_t)(n + 1) * 4, (const void **)&d_boff);
        if (rc == AP_OK) rc = up(4, b_idx, (size_t)hb[n] * 4, (const void **)&d_bidx);
        if (rc == AP_OK) rc = up(5, b_val, (size_t)hb[n] * 4, (const void **)&d_bval);
    }
    if (rc == AP_OK && feed) {   // the arrays the uploads above left empty come from the feed
        rc = sg.init((size_t)16384 * (kDim + 1) * 4, true);
        if (rc == AP_OK) rc = stream_array(*feed, 1, (size_t)hs[n] * 4, tmp[1], sg);
        if (rc == AP_OK) rc = stream_array(*feed, 2, (size_t)hs[n] * 4, tmp[2], sg);
        if (rc == AP_OK) rc = stream_array(*feed, 3, (size_t)hb[n] * 4, tmp[4], sg);
        if (rc == AP_OK) rc = stream_array(*feed, 4, (size_t)hb[n] * 4, tmp[5], sg);
        if (rc == AP_OK) rc = pack_from_feed(ix, *feed, sg, for_build, d_soff, d_sidx, d_sval, d_boff, d_bidx, d_bval);
    }
    // dense: straight from device memory, or through a staging buffer in chunks of rows
    const uint32_t chunk = on_device ? n : std::min(n, 65536u);
    float *stage = nullptr;
    if (rc == AP_OK && !on_device && !feed) {
        cudaError_t e = cudaMalloc(&stage, (size_t)chunk * kDim * 4);
        if (e != cudaSuccess) rc = fail(AP_ERR_CUDA, "cudaMalloc(staging) failed: %s", cudaGetErrorString(e));
    }
    for (uint32_t r0 = 0; rc == AP_OK && !feed && r0 < n; r0 += chunk) {
        const uint32_t rows = std::min(chunk, n - r0);
        const float *src = dense + (size_t)r0 * kDim;
        if (!on_device) {
            cudaError_t e = cudaMemcpy(stage, src, (size_t)rows * kDim * 4, cudaMemcpyHostToDevice);
            if (e != cudaSuccess) { rc = fail(AP_ERR_CUDA, "dense upload failed: %s", cudaGetErrorString(e)); break; }
            src = stage;
        }
        const uint32_t blocks = (rows + 7) / 8;
        pack_records_kernel<<<blocks, 256>>>(r0, rows, src, 1.0f, d_soff, d_sidx, d_sval, d_boff, d_bidx, d_bval, ix->meta, ix->rec, 1);
        if (for_build)
            pack_records_kernel<<<blocks, 256>>>(r0, rows, src, 7.0f, d_soff, d_sidx, d_sval, d_boff, d_bidx, d_bval, ix->meta, ix->rec_build, 1);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(AP_ERR_CUDA, "pack kernel launch failed: %s", cudaGetErrorString(e));
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (rc == AP_OK && e != cudaSuccess) rc = fail(AP_ERR_CUDA, "packing failed: %s", cudaGetErrorString(e));
    if (stage) cudaFree(stage);
    for (void *p : tmp) if (p) cudaFree(p);
    if (on_device && for_build) ix->dense_src = dense;
    return rc;
}

// Make sure the build-time copy holds dense x scale (re-converted from the caller's fp32 rows when possible).
int ensure_build_copy(ap_index *ix, float scale) {
    if (!ix->rec_build) return fail(AP_ERR_STATE, "the index was created without AP_CREATE_FOR_BUILD");
    if (ix->build_scale == scale) return AP_OK;
    if (!ix->dense_src) return fail(AP_ERR_STATE, "dense_scale %g differs from the packed copy (%g) and the fp32 rows are gone", scale, ix->build_scale);
    const uint32_t blocks = (ix->n + 7) / 8;
    pack_records_kernel<<<blocks, 256>>>(0, ix->n, ix->dense_src, scale, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, ix->meta, ix->rec_build, 0);
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaDeviceSynchronize());
    ix->build_scale = scale;
    return AP_OK;
}

int index_install_graph(ap_index *ix) {
    const size_t total = (size_t)ix->n * AP_ROW;
    if (!ix->fat) AP_CUDA(cudaMalloc(&ix->fat, total * sizeof(FatEdge)));
    if (!ix->ep_fat) AP_CUDA(cudaMalloc(&ix->ep_fat, AP_ENTRY_POINTS * sizeof(FatEdge)));
    fat_graph_kernel<<<(uint32_t)((total + 255) / 256), 256>>>(ix->n, ix->graph, ix->meta, ix->fat, total);
    // entry points as one more "row" of 32 edges; slot 32 does not exist there, so reuse the kernel with a
    // row width trick: 32 < AP_ROW keeps every slot on the id path
    fat_graph_kernel<<<1, 32>>>(ix->n, ix->ep, ix->meta, ix->ep_fat, AP_ENTRY_POINTS);
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaDeviceSynchronize());
    ix->has_graph = true;
    return AP_OK;
}

static int check_graph_rows(uint32_t n, const uint32_t *rows, const uint32_t *ep) {
    for (uint32_t i = 0; i < AP_ENTRY_POINTS; ++i)
        if (ep[i] >= n) return fail(AP_ERR_ARG, "entry point %u = %u is not a document id (n = %u)", i, ep[i], n);
    for (uint32_t d = 0; d < n; ++d) {
        const uint32_t *r = rows + (size_t)d * AP_ROW;
        for (uint32_t j = 0; j < AP_DEGREE; ++j)
            if (r[j] >= n) return fail(AP_ERR_ARG, "graph row %u slot %u = %u is not a document id (n = %u)", d, j, r[j], n);
        if (r[AP_DEGREE] > AP_ROW - AP_DEGREE - 1) return fail(AP_ERR_ARG, "graph row %u holds keyword-edge count %u", d, r[AP_DEGREE]);
        for (uint32_t j = 0; j < r[AP_DEGREE]; ++j)
            if (r[AP_DEGREE + 1 + j] >= n) return fail(AP_ERR_ARG, "graph row %u keyword edge %u = %u is not a document id", d, j, r[AP_DEGREE + 1 + j]);
    }
    return AP_OK;
}

// ---------------------------------------------------------------------------------------------------------
// weights, dispatch
// ---------------------------------------------------------------------------------------------------------
static float dot_seq(const float *a, const float *b) { float r = 0.f; for (uint32_t i = 0; i < kDim; ++i) r += a[i] * b[i]; return r; }
static float merge_ip(const uint32_t *i1, const float *v1, uint32_t n1, const uint32_t *i2, const float *v2, uint32_t n2) {
    float r = 0.f; uint32_t p1 = 0, p2 = 0;
    while (p1 < n1 && p2 < n2) {
        const uint32_t x = i1[p1], y = i2[p2] & 0x7FFFFFFFu;
        if (x < y) ++p1; else if (x > y) ++p2; else { r += v1[p1] * v2[p2]; ++p1; ++p2; }
    }
    return r;
}

// ref: src/query.cu:1847-1869 (first 100 docs x first 100 queries, exact fp32 inner products per path)
static int effective_weights_host(const ap_index *ix, const ap_queries *q, float *ws, float *wb, float *wd) {
    const HostSample &sm = ix->sample;
    const uint32_t nd = std::min(sm.n, std::min(q->nq, 100u)), nqq = std::min(q->nq, std::min(ix->n, 100u));
    if (nd == 0 || nqq == 0) return AP_OK;
    float r1 = 0, r2 = 0, r3 = 0; bool first = true;
    for (uint32_t bb = 0; bb < nqq; ++bb)
        for (uint32_t aa = 0; aa < nd; ++aa) {
            const float d = -dot_seq(sm.dense.data() + (size_t)aa * kDim, q->dense + (size_t)bb * kDim);
            const float s = -merge_ip(sm.s_idx.data() + sm.s_off[aa], sm.s_val.data() + sm.s_off[aa], sm.s_off[aa + 1] - sm.s_off[aa],
                                      q->sparse.idx + q->sparse.off[bb], q->sparse.val + q->sparse.off[bb], q->sparse.off[bb + 1] - q->sparse.off[bb]);
            const float b = -merge_ip(sm.b_idx.data() + sm.b_off[aa], sm.b_val.data() + sm.b_off[aa], sm.b_off[aa + 1] - sm.b_off[aa],
                                      q->bm25.idx + q->bm25.off[bb], q->bm25.val + q->bm25.off[bb], q->bm25.off[bb + 1] - q->bm25.off[bb]);
            if (first || d < r1) r1 = d;
            if (first || s < r2) r2 = s;
            if (first || b < r3) r3 = b;
            first = false;
        }
    if ((-r2) > (-r3) && (-r2) > (-r1)) { *wb *= (r2 / r3); *wd *= (r2 / r1); }
    else if ((-r3) > (-r2) && (-r3) > (-r1)) { *ws *= (r3 / r2); *wd *= (r3 / r1); }
    else if ((-r1) > (-r2) && (-r1) > (-r3)) { *ws *= (r1 / r2); *wb *= (r1 / r3); }
    return AP_OK;
}

// ref: the kernel dispatch of src/query.cu:2004-2047 on the rescaled weights, thresholds 1e-5
static int dispatch_path(uint32_t flags, float ws, float wb, float wd, float kg_weight, uint32_t *path, uint32_t *mode) {
    *mode = 0;
    if (!(kg_weight < 1e-5f)) { *path = 7; *mode = AP_SEARCH_KG; return AP_OK; }
    if (flags & AP_SEARCH_KEYWORD) { *path = 7; *mode = AP_SEARCH_KEYWORD; return AP_OK; }
    if (wb < 1e-5f) {
        if (ws > 1e-5f && wd > 1e-5f) *path = AP_PATH_DENSE | AP_PATH_SPARSE;
        else if (ws < 1e-5f && wd > 1e-5f) *path = AP_PATH_DENSE;
        else if (ws > 1e-5f && wd < 1e-5f) *path = AP_PATH_SPARSE;
        else return fail(AP_ERR_ARG, "no path has a weight above 1e-5 (the reference launches nothing in this case)");
    } else {
        if (ws > 1e-5f && wd > 1e-5f) *path = 7;
        else if (ws < 1e-5f && wd > 1e-5f) *path = AP_PATH_DENSE | AP_PATH_BM25;
        else if (ws > 1e-5f && wd < 1e-5f) *path = AP_PATH_SPARSE | AP_PATH_BM25;
        else *path = AP_PATH_BM25;
    }
    return AP_OK;
}

static int check_search_args(const ap_index *ix, const ap_queries *q, const ap_search_opts *o) {
    if (!ix || !q || !o) return fail(AP_ERR_ARG, "null argument");
    if (!ix->has_graph) return fail(AP_ERR_STATE, "no graph installed: build, load or set one first");
    if (o->cands < 32 || o->cands > AP_MAX_CANDS || (o->cands % 32) != 0)
        return fail(AP_ERR_ARG, "cands = %u: must be a multiple of 32 in [32, %d]", o->cands, AP_MAX_CANDS);
    if (q->nq == 0) return fail(AP_ERR_ARG, "no queries");
    if (!q->dense || !q->sparse.off || !q->bm25.off) return fail(AP_ERR_ARG, "null query pointer");
    return AP_OK;
}

static int read_back_status(ap_index *ix, ap_search_stats *stats, cudaStream_t stream) {
    uint32_t ctl[2] = {0, 0};
    unsigned long long cnt[3] = {0, 0, 0};
    AP_CUDA(cudaMemcpyAsync(ctl, ix->d_ctl, 8, cudaMemcpyDeviceToHost, stream));
    AP_CUDA(cudaMemcpyAsync(cnt, ix->d_cnt, 24, cudaMemcpyDeviceToHost, stream));
    AP_CUDA(cudaStreamSynchronize(stream));
    if (stats) { stats->expansions = cnt[0]; stats->evaluations = cnt[1]; stats->gathered_bytes = cnt[2]; }
    if (ctl[1] != 0) {
        const uint32_t code = ctl[1];
        cudaMemset(ix->d_ctl + 1, 0, 4);
        return fail(AP_ERR_DEVICE, "search kernel raised error word %u (%s)", code,
                    code == 1 ? "a bulk copy did not complete within the wait limit" : "a record is larger than the staging arena");
    }
    return AP_OK;
}

}  // namespace apoe

using namespace apoe;

// ---------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------
extern "C" {

const char *ap_last_error(void) { return g_err; }
int ap_version(void) { return 100; }

int ap_index_create_host(ap_index **out, int device, uint32_t n, const float *dense, ap_csr sparse, ap_csr bm25, uint32_t flags) {
    AP_TRY(index_alloc(out, device, n));
    const int rc = index_pack(*out, dense, sparse.off, sparse.idx, sparse.val, bm25.off, bm25.idx, bm25.val, false, flags);
    if (rc != AP_OK) { ap_index_destroy(*out); *out = nullptr; }
    return rc;
}
int ap_index_create_device(ap_index **out, int device, uint32_t n, const float *dense, ap_csr sparse, ap_csr bm25, uint32_t flags) {
    AP_TRY(index_alloc(out, device, n));
    const int rc = index_pack(*out, dense, sparse.off, sparse.idx, sparse.val, bm25.off, bm25.idx, bm25.val, true, flags);
    if (rc != AP_OK) { ap_index_destroy(*out); *out = nullptr; }
    return rc;
}

int ap_index_destroy(ap_index *ix) {
    if (!ix) return AP_OK;
    cudaSetDevice(ix->device);
    exact_release(ix);
    void *ptrs[] = {ix->rec, ix->rec_build, ix->meta, ix->graph, ix->fat, ix->ep, ix->ep_fat, ix->knn_ids, ix->knn_dis, ix->power,
                    ix->e2e_off, ix->e2e_idx, ix->e2d_off, ix->e2d_idx, ix->d_ctl, ix->d_cnt};
    for (void *p : ptrs) if (p) cudaFree(p);
    for (void *p : ix->ws.buf) if (p) cudaFree(p);
    if (ix->ev0) cudaEventDestroy(ix->ev0);
    if (ix->ev1) cudaEventDestroy(ix->ev1);
    delete ix;
    return AP_OK;
}

uint32_t ap_index_size(const ap_index *ix) { return ix ? ix->n : 0; }

int ap_index_set_graph(ap_index *ix, const uint32_t *rows, const uint32_t *entry_points) {
    if (!ix || !rows || !entry_points) return fail(AP_ERR_ARG, "null argument");
    AP_TRY(check_graph_rows(ix->n, rows, entry_points));
    AP_CUDA(cudaSetDevice(ix->device));
    if (!ix->graph) AP_CUDA(cudaMalloc(&ix->graph, (size_t)ix->n * AP_ROW * 4));
    if (!ix->ep) AP_CUDA(cudaMalloc(&ix->ep, AP_ENTRY_POINTS * 4));
    AP_CUDA(cudaMemcpy(ix->graph, rows, (size_t)ix->n * AP_ROW * 4, cudaMemcpyHostToDevice));
    AP_CUDA(cudaMemcpy(ix->ep, entry_points, AP_ENTRY_POINTS * 4, cudaMemcpyHostToDevice));
    return index_install_graph(ix);
}

int ap_index_get_graph(const ap_index *ix, uint32_t *rows, uint32_t *entry_points) {
    if (!ix) return fail(AP_ERR_ARG, "null index");
    if (!ix->has_graph) return fail(AP_ERR_STATE, "no graph installed");
    AP_CUDA(cudaSetDevice(ix->device));
    if (rows) AP_CUDA(cudaMemcpy(rows, ix->graph, (size_t)ix->n * AP_ROW * 4, cudaMemcpyDeviceToHost));
    if (entry_points) AP_CUDA(cudaMemcpy(entry_points, ix->ep, AP_ENTRY_POINTS * 4, cudaMemcpyDeviceToHost));
    return AP_OK;
}

int ap_index_set_kg(ap_index *ix, uint32_t n_entities, const uint32_t *e2e_off, const uint32_t *e2e_idx,
                    const uint32_t *e2d_off, const uint32_t *e2d_idx) {
    if (!ix || !e2e_off || !e2d_off) return fail(AP_ERR_ARG, "null argument");
    uint32_t mx;
    AP_TRY(validate_offsets(e2e_off, n_entities, "entity graph", &mx));
    AP_TRY(validate_offsets(e2d_off, n_entities, "entity->doc map", &mx));
    for (uint32_t i = 0; i < e2e_off[n_entities]; ++i)
        if (e2e_idx[i] >= n_entities) return fail(AP_ERR_ARG, "entity graph edge %u points at entity %u of %u", i, e2e_idx[i], n_entities);
    for (uint32_t i = 0; i < e2d_off[n_entities]; ++i)
        if (e2d_idx[i] >= ix->n) return fail(AP_ERR_ARG, "entity->doc entry %u = %u is not a document id", i, e2d_idx[i]);
    AP_CUDA(cudaSetDevice(ix->device));
    void *old[] = {ix->e2e_off, ix->e2e_idx, ix->e2d_off, ix->e2d_idx};
    for (void *p : old) if (p) cudaFree(p);
    ix->e2e_off = ix->e2e_idx = ix->e2d_off = ix->e2d_idx = nullptr;
    auto up = [&](uint32_t **dst, const uint32_t *src, size_t cnt) -> int {
        AP_CUDA(cudaMalloc(dst, std::max<size_t>(cnt, 4) * 4));
        if (cnt) AP_CUDA(cudaMemcpy(*dst, src, cnt * 4, cudaMemcpyHostToDevice));
        return AP_OK;
    };
    AP_TRY(up(&ix->e2e_off, e2e_off, n_entities + 1));
    AP_TRY(up(&ix->e2e_idx, e2e_idx, e2e_off[n_entities]));
    AP_TRY(up(&ix->e2d_off, e2d_off, n_entities + 1));
    AP_TRY(up(&ix->e2d_idx, e2d_idx, e2d_off[n_entities]));
    ix->n_ent = n_entities;
    return AP_OK;
}

int ap_index_check_status(ap_index *ix) {
    if (!ix) return fail(AP_ERR_ARG, "null index");
    AP_CUDA(cudaSetDevice(ix->device));
    uint32_t word = 0;
    AP_CUDA(cudaMemcpy(&word, ix->d_ctl + 1, 4, cudaMemcpyDeviceToHost));   // default stream: after the work queued there
    if (word != 0) {
        AP_CUDA(cudaMemset(ix->d_ctl + 1, 0, 4));
        return fail(AP_ERR_DEVICE, "a kernel raised error word %u (%s)", word,
                    word == 1 ? "a bulk copy did not complete within the wait limit" : word == 2 ? "a record is larger than the staging arena" : "a bounded wait ran out");
    }
    return AP_OK;
}

int ap_debug_wait_timeout(ap_index *ix, uint32_t polls) {
    if (!ix) return fail(AP_ERR_ARG, "null index");
    AP_CUDA(cudaSetDevice(ix->device));
    wait_timeout_kernel<<<1, 32>>>(ix->d_ctl + 1, polls > 4096u ? 4096u : polls);
    AP_CUDA(cudaGetLastError());
    AP_CUDA(cudaDeviceSynchronize());
    return AP_OK;
}

int ap_effective_weights(const ap_index *ix, const ap_queries *q, float *sparse_weight, float *bm25_weight, float *dense_weight) {
    if (!ix || !q || !sparse_weight || !bm25_weight || !dense_weight) return fail(AP_ERR_ARG, "null argument");
    return effective_weights_host(ix, q, sparse_weight, bm25_weight, dense_weight);
}

static int host_query_limits(const ap_index *ix, const ap_queries *q, uint32_t flags, uint32_t *mqs, uint32_t *mqb) {
    AP_TRY(validate_offsets(q->sparse.off, q->nq, "sparse queries", mqs));
    AP_TRY(validate_offsets(q->bm25.off, q->nq, "bm25 queries", mqb));
    if (*mqs > 2048 || *mqb > 2048) return fail(AP_ERR_LIMIT, "a query row holds more than 2048 terms");
    if (flags & AP_SEARCH_KG) {
        if (!q->ent_off || !q->ent_idx) return fail(AP_ERR_ARG, "KG search needs the query->entity CSR");
        uint32_t mx;
        AP_TRY(validate_offsets(q->ent_off, q->nq, "query entities", &mx));
        for (uint32_t i = 0; i < q->ent_off[q->nq]; ++i)
            if (q->ent_idx[i] >= ix->n_ent) return fail(AP_ERR_ARG, "query entity %u is not an entity id", q->ent_idx[i]);
    }
    return AP_OK;
}

static int search_host_impl(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids, float *out_dis,
                            unsigned long long *out_keys, uint32_t key_top_k, uint32_t id_base, ap_search_stats *stats) {
    const auto t0 = std::chrono::high_resolution_clock::now();
    AP_TRY(check_search_args(ix, q, opts));
    if ((!out_ids || !out_dis) && !out_keys) return fail(AP_ERR_ARG, "null output pointer");
    if (out_keys && (key_top_k == 0 || key_top_k > opts->cands)) return fail(AP_ERR_ARG, "top_k = %u must lie in [1, cands = %u]", key_top_k, opts->cands);
    AP_CUDA(cudaSetDevice(ix->device));
    float ws = opts->sparse_weight, wb = opts->bm25_weight, wd = opts->dense_weight;
    if (!(opts->flags & AP_SEARCH_RAW_WEIGHTS)) AP_TRY(effective_weights_host(ix, q, &ws, &wb, &wd));
    uint32_t path = 0, mode = 0;
    AP_TRY(dispatch_path(opts->flags, ws, wb, wd, opts->kg_weight, &path, &mode));
    if ((mode & AP_SEARCH_KG) && ix->n_ent == 0) return fail(AP_ERR_STATE, "kg_weight >= 1e-5 but no knowledge graph is loaded");
    uint32_t mqs = 0, mqb = 0;
    AP_TRY(host_query_limits(ix, q, mode, &mqs, &mqb));

    const uint32_t nq = q->nq, cands = opts->cands;
    const size_t nzs = q->sparse.off[nq], nzb = q->bm25.off[nq];
    SearchLaunch L{};
    void *p;
    cudaStream_t st = 0;
    size_t h2d = 0;
    auto upload = [&](int slot, const void *src, size_t bytes, const void **dst) -> int {
        AP_TRY(ws_reserve(ix, slot, bytes, &p));
        if (bytes) AP_CUDA(cudaMemcpyAsync(p, src, bytes, cudaMemcpyHostToDevice, st));
        h2d += bytes;
        *dst = p;
        return AP_OK;
    };
    AP_TRY(upload(0, q->dense, (size_t)nq * kDim * 4, (const void **)&L.qdense));
    AP_TRY(upload(1, q->sparse.off, (size_t)(nq + 1) * 4, (const void **)&L.qs_off));
    AP_TRY(upload(2, q->sparse.idx, nzs * 4, (const void **)&L.qs_idx));
    AP_TRY(upload(3, q->sparse.val, nzs * 4, (const void **)&L.qs_val));
    AP_TRY(upload(4, q->bm25.off, (size_t)(nq + 1) * 4, (const void **)&L.qb_off));
    AP_TRY(upload(5, q->bm25.idx, nzb * 4, (const void **)&L.qb_idx));
    AP_TRY(upload(6, q->bm25.val, nzb * 4, (const void **)&L.qb_val));
    if (mode & AP_SEARCH_KG) {
        AP_TRY(upload(7, q->ent_off, (size_t)(nq + 1) * 4, (const void **)&L.qe_off));
        AP_TRY(upload(8, q->ent_idx, (size_t)q->ent_off[nq] * 4, (const void **)&L.qe_idx));
    }
    const bool want_lists = out_ids && out_dis;
    if (want_lists) {
        AP_TRY(ws_reserve(ix, 9, (size_t)nq * cands * 4, &p)); L.out_ids = (uint32_t *)p;
        AP_TRY(ws_reserve(ix, 10, (size_t)nq * cands * 4, &p)); L.out_dis = (float *)p;
    }
    if (out_keys) {
        AP_TRY(ws_reserve(ix, 14, (size_t)nq * key_top_k * 8, &p)); L.out_keys = (unsigned long long *)p;
        L.key_top_k = key_top_k; L.id_base = id_base;
    }
    L.nq = nq; L.max_qs = mqs; L.max_qb = mqb;
    L.w_sparse = ws; L.w_bm25 = wb; L.w_dense = wd; L.kg_weight = opts->kg_weight;
    L.cands = cands; L.flags = (opts->flags & ~(AP_SEARCH_KEYWORD | AP_SEARCH_KG)) | mode; L.path = path;
    L.arena_bytes = opts->arena_bytes; L.ctas_per_sm = opts->ctas_per_sm; L.stream = st;
    uint32_t launches = 0;
    AP_CUDA(cudaMemsetAsync(ix->d_cnt, 0, 64, st));
    AP_CUDA(cudaEventRecord(ix->ev0, st));
    AP_TRY(search_launch(ix, L, &launches));
    AP_CUDA(cudaEventRecord(ix->ev1, st));
    if (want_lists) {
        AP_CUDA(cudaMemcpyAsync(out_ids, L.out_ids, (size_t)nq * cands * 4, cudaMemcpyDeviceToHost, st));
        AP_CUDA(cudaMemcpyAsync(out_dis, L.out_dis, (size_t)nq * cands * 4, cudaMemcpyDeviceToHost, st));
    }
    if (out_keys) AP_CUDA(cudaMemcpyAsync(out_keys, L.out_keys, (size_t)nq * key_top_k * 8, cudaMemcpyDeviceToHost, st));
    AP_TRY(read_back_status(ix, stats, st));
    if (stats) {
        float ms = 0.f;
        AP_CUDA(cudaEventElapsedTime(&ms, ix->ev0, ix->ev1));
        stats->kernel_ms = ms;
        stats->eff_sparse = ws; stats->eff_bm25 = wb; stats->eff_dense = wd; stats->path = path; stats->launches = launches;
        const size_t d2h = (want_lists ? (size_t)nq * cands * 8 : 0) + (out_keys ? (size_t)nq * key_top_k * 8 : 0);
        stats->h2d_bytes_lo = (uint32_t)h2d; stats->h2d_bytes_hi = (uint32_t)((uint64_t)h2d >> 32);
        stats->d2h_bytes_lo = (uint32_t)d2h; stats->d2h_bytes_hi = (uint32_t)((uint64_t)d2h >> 32);
        stats->total_ms = std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count();
    }
    return AP_OK;
}

int ap_search_host(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids, float *out_dis,
                   ap_search_stats *stats) {
    if (!out_ids || !out_dis) return fail(AP_ERR_ARG, "null output pointer");
    return search_host_impl(ix, q, opts, out_ids, out_dis, nullptr, 0, 0, stats);
}

int ap_search_shard_host(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t id_base, uint32_t top_k,
                         unsigned long long *out_keys, uint32_t *out_ids, float *out_dis, ap_search_stats *stats) {
    if (!out_keys) return fail(AP_ERR_ARG, "null output pointer");
    if (ix && (uint64_t)id_base + ix->n > 0xFFFFFFFFull) return fail(AP_ERR_ARG, "id base %u + %u documents leaves the 32-bit id range", id_base, ix->n);
    return search_host_impl(ix, q, opts, out_ids, out_dis, out_keys, top_k, id_base, stats);
}

static int search_device_impl(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids, float *out_dis,
                              unsigned long long *out_keys, uint32_t key_top_k, uint32_t id_base, void *stream, ap_search_stats *stats) {
    const auto t0 = std::chrono::high_resolution_clock::now();
    AP_TRY(check_search_args(ix, q, opts));
    if ((!out_ids || !out_dis) && !out_keys) return fail(AP_ERR_ARG, "null output pointer");
    if (out_keys && (key_top_k == 0 || key_top_k > opts->cands)) return fail(AP_ERR_ARG, "top_k = %u must lie in [1, cands = %u]", key_top_k, opts->cands);
    AP_CUDA(cudaSetDevice(ix->device));
    cudaStream_t st = (cudaStream_t)stream;
    const float ws = opts->sparse_weight, wb = opts->bm25_weight, wd = opts->dense_weight;
    uint32_t path = 0, mode = 0;
    AP_TRY(dispatch_path(opts->flags, ws, wb, wd, opts->kg_weight, &path, &mode));
    if ((mode & AP_SEARCH_KG) && (ix->n_ent == 0 || !q->ent_off || !q->ent_idx)) return fail(AP_ERR_STATE, "KG search without a knowledge graph or query entities");
    uint32_t mqs = q->max_sparse_nnz, mqb = q->max_bm25_nnz;
    if (mqs == 0 || mqb == 0) {  // read the offsets back and check them
        std::vector<uint32_t> so(q->nq + 1), bo(q->nq + 1);
        AP_CUDA(cudaMemcpyAsync(so.data(), q->sparse.off, (size_t)(q->nq + 1) * 4, cudaMemcpyDeviceToHost, st));
        AP_CUDA(cudaMemcpyAsync(bo.data(), q->bm25.off, (size_t)(q->nq + 1) * 4, cudaMemcpyDeviceToHost, st));
        AP_CUDA(cudaStreamSynchronize(st));
        AP_TRY(validate_offsets(so.data(), q->nq, "sparse queries", &mqs));
        AP_TRY(validate_offsets(bo.data(), q->nq, "bm25 queries", &mqb));
    }
    if (mqs > 2048 || mqb > 2048) return fail(AP_ERR_LIMIT, "a query row holds more than 2048 terms");
    SearchLaunch L{};
    L.qdense = q->dense; L.qs_off = q->sparse.off; L.qs_idx = q->sparse.idx; L.qs_val = q->sparse.val;
    L.qb_off = q->bm25.off; L.qb_idx = q->bm25.idx; L.qb_val = q->bm25.val; L.qe_off = q->ent_off; L.qe_idx = q->ent_idx;
    L.nq = q->nq; L.max_qs = mqs; L.max_qb = mqb;
    L.w_sparse = ws; L.w_bm25 = wb; L.w_dense = wd; L.kg_weight = opts->kg_weight;
    L.cands = opts->cands; L.flags = (opts->flags & ~(AP_SEARCH_KEYWORD | AP_SEARCH_KG)) | mode; L.path = path;
    L.arena_bytes = opts->arena_bytes; L.ctas_per_sm = opts->ctas_per_sm; L.stream = st;
    L.out_ids = out_dis ? out_ids : nullptr; L.out_dis = out_ids ? out_dis : nullptr;
    L.out_keys = out_keys; L.key_top_k = key_top_k; L.id_base = id_base;
    uint32_t launches = 0;
    AP_CUDA(cudaMemsetAsync(ix->d_cnt, 0, 64, st));
    if (stats) AP_CUDA(cudaEventRecord(ix->ev0, st));
    AP_TRY(search_launch(ix, L, &launches));
    if (stats) {
        AP_CUDA(cudaEventRecord(ix->ev1, st));
        AP_TRY(read_back_status(ix, stats, st));
        float ms = 0.f;
        AP_CUDA(cudaEventElapsedTime(&ms, ix->ev0, ix->ev1));
        stats->kernel_ms = ms;
        stats->eff_sparse = ws; stats->eff_bm25 = wb; stats->eff_dense = wd; stats->path = path; stats->launches = launches;
        stats->total_ms = std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count();
    }
    return AP_OK;
}

int ap_search_device(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids, float *out_dis,
                     void *stream, ap_search_stats *stats) {
    if (!out_ids || !out_dis) return fail(AP_ERR_ARG, "null output pointer");
    return search_device_impl(ix, q, opts, out_ids, out_dis, nullptr, 0, 0, stream, stats);
}

int ap_search_shard_device(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t id_base, uint32_t top_k,
                           unsigned long long *out_keys, uint32_t *out_ids, float *out_dis, void *stream, ap_search_stats *stats) {
    if (!out_keys) return fail(AP_ERR_ARG, "null output pointer");
    if (ix && (uint64_t)id_base + ix->n > 0xFFFFFFFFull) return fail(AP_ERR_ARG, "id base %u + %u documents leaves the 32-bit id range", id_base, ix->n);
    return search_device_impl(ix, q, opts, out_ids, out_dis, out_keys, top_k, id_base, stream, stats);
}

int ap_fused_distances(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, size_t n_pairs,
                       const uint32_t *pair_query, const uint32_t *pair_doc, float *out) {
    if (!ix || !q || !opts || !pair_query || !pair_doc || !out) return fail(AP_ERR_ARG, "null argument");
    AP_CUDA(cudaSetDevice(ix->device));
    uint32_t mqs = 0, mqb = 0;
    AP_TRY(host_query_limits(ix, q, 0, &mqs, &mqb));
    for (size_t i = 0; i < n_pairs; ++i)
        if (pair_query[i] >= q->nq || pair_doc[i] >= ix->n) return fail(AP_ERR_ARG, "pair %zu out of range", i);
    uint32_t path = 0, mode = 0;
    AP_TRY(dispatch_path(0, opts->sparse_weight, opts->bm25_weight, opts->dense_weight, 0.f, &path, &mode));
    const uint32_t nq = q->nq;
    SearchLaunch L{};
    void *p;
    auto upload = [&](int slot, const void *src, size_t bytes, const void **dst) -> int {
        AP_TRY(ws_reserve(ix, slot, bytes, &p));
        if (bytes) AP_CUDA(cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice));
        *dst = p;
        return AP_OK;
    };
    const uint32_t *dq, *dd;
    AP_TRY(upload(0, q->dense, (size_t)nq * kDim * 4, (const void **)&L.qdense));
    AP_TRY(upload(1, q->sparse.off, (size_t)(nq + 1) * 4, (const void **)&L.qs_off));
    AP_TRY(upload(2, q->sparse.idx, (size_t)q->sparse.off[nq] * 4, (const void **)&L.qs_idx));
    AP_TRY(upload(3, q->sparse.val, (size_t)q->sparse.off[nq] * 4, (const void **)&L.qs_val));
    AP_TRY(upload(4, q->bm25.off, (size_t)(nq + 1) * 4, (const void **)&L.qb_off));
    AP_TRY(upload(5, q->bm25.idx, (size_t)q->bm25.off[nq] * 4, (const void **)&L.qb_idx));
    AP_TRY(upload(6, q->bm25.val, (size_t)q->bm25.off[nq] * 4, (const void **)&L.qb_val));
    AP_TRY(upload(11, pair_query, n_pairs * 4, (const void **)&dq));
    AP_TRY(upload(12, pair_doc, n_pairs * 4, (const void **)&dd));
    AP_TRY(ws_reserve(ix, 13, n_pairs * 4, &p));
    float *dout = (float *)p;
    L.nq = nq; L.max_qs = mqs; L.max_qb = mqb;
    L.w_sparse = opts->sparse_weight; L.w_bm25 = opts->bm25_weight; L.w_dense = opts->dense_weight;
    L.cands = 32; L.flags = opts->flags & AP_SEARCH_UNFUSED_DENSE; L.path = path; L.stream = 0;
    AP_TRY(distances_launch(ix, L, n_pairs, dq, dd, dout));
    AP_CUDA(cudaMemcpy(out, dout, n_pairs * 4, cudaMemcpyDeviceToHost));
    return AP_OK;
}

// Test / profiling hook: the counters of the last search on this index: expansions, evaluations, gathered bytes, then
// clock cycles thread 0 of every CTA spent in: control (select, row staging, copy planning), waiting for copies,
// scoring, the 32-wide sort, the pool merge (summed over CTAs).
int ap_debug_counters(ap_index *ix, uint64_t *out8) {
    if (!ix || !out8) return fail(AP_ERR_ARG, "null argument");
    AP_CUDA(cudaSetDevice(ix->device));
    AP_CUDA(cudaMemcpy(out8, ix->d_cnt, 64, cudaMemcpyDeviceToHost));
    return AP_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Search from host buffers without any allocation.
//
// ap_search_host stages a batch's queries and results in grow-only device buffers that it cudaMalloc's on demand.
// Some callers must not allocate once they are serving: a process that has handed the whole GPU to another memory
// pool has nothing left for cudaMalloc to give, and cudaMalloc / cudaFree may synchronise the device, which a
// latency-bound query loop cannot afford.  For them the staging area below is part of the library image itself: a
// file-scope device array that every GPU loading the library holds until the process exits.
// ---------------------------------------------------------------------------------------------------------
namespace apoe {

constexpr size_t kStaticScratchBytes = AP_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, never an address a kernel could use: the device
// address is asked for once per device, with that device current, and cached.
constexpr int kMaxDevices = 64;
static unsigned char *g_static_ptr[kMaxDevices] = {nullptr};

static int static_scratch_address(int device, unsigned char **out) {
    if (device < 0 || device >= kMaxDevices) return fail(AP_ERR_ARG, "device %d out of range", device);
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!g_static_ptr[device]) {
        AP_CUDA(cudaSetDevice(device));
        void *p = nullptr;
        AP_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return fail(AP_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the static scratch");
        g_static_ptr[device] = static_cast<unsigned char *>(p);
    }
    *out = g_static_ptr[device];
    return AP_OK;
}

}  // namespace apoe

extern "C" int ap_search_host_static(ap_index *ix, const ap_queries *q, const ap_search_opts *opts, uint32_t *out_ids,
                                     float *out_dis, ap_search_stats *stats) {
    using namespace apoe;
    const auto t0 = std::chrono::high_resolution_clock::now();
    AP_TRY(check_search_args(ix, q, opts));
    if (!out_ids || !out_dis) return fail(AP_ERR_ARG, "null output pointer");
    AP_CUDA(cudaSetDevice(ix->device));
    float ws = opts->sparse_weight, wb = opts->bm25_weight, wd = opts->dense_weight;
    if (!(opts->flags & AP_SEARCH_RAW_WEIGHTS)) AP_TRY(effective_weights_host(ix, q, &ws, &wb, &wd));
    uint32_t path = 0, mode = 0;
    AP_TRY(dispatch_path(opts->flags, ws, wb, wd, opts->kg_weight, &path, &mode));
    if ((mode & AP_SEARCH_KG) && ix->n_ent == 0) return fail(AP_ERR_STATE, "kg_weight >= 1e-5 but no knowledge graph is loaded");
    uint32_t mqs = 0, mqb = 0;
    AP_TRY(host_query_limits(ix, q, mode, &mqs, &mqb));

    // carve the static array: control words and counters first, then the batch, every piece 256-byte aligned
    const uint32_t nq = q->nq, cands = opts->cands;
    const size_t nzs = q->sparse.off[nq], nzb = q->bm25.off[nq];
    const size_t nze = (mode & AP_SEARCH_KG) ? q->ent_off[nq] : 0;
    size_t need = 0;
    auto carve = [&](size_t bytes) { const size_t at = need; need = (need + bytes + 255) / 256 * 256; return at; };
    const size_t o_ctl = carve(64), o_cnt = carve(64);
    const size_t o_qd = carve((size_t)nq * kDim * 4), o_so = carve((size_t)(nq + 1) * 4), o_si = carve(nzs * 4), o_sv = carve(nzs * 4);
    const size_t o_bo = carve((size_t)(nq + 1) * 4), o_bi = carve(nzb * 4), o_bv = carve(nzb * 4);
    const size_t o_eo = carve((mode & AP_SEARCH_KG) ? (size_t)(nq + 1) * 4 : 0), o_ei = carve(nze * 4);
    const size_t o_ids = carve((size_t)nq * cands * 4), o_dis = carve((size_t)nq * cands * 4);
    if (need > kStaticScratchBytes)
        return fail(AP_ERR_LIMIT, "this batch needs %zu bytes of device staging, the static area holds %zu (%u queries, cands %u): "
                                  "send fewer queries per call or use ap_search_host", need, (size_t)kStaticScratchBytes, nq, cands);
    unsigned char *base = nullptr;
    AP_TRY(static_scratch_address(ix->device, &base));

    cudaStream_t st = 0;
    // the area keeps whatever the previous call left: next-query counter, error word and counters start at zero
    AP_CUDA(cudaMemsetAsync(base + o_ctl, 0, 64, st));
    AP_CUDA(cudaMemsetAsync(base + o_cnt, 0, 64, st));
    size_t h2d = 0;
    auto put = [&](size_t at, const void *src, size_t bytes) -> int {
        if (bytes) AP_CUDA(cudaMemcpyAsync(base + at, src, bytes, cudaMemcpyHostToDevice, st));
        h2d += bytes;
        return AP_OK;
    };
    AP_TRY(put(o_qd, q->dense, (size_t)nq * kDim * 4));
    AP_TRY(put(o_so, q->sparse.off, (size_t)(nq + 1) * 4)); AP_TRY(put(o_si, q->sparse.idx, nzs * 4)); AP_TRY(put(o_sv, q->sparse.val, nzs * 4));
    AP_TRY(put(o_bo, q->bm25.off, (size_t)(nq + 1) * 4)); AP_TRY(put(o_bi, q->bm25.idx, nzb * 4)); AP_TRY(put(o_bv, q->bm25.val, nzb * 4));
    if (mode & AP_SEARCH_KG) { AP_TRY(put(o_eo, q->ent_off, (size_t)(nq + 1) * 4)); AP_TRY(put(o_ei, q->ent_idx, nze * 4)); }

    SearchLaunch L{};
    L.qdense = reinterpret_cast<const float *>(base + o_qd);
    L.qs_off = reinterpret_cast<const uint32_t *>(base + o_so); L.qs_idx = reinterpret_cast<const uint32_t *>(base + o_si);
    L.qs_val = reinterpret_cast<const float *>(base + o_sv);
    L.qb_off = reinterpret_cast<const uint32_t *>(base + o_bo); L.qb_idx = reinterpret_cast<const uint32_t *>(base + o_bi);
    L.qb_val = reinterpret_cast<const float *>(base + o_bv);
    if (mode & AP_SEARCH_KG) { L.qe_off = reinterpret_cast<const uint32_t *>(base + o_eo); L.qe_idx = reinterpret_cast<const uint32_t *>(base + o_ei); }
    L.out_ids = reinterpret_cast<uint32_t *>(base + o_ids); L.out_dis = reinterpret_cast<float *>(base + o_dis);
    L.ctl = reinterpret_cast<uint32_t *>(base + o_ctl); L.cnt = reinterpret_cast<unsigned long long *>(base + o_cnt);
    L.nq = nq; L.max_qs = mqs; L.max_qb = mqb;
    L.w_sparse = ws; L.w_bm25 = wb; L.w_dense = wd; L.kg_weight = opts->kg_weight;
    L.cands = cands; L.flags = (opts->flags & ~(AP_SEARCH_KEYWORD | AP_SEARCH_KG)) | mode; L.path = path;
    L.arena_bytes = opts->arena_bytes; L.ctas_per_sm = opts->ctas_per_sm; L.stream = st;
    uint32_t launches = 0;
    AP_CUDA(cudaEventRecord(ix->ev0, st));
    AP_TRY(search_launch(ix, L, &launches));
    AP_CUDA(cudaEventRecord(ix->ev1, st));
    AP_CUDA(cudaMemcpyAsync(out_ids, L.out_ids, (size_t)nq * cands * 4, cudaMemcpyDeviceToHost, st));
    AP_CUDA(cudaMemcpyAsync(out_dis, L.out_dis, (size_t)nq * cands * 4, cudaMemcpyDeviceToHost, st));
    uint32_t ctl[2] = {0, 0};
    unsigned long long cnt[3] = {0, 0, 0};
    AP_CUDA(cudaMemcpyAsync(ctl, L.ctl, 8, cudaMemcpyDeviceToHost, st));
    AP_CUDA(cudaMemcpyAsync(cnt, L.cnt, 24, cudaMemcpyDeviceToHost, st));
    AP_CUDA(cudaStreamSynchronize(st));
    if (ctl[1] != 0) return fail(AP_ERR_DEVICE, "search kernel raised error word %u (a bounded wait ran out or a record exceeds the arena)", ctl[1]);
    if (stats) {
        float ms = 0.f;
        AP_CUDA(cudaEventElapsedTime(&ms, ix->ev0, ix->ev1));
        stats->kernel_ms = ms; stats->expansions = cnt[0]; stats->evaluations = cnt[1]; stats->gathered_bytes = cnt[2];
        stats->eff_sparse = ws; stats->eff_bm25 = wb; stats->eff_dense = wd; stats->path = path; stats->launches = launches;
        const size_t d2h = (size_t)nq * cands * 8;
        stats->h2d_bytes_lo = (uint32_t)h2d; stats->h2d_bytes_hi = (uint32_t)((uint64_t)h2d >> 32);
        stats->d2h_bytes_lo = (uint32_t)d2h; stats->d2h_bytes_hi = (uint32_t)((uint64_t)d2h >> 32);
        stats->total_ms = std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count();
    }
    return AP_OK;
}
