// TEST / BASELINE INFRASTRUCTURE ONLY.
//
// Drives the reference's own index-construction kernels, compiled unmodified from the reference tree
// (`#include "index.cu"`, found through -I<reference>/src), so that their intermediate state can be read back:
// the k-NN lists after merge_reverse_plus, the forward / keyword-edge lists after allan_poe and the final rows.
// The launch sequence below is the one of build_index_impl (src/index.cu:842-903).  Two things differ from it,
// both outside the kernels: reverse_graph_dev is zeroed before use (the reference reads it uninitialised in
// round 0, src/index.cu:188,845-846) and the Keyword_edge counters are cleared so that more than one build can run
// in a process (src/index.cu:536).  Nothing from the reference is copied into this repository; the shared
// library built from this file lives under oracle/_ref/ only.
#include "index.cu"

extern "C" int ref_build(unsigned points_num, const float *dense_unscaled, const unsigned *sparse_off, const unsigned *sparse_idx,
                         const float *sparse_val, const unsigned *bm25_off, const unsigned *bm25_idx, const float *bm25_val,
                         unsigned *knn_out, float *knn_dis_out, float *power_out, unsigned *new_list_out, unsigned *kw_out,
                         unsigned *graph_out, unsigned *ep_out, double *seconds) {
    if (points_num > POINTS || points_num < 64) return 1;
    const unsigned dim = DIM, non_zero_num = sparse_off[points_num], bm25_non_zero = bm25_off[points_num];
    std::vector<float> data_load((size_t)points_num * dim);
    for (size_t i = 0; i < (size_t)points_num * dim; i++) data_load[i] = dense_unscaled[i] * 7;  // src/index.cu:836-840

    unsigned *graph_dev, *reverse_graph_dev, *sparse_off_dev, *sparse_idx_dev, *bm25_off_dev, *bm25_idx_dev;
    float *data_dev, *sparse_val_dev, *bm25_val_dev, *data_power_dev;
    half *data_half_dev;
    cudaMalloc((void **)&graph_dev, (size_t)points_num * K * sizeof(unsigned));
    cudaMalloc((void **)&reverse_graph_dev, (size_t)points_num * K * sizeof(unsigned));
    cudaMemset(reverse_graph_dev, 0, (size_t)points_num * K * sizeof(unsigned));
    cudaMalloc((void **)&data_dev, (size_t)points_num * dim * sizeof(float));
    cudaMemcpy(data_dev, data_load.data(), (size_t)points_num * dim * sizeof(float), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&data_half_dev, (size_t)points_num * dim * sizeof(half));
    cudaMalloc((void **)&sparse_off_dev, (points_num + 1) * sizeof(unsigned));
    cudaMemcpy(sparse_off_dev, sparse_off, (points_num + 1) * sizeof(unsigned), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&sparse_idx_dev, (size_t)non_zero_num * sizeof(unsigned));
    cudaMemcpy(sparse_idx_dev, sparse_idx, (size_t)non_zero_num * sizeof(unsigned), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&sparse_val_dev, (size_t)non_zero_num * sizeof(float));
    cudaMemcpy(sparse_val_dev, sparse_val, (size_t)non_zero_num * sizeof(float), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&bm25_off_dev, (points_num + 1) * sizeof(unsigned));
    cudaMemcpy(bm25_off_dev, bm25_off, (points_num + 1) * sizeof(unsigned), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&bm25_idx_dev, (size_t)bm25_non_zero * sizeof(unsigned));
    cudaMemcpy(bm25_idx_dev, bm25_idx, (size_t)bm25_non_zero * sizeof(unsigned), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&bm25_val_dev, (size_t)bm25_non_zero * sizeof(float));
    cudaMemcpy(bm25_val_dev, bm25_val, (size_t)bm25_non_zero * sizeof(float), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&data_power_dev, points_num * sizeof(float));
    cudaMemset(data_power_dev, 0, points_num * sizeof(float));
    {
        void *ke = nullptr, *rn = nullptr;
        cudaGetSymbolAddress(&ke, Keyword_edge);
        cudaMemset(ke, 0, sizeof(unsigned) * (size_t)POINTS * (KEYEDGE + 1));
        cudaGetSymbolAddress(&rn, reverse_num);
        cudaMemset(rn, 0, sizeof(unsigned) * (size_t)POINTS);
    }
    if (cudaGetLastError() != cudaSuccess) return 2;

    dim3 grid(points_num, 1, 1), block(32, MAX_P / 32, 1), block3(32, 3, 1), grid_s(points_num, 1, 1), block_s(32, 3, 1),
        block_m(32, 16, 1);
    const unsigned all_it = 25, degree = 32;
    cudaDeviceSynchronize();
    auto start = std::chrono::high_resolution_clock::now();
    initialize_graph<<<points_num, 32>>>(graph_dev, points_num, data_dev);
    f2h<<<points_num, 256>>>(data_dev, data_half_dev, points_num);
    cal_power<<<points_num, 32>>>(data_half_dev, data_power_dev, dim, sparse_off_dev, sparse_idx_dev, sparse_val_dev, bm25_off_dev,
                                  bm25_idx_dev, bm25_val_dev, points_num);
    for (unsigned it = 0; it < all_it; it++) {
        nn_descent_gpu<<<grid, block>>>(graph_dev, reverse_graph_dev, it, data_half_dev, points_num, all_it, sparse_off_dev,
                                        sparse_idx_dev, sparse_val_dev, bm25_off_dev, bm25_idx_dev, bm25_val_dev, data_power_dev);
        if (it < all_it - 1) reset_reverse_num<<<1000, 1024>>>(points_num);
    }
    merge_reverse_plus<<<grid, block3>>>(graph_dev, reverse_graph_dev);
    reset_reverse_num<<<1000, 1024>>>(points_num);
    // read-back point 1 (not part of the reference's timed region; the clock is stopped around it)
    cudaDeviceSynchronize();
    auto mid0 = std::chrono::high_resolution_clock::now();
    if (knn_out) cudaMemcpy(knn_out, graph_dev, (size_t)points_num * K * sizeof(unsigned), cudaMemcpyDeviceToHost);
    if (knn_dis_out) cudaMemcpyFromSymbol(knn_dis_out, nei_distance, (size_t)points_num * K * sizeof(float));
    if (power_out) cudaMemcpy(power_out, data_power_dev, points_num * sizeof(float), cudaMemcpyDeviceToHost);
    auto mid1 = std::chrono::high_resolution_clock::now();
    allan_poe<<<grid_s, block_m>>>(graph_dev, degree, reverse_graph_dev, data_half_dev, data_power_dev, sparse_off_dev, sparse_idx_dev,
                                   sparse_val_dev, bm25_off_dev, bm25_idx_dev, bm25_val_dev);
    cudaDeviceSynchronize();
    auto mid2 = std::chrono::high_resolution_clock::now();
    if (new_list_out) {  // new_list rows are K = 64 wide, the first 32 entries are the forward list
        std::vector<unsigned> tmp((size_t)points_num * K);
        cudaMemcpyFromSymbol(tmp.data(), new_list, (size_t)points_num * K * sizeof(unsigned));
        for (size_t i = 0; i < points_num; i++) memcpy(new_list_out + i * 32, tmp.data() + i * K, 32 * sizeof(unsigned));
    }
    if (kw_out) cudaMemcpyFromSymbol(kw_out, Keyword_edge, (size_t)points_num * (KEYEDGE + 1) * sizeof(unsigned));
    auto mid3 = std::chrono::high_resolution_clock::now();
    allan_poe_final_graph<<<grid_s, block_s>>>(graph_dev, reverse_graph_dev, degree, degree + KEYEDGEFINAL);
    cudaDeviceSynchronize();
    auto end = std::chrono::high_resolution_clock::now();
    const cudaError_t err = cudaGetLastError();
    if (seconds)
        *seconds = std::chrono::duration<double>(end - start).count() - std::chrono::duration<double>(mid1 - mid0).count() -
                   std::chrono::duration<double>(mid3 - mid2).count();
    if (graph_out) cudaMemcpy(graph_out, graph_dev, (size_t)points_num * (degree + KEYEDGEFINAL) * sizeof(unsigned), cudaMemcpyDeviceToHost);
    if (ep_out) {  // src/index.cu:916-925
        std::vector<float> data_p(points_num);
        cudaMemcpy(data_p.data(), data_power_dev, points_num * sizeof(float), cudaMemcpyDeviceToHost);
        std::vector<std::pair<float, unsigned>> dp;
        for (unsigned i = 0; i < points_num; i++) dp.push_back(std::pair<float, unsigned>(data_p[i], i));
        std::sort(dp.begin(), dp.end());
        for (unsigned i = 0; i < degree; i++) ep_out[i] = dp[i].second;
    }
    cudaFree(graph_dev); cudaFree(reverse_graph_dev); cudaFree(data_dev); cudaFree(data_half_dev); cudaFree(sparse_off_dev);
    cudaFree(sparse_idx_dev); cudaFree(sparse_val_dev); cudaFree(bm25_off_dev); cudaFree(bm25_idx_dev); cudaFree(bm25_val_dev);
    cudaFree(data_power_dev);
    return err == cudaSuccess ? 0 : 3;
}

// The reference's corpus loaders (include/utils.cuh:361-398) followed by the uploads build_index_impl makes
// (src/index.cu:845-887), timed: seconds[0] = the three loads, seconds[1] = loads + uploads.
extern "C" int ref_load(const char *dense_path, const char *sparse_path, const char *bm25_path, unsigned *rows_out, double *seconds) {
    auto t0 = std::chrono::high_resolution_clock::now();
    float *data = nullptr, *sparse_val = nullptr, *bm25_val = nullptr;
    unsigned *sparse_off = nullptr, *sparse_idx = nullptr, *bm25_off = nullptr, *bm25_idx = nullptr;
    unsigned num = 0, dim = 0, nnz_s = 0, nnz_b = 0;
    load_data(const_cast<char *>(dense_path), data, num, dim);
    load_sparse_data(const_cast<char *>(sparse_path), sparse_off, sparse_idx, sparse_val, num + 1, nnz_s);
    load_sparse_data(const_cast<char *>(bm25_path), bm25_off, bm25_idx, bm25_val, num + 1, nnz_b);
    auto t1 = std::chrono::high_resolution_clock::now();
    float *data_dev, *sv_dev, *bv_dev;
    unsigned *so_dev, *si_dev, *bo_dev, *bi_dev;
    cudaMalloc((void **)&data_dev, (size_t)num * dim * sizeof(float));
    cudaMemcpy(data_dev, data, (size_t)num * dim * sizeof(float), cudaMemcpyHostToDevice);
    cudaMalloc((void **)&so_dev, (size_t)(num + 1) * 4); cudaMemcpy(so_dev, sparse_off, (size_t)(num + 1) * 4, cudaMemcpyHostToDevice);
    cudaMalloc((void **)&si_dev, (size_t)nnz_s * 4); cudaMemcpy(si_dev, sparse_idx, (size_t)nnz_s * 4, cudaMemcpyHostToDevice);
    cudaMalloc((void **)&sv_dev, (size_t)nnz_s * 4); cudaMemcpy(sv_dev, sparse_val, (size_t)nnz_s * 4, cudaMemcpyHostToDevice);
    cudaMalloc((void **)&bo_dev, (size_t)(num + 1) * 4); cudaMemcpy(bo_dev, bm25_off, (size_t)(num + 1) * 4, cudaMemcpyHostToDevice);
    cudaMalloc((void **)&bi_dev, (size_t)nnz_b * 4); cudaMemcpy(bi_dev, bm25_idx, (size_t)nnz_b * 4, cudaMemcpyHostToDevice);
    cudaMalloc((void **)&bv_dev, (size_t)nnz_b * 4); cudaMemcpy(bv_dev, bm25_val, (size_t)nnz_b * 4, cudaMemcpyHostToDevice);
    cudaDeviceSynchronize();
    auto t2 = std::chrono::high_resolution_clock::now();
    const cudaError_t err = cudaGetLastError();
    cudaFree(data_dev); cudaFree(so_dev); cudaFree(si_dev); cudaFree(sv_dev); cudaFree(bo_dev); cudaFree(bi_dev); cudaFree(bv_dev);
    delete[] data; delete[] sparse_off; delete[] sparse_idx; delete[] sparse_val; delete[] bm25_off; delete[] bm25_idx; delete[] bm25_val;
    if (rows_out) *rows_out = num;
    if (seconds) { seconds[0] = std::chrono::duration<double>(t1 - t0).count(); seconds[1] = std::chrono::duration<double>(t2 - t0).count(); }
    return err == cudaSuccess ? 0 : 3;
}
