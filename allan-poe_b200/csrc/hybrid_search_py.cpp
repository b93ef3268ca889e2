// Python module `hybrid_search`: the reference's two entry points with unchanged keyword names and order
// (ref: src/bindings.cpp:7-38), as a thin shim over the C ABI.  Failures raise RuntimeError instead of
// ending the interpreter.
#include <pybind11/pybind11.h>

#include <stdexcept>
#include <string>

#include "../../include/allan_poe.h"

namespace py = pybind11;

static void check(int rc) {
    if (rc != AP_OK) throw std::runtime_error(std::string("allan-poe: ") + ap_last_error());
}

static void build_index_impl(const std::string &dense_data_path, const std::string &sparse_data_path,
                             const std::string &bm25_data_path, const std::string &output_graph_path) {
    py::gil_scoped_release release;
    check(ap_build_index(dense_data_path.c_str(), sparse_data_path.c_str(), bm25_data_path.c_str(),
                         output_graph_path.c_str(), 0, nullptr, nullptr));
}

static void search_index_impl(const std::string &dense_data_path, const std::string &dense_query_path,
                              const std::string &sparse_data_path, const std::string &sparse_query_path,
                              const std::string &bm25_data_path, const std::string &bm25_query_path,
                              const std::string &keyword_id_path, const std::string &knowledge_path,
                              const std::string &entity2doc_path, const std::string &query_entity_path,
                              const std::string &graph_path, const std::string &ground_truth_path, int top_k, int cands,
                              float sparse_weight, float bm25_weight, float dense_weight, float kg_weight) {
    py::gil_scoped_release release;
    check(ap_search_index(dense_data_path.c_str(), dense_query_path.c_str(), sparse_data_path.c_str(),
                          sparse_query_path.c_str(), bm25_data_path.c_str(), bm25_query_path.c_str(),
                          keyword_id_path.c_str(), knowledge_path.c_str(), entity2doc_path.c_str(),
                          query_entity_path.c_str(), graph_path.c_str(), ground_truth_path.c_str(), top_k, cands,
                          sparse_weight, bm25_weight, dense_weight, kg_weight, 0, 0, nullptr, nullptr, nullptr, nullptr,
                          nullptr));
}

PYBIND11_MODULE(hybrid_search, m) {
    m.doc() = "Hybrid Search with Allan-Poe (B200-native)";
    m.def("build_index", &build_index_impl, "Build the hybrid index", py::arg("dense_data_path"),
          py::arg("sparse_data_path"), py::arg("bm25_data_path"), py::arg("output_graph_path"));
    m.def("search_index", &search_index_impl, "Search the hybrid index", py::arg("dense_data_path"),
          py::arg("dense_query_path"), py::arg("sparse_data_path"), py::arg("sparse_query_path"),
          py::arg("bm25_data_path"), py::arg("bm25_query_path"), py::arg("keyword_id_path"), py::arg("knowledge_path"),
          py::arg("entity2doc_path"), py::arg("query_entity_path"), py::arg("graph_path"), py::arg("ground_truth_path"),
          py::arg("top_k"), py::arg("cands"), py::arg("sparse_weight"), py::arg("bm25_weight"), py::arg("dense_weight"),
          py::arg("kg_weight"));
}
