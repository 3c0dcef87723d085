// Entry points of the CUDA-core (exact fp32) trimul path; see trimul_simt.cu.
#pragma once
#include "common.cuh"

namespace tri {
namespace simt {
size_t saved_bytes(const TriMulDesc* d);
size_t ws_bytes(const TriMulDesc* d, int is_bwd);
int forward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out,
            void* saved, void* ws, size_t ws_size, cudaStream_t st);
int backward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, const void* saved,
             const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws, size_t ws_size, cudaStream_t st);
}  // namespace simt
}  // namespace tri
