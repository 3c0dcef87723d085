// Entry points of the CUDA-core (exact fp32) triangle-attention path; see attn_simt.cu.
#pragma once
#include "common.cuh"

namespace tri {
namespace simt {
size_t attn_ws_bytes(const TriAttnDesc* d, int is_bwd);
int attn_forward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                 const uint8_t* mask, void* o, float* lse, cudaStream_t st);
int attn_backward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                  const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                  void* dv, float* dbias, void* ws, size_t ws_size, cudaStream_t st);
// Backward whose scratch is a built-in device array (no workspace argument); see attn_simt.cu.
size_t attn_static_scratch_rows();
int attn_backward_static(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                         const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                         void* dv, float* dbias, cudaStream_t st);
}  // namespace simt
}  // namespace tri
