// Entry points of the tensor-core (tcgen05 / TMEM / TMA) paths.
#pragma once
#include "common.cuh"

namespace tri {
namespace tc {
// True when the tensor-core kernels cover this problem (dtype, precision, shape, strides).
bool attn_fwd_supported(const TriAttnDesc* d);
bool attn_bwd_supported(const TriAttnDesc* d);
size_t attn_ws_bytes(const TriAttnDesc* d, int is_bwd);
int attn_forward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                 const uint8_t* mask, void* o, float* lse, void* ws, size_t ws_size, cudaStream_t st);
int attn_backward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                  const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                  void* dv, float* dbias, void* ws, size_t ws_size, cudaStream_t st);

bool mul_supported(const TriMulDesc* d);
size_t mul_saved_bytes(const TriMulDesc* d);
size_t mul_ws_bytes(const TriMulDesc* d, int is_bwd);
int mul_forward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out,
                void* saved, void* ws, size_t ws_size, cudaStream_t st);
int mul_backward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, const void* saved,
                 const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws, size_t ws_size, cudaStream_t st);
// Row-sharded trimul: the pixel-wise phases on their own (see tri_mul_shard_phase in the C header).
bool mul_shard_supported(const TriMulShardDesc* d);
size_t mul_shard_saved_bytes(const TriMulShardDesc* d);
size_t mul_shard_ws_bytes(const TriMulShardDesc* d, int phase);
size_t mul_shard_prep_bytes(const TriMulShardDesc* d);
int mul_shard_phase(const TriMulShardDesc* d, int phase, const TriMulShardBufs* bufs, void* ws, size_t ws_size,
                    cudaStream_t st);
// Fused LayerNorm + q / k / v / pair-bias projection feeding triangle attention (see tri_attn_project in the C header).
bool attn_project_supported(const TriAttnProjDesc* d);
size_t attn_project_ws_bytes(const TriAttnProjDesc* d);
int attn_project(const TriAttnProjDesc* d, const void* z, const void* ln_w, const void* ln_b, const void* w_qkv,
                 const void* w_bias, void* qkv, void* bias, void* ws, size_t ws_size, cudaStream_t st);
}  // namespace tc
}  // namespace tri
