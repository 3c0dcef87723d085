// LayerNorm fused into the projection GEMMs of the triangle multiplicative update (16-bit dtypes, 128 channels).
//
//   ln_gate_in   x -> z = LayerNorm(x) normalised in shared memory, then both halves of
//                a | b = (z Wp^T + bp) * sigmoid(z Wg^T + bg) * mask, channel-major; z and the row statistics are
//                written out for the output gate and the backward pass.
//   ln_gate_out  t (channel-major) -> u = LayerNorm over channels, normalised in shared memory in the layout the
//                contraction left it in (the MMA reads it as an MN-major operand, so nothing is transposed), then
//                out = (u Wo^T + bo) * sigmoid(z Wgo^T + bgo); u is kept channel-major for the backward pass.
#pragma once

#include "tc_common.cuh"

namespace tri {
namespace tc {

struct LnGateIn {
  int dtype;                 // TRI_BF16 / TRI_F16
  long long M, plane;        // pixels in all; pixels per batch entry (channel-plane stride of a / b)
  float eps;
  const void* x;             // [M, 128]
  const void* gamma;         // [128] or null
  const void* beta;          // [128] or null
  const void* wcat;          // [512, 128]: rows [Wp_a; Wg_a; Wp_b; Wg_b]
  const float* bias_cat;     // [512] in the same row order, or null
  const void* mask;          // [M] in the input dtype, or null
  void* z;                   // [M, 128]
  float* mean;               // [M]
  float* rstd;               // [M]
  void* a_cm;                // [B, 128, plane]
  void* b_cm;
  int* err;                  // device status word (zeroed by the caller)
};

bool ln_gate_in_supported(int dtype, long long M, long long plane);
int ln_gate_in(cudaStream_t st, const LnGateIn& p);

struct LnGateOut {
  int dtype;                 // TRI_BF16 / TRI_F16
  long long M;               // pixels (one batch entry: the channel planes of t are M pixels apart)
  float eps;
  const void* t_cm;          // [128, M]
  const void* z;             // [M, 128]
  const void* gamma;         // [128] or null
  const void* beta;          // [128] or null
  const void* w_out;         // [128, 128], rows = output channel
  const void* w_gate;        // [128, 128]
  const float* bias_out;     // [256]: output bias, gate bias; or null
  void* u_cm;                // [128, M] or null (inference: nothing to keep)
  float* mean;               // [M]
  float* rstd;               // [M]
  void* out;                 // [M, 128]
  int* err;
};

// One batch entry, 64-pixel groups aligned: M a multiple of 64.
bool ln_gate_out_supported(int dtype, long long M, long long plane);
int ln_gate_out(cudaStream_t st, const LnGateOut& p);

}  // namespace tc
}  // namespace tri
