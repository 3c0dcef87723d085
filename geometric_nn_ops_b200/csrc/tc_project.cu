// Fused attention-input projection for the pair stack: LayerNorm(z) and the q / k / v / pair-bias projections in two
// launches, written in the layouts the triangle-attention kernels read.
//
//   ln_bias_kernel   z [M, 128] -> zn = LayerNorm(z) [M, 128] (input dtype), and the pair bias
//                    bias[h][m] = sum_c zn[m][c] Wb[h][c] for h < H, computed from the fp32 row while it is in
//                    registers (H <= 8 dot products per pixel are not worth a GEMM) and stored head-major, which is
//                    the [B, 1, H, N, N] layout the attention takes.
//   tc_gemm          qkv[m][0:384] = zn[m][:] Wqkv^T on tcgen05 (M = pixels, N = 3 * H * D = 384, K = 128): one
//                    [M, 384] buffer whose three 128-column groups are q, k and v with a row stride of 384 elements;
//                    the attention kernels take strides, so no copy follows.
// The reference has no such op (its attention takes pre-projected tensors,
// geometric_nn_ops_torch/triangle/_triattn.py:36-44); eager torch does the same work in a LayerNorm, four linears and
// a permute, about 10 pair-sized tensors of HBM traffic against 6 here.
#include "tc_gemm.cuh"
#include "tc_paths.cuh"

namespace tri {
namespace tc {

namespace {

constexpr int CW = 128;
constexpr int kMaxHeads = 8;
constexpr int kRowPairs = 4;   // row pairs per warp and pass

template <typename T> __device__ __forceinline__ void ld8(const T* p, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    union { uint4 u; T h[8]; } pk;
    pk.u = *reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = to_f32(pk.h[e]);
  }
}
template <typename T> __device__ __forceinline__ void st8(T* p, const float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    union { uint4 u; T h[8]; } pk;
#pragma unroll
    for (int e = 0; e < 8; ++e) pk.h[e] = from_f32<T>(v[e]);
    *reinterpret_cast<uint4*>(p) = pk.u;
  }
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// A row of 128 channels is held by 16 lanes (8 channels each), two rows per warp access, kRowPairs pairs in flight.
// H4 = true is the common four-head case: the lane's 32 bias weights live in registers and the four dot products are
// reduced over the 16 lanes with a halving butterfly (each step keeps half of the values and adds the partner's),
// 5 shuffles per row instead of 16.
template <typename T, bool H4>
__global__ void __launch_bounds__(256) ln_bias_kernel(const T* __restrict__ z, const T* gamma, const T* beta, float eps,
                                                       long long M, const T* __restrict__ wb, int H, T* __restrict__ zn,
                                                       T* __restrict__ bias) {
  __shared__ float sWb[H4 ? 1 : kMaxHeads][CW];
  const int lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
  float wr[4][8];
  if constexpr (H4) {
#pragma unroll
    for (int h = 0; h < 4; ++h) ld8(wb + h * CW + sub * 8, wr[h]);
  } else {
    for (int i = threadIdx.x; i < H * CW; i += 256) sWb[i / CW][i % CW] = to_f32(wb[i]);
    __syncthreads();
  }
  const long long row0 = (blockIdx.x * 8LL + (threadIdx.x >> 5)) * (2 * kRowPairs) + half;
  float gm[8], bt[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { gm[i] = 1.f; bt[i] = 0.f; }
  if (gamma) ld8(gamma + sub * 8, gm);
  if (beta) ld8(beta + sub * 8, bt);
  float v[kRowPairs][8];
#pragma unroll
  for (int p = 0; p < kRowPairs; ++p) {
    const long long row = row0 + 2 * p;
    if (row < M) ld8(z + row * CW + sub * 8, v[p]);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[p][i] = 0.f;
    }
  }
#pragma unroll
  for (int p = 0; p < kRowPairs; ++p) {
    const long long row = row0 + 2 * p;
    float sm = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sm += v[p][i];
    const float mu = half_warp_sum(sm) * (1.0f / CW);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[p][i] -= mu; q += v[p][i] * v[p][i]; }
    const float rs = 1.0f / sqrtf(half_warp_sum(q) * (1.0f / CW) + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[p][i] = v[p][i] * rs * gm[i] + bt[i];
    if (row < M) st8(zn + row * CW + sub * 8, v[p]);
    // the bias is projected from the values the GEMM will see: zn rounded to the storage dtype
#pragma unroll
    for (int i = 0; i < 8; ++i) v[p][i] = to_f32(from_f32<T>(v[p][i]));
    if constexpr (H4) {
      float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) d[h] += v[p][i] * wr[h][i];
      // lanes with bit 3 clear keep heads 0, 1 and those with it set heads 2, 3; then bit 2 picks one of the two
      const bool hi8 = (sub & 8) != 0, hi4 = (sub & 4) != 0;
      const float a = (hi8 ? d[2] : d[0]) + __shfl_xor_sync(0xffffffffu, hi8 ? d[0] : d[2], 8);
      const float b = (hi8 ? d[3] : d[1]) + __shfl_xor_sync(0xffffffffu, hi8 ? d[1] : d[3], 8);
      float c = (hi4 ? b : a) + __shfl_xor_sync(0xffffffffu, hi4 ? a : b, 4);
      c += __shfl_xor_sync(0xffffffffu, c, 2);
      c += __shfl_xor_sync(0xffffffffu, c, 1);
      const int h = (hi8 ? 2 : 0) + (hi4 ? 1 : 0);
      if ((sub & 3) == 0 && row < M) bias[(long long)h * M + row] = from_f32<T>(c);
    } else {
      for (int h = 0; h < H; ++h) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d += v[p][i] * sWb[h][sub * 8 + i];
        d = half_warp_sum(d);
        if (sub == 0 && row < M) bias[(long long)h * M + row] = from_f32<T>(d);
      }
    }
  }
}

template <typename T>
int project_t(const TriAttnProjDesc* d, const void* z, const void* ln_w, const void* ln_b, const void* w_qkv,
              const void* w_bias, void* qkv, void* bias, void* ws, cudaStream_t st) {
  const long long M = d->M;
  int* err = static_cast<int*>(ws);
  void* zn = static_cast<char*>(ws) + 256;
  TRI_CUDA_OK(cudaMemsetAsync(ws, 0, 256, st));
  const double unit = (double)M * CW * sizeof(T);
  {
    KernelTimer kt("tc_ln_bias", st, 2.0 * M * CW * d->H, 2.0 * unit);
    auto kern = d->H == 4 ? ln_bias_kernel<T, true> : ln_bias_kernel<T, false>;
    kern<<<cdiv(M, 8 * 2 * kRowPairs), 256, 0, st>>>((const T*)z, (const T*)ln_w, (const T*)ln_b, d->eps, M, (const T*)w_bias,
                                                      d->H, (T*)zn, (T*)bias);
    TRI_LAUNCH_OK();
  }
  const int n_out = 3 * d->H * d->D;
  GemmPlan p;
  p.a[0].ptr = zn; p.a[0].mn_major = false; p.a[0].inner = CW; p.a[0].outer = M; p.a[0].batch = 1; p.a[0].st_outer = CW;
  p.b[0].ptr = w_qkv; p.b[0].mn_major = false; p.b[0].inner = CW; p.b[0].outer = n_out; p.b[0].batch = 1; p.b[0].st_outer = CW;
  p.M = (int)M; p.N = n_out; p.K0 = CW; p.out0 = qkv; p.ld_out = n_out;
  p.name = "tc_gemm_qkv"; p.flops = 2.0 * M * CW * n_out; p.bytes = unit * (1.0 + n_out / (double)CW);
  return launch_gemm(st, d->dtype, EPI_STORE, 128, false, p, err);
}

}  // namespace

bool attn_project_supported(const TriAttnProjDesc* d) {
  if (d->C != CW || d->H < 1 || d->H > kMaxHeads || d->D < 8 || (d->H * d->D) % 8 != 0) return false;
  if (d->dtype == TRI_F32 && d->precision != TRI_PREC_TF32) return false;   // exact fp32 has no tensor-core form
  return d->M > 0 && d->M <= 2147483647LL;
}

size_t attn_project_ws_bytes(const TriAttnProjDesc* d) {
  return 256 + align_up((size_t)d->M * CW * (d->dtype == TRI_F32 ? 4 : 2));
}

int attn_project(const TriAttnProjDesc* d, const void* z, const void* ln_w, const void* ln_b, const void* w_qkv,
                 const void* w_bias, void* qkv, void* bias, void* ws, size_t ws_size, cudaStream_t st) {
  if (ws_size < attn_project_ws_bytes(d)) return fail(TRI_ERR_WORKSPACE, "projection workspace too small");
  switch (d->dtype) {
    case TRI_F32: return project_t<float>(d, z, ln_w, ln_b, w_qkv, w_bias, qkv, bias, ws, st);
    case TRI_BF16: return project_t<__nv_bfloat16>(d, z, ln_w, ln_b, w_qkv, w_bias, qkv, bias, ws, st);
    case TRI_F16: return project_t<__half>(d, z, ln_w, ln_b, w_qkv, w_bias, qkv, bias, ws, st);
  }
  return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
}

}  // namespace tc
}  // namespace tri
