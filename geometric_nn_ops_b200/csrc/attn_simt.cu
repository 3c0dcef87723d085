// Exact-fp32 (CUDA-core) path of triangle attention, forward and backward.
//
// Flash-style: 64 queries x 64 keys per tile, online softmax over the key axis,
// additive pair bias and key mask fused in, fp32 everywhere.  Serves fp32 inputs
// with matmul precision "ieee", and every shape the tensor-core path does not
// cover.  With precision tf32 the operands of each product are rounded to tf32.
//
// Math follows triangle_attention_torch
// (geometric_nn_ops_torch/triangle/_reference/triangle_attention.py:28-44):
//   logits = (q*scale).k + bias + mask_bias,  mask_bias = 1e9*(mask-1)
// added in that order in fp32, so a fully masked row degenerates to a uniform
// softmax exactly as the reference's does (_masking.py:13-42).
// The backward recomputes P from the saved log-sum-exp; dbias is reduced over the
// row axis inside one kernel, in a fixed order (no atomics, deterministic).
#include <algorithm>
#include <mutex>

#include "attn_simt.cuh"
#include "common.cuh"

namespace tri {
namespace simt {

namespace {

constexpr int TQ = 64, TK = 64;

__device__ __forceinline__ long long off4(const int64_t* st, int b, int s, int i, int h) {
  return b * st[0] + s * st[1] + i * st[2] + h * st[3];
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Load a [64, D] tile (rows i0..i0+63 of one (b, s, h) slice) into smem as fp32, zero padded.
template <typename T, bool TF32>
__device__ __forceinline__ void load_tile(float* dst, int DP, const T* base, const int64_t* st, int b, int s,
                                          int h, int i0, int n, int D, float mul) {
  const int tid = threadIdx.y * 16 + threadIdx.x;
  for (int idx = tid; idx < 64 * D; idx += 256) {
    int i = idx / D, dd = idx - i * D;
    float v = 0.f;
    if (i0 + i < n) v = to_f32(base[off4(st, b, s, i0 + i, h) + dd]) * mul;
    dst[i * DP + dd] = TF32 ? round_tf32(v) : v;
  }
}

// The reference's torch path accumulates in fp32 for every 16/32-bit dtype and takes the sentinel of
// that accumulate dtype (triangle_attention.py:28,40 of its _reference package): 1e9.
constexpr float kMaskSentinel = 1e9f;

template <typename T>
__device__ __forceinline__ void add_bias_mask(const TriAttnDesc& d, const T* bias, const uint8_t* mask, int b, int s,
                                              int h, int q0, int k0, float sc[4][4]) {
  const int tx = threadIdx.x, ty = threadIdx.y;
  const float sentinel = kMaskSentinel;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int qi = q0 + ty + 16 * r;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int kj = k0 + tx + 16 * c;
      float v = sc[r][c];
      if (kj >= d.n_res) { sc[r][c] = -INFINITY; continue; }
      if (bias != nullptr && qi < d.n_res)
        v += to_f32(bias[b * d.bias_st[0] + h * d.bias_st[1] + qi * d.bias_st[2] + kj]);
      if (mask != nullptr) {
        // 1e9 * (float(mask) - 1): +0.0 when kept, -1e9 when masked
        float mb = sentinel * ((mask[b * d.mask_st[0] + s * d.mask_st[1] + kj] ? 1.0f : 0.0f) - 1.0f);
        v += mb;
      }
      sc[r][c] = v;
    }
  }
}

template <int DC>
__device__ __forceinline__ void qk_dot(const float* Qs, const float* Ks, int DP, int D, float sc[4][4]) {
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) sc[r][c] = 0.f;
  for (int dd = 0; dd < D; ++dd) {
    float a[4], bb[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) a[r] = Qs[(ty + 16 * r) * DP + dd];
#pragma unroll
    for (int c = 0; c < 4; ++c) bb[c] = Ks[(tx + 16 * c) * DP + dd];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[r][c] = fmaf(a[r], bb[c], sc[r][c]);
  }
}

// acc[r][c] += sum_j L[(ty+16r)][j] * R[j][(tx+16c)]   with L [64][65], R [64][DP]
template <int DC>
__device__ __forceinline__ void rows_times_tile(const float* L, const float* R, int DP, float acc[4][DC]) {
  const int tx = threadIdx.x, ty = threadIdx.y;
  for (int j = 0; j < 64; ++j) {
    float l[4], rr[DC];
#pragma unroll
    for (int r = 0; r < 4; ++r) l[r] = L[(ty + 16 * r) * 65 + j];
#pragma unroll
    for (int c = 0; c < DC; ++c) rr[c] = R[j * DP + tx + 16 * c];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[r][c] = fmaf(l[r], rr[c], acc[r][c]);
  }
}

// acc[r][c] += sum_i L[i][(ty+16r)] * R[i][(tx+16c)]   (L transposed: reduce over the tile's rows)
template <int DC>
__device__ __forceinline__ void cols_times_tile(const float* L, const float* R, int DP, float acc[4][DC]) {
  const int tx = threadIdx.x, ty = threadIdx.y;
  for (int i = 0; i < 64; ++i) {
    float l[4], rr[DC];
#pragma unroll
    for (int r = 0; r < 4; ++r) l[r] = L[i * 65 + ty + 16 * r];
#pragma unroll
    for (int c = 0; c < DC; ++c) rr[c] = R[i * DP + tx + 16 * c];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[r][c] = fmaf(l[r], rr[c], acc[r][c]);
  }
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T, int DC, bool TF32>
__global__ void __launch_bounds__(256) attn_fwd_kernel(TriAttnDesc d, const T* q, const T* k, const T* v,
                                                        const T* bias, const uint8_t* mask, T* o, float* lse) {
  extern __shared__ float sm[];
  const int D = d.D, DP = 16 * DC + 1;
  float* Qs = sm;
  float* Ks = Qs + 64 * DP;
  float* Vs = Ks + 64 * DP;
  float* Ps = Vs + 64 * DP;  // [64][65]
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int q0 = blockIdx.x * TQ;
  int z = blockIdx.y;
  const int h = z % d.H; z /= d.H;
  const int s = z % d.n_seq;
  const int b = z / d.n_seq;
  // zero the padding columns once so D < 16*DC reads zeros
  for (int idx = ty * 16 + tx; idx < 3 * 64 * DP; idx += 256) sm[idx] = 0.f;
  __syncthreads();
  load_tile<T, TF32>(Qs, DP, q, d.q_st, b, s, h, q0, d.n_res, D, d.scale);
  float m[4], l[4], acc[4][DC];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[r][c] = 0.f;
  }
  for (int k0 = 0; k0 < d.n_res; k0 += TK) {
    load_tile<T, TF32>(Ks, DP, k, d.k_st, b, s, h, k0, d.n_res, D, 1.0f);
    load_tile<T, TF32>(Vs, DP, v, d.v_st, b, s, h, k0, d.n_res, D, 1.0f);
    __syncthreads();
    float sc[4][4];
    qk_dot<DC>(Qs, Ks, DP, D, sc);
    add_bias_mask<T>(d, bias, mask, b, s, h, q0, k0, sc);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float mx = fmaxf(fmaxf(sc[r][0], sc[r][1]), fmaxf(sc[r][2], sc[r][3]));
      mx = half_warp_max(mx);
      const float mn = fmaxf(m[r], mx);
      const float alpha = expf(m[r] - mn);
      float ps = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float p = expf(sc[r][c] - mn);
        ps += p;
        Ps[(ty + 16 * r) * 65 + tx + 16 * c] = TF32 ? round_tf32(p) : p;
      }
      ps = half_warp_sum(ps);
      l[r] = l[r] * alpha + ps;
      m[r] = mn;
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[r][c] *= alpha;
    }
    __syncthreads();
    rows_times_tile<DC>(Ps, Vs, DP, acc);
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int qi = q0 + ty + 16 * r;
    if (qi >= d.n_res) continue;
    const float inv = 1.0f / l[r];
    T* orow = o + off4(d.o_st, b, s, qi, h);
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      int dd = tx + 16 * c;
      if (dd < D) orow[dd] = from_f32<T>(acc[r][c] * inv);
    }
    if (tx == 0) {
      const long long row = (((long long)b * d.n_seq + s) * d.H + h) * d.n_res + qi;
      lse[row] = m[r];
      lse[(long long)d.B * d.n_seq * d.H * d.n_res + row] = logf(l[r]);
    }
  }
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
// delta[b,s,h,i] = sum_d dO * O
template <typename T>
__global__ void attn_delta_kernel(TriAttnDesc d, const T* o, const T* d_o, float* delta) {
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long total = (long long)d.B * d.n_seq * d.H * d.n_res;
  if (idx >= total) return;
  int i = idx % d.n_res; long long z = idx / d.n_res;
  int h = z % d.H; z /= d.H;
  int s = z % d.n_seq; int b = z / d.n_seq;
  const T* orow = o + off4(d.o_st, b, s, i, h);
  const T* grow = d_o + off4(d.do_st, b, s, i, h);
  float acc = 0.f;
  for (int dd = 0; dd < d.D; ++dd) acc = fmaf(to_f32(orow[dd]), to_f32(grow[dd]), acc);
  delta[idx] = acc;
}

// P and dS for this thread's 4x4 patch.  Qs is pre-scaled, dOs/Vs give dP.
template <typename T, int DC>
__device__ __forceinline__ void p_and_ds(const TriAttnDesc& d, const float* Qs, const float* Ks, const float* Vs,
                                         const float* dOs, int DP, const T* bias, const uint8_t* mask,
                                         const float* lse_s, const float* delta_s, int b, int s, int h, int q0, int k0,
                                         float p[4][4], float ds[4][4]) {
  const int tx = threadIdx.x, ty = threadIdx.y;
  float sc[4][4], dp[4][4];
  qk_dot<DC>(Qs, Ks, DP, d.D, sc);
  add_bias_mask<T>(d, bias, mask, b, s, h, q0, k0, sc);
  qk_dot<DC>(dOs, Vs, DP, d.D, dp);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int ql = ty + 16 * r;
    const bool q_ok = q0 + ql < d.n_res;
    // P = exp((S - m) - log l): the two statistics stay separate because m + log l would round
    // log l away when m is the -1e9 of a fully masked row.
    const float ls = lse_s[ql], ll = lse_s[128 + ql], dl = delta_s[ql];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const bool ok = q_ok && (k0 + tx + 16 * c < d.n_res);
      float pv = ok ? expf((sc[r][c] - ls) - ll) : 0.f;
      p[r][c] = pv;
      ds[r][c] = ok ? pv * (dp[r][c] - dl) : 0.f;
    }
  }
}

__device__ __forceinline__ void load_row_stats(const TriAttnDesc& d, const float* lse, const float* delta, int b, int s,
                                               int h, int q0, float* lse_s, float* delta_s) {
  const int tid = threadIdx.y * 16 + threadIdx.x;
  if (tid < 64) {
    int qi = q0 + tid;
    long long o = (((long long)b * d.n_seq + s) * d.H + h) * d.n_res + qi;
    lse_s[tid] = qi < d.n_res ? lse[o] : 0.f;
    lse_s[128 + tid] = qi < d.n_res ? lse[(long long)d.B * d.n_seq * d.H * d.n_res + o] : 0.f;
    delta_s[tid] = qi < d.n_res ? delta[o] : 0.f;
  }
}

template <typename T, int DC, bool TF32>
__global__ void __launch_bounds__(256) attn_bwd_dkdv_kernel(TriAttnDesc d, const T* q, const T* k, const T* v,
                                                             const T* bias, const uint8_t* mask, const T* d_o,
                                                             const float* lse, const float* delta, T* dk, T* dv) {
  extern __shared__ float sm[];
  const int D = d.D, DP = 16 * DC + 1;
  float* Qs = sm;
  float* Ks = Qs + 64 * DP;
  float* Vs = Ks + 64 * DP;
  float* dOs = Vs + 64 * DP;
  float* Ps = dOs + 64 * DP;   // [64][65]
  float* dSs = Ps + 64 * 65;   // [64][65]
  float* lse_s = dSs + 64 * 65;
  float* delta_s = lse_s + 64;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int k0 = blockIdx.x * TK;
  int z = blockIdx.y;
  const int h = z % d.H; z /= d.H;
  const int s = z % d.n_seq;
  const int b = z / d.n_seq;
  for (int idx = ty * 16 + tx; idx < 4 * 64 * DP; idx += 256) sm[idx] = 0.f;
  __syncthreads();
  load_tile<T, TF32>(Ks, DP, k, d.k_st, b, s, h, k0, d.n_res, D, 1.0f);
  load_tile<T, TF32>(Vs, DP, v, d.v_st, b, s, h, k0, d.n_res, D, 1.0f);
  float acc_k[4][DC], acc_v[4][DC];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < DC; ++c) { acc_k[r][c] = 0.f; acc_v[r][c] = 0.f; }
  for (int q0 = 0; q0 < d.n_res; q0 += TQ) {
    load_tile<T, TF32>(Qs, DP, q, d.q_st, b, s, h, q0, d.n_res, D, d.scale);
    load_tile<T, TF32>(dOs, DP, d_o, d.do_st, b, s, h, q0, d.n_res, D, 1.0f);
    load_row_stats(d, lse, delta, b, s, h, q0, lse_s, delta_s);
    __syncthreads();
    float p[4][4], ds[4][4];
    p_and_ds<T, DC>(d, Qs, Ks, Vs, dOs, DP, bias, mask, lse_s, delta_s, b, s, h, q0, k0, p, ds);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        Ps[(ty + 16 * r) * 65 + tx + 16 * c] = TF32 ? round_tf32(p[r][c]) : p[r][c];
        dSs[(ty + 16 * r) * 65 + tx + 16 * c] = TF32 ? round_tf32(ds[r][c]) : ds[r][c];
      }
    __syncthreads();
    cols_times_tile<DC>(Ps, dOs, DP, acc_v);   // dV[k] += sum_q P[q,k] dO[q]
    cols_times_tile<DC>(dSs, Qs, DP, acc_k);   // dK[k] += sum_q dS[q,k] (scale q)
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int kj = k0 + ty + 16 * r;
    if (kj >= d.n_res) continue;
    T* krow = dk + off4(d.dk_st, b, s, kj, h);
    T* vrow = dv + off4(d.dv_st, b, s, kj, h);
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      int dd = tx + 16 * c;
      if (dd < D) { krow[dd] = from_f32<T>(acc_k[r][c]); vrow[dd] = from_f32<T>(acc_v[r][c]); }
    }
  }
}

template <typename T, int DC, bool TF32>
__global__ void __launch_bounds__(256) attn_bwd_dq_kernel(TriAttnDesc d, const T* q, const T* k, const T* v,
                                                           const T* bias, const uint8_t* mask, const T* d_o,
                                                           const float* lse, const float* delta, T* dq) {
  extern __shared__ float sm[];
  const int D = d.D, DP = 16 * DC + 1;
  float* Qs = sm;
  float* Ks = Qs + 64 * DP;
  float* Vs = Ks + 64 * DP;
  float* dOs = Vs + 64 * DP;
  float* dSs = dOs + 64 * DP;  // [64][65]
  float* lse_s = dSs + 64 * 65;
  float* delta_s = lse_s + 64;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int q0 = blockIdx.x * TQ;
  int z = blockIdx.y;
  const int h = z % d.H; z /= d.H;
  const int s = z % d.n_seq;
  const int b = z / d.n_seq;
  for (int idx = ty * 16 + tx; idx < 4 * 64 * DP; idx += 256) sm[idx] = 0.f;
  __syncthreads();
  load_tile<T, TF32>(Qs, DP, q, d.q_st, b, s, h, q0, d.n_res, D, d.scale);
  load_tile<T, TF32>(dOs, DP, d_o, d.do_st, b, s, h, q0, d.n_res, D, 1.0f);
  load_row_stats(d, lse, delta, b, s, h, q0, lse_s, delta_s);
  float acc[4][DC];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[r][c] = 0.f;
  for (int k0 = 0; k0 < d.n_res; k0 += TK) {
    load_tile<T, TF32>(Ks, DP, k, d.k_st, b, s, h, k0, d.n_res, D, 1.0f);
    load_tile<T, TF32>(Vs, DP, v, d.v_st, b, s, h, k0, d.n_res, D, 1.0f);
    __syncthreads();
    float p[4][4], ds[4][4];
    p_and_ds<T, DC>(d, Qs, Ks, Vs, dOs, DP, bias, mask, lse_s, delta_s, b, s, h, q0, k0, p, ds);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) dSs[(ty + 16 * r) * 65 + tx + 16 * c] = TF32 ? round_tf32(ds[r][c]) : ds[r][c];
    __syncthreads();
    rows_times_tile<DC>(dSs, Ks, DP, acc);  // dQ[q] += sum_k dS[q,k] K[k]
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int qi = q0 + ty + 16 * r;
    if (qi >= d.n_res) continue;
    T* row = dq + off4(d.dq_st, b, s, qi, h);
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      int dd = tx + 16 * c;
      if (dd < D) row[dd] = from_f32<T>(acc[r][c] * d.scale);
    }
  }
}

// dbias[b,h,i,j] = sum over rows s of dS; one CTA per (query tile, key tile, b, h), rows in order.
template <typename T, int DC, bool TF32>
__global__ void __launch_bounds__(256) attn_bwd_dbias_kernel(TriAttnDesc d, const T* q, const T* k, const T* v,
                                                              const T* bias, const uint8_t* mask, const T* d_o,
                                                              const float* lse, const float* delta, float* dbias) {
  extern __shared__ float sm[];
  const int D = d.D, DP = 16 * DC + 1;
  float* Qs = sm;
  float* Ks = Qs + 64 * DP;
  float* Vs = Ks + 64 * DP;
  float* dOs = Vs + 64 * DP;
  float* lse_s = dOs + 64 * DP;
  float* delta_s = lse_s + 64;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int q0 = blockIdx.x * TQ, k0 = blockIdx.y * TK;
  const int h = blockIdx.z % d.H, b = blockIdx.z / d.H;
  for (int idx = ty * 16 + tx; idx < 4 * 64 * DP; idx += 256) sm[idx] = 0.f;
  __syncthreads();
  float acc[4][4] = {};
  for (int s = 0; s < d.n_seq; ++s) {
    load_tile<T, TF32>(Qs, DP, q, d.q_st, b, s, h, q0, d.n_res, D, d.scale);
    load_tile<T, TF32>(dOs, DP, d_o, d.do_st, b, s, h, q0, d.n_res, D, 1.0f);
    load_tile<T, TF32>(Ks, DP, k, d.k_st, b, s, h, k0, d.n_res, D, 1.0f);
    load_tile<T, TF32>(Vs, DP, v, d.v_st, b, s, h, k0, d.n_res, D, 1.0f);
    load_row_stats(d, lse, delta, b, s, h, q0, lse_s, delta_s);
    __syncthreads();
    float p[4][4], ds[4][4];
    p_and_ds<T, DC>(d, Qs, Ks, Vs, dOs, DP, bias, mask, lse_s, delta_s, b, s, h, q0, k0, p, ds);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][c] += ds[r][c];
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int qi = q0 + ty + 16 * r;
    if (qi >= d.n_res) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int kj = k0 + tx + 16 * c;
      if (kj < d.n_res) dbias[(((long long)b * d.H + h) * d.n_res + qi) * d.n_res + kj] = acc[r][c];
    }
  }
}

template <typename KernelT>
int set_smem(KernelT kern, size_t bytes) {
  if (bytes > 48 * 1024) TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return 0;
}

template <typename T, int DC, bool TF32>
int fwd_launch(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
               const uint8_t* mask, void* o, float* lse, cudaStream_t st) {
  const int DP = 16 * DC + 1;
  size_t smem = (3 * 64 * DP + 64 * 65) * sizeof(float);
  auto kern = attn_fwd_kernel<T, DC, TF32>;
  TRI_TRY(set_smem(kern, smem));
  dim3 grid(cdiv(d->n_res, TQ), d->B * d->n_seq * d->H);
  const double pairs = (double)d->B * d->n_seq * d->H * d->n_res * (double)d->n_res;
  KernelTimer kt("simt_attn_fwd", st, 4.0 * pairs * d->D, 4.0 * sizeof(T) * d->B * d->n_seq * (double)d->n_res * d->H * d->D);
  kern<<<grid, dim3(16, 16), smem, st>>>(*d, (const T*)q, (const T*)k, (const T*)v, (const T*)bias, mask, (T*)o, lse);
  TRI_LAUNCH_OK();
  return 0;
}

template <typename T, int DC, bool TF32>
int bwd_launch(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
               const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk, void* dv,
               float* dbias, float* delta, cudaStream_t st) {
  const int DP = 16 * DC + 1;
  const long long rows = (long long)d->B * d->n_seq * d->H * d->n_res;
  const double pairs = (double)d->B * d->n_seq * d->H * d->n_res * (double)d->n_res;
  const double tensor_bytes = sizeof(T) * (double)d->B * d->n_seq * d->n_res * d->H * d->D;
  {
    KernelTimer kt("simt_attn_delta", st, 0.0, 2.0 * tensor_bytes);
    attn_delta_kernel<T><<<cdiv(rows, 256), 256, 0, st>>>(*d, (const T*)o, (const T*)d_o, delta);
    TRI_LAUNCH_OK();
  }
  const dim3 block(16, 16);
  {
    size_t smem = (4 * 64 * DP + 2 * 64 * 65 + 192) * sizeof(float);
    auto kern = attn_bwd_dkdv_kernel<T, DC, TF32>;
    TRI_TRY(set_smem(kern, smem));
    dim3 grid(cdiv(d->n_res, TK), d->B * d->n_seq * d->H);
    KernelTimer kt("simt_attn_bwd_dkdv", st, 8.0 * pairs * d->D, 6.0 * tensor_bytes);
    kern<<<grid, block, smem, st>>>(*d, (const T*)q, (const T*)k, (const T*)v, (const T*)bias, mask, (const T*)d_o,
                                    lse, delta, (T*)dk, (T*)dv);
    TRI_LAUNCH_OK();
  }
  {
    size_t smem = (4 * 64 * DP + 64 * 65 + 192) * sizeof(float);
    auto kern = attn_bwd_dq_kernel<T, DC, TF32>;
    TRI_TRY(set_smem(kern, smem));
    dim3 grid(cdiv(d->n_res, TQ), d->B * d->n_seq * d->H);
    KernelTimer kt("simt_attn_bwd_dq", st, 2.0 * pairs * d->D, 5.0 * tensor_bytes);
    kern<<<grid, block, smem, st>>>(*d, (const T*)q, (const T*)k, (const T*)v, (const T*)bias, mask, (const T*)d_o,
                                    lse, delta, (T*)dq);
    TRI_LAUNCH_OK();
  }
  if (dbias != nullptr) {
    size_t smem = (4 * 64 * DP + 192) * sizeof(float);
    auto kern = attn_bwd_dbias_kernel<T, DC, TF32>;
    TRI_TRY(set_smem(kern, smem));
    dim3 grid(cdiv(d->n_res, TQ), cdiv(d->n_res, TK), d->B * d->H);
    KernelTimer kt("simt_attn_bwd_dbias", st, 0.0, 4.0 * tensor_bytes);
    kern<<<grid, block, smem, st>>>(*d, (const T*)q, (const T*)k, (const T*)v, (const T*)bias, mask, (const T*)d_o,
                                    lse, delta, dbias);
    TRI_LAUNCH_OK();
  }
  return 0;
}

#define TRI_ATTN_DISPATCH(FN, ...)                                                            \
  do {                                                                                        \
    const bool tf32 = d->dtype == TRI_F32 && d->precision == TRI_PREC_TF32;                   \
    const int dc = d->D <= 32 ? 2 : (d->D <= 64 ? 4 : 8);                                     \
    if (d->dtype == TRI_F32) {                                                                \
      if (tf32) {                                                                             \
        if (dc == 2) return FN<float, 2, true>(__VA_ARGS__);                                  \
        if (dc == 4) return FN<float, 4, true>(__VA_ARGS__);                                  \
        return FN<float, 8, true>(__VA_ARGS__);                                               \
      }                                                                                       \
      if (dc == 2) return FN<float, 2, false>(__VA_ARGS__);                                   \
      if (dc == 4) return FN<float, 4, false>(__VA_ARGS__);                                   \
      return FN<float, 8, false>(__VA_ARGS__);                                                \
    }                                                                                         \
    if (d->dtype == TRI_BF16) {                                                               \
      if (dc == 2) return FN<__nv_bfloat16, 2, false>(__VA_ARGS__);                           \
      if (dc == 4) return FN<__nv_bfloat16, 4, false>(__VA_ARGS__);                           \
      return FN<__nv_bfloat16, 8, false>(__VA_ARGS__);                                        \
    }                                                                                         \
    if (dc == 2) return FN<__half, 2, false>(__VA_ARGS__);                                    \
    if (dc == 4) return FN<__half, 4, false>(__VA_ARGS__);                                    \
    return FN<__half, 8, false>(__VA_ARGS__);                                                 \
  } while (0)

}  // namespace

size_t attn_ws_bytes(const TriAttnDesc* d, int is_bwd) {
  if (!is_bwd) return 256;
  return align_up((size_t)d->B * d->n_seq * d->H * d->n_res * sizeof(float)) + 256;
}

int attn_forward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                 const uint8_t* mask, void* o, float* lse, cudaStream_t st) {
  TRI_ATTN_DISPATCH(fwd_launch, d, q, k, v, bias, mask, o, lse, st);
}

int attn_backward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                  const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                  void* dv, float* dbias, void* ws, size_t ws_size, cudaStream_t st) {
  if (ws_size < attn_ws_bytes(d, 1)) return fail(TRI_ERR_WORKSPACE, "attention backward workspace too small");
  float* delta = (float*)ws;
  TRI_ATTN_DISPATCH(bwd_launch, d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, delta, st);
}

// ---------------------------------------------------------------------------------------------
// Backward without any caller- or library-allocated scratch.
//
// Some callers cannot hand this library a workspace: code running where device allocation is
// forbidden or impossible (a real-time serving loop with a frozen memory pool, a plugin host that
// gives operators no allocator, a process already at its memory limit).  For them the one scratch
// buffer the backward needs, delta[b,s,h,i] = sum_d dO*O, lives in this file-scope device array.
// Every GPU that loads the library carries these 4 MiB until the process exits.
//
// The array's name is only a host-side handle.  Its device address is looked up once per device, with
// that device current, through cudaGetSymbolAddress, and that address is what the kernels get.
// ---------------------------------------------------------------------------------------------
constexpr size_t kStaticDeltaFloats = size_t(1) << 20;  // B * n_seq * H * n_res may not exceed this
static __device__ __align__(256) float g_static_delta[kStaticDeltaFloats];

size_t attn_static_scratch_rows() { return kStaticDeltaFloats; }

int attn_backward_static(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                         const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                         void* dv, float* dbias, cudaStream_t st) {
  const size_t rows = (size_t)d->B * d->n_seq * d->H * d->n_res;
  if (rows > kStaticDeltaFloats)
    return fail(TRI_ERR_UNSUPPORTED,
                "B*n_seq*H*n_res = %zu exceeds the built-in scratch of %zu rows; use tri_attn_bwd with a workspace",
                rows, kStaticDeltaFloats);
  constexpr int kMaxDevices = 64;
  static float* device_ptr[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  TRI_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(TRI_ERR_UNSUPPORTED, "device index %d out of range", dev);
  float* delta = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (device_ptr[dev] == nullptr) {
      void* p = nullptr;
      TRI_CUDA_OK(cudaGetSymbolAddress(&p, g_static_delta));  // first call on this device: set-up
      device_ptr[dev] = static_cast<float*>(p);
    }
    delta = device_ptr[dev];
  }
  // delta is written in full by the first kernel before anything reads it: nothing to clear.
  TRI_ATTN_DISPATCH(bwd_launch, d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, delta, st);
}

}  // namespace simt
}  // namespace tri
