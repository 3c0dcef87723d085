// Exact-fp32 (CUDA-core) path of the triangle multiplicative update.
//
// This is the path behind fp32 inputs with matmul precision "ieee" (no tensor
// core offers exact fp32 products) and behind every shape the tensor-core path
// does not cover.  All intermediates are fp32 and pixel-major ([B*N*N, channels]);
// only the tensors that cross the ABI (x, mask, weights, out, d_out, dx) are in
// the caller's dtype.  With precision == tf32 the operands of every product are
// rounded to the tf32 grid first, so the two precisions differ bitwise as the
// reference's do (tests/test_trimul.py:185-201 of the reference).
//
// Math follows trimul_torch (geometric_nn_ops_torch/triangle/_reference/trimul.py:57-97).
#include <algorithm>

#include "common.cuh"
#include "trimul_simt.cuh"

namespace tri {
namespace simt {

// ============================================================================
// generic strided GEMM   C[m,n] (+)= sum_k A(m,k) * B(n,k)  (+ bias[n])
// ============================================================================
struct GemmP {
  const float* A;
  const float* B;
  float* C;
  const float* bias;
  int M, N, K;
  long long a_m, a_k, b_n, b_k, c_m, c_n;
  int ksplit;
  long long c_split;
  int accumulate;
};

template <bool TF32>
__global__ void __launch_bounds__(256) gemm_kernel(GemmP p) {
  __shared__ float As[16][65];
  __shared__ float Bs[16][65];
  const int tid = threadIdx.y * 16 + threadIdx.x;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  int kper = (p.K + p.ksplit - 1) / p.ksplit;
  kper = (kper + 15) / 16 * 16;
  const int kbeg = blockIdx.z * kper;
  const int kend = min(p.K, kbeg + kper);
  float acc[4][4] = {};
  for (int k0 = kbeg; k0 < kend; k0 += 16) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + 256 * e;
      int mm, kk;
      if (p.a_k == 1) { kk = idx & 15; mm = idx >> 4; } else { mm = idx & 63; kk = idx >> 6; }
      float v = 0.f;
      if (m0 + mm < p.M && k0 + kk < kend) v = p.A[(long long)(m0 + mm) * p.a_m + (long long)(k0 + kk) * p.a_k];
      As[kk][mm] = TF32 ? round_tf32(v) : v;
      int nn;
      if (p.b_k == 1) { kk = idx & 15; nn = idx >> 4; } else { nn = idx & 63; kk = idx >> 6; }
      v = 0.f;
      if (n0 + nn < p.N && k0 + kk < kend) v = p.B[(long long)(n0 + nn) * p.b_n + (long long)(k0 + kk) * p.b_k];
      Bs[kk][nn] = TF32 ? round_tf32(v) : v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = As[kk][ty + 16 * r];
#pragma unroll
      for (int c = 0; c < 4; ++c) b[c] = Bs[kk][tx + 16 * c];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
    }
    __syncthreads();
  }
  float* C = p.C + (long long)blockIdx.z * p.c_split;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    int m = m0 + ty + 16 * r;
    if (m >= p.M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int n = n0 + tx + 16 * c;
      if (n >= p.N) continue;
      float v = acc[r][c];
      if (p.bias != nullptr && blockIdx.z == 0) v += p.bias[n];
      long long o = (long long)m * p.c_m + (long long)n * p.c_n;
      if (p.accumulate) v += C[o];
      C[o] = v;
    }
  }
}

static int gemm(cudaStream_t st, bool tf32, GemmP p) {
  if (p.M <= 0 || p.N <= 0) return 0;
  dim3 grid(cdiv(p.N, 64), cdiv(p.M, 64), p.ksplit);
  dim3 block(16, 16);
  KernelTimer kt("simt_gemm", st, 2.0 * p.M * p.N * p.K, 4.0 * ((double)p.M * p.K + (double)p.N * p.K + (double)p.M * p.N));
  if (tf32) gemm_kernel<true><<<grid, block, 0, st>>>(p);
  else gemm_kernel<false><<<grid, block, 0, st>>>(p);
  TRI_LAUNCH_OK();
  return 0;
}

// out[j] = sum_p partial[p*n + j]
__global__ void reduce_partials_kernel(const float* partial, int nparts, long long n, float* out) {
  long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (j >= n) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * n + j];
  out[j] = s;
}

static int reduce_partials(cudaStream_t st, const float* partial, int nparts, long long n, float* out) {
  KernelTimer kt("simt_reduce_partials", st, 0.0, 4.0 * (nparts + 1) * n);
  reduce_partials_kernel<<<cdiv(n, 256), 256, 0, st>>>(partial, nparts, n, out);
  TRI_LAUNCH_OK();
  return 0;
}

// dW[n_out, n_in] = sum_rows D[row, n_out] * Z[row, n_in], split over rows, deterministic.
static int weight_grad(cudaStream_t st, bool tf32, const float* D, int ldd, int n_out, const float* Z,
                       int ldz, int n_in, long long rows, float* partial, int ksplit, float* out) {
  GemmP p{};
  p.A = D; p.a_m = 1; p.a_k = ldd;
  p.B = Z; p.b_n = 1; p.b_k = ldz;
  p.C = partial; p.c_m = n_in; p.c_n = 1;
  p.M = n_out; p.N = n_in; p.K = (int)rows;
  p.ksplit = ksplit; p.c_split = (long long)n_out * n_in;
  TRI_TRY(gemm(st, tf32, p));
  return reduce_partials(st, partial, ksplit, (long long)n_out * n_in, out);
}

// ============================================================================
// per-channel contraction  O[p,q,c] = sum_r X(p,r,c) * Y(q,r,c)
// One thread per channel (coalesced along c), 8x8 output pixels per thread.
// ============================================================================
struct ContractP {
  const float* X;
  const float* Y;
  float* O;
  int N, Ch, cblocks;
  long long xs_p, xs_r, ys_q, ys_r, os_p, os_q;  // pixel strides inside one N x N plane
  int ldx, ldy, ldo;                             // channels per pixel in each buffer
  int xoff, yoff, ooff;                          // first channel inside the buffer
};

template <bool TF32>
__global__ void __launch_bounds__(128) contract_kernel(ContractP p) {
  const int cb = blockIdx.z % p.cblocks;
  const int b = blockIdx.z / p.cblocks;
  const int c = cb * blockDim.x + threadIdx.x;
  const bool c_ok = c < p.Ch;
  const int p0 = blockIdx.x * 8;
  const int q0 = (blockIdx.y * blockDim.y + threadIdx.y) * 8;
  const long long plane = (long long)b * p.N * p.N;
  float acc[8][8] = {};
  const float* X = p.X + p.xoff + (c_ok ? c : 0);
  const float* Y = p.Y + p.yoff + (c_ok ? c : 0);
  for (int r = 0; r < p.N; ++r) {
    float xv[8], yv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int pp = p0 + i;
      xv[i] = (c_ok && pp < p.N) ? X[(plane + pp * p.xs_p + r * p.xs_r) * p.ldx] : 0.f;
      int qq = q0 + i;
      yv[i] = (c_ok && qq < p.N) ? Y[(plane + qq * p.ys_q + r * p.ys_r) * p.ldy] : 0.f;
      if (TF32) { xv[i] = round_tf32(xv[i]); yv[i] = round_tf32(yv[i]); }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(xv[i], yv[j], acc[i][j]);
  }
  if (!c_ok) return;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (p0 + i >= p.N) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (q0 + j >= p.N) continue;
      p.O[(plane + (p0 + i) * p.os_p + (q0 + j) * p.os_q) * p.ldo + p.ooff + c] = acc[i][j];
    }
  }
}

static int contract(cudaStream_t st, bool tf32, int B, ContractP p) {
  int bx = p.Ch >= 128 ? 128 : (p.Ch + 31) / 32 * 32;
  int by = 128 / bx;
  p.cblocks = cdiv(p.Ch, bx);
  dim3 block(bx, by);
  dim3 grid(cdiv(p.N, 8), cdiv(p.N, 8 * by), B * p.cblocks);
  KernelTimer kt("simt_contract", st, 2.0 * B * p.N * (double)p.N * p.N * p.Ch, 12.0 * B * (double)p.N * p.N * p.Ch);
  if (tf32) contract_kernel<true><<<grid, block, 0, st>>>(p);
  else contract_kernel<false><<<grid, block, 0, st>>>(p);
  TRI_LAUNCH_OK();
  return 0;
}

// ============================================================================
// LayerNorm forward / backward (one warp per row)
// ============================================================================
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename TI>
__global__ void __launch_bounds__(256) ln_fwd_kernel(const TI* x, const float* gamma, const float* beta,
                                                      float eps, long long M, int C, float* z,
                                                      float* mean, float* rstd) {
  const int lane = threadIdx.x & 31;
  long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= M) return;
  const TI* xr = x + row * C;
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += to_f32(xr[c]);
  const float mu = warp_sum(s) / C;
  float v = 0.f;
  for (int c = lane; c < C; c += 32) { float d = to_f32(xr[c]) - mu; v += d * d; }
  const float rs = 1.0f / sqrtf(warp_sum(v) / C + eps);
  for (int c = lane; c < C; c += 32) {
    float h = (to_f32(xr[c]) - mu) * rs;
    if (gamma) h *= gamma[c];
    if (beta) h += beta[c];
    z[row * C + c] = h;
  }
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
}

// d_in = rstd * (dhat - mean(dhat) - xhat * mean(dhat * xhat)), dhat = d_out * gamma.
// Per-block partial sums of d_out*xhat and d_out go to pg/pb [gridDim.x, C].
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const float* d_out, const TI* x, const float* mean,
                                                      const float* rstd, const float* gamma, long long M,
                                                      int C, TO* d_in, float* pg, float* pb) {
  extern __shared__ float sm[];  // [8][C] dgamma, [8][C] dbeta
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* sg = sm + warp * C;
  float* sb = sm + (8 + warp) * C;
  for (int c = lane; c < C; c += 32) { sg[c] = 0.f; sb[c] = 0.f; }
  for (long long row = blockIdx.x * 8LL + warp; row < M; row += gridDim.x * 8LL) {
    const float mu = mean[row], rs = rstd[row];
    const TI* xr = x + row * C;
    const float* dr = d_out + row * C;
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < C; c += 32) {
      float h = (to_f32(xr[c]) - mu) * rs;
      float d = dr[c];
      float dh = gamma ? d * gamma[c] : d;
      s1 += dh;
      s2 += dh * h;
      sg[c] += d * h;
      sb[c] += d;
    }
    const float m1 = warp_sum(s1) / C, m2 = warp_sum(s2) / C;
    for (int c = lane; c < C; c += 32) {
      float h = (to_f32(xr[c]) - mu) * rs;
      float dh = gamma ? dr[c] * gamma[c] : dr[c];
      d_in[row * C + c] = from_f32<TO>(rs * (dh - m1 - h * m2));
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += 256) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { g += sm[w * C + c]; b += sm[(8 + w) * C + c]; }
    pg[(long long)blockIdx.x * C + c] = g;
    pb[(long long)blockIdx.x * C + c] = b;
  }
}

constexpr int kLnBwdBlocks = 296;

template <typename TI, typename TO>
static int ln_bwd(cudaStream_t st, const float* d_out, const TI* x, const float* mean, const float* rstd,
                  const float* gamma, long long M, int C, TO* d_in, float* partial /*2*blocks*C*/,
                  float* dgamma, float* dbeta) {
  int blocks = (int)std::min<long long>(kLnBwdBlocks, (M + 7) / 8);
  size_t smem = 16 * (size_t)C * sizeof(float);
  auto kern = ln_bwd_kernel<TI, TO>;
  if (smem > 48 * 1024) TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  float* pg = partial;
  float* pb = partial + (size_t)blocks * C;
  {
    KernelTimer kt("simt_ln_bwd", st, 0.0, (double)M * C * (4.0 + sizeof(TI) + sizeof(TO)));
    kern<<<blocks, 256, smem, st>>>(d_out, x, mean, rstd, gamma, M, C, d_in, pg, pb);
    TRI_LAUNCH_OK();
  }
  if (dgamma) TRI_TRY(reduce_partials(st, pg, blocks, C, dgamma));
  if (dbeta) TRI_TRY(reduce_partials(st, pb, blocks, C, dbeta));
  return 0;
}

// ============================================================================
// elementwise stages
// ============================================================================
template <typename T>
__global__ void convert_kernel(const T* src, float* dst, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) dst[i] = to_f32(src[i]);
}

// ab = P * sigmoid(G) * mask  over [M, W]
__global__ void gate_in_kernel(const float* P, const float* G, const float* mask, long long M, int W, float* ab) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= M * W) return;
  float v = P[i] * sigmoidf_acc(G[i]);
  if (mask) v *= mask[i / W];
  ab[i] = v;
}

__global__ void gate_in_bwd_kernel(const float* dab, const float* P, const float* G, const float* mask,
                                   long long M, int W, float* dP, float* dG) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= M * W) return;
  float d = dab[i];
  if (mask) d *= mask[i / W];
  float g = sigmoidf_acc(G[i]);
  dP[i] = d * g;
  dG[i] = d * P[i] * g * (1.0f - g);
}

template <typename T>
__global__ void gate_out_kernel(const float* y, const float* go, long long n, T* out) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f32<T>(y[i] * sigmoidf_acc(go[i]));
}

template <typename T>
__global__ void gate_out_bwd_kernel(const T* d_out, const float* y, const float* go, long long n, float* dy, float* dgo) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  float d = to_f32(d_out[i]);
  float g = sigmoidf_acc(go[i]);
  dy[i] = d * g;
  dgo[i] = d * y[i] * g * (1.0f - g);
}

// partial[blockIdx.x][c] = sum over this block's rows of X[row, c]
__global__ void colsum_kernel(const float* X, long long M, int C, float* partial) {
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  long long per = (M + gridDim.x - 1) / gridDim.x;
  long long r0 = blockIdx.x * per, r1 = min(M, r0 + per);
  float s = 0.f;
  for (long long r = r0; r < r1; ++r) s += X[r * C + c];
  partial[(long long)blockIdx.x * C + c] = s;
}

constexpr int kColsumBlocks = 256;
static int colsum(cudaStream_t st, const float* X, long long M, int C, float* partial, float* out) {
  dim3 grid(kColsumBlocks, cdiv(C, 128));
  KernelTimer kt("simt_colsum", st, 0.0, 4.0 * M * C);
  colsum_kernel<<<grid, 128, 0, st>>>(X, M, C, partial);
  TRI_LAUNCH_OK();
  return reduce_partials(st, partial, kColsumBlocks, C, out);
}

#define EW_GRID(n) cdiv((n), 256), 256, 0, st

// ============================================================================
// memory plan
// ============================================================================
struct WeightsF32 {
  float *norm_in_w, *norm_in_b, *p_in_w, *p_in_b, *g_in_w, *g_in_b;
  float *norm_out_w, *norm_out_b, *p_out_w, *p_out_b, *g_out_w, *g_out_b, *mask;
};

struct Saved {
  float *z, *P, *G, *ab, *t, *y, *go, *mean_in, *rstd_in, *mean_out, *rstd_out;
};

static size_t carve_saved(Arena& a, const TriMulDesc* d, Saved* s) {
  const size_t M = (size_t)d->B * d->N * d->N;
  s->z = a.take<float>(M * d->C);
  s->P = a.take<float>(M * 2 * d->Ch);
  s->G = a.take<float>(M * 2 * d->Ch);
  s->ab = a.take<float>(M * 2 * d->Ch);
  s->t = a.take<float>(M * d->Ch);
  s->y = a.take<float>(M * d->C);
  s->go = a.take<float>(M * d->C);
  s->mean_in = a.take<float>(M);
  s->rstd_in = a.take<float>(M);
  s->mean_out = a.take<float>(M);
  s->rstd_out = a.take<float>(M);
  return a.off;
}

static void carve_weights(Arena& a, const TriMulDesc* d, WeightsF32* w) {
  const size_t C = d->C, Ch = d->Ch;
  w->norm_in_w = a.take<float>(C); w->norm_in_b = a.take<float>(C);
  w->p_in_w = a.take<float>(2 * Ch * C); w->p_in_b = a.take<float>(2 * Ch);
  w->g_in_w = a.take<float>(2 * Ch * C); w->g_in_b = a.take<float>(2 * Ch);
  w->norm_out_w = a.take<float>(Ch); w->norm_out_b = a.take<float>(Ch);
  w->p_out_w = a.take<float>(C * Ch); w->p_out_b = a.take<float>(C);
  w->g_out_w = a.take<float>(C * C); w->g_out_b = a.take<float>(C);
  w->mask = a.take<float>((size_t)d->B * d->N * d->N);
}

constexpr int kWgradSplit = 128;

size_t saved_bytes(const TriMulDesc* d) {
  Arena a(nullptr, 0);
  Saved s;
  return carve_saved(a, d, &s);
}

size_t ws_bytes(const TriMulDesc* d, int is_bwd) {
  Arena a(nullptr, 0);
  WeightsF32 w;
  carve_weights(a, d, &w);
  Saved s;
  carve_saved(a, d, &s);  // forward without a saved block keeps its intermediates here
  if (is_bwd) {
    const size_t M = (size_t)d->B * d->N * d->N, C = d->C, Ch = d->Ch;
    a.take<float>(M * Ch);      // u
    a.take<float>(M * C);       // dy
    a.take<float>(M * C);       // dgo
    a.take<float>(M * Ch);      // du
    a.take<float>(M * Ch);      // dt
    a.take<float>(M * 2 * Ch);  // dab
    a.take<float>(M * 2 * Ch);  // dP
    a.take<float>(M * 2 * Ch);  // dG
    a.take<float>(M * C);       // dz
    size_t wmax = std::max((size_t)2 * Ch * C, std::max(C * Ch, C * C));
    a.take<float>(std::max((size_t)kWgradSplit * wmax, (size_t)2 * kLnBwdBlocks * std::max(C, Ch)));
  }
  return a.off + 256;
}

template <typename T>
static int convert_weights(cudaStream_t st, const TriMulDesc* d, const TriMulWeights* w, const void* mask, WeightsF32* f) {
  struct Item { const void* src; float** dst; size_t n; };
  const size_t C = d->C, Ch = d->Ch;
  Item items[] = {
      {w->norm_in_w, &f->norm_in_w, C},       {w->norm_in_b, &f->norm_in_b, C},
      {w->p_in_w, &f->p_in_w, 2 * Ch * C},    {w->p_in_b, &f->p_in_b, 2 * Ch},
      {w->g_in_w, &f->g_in_w, 2 * Ch * C},    {w->g_in_b, &f->g_in_b, 2 * Ch},
      {w->norm_out_w, &f->norm_out_w, Ch},    {w->norm_out_b, &f->norm_out_b, Ch},
      {w->p_out_w, &f->p_out_w, C * Ch},      {w->p_out_b, &f->p_out_b, C},
      {w->g_out_w, &f->g_out_w, C * C},       {w->g_out_b, &f->g_out_b, C},
      {mask, &f->mask, (size_t)d->B * d->N * d->N},
  };
  for (auto& it : items) {
    if (it.src == nullptr) { *it.dst = nullptr; continue; }
    convert_kernel<T><<<EW_GRID((long long)it.n)>>>((const T*)it.src, *it.dst, (long long)it.n);
    TRI_LAUNCH_OK();
  }
  return 0;
}

static GemmP linear_p(const float* in, int ld_in, const float* W, const float* bias, float* out, int ld_out,
                      long long rows, int n_out, int n_in) {
  GemmP p{};
  p.A = in; p.a_m = ld_in; p.a_k = 1;
  p.B = W; p.b_n = n_in; p.b_k = 1;
  p.C = out; p.c_m = ld_out; p.c_n = 1;
  p.bias = bias;
  p.M = (int)rows; p.N = n_out; p.K = n_in; p.ksplit = 1;
  return p;
}

// out[rows, n_in] (+)= D[rows, n_out] * W[n_out, n_in]
static GemmP linear_t_p(const float* D, int ldd, const float* W, float* out, long long rows, int n_out, int n_in, int accumulate) {
  GemmP p{};
  p.A = D; p.a_m = ldd; p.a_k = 1;
  p.B = W; p.b_n = 1; p.b_k = n_in;
  p.C = out; p.c_m = n_in; p.c_n = 1;
  p.M = (int)rows; p.N = n_in; p.K = n_out; p.ksplit = 1; p.accumulate = accumulate;
  return p;
}

template <typename T>
static int forward_t(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out,
                     void* saved, void* ws, size_t ws_size, cudaStream_t st) {
  const long long M = (long long)d->B * d->N * d->N;
  const int C = d->C, Ch = d->Ch, N = d->N;
  const bool tf32 = d->dtype == TRI_F32 && d->precision == TRI_PREC_TF32;
  Arena a(ws, ws_size);
  WeightsF32 f;
  carve_weights(a, d, &f);
  Saved s;
  if (saved) { Arena sa(saved, saved_bytes(d)); carve_saved(sa, d, &s); }
  else carve_saved(a, d, &s);
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul forward workspace too small: need %zu, got %zu", a.off, ws_size);
  TRI_TRY(convert_weights<T>(st, d, w, mask, &f));

  {
    KernelTimer kt("simt_ln_fwd", st, 0.0, (double)M * C * (sizeof(T) + 4.0));
    ln_fwd_kernel<T><<<cdiv(M, 8), 256, 0, st>>>((const T*)x, f.norm_in_w, f.norm_in_b, d->eps, M, C, s.z, s.mean_in, s.rstd_in);
    TRI_LAUNCH_OK();
  }
  TRI_TRY(gemm(st, tf32, linear_p(s.z, C, f.p_in_w, f.p_in_b, s.P, 2 * Ch, M, 2 * Ch, C)));
  TRI_TRY(gemm(st, tf32, linear_p(s.z, C, f.g_in_w, f.g_in_b, s.G, 2 * Ch, M, 2 * Ch, C)));
  {
    KernelTimer kt("simt_gate_in", st, 0.0, 24.0 * M * Ch);
    gate_in_kernel<<<EW_GRID(M * 2 * Ch)>>>(s.P, s.G, f.mask, M, 2 * Ch, s.ab);
    TRI_LAUNCH_OK();
  }
  ContractP cp{};
  cp.X = s.ab; cp.Y = s.ab; cp.O = s.t; cp.N = N; cp.Ch = Ch;
  cp.ldx = cp.ldy = 2 * Ch; cp.ldo = Ch; cp.xoff = 0; cp.yoff = Ch; cp.ooff = 0;
  cp.os_p = N; cp.os_q = 1;
  if (d->direction == TRI_OUTGOING) { cp.xs_p = N; cp.xs_r = 1; cp.ys_q = N; cp.ys_r = 1; }
  else { cp.xs_p = 1; cp.xs_r = N; cp.ys_q = 1; cp.ys_r = N; }
  TRI_TRY(contract(st, tf32, d->B, cp));
  // LayerNormed contraction output: P is dead by now in inference, so it doubles as scratch there;
  // with a saved block P must survive, and the workspace region that would have held it is free.
  float* u_buf = saved ? a.take<float>((size_t)M * Ch) : s.P;
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul forward workspace too small: need %zu, got %zu", a.off, ws_size);
  {
    KernelTimer kt("simt_ln_fwd", st, 0.0, 8.0 * M * Ch);
    ln_fwd_kernel<float><<<cdiv(M, 8), 256, 0, st>>>(s.t, f.norm_out_w, f.norm_out_b, d->eps, M, Ch, u_buf, s.mean_out, s.rstd_out);
    TRI_LAUNCH_OK();
  }
  TRI_TRY(gemm(st, tf32, linear_p(u_buf, Ch, f.p_out_w, f.p_out_b, s.y, C, M, C, Ch)));
  TRI_TRY(gemm(st, tf32, linear_p(s.z, C, f.g_out_w, f.g_out_b, s.go, C, M, C, C)));
  {
    KernelTimer kt("simt_gate_out", st, 0.0, (double)M * C * (8.0 + sizeof(T)));
    gate_out_kernel<T><<<EW_GRID(M * C)>>>(s.y, s.go, M * C, (T*)out);
    TRI_LAUNCH_OK();
  }
  return 0;
}

template <typename T>
static int backward_t(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w,
                      const void* saved, const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws,
                      size_t ws_size, cudaStream_t st) {
  const long long M = (long long)d->B * d->N * d->N;
  const int C = d->C, Ch = d->Ch, N = d->N;
  const bool tf32 = d->dtype == TRI_F32 && d->precision == TRI_PREC_TF32;
  Arena a(ws, ws_size);
  WeightsF32 f;
  carve_weights(a, d, &f);
  Saved s;
  { Arena sa(const_cast<void*>(saved), saved_bytes(d)); carve_saved(sa, d, &s); }
  float* u = a.take<float>((size_t)M * Ch);
  float* dy = a.take<float>((size_t)M * C);
  float* dgo = a.take<float>((size_t)M * C);
  float* du = a.take<float>((size_t)M * Ch);
  float* dt = a.take<float>((size_t)M * Ch);
  float* dab = a.take<float>((size_t)M * 2 * Ch);
  float* dP = a.take<float>((size_t)M * 2 * Ch);
  float* dG = a.take<float>((size_t)M * 2 * Ch);
  float* dz = a.take<float>((size_t)M * C);
  size_t wmax = std::max((size_t)2 * Ch * C, std::max((size_t)C * Ch, (size_t)C * C));
  float* partial = a.take<float>(std::max((size_t)kWgradSplit * wmax, (size_t)2 * kLnBwdBlocks * std::max(C, Ch)));
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul backward workspace too small: need %zu, got %zu", a.off, ws_size);
  TRI_TRY(convert_weights<T>(st, d, w, mask, &f));

  // output gate and projection
  {
    KernelTimer kt("simt_gate_out_bwd", st, 0.0, (double)M * C * (16.0 + sizeof(T)));
    gate_out_bwd_kernel<T><<<EW_GRID(M * C)>>>((const T*)d_out, s.y, s.go, M * C, dy, dgo);
    TRI_LAUNCH_OK();
  }
  {
    KernelTimer kt("simt_ln_fwd", st, 0.0, 8.0 * M * Ch);
    ln_fwd_kernel<float><<<cdiv(M, 8), 256, 0, st>>>(s.t, f.norm_out_w, f.norm_out_b, d->eps, M, Ch, u, s.mean_out, s.rstd_out);
    TRI_LAUNCH_OK();
  }
  if (g->p_out_w) TRI_TRY(weight_grad(st, tf32, dy, C, C, u, Ch, Ch, M, partial, kWgradSplit, g->p_out_w));
  if (g->p_out_b) TRI_TRY(colsum(st, dy, M, C, partial, g->p_out_b));
  if (g->g_out_w) TRI_TRY(weight_grad(st, tf32, dgo, C, C, s.z, C, C, M, partial, kWgradSplit, g->g_out_w));
  if (g->g_out_b) TRI_TRY(colsum(st, dgo, M, C, partial, g->g_out_b));
  TRI_TRY(gemm(st, tf32, linear_t_p(dy, C, f.p_out_w, du, M, C, Ch, 0)));
  TRI_TRY((ln_bwd<float, float>(st, du, s.t, s.mean_out, s.rstd_out, f.norm_out_w, M, Ch, dt, partial, g->norm_out_w, g->norm_out_b)));

  // contraction backward: da -> dab[:, :Ch], db -> dab[:, Ch:]
  ContractP ca{}, cb{};
  ca.N = cb.N = N; ca.Ch = cb.Ch = Ch;
  ca.O = cb.O = dab; ca.ldo = cb.ldo = 2 * Ch; ca.ooff = 0; cb.ooff = Ch;
  ca.X = dt; ca.ldx = Ch; ca.xoff = 0; ca.Y = s.ab; ca.ldy = 2 * Ch; ca.yoff = Ch;   // dt with b
  if (d->direction == TRI_OUTGOING) {
    // da[i,k] = sum_j dt[i,j] b[j,k]        (p=i, q=k, r=j)
    ca.xs_p = N; ca.xs_r = 1; ca.ys_q = 1; ca.ys_r = N; ca.os_p = N; ca.os_q = 1;
    // db[j,k] = sum_i dt[i,j] a[i,k]        (p=j, q=k, r=i)
    cb.X = dt; cb.ldx = Ch; cb.xoff = 0; cb.Y = s.ab; cb.ldy = 2 * Ch; cb.yoff = 0;
    cb.xs_p = 1; cb.xs_r = N; cb.ys_q = 1; cb.ys_r = N; cb.os_p = N; cb.os_q = 1;
  } else {
    // da[k,i] = sum_j dt[i,j] b[k,j]        (p=i, q=k, r=j), stored at pixel (k,i)
    ca.xs_p = N; ca.xs_r = 1; ca.ys_q = N; ca.ys_r = 1; ca.os_p = 1; ca.os_q = N;
    // db[k,j] = sum_i a[k,i] dt[i,j]        (p=k, q=j, r=i)
    cb.X = s.ab; cb.ldx = 2 * Ch; cb.xoff = 0; cb.Y = dt; cb.ldy = Ch; cb.yoff = 0;
    cb.xs_p = N; cb.xs_r = 1; cb.ys_q = 1; cb.ys_r = N; cb.os_p = N; cb.os_q = 1;
  }
  TRI_TRY(contract(st, tf32, d->B, ca));
  TRI_TRY(contract(st, tf32, d->B, cb));

  // input gate and projections
  {
    KernelTimer kt("simt_gate_in_bwd", st, 0.0, 40.0 * M * Ch);
    gate_in_bwd_kernel<<<EW_GRID(M * 2 * Ch)>>>(dab, s.P, s.G, f.mask, M, 2 * Ch, dP, dG);
    TRI_LAUNCH_OK();
  }
  if (g->p_in_w) TRI_TRY(weight_grad(st, tf32, dP, 2 * Ch, 2 * Ch, s.z, C, C, M, partial, kWgradSplit, g->p_in_w));
  if (g->p_in_b) TRI_TRY(colsum(st, dP, M, 2 * Ch, partial, g->p_in_b));
  if (g->g_in_w) TRI_TRY(weight_grad(st, tf32, dG, 2 * Ch, 2 * Ch, s.z, C, C, M, partial, kWgradSplit, g->g_in_w));
  if (g->g_in_b) TRI_TRY(colsum(st, dG, M, 2 * Ch, partial, g->g_in_b));
  TRI_TRY(gemm(st, tf32, linear_t_p(dP, 2 * Ch, f.p_in_w, dz, M, 2 * Ch, C, 0)));
  TRI_TRY(gemm(st, tf32, linear_t_p(dG, 2 * Ch, f.g_in_w, dz, M, 2 * Ch, C, 1)));
  TRI_TRY(gemm(st, tf32, linear_t_p(dgo, C, f.g_out_w, dz, M, C, C, 1)));
  TRI_TRY((ln_bwd<T, T>(st, dz, (const T*)x, s.mean_in, s.rstd_in, f.norm_in_w, M, C, (T*)dx, partial, g->norm_in_w, g->norm_in_b)));
  return 0;
}

int forward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out,
            void* saved, void* ws, size_t ws_size, cudaStream_t st) {
  switch (d->dtype) {
    case TRI_F32: return forward_t<float>(d, x, mask, w, out, saved, ws, ws_size, st);
    case TRI_BF16: return forward_t<__nv_bfloat16>(d, x, mask, w, out, saved, ws, ws_size, st);
    case TRI_F16: return forward_t<__half>(d, x, mask, w, out, saved, ws, ws_size, st);
  }
  return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
}

int backward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, const void* saved,
             const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws, size_t ws_size, cudaStream_t st) {
  switch (d->dtype) {
    case TRI_F32: return backward_t<float>(d, x, mask, w, saved, d_out, dx, g, ws, ws_size, st);
    case TRI_BF16: return backward_t<__nv_bfloat16>(d, x, mask, w, saved, d_out, dx, g, ws, ws_size, st);
    case TRI_F16: return backward_t<__half>(d, x, mask, w, saved, d_out, dx, g, ws, ws_size, st);
  }
  return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
}

}  // namespace simt
}  // namespace tri
