// Tensor-core path of the triangle multiplicative update (C_z = C_hidden = 128), forward and backward.
//
// Every product runs on tcgen05 through tc_gemm (bf16 / fp16 operands, or tf32 for fp32 inputs with
// precision "tf32"); LayerNorm, transposes and reductions are memory-bound kernels with 8/16-byte
// accesses and warp-shuffle reductions.  Intermediates are stored in the input dtype.
//
// Data layout in HBM (M = B*N*N pixels, NN = N*N):
//   z, u, dy, dgo, du, dz   pixel-major   [M, 128]
//   dPG                     pixel-major   [M, 512], columns [dP_a | dG_a | dP_b | dG_b]
//   a, b, t, dt, da, db     channel-major [B, 128, N, N]: one N x N plane per channel, so the per-channel
//                           contraction is a plain batched GEMM and both directions (and all four
//                           backward products) differ only in which operand is read K-major / MN-major.
//
// forward : ln_rows -> GEMM[z Wcat^T | gate-in epilogue -> a,b] -> GEMM[contraction -> t] -> ln_cm -> u
//           -> GEMM[u Wo^T | z Wgo^T, gate-out epilogue -> out]
// backward: GEMM[gate-out bwd epilogue -> dy,dgo] -> split-K GEMMs dWo,dWgo -> GEMM du -> ln_cm_bwd -> dt
//           -> 2 contraction GEMMs -> GEMM[z Wcat^T | gate-in bwd epilogue -> dPG] -> split-K GEMM dWcat
//           -> GEMM[dPG Wcat + dgo Wgo -> dz] -> ln_rows_bwd -> dx
// Math follows trimul_torch (geometric_nn_ops_torch/triangle/_reference/trimul.py:57-97).
#include <algorithm>
#include <cstdlib>

#include "tc_gemm.cuh"
#include "tc_paths.cuh"

namespace tri {
namespace tc {

namespace {

constexpr int CW = 128;        // channel width this path is built for
constexpr int kPersist = 592;  // blocks of the persistent memory-bound kernels (4 per SM)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]) {
  if constexpr (sizeof(T) == 4) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    union { uint2 u; T h[4]; } pk;
    pk.u = *reinterpret_cast<const uint2*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = to_f32(pk.h[i]);
  }
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
    union { uint2 u; T h[4]; } pk;
#pragma unroll
    for (int i = 0; i < 4; ++i) pk.h[i] = from_f32<T>(v[i]);
    *reinterpret_cast<uint2*>(p) = pk.u;
  }
}

// ---------------------------------------------------------------------------------------------
// weight preparation: Wcat rows [Wp_a; Wg_a; Wp_b; Wg_b], fp32 bias vectors in accumulator-column order
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void prep_weights_kernel(const T* wp, const T* wg, const T* bp, const T* bg, const T* bo, const T* bgo,
                                    T* wcat, float* bias_cat, float* bias_out) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < 4 * CW * CW) {
    const int r = idx / CW, k = idx % CW, blk = r / CW, c = r % CW;
    const T* src = (blk & 1) ? wg : wp;
    wcat[idx] = src[((blk >> 1) * CW + c) * CW + k];
  }
  if (idx < 4 * CW) {
    const int blk = idx / CW, c = idx % CW;
    const T* src = (blk & 1) ? bg : bp;
    bias_cat[idx] = src ? to_f32(src[(blk >> 1) * CW + c]) : 0.f;
  }
  if (idx < 2 * CW) {
    const T* src = idx < CW ? bo : bgo;
    bias_out[idx] = src ? to_f32(src[idx % CW]) : 0.f;
  }
}

// ---------------------------------------------------------------------------------------------
// LayerNorm over pixel-major rows (x -> z)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) ln_rows_kernel(const T* x, const T* gamma, const T* beta, float eps,
                                                       long long M, T* z, float* mean, float* rstd) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= M) return;
  float v[4];
  load4(x + row * CW + lane * 4, v);
  const float mu = warp_sum(v[0] + v[1] + v[2] + v[3]) * (1.0f / CW);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[i] -= mu; q += v[i] * v[i]; }
  const float rs = 1.0f / sqrtf(warp_sum(q) * (1.0f / CW) + eps);
  float gm[4] = {1.f, 1.f, 1.f, 1.f}, bt[4] = {0.f, 0.f, 0.f, 0.f};
  if (gamma) load4(gamma + lane * 4, gm);
  if (beta) load4(beta + lane * 4, bt);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = v[i] * rs * gm[i] + bt[i];
  store4(z + row * CW + lane * 4, v);
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
}

// dx = rstd * (dhat - mean(dhat) - xhat * mean(dhat*xhat)); per-block partial dgamma / dbeta
template <typename T>
__global__ void __launch_bounds__(256) ln_rows_bwd_kernel(const T* dz, const T* x, const float* mean,
                                                           const float* rstd, const T* gamma, long long M, T* dx,
                                                           float* pg, float* pb) {
  __shared__ float sg[8][CW], sb[8][CW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float gm[4] = {1.f, 1.f, 1.f, 1.f};
  if (gamma) load4(gamma + lane * 4, gm);
  float ag[4] = {}, ab[4] = {};
  for (long long row = blockIdx.x * 8LL + warp; row < M; row += gridDim.x * 8LL) {
    float xv[4], dv[4];
    load4(x + row * CW + lane * 4, xv);
    load4(dz + row * CW + lane * 4, dv);
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f, dh[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xv[i] = (xv[i] - mu) * rs;
      dh[i] = dv[i] * gm[i];
      s1 += dh[i];
      s2 += dh[i] * xv[i];
      ag[i] += dv[i] * xv[i];
      ab[i] += dv[i];
    }
    s1 = warp_sum(s1) * (1.0f / CW);
    s2 = warp_sum(s2) * (1.0f / CW);
#pragma unroll
    for (int i = 0; i < 4; ++i) dh[i] = rs * (dh[i] - s1 - xv[i] * s2);
    store4(dx + row * CW + lane * 4, dh);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) { sg[warp][lane * 4 + i] = ag[i]; sb[warp][lane * 4 + i] = ab[i]; }
  __syncthreads();
  if (threadIdx.x < CW) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { g += sg[w][threadIdx.x]; b += sb[w][threadIdx.x]; }
    pg[blockIdx.x * CW + threadIdx.x] = g;
    pb[blockIdx.x * CW + threadIdx.x] = b;
  }
}

// ---------------------------------------------------------------------------------------------
// LayerNorm over channels of a channel-major tensor (t -> u pixel-major), and its backward (du -> dt)
// ---------------------------------------------------------------------------------------------
constexpr int TP = 64;  // pixels per tile

template <typename T>
__device__ __forceinline__ void load_cm_tile(float (*tile)[TP + 1], const T* src, long long m0, long long M,
                                             long long NN) {
  const int pl = threadIdx.x & (TP - 1);
  const long long m = m0 + pl;
  const long long bb = m / NN, pix = m % NN;
  for (int c = threadIdx.x / TP; c < CW; c += 256 / TP)
    tile[c][pl] = m < M ? to_f32(src[(bb * CW + c) * NN + pix]) : 0.f;
}

template <typename T>
__global__ void __launch_bounds__(256) ln_cm_kernel(const T* t_cm, const T* gamma, const T* beta, float eps,
                                                     long long M, long long NN, T* u, float* mean, float* rstd) {
  __shared__ float tile[CW][TP + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float gm[4], bt[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    gm[k] = gamma ? to_f32(gamma[lane + 32 * k]) : 1.f;
    bt[k] = beta ? to_f32(beta[lane + 32 * k]) : 0.f;
  }
  const long long tiles = (M + TP - 1) / TP;
  for (long long tl = blockIdx.x; tl < tiles; tl += gridDim.x) {
    const long long m0 = tl * TP;
    __syncthreads();
    load_cm_tile(tile, t_cm, m0, M, NN);
    __syncthreads();
    for (int pl = warp; pl < TP; pl += 8) {
      const long long m = m0 + pl;
      if (m >= M) break;
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = tile[lane + 32 * k][pl];
      const float mu = warp_sum(v[0] + v[1] + v[2] + v[3]) * (1.0f / CW);
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) { v[k] -= mu; q += v[k] * v[k]; }
      const float rs = 1.0f / sqrtf(warp_sum(q) * (1.0f / CW) + eps);
#pragma unroll
      for (int k = 0; k < 4; ++k) u[m * CW + lane + 32 * k] = from_f32<T>(v[k] * rs * gm[k] + bt[k]);
      if (lane == 0) { mean[m] = mu; rstd[m] = rs; }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ln_cm_bwd_kernel(const T* du, const T* t_cm, const float* mean,
                                                         const float* rstd, const T* gamma, long long M,
                                                         long long NN, T* dt_cm, float* pg, float* pb) {
  __shared__ float tile[CW][TP + 1];
  __shared__ float sg[8][CW], sb[8][CW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float gm[4], ag[4] = {}, ab[4] = {};
#pragma unroll
  for (int k = 0; k < 4; ++k) gm[k] = gamma ? to_f32(gamma[lane + 32 * k]) : 1.f;
  const long long tiles = (M + TP - 1) / TP;
  for (long long tl = blockIdx.x; tl < tiles; tl += gridDim.x) {
    const long long m0 = tl * TP;
    __syncthreads();
    load_cm_tile(tile, t_cm, m0, M, NN);
    __syncthreads();
    for (int pl = warp; pl < TP; pl += 8) {
      const long long m = m0 + pl;
      if (m >= M) break;
      const float mu = mean[m], rs = rstd[m];
      float th[4], dh[4], s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        th[k] = (tile[lane + 32 * k][pl] - mu) * rs;
        const float d = to_f32(du[m * CW + lane + 32 * k]);
        dh[k] = d * gm[k];
        s1 += dh[k];
        s2 += dh[k] * th[k];
        ag[k] += d * th[k];
        ab[k] += d;
      }
      s1 = warp_sum(s1) * (1.0f / CW);
      s2 = warp_sum(s2) * (1.0f / CW);
#pragma unroll
      for (int k = 0; k < 4; ++k) tile[lane + 32 * k][pl] = rs * (dh[k] - s1 - th[k] * s2);
    }
    __syncthreads();
    {
      const int pl = threadIdx.x & (TP - 1);
      const long long m = m0 + pl;
      const long long bb = m / NN, pix = m % NN;
      if (m < M)
        for (int c = threadIdx.x / TP; c < CW; c += 256 / TP) dt_cm[(bb * CW + c) * NN + pix] = from_f32<T>(tile[c][pl]);
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) { sg[warp][lane + 32 * k] = ag[k]; sb[warp][lane + 32 * k] = ab[k]; }
  __syncthreads();
  if (threadIdx.x < CW) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { g += sg[w][threadIdx.x]; b += sb[w][threadIdx.x]; }
    pg[blockIdx.x * CW + threadIdx.x] = g;
    pb[blockIdx.x * CW + threadIdx.x] = b;
  }
}

// ---------------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------------
// partial[blockIdx.x][w] = column sums of this block's rows of X [M, W]
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(const T* X, long long M, int W, float* partial) {
  const long long per = (M + gridDim.x - 1) / gridDim.x;
  const long long r0 = blockIdx.x * per, r1 = min(M, r0 + per);
  for (int c = threadIdx.x; c < W; c += 256) {
    float s = 0.f;
    for (long long r = r0; r < r1; ++r) s += to_f32(X[r * W + c]);
    partial[(long long)blockIdx.x * W + c] = s;
  }
}

__global__ void reduce_kernel(const float* partial, int nparts, int n, float* out) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * n + j];
  out[j] = s;
}

// Sum partials of a [512, rowlen] tensor in Wcat row order and scatter the rows to the p_in / g_in gradients.
__global__ void reduce_wcat_kernel(const float* partial, int nparts, int rowlen, float* d_p, float* d_g) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = 4 * CW * rowlen;
  if (j >= n) return;
  const int r = j / rowlen, k = j % rowlen, blk = r / CW, c = r % CW;
  float* dst = (blk & 1) ? d_g : d_p;
  if (dst == nullptr) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * n + j];
  dst[((blk >> 1) * CW + c) * rowlen + k] = s;
}

// ---------------------------------------------------------------------------------------------
// memory plan
// ---------------------------------------------------------------------------------------------
struct Prep { int* err; void* wcat; float* bias_cat; float* bias_out; };
struct SavedT { void *z, *a, *b, *t, *u; float *mean_in, *rstd_in, *mean_out, *rstd_out; };

size_t es_of(const TriMulDesc* d) { return d->dtype == TRI_F32 ? 4 : 2; }

void carve_prep(Arena& a, const TriMulDesc* d, Prep* p) {
  p->err = a.take<int>(64);
  p->wcat = a.take<char>(4 * CW * CW * es_of(d));
  p->bias_cat = a.take<float>(4 * CW);
  p->bias_out = a.take<float>(2 * CW);
}

void carve_saved(Arena& a, const TriMulDesc* d, SavedT* s) {
  const size_t M = (size_t)d->B * d->N * d->N, unit = M * CW * es_of(d);
  s->z = a.take<char>(unit); s->a = a.take<char>(unit); s->b = a.take<char>(unit);
  s->t = a.take<char>(unit); s->u = a.take<char>(unit);
  s->mean_in = a.take<float>(M); s->rstd_in = a.take<float>(M);
  s->mean_out = a.take<float>(M); s->rstd_out = a.take<float>(M);
}

constexpr int kSplitK = 148;

struct BwdBufs { void *dy, *dgo, *du, *dt, *da, *db, *dpg, *dz; float* partial; };
void carve_bwd(Arena& a, const TriMulDesc* d, BwdBufs* w) {
  const size_t M = (size_t)d->B * d->N * d->N, unit = M * CW * es_of(d);
  w->dy = a.take<char>(unit); w->dgo = a.take<char>(unit); w->du = a.take<char>(unit);
  w->dt = a.take<char>(unit); w->da = a.take<char>(unit); w->db = a.take<char>(unit);
  w->dpg = a.take<char>(4 * unit); w->dz = a.take<char>(unit);
  w->partial = a.take<float>(std::max((size_t)kSplitK * 4 * CW * CW, (size_t)2 * kPersist * 4 * CW));
}

Operand rows_operand(const void* p, int width, long long rows, bool as_mn) {
  // pixel-major [rows, width]: K-major with K = width, or MN-major with MN = width and K = rows
  Operand o;
  o.ptr = p; o.mn_major = as_mn; o.inner = width; o.outer = rows; o.batch = 1; o.st_outer = width; o.st_batch = 0;
  return o;
}

Operand plane_operand(const void* p, int n, int planes, bool mn) {
  Operand o;
  o.ptr = p; o.mn_major = mn; o.inner = n; o.outer = n; o.batch = planes; o.st_outer = n; o.st_batch = (uint64_t)n * n;
  return o;
}

int contraction(cudaStream_t st, const TriMulDesc* d, const void* a, bool a_mn, const void* b, bool b_mn, void* out,
                int* err, const char* name) {
  GemmPlan p;
  const int planes = d->B * CW, n = d->N;
  p.a[0] = plane_operand(a, n, planes, a_mn);
  p.b[0] = plane_operand(b, n, planes, b_mn);
  p.M = n; p.N = n; p.K0 = n; p.batches = planes;
  p.out0 = out; p.ld_out = n; p.batch_out = (long long)n * n;
  p.name = name;
  p.flops = 2.0 * planes * n * (double)n * n;
  p.bytes = 3.0 * planes * (double)n * n * es_of(d);
  return launch_gemm(st, d->dtype, EPI_STORE, n > 128 ? 256 : 128, false, p, err);
}

template <typename T>
int run_prep(cudaStream_t st, const TriMulWeights* w, const Prep& pr) {
  TRI_CUDA_OK(cudaMemsetAsync(pr.err, 0, 256, st));
  KernelTimer kt("tc_prep_weights", st, 0.0, 0.0);
  prep_weights_kernel<T><<<cdiv(4 * CW * CW, 256), 256, 0, st>>>(
      (const T*)w->p_in_w, (const T*)w->g_in_w, (const T*)w->p_in_b, (const T*)w->g_in_b, (const T*)w->p_out_b,
      (const T*)w->g_out_b, (T*)pr.wcat, pr.bias_cat, pr.bias_out);
  TRI_LAUNCH_OK();
  return 0;
}

template <typename T>
int forward_t(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out, void* saved,
              void* ws, size_t ws_size, cudaStream_t st) {
  const long long M = (long long)d->B * d->N * d->N, NN = (long long)d->N * d->N;
  const double unit = (double)M * CW * sizeof(T);
  Arena a(ws, ws_size);
  Prep pr;
  carve_prep(a, d, &pr);
  SavedT s;
  if (saved) { Arena sa(saved, mul_saved_bytes(d)); carve_saved(sa, d, &s); }
  else carve_saved(a, d, &s);
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul forward workspace too small: need %zu, got %zu", a.off, ws_size);
  TRI_TRY(run_prep<T>(st, w, pr));
  const bool in_bias = w->p_in_b || w->g_in_b, out_bias = w->p_out_b || w->g_out_b;
  {
    KernelTimer kt("tc_ln_rows", st, 0.0, 2.0 * unit);
    ln_rows_kernel<T><<<cdiv(M, 8), 256, 0, st>>>((const T*)x, (const T*)w->norm_in_w, (const T*)w->norm_in_b, d->eps,
                                                  M, (T*)s.z, s.mean_in, s.rstd_in);
    TRI_LAUNCH_OK();
  }
  {
    GemmPlan p;
    p.a[0] = rows_operand(s.z, CW, M, false);
    p.b[0] = rows_operand(pr.wcat, CW, 4 * CW, false);
    p.M = (int)M; p.N = 4 * CW; p.K0 = CW;
    p.out0 = s.a; p.out1 = s.b; p.bias0 = in_bias ? pr.bias_cat : nullptr; p.aux = mask; p.plane = NN;
    p.name = "tc_gemm_gate_in"; p.flops = 2.0 * M * CW * 4 * CW; p.bytes = 3.0 * unit;
    TRI_TRY(launch_gemm(st, d->dtype, EPI_GATE_IN, 256, false, p, pr.err));
  }
  const bool incoming = d->direction == TRI_INCOMING;
  TRI_TRY(contraction(st, d, s.a, incoming, s.b, incoming, s.t, pr.err, "tc_gemm_contract"));
  {
    KernelTimer kt("tc_ln_cm", st, 0.0, 2.0 * unit);
    ln_cm_kernel<T><<<kPersist, 256, 0, st>>>((const T*)s.t, (const T*)w->norm_out_w, (const T*)w->norm_out_b, d->eps,
                                              M, NN, (T*)s.u, s.mean_out, s.rstd_out);
    TRI_LAUNCH_OK();
  }
  {
    GemmPlan p;
    p.a[0] = rows_operand(s.u, CW, M, false);
    p.b[0] = rows_operand(w->p_out_w, CW, CW, false);
    p.a[1] = rows_operand(s.z, CW, M, false);
    p.b[1] = rows_operand(w->g_out_w, CW, CW, false);
    p.M = (int)M; p.N = 2 * CW; p.K0 = CW; p.K1 = CW; p.seg1_col = CW;
    p.out0 = out; p.bias0 = out_bias ? pr.bias_out : nullptr;
    p.name = "tc_gemm_gate_out"; p.flops = 2.0 * M * CW * 2 * CW; p.bytes = 3.0 * unit;
    TRI_TRY(launch_gemm(st, d->dtype, EPI_GATE_OUT, 256, false, p, pr.err));
  }
  return 0;
}

int split_k_grad(cudaStream_t st, const TriMulDesc* d, const void* lhs, int lhs_w, const void* rhs, long long M,
                 float* partial, int* err, const char* name, int* nparts) {
  // partial[s][lhs_w][128] = sum over the rows of split s of lhs[row][:]^T rhs[row][:]
  const int bke = d->dtype == TRI_F32 ? 32 : 64;
  int splits = (int)std::min<long long>(kSplitK, (M + bke - 1) / bke);
  long long kper = ((M + splits - 1) / splits + bke - 1) / bke * bke;
  splits = (int)((M + kper - 1) / kper);
  GemmPlan p;
  p.a[0] = rows_operand(lhs, lhs_w, M, true);
  p.b[0] = rows_operand(rhs, CW, M, true);
  p.M = lhs_w; p.N = CW; p.K0 = (int)kper; p.batches = splits; p.split_k = 1;
  p.out0 = partial; p.ld_out = CW; p.batch_out = (long long)lhs_w * CW;
  p.name = name; p.flops = 2.0 * M * lhs_w * CW; p.bytes = (double)M * (lhs_w + CW) * es_of(d);
  *nparts = splits;
  return launch_gemm(st, d->dtype, EPI_STORE, 128, true, p, err);
}

int reduce_to(cudaStream_t st, const float* partial, int nparts, int n, float* out) {
  KernelTimer kt("tc_reduce", st, 0.0, 4.0 * (nparts + 1) * n);
  reduce_kernel<<<cdiv(n, 256), 256, 0, st>>>(partial, nparts, n, out);
  TRI_LAUNCH_OK();
  return 0;
}

template <typename T>
int colsum_to(cudaStream_t st, const void* X, long long M, int W, float* partial, int* nparts) {
  const int blocks = (int)std::min<long long>(kPersist, M);
  KernelTimer kt("tc_colsum", st, 0.0, (double)M * W * sizeof(T));
  colsum_kernel<T><<<blocks, 256, 0, st>>>((const T*)X, M, W, partial);
  TRI_LAUNCH_OK();
  *nparts = blocks;
  return 0;
}

template <typename T>
int backward_t(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, const void* saved,
               const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws, size_t ws_size, cudaStream_t st) {
  const long long M = (long long)d->B * d->N * d->N, NN = (long long)d->N * d->N;
  const double unit = (double)M * CW * sizeof(T);
  Arena a(ws, ws_size);
  Prep pr;
  carve_prep(a, d, &pr);
  BwdBufs b;
  carve_bwd(a, d, &b);
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul backward workspace too small: need %zu, got %zu", a.off, ws_size);
  SavedT s;
  { Arena sa(const_cast<void*>(saved), mul_saved_bytes(d)); carve_saved(sa, d, &s); }
  TRI_TRY(run_prep<T>(st, w, pr));
  const bool in_bias = w->p_in_b || w->g_in_b, out_bias = w->p_out_b || w->g_out_b;
  int nparts = 0;

  // output gate: dy = d_out * sig(go), dgo = d_out * y * sig * (1 - sig), with y and go recomputed
  {
    GemmPlan p;
    p.a[0] = rows_operand(s.u, CW, M, false);
    p.b[0] = rows_operand(w->p_out_w, CW, CW, false);
    p.a[1] = rows_operand(s.z, CW, M, false);
    p.b[1] = rows_operand(w->g_out_w, CW, CW, false);
    p.M = (int)M; p.N = 2 * CW; p.K0 = CW; p.K1 = CW; p.seg1_col = CW;
    p.out0 = b.dy; p.out1 = b.dgo; p.aux = d_out; p.bias0 = out_bias ? pr.bias_out : nullptr;
    p.name = "tc_gemm_gate_out_bwd"; p.flops = 0.0; p.bytes = 5.0 * unit;  // recompute: no algorithmic flops
    TRI_TRY(launch_gemm(st, d->dtype, EPI_GATE_OUT_BWD, 256, false, p, pr.err));
  }
  if (g->p_out_w) {
    TRI_TRY(split_k_grad(st, d, b.dy, CW, s.u, M, b.partial, pr.err, "tc_gemm_wgrad", &nparts));
    TRI_TRY(reduce_to(st, b.partial, nparts, CW * CW, g->p_out_w));
  }
  if (g->g_out_w) {
    TRI_TRY(split_k_grad(st, d, b.dgo, CW, s.z, M, b.partial, pr.err, "tc_gemm_wgrad", &nparts));
    TRI_TRY(reduce_to(st, b.partial, nparts, CW * CW, g->g_out_w));
  }
  if (g->p_out_b) {
    TRI_TRY(colsum_to<T>(st, b.dy, M, CW, b.partial, &nparts));
    TRI_TRY(reduce_to(st, b.partial, nparts, CW, g->p_out_b));
  }
  if (g->g_out_b) {
    TRI_TRY(colsum_to<T>(st, b.dgo, M, CW, b.partial, &nparts));
    TRI_TRY(reduce_to(st, b.partial, nparts, CW, g->g_out_b));
  }
  // du = dy Wo
  {
    GemmPlan p;
    p.a[0] = rows_operand(b.dy, CW, M, false);
    p.b[0] = rows_operand(w->p_out_w, CW, CW, true);  // B(n = ch, k = c) = Wo[c][ch]: n contiguous
    p.M = (int)M; p.N = CW; p.K0 = CW; p.out0 = b.du; p.ld_out = CW;
    p.name = "tc_gemm_du"; p.flops = 2.0 * M * CW * CW; p.bytes = 2.0 * unit;
    TRI_TRY(launch_gemm(st, d->dtype, EPI_STORE, 128, false, p, pr.err));
  }
  {
    float* pg = b.partial;
    float* pb = b.partial + (size_t)kPersist * CW;
    {
      KernelTimer kt("tc_ln_cm_bwd", st, 0.0, 3.0 * unit);
      ln_cm_bwd_kernel<T><<<kPersist, 256, 0, st>>>((const T*)b.du, (const T*)s.t, s.mean_out, s.rstd_out,
                                                    (const T*)w->norm_out_w, M, NN, (T*)b.dt, pg, pb);
      TRI_LAUNCH_OK();
    }
    if (g->norm_out_w) TRI_TRY(reduce_to(st, pg, kPersist, CW, g->norm_out_w));
    if (g->norm_out_b) TRI_TRY(reduce_to(st, pb, kPersist, CW, g->norm_out_b));
  }
  // contraction backward (operand majors per direction; see the header comment)
  if (d->direction == TRI_OUTGOING) {
    TRI_TRY(contraction(st, d, b.dt, false, s.b, true, b.da, pr.err, "tc_gemm_contract_bwd"));  // da[i,k] = sum_j dt[i,j] b[j,k]
    TRI_TRY(contraction(st, d, b.dt, true, s.a, true, b.db, pr.err, "tc_gemm_contract_bwd"));   // db[j,k] = sum_i dt[i,j] a[i,k]
  } else {
    TRI_TRY(contraction(st, d, s.b, false, b.dt, false, b.da, pr.err, "tc_gemm_contract_bwd")); // da[k,i] = sum_j b[k,j] dt[i,j]
    TRI_TRY(contraction(st, d, s.a, false, b.dt, true, b.db, pr.err, "tc_gemm_contract_bwd"));  // db[k,j] = sum_i a[k,i] dt[i,j]
  }
  // input gate backward fused into the recomputed projection GEMM
  {
    GemmPlan p;
    p.a[0] = rows_operand(s.z, CW, M, false);
    p.b[0] = rows_operand(pr.wcat, CW, 4 * CW, false);
    p.M = (int)M; p.N = 4 * CW; p.K0 = CW;
    p.out0 = b.dpg; p.ld_out = 4 * CW; p.bias0 = in_bias ? pr.bias_cat : nullptr;
    p.aux = mask; p.aux2 = b.da; p.aux3 = b.db; p.plane = NN;
    p.name = "tc_gemm_gate_in_bwd"; p.flops = 0.0; p.bytes = 7.0 * unit;
    TRI_TRY(launch_gemm(st, d->dtype, EPI_GATE_IN_BWD, 256, false, p, pr.err));
  }
  if (g->p_in_w || g->g_in_w) {
    TRI_TRY(split_k_grad(st, d, b.dpg, 4 * CW, s.z, M, b.partial, pr.err, "tc_gemm_wgrad", &nparts));
    KernelTimer kt("tc_reduce", st, 0.0, 4.0 * (nparts + 1) * 4 * CW * CW);
    reduce_wcat_kernel<<<cdiv(4 * CW * CW, 256), 256, 0, st>>>(b.partial, nparts, CW, g->p_in_w, g->g_in_w);
    TRI_LAUNCH_OK();
  }
  if (g->p_in_b || g->g_in_b) {
    TRI_TRY(colsum_to<T>(st, b.dpg, M, 4 * CW, b.partial, &nparts));
    KernelTimer kt("tc_reduce", st, 0.0, 4.0 * (nparts + 1) * 4 * CW);
    reduce_wcat_kernel<<<cdiv(4 * CW, 256), 256, 0, st>>>(b.partial, nparts, 1, g->p_in_b, g->g_in_b);
    TRI_LAUNCH_OK();
  }
  // dz = dPG Wcat + dgo Wgo
  {
    GemmPlan p;
    p.a[0] = rows_operand(b.dpg, 4 * CW, M, false);
    p.b[0] = rows_operand(pr.wcat, CW, 4 * CW, true);   // B(n = c, k = row of Wcat): n contiguous
    p.a[1] = rows_operand(b.dgo, CW, M, false);
    p.b[1] = rows_operand(w->g_out_w, CW, CW, true);
    p.M = (int)M; p.N = CW; p.K0 = 4 * CW; p.K1 = CW; p.seg1_col = 0;
    p.out0 = b.dz; p.ld_out = CW;
    p.name = "tc_gemm_dz"; p.flops = 2.0 * M * CW * 5 * CW; p.bytes = 6.0 * unit;
    TRI_TRY(launch_gemm(st, d->dtype, EPI_STORE, 128, false, p, pr.err));
  }
  {
    const int blocks = (int)std::min<long long>(kPersist, (M + 7) / 8);
    float* pg = b.partial;
    float* pb = b.partial + (size_t)kPersist * CW;
    {
      KernelTimer kt("tc_ln_rows_bwd", st, 0.0, 3.0 * unit);
      ln_rows_bwd_kernel<T><<<blocks, 256, 0, st>>>((const T*)b.dz, (const T*)x, s.mean_in, s.rstd_in,
                                                    (const T*)w->norm_in_w, M, (T*)dx, pg, pb);
      TRI_LAUNCH_OK();
    }
    if (g->norm_in_w) TRI_TRY(reduce_to(st, pg, blocks, CW, g->norm_in_w));
    if (g->norm_in_b) TRI_TRY(reduce_to(st, pb, blocks, CW, g->norm_in_b));
  }
  return 0;
}

bool forced_simt() {
  const char* e = getenv("TRI_B200_FORCE_SIMT");
  return e != nullptr && e[0] == '1';
}

}  // namespace

bool mul_supported(const TriMulDesc* d) {
  if (forced_simt()) return false;
  if (d->C != CW || d->Ch != CW) return false;
  if (d->dtype == TRI_F32 && d->precision != TRI_PREC_TF32) return false;  // exact fp32 has no tensor-core form
  if (d->N % 8 != 0) return false;                                          // TMA strides: multiples of 16 bytes
  return true;
}

size_t mul_saved_bytes(const TriMulDesc* d) {
  Arena a(nullptr, 0);
  SavedT s;
  carve_saved(a, d, &s);
  return a.off;
}

size_t mul_ws_bytes(const TriMulDesc* d, int is_bwd) {
  Arena a(nullptr, 0);
  Prep p;
  carve_prep(a, d, &p);
  if (is_bwd) { BwdBufs b; carve_bwd(a, d, &b); }
  else { SavedT s; carve_saved(a, d, &s); }
  return a.off + 256;
}

int mul_forward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out, void* saved,
                void* ws, size_t ws_size, cudaStream_t st) {
  switch (d->dtype) {
    case TRI_F32: return forward_t<float>(d, x, mask, w, out, saved, ws, ws_size, st);
    case TRI_BF16: return forward_t<__nv_bfloat16>(d, x, mask, w, out, saved, ws, ws_size, st);
    case TRI_F16: return forward_t<__half>(d, x, mask, w, out, saved, ws, ws_size, st);
  }
  return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
}

int mul_backward(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, const void* saved,
                 const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws, size_t ws_size, cudaStream_t st) {
  switch (d->dtype) {
    case TRI_F32: return backward_t<float>(d, x, mask, w, saved, d_out, dx, g, ws, ws_size, st);
    case TRI_BF16: return backward_t<__nv_bfloat16>(d, x, mask, w, saved, d_out, dx, g, ws, ws_size, st);
    case TRI_F16: return backward_t<__half>(d, x, mask, w, saved, d_out, dx, g, ws, ws_size, st);
  }
  return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
}

}  // namespace tc
}  // namespace tri
