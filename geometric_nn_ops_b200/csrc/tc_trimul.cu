// Tensor-core path of the triangle multiplicative update (C_z = C_hidden = 128), forward and backward.
//
// Every product runs on tcgen05 through tc_gemm (bf16 / fp16 operands, or tf32 for fp32 inputs with
// precision "tf32"); LayerNorm, transposes and reductions are memory-bound kernels with 8/16-byte
// accesses and warp-shuffle reductions.  Intermediates are stored in the input dtype.
//
// Data layout in HBM (M = B*N*N pixels, NN = N*N):
//   z, u, dy, dgo, du, dz   pixel-major   [M, 128]
//   dPG                     channel-major [512, M], rows [dP_a | dG_a | dP_b | dG_b]
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
#include <initializer_list>

#include "tc_gemm.cuh"
#include "tc_lngemm.cuh"
#include "tc_paths.cuh"

namespace tri {
namespace tc {

namespace {

constexpr int CW = 128;        // channel width this path is built for
constexpr int kPersist = 592;  // blocks of the persistent memory-bound kernels (4 per SM)
constexpr int kLnCmBlocks = 592;    // ln_cm: 4 per SM (64 registers per thread hold the next tile's loads)
constexpr int kLnCmBwdBlocks = 444; // ln_cm_bwd: 3 per SM (80 registers: next tile, eight pixels' gradients and statistics)

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
template <typename T> __device__ __forceinline__ void load8v(const T* p, float (&v)[8]) {
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
template <typename T> __device__ __forceinline__ void store8v(T* p, const float (&v)[8]) {
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

// A row of 128 channels is held by 16 lanes (8 channels, one 16-byte access each), so a warp covers two rows per
// access and keeps several row pairs in flight: with one 8-byte access per thread these kernels were bound by
// load latency (3.0 of 6.6 TB/s).
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
constexpr int kLnRowPairs = 4;   // row pairs per warp and pass (8 rows)

template <typename T>
__global__ void __launch_bounds__(256) ln_rows_kernel(const T* __restrict__ x, const T* gamma, const T* beta, float eps,
                                                       long long M, T* __restrict__ z, float* mean, float* rstd) {
  const int lane = threadIdx.x & 31, sub = lane & 15, half = lane >> 4;
  const long long row0 = (blockIdx.x * 8LL + (threadIdx.x >> 5)) * (2 * kLnRowPairs) + half;
  float gm[8], bt[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { gm[i] = 1.f; bt[i] = 0.f; }
  if (gamma) load8v(gamma + sub * 8, gm);
  if (beta) load8v(beta + sub * 8, bt);
  float v[kLnRowPairs][8];
#pragma unroll
  for (int p = 0; p < kLnRowPairs; ++p) {
    const long long row = row0 + 2 * p;
    if (row < M) load8v(x + row * CW + sub * 8, v[p]);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[p][i] = 0.f;
    }
  }
#pragma unroll
  for (int p = 0; p < kLnRowPairs; ++p) {
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
    if (row < M) {
      store8v(z + row * CW + sub * 8, v[p]);
      if (sub == 0) { mean[row] = mu; rstd[row] = rs; }
    }
  }
}

// dx = rstd * (dhat - mean(dhat) - xhat * mean(dhat*xhat)); per-block partial dgamma / dbeta
template <typename T>
__global__ void __launch_bounds__(256, 4) ln_rows_bwd_kernel(const T* __restrict__ dz, const T* __restrict__ x,
                                                           const float* __restrict__ mean, const float* __restrict__ rstd,
                                                           const T* gamma, long long M, T* __restrict__ dx, float* pg,
                                                           float* pb) {
  __shared__ float sg[16][CW], sb[16][CW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 15, half = lane >> 4;
  constexpr int RP = 1;   // row pairs per warp and pass (more would cost the registers of a fourth resident block)
  float gm[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) gm[i] = 1.f;
  if (gamma) load8v(gamma + sub * 8, gm);
  float ag[8] = {}, ab[8] = {};
  for (long long base = (blockIdx.x * 8LL + warp) * (2 * RP); base < M; base += gridDim.x * 8LL * (2 * RP)) {
    float xv[RP][8], dv[RP][8], mu[RP], rs[RP];
#pragma unroll
    for (int p = 0; p < RP; ++p) {
      const long long row = base + 2 * p + half;
      if (row < M) {
        load8v(x + row * CW + sub * 8, xv[p]);
        load8v(dz + row * CW + sub * 8, dv[p]);
        mu[p] = mean[row]; rs[p] = rstd[row];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) { xv[p][i] = 0.f; dv[p][i] = 0.f; }
        mu[p] = 0.f; rs[p] = 0.f;
      }
    }
#pragma unroll
    for (int p = 0; p < RP; ++p) {
      const long long row = base + 2 * p + half;
      float s1 = 0.f, s2 = 0.f, dh[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xv[p][i] = (xv[p][i] - mu[p]) * rs[p];
        dh[i] = dv[p][i] * gm[i];
        s1 += dh[i];
        s2 += dh[i] * xv[p][i];
        ag[i] += dv[p][i] * xv[p][i];
        ab[i] += dv[p][i];
      }
      s1 = half_warp_sum(s1) * (1.0f / CW);
      s2 = half_warp_sum(s2) * (1.0f / CW);
#pragma unroll
      for (int i = 0; i < 8; ++i) dh[i] = rs[p] * (dh[i] - s1 - xv[p][i] * s2);
      if (row < M) store8v(dx + row * CW + sub * 8, dh);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) { sg[warp * 2 + half][sub * 8 + i] = ag[i]; sb[warp * 2 + half][sub * 8 + i] = ab[i]; }
  __syncthreads();
  if (threadIdx.x < CW) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < 16; ++w) { g += sg[w][threadIdx.x]; b += sb[w][threadIdx.x]; }
    pg[blockIdx.x * CW + threadIdx.x] = g;
    pb[blockIdx.x * CW + threadIdx.x] = b;
  }
}

// ---------------------------------------------------------------------------------------------
// LayerNorm over channels of a channel-major tensor (t -> u pixel-major), and its backward (du -> dt)
// ---------------------------------------------------------------------------------------------
constexpr int TP = 64;        // pixels per tile
constexpr int TROW = CW + 5;  // floats per tile row: 128 channels, one pad word after every 32, one more for the row

// The transposing tile lives in shared memory pixel-major, tile[pixel][channel], with two twists that make both
// sides free of bank conflicts (row stride 133 words = 5 mod 32):
//  * a pad word after every 32 channels: on the pixel-major side a warp reads one pixel, lane l channels 4l..4l+3,
//    one word per instruction; lanes l, l+8, l+16, l+24 would share a bank (4l mod 32), the pads shift them apart;
//  * the channel index of pixels 32..63 XOR-ed with 4: on the channel-major side a lane holds 8 consecutive pixels of
//    one channel and the 32 lanes of an access are 4 channels x 8 pixel groups; groups pg and pg + 4 would collide
//    (40 pg = 8 pg mod 32), the XOR moves the upper four onto the neighbouring channels' banks.
// The first version kept tile[channel][pixel + 1]: 2-way conflicts on one side and 4-way on the other held the LSU
// pipe at 85 % and these kernels at 2.5 TB/s.
__device__ __forceinline__ int tile_at(int pixel, int channel) {
  return pixel * TROW + (channel ^ ((pixel >> 5) << 2)) + (channel >> 5);
}

// 64 pixels x 128 channels of a channel-major tensor <-> smem tile (fp32), 8 pixels (16 or 32 bytes) per access, four
// accesses per thread.  The plane size is a multiple of 8 pixels, so a group of 8 never straddles two batch entries.
// The global loads of a tile are issued into registers (fetch_cm_tile) while the block still works on the previous
// tile and written to shared memory afterwards (put_cm_tile): with the loads issued at the top of a tile's own
// phase, a block had nothing in flight during its arithmetic and the kernels sat at 2.1-2.5 TB/s.
// four consecutive elements as raw words (converted when used)
template <typename T> struct Raw4 { uint32_t w[sizeof(T) == 4 ? 4 : 2]; };
template <typename T> __device__ __forceinline__ Raw4<T> ldraw4(const T* p) {
  Raw4<T> r;
  if constexpr (sizeof(T) == 4) {
    const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
    r.w[0] = t.x; r.w[1] = t.y; r.w[2] = t.z; r.w[3] = t.w;
  } else {
    const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
    r.w[0] = t.x; r.w[1] = t.y;
  }
  return r;
}
template <typename T> __device__ __forceinline__ void cvtraw4(const Raw4<T>& r, float (&v)[4]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r.w[i]);
  } else {
    union { uint2 u; T h[4]; } pk;
    pk.u = make_uint2(r.w[0], r.w[1]);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = to_f32(pk.h[i]);
  }
}

template <typename T> struct CmRegs { Raw8<T> v[4]; bool ok[4]; };   // raw 16-byte words: converted when written to the tile

template <typename T>
__device__ __forceinline__ void fetch_cm_tile(CmRegs<T>& r, const T* src, long long m0, long long M, long long NN) {
  const long long b0 = m0 / NN, p0 = m0 - b0 * NN;   // one division per tile, not one per access
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int item = threadIdx.x + k * 256;
    const int c = item / (TP / 8), pg = item % (TP / 8);
    const long long m = m0 + pg * 8;
    long long bb = b0, pix = p0 + pg * 8;
    while (pix >= NN) { pix -= NN; ++bb; }
    r.ok[k] = m < M;
    if (r.ok[k]) r.v[k] = ldraw8<T>(src + (bb * CW + c) * NN + pix);
  }
}
template <typename T>
__device__ __forceinline__ void put_cm_tile(float* tile, const CmRegs<T>& r) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int item = threadIdx.x + k * 256;
    const int c = item / (TP / 8), pg = item % (TP / 8);
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (r.ok[k]) cvtraw8<T>(r.v[k], v);
#pragma unroll
    for (int e = 0; e < 8; ++e) tile[tile_at(pg * 8 + e, c)] = v[e];
  }
}
template <typename T>
__device__ __forceinline__ void store_cm_tile(const float* tile, T* dst, long long m0, long long M, long long NN) {
  const long long b0 = m0 / NN, p0 = m0 - b0 * NN;
  for (int item = threadIdx.x; item < CW * (TP / 8); item += 256) {
    const int c = item / (TP / 8), pg = item % (TP / 8);
    const long long m = m0 + pg * 8;
    if (m >= M) continue;
    long long bb = b0, pix = p0 + pg * 8;
    while (pix >= NN) { pix -= NN; ++bb; }
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = tile[tile_at(pg * 8 + e, c)];
    store8v<T>(dst + (bb * CW + c) * NN + pix, v);
  }
}

// One warp per pixel; lane l owns channels 4l..4l+3, so the pixel-major side is read / written 8 or 16
// bytes per lane (256 or 512 contiguous bytes per warp).
template <typename T>
__global__ void __launch_bounds__(256, 4) ln_cm_kernel(const T* t_cm, const T* gamma, const T* beta, float eps,
                                                        long long M, long long NN, T* u, float* mean, float* rstd) {
  __shared__ float tile[TP * TROW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float gm[4] = {1.f, 1.f, 1.f, 1.f}, bt[4] = {0.f, 0.f, 0.f, 0.f};
  if (gamma) load4(gamma + lane * 4, gm);
  if (beta) load4(beta + lane * 4, bt);
  const long long tiles = (M + TP - 1) / TP;
  CmRegs<T> next;
  if ((long long)blockIdx.x < tiles) fetch_cm_tile(next, t_cm, (long long)blockIdx.x * TP, M, NN);
  for (long long tl = blockIdx.x; tl < tiles; tl += gridDim.x) {
    const long long m0 = tl * TP;
    __syncthreads();                       // the previous tile has been read out of shared memory
    put_cm_tile(tile, next);
    __syncthreads();
    if (tl + gridDim.x < tiles) fetch_cm_tile(next, t_cm, (tl + gridDim.x) * TP, M, NN);   // in flight during the arithmetic
    for (int pl = warp; pl < TP; pl += 8) {
      const long long m = m0 + pl;
      if (m >= M) break;
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = tile[tile_at(pl, lane * 4 + k)];
      const float mu = warp_sum(v[0] + v[1] + v[2] + v[3]) * (1.0f / CW);
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) { v[k] -= mu; q += v[k] * v[k]; }
      const float rs = 1.0f / sqrtf(warp_sum(q) * (1.0f / CW) + eps);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = v[k] * rs * gm[k] + bt[k];
      store4(u + m * CW + lane * 4, v);
      if (lane == 0) { mean[m] = mu; rstd[m] = rs; }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256, 3) ln_cm_bwd_kernel(const T* du, const T* t_cm, const float* mean,
                                                            const float* rstd, const T* gamma, long long M,
                                                            long long NN, T* dt_cm, float* pg, float* pb) {
  __shared__ float tile[TP * TROW];
  __shared__ float sg[8][CW], sb[8][CW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float gm[4] = {1.f, 1.f, 1.f, 1.f}, ag[4] = {}, ab[4] = {};
  if (gamma) load4(gamma + lane * 4, gm);
  const long long tiles = (M + TP - 1) / TP;
  CmRegs<T> next;
  if ((long long)blockIdx.x < tiles) fetch_cm_tile(next, t_cm, (long long)blockIdx.x * TP, M, NN);
  for (long long tl = blockIdx.x; tl < tiles; tl += gridDim.x) {
    const long long m0 = tl * TP;
    __syncthreads();                       // the previous tile has been stored from shared memory
    put_cm_tile(tile, next);
    // this warp's eight pixels: their upstream gradients and statistics, fetched together instead of one pixel at a
    // time in front of their use (eight exposed load latencies per tile)
    Raw4<T> d8[TP / 8];
    float mu8[TP / 8], rs8[TP / 8];
#pragma unroll
    for (int i = 0; i < TP / 8; ++i) {
      const long long m = m0 + warp + 8 * i;
      mu8[i] = 0.f; rs8[i] = 0.f;
      if (m < M) { d8[i] = ldraw4<T>(du + m * CW + lane * 4); mu8[i] = mean[m]; rs8[i] = rstd[m]; }
    }
    __syncthreads();
    if (tl + gridDim.x < tiles) fetch_cm_tile(next, t_cm, (tl + gridDim.x) * TP, M, NN);   // in flight during the arithmetic
#pragma unroll
    for (int i = 0; i < TP / 8; ++i) {
      const int pl = warp + 8 * i;
      if (m0 + pl >= M) break;
      const float mu = mu8[i], rs = rs8[i];
      float d[4], th[4], dh[4], s1 = 0.f, s2 = 0.f;
      cvtraw4<T>(d8[i], d);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        th[k] = (tile[tile_at(pl, lane * 4 + k)] - mu) * rs;
        dh[k] = d[k] * gm[k];
        s1 += dh[k];
        s2 += dh[k] * th[k];
        ag[k] += d[k] * th[k];
        ab[k] += d[k];
      }
      s1 = warp_sum(s1) * (1.0f / CW);
      s2 = warp_sum(s2) * (1.0f / CW);
#pragma unroll
      for (int k = 0; k < 4; ++k) tile[tile_at(pl, lane * 4 + k)] = rs * (dh[k] - s1 - th[k] * s2);
    }
    __syncthreads();
    store_cm_tile(tile, dt_cm, m0, M, NN);
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) { sg[warp][lane * 4 + k] = ag[k]; sb[warp][lane * 4 + k] = ab[k]; }
  __syncthreads();
  if (threadIdx.x < CW) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { g += sg[w][threadIdx.x]; b += sb[w][threadIdx.x]; }
    pg[blockIdx.x * CW + threadIdx.x] = g;
    pb[blockIdx.x * CW + threadIdx.x] = b;
  }
}

// The same backward with every tensor channel-major ([128][M]: du from the transposed du GEMM, t, dt): nothing is
// transposed.  A block of 256 threads takes 64 pixels; a thread holds 8 pixels (16 bytes of a channel row) of 4
// channels in registers, raw, for both passes.  A pixel's two sums over its 128 channels are combined from the 32
// channel parts through shared memory; the per-channel sums over pixels (gradients of the LayerNorm weight and bias)
// stay in the thread's registers across tiles, since its 4 channels never change.
constexpr int kLnCmCmBlocks = 296;   // 2 per SM (about 100 registers per thread)
template <typename T>
__global__ void __launch_bounds__(256, 2) ln_cm_bwd_cm_kernel(const T* __restrict__ du, const T* __restrict__ t,
                                                              const float* __restrict__ mean, const float* __restrict__ rstd,
                                                              const T* gamma, long long M, T* __restrict__ dt, float* pg,
                                                              float* pb) {
  static_assert(sizeof(T) == 2, "16-bit types");
  __shared__ __align__(16) float s_p1[32][64], s_p2[32][64], s_s1[64], s_s2[64];
  const int tid = threadIdx.x, pgp = tid & 7, kp = tid >> 3;   // 8-pixel group of the tile; 4-channel part
  float gm[4], dg[4] = {}, db[4] = {};
#pragma unroll
  for (int r = 0; r < 4; ++r) gm[r] = gamma ? to_f32(gamma[kp * 4 + r]) : 1.f;
  const long long tiles = (M + 63) / 64;
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const long long px0 = tile * 64 + pgp * 8;   // 8 pixels: all inside the tensor or none (M is a multiple of 8)
    const bool valid = px0 < M;
    uint4 tw[4], dw[4];
    float mu[8], rs[8];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      tw[r] = make_uint4(0, 0, 0, 0); dw[r] = tw[r];
      if (valid) {
        tw[r] = __ldg(reinterpret_cast<const uint4*>(t + (long long)(kp * 4 + r) * M + px0));
        dw[r] = __ldg(reinterpret_cast<const uint4*>(du + (long long)(kp * 4 + r) * M + px0));
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) { mu[e] = 0.f; rs[e] = 0.f; }
    if (valid) {
      const float4 a = *reinterpret_cast<const float4*>(mean + px0), b = *reinterpret_cast<const float4*>(mean + px0 + 4);
      const float4 c = *reinterpret_cast<const float4*>(rstd + px0), d = *reinterpret_cast<const float4*>(rstd + px0 + 4);
      mu[0] = a.x; mu[1] = a.y; mu[2] = a.z; mu[3] = a.w; mu[4] = b.x; mu[5] = b.y; mu[6] = b.z; mu[7] = b.w;
      rs[0] = c.x; rs[1] = c.y; rs[2] = c.z; rs[3] = c.w; rs[4] = d.x; rs[5] = d.y; rs[6] = d.z; rs[7] = d.w;
    }
    {
      float p1[8] = {}, p2[8] = {};
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        union { uint4 u; T h[8]; } xt, xd;
        xt.u = tw[r]; xd.u = dw[r];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = (to_f32(xt.h[e]) - mu[e]) * rs[e], gd = to_f32(xd.h[e]) * gm[r];
          p1[e] += gd;
          p2[e] = fmaf(gd, xh, p2[e]);
        }
      }
      float4* d1 = reinterpret_cast<float4*>(&s_p1[kp][pgp * 8]);
      float4* d2 = reinterpret_cast<float4*>(&s_p2[kp][pgp * 8]);
      d1[0] = make_float4(p1[0], p1[1], p1[2], p1[3]); d1[1] = make_float4(p1[4], p1[5], p1[6], p1[7]);
      d2[0] = make_float4(p2[0], p2[1], p2[2], p2[3]); d2[1] = make_float4(p2[4], p2[5], p2[6], p2[7]);
    }
    __syncthreads();
    if (tid < 128) {   // 64 pixels x 2 sums
      const int px = tid & 63;
      const float(*src)[64] = tid < 64 ? s_p1 : s_p2;
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int k = 0; k < 32; k += 2) { a += src[k][px]; b += src[k + 1][px]; }
      (tid < 64 ? s_s1 : s_s2)[px] = (a + b) * (1.0f / CW);
    }
    __syncthreads();
    {
      const float4 a = *reinterpret_cast<const float4*>(&s_s1[pgp * 8]), b = *reinterpret_cast<const float4*>(&s_s1[pgp * 8 + 4]);
      const float4 c = *reinterpret_cast<const float4*>(&s_s2[pgp * 8]), d = *reinterpret_cast<const float4*>(&s_s2[pgp * 8 + 4]);
      const float s1[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w}, s2[8] = {c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        union { uint4 u; T h[8]; } xt, xd, o;
        xt.u = tw[r]; xd.u = dw[r];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float dv = to_f32(xd.h[e]), xh = (to_f32(xt.h[e]) - mu[e]) * rs[e];
          o.h[e] = from_f32<T>(rs[e] * (dv * gm[r] - s1[e] - xh * s2[e]));
          dg[r] = fmaf(dv, xh, dg[r]);
          db[r] += dv;
        }
        if (valid) *reinterpret_cast<uint4*>(dt + (long long)(kp * 4 + r) * M + px0) = o.u;
      }
    }
  }
  // the 8 threads of a channel part are a quarter of a warp
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float a = dg[r], b = db[r];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
    if (pgp == 0) { pg[blockIdx.x * CW + kp * 4 + r] = a; pb[blockIdx.x * CW + kp * 4 + r] = b; }
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

// out[j] = sum_p partial[p][j].  64 outputs per block, four threads per output each summing every fourth
// partial; the four sub-sums are added in a fixed order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) reduce_kernel(const float* partial, int nparts, int n, float* out) {
  __shared__ float sub[4][64];
  const int o = threadIdx.x & 63, lane4 = threadIdx.x >> 6;
  const int j = blockIdx.x * 64 + o;
  float s = 0.f;
  if (j < n)
    for (int p = lane4; p < nparts; p += 4) s += partial[(long long)p * n + j];
  sub[lane4][o] = s;
  __syncthreads();
  if (lane4 == 0 && j < n) out[j] = (sub[0][o] + sub[1][o]) + (sub[2][o] + sub[3][o]);
}

// Up to six such reductions in one launch (blockIdx.y selects the job): the backward has groups of small reductions
// (weight gradients, LayerNorm weight and bias) whose launches cost more than their work.  A job with `rowlen` set
// sums partials of a [512, rowlen] tensor in Wcat row order and scatters its rows to the p_in (out) and g_in (out2)
// gradients; either may be null.
constexpr int kReduceJobs = 6;
struct ReduceJobs {
  const float* partial[kReduceJobs];
  float* out[kReduceJobs];
  float* out2[kReduceJobs];
  int nparts[kReduceJobs], n[kReduceJobs], rowlen[kReduceJobs];
};
// 32 outputs per block (one warp reads 128 contiguous bytes of a partial), 8 warps each summing every eighth
// partial with eight independent accumulators so that loads overlap (the first version walked 37 partials with one
// dependent load each: 16 us per launch of pure latency); the warps' sums are added in a fixed order, so the
// result does not depend on scheduling.
__global__ void __launch_bounds__(256) reduce_multi_kernel(const ReduceJobs jobs) {
  __shared__ float sub[8][32];
  const int job = blockIdx.y, n = jobs.n[job], nparts = jobs.nparts[job];
  if (blockIdx.x * 32 >= n) return;
  const float* partial = jobs.partial[job];
  const int o = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + o;
  float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (j < n) {
    int p = w;
    for (; p + 56 < nparts; p += 64) {   // eight independent loads in flight
#pragma unroll
      for (int u = 0; u < 8; ++u) a[u] += partial[(long long)(p + 8 * u) * n + j];
    }
    for (; p < nparts; p += 8) a[0] += partial[(long long)p * n + j];
  }
  sub[w][o] = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
  __syncthreads();
  if (w != 0 || j >= n) return;
  const float sum = ((sub[0][o] + sub[1][o]) + (sub[2][o] + sub[3][o])) + ((sub[4][o] + sub[5][o]) + (sub[6][o] + sub[7][o]));
  const int rowlen = jobs.rowlen[job];
  if (rowlen == 0) {
    jobs.out[job][j] = sum;
  } else {
    const int r = j / rowlen, k = j % rowlen, blk = r / CW, c = r % CW;
    float* dst = (blk & 1) ? jobs.out2[job] : jobs.out[job];
    if (dst != nullptr) dst[((blk >> 1) * CW + c) * rowlen + k] = sum;
  }
}

// Row sums of the channel-major dPG [512, M] scattered to the p_in / g_in bias gradients (one block per row,
// fixed summation order).
template <typename T>
__global__ void __launch_bounds__(256) rowsum_wcat_kernel(const T* dpg, long long M, float* d_p, float* d_g) {
  __shared__ float red[256];
  const int r = blockIdx.x, blk = r / CW, c = r % CW;
  float* dst = (blk & 1) ? d_g : d_p;
  float s = 0.f;
  for (long long i = threadIdx.x; i < M; i += 256) s += to_f32(dpg[(long long)r * M + i]);
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0 && dst != nullptr) dst[(blk >> 1) * CW + c] = red[0];
}

// ---------------------------------------------------------------------------------------------
// memory plan
// ---------------------------------------------------------------------------------------------
// Geometry of the pixel-wise phases: M pixels in all, `plane` pixels per batch entry (the stride between
// channel planes of a channel-major buffer).  For the single-GPU op plane = N*N; for a row shard
// plane = rows*N.  Nothing in these phases knows about the pair structure beyond that.
struct Geom {
  int dtype;
  float eps;
  long long M, plane;
  bool sharded = false;      // a row shard of a multi-GPU op (other streams' kernels run beside this one's)
  size_t es() const { return dtype == TRI_F32 ? 4 : 2; }
  double unit() const { return (double)M * CW * es(); }
};

struct Prep { int* err; void* wcat; float* bias_cat; float* bias_out; };

void carve_prep_weights(Arena& a, size_t es, Prep* p) {
  p->wcat = a.take<char>(4 * CW * CW * es);
  p->bias_cat = a.take<float>(4 * CW);
  p->bias_out = a.take<float>(2 * CW);
}
void carve_prep(Arena& a, size_t es, Prep* p) {
  p->err = a.take<int>(64);
  carve_prep_weights(a, es, p);
}

// The layout of the saved u = LayerNorm(t): channel-major [128, M] where the fused output kernel runs (it never
// transposes t), pixel-major [M, 128] otherwise.  Forward and backward decide from the same geometry.
bool u_channel_major(const Geom& gm) { return ln_gate_out_supported(gm.dtype, gm.M, gm.plane); }

constexpr int kSplitK = 148;
// The partials of one backward phase live side by side until the phase's single reduction launch: the split-K
// weight-gradient partials (dWcat, or dWo | dWgo) first, then the LayerNorm weight / bias partials.
constexpr size_t kWgradPartialFloats = (size_t)kSplitK * 4 * CW * CW;
constexpr size_t kLnPartialFloats = (size_t)2 * kPersist * CW;
size_t partial_floats() { return kWgradPartialFloats + kLnPartialFloats; }

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

// One N x N x N product per channel plane: out[p] = A[p] B[p]^T with the given operand majors.
int contraction(cudaStream_t st, int dtype, int planes, int n, const void* a, bool a_mn, const void* b, bool b_mn,
                void* out, int* err, const char* name) {
  GemmPlan p;
  p.a[0] = plane_operand(a, n, planes, a_mn);
  p.b[0] = plane_operand(b, n, planes, b_mn);
  p.M = n; p.N = n; p.K0 = n; p.batches = planes;
  p.out0 = out; p.ld_out = n; p.batch_out = (long long)n * n;
  p.name = name;
  p.flops = 2.0 * planes * n * (double)n * n;
  p.bytes = 3.0 * planes * (double)n * n * (dtype == TRI_F32 ? 4 : 2);
  return launch_gemm(st, dtype, EPI_STORE, n > 128 ? 256 : 128, false, p, err);
}

template <typename T>
int run_prep(cudaStream_t st, const TriMulWeights* w, const Prep& pr, bool weights_ready = false) {
  TRI_CUDA_OK(cudaMemsetAsync(pr.err, 0, 256, st));
  if (weights_ready) return 0;   // the caller kept the prepared weights of an earlier phase of the same call
  KernelTimer kt("tc_prep_weights", st, 0.0, 0.0);
  prep_weights_kernel<T><<<cdiv(4 * CW * CW, 256), 256, 0, st>>>(
      (const T*)w->p_in_w, (const T*)w->g_in_w, (const T*)w->p_in_b, (const T*)w->g_in_b, (const T*)w->p_out_b,
      (const T*)w->g_out_b, (T*)pr.wcat, pr.bias_cat, pr.bias_out);
  TRI_LAUNCH_OK();
  return 0;
}

// The input-gate GEMM runs transposed: M = the 128 channels of one half (tile_m = a or b; P and G blocks of
// Wcat side by side as the two segments), N = pixels.  A thread then owns a channel and holds consecutive
// pixels, which is the order of the channel-major tensors it writes (a, b, dPG) or reads (da, db).
void gate_in_operands(GemmPlan* p, const Geom& gm, const Prep& pr, const void* z) {
  for (int seg = 0; seg < 2; ++seg) {
    Operand& a = p->a[seg];
    a.ptr = static_cast<const char*>(pr.wcat) + (size_t)seg * CW * CW * gm.es();   // P block / G block of each half
    a.mn_major = false; a.inner = CW; a.outer = CW; a.batch = 2; a.st_outer = CW; a.st_batch = 2 * CW * CW;
    p->b[seg] = rows_operand(z, CW, gm.M, false);
  }
  p->M = CW; p->N = (int)gm.M; p->K0 = CW; p->K1 = CW; p->seg1_col = CW; p->a_tiles = 2;
}

// ---- phase 1: x -> z (LayerNorm), a / b (gated, masked projections, channel-major) ---------------------
template <typename T>
int phase_project(cudaStream_t st, const Geom& gm, const void* x, const void* mask, const TriMulWeights* w,
                  const Prep& pr, void* z, float* mean_in, float* rstd_in, void* a_cm, void* b_cm,
                  void* const* peer_ab = nullptr, int peer_world = 0, int peer_rank = 0) {
  const long long M = gm.M;
  if (peer_ab == nullptr && ln_gate_in_supported(gm.dtype, M, gm.plane)) {
    // 16-bit dtypes: one kernel normalises each x tile in shared memory and feeds both halves' products from it
    LnGateIn f;
    f.dtype = gm.dtype; f.M = M; f.plane = gm.plane; f.eps = gm.eps;
    f.x = x; f.gamma = w->norm_in_w; f.beta = w->norm_in_b; f.wcat = pr.wcat;
    f.bias_cat = (w->p_in_b || w->g_in_b) ? pr.bias_cat : nullptr; f.mask = mask;
    f.z = z; f.mean = mean_in; f.rstd = rstd_in; f.a_cm = a_cm; f.b_cm = b_cm; f.err = pr.err;
    return ln_gate_in(st, f);
  }
  {
    KernelTimer kt("tc_ln_rows", st, 0.0, 2.0 * gm.unit());
    ln_rows_kernel<T><<<cdiv(M, 8 * 2 * kLnRowPairs), 256, 0, st>>>((const T*)x, (const T*)w->norm_in_w, (const T*)w->norm_in_b, gm.eps,
                                                  M, (T*)z, mean_in, rstd_in);
    TRI_LAUNCH_OK();
  }
  GemmPlan p;
  gate_in_operands(&p, gm, pr, z);
  p.out0 = a_cm; p.out1 = b_cm; p.bias0 = (w->p_in_b || w->g_in_b) ? pr.bias_cat : nullptr; p.aux = mask;
  p.plane = gm.plane;
  p.peer_out = peer_ab; p.peer_world = peer_world; p.peer_rank = peer_rank; p.peer_batches = (int)(M / gm.plane);
  p.name = "tc_gemm_gate_in"; p.flops = 2.0 * M * CW * 4 * CW; p.bytes = 3.0 * gm.unit();
  return launch_gemm(st, gm.dtype, EPI_GATE_IN, 256, false, p, pr.err);
}

// ---- phase 3: t -> u (LayerNorm over channels), out = (u Wo^T + bo) * sigmoid(z Wgo^T + bgo) --------------
template <typename T>
int phase_output(cudaStream_t st, const Geom& gm, const void* t_cm, const void* z, const TriMulWeights* w,
                 const Prep& pr, void* u, float* mean_out, float* rstd_out, void* out, bool keep_u = true) {
  const long long M = gm.M;
  if (u_channel_major(gm)) {
    // one batch entry, 16-bit dtype: t is normalised in shared memory as the MMA's MN-major operand; u (kept for
    // the backward pass only) stays channel-major
    LnGateOut f;
    f.dtype = gm.dtype; f.M = M; f.eps = gm.eps; f.t_cm = t_cm; f.z = z;
    f.gamma = w->norm_out_w; f.beta = w->norm_out_b; f.w_out = w->p_out_w; f.w_gate = w->g_out_w;
    f.bias_out = (w->p_out_b || w->g_out_b) ? pr.bias_out : nullptr;
    f.u_cm = keep_u ? u : nullptr; f.mean = mean_out; f.rstd = rstd_out; f.out = out; f.err = pr.err;
    return ln_gate_out(st, f);
  }
  {
    KernelTimer kt("tc_ln_cm", st, 0.0, 2.0 * gm.unit());
    ln_cm_kernel<T><<<kLnCmBlocks, 256, 0, st>>>((const T*)t_cm, (const T*)w->norm_out_w, (const T*)w->norm_out_b, gm.eps,
                                              M, gm.plane, (T*)u, mean_out, rstd_out);
    TRI_LAUNCH_OK();
  }
  GemmPlan p;
  p.a[0] = rows_operand(u, CW, M, false);
  p.b[0] = rows_operand(w->p_out_w, CW, CW, false);
  p.a[1] = rows_operand(z, CW, M, false);
  p.b[1] = rows_operand(w->g_out_w, CW, CW, false);
  p.M = (int)M; p.N = CW; p.K0 = CW; p.K1 = CW; p.seg1_col = CW;
  p.out0 = out; p.bias0 = (w->p_out_b || w->g_out_b) ? pr.bias_out : nullptr;
  p.name = "tc_gemm_gate_out"; p.flops = 2.0 * M * CW * 2 * CW; p.bytes = 3.0 * gm.unit();
  return launch_gemm(st, gm.dtype, EPI_GATE_OUT, 256, false, p, pr.err);
}

int split_k_grad(cudaStream_t st, const Geom& gm, const void* lhs, int lhs_w, const void* rhs, float* partial,
                 int* err, const char* name, int* nparts, bool lhs_channel_major = false,
                 bool rhs_channel_major = false) {
  // partial[s][lhs_w][128] = sum over the pixels of split s of lhs[pixel][:]^T rhs[pixel][:]
  // (lhs pixel-major [M, lhs_w], or channel-major [lhs_w, M]; rhs pixel-major [M, 128], or channel-major [128, M])
  const long long M = gm.M;
  const int bke = gm.dtype == TRI_F32 ? 32 : 64;
  // One split per SM for the single-GPU op.  A row shard gets proportionally fewer (at least 2048 pixels per split,
  // never under 37 splits), so that the partials written here and summed by the reduction shrink with the shard
  // instead of staying sized for 148 SMs; the SMs this leaves idle run the other streams' kernels of the sharded step.
  int splits = gm.sharded ? (int)std::min<long long>(kSplitK, std::max<long long>(37, M / 2048)) : kSplitK;
  splits = (int)std::min<long long>(splits, (M + bke - 1) / bke);
  long long kper = ((M + splits - 1) / splits + bke - 1) / bke * bke;
  splits = (int)((M + kper - 1) / kper);
  GemmPlan p;
  p.a[0] = rows_operand(lhs, lhs_w, M, true);
  if (lhs_channel_major) {  // K (pixels) contiguous: a K-major operand with lhs_w rows
    p.a[0].mn_major = false; p.a[0].inner = M; p.a[0].outer = lhs_w; p.a[0].st_outer = M;
  }
  p.b[0] = rows_operand(rhs, CW, M, true);
  if (rhs_channel_major) {  // K (pixels) contiguous: a K-major operand with 128 rows
    p.b[0].mn_major = false; p.b[0].inner = M; p.b[0].outer = CW; p.b[0].st_outer = M;
  }
  p.M = lhs_w; p.N = CW; p.K0 = (int)kper; p.batches = splits; p.split_k = 1;
  p.out0 = partial; p.ld_out = CW; p.batch_out = (long long)lhs_w * CW;
  p.name = name; p.flops = 2.0 * M * lhs_w * CW; p.bytes = (double)M * (lhs_w + CW) * gm.es();
  *nparts = splits;
  return launch_gemm(st, gm.dtype, EPI_STORE, 128, true, p, err);
}

// reduce_to for several (partial, nparts, n, out) jobs at once; jobs with nothing to write are dropped
struct ReduceJob { const float* partial; int nparts, n; float* out; float* out2 = nullptr; int rowlen = 0; };
int reduce_many(cudaStream_t st, std::initializer_list<ReduceJob> list) {
  ReduceJobs jobs = {};
  int count = 0, nmax = 0;
  double bytes = 0.0;
  for (const ReduceJob& j : list) {
    if ((j.out == nullptr && j.out2 == nullptr) || j.nparts == 0) continue;
    jobs.partial[count] = j.partial; jobs.out[count] = j.out; jobs.out2[count] = j.out2;
    jobs.nparts[count] = j.nparts; jobs.n[count] = j.n; jobs.rowlen[count] = j.rowlen;
    nmax = std::max(nmax, j.n);
    bytes += 4.0 * (j.nparts + 1) * j.n;
    ++count;
  }
  if (count == 0) return 0;
  KernelTimer kt("tc_reduce", st, 0.0, bytes);
  reduce_multi_kernel<<<dim3(cdiv(nmax, 32), count), 256, 0, st>>>(jobs);
  TRI_LAUNCH_OK();
  return 0;
}

int reduce_to(cudaStream_t st, const float* partial, int nparts, int n, float* out) {
  KernelTimer kt("tc_reduce", st, 0.0, 4.0 * (nparts + 1) * n);
  reduce_kernel<<<cdiv(n, 64), 256, 0, st>>>(partial, nparts, n, out);
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

// ---- backward of phase 3: d_out -> dy, dgo, gradients of the output weights, dt (channel-major) ------------
template <typename T>
int phase_output_bwd(cudaStream_t st, const Geom& gm, const void* d_out, const void* u, const void* z,
                     const void* t_cm, const float* mean_out, const float* rstd_out, const TriMulWeights* w,
                     const Prep& pr, const TriMulWeightGrads* g, void* dy, void* dgo, void* du, void* dt_cm,
                     float* partial) {
  const long long M = gm.M;
  int nparts = 0;
  {
    GemmPlan p;   // dy = d_out * sig(go), dgo = d_out * y * sig * (1 - sig), with y and go recomputed
    p.a[0] = rows_operand(u, CW, M, false);
    if (u_channel_major(gm)) {   // A(m = pixel, k = channel) with the pixels contiguous
      p.a[0].mn_major = true; p.a[0].inner = M; p.a[0].outer = CW; p.a[0].st_outer = M;
    }
    p.b[0] = rows_operand(w->p_out_w, CW, CW, false);
    p.a[1] = rows_operand(z, CW, M, false);
    p.b[1] = rows_operand(w->g_out_w, CW, CW, false);
    p.M = (int)M; p.N = CW; p.K0 = CW; p.K1 = CW; p.seg1_col = CW;
    p.out0 = dy; p.out1 = dgo; p.aux = d_out; p.bias0 = (w->p_out_b || w->g_out_b) ? pr.bias_out : nullptr;
    p.name = "tc_gemm_gate_out_bwd"; p.flops = 0.0; p.bytes = 5.0 * gm.unit();  // recompute: no algorithmic flops
    TRI_TRY(launch_gemm(st, gm.dtype, EPI_GATE_OUT_BWD, 256, false, p, pr.err));
  }
  // the two output weight gradients: split-K partials side by side, reduced at the end of the phase together
  // with the LayerNorm partials
  float* part2 = partial + (size_t)kSplitK * CW * CW;
  float* scratch = partial + (size_t)2 * kSplitK * CW * CW;   // the rest of the weight-gradient area
  int n1 = 0, n2 = 0;
  if (g->p_out_w)
    TRI_TRY(split_k_grad(st, gm, dy, CW, u, partial, pr.err, "tc_gemm_wgrad", &n1, false, u_channel_major(gm)));
  if (g->g_out_w) TRI_TRY(split_k_grad(st, gm, dgo, CW, z, part2, pr.err, "tc_gemm_wgrad", &n2));
  if (g->p_out_b) {
    TRI_TRY(colsum_to<T>(st, dy, M, CW, scratch, &nparts));
    TRI_TRY(reduce_to(st, scratch, nparts, CW, g->p_out_b));
  }
  if (g->g_out_b) {
    TRI_TRY(colsum_to<T>(st, dgo, M, CW, scratch, &nparts));
    TRI_TRY(reduce_to(st, scratch, nparts, CW, g->g_out_b));
  }
  float* pg = partial + kWgradPartialFloats;
  if (u_channel_major(gm)) {
    // du^T = Wo^T dy^T: a thread of the store epilogue owns a channel and consecutive pixels, so du comes out
    // channel-major like t and dt, and the LayerNorm backward needs no transposition
    GemmPlan p;
    p.a[0] = rows_operand(w->p_out_w, CW, CW, true);   // A(m = ch, k = c) = Wo[c][ch]: m contiguous
    p.b[0] = rows_operand(dy, CW, M, false);           // B(n = pixel, k = c)
    p.M = CW; p.N = (int)M; p.K0 = CW; p.out0 = du; p.ld_out = M;
    p.name = "tc_gemm_du"; p.flops = 2.0 * M * CW * CW; p.bytes = 2.0 * gm.unit();
    TRI_TRY(launch_gemm(st, gm.dtype, EPI_STORE, 256, false, p, pr.err));
    const int blocks = (int)std::min<long long>(kLnCmCmBlocks, (M + 63) / 64);
    float* pb = pg + (size_t)blocks * CW;
    {
      KernelTimer kt("tc_ln_cm_bwd", st, 0.0, 3.0 * gm.unit());
      if constexpr (sizeof(T) == 2)
        ln_cm_bwd_cm_kernel<T><<<blocks, 256, 0, st>>>((const T*)du, (const T*)t_cm, mean_out, rstd_out,
                                                       (const T*)w->norm_out_w, M, (T*)dt_cm, pg, pb);
      TRI_LAUNCH_OK();
    }
    return reduce_many(st, {{partial, n1, CW * CW, g->p_out_w}, {part2, n2, CW * CW, g->g_out_w},
                            {pg, blocks, CW, g->norm_out_w}, {pb, blocks, CW, g->norm_out_b}});
  }
  {
    GemmPlan p;   // du = dy Wo
    p.a[0] = rows_operand(dy, CW, M, false);
    p.b[0] = rows_operand(w->p_out_w, CW, CW, true);  // B(n = ch, k = c) = Wo[c][ch]: n contiguous
    p.M = (int)M; p.N = CW; p.K0 = CW; p.out0 = du; p.ld_out = CW;
    p.name = "tc_gemm_du"; p.flops = 2.0 * M * CW * CW; p.bytes = 2.0 * gm.unit();
    TRI_TRY(launch_gemm(st, gm.dtype, EPI_STORE, 128, false, p, pr.err));
  }
  float* pb = pg + (size_t)kLnCmBwdBlocks * CW;
  {
    KernelTimer kt("tc_ln_cm_bwd", st, 0.0, 3.0 * gm.unit());
    ln_cm_bwd_kernel<T><<<kLnCmBwdBlocks, 256, 0, st>>>((const T*)du, (const T*)t_cm, mean_out, rstd_out,
                                                  (const T*)w->norm_out_w, M, gm.plane, (T*)dt_cm, pg, pb);
    TRI_LAUNCH_OK();
  }
  return reduce_many(st, {{partial, n1, CW * CW, g->p_out_w}, {part2, n2, CW * CW, g->g_out_w},
                          {pg, kLnCmBwdBlocks, CW, g->norm_out_w}, {pb, kLnCmBwdBlocks, CW, g->norm_out_b}});
}

// ---- backward of phase 1: da, db (channel-major), dgo -> gradients of the input weights, dx ---------------
template <typename T>
int phase_project_bwd(cudaStream_t st, const Geom& gm, const void* x, const void* mask, const void* z,
                      const void* da_cm, const void* db_cm, const void* dgo, const float* mean_in,
                      const float* rstd_in, const TriMulWeights* w, const Prep& pr, const TriMulWeightGrads* g,
                      void* dpg, void* dz, void* dx, float* partial) {
  const long long M = gm.M;
  int nparts = 0;
  {
    GemmPlan p;   // input gate backward fused into the recomputed projection GEMM
    gate_in_operands(&p, gm, pr, z);
    p.out0 = dpg; p.ld_out = M; p.bias0 = (w->p_in_b || w->g_in_b) ? pr.bias_cat : nullptr;
    p.aux = mask; p.aux2 = da_cm; p.aux3 = db_cm; p.plane = gm.plane;
    p.name = "tc_gemm_gate_in_bwd"; p.flops = 0.0; p.bytes = 7.0 * gm.unit();
    TRI_TRY(launch_gemm(st, gm.dtype, EPI_GATE_IN_BWD, 256, false, p, pr.err));
  }
  if (g->p_in_w || g->g_in_w)   // reduced at the end of the phase together with the LayerNorm partials
    TRI_TRY(split_k_grad(st, gm, dpg, 4 * CW, z, partial, pr.err, "tc_gemm_wgrad", &nparts, /*lhs_channel_major=*/true));
  if (g->p_in_b || g->g_in_b) {
    KernelTimer kt("tc_rowsum", st, 0.0, 4.0 * gm.unit());
    rowsum_wcat_kernel<T><<<4 * CW, 256, 0, st>>>((const T*)dpg, M, g->p_in_b, g->g_in_b);
    TRI_LAUNCH_OK();
  }
  {
    GemmPlan p;   // dz = dPG Wcat + dgo Wgo
    p.a[0] = rows_operand(dpg, 4 * CW, M, false);
    p.a[0].mn_major = true; p.a[0].inner = M; p.a[0].outer = 4 * CW; p.a[0].st_outer = M;   // A(m = pixel, k = row of dPG): m contiguous
    p.b[0] = rows_operand(pr.wcat, CW, 4 * CW, true);   // B(n = c, k = row of Wcat): n contiguous
    p.a[1] = rows_operand(dgo, CW, M, false);
    p.b[1] = rows_operand(w->g_out_w, CW, CW, true);
    p.M = (int)M; p.N = CW; p.K0 = 4 * CW; p.K1 = CW; p.seg1_col = 0;
    p.out0 = dz; p.ld_out = CW;
    p.name = "tc_gemm_dz"; p.flops = 2.0 * M * CW * 5 * CW; p.bytes = 6.0 * gm.unit();
    TRI_TRY(launch_gemm(st, gm.dtype, EPI_STORE, 128, false, p, pr.err));
  }
  const int blocks = (int)std::min<long long>(kPersist, (M + 7) / 8);
  float* pg = partial + kWgradPartialFloats;
  float* pb = pg + (size_t)kPersist * CW;
  {
    KernelTimer kt("tc_ln_rows_bwd", st, 0.0, 3.0 * gm.unit());
    ln_rows_bwd_kernel<T><<<blocks, 256, 0, st>>>((const T*)dz, (const T*)x, mean_in, rstd_in, (const T*)w->norm_in_w,
                                                  M, (T*)dx, pg, pb);
    TRI_LAUNCH_OK();
  }
  return reduce_many(st, {{partial, nparts, 4 * CW * CW, g->p_in_w, g->g_in_w, CW},
                          {pg, blocks, CW, g->norm_in_w}, {pb, blocks, CW, g->norm_in_b}});
}

// ---------------------------------------------------------------------------------------------
// single-GPU op: memory plan and drivers
// ---------------------------------------------------------------------------------------------
struct SavedT { void *z, *a, *b, *t, *u; float *mean_in, *rstd_in, *mean_out, *rstd_out; };

Geom geom_of(const TriMulDesc* d) {
  Geom g;
  g.dtype = d->dtype; g.eps = d->eps;
  g.plane = (long long)d->N * d->N; g.M = g.plane * d->B;
  return g;
}

void carve_saved(Arena& a, const Geom& gm, SavedT* s) {
  const size_t M = (size_t)gm.M, unit = M * CW * gm.es();
  s->z = a.take<char>(unit); s->a = a.take<char>(unit); s->b = a.take<char>(unit);
  s->t = a.take<char>(unit); s->u = a.take<char>(unit);
  s->mean_in = a.take<float>(M); s->rstd_in = a.take<float>(M);
  s->mean_out = a.take<float>(M); s->rstd_out = a.take<float>(M);
}

struct BwdBufs { void *dy, *dgo, *du, *dt, *da, *db, *dpg, *dz; float* partial; };
void carve_bwd(Arena& a, const Geom& gm, BwdBufs* w) {
  const size_t unit = (size_t)gm.M * CW * gm.es();
  w->dy = a.take<char>(unit); w->dgo = a.take<char>(unit); w->du = a.take<char>(unit);
  w->dt = a.take<char>(unit); w->da = a.take<char>(unit); w->db = a.take<char>(unit);
  w->dpg = a.take<char>(4 * unit); w->dz = a.take<char>(unit);
  w->partial = a.take<float>(partial_floats());
}

template <typename T>
int forward_t(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out, void* saved,
              void* ws, size_t ws_size, cudaStream_t st) {
  const Geom gm = geom_of(d);
  Arena a(ws, ws_size);
  Prep pr;
  carve_prep(a, gm.es(), &pr);
  SavedT s;
  if (saved) { Arena sa(saved, mul_saved_bytes(d)); carve_saved(sa, gm, &s); }
  else carve_saved(a, gm, &s);
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul forward workspace too small: need %zu, got %zu", a.off, ws_size);
  TRI_TRY(run_prep<T>(st, w, pr));
  TRI_TRY(phase_project<T>(st, gm, x, mask, w, pr, s.z, s.mean_in, s.rstd_in, s.a, s.b));
  const bool incoming = d->direction == TRI_INCOMING;
  TRI_TRY(contraction(st, d->dtype, d->B * CW, d->N, s.a, incoming, s.b, incoming, s.t, pr.err, "tc_gemm_contract"));
  return phase_output<T>(st, gm, s.t, s.z, w, pr, s.u, s.mean_out, s.rstd_out, out, /*keep_u=*/saved != nullptr);
}

template <typename T>
int backward_t(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, const void* saved,
               const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws, size_t ws_size, cudaStream_t st) {
  const Geom gm = geom_of(d);
  Arena a(ws, ws_size);
  Prep pr;
  carve_prep(a, gm.es(), &pr);
  BwdBufs b;
  carve_bwd(a, gm, &b);
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul backward workspace too small: need %zu, got %zu", a.off, ws_size);
  SavedT s;
  { Arena sa(const_cast<void*>(saved), mul_saved_bytes(d)); carve_saved(sa, gm, &s); }
  TRI_TRY(run_prep<T>(st, w, pr));
  TRI_TRY(phase_output_bwd<T>(st, gm, d_out, s.u, s.z, s.t, s.mean_out, s.rstd_out, w, pr, g, b.dy, b.dgo, b.du, b.dt,
                              b.partial));
  // contraction backward: the same batched GEMM, only the operand majors change
  const int planes = d->B * CW, n = d->N, dt = d->dtype;
  if (d->direction == TRI_OUTGOING) {
    TRI_TRY(contraction(st, dt, planes, n, b.dt, false, s.b, true, b.da, pr.err, "tc_gemm_contract_bwd"));  // da[i,k] = sum_j dt[i,j] b[j,k]
    TRI_TRY(contraction(st, dt, planes, n, b.dt, true, s.a, true, b.db, pr.err, "tc_gemm_contract_bwd"));   // db[j,k] = sum_i dt[i,j] a[i,k]
  } else {
    TRI_TRY(contraction(st, dt, planes, n, s.b, false, b.dt, false, b.da, pr.err, "tc_gemm_contract_bwd")); // da[k,i] = sum_j b[k,j] dt[i,j]
    TRI_TRY(contraction(st, dt, planes, n, s.a, false, b.dt, true, b.db, pr.err, "tc_gemm_contract_bwd"));  // db[k,j] = sum_i a[k,i] dt[i,j]
  }
  return phase_project_bwd<T>(st, gm, x, mask, s.z, b.da, b.db, b.dgo, s.mean_in, s.rstd_in, w, pr, g, b.dpg, b.dz, dx,
                              b.partial);
}

// ---------------------------------------------------------------------------------------------
// row-sharded op: the four pixel-wise phases on their own (the contraction runs through tri_bgemm)
// ---------------------------------------------------------------------------------------------
struct ShardSaved { void *z, *u, *dgo; float *mean_in, *rstd_in, *mean_out, *rstd_out; };

Geom geom_of(const TriMulShardDesc* d) {
  Geom g;
  g.dtype = d->dtype; g.eps = d->eps;
  g.plane = (long long)d->rows * d->N; g.M = g.plane * d->B;
  g.sharded = true;
  return g;
}

void carve_shard_saved(Arena& a, const Geom& gm, ShardSaved* s) {
  const size_t M = (size_t)gm.M, unit = M * CW * gm.es();
  s->z = a.take<char>(unit); s->u = a.take<char>(unit); s->dgo = a.take<char>(unit);
  s->mean_in = a.take<float>(M); s->rstd_in = a.take<float>(M);
  s->mean_out = a.take<float>(M); s->rstd_out = a.take<float>(M);
}

struct ShardWs { void *dy, *du, *dpg, *dz; float* partial; };
void carve_shard_ws(Arena& a, const Geom& gm, int phase, ShardWs* w) {
  const size_t unit = (size_t)gm.M * CW * gm.es();
  *w = ShardWs{};
  if (phase == TRI_PHASE_OUTPUT_BWD) { w->dy = a.take<char>(unit); w->du = a.take<char>(unit); }
  if (phase == TRI_PHASE_PROJECT_BWD) { w->dpg = a.take<char>(4 * unit); w->dz = a.take<char>(unit); }
  if (phase >= TRI_PHASE_OUTPUT_BWD) w->partial = a.take<float>(partial_floats());
}

template <typename T>
int shard_phase_t(const TriMulShardDesc* d, int phase, const TriMulShardBufs* bf, void* ws, size_t ws_size,
                  cudaStream_t st) {
  const Geom gm = geom_of(d);
  Arena a(ws, ws_size);
  Prep pr;
  carve_prep(a, gm.es(), &pr);
  if (bf->prep != nullptr) {   // prepared weights kept by the caller across the phases of one forward + backward
    Arena pa(bf->prep, mul_shard_prep_bytes(d));
    carve_prep_weights(pa, gm.es(), &pr);
  }
  ShardWs sw;
  carve_shard_ws(a, gm, phase, &sw);
  if (!a.ok()) return fail(TRI_ERR_WORKSPACE, "trimul shard workspace too small: need %zu, got %zu", a.off, ws_size);
  ShardSaved s;
  { Arena sa(bf->saved, mul_shard_saved_bytes(d)); carve_shard_saved(sa, gm, &s); }
  TRI_TRY(run_prep<T>(st, bf->w, pr, bf->prep != nullptr && bf->prep_ready != 0));
  switch (phase) {
    case TRI_PHASE_PROJECT:
      if (!bf->x || ((!bf->a_cm || !bf->b_cm) && !(bf->peer_ab != nullptr && bf->peer_world > 1)))
        return fail(TRI_ERR_ARG, "project phase needs x and either a_cm, b_cm or the peer buffers");
      return phase_project<T>(st, gm, bf->x, bf->mask, bf->w, pr, s.z, s.mean_in, s.rstd_in, bf->a_cm, bf->b_cm,
                              bf->peer_ab, bf->peer_world, bf->peer_rank);
    case TRI_PHASE_OUTPUT:
      if (!bf->t_cm || !bf->out) return fail(TRI_ERR_ARG, "output phase needs t_cm, out");
      return phase_output<T>(st, gm, bf->t_cm, s.z, bf->w, pr, s.u, s.mean_out, s.rstd_out, bf->out);
    case TRI_PHASE_OUTPUT_BWD:
      if (!bf->d_out || !bf->t_cm || !bf->dt_cm || !bf->g) return fail(TRI_ERR_ARG, "output backward needs d_out, t_cm, dt_cm, g");
      return phase_output_bwd<T>(st, gm, bf->d_out, s.u, s.z, bf->t_cm, s.mean_out, s.rstd_out, bf->w, pr, bf->g, sw.dy,
                                 s.dgo, sw.du, bf->dt_cm, sw.partial);
    case TRI_PHASE_PROJECT_BWD:
      if (!bf->x || !bf->a_cm || !bf->b_cm || !bf->dx || !bf->g) return fail(TRI_ERR_ARG, "project backward needs x, a_cm, b_cm (gradients), dx, g");
      return phase_project_bwd<T>(st, gm, bf->x, bf->mask, s.z, bf->a_cm, bf->b_cm, s.dgo, s.mean_in, s.rstd_in, bf->w,
                                  pr, bf->g, sw.dpg, sw.dz, bf->dx, sw.partial);
  }
  return fail(TRI_ERR_ARG, "bad phase %d", phase);
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
  carve_saved(a, geom_of(d), &s);
  return a.off;
}

size_t mul_ws_bytes(const TriMulDesc* d, int is_bwd) {
  Arena a(nullptr, 0);
  Prep p;
  const Geom gm = geom_of(d);
  carve_prep(a, gm.es(), &p);
  if (is_bwd) { BwdBufs b; carve_bwd(a, gm, &b); }
  else { SavedT s; carve_saved(a, gm, &s); }
  return a.off + 256;
}

bool mul_shard_supported(const TriMulShardDesc* d) {
  if (d->C != CW || d->Ch != CW) return false;
  if (d->dtype == TRI_F32 && d->precision != TRI_PREC_TF32) return false;
  return d->N % 8 == 0 && d->rows > 0 && d->rows <= d->N;
}

size_t mul_shard_saved_bytes(const TriMulShardDesc* d) {
  Arena a(nullptr, 0);
  ShardSaved s;
  carve_shard_saved(a, geom_of(d), &s);
  return a.off;
}

size_t mul_shard_prep_bytes(const TriMulShardDesc* d) {
  Arena a(nullptr, 0);
  Prep p;
  carve_prep_weights(a, geom_of(d).es(), &p);
  return a.off;
}

size_t mul_shard_ws_bytes(const TriMulShardDesc* d, int phase) {
  Arena a(nullptr, 0);
  Prep p;
  const Geom gm = geom_of(d);
  carve_prep(a, gm.es(), &p);
  ShardWs w;
  carve_shard_ws(a, gm, phase, &w);
  return a.off + 256;
}

int mul_shard_phase(const TriMulShardDesc* d, int phase, const TriMulShardBufs* bf, void* ws, size_t ws_size,
                    cudaStream_t st) {
  switch (d->dtype) {
    case TRI_F32: return shard_phase_t<float>(d, phase, bf, ws, ws_size, st);
    case TRI_BF16: return shard_phase_t<__nv_bfloat16>(d, phase, bf, ws, ws_size, st);
    case TRI_F16: return shard_phase_t<__half>(d, phase, bf, ws, ws_size, st);
  }
  return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
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
