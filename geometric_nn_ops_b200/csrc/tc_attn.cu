// Tensor-core triangle attention (tcgen05 + TMEM + TMA), bf16 / fp16, head dim 32 or 64.
//
// Forward: one CTA (128 threads, one query row per thread) per (batch, row, head, 128-query block).
// Per 128-key tile:
//   S   = Q K^T             tcgen05.mma, A/B from TMA-staged swizzled smem, accumulator in TMEM (128 cols)
//   x   = scale*S + bias + mask_bias        tcgen05.ld to registers; bias tile TMA-staged in smem
//   P   = exp2((x - m) log2e), online max / sum per row; P rounded to the input dtype into smem
//   PV  = P V               tcgen05.mma (P K-major from smem, V MN-major), fresh TMEM accumulator (D cols)
//   O   = O*alpha + PV      in registers (so no TMEM read-modify-write for the rescale)
// Two CTAs per SM overlap each other's MMA / softmax phases.  K/V tiles are double buffered.
// Semantics follow triangle_attention_torch (geometric_nn_ops_torch/triangle/_reference/triangle_attention.py:28-44):
// bias and the finite -1e9 key-mask sentinel are added in fp32 in that order; keys beyond N_res get -inf.
#include <algorithm>
#include <cstdlib>

#include "tc_common.cuh"
#include "tc_paths.cuh"

namespace tri {
namespace tc {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMaskSentinel = 1e9f;

struct AttnArgs {
  int B, S, N, H;
  float scale;
  void* o;
  int64_t o_st[4];
  float* stats;          // [2][B][S][H][N]: row max, log row sum
  const uint8_t* mask;   // nullable
  int64_t mask_st[2];
  int has_bias;
  int bias_b_mul;        // 0 when the bias is broadcast over the batch
  uint32_t idesc_s, idesc_pv;
  int* err;
};

template <int HD> struct Geo {
  static constexpr int RB = HD * 2;                      // bytes per tile row (16-bit elements)
  static constexpr int TILE = 128 * RB;                  // one [128 x HD] tile
  static constexpr uint32_t LAYOUT = RB == 128 ? 2 : 4;  // SWIZZLE_128B or SWIZZLE_64B
  static constexpr uint32_t SBO = 8 * RB;                // 8-row group
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + TILE;
  static constexpr int OFF_V = OFF_K + 2 * TILE;
  static constexpr int OFF_P = OFF_V + 2 * TILE;         // [128 x 128] as two SW128 blocks of 64 keys
  static constexpr int OFF_BIAS = OFF_P + 32768;         // same shape
  static constexpr int OFF_MB = OFF_BIAS + 32768;        // 128 floats
  static constexpr int OFF_BAR = OFF_MB + 512;
  static constexpr int SMEM = OFF_BAR + 128 + 1024;      // + alignment slack
};

// byte offset of 16-byte chunk `g` (0..15, 8 elements each) of row r inside a [128 x 128] two-block SW128 tile
__device__ __forceinline__ int sw128_chunk(int r, int g) {
  return (g >> 3) * 16384 + r * 128 + (((g & 7) ^ (r & 7)) << 4);
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  union { uint32_t u; T h[2]; } pk;
  pk.h[0] = from_f32<T>(a);
  pk.h[1] = from_f32<T>(b);
  return pk.u;
}
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  union { uint4 u; T h[8]; } pk;
  pk.u = v;
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f32(pk.h[i]);
}

template <typename T, int HD>
__global__ void __launch_bounds__(128, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmBias,
                   const AttnArgs a) {
  using G = Geo<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + G::OFF_Q;
  uint8_t* sK = smem + G::OFF_K;
  uint8_t* sV = smem + G::OFF_V;
  uint8_t* sP = smem + G::OFF_P;
  uint8_t* sBias = smem + G::OFF_BIAS;
  float* sMb = reinterpret_cast<float*>(smem + G::OFF_MB);
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + G::OFF_BAR);
  uint64_t* bar_kv = bar_q + 1;  // [2]
  uint64_t* bar_bias = bar_q + 3;
  uint64_t* bar_s = bar_q + 4;
  uint64_t* bar_pv = bar_q + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 6);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qblocks = (a.N + 127) / 128;
  int z = blockIdx.x;
  const int qb = z % qblocks; z /= qblocks;
  const int h = z % a.H; z /= a.H;
  const int s = z % a.S;
  const int b = z / a.S;
  const int q0 = qb * 128;
  const int ntiles = (a.N + 127) / 128;

  if (tid == 0) {
    mbar_init(bar_q, 1); mbar_init(&bar_kv[0], 1); mbar_init(&bar_kv[1], 1);
    mbar_init(bar_bias, 1); mbar_init(bar_s, 1); mbar_init(bar_pv, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);

  if (tid == 0) {
    mbar_expect_tx(bar_q, G::TILE);
    tma_load_5d(sQ, &tmQ, bar_q, 0, h, q0, s, b);
    for (int st = 0; st < 2 && st < ntiles; ++st) {
      mbar_expect_tx(&bar_kv[st], 2 * G::TILE);
      tma_load_5d(sK + st * G::TILE, &tmK, &bar_kv[st], 0, h, st * 128, s, b);
      tma_load_5d(sV + st * G::TILE, &tmV, &bar_kv[st], 0, h, st * 128, s, b);
    }
    if (a.has_bias) {
      mbar_expect_tx(bar_bias, 32768);
      tma_load_4d(sBias, &tmBias, bar_bias, 0, q0, h, b * a.bias_b_mul);
      tma_load_4d(sBias + 16384, &tmBias, bar_bias, 64, q0, h, b * a.bias_b_mul);
    }
  }

  float m_run = -INFINITY, l_run = 0.f;
  float o_acc[HD];
#pragma unroll
  for (int i = 0; i < HD; ++i) o_acc[i] = 0.f;
  bool ok = true;

  for (int j = 0; j < ntiles; ++j) {
    const int stg = j & 1, k0 = j * 128;
    const uint32_t par = j & 1, kv_par = (j >> 1) & 1;
    if (tid == 0) {
      if (j == 0) ok = mbar_wait(bar_q, 0, a.err, 11);
      ok = ok && mbar_wait(&bar_kv[stg], kv_par, a.err, 12);
      tc_fence_after_sync();
      const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + stg * G::TILE);
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        umma<KIND_F16>(tmem_base, make_smem_desc(qa + ks * 32, 16, G::SBO, G::LAYOUT),
                       make_smem_desc(ka + ks * 32, 16, G::SBO, G::LAYOUT), a.idesc_s, ks > 0);
      umma_commit(bar_s);
    }
    {  // additive key-mask term for this tile's 128 keys (thread t handles key t)
      const int kj = k0 + tid;
      float mb = 0.f;
      if (kj >= a.N) mb = -INFINITY;
      else if (a.mask != nullptr) mb = kMaskSentinel * ((a.mask[b * a.mask_st[0] + s * a.mask_st[1] + kj] ? 1.0f : 0.0f) - 1.0f);
      sMb[tid] = mb;
    }
    __syncthreads();
    ok = mbar_wait(bar_s, par, a.err, 13) && ok;
    tc_fence_after_sync();
    if (a.has_bias) ok = mbar_wait(bar_bias, par, a.err, 14) && ok;

    // ---- logits into registers, running max --------------------------------------------------
    float x[128];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(t_row + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float bv[8];
        if (a.has_bias) {
          const uint4 raw = *reinterpret_cast<const uint4*>(sBias + sw128_chunk(tid, c * 4 + u));
          unpack8<T>(raw, bv);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int col = c * 32 + u * 8 + i;
          float v = __uint_as_float(r[u * 8 + i]) * a.scale;
          if (a.has_bias) v += bv[i];
          v += sMb[col];
          x[col] = v;
          mx = fmaxf(mx, v);
        }
      }
    }
    const float m_new = fmaxf(m_run, mx);
    const float alpha = ex2_approx((m_run - m_new) * kLog2e);
    float psum = 0.f;
#pragma unroll
    for (int g = 0; g < 16; ++g) {
      float p[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        p[i] = ex2_approx((x[g * 8 + i] - m_new) * kLog2e);
        psum += p[i];
      }
      uint4 pk;
      pk.x = pack2<T>(p[0], p[1]); pk.y = pack2<T>(p[2], p[3]);
      pk.z = pack2<T>(p[4], p[5]); pk.w = pack2<T>(p[6], p[7]);
      *reinterpret_cast<uint4*>(sP + sw128_chunk(tid, g)) = pk;
    }
    l_run = l_run * alpha + psum;
    m_run = m_new;
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();

    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t pa = smem_u32(sP), va = smem_u32(sV + stg * G::TILE);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma<KIND_F16>(tmem_base + 128, make_smem_desc(pa + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024, 2),
                       make_smem_desc(va + kk * 16 * G::RB, 128 * G::RB, G::SBO, G::LAYOUT), a.idesc_pv, kk > 0);
      umma_commit(bar_pv);
      if (a.has_bias && j + 1 < ntiles) {  // every thread has finished reading this tile's bias
        mbar_expect_tx(bar_bias, 32768);
        tma_load_4d(sBias, &tmBias, bar_bias, k0 + 128, q0, h, b * a.bias_b_mul);
        tma_load_4d(sBias + 16384, &tmBias, bar_bias, k0 + 192, q0, h, b * a.bias_b_mul);
      }
    }
    ok = mbar_wait(bar_pv, par, a.err, 15) && ok;
    tc_fence_after_sync();
    if (tid == 0 && j + 2 < ntiles) {  // the PV product has consumed this K/V stage
      mbar_expect_tx(&bar_kv[stg], 2 * G::TILE);
      tma_load_5d(sK + stg * G::TILE, &tmK, &bar_kv[stg], 0, h, k0 + 256, s, b);
      tma_load_5d(sV + stg * G::TILE, &tmV, &bar_kv[stg], 0, h, k0 + 256, s, b);
    }
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(t_row + 128 + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(r[i]);
    }
    tc_fence_before_sync();
    if (!ok) break;
  }

  const int qi = q0 + tid;
  if (qi < a.N && ok) {
    const float inv = 1.0f / l_run;
    T* orow = reinterpret_cast<T*>(a.o) + b * a.o_st[0] + s * a.o_st[1] + qi * a.o_st[2] + h * a.o_st[3];
#pragma unroll
    for (int g = 0; g < HD / 8; ++g) {
      uint4 pk;
      pk.x = pack2<T>(o_acc[g * 8 + 0] * inv, o_acc[g * 8 + 1] * inv);
      pk.y = pack2<T>(o_acc[g * 8 + 2] * inv, o_acc[g * 8 + 3] * inv);
      pk.z = pack2<T>(o_acc[g * 8 + 4] * inv, o_acc[g * 8 + 5] * inv);
      pk.w = pack2<T>(o_acc[g * 8 + 6] * inv, o_acc[g * 8 + 7] * inv);
      reinterpret_cast<uint4*>(orow)[g] = pk;
    }
    const long long row = (((long long)b * a.S + s) * a.H + h) * a.N + qi;
    a.stats[row] = m_run;
    a.stats[(long long)a.B * a.S * a.H * a.N + row] = logf(l_run);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

bool forced_simt() {
  const char* e = getenv("TRI_B200_FORCE_SIMT");
  return e != nullptr && e[0] == '1';
}

bool strides_ok(const int64_t* st) {
  for (int i = 0; i < 4; ++i)
    if (st[i] % 8 != 0) return false;
  return true;
}

// rank-5 map over a [B, S, N, H, D] tensor given its (batch, row, residue, head) strides; box = [128 residues x D]
int qkv_map(CUtensorMap* out, const void* p, const TriAttnDesc* d, const int64_t* st) {
  const uint64_t dims[5] = {(uint64_t)d->D, (uint64_t)d->H, (uint64_t)d->n_res, (uint64_t)d->n_seq, (uint64_t)d->B};
  const uint64_t str[4] = {(uint64_t)st[3], (uint64_t)st[2], (uint64_t)st[1], (uint64_t)st[0]};
  const uint32_t box[5] = {(uint32_t)d->D, 1, 128, 1, 1};
  return make_tmap(out, p, d->dtype, 5, dims, str, box, d->D * 2);
}

template <typename T, int HD>
int fwd_launch(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
               const uint8_t* mask, void* o, float* stats, int* err, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tb;
  TRI_TRY(qkv_map(&tq, q, d, d->q_st));
  TRI_TRY(qkv_map(&tk, k, d, d->k_st));
  TRI_TRY(qkv_map(&tv, v, d, d->v_st));
  AttnArgs a;
  a.B = d->B; a.S = d->n_seq; a.N = d->n_res; a.H = d->H; a.scale = d->scale;
  a.o = o; for (int i = 0; i < 4; ++i) a.o_st[i] = d->o_st[i];
  a.stats = stats; a.mask = mask; a.mask_st[0] = d->mask_st[0]; a.mask_st[1] = d->mask_st[1];
  a.has_bias = bias != nullptr; a.bias_b_mul = d->bias_st[0] != 0 ? 1 : 0;
  const int kind = d->dtype == TRI_BF16 ? KIND_BF16 : KIND_F16;
  a.idesc_s = make_idesc(kind, 128, 128, false, false);
  a.idesc_pv = make_idesc(kind, 128, HD, false, true);
  a.err = err;
  if (bias != nullptr) {
    const uint64_t nb = a.bias_b_mul ? (uint64_t)d->B : 1;
    const uint64_t dims[4] = {(uint64_t)d->n_res, (uint64_t)d->n_res, (uint64_t)d->H, nb};
    const uint64_t str[3] = {(uint64_t)d->bias_st[2], (uint64_t)d->bias_st[1], (uint64_t)d->bias_st[0]};
    const uint32_t box[4] = {64, 128, 1, 1};
    TRI_TRY(make_tmap(&tb, bias, d->dtype, 4, dims, str, box, 128));
  } else {
    tb = tq;
  }
  auto kern = attn_fwd_tc_kernel<T, HD>;
  static bool configured = false;
  if (!configured) {
    TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<HD>::SMEM));
    configured = true;
  }
  const long long blocks = (long long)((d->n_res + 127) / 128) * d->B * d->n_seq * d->H;
  const double pairs = (double)d->B * d->n_seq * d->H * d->n_res * (double)d->n_res;
  KernelTimer kt("tc_attn_fwd", st, 4.0 * pairs * d->D, 2.0 * 4.0 * d->B * d->n_seq * (double)d->n_res * d->H * d->D);
  kern<<<(unsigned)blocks, 128, Geo<HD>::SMEM, st>>>(tq, tk, tv, tb, a);
  TRI_LAUNCH_OK();
  return 0;
}

}  // namespace

bool attn_fwd_supported(const TriAttnDesc* d) {
  if (forced_simt()) return false;
  if (d->dtype != TRI_BF16 && d->dtype != TRI_F16) return false;
  if (d->D != 32 && d->D != 64) return false;
  if (d->n_res % 8 != 0) return false;
  if (!strides_ok(d->q_st) || !strides_ok(d->k_st) || !strides_ok(d->v_st) || !strides_ok(d->o_st)) return false;
  if (d->bias_st[1] % 8 != 0 || d->bias_st[2] % 8 != 0 || d->bias_st[0] % 8 != 0) return false;
  if ((long long)((d->n_res + 127) / 128) * d->B * d->n_seq * d->H > 2147483647LL) return false;
  return true;
}

bool attn_bwd_supported(const TriAttnDesc* d) { (void)d; return false; }

size_t attn_ws_bytes(const TriAttnDesc* d, int is_bwd) { (void)d; (void)is_bwd; return 512; }

int attn_forward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                 const uint8_t* mask, void* o, float* lse, void* ws, size_t ws_size, cudaStream_t st) {
  if (ws == nullptr || ws_size < 256) return fail(TRI_ERR_WORKSPACE, "attention forward needs a 256-byte workspace");
  TRI_CUDA_OK(cudaMemsetAsync(ws, 0, 256, st));
  int* err = static_cast<int*>(ws);
  if (d->dtype == TRI_BF16) {
    if (d->D == 32) return fwd_launch<__nv_bfloat16, 32>(d, q, k, v, bias, mask, o, lse, err, st);
    return fwd_launch<__nv_bfloat16, 64>(d, q, k, v, bias, mask, o, lse, err, st);
  }
  if (d->D == 32) return fwd_launch<__half, 32>(d, q, k, v, bias, mask, o, lse, err, st);
  return fwd_launch<__half, 64>(d, q, k, v, bias, mask, o, lse, err, st);
}

int attn_backward(const TriAttnDesc*, const void*, const void*, const void*, const void*, const uint8_t*,
                  const void*, const float*, const void*, void*, void*, void*, float*, void*, size_t, cudaStream_t) {
  return fail(TRI_ERR_UNSUPPORTED, "no tensor-core attention backward for this problem");
}

}  // namespace tc
}  // namespace tri
