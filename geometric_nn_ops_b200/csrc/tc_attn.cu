// Tensor-core triangle attention (tcgen05 + TMEM + TMA), bf16 / fp16, head dim 32 or 64.
//
// All four kernels share one shape: 320 threads, of which warps 0-7 do the elementwise arithmetic (two threads per
// tile row, each owning half of the tile's columns), warp 8 issues every tcgen05.mma and warp 9 every TMA / bulk
// copy.  The three sides meet only on mbarriers, so the serial issue code never sits between the arithmetic warps'
// steps, and score products for the next tile are issued as soon as the accumulators have been read into registers.
// The arithmetic is packed fp32x2 (fma.rn.f32x2 and friends); row constants arrive in the form it adds
// (-m, -log l * log2e, -delta), and additive key-mask terms (0, -1e9, -inf beyond N) come from a small array
// prepared once per call.  With head dim 32 the probabilities (forward) and dS / P^T / dS^T (backward) never touch
// shared memory: they are stored packed into TMEM and read from there as the A operand of the next product, which
// halves the shared-memory traffic that otherwise bounds these kernels.
//
// Forward, per (batch, row, head, 128-query block), per 128-key tile:
//   S = Q K^T (TMEM) -> x = scale*S + mask + bias -> running maximum -> P = 2^((x - m) log2e) -> O_half += P V.
//   Each half of the key tile keeps its own maximum, sum and O accumulator (merged at the end); O stays in TMEM
//   and is rescaled only when a maximum grows by more than 8 ln 2.
// Backward: three deterministic passes, each recomputing P from the saved statistics (see below).
// Semantics follow triangle_attention_torch (geometric_nn_ops_torch/triangle/_reference/triangle_attention.py:28-44):
// bias and the finite -1e9 key-mask sentinel are added in fp32; keys beyond N_res get -inf.
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
  const float* mask_terms;   // [B][S][npad] additive key-mask terms (0, -1e9, or -inf beyond N)
  int npad;                  // N rounded up to 128
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
  static constexpr int OFF_K = OFF_Q + TILE;             // [2]
  static constexpr int OFF_V = OFF_K + 2 * TILE;         // [2]
  static constexpr int OFF_P = OFF_V + 2 * TILE;         // [2] x [128 x 128] (two SW128 blocks of 64 keys): the bias tile
                                                         // arrives here and each thread overwrites it with its P values
  static constexpr int OFF_MB = OFF_P + 2 * 32768;       // [2] x 128 additive key-mask terms
  static constexpr int OFF_X = OFF_MB + 1024;            // [128][2] floats exchanged when the key halves are merged
  static constexpr int OFF_BAR = OFF_X + 1024;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;      // + alignment slack
};

// byte offset of 16-byte chunk `g` (0..15, 8 elements each) of row r inside a [128 x 128] two-block SW128 tile
__device__ __forceinline__ int sw128_chunk(int r, int g) {
  return (g >> 3) * 16384 + r * 128 + (((g & 7) ^ (r & 7)) << 4);
}

// two fp32 -> one packed pair of 16-bit values with a single conversion instruction
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// one packed pair of 16-bit values -> two fp32
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 pair(uint32_t lo, uint32_t hi) { return make_float2(__uint_as_float(lo), __uint_as_float(hi)); }
__device__ __forceinline__ float2 splat(float v) { return make_float2(v, v); }

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  union { uint4 u; T h[8]; } pk;
  pk.u = v;
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f32(pk.h[i]);
}

// additive key-mask terms of every (batch, row): 0 for a kept key, -1e9 for a masked key, -inf beyond N; rows of npad
__global__ void mask_terms_kernel(const uint8_t* __restrict__ mask, int64_t st_b, int64_t st_s, int B, int S, int N, int npad,
                                  float* __restrict__ out) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)B * S * npad) return;
  const int k = idx % npad;
  const long long bs = idx / npad;
  const int s = bs % S, b = bs / S;
  float v = 0.f;
  if (k >= N) v = -INFINITY;
  else if (mask != nullptr) v = kMaskSentinel * ((mask[b * st_b + s * st_s + k] ? 1.0f : 0.0f) - 1.0f);
  out[idx] = v;
}

// 320 threads.  Warps 0-7 do the softmax arithmetic: thread (r, hh) owns query row r and the 64-key half hh of each
// 128-key tile, with its own running maximum and sum and its own output accumulator O_hh in TMEM; the halves are
// merged once at the end.  Warp 8 issues the MMAs, warp 9 the TMA copies.  The sides meet on mbarriers:
//   bar_s    MMA -> threads      S = Q K^T of a tile is in TMEM
//   bar_free threads -> MMA, TMA every warp has its logits in registers (next tile's S and K may follow)
//   bar_p    threads -> MMA      P of the tile is in shared memory and O has its final scale (P V may start)
//   bar_pv   MMA -> TMA, threads P V is done: its V stage and P buffer are free and O is current
// The bias tile of step j lands in buffer j & 1 and each thread overwrites its own part with P, so P is double
// buffered at no cost and the threads never wait for P V except to rescale O.
// O stays in TMEM across tiles.  It is rescaled only when a row's maximum grows by more than kRescale, so the
// stored maximum may be stale by up to that much: P <= e^kRescale = 256, and the row sum uses the same maximum.
constexpr float kRescale = 5.545177444f;   // 8 ln 2

template <typename T, int HD, bool HB>
__global__ void __launch_bounds__(320, 2)
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
  float* sMb = reinterpret_cast<float*>(smem + G::OFF_MB);
  float* sX = reinterpret_cast<float*>(smem + G::OFF_X);   // [128][2]: maximum and sum of key half 1, for the merge
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + G::OFF_BAR);
  uint64_t* bar_k = bar_q + 1;      // [2] K tile + mask terms
  uint64_t* bar_v = bar_q + 3;      // [2]
  uint64_t* bar_bias = bar_q + 5;   // [2]
  uint64_t* bar_s = bar_q + 7;
  uint64_t* bar_pv = bar_q + 8;     // [2]: tile c commits to bar_pv[c & 1]
  uint64_t* bar_free = bar_q + 10;  // [4]: tile c arrives on bar_free[c & 3] (the copy warp may lag the threads by up to
                                    // two tiles, so two tiles that share a barrier are never both pending)
  uint64_t* bar_p = bar_q + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 15);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = tid & 127, hh = (tid >> 7) & 1;
  const int qblocks = (a.N + 127) / 128;
  const int nt = (a.N + 127) / 128;
  // Persistent: this CTA takes work items blockIdx.x, blockIdx.x + gridDim.x, ... (an item = one (batch, row, head,
  // 128-query block)) and treats their key tiles as one stream c = 0, 1, ...: the copy warp runs two tiles ahead
  // across item boundaries, and TMEM, barriers and the pipeline survive from one item to the next.
  const long long items = (long long)qblocks * a.H * a.S * a.B;
  const int my_items = blockIdx.x < items ? (int)((items - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
  const int total = my_items * nt;
  struct Item { int q0, h, s, b; };
  auto item_of = [&](int n) {   // (the item count fits 31 bits: 32-bit divisions)
    unsigned z = blockIdx.x + (unsigned)n * gridDim.x;
    Item it;
    it.q0 = (int)(z % (unsigned)qblocks) * 128; z /= (unsigned)qblocks;
    it.h = (int)(z % (unsigned)a.H); z /= (unsigned)a.H;
    it.s = (int)(z % (unsigned)a.S);
    it.b = (int)(z / (unsigned)a.S);
    return it;
  };

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bar_k[i], 1); mbar_init(&bar_v[i], 1); mbar_init(&bar_bias[i], 1); mbar_init(&bar_pv[i], 1); }
    mbar_init(bar_s, 1); mbar_init(bar_p, 8);
    for (int i = 0; i < 4; ++i) mbar_init(&bar_free[i], 8);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t COL_O = 128;   // O_0 at [128, 128 + HD), O_1 at [128 + HD, 128 + 2 HD)
  // With head dim 32 the 256 TMEM columns have room for P itself (two 16-bit values per column) and P V reads it
  // from there, which halves the step's shared-memory traffic.  P is single buffered then: a tile's values are
  // stored once the previous tile's P V is done.
  constexpr bool TMEM_P = HD == 32;
  constexpr uint32_t COL_P = 192;
  bool ok = true;

  if (warp == 9) {
    if (lane == 0) {
      // ---------------------------------- TMA copies ---------------------------------------------
      auto load_q = [&](int n) {
        const Item it = item_of(n);
        mbar_expect_tx(bar_q, G::TILE);
        tma_load_5d(sQ, &tmQ, bar_q, 0, it.h, it.q0, it.s, it.b);
      };
      // tile c of the stream: item `it`, key tile t of that item
      auto load_k = [&](int c, const Item& it, int t) {
        const int stg = c & 1;
        mbar_expect_tx(&bar_k[stg], G::TILE + 512);
        tma_load_5d(sK + stg * G::TILE, &tmK, &bar_k[stg], 0, it.h, t * 128, it.s, it.b);
        bulk_load(sMb + stg * 128, a.mask_terms + ((long long)it.b * a.S + it.s) * a.npad + t * 128, 512, &bar_k[stg]);
      };
      auto load_v = [&](int c, const Item& it, int t) {
        const int stg = c & 1;
        mbar_expect_tx(&bar_v[stg], G::TILE);
        tma_load_5d(sV + stg * G::TILE, &tmV, &bar_v[stg], 0, it.h, t * 128, it.s, it.b);
      };
      auto load_bias = [&](int c, const Item& it, int t) {
        uint64_t* bb = &bar_bias[c & 1];
        uint8_t* dst = sP + (c & 1) * 32768;
        mbar_expect_tx(bb, 32768);
        tma_load_4d(dst, &tmBias, bb, t * 128, it.q0, it.h, it.b * a.bias_b_mul);
        tma_load_4d(dst + 16384, &tmBias, bb, t * 128 + 64, it.q0, it.h, it.b * a.bias_b_mul);
      };
      // (la_n, la_t): item and key tile of the stream position being loaded, two tiles ahead of the consumers
      int la_n = 0, la_t = 0;
      Item la = item_of(0);
      auto advance = [&]() {
        if (++la_t == nt) { la_t = 0; ++la_n; if (la_n < my_items) la = item_of(la_n); }
      };
      if (total > 0) load_q(0);
      for (int c = 0; c < 2 && c < total; ++c) {
        load_k(c, la, la_t);
        if (HB) load_bias(c, la, la_t);
        load_v(c, la, la_t);
        advance();
      }
      int jt = 0, n_cur = 0;   // key tile and item of stream position c
      for (int c = 0; c < total && ok; ++c) {
        ok = mbar_wait(&bar_free[c & 3], (c >> 2) & 1, a.err, 16) && ok;   // S(c) has been read: its K stage and mask terms are free
        if (++jt == nt) {                                    // ... and it was the item's last use of Q
          jt = 0;
          if (++n_cur < my_items) load_q(n_cur);
        }
        if (c + 2 < total) {
          load_k(c + 2, la, la_t);
          if (HB && TMEM_P) load_bias(c + 2, la, la_t);      // the bias tile has been read too and P does not replace it
          ok = mbar_wait(&bar_pv[c & 1], (c >> 1) & 1, a.err, 15) && ok;   // P V(c) done: its V stage and P buffer are free
          if (HB && !TMEM_P) load_bias(c + 2, la, la_t);
          load_v(c + 2, la, la_t);
          advance();
        }
      }
    }
  } else if (warp == 8) {
    if (lane == 0) {
      // ---------------------------------- MMA issue ----------------------------------------------
      constexpr uint32_t HI_KMAJ = desc_hi(G::SBO, G::LAYOUT);
      constexpr uint32_t HI_P = desc_hi(1024, 2);
      const uint32_t q_lo = desc_lo(smem_u32(sQ), 16), k_lo = desc_lo(smem_u32(sK), 16);
      const uint32_t p_lo = desc_lo(smem_u32(sP), 16), vmn_lo = desc_lo(smem_u32(sV), 128 * G::RB);   // V as [n = d, k = key]
      int s_t = 0, s_n = 0;   // key tile and item of the next S product
      auto issue_s = [&](int c) {
        if (s_t == 0) ok = mbar_wait(bar_q, s_n & 1, a.err, 11) && ok;   // first tile of an item: its Q
        if (++s_t == nt) { s_t = 0; ++s_n; }
        ok = mbar_wait(&bar_k[c & 1], (c >> 1) & 1, a.err, 12) && ok;
        tc_fence_after_sync();
        const uint32_t so = (c & 1) * (G::TILE >> 4);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma<KIND_F16>(tmem_base, desc_join(q_lo + ks * 2, HI_KMAJ), desc_join(k_lo + so + ks * 2, HI_KMAJ), a.idesc_s, ks > 0);
        umma_commit(bar_s);
      };
      if (total > 0) issue_s(0);
      int j = 0;
      for (int c = 0; c < total && ok; ++c, j = (j + 1 == nt ? 0 : j + 1)) {
        const int stg = c & 1;
        ok = mbar_wait(&bar_free[c & 3], (c >> 2) & 1, a.err, 16) && ok;   // logits of tile c are in registers
        if (c + 1 < total) issue_s(c + 1);
        ok = mbar_wait(bar_p, c & 1, a.err, 17) && ok;
        ok = mbar_wait(&bar_v[stg], (c >> 1) & 1, a.err, 18) && ok;
        tc_fence_after_sync();
        const uint32_t so = stg * (G::TILE >> 4), po = stg * (32768 >> 4);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // O_half += P[:, half] V[half]: keys 64 * (kk >> 2) + 16 * (kk & 3) ...
          const uint64_t vd = desc_join(vmn_lo + so + kk * G::RB, HI_KMAJ);
          const uint32_t accf = (j > 0 || (kk & 3) > 0) ? 1u : 0u;
          if constexpr (TMEM_P) umma_ts_f16(tmem_base + COL_O + (kk >> 2) * HD, tmem_base + COL_P + kk * 8, vd, a.idesc_pv, accf);
          else umma<KIND_F16>(tmem_base + COL_O + (kk >> 2) * HD, desc_join(p_lo + po + (kk >> 2) * 1024 + (kk & 3) * 2, HI_P), vd, a.idesc_pv, accf);
        }
        umma_commit(&bar_pv[stg]);
      }
    }
  } else {
    // ------------------------------------ softmax warps ------------------------------------------
    const float2 sc2 = splat(a.scale), l2e2 = splat(kLog2e);
    const uint32_t t_o = t_row + COL_O + hh * HD;   // this thread's output accumulator row
    for (int n = 0; n < my_items; ++n) {
      const Item it = item_of(n);
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < nt; ++j) {
        const int c = n * nt + j, stg = c & 1;
        ok = mbar_wait(bar_s, c & 1, a.err, 13) && ok;
        tc_fence_after_sync();
        ok = mbar_wait(&bar_k[stg], (c >> 1) & 1, a.err, 12) && ok;   // the tile's mask terms
        if (HB) ok = mbar_wait(&bar_bias[stg], (c >> 1) & 1, a.err, 14) && ok;
        uint8_t* sPj = sP + stg * 32768;   // holds the bias tile; with P in shared memory, P when this step is done

        // ---- logits of this thread's 64 keys into registers, their maximum ----------------------------
        float2 x2[32];
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains
        const float4* sMb4 = reinterpret_cast<const float4*>(sMb + stg * 128 + hh * 64);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t rr[32];
          tmem_ld_32x32(t_row + hh * 64 + cc * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if constexpr (HB) raw = *reinterpret_cast<const uint4*>(sPj + sw128_chunk(r, hh * 8 + cc * 4 + u));
            const uint32_t bw[4] = {raw.x, raw.y, raw.z, raw.w};
            const float4 mA = sMb4[cc * 8 + u * 2], mB = sMb4[cc * 8 + u * 2 + 1];
            const float2 mk[4] = {make_float2(mA.x, mA.y), make_float2(mA.z, mA.w), make_float2(mB.x, mB.y),
                                  make_float2(mB.z, mB.w)};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float2 v = __ffma2_rn(pair(rr[u * 8 + 2 * i], rr[u * 8 + 2 * i + 1]), sc2, mk[i]);
              if constexpr (HB) v = __fadd2_rn(v, unpack2<T>(bw[i]));
              x2[cc * 16 + u * 4 + i] = v;
              mx4[i] = fmax3(mx4[i], v.x, v.y);
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_free[c & 3]);

        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const bool grow = mx > m_run + kRescale;          // (always true on the first tile with a key in range)
        const float m_new = grow ? mx : m_run;
        if (j > 0 && __any_sync(0xffffffffu, grow)) {     // tcgen05.ld / st are warp-wide: rows that keep their maximum scale by 1
          ok = mbar_wait(&bar_pv[(c - 1) & 1], ((c - 1) >> 1) & 1, a.err, 15) && ok;   // O is current
          tc_fence_after_sync();
          const float alpha = grow ? ex2_approx((m_run - m_new) * kLog2e) : 1.0f;   // m_run = -inf gives 0 (O_hh is 0 then)
          l_run *= alpha;
#pragma unroll
          for (int cc = 0; cc < HD / 16; ++cc) {
            uint32_t o[16];
            tmem_ld_32x16(t_o + cc * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(t_o + cc * 16, o);
          }
          tmem_st_wait();
        }
        m_run = m_new;

        // ---- P = 2^((x - m) log2e), its row sum; P rounded to the input dtype -----------------------------
        const float2 nm2 = splat(m_new == -INFINITY ? 0.f : -m_new);   // a half with no key in range yet: P = 2^-inf = 0
        float2 ps2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        uint32_t pw[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 e = __fmul2_rn(__fadd2_rn(x2[g * 4 + i], nm2), l2e2);
            const float2 pp = make_float2(ex2_approx(e.x), ex2_approx(e.y));
            ps2[i & 1] = __fadd2_rn(ps2[i & 1], pp);
            pw[g * 4 + i] = pack2<T>(pp.x, pp.y);
          }
          if constexpr (!TMEM_P)
            *reinterpret_cast<uint4*>(sPj + sw128_chunk(r, hh * 8 + g)) = make_uint4(pw[g * 4], pw[g * 4 + 1], pw[g * 4 + 2], pw[g * 4 + 3]);
        }
        l_run += (ps2[0].x + ps2[0].y) + (ps2[1].x + ps2[1].y);
        if constexpr (TMEM_P) {
          if (c > 0) ok = mbar_wait(&bar_pv[(c - 1) & 1], ((c - 1) >> 1) & 1, a.err, 15) && ok;   // the previous P has been read
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {   // this thread's query row, its 64 keys as 32 packed columns
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) w[i] = pw[cc * 16 + i];
            tmem_st_32x16(t_row + COL_P + hh * 32 + cc * 16, w);
          }
          tmem_st_wait();
        } else {
          fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p);
        if (!ok) break;
      }
      if (!ok) break;

      // ---- merge the two key halves of each row and write O, the row maximum and log row sum -------------
      // Both halves' accumulators sit in this row's TMEM lane; only the maximum and sum of half 1 cross threads.
      // The next item's first P V, which overwrites O, is issued only after every warp has arrived on bar_p
      // for that tile, hence after this.
      const int cl = n * nt + nt - 1;
      ok = mbar_wait(&bar_pv[cl & 1], (cl >> 1) & 1, a.err, 15) && ok;
      tc_fence_after_sync();
      if (hh == 1) { sX[2 * r] = m_run; sX[2 * r + 1] = l_run; }
      named_barrier(1, 256);
      if (hh == 0) {
        const float m1 = sX[2 * r], l1 = sX[2 * r + 1];
        const float m = fmaxf(m_run, m1);   // finite: key 0 is in range and belongs to half 0
        const float a0 = ex2_approx((m_run - m) * kLog2e), a1 = ex2_approx((m1 - m) * kLog2e);
        const float l = l_run * a0 + l1 * a1;
        const float inv = 1.0f / l, w0 = a0 * inv, w1 = a1 * inv;
        const int qi = it.q0 + r;
        const bool st_ok = qi < a.N && ok;
        T* orow = reinterpret_cast<T*>(a.o) + it.b * a.o_st[0] + it.s * a.o_st[1] + qi * a.o_st[2] + it.h * a.o_st[3];
#pragma unroll
        for (int cc = 0; cc < HD / 16; ++cc) {   // tcgen05.ld is warp-wide: every row loads, valid rows store
          uint32_t o0[16], o1[16];
          tmem_ld_32x16(t_row + COL_O + cc * 16, o0);
          tmem_ld_32x16(t_row + COL_O + HD + cc * 16, o1);
          tmem_ld_wait();
          if (st_ok) {
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o0[g * 8 + i]) * w0 + __uint_as_float(o1[g * 8 + i]) * w1;
              uint4 pk;
              pk.x = pack2<T>(f[0], f[1]); pk.y = pack2<T>(f[2], f[3]);
              pk.z = pack2<T>(f[4], f[5]); pk.w = pack2<T>(f[6], f[7]);
              reinterpret_cast<uint4*>(orow)[cc * 2 + g] = pk;
            }
          }
        }
        if (st_ok) {
          const long long srow = (((long long)it.b * a.S + it.s) * a.H + it.h) * a.N + qi;
          a.stats[srow] = m;
          a.stats[(long long)a.B * a.S * a.H * a.N + srow] = logf(l);
        }
      }
      tc_fence_before_sync();   // orders this item's TMEM reads before the arrivals that let the next item overwrite O
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// =================================================================================================
// Backward.  Three deterministic passes, each recomputing P from the saved statistics:
//   dK/dV : one CTA per (b, row, head, 128-key block), thread = key.  Per 64-query tile:
//           S^T = K Q^T and dP^T = V dO^T (TMEM), P^T and dS^T packed (TMEM or smem), dV += P^T dO, dK += dS^T Q.
//           The bias is read from a transposed copy so that a thread's queries are contiguous.
//   dQ    : one CTA per (b, row, head, 128-query block), thread = query.  Per 64-key tile:
//           S = Q K^T, dP = dO V^T, dS packed into TMEM, dQ += dS K.
//   dbias : one CTA per (row chunk, b, head, 128-query block, 64-key block) looping over its rows in order and
//           summing dS in registers (no atomics: fixed order), S / dP double buffered in TMEM.
// P = exp((x - m) - log l), dS = P * (dP - delta), delta = sum_d dO*O (computed by a small kernel first).
// =================================================================================================
struct AttnBwdArgs {
  int B, S, N, H;
  float scale;
  const float* stats;    // [2][B][S][H][N]
  const float* delta;    // [B][S][H][N]
  const float* prep;     // [3][B][S][H][npad]: -m, -log l * log2e, -delta, zero in the padding
  long long prep_plane;  // B*S*H*npad
  int npad;              // N rounded up to 128
  const float* mask_terms;   // [B][S][npad] additive key-mask terms (0, -1e9, or -inf beyond N)
  const uint8_t* mask;
  int64_t mask_st[2];
  int bias_b_mul;        // 0 when the bias is broadcast over the batch
  void* out0;            // dq (MODE_DQ), dk (dK/dV kernel), dbias fp32 (MODE_DBIAS)
  void* out1;            // dv
  int64_t out0_st[4], out1_st[4];
  uint32_t idesc_a, idesc_b;   // the two MMA shapes of the kernel
  uint32_t idesc_c;            // merged dK/dV + dQ pass: the dQ product (both operands MN-major)
  void* dq_part;               // merged pass: per key block, dS K of that block: [key blocks][B][S][N][H][D] in the input dtype
  long long dq_part_plane;     // elements per key block
  int row_chunks;              // MODE_DBIAS: the row loop is split into this many CTAs, each writing its own partial
  int* err;
};

// byte offset of 16-byte chunk g (0..7) of row r inside a one-block SW128 tile (rows of 64 16-bit elements)
__device__ __forceinline__ int sw128_chunk1(int r, int g) { return r * 128 + ((g ^ (r & 7)) << 4); }

template <int HD> struct GeoC {
  static constexpr int RB = HD * 2;
  static constexpr int TK = 128 * RB;   // K / V tile
  static constexpr int TQ = 64 * RB;    // Q / dO tile
  static constexpr uint32_t LAYOUT = RB == 128 ? 2 : 4;
  static constexpr uint32_t SBO = 8 * RB;
  static constexpr int NQ = 3;                      // query-tile stages: tiles are fetched two steps ahead
  static constexpr int ST = 3 * 64 * 4;             // one stage of row statistics: -m, -log l log2e, -delta for 64 queries
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TK;
  static constexpr int OFF_Q = OFF_V + TK;          // [NQ]
  static constexpr int OFF_DO = OFF_Q + NQ * TQ;    // [NQ]
  static constexpr int OFF_PT = OFF_DO + NQ * TQ;   // [2] x [128 keys x 64 queries] SW128: the transposed bias tile arrives
                                                    // here and each thread overwrites its part with P^T
  static constexpr int OFF_DST = OFF_PT + 2 * 16384;    // [2] x dS^T, same shape
  static constexpr int OFF_ST = OFF_DST + 2 * 16384;    // [NQ] statistics stages
  static constexpr int OFF_BAR = OFF_ST + NQ * ST;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
};

// 320 threads.  Warps 0-7 do the arithmetic: thread (r, hh) owns key r of the block and query half hh of each
// 64-query tile.  Warp 8 issues the MMAs and warp 9 the TMA copies, so none of that serial code sits between the
// arithmetic warps' steps; the sides meet only on mbarriers:
//   bar_s    MMA -> threads      S^T and dP^T of a tile are in TMEM
//   bar_free threads -> MMA      every warp has read them into registers (the next tile's products may start)
//   bar_p    threads -> MMA      P^T and dS^T of the tile are in shared memory (dV, dK products may start)
//   bar_acc  MMA -> TMA, threads those products are done: the tile's stage and its P^T / dS^T buffers are free
// P^T and dS^T are double buffered (P^T over the bias tile it was computed from), so the threads do not wait for
// the dV / dK products of one tile before the arithmetic of the next.
//
// MERGE (head dim 32): the same pass also produces this key block's share of dQ, so that S, the exponentials and dP
// are computed once for dK, dV and dQ instead of once per gradient.  dS^T then goes to shared memory ([128 keys x 64
// queries], the two buffers of a pair of query tiles 16 KB apart) instead of TMEM: dK reads it K-major as before, and
// after every second tile one product dQ_pair[128 queries x D] = dS_pair K reads the pair MN-major (M = queries) with
// K as the MN-major B operand, into the TMEM columns dS^T no longer needs.  The arithmetic warps fetch that
// accumulator one step later and store it, unscaled, as this key block's partial; attn_dq_sum_kernel adds the key
// blocks' partials in fixed order.  A last tile without a partner is paired with a buffer of zeros.
template <typename T, int HD, bool HB, bool MERGE>
__global__ void __launch_bounds__(320, 2)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmBias, const AttnBwdArgs a) {
  using G = GeoC<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + G::OFF_K;
  uint8_t* sV = smem + G::OFF_V;
  uint8_t* sQ = smem + G::OFF_Q;
  uint8_t* sDO = smem + G::OFF_DO;
  uint8_t* sPT = smem + G::OFF_PT;
  uint8_t* sDST = smem + G::OFF_DST;
  float* sStats = reinterpret_cast<float*>(smem + G::OFF_ST);   // [NQ][3][64]
  uint64_t* bar_kv = reinterpret_cast<uint64_t*>(smem + G::OFF_BAR);
  uint64_t* bar_in = bar_kv + 1;     // [NQ]
  uint64_t* bar_bias = bar_kv + 4;   // [2]
  uint64_t* bar_s = bar_kv + 6;
  uint64_t* bar_acc = bar_kv + 7;    // [4]: tile j commits to bar_acc[j & 3] (the copy warp may lag the MMA warp by up to
                                     // three tiles, so two tiles that share a barrier are never both pending)
  uint64_t* bar_free = bar_kv + 11;
  uint64_t* bar_p = bar_kv + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_kv + 13);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = tid & 127, hh = (tid >> 7) & 1;
  const int kblocks = (a.N + 127) / 128;
  int z = blockIdx.x;
  const int kvb = z % kblocks; z /= kblocks;
  const int h = z % a.H; z /= a.H;
  const int s = z % a.S;
  const int b = z / a.S;
  const int k0 = kvb * 128;
  const int nsteps = (a.N + 63) / 64;
  const int bias_b = b * a.bias_b_mul;

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    for (int i = 0; i < G::NQ; ++i) mbar_init(&bar_in[i], 1);
    mbar_init(&bar_bias[0], 1); mbar_init(&bar_bias[1], 1); mbar_init(bar_s, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bar_acc[i], 1);
    mbar_init(bar_free, 8); mbar_init(bar_p, 8);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t COL_DP = 64, COL_DV = 128, COL_DK = 128 + HD;
  // With head dim 32 the 256 TMEM columns have room for P^T and dS^T themselves (two 16-bit values per column), and
  // the dV / dK products read them from there: half the shared-memory traffic of the step, which is what bounds it.
  // They are single buffered, so a tile's values are stored once the previous tile's products are done.
  constexpr bool TMEM_A = HD == 32;
  constexpr uint32_t COL_PT = 192, COL_DST = 224;
  constexpr uint32_t COL_DQ = COL_DST;   // MERGE: dS^T lives in shared memory and its columns hold the dQ accumulator
  static_assert(!MERGE || TMEM_A, "the merged pass is built for head dim 32");
  bool ok = true;

  if (warp == 9) {
    if (lane == 0) {
      // ---------------------------------- TMA copies ---------------------------------------------
      const float* prep_row = a.prep + ((((long long)b * a.S + s) * a.H + h) * (long long)a.npad);
      auto load_step = [&](int step) {
        const int stg = step % G::NQ;
        float* st = sStats + stg * 192;
        mbar_expect_tx(&bar_in[stg], 2 * G::TQ + G::ST);
        tma_load_5d(sQ + stg * G::TQ, &tmQ, &bar_in[stg], 0, h, step * 64, s, b);
        tma_load_5d(sDO + stg * G::TQ, &tmDO, &bar_in[stg], 0, h, step * 64, s, b);
        bulk_load(st, prep_row + step * 64, 256, &bar_in[stg]);
        bulk_load(st + 64, prep_row + a.prep_plane + step * 64, 256, &bar_in[stg]);
        bulk_load(st + 128, prep_row + 2 * a.prep_plane + step * 64, 256, &bar_in[stg]);
      };
      auto load_bias = [&](int step) {
        uint64_t* bb = &bar_bias[step & 1];
        mbar_expect_tx(bb, 16384);
        tma_load_4d(sPT + (step & 1) * 16384, &tmBias, bb, step * 64, k0, h, bias_b);   // transposed copy: queries inner
      };
      mbar_expect_tx(bar_kv, 2 * G::TK);
      tma_load_5d(sK, &tmK, bar_kv, 0, h, k0, s, b);
      tma_load_5d(sV, &tmV, bar_kv, 0, h, k0, s, b);
      for (int st = 0; st < G::NQ && st < nsteps; ++st) {
        load_step(st);
        if (HB && st < 2) load_bias(st);
      }
      for (int j = 0; j + 2 < nsteps && ok; ++j) {
        ok = mbar_wait(&bar_acc[j & 3], (j >> 2) & 1, a.err, 39) && ok;   // tile j's dV / dK products are done
        if (HB) load_bias(j + 2);                                         // its P^T buffer is free
        if (j + 3 < nsteps) load_step(j + 3);                             // ... and its Q / dO / statistics stage
      }
    }
  } else if (warp == 8) {
    if (lane == 0) {
      // ---------------------------------- MMA issue ----------------------------------------------
      // Descriptors are built once: the high word is a constant per operand kind, the low word is
      // (address >> 4) plus the leading-dimension field, so a k-step or a stage only adds to it.
      constexpr uint32_t HI_KMAJ = desc_hi(G::SBO, G::LAYOUT);   // K, V, Q, dO as K-major rows of RB bytes
      constexpr uint32_t HI_PT = desc_hi(1024, 2);               // P^T, dS^T: [128 x 64] SW128
      const uint32_t k_lo = desc_lo(smem_u32(sK), 16), v_lo = desc_lo(smem_u32(sV), 16);
      const uint32_t q_lo = desc_lo(smem_u32(sQ), 16), do_lo = desc_lo(smem_u32(sDO), 16);
      const uint32_t qmn_lo = desc_lo(smem_u32(sQ), 64 * G::RB), domn_lo = desc_lo(smem_u32(sDO), 64 * G::RB);   // MN-major view
      const uint32_t pt_lo = desc_lo(smem_u32(sPT), 16), dst_lo = desc_lo(smem_u32(sDST), 16);
      const uint32_t dsmn_lo = desc_lo(smem_u32(sDST), 16384);      // dS of a tile pair as [m = query, k = key]: MN-major A
      const uint32_t kmn_lo = desc_lo(smem_u32(sK), 128 * G::RB);   // K as [n = d, k = key]: MN-major B
      // S^T = K Q^T and dP^T = V dO^T of one 64-query tile
      auto issue_scores = [&](int step) {
        const int stg = step % G::NQ;
        ok = mbar_wait(&bar_in[stg], (step / G::NQ) & 1, a.err, 32) && ok;
        tc_fence_after_sync();
        const uint32_t so = stg * (G::TQ >> 4);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma<KIND_F16>(tmem_base, desc_join(k_lo + ks * 2, HI_KMAJ), desc_join(q_lo + so + ks * 2, HI_KMAJ), a.idesc_a, ks > 0);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma<KIND_F16>(tmem_base + COL_DP, desc_join(v_lo + ks * 2, HI_KMAJ), desc_join(do_lo + so + ks * 2, HI_KMAJ), a.idesc_a, ks > 0);
        umma_commit(bar_s);
      };
      ok = mbar_wait(bar_kv, 0, a.err, 31);
      issue_scores(0);
      for (int j = 0; j < nsteps && ok; ++j) {
        const int qstg = j % G::NQ;
        ok = mbar_wait(bar_free, j & 1, a.err, 37) && ok;
        if (j + 1 < nsteps) issue_scores(j + 1);
        ok = mbar_wait(bar_p, j & 1, a.err, 38) && ok;
        tc_fence_after_sync();
        const uint32_t so = qstg * (G::TQ >> 4), bo = (j & 1) * (16384 >> 4);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {   // dV += P^T dO   (B = dO as [n = d, k = query]: MN-major)
          const uint64_t bd = desc_join(domn_lo + so + kk * G::RB, HI_KMAJ);
          const uint32_t accf = (j > 0 || kk > 0) ? 1u : 0u;
          if constexpr (TMEM_A) umma_ts_f16(tmem_base + COL_DV, tmem_base + COL_PT + kk * 8, bd, a.idesc_b, accf);
          else umma<KIND_F16>(tmem_base + COL_DV, desc_join(pt_lo + bo + kk * 2, HI_PT), bd, a.idesc_b, accf);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {   // dK += dS^T Q
          const uint64_t bd = desc_join(qmn_lo + so + kk * G::RB, HI_KMAJ);
          const uint32_t accf = (j > 0 || kk > 0) ? 1u : 0u;
          if constexpr (TMEM_A && !MERGE) umma_ts_f16(tmem_base + COL_DK, tmem_base + COL_DST + kk * 8, bd, a.idesc_b, accf);
          else umma<KIND_F16>(tmem_base + COL_DK, desc_join(dst_lo + bo + kk * 2, HI_PT), bd, a.idesc_b, accf);
        }
        if constexpr (MERGE) {
          if ((j & 1) || j == nsteps - 1) {   // a pair of query tiles is complete: dQ_pair = dS_pair K (16 keys per product)
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma<KIND_F16>(tmem_base + COL_DQ, desc_join(dsmn_lo + ks * 128, HI_PT), desc_join(kmn_lo + ks * G::RB, HI_KMAJ),
                             a.idesc_c, ks > 0);
          }
        }
        umma_commit(&bar_acc[j & 3]);
      }
    }
  } else {
    // ------------------------------------ arithmetic warps ---------------------------------------
    const int kj = k0 + r;
    float mb = 0.f;
    if (kj >= a.N) mb = -INFINITY;
    else if (a.mask != nullptr) mb = kMaskSentinel * ((a.mask[b * a.mask_st[0] + s * a.mask_st[1] + kj] ? 1.0f : 0.0f) - 1.0f);
    const float2 sc2 = splat(a.scale), mk2 = splat(mb), l2e2 = splat(kLog2e);
    // MERGE: fetch the dQ accumulator of query-tile pair `pair` (row r = query 128 pair + r, this thread's half of the
    // head dim) and store it, unscaled, as this key block's partial.  tcgen05.ld is warp-wide: every thread loads.
    auto store_dq_pair = [&](int pair) {
      uint32_t v[16];
      tmem_ld_32x16(t_row + COL_DQ + hh * 16, v);
      tmem_ld_wait();
      const int qi = pair * 128 + r;
      if (qi < a.N && ok) {
        T* dst = reinterpret_cast<T*>(a.dq_part) + kvb * a.dq_part_plane +
                 ((((long long)b * a.S + s) * a.N + qi) * a.H + h) * HD + hh * 16;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint4 pk;
          pk.x = pack2<T>(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
          pk.y = pack2<T>(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
          pk.z = pack2<T>(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
          pk.w = pack2<T>(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
          reinterpret_cast<uint4*>(dst)[g] = pk;
        }
      }
    };

    for (int j = 0; j < nsteps; ++j) {
      const int stg = j & 1, qstg = j % G::NQ;
      ok = mbar_wait(bar_s, j & 1, a.err, 33) && ok;
      tc_fence_after_sync();
      ok = mbar_wait(&bar_in[qstg], (j / G::NQ) & 1, a.err, 32) && ok;   // the tile's row statistics
      if (HB) ok = mbar_wait(&bar_bias[stg], (j >> 1) & 1, a.err, 34) && ok;

      // packed fp32x2 arithmetic: P = 2^((x - m) log2e - log l log2e), dS = P (dP - delta); thread = key, columns = queries
      uint8_t* sPTj = sPT + stg * 16384;     // holds the transposed bias tile now, P^T when this step is done
      uint8_t* sDSTj = sDST + stg * 16384;   // (its last readers, tile j-2's products, finished before S^T(j) did)
      const float4* sM4 = reinterpret_cast<const float4*>(sStats + qstg * 192);
      const float4* sL4 = sM4 + 16;
      const float4* sD4 = sM4 + 32;
      const int c = hh;
      uint32_t pw[16], dw[16];
      // 16 of this thread's 32 queries
      auto half = [&](const uint32_t (&rs)[16], const uint32_t (&rp)[16], int h2) {
#pragma unroll
        for (int uu = 0; uu < 2; ++uu) {
          const int u = h2 * 2 + uu;
          uint4 raw = make_uint4(0, 0, 0, 0);
          if constexpr (HB) raw = *reinterpret_cast<const uint4*>(sPTj + sw128_chunk1(r, c * 4 + u));
          const uint32_t bw[4] = {raw.x, raw.y, raw.z, raw.w};
          const float4 m0 = sM4[c * 8 + u * 2], m1 = sM4[c * 8 + u * 2 + 1];
          const float4 l0 = sL4[c * 8 + u * 2], l1 = sL4[c * 8 + u * 2 + 1];
          const float4 d0 = sD4[c * 8 + u * 2], d1 = sD4[c * 8 + u * 2 + 1];
          const float2 nm[4] = {make_float2(m0.x, m0.y), make_float2(m0.z, m0.w), make_float2(m1.x, m1.y), make_float2(m1.z, m1.w)};
          const float2 nl[4] = {make_float2(l0.x, l0.y), make_float2(l0.z, l0.w), make_float2(l1.x, l1.y), make_float2(l1.z, l1.w)};
          const float2 nd[4] = {make_float2(d0.x, d0.y), make_float2(d0.z, d0.w), make_float2(d1.x, d1.y), make_float2(d1.z, d1.w)};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 x = __ffma2_rn(pair(rs[uu * 8 + 2 * i], rs[uu * 8 + 2 * i + 1]), sc2, mk2);
            if constexpr (HB) x = __fadd2_rn(x, unpack2<T>(bw[i]));
            const float2 e = __ffma2_rn(__fadd2_rn(x, nm[i]), l2e2, nl[i]);
            const float2 pp = make_float2(ex2_approx(e.x), ex2_approx(e.y));
            const float2 ds = __fmul2_rn(pp, __fadd2_rn(pair(rp[uu * 8 + 2 * i], rp[uu * 8 + 2 * i + 1]), nd[i]));
            pw[u * 4 + i] = pack2<T>(pp.x, pp.y);
            dw[u * 4 + i] = pack2<T>(ds.x, ds.y);
          }
          if constexpr (!TMEM_A) {
            *reinterpret_cast<uint4*>(sPTj + sw128_chunk1(r, c * 4 + u)) = make_uint4(pw[u * 4], pw[u * 4 + 1], pw[u * 4 + 2], pw[u * 4 + 3]);
            *reinterpret_cast<uint4*>(sDSTj + sw128_chunk1(r, c * 4 + u)) = make_uint4(dw[u * 4], dw[u * 4 + 1], dw[u * 4 + 2], dw[u * 4 + 3]);
          }
        }
      };
      // the second half's TMEM loads are in flight while the first half is computed
      uint32_t rsA[16], rpA[16], rsB[16], rpB[16];
      tmem_ld_32x16(t_row + hh * 32, rsA);
      tmem_ld_32x16(t_row + COL_DP + hh * 32, rpA);
      tmem_ld_wait();
      tmem_ld_32x16(t_row + hh * 32 + 16, rsB);
      tmem_ld_32x16(t_row + COL_DP + hh * 32 + 16, rpB);
      half(rsA, rpA, 0);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_free);   // this warp holds its logits: the accumulators can take the next tile
      half(rsB, rpB, 1);
      if constexpr (TMEM_A) {
        if (j > 0) ok = mbar_wait(&bar_acc[(j - 1) & 3], ((j - 1) >> 2) & 1, a.err, 35) && ok;   // the previous tile's products have read theirs
        tc_fence_after_sync();
        if constexpr (MERGE) {
          if (j >= 2 && (j & 1) == 0) store_dq_pair(j / 2 - 1);   // the pair before this tile: its dQ product is done too
        }
        tmem_st_32x16(t_row + COL_PT + hh * 16, pw);    // this thread's key row, its 32 queries as 16 packed columns
        if constexpr (MERGE) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            *reinterpret_cast<uint4*>(sDSTj + sw128_chunk1(r, c * 4 + u)) = make_uint4(dw[u * 4], dw[u * 4 + 1], dw[u * 4 + 2], dw[u * 4 + 3]);
          if (j == nsteps - 1 && (j & 1) == 0) {   // no partner tile: the pair's second buffer reads as zeros
#pragma unroll
            for (int u = 0; u < 4; ++u)
              *reinterpret_cast<uint4*>(sDST + 16384 + sw128_chunk1(r, c * 4 + u)) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
        } else {
          tmem_st_32x16(t_row + COL_DST + hh * 16, dw);
        }
        tmem_st_wait();
      } else {
        fence_proxy_async_smem();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      if (!ok) break;
    }
    ok = mbar_wait(&bar_acc[(nsteps - 1) & 3], ((nsteps - 1) >> 2) & 1, a.err, 36) && ok;
    tc_fence_after_sync();
    if constexpr (MERGE) store_dq_pair((nsteps - 1) / 2);   // the last pair
    {
      const bool st_ok = kj < a.N && ok && hh == 0;
      T* krow = reinterpret_cast<T*>(a.out0) + b * a.out0_st[0] + s * a.out0_st[1] + kj * a.out0_st[2] + h * a.out0_st[3];
      T* vrow = reinterpret_cast<T*>(a.out1) + b * a.out1_st[0] + s * a.out1_st[1] + kj * a.out1_st[2] + h * a.out1_st[3];
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t rk[32], rv[32];
        tmem_ld_32x32(t_row + COL_DK + c * 32, rk);
        tmem_ld_32x32(t_row + COL_DV + c * 32, rv);
        tmem_ld_wait();
        if (st_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 pk;
            pk.x = pack2<T>(__uint_as_float(rk[g * 8 + 0]) * a.scale, __uint_as_float(rk[g * 8 + 1]) * a.scale);
            pk.y = pack2<T>(__uint_as_float(rk[g * 8 + 2]) * a.scale, __uint_as_float(rk[g * 8 + 3]) * a.scale);
            pk.z = pack2<T>(__uint_as_float(rk[g * 8 + 4]) * a.scale, __uint_as_float(rk[g * 8 + 5]) * a.scale);
            pk.w = pack2<T>(__uint_as_float(rk[g * 8 + 6]) * a.scale, __uint_as_float(rk[g * 8 + 7]) * a.scale);
            reinterpret_cast<uint4*>(krow)[c * 4 + g] = pk;
            pk.x = pack2<T>(__uint_as_float(rv[g * 8 + 0]), __uint_as_float(rv[g * 8 + 1]));
            pk.y = pack2<T>(__uint_as_float(rv[g * 8 + 2]), __uint_as_float(rv[g * 8 + 3]));
            pk.z = pack2<T>(__uint_as_float(rv[g * 8 + 4]), __uint_as_float(rv[g * 8 + 5]));
            pk.w = pack2<T>(__uint_as_float(rv[g * 8 + 6]), __uint_as_float(rv[g * 8 + 7]));
            reinterpret_cast<uint4*>(vrow)[c * 4 + g] = pk;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------------
// dQ pass: one CTA per (batch, row, head, 128-query block), 64-key tiles.  320 threads: warps 0-7 do the arithmetic
// (thread (r, hh) owns query r and key half hh of each tile), warp 8 issues the MMAs, warp 9 the TMA copies.
//   S = Q K^T, dP = dO V^T (TMEM) -> dS = P (dP - delta) packed into TMEM -> dQ += dS K (A operand read from TMEM).
// Barriers as in the dK/dV pass: bar_s, bar_free, bar_p, and a ring bar_dq[4] for the dQ products.
// ------------------------------------------------------------------------------------------------
template <int HD> struct GeoQ {
  static constexpr int RB = HD * 2;
  static constexpr int TA = 128 * RB;                    // Q / dO tile
  static constexpr int TB = 64 * RB;                     // K / V tile
  static constexpr uint32_t LAYOUT = RB == 128 ? 2 : 4;
  static constexpr uint32_t SBO = 8 * RB;
  static constexpr int NS = 3;                           // K / V stages: tiles are fetched two steps ahead
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + TA;
  static constexpr int OFF_K = OFF_DO + TA;              // [NS]
  static constexpr int OFF_V = OFF_K + NS * TB;          // [NS]
  static constexpr int OFF_BIAS = OFF_V + NS * TB;       // [2] x [128 queries x 64 keys] SW128
  static constexpr int OFF_MB = OFF_BIAS + 2 * 16384;    // [NS] x 64 additive key-mask terms
  static constexpr int OFF_BAR = OFF_MB + NS * 256;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
};

template <typename T, int HD, bool HB>
__global__ void __launch_bounds__(320, 2)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmBias, const AttnBwdArgs a) {
  using G = GeoQ<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + G::OFF_Q;
  uint8_t* sDO = smem + G::OFF_DO;
  uint8_t* sK = smem + G::OFF_K;
  uint8_t* sV = smem + G::OFF_V;
  uint8_t* sBias = smem + G::OFF_BIAS;
  float* sMb = reinterpret_cast<float*>(smem + G::OFF_MB);
  uint64_t* bar_once = reinterpret_cast<uint64_t*>(smem + G::OFF_BAR);   // Q + dO
  uint64_t* bar_in = bar_once + 1;    // [NS] K, V and mask terms of a tile
  uint64_t* bar_bias = bar_once + 4;  // [2]
  uint64_t* bar_s = bar_once + 6;
  uint64_t* bar_dq = bar_once + 7;    // [4]: tile j commits to bar_dq[j & 3]
  uint64_t* bar_free = bar_once + 11;
  uint64_t* bar_p = bar_once + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_once + 13);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = tid & 127, hh = (tid >> 7) & 1;
  const int qblocks = (a.N + 127) / 128;
  int z = blockIdx.x;
  const int qb = z % qblocks; z /= qblocks;
  const int h = z % a.H; z /= a.H;
  const int s = z % a.S;
  const int b = z / a.S;
  const int q0 = qb * 128;
  const int nsteps = (a.N + 63) / 64;
  const int bias_b = b * a.bias_b_mul;

  if (tid == 0) {
    mbar_init(bar_once, 1);
    for (int i = 0; i < G::NS; ++i) mbar_init(&bar_in[i], 1);
    mbar_init(&bar_bias[0], 1); mbar_init(&bar_bias[1], 1); mbar_init(bar_s, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bar_dq[i], 1);
    mbar_init(bar_free, 8); mbar_init(bar_p, 8);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t COL_DP = 64, COL_DQ = 128, COL_DS = 128 + HD;   // dS: 64 keys as 32 packed columns
  bool ok = true;

  if (warp == 9) {
    if (lane == 0) {
      // ---------------------------------- TMA copies ---------------------------------------------
      const float* mrow = a.mask_terms + ((long long)b * a.S + s) * a.npad;
      auto load_step = [&](int step) {
        const int stg = step % G::NS;
        mbar_expect_tx(&bar_in[stg], 2 * G::TB + 256);
        tma_load_5d(sK + stg * G::TB, &tmK, &bar_in[stg], 0, h, step * 64, s, b);
        tma_load_5d(sV + stg * G::TB, &tmV, &bar_in[stg], 0, h, step * 64, s, b);
        bulk_load(sMb + stg * 64, mrow + step * 64, 256, &bar_in[stg]);
      };
      auto load_bias = [&](int step) {
        uint64_t* bb = &bar_bias[step & 1];
        mbar_expect_tx(bb, 16384);
        tma_load_4d(sBias + (step & 1) * 16384, &tmBias, bb, step * 64, q0, h, bias_b);
      };
      mbar_expect_tx(bar_once, 2 * G::TA);
      tma_load_5d(sQ, &tmQ, bar_once, 0, h, q0, s, b);
      tma_load_5d(sDO, &tmDO, bar_once, 0, h, q0, s, b);
      for (int st = 0; st < G::NS && st < nsteps; ++st) {
        load_step(st);
        if (HB && st < 2) load_bias(st);
      }
      for (int j = 0; j + 2 < nsteps && ok; ++j) {
        ok = mbar_wait(&bar_dq[j & 3], (j >> 2) & 1, a.err, 26) && ok;   // tile j's dQ product is done
        if (HB) load_bias(j + 2);                                        // (its bias tile was read before that)
        if (j + 3 < nsteps) load_step(j + 3);                            // its K / V stage is free
      }
    }
  } else if (warp == 8) {
    if (lane == 0) {
      // ---------------------------------- MMA issue ----------------------------------------------
      constexpr uint32_t HI_KMAJ = desc_hi(G::SBO, G::LAYOUT);
      const uint32_t q_lo = desc_lo(smem_u32(sQ), 16), do_lo = desc_lo(smem_u32(sDO), 16);
      const uint32_t k_lo = desc_lo(smem_u32(sK), 16), v_lo = desc_lo(smem_u32(sV), 16);
      const uint32_t kmn_lo = desc_lo(smem_u32(sK), 64 * G::RB);   // K as [n = d, k = key]
      auto issue_scores = [&](int step) {
        const int stg = step % G::NS;
        ok = mbar_wait(&bar_in[stg], (step / G::NS) & 1, a.err, 23) && ok;
        tc_fence_after_sync();
        const uint32_t so = stg * (G::TB >> 4);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma<KIND_F16>(tmem_base, desc_join(q_lo + ks * 2, HI_KMAJ), desc_join(k_lo + so + ks * 2, HI_KMAJ), a.idesc_a, ks > 0);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma<KIND_F16>(tmem_base + COL_DP, desc_join(do_lo + ks * 2, HI_KMAJ), desc_join(v_lo + so + ks * 2, HI_KMAJ), a.idesc_a, ks > 0);
        umma_commit(bar_s);
      };
      ok = mbar_wait(bar_once, 0, a.err, 22);
      issue_scores(0);
      for (int j = 0; j < nsteps && ok; ++j) {
        ok = mbar_wait(bar_free, j & 1, a.err, 28) && ok;
        if (j + 1 < nsteps) issue_scores(j + 1);
        ok = mbar_wait(bar_p, j & 1, a.err, 29) && ok;
        tc_fence_after_sync();
        const uint32_t so = (j % G::NS) * (G::TB >> 4);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)   // dQ += dS K   (A = dS from TMEM, B = K as [n = d, k = key]: MN-major)
          umma_ts_f16(tmem_base + COL_DQ, tmem_base + COL_DS + kk * 8, desc_join(kmn_lo + so + kk * G::RB, HI_KMAJ), a.idesc_b,
                      (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bar_dq[j & 3]);
      }
    }
  } else {
    // ------------------------------------ arithmetic warps ---------------------------------------
    const int qi = q0 + r;
    const bool q_ok = qi < a.N;
    float m_row = 0.f, l_row = 0.f, d_row = 0.f;
    if (q_ok) {
      const long long plane = (long long)a.B * a.S * a.H * a.N;
      const long long row = (((long long)b * a.S + s) * a.H + h) * a.N + qi;
      m_row = a.stats[row]; l_row = a.stats[plane + row]; d_row = a.delta[row];
    }
    // packed fp32x2 arithmetic: P = 2^((x - m) log2e - log l log2e), dS = P (dP - delta)
    const float2 sc2 = splat(a.scale), nm2 = splat(-m_row), nl2 = splat(-l_row * kLog2e), l2e2 = splat(kLog2e),
                 nd2 = splat(-d_row);

    for (int j = 0; j < nsteps; ++j) {
      const int stg = j & 1, kstg = j % G::NS;
      ok = mbar_wait(bar_s, j & 1, a.err, 24) && ok;
      tc_fence_after_sync();
      ok = mbar_wait(&bar_in[kstg], (j / G::NS) & 1, a.err, 23) && ok;   // the tile's mask terms
      if (HB) ok = mbar_wait(&bar_bias[stg], (j >> 1) & 1, a.err, 25) && ok;
      const float4* sMb4 = reinterpret_cast<const float4*>(sMb + kstg * 64 + hh * 32);
      const uint8_t* bias_t = sBias + stg * 16384;
      uint32_t dw[16];
      // 16 of this thread's 32 columns: dS = P (dP - delta), packed
      auto half = [&](const uint32_t (&rs)[16], const uint32_t (&rp)[16], int h2) {
#pragma unroll
        for (int uu = 0; uu < 2; ++uu) {
          const int u = h2 * 2 + uu;
          uint4 raw = make_uint4(0, 0, 0, 0);
          if constexpr (HB) raw = *reinterpret_cast<const uint4*>(bias_t + sw128_chunk1(r, hh * 4 + u));
          const uint32_t bw[4] = {raw.x, raw.y, raw.z, raw.w};
          const float4 mA = sMb4[u * 2], mB = sMb4[u * 2 + 1];
          const float2 mk[4] = {make_float2(mA.x, mA.y), make_float2(mA.z, mA.w), make_float2(mB.x, mB.y),
                                make_float2(mB.z, mB.w)};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 x = __ffma2_rn(pair(rs[uu * 8 + 2 * i], rs[uu * 8 + 2 * i + 1]), sc2, mk[i]);
            if constexpr (HB) x = __fadd2_rn(x, unpack2<T>(bw[i]));
            const float2 e = __ffma2_rn(__fadd2_rn(x, nm2), l2e2, nl2);
            const float2 p = make_float2(ex2_approx(e.x), ex2_approx(e.y));
            const float2 ds = __fmul2_rn(p, __fadd2_rn(pair(rp[uu * 8 + 2 * i], rp[uu * 8 + 2 * i + 1]), nd2));
            dw[u * 4 + i] = pack2<T>(ds.x, ds.y);
          }
        }
      };
      // the second half's TMEM loads are in flight while the first half is computed
      uint32_t rsA[16], rpA[16], rsB[16], rpB[16];
      tmem_ld_32x16(t_row + hh * 32, rsA);
      tmem_ld_32x16(t_row + COL_DP + hh * 32, rpA);
      tmem_ld_wait();
      tmem_ld_32x16(t_row + hh * 32 + 16, rsB);
      tmem_ld_32x16(t_row + COL_DP + hh * 32 + 16, rpB);
      half(rsA, rpA, 0);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_free);   // this warp holds its logits: the accumulators can take the next tile
      half(rsB, rpB, 1);
      if (j > 0) ok = mbar_wait(&bar_dq[(j - 1) & 3], ((j - 1) >> 2) & 1, a.err, 26) && ok;   // the previous dS has been read
      tc_fence_after_sync();
      tmem_st_32x16(t_row + COL_DS + hh * 16, dw);   // this thread's query row, its 32 keys as 16 packed columns
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      if (!ok) break;
    }
    ok = mbar_wait(&bar_dq[(nsteps - 1) & 3], ((nsteps - 1) >> 2) & 1, a.err, 27) && ok;
    tc_fence_after_sync();
    {
      // tcgen05.ld is warp-collective: every thread loads, only valid rows store; the halves split the head dim
      const bool st_ok = q_ok && ok;
      T* row = reinterpret_cast<T*>(a.out0) + b * a.out0_st[0] + s * a.out0_st[1] + qi * a.out0_st[2] + h * a.out0_st[3];
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[16];
        tmem_ld_32x16(t_row + COL_DQ + hh * (HD / 2) + c * 16, v);
        tmem_ld_wait();
        if (st_ok) {
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            uint4 pk;
            pk.x = pack2<T>(__uint_as_float(v[g * 8 + 0]) * a.scale, __uint_as_float(v[g * 8 + 1]) * a.scale);
            pk.y = pack2<T>(__uint_as_float(v[g * 8 + 2]) * a.scale, __uint_as_float(v[g * 8 + 3]) * a.scale);
            pk.z = pack2<T>(__uint_as_float(v[g * 8 + 4]) * a.scale, __uint_as_float(v[g * 8 + 5]) * a.scale);
            pk.w = pack2<T>(__uint_as_float(v[g * 8 + 6]) * a.scale, __uint_as_float(v[g * 8 + 7]) * a.scale);
            reinterpret_cast<uint4*>(row)[(hh * (HD / 2) + c * 16) / 8 + g] = pk;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------------
// dbias pass: one CTA per (row chunk, batch, head, 128-query block, 64-key block) looping over the rows of its chunk
// in order and summing dS = P (dP - delta) in registers (no atomics: the sum over rows has a fixed order; the chunks'
// partial sums are added by sum_partials_kernel).  320 threads: warps 0-7 do the arithmetic (thread (r, hh) owns
// query r and key half hh), warp 8 issues the MMAs, warp 9 the TMA copies.  S and dP are double buffered in TMEM,
// so the products of the next two rows run under the arithmetic of this one.
//   bar_s[2]    MMA -> threads        S, dP of a row are in TMEM buffer (row & 1)
//   bar_free[4] threads -> MMA, TMA   the row's accumulators, statistics and mask terms have been read
// ------------------------------------------------------------------------------------------------
template <int HD> struct GeoB {
  static constexpr int RB = HD * 2;
  static constexpr int TA = 128 * RB;                    // Q / dO tile
  static constexpr int TB = 64 * RB;                     // K / V tile
  static constexpr uint32_t LAYOUT = RB == 128 ? 2 : 4;
  static constexpr uint32_t SBO = 8 * RB;
  static constexpr int NS = 3;                           // row stages
  static constexpr int STAT = 2048;                      // -m, -log l log2e, -delta of 128 queries; 64 mask terms; padding
                                                         // (stages stay 1024-byte aligned for the swizzled tiles)
  static constexpr int STAGE = 2 * TA + 2 * TB + STAT;
  static constexpr int OFF_BIAS = NS * STAGE;            // [128 queries x 64 keys] SW128, loaded once
  static constexpr int OFF_BAR = OFF_BIAS + 16384;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
};

template <typename T, int HD>
__global__ void __launch_bounds__(320, HD == 32 ? 2 : 1)
attn_bwd_dbias_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmBias, const AttnBwdArgs a) {
  using G = GeoB<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sBias = smem + G::OFF_BIAS;
  uint64_t* bar_once = reinterpret_cast<uint64_t*>(smem + G::OFF_BAR);   // bias tile
  uint64_t* bar_in = bar_once + 1;     // [NS]
  uint64_t* bar_s = bar_once + 4;      // [2]
  uint64_t* bar_free = bar_once + 6;   // [4]: row j arrives on bar_free[j & 3]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_once + 10);
  auto stage_q = [&](int stg) { return smem + stg * G::STAGE; };
  auto stage_do = [&](int stg) { return smem + stg * G::STAGE + G::TA; };
  auto stage_k = [&](int stg) { return smem + stg * G::STAGE + 2 * G::TA; };
  auto stage_v = [&](int stg) { return smem + stg * G::STAGE + 2 * G::TA + G::TB; };
  auto stage_stat = [&](int stg) { return reinterpret_cast<float*>(smem + stg * G::STAGE + 2 * G::TA + 2 * G::TB); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = tid & 127, hh = (tid >> 7) & 1;
  const int qblocks = (a.N + 127) / 128, kblocks = (a.N + 63) / 64;
  int z = blockIdx.x;
  const int kvb = z % kblocks; z /= kblocks;
  const int qb = z % qblocks; z /= qblocks;
  const int h = z % a.H; z /= a.H;
  const int b = z % a.B;
  const int rc = z / a.B;
  const int per = (a.S + a.row_chunks - 1) / a.row_chunks;
  const int s_lo = rc * per;
  const int nsteps = max(0, min(a.S, s_lo + per) - s_lo);
  const int q0 = qb * 128, k0 = kvb * 64;

  if (tid == 0) {
    mbar_init(bar_once, 1);
    for (int i = 0; i < G::NS; ++i) mbar_init(&bar_in[i], 1);
    mbar_init(&bar_s[0], 1); mbar_init(&bar_s[1], 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bar_free[i], 8);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  bool ok = true;

  if (warp == 9) {
    if (lane == 0) {
      // ---------------------------------- TMA copies ---------------------------------------------
      auto load_step = [&](int step) {
        const int stg = step % G::NS, s = s_lo + step;
        const float* prow = a.prep + ((((long long)b * a.S + s) * a.H + h) * (long long)a.npad) + q0;
        float* st = stage_stat(stg);
        mbar_expect_tx(&bar_in[stg], 2 * G::TA + 2 * G::TB + 3 * 512 + 256);
        tma_load_5d(stage_q(stg), &tmQ, &bar_in[stg], 0, h, q0, s, b);
        tma_load_5d(stage_do(stg), &tmDO, &bar_in[stg], 0, h, q0, s, b);
        tma_load_5d(stage_k(stg), &tmK, &bar_in[stg], 0, h, k0, s, b);
        tma_load_5d(stage_v(stg), &tmV, &bar_in[stg], 0, h, k0, s, b);
        bulk_load(st, prow, 512, &bar_in[stg]);
        bulk_load(st + 128, prow + a.prep_plane, 512, &bar_in[stg]);
        bulk_load(st + 256, prow + 2 * a.prep_plane, 512, &bar_in[stg]);
        bulk_load(st + 384, a.mask_terms + ((long long)b * a.S + s) * a.npad + k0, 256, &bar_in[stg]);
      };
      if (nsteps > 0) {   // (a CTA with no rows must not leave a copy in flight)
        mbar_expect_tx(bar_once, 16384);
        tma_load_4d(sBias, &tmBias, bar_once, k0, q0, h, b * a.bias_b_mul);
      }
      for (int st = 0; st < G::NS && st < nsteps; ++st) load_step(st);
      for (int j = 0; j + G::NS < nsteps && ok; ++j) {
        ok = mbar_wait(&bar_free[j & 3], (j >> 2) & 1, a.err, 41) && ok;   // row j has been consumed: its stage is free
        load_step(j + G::NS);
      }
    }
  } else if (warp == 8) {
    if (lane == 0) {
      // ---------------------------------- MMA issue ----------------------------------------------
      constexpr uint32_t HI_KMAJ = desc_hi(G::SBO, G::LAYOUT);
      const uint32_t base_lo = desc_lo(smem_u32(smem), 16);
      for (int j = 0; j < nsteps && ok; ++j) {
        const int stg = j % G::NS, buf = j & 1;
        if (j >= 2) ok = mbar_wait(&bar_free[(j - 2) & 3], ((j - 2) >> 2) & 1, a.err, 42) && ok;   // TMEM buffer is free
        ok = mbar_wait(&bar_in[stg], (j / G::NS) & 1, a.err, 43) && ok;
        tc_fence_after_sync();
        const uint32_t q_lo = base_lo + stg * (G::STAGE >> 4), do_lo = q_lo + (G::TA >> 4), k_lo = do_lo + (G::TA >> 4),
                       v_lo = k_lo + (G::TB >> 4);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma<KIND_F16>(tmem_base + buf * 128, desc_join(q_lo + ks * 2, HI_KMAJ), desc_join(k_lo + ks * 2, HI_KMAJ), a.idesc_a, ks > 0);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma<KIND_F16>(tmem_base + buf * 128 + 64, desc_join(do_lo + ks * 2, HI_KMAJ), desc_join(v_lo + ks * 2, HI_KMAJ), a.idesc_a, ks > 0);
        umma_commit(&bar_s[buf]);
      }
    }
  } else {
    // ------------------------------------ arithmetic warps ---------------------------------------
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    const float2 sc2 = splat(a.scale), l2e2 = splat(kLog2e);
    if (nsteps > 0) ok = mbar_wait(bar_once, 0, a.err, 21);

    for (int j = 0; j < nsteps; ++j) {
      const int stg = j % G::NS, buf = j & 1;
      ok = mbar_wait(&bar_in[stg], (j / G::NS) & 1, a.err, 43) && ok;   // statistics and mask terms of the row
      const float* st = stage_stat(stg);
      const float2 nm2 = splat(st[r]), nl2 = splat(st[128 + r]), nd2 = splat(st[256 + r]);
      const float4* sMb4 = reinterpret_cast<const float4*>(st + 384 + hh * 32);
      ok = mbar_wait(&bar_s[buf], (j >> 1) & 1, a.err, 24) && ok;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[16], rp[16];
        tmem_ld_32x16(t_row + buf * 128 + hh * 32 + c * 16, rs);
        tmem_ld_32x16(t_row + buf * 128 + 64 + hh * 32 + c * 16, rp);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint4 raw = *reinterpret_cast<const uint4*>(sBias + sw128_chunk1(r, hh * 4 + c * 2 + u));   // same tile for every row
          const uint32_t bw[4] = {raw.x, raw.y, raw.z, raw.w};
          const float4 mA = sMb4[c * 4 + u * 2], mB = sMb4[c * 4 + u * 2 + 1];
          const float2 mk[4] = {make_float2(mA.x, mA.y), make_float2(mA.z, mA.w), make_float2(mB.x, mB.y),
                                make_float2(mB.z, mB.w)};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 x = __ffma2_rn(pair(rs[u * 8 + 2 * i], rs[u * 8 + 2 * i + 1]), sc2, mk[i]);
            x = __fadd2_rn(x, unpack2<T>(bw[i]));
            const float2 e = __ffma2_rn(__fadd2_rn(x, nm2), l2e2, nl2);
            const float2 p = make_float2(ex2_approx(e.x), ex2_approx(e.y));
            const float2 ds = __fmul2_rn(p, __fadd2_rn(pair(rp[u * 8 + 2 * i], rp[u * 8 + 2 * i + 1]), nd2));
            const int k = c * 16 + u * 8 + 2 * i;
            const float2 t = __fadd2_rn(make_float2(acc[k], acc[k + 1]), ds);
            acc[k] = t.x;
            acc[k + 1] = t.y;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_free[j & 3]);   // accumulators, statistics and mask terms of the row are consumed
      if (!ok) break;
    }

    const int qi = q0 + r;
    if (qi < a.N && ok) {
      float* row = reinterpret_cast<float*>(a.out0) + (long long)rc * a.B * a.H * a.N * a.N +
                   (((long long)b * a.H + h) * a.N + qi) * a.N + k0 + hh * 32;
      const int valid = a.N - k0 - hh * 32;
      if (valid >= 32 && (a.N % 4) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          reinterpret_cast<float4*>(row)[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < valid) row[i] = acc[i];
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// delta[b,s,h,i] = sum_d dO * O; also the per-row constants of the backward passes in the form their packed
// arithmetic adds (prep[0] = -m, prep[1] = -log l * log2e, prep[2] = -delta), rows padded to npad entries.
template <typename T>
__global__ void attn_delta_tc_kernel(TriAttnDesc d, const T* o, const T* d_o, const float* stats, float* delta,
                                     float* prep, int npad) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)d.B * d.n_seq * d.H * d.n_res;
  if (idx >= total) return;
  const int i = idx % d.n_res; long long z = idx / d.n_res;
  const int h = z % d.H; z /= d.H;
  const int s = z % d.n_seq; const int b = z / d.n_seq;
  const T* orow = o + b * d.o_st[0] + s * d.o_st[1] + i * d.o_st[2] + h * d.o_st[3];
  const T* grow = d_o + b * d.do_st[0] + s * d.do_st[1] + i * d.do_st[2] + h * d.do_st[3];
  float acc = 0.f;
  for (int g = 0; g < d.D / 8; ++g) {
    float x[8], y[8];
    unpack8<T>(reinterpret_cast<const uint4*>(orow)[g], x);
    unpack8<T>(reinterpret_cast<const uint4*>(grow)[g], y);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = fmaf(x[e], y[e], acc);
  }
  delta[idx] = acc;
  const long long pi = (idx / d.n_res) * npad + i, plane = (total / d.n_res) * npad;
  prep[pi] = -stats[idx];
  prep[plane + pi] = -stats[total + idx] * kLog2e;
  prep[2 * plane + pi] = -acc;
}

// dq = scale * sum over key blocks of the merged pass's partials ([nparts][B][S][N][H][D] contiguous), added in key
// block order in fp32; 8 elements per thread.
template <typename T>
__global__ void attn_dq_sum_kernel(const T* __restrict__ part, int nparts, long long plane, TriAttnDesc d, T* __restrict__ dq) {
  const long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (c >= plane / 8) return;
  const int dc = d.D / 8;
  long long z = c;
  const int d8 = z % dc; z /= dc;
  const int h = z % d.H; z /= d.H;
  const int q = z % d.n_res; z /= d.n_res;
  const int s = z % d.n_seq; const int b = z / d.n_seq;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int p = 0; p < nparts; ++p) {
    float v[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(part + p * plane + c * 8), v);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += v[e];
  }
  uint4 pk;
  pk.x = pack2<T>(acc[0] * d.scale, acc[1] * d.scale); pk.y = pack2<T>(acc[2] * d.scale, acc[3] * d.scale);
  pk.z = pack2<T>(acc[4] * d.scale, acc[5] * d.scale); pk.w = pack2<T>(acc[6] * d.scale, acc[7] * d.scale);
  T* row = dq + b * d.dq_st[0] + s * d.dq_st[1] + q * d.dq_st[2] + h * d.dq_st[3];
  reinterpret_cast<uint4*>(row)[d8] = pk;
}

__global__ void sum_partials_kernel(const float* partial, int nparts, long long n, float* out) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[p * n + i];
  out[i] = s;
}

constexpr int kDbiasRowChunks = 8;   // at most this many row chunks (the workspace holds one partial sum per chunk)

// rank-5 map with a caller-chosen number of residues per box
int qkv_map_rows(CUtensorMap* out, const void* p, const TriAttnDesc* d, const int64_t* st, int rows) {
  const uint64_t dims[5] = {(uint64_t)d->D, (uint64_t)d->H, (uint64_t)d->n_res, (uint64_t)d->n_seq, (uint64_t)d->B};
  const uint64_t str[4] = {(uint64_t)st[3], (uint64_t)st[2], (uint64_t)st[1], (uint64_t)st[0]};
  const uint32_t box[5] = {(uint32_t)d->D, 1, (uint32_t)rows, 1, 1};
  return make_tmap(out, p, d->dtype, 5, dims, str, box, d->D * 2);
}

int bias_map(CUtensorMap* out, const void* bias, const TriAttnDesc* d, int rows) {
  const uint64_t nb = d->bias_st[0] != 0 ? (uint64_t)d->B : 1;
  const uint64_t dims[4] = {(uint64_t)d->n_res, (uint64_t)d->n_res, (uint64_t)d->H, nb};
  const uint64_t str[3] = {(uint64_t)d->bias_st[2], (uint64_t)d->bias_st[1], (uint64_t)d->bias_st[0]};
  const uint32_t box[4] = {64, (uint32_t)rows, 1, 1};
  return make_tmap(out, bias, d->dtype, 4, dims, str, box, 128);
}

// out[b][h][k][q] = bias[b][h][q][k] for 16-bit elements (the dK/dV pass reads keys as rows)
__global__ void transpose_bias_kernel(const uint16_t* __restrict__ in, int64_t st_b, int64_t st_h, int64_t st_q, int n, int H,
                                      uint16_t* __restrict__ out) {
  __shared__ uint16_t tile[64][66];
  const int bh = blockIdx.z, b = bh / H, h = bh % H;
  const uint16_t* src = in + b * st_b + h * st_h;
  uint16_t* dst = out + (int64_t)bh * n * n;
  const int q0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int q = q0 + i;
    for (int jj = threadIdx.x; jj < 64; jj += 32) {
      const int k = k0 + jj;
      tile[i][jj] = (q < n && k < n) ? src[q * st_q + k] : (uint16_t)0;
    }
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int k = k0 + i;
    for (int jj = threadIdx.x; jj < 64; jj += 32) {
      const int q = q0 + jj;
      if (k < n && q < n) dst[(int64_t)k * n + q] = tile[jj][i];
    }
  }
}

template <typename KernelT>
int set_dyn_smem(KernelT kern, int bytes) {
  TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return 0;
}

template <typename T, int HD>
int bwd_launch(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
               const uint8_t* mask, const void* o, const float* stats, const void* d_o, void* dq, void* dk, void* dv,
               float* dbias, int* err, float* delta, float* dbias_partial, void* bias_t, float* prep, float* mask_terms,
               void* dq_part, cudaStream_t st) {
  const long long rows = (long long)d->B * d->n_seq * d->H * d->n_res;
  const double pairs = (double)rows * d->n_res;
  const double tensor_bytes = 2.0 * d->B * d->n_seq * (double)d->n_res * d->H * d->D;
  const int npad = (d->n_res + 127) / 128 * 128;
  const long long prep_plane = (long long)d->B * d->n_seq * d->H * npad;
  {
    KernelTimer kt("tc_attn_delta", st, 0.0, 2.0 * tensor_bytes);
    {
      const long long n = (long long)d->B * d->n_seq * npad;
      mask_terms_kernel<<<cdiv(n, 256), 256, 0, st>>>(mask, d->mask_st[0], d->mask_st[1], d->B, d->n_seq, d->n_res, npad, mask_terms);
      TRI_LAUNCH_OK();
    }
    if (npad != d->n_res) TRI_CUDA_OK(cudaMemsetAsync(prep, 0, 3 * prep_plane * sizeof(float), st));
    attn_delta_tc_kernel<T><<<cdiv(rows, 256), 256, 0, st>>>(*d, (const T*)o, (const T*)d_o, stats, delta, prep, npad);
    TRI_LAUNCH_OK();
  }
  const int kind = d->dtype == TRI_BF16 ? KIND_BF16 : KIND_F16;
  AttnBwdArgs a;
  a.B = d->B; a.S = d->n_seq; a.N = d->n_res; a.H = d->H; a.scale = d->scale;
  a.stats = stats; a.delta = delta; a.prep = prep; a.prep_plane = prep_plane; a.npad = npad; a.mask_terms = mask_terms; a.mask = mask; a.mask_st[0] = d->mask_st[0]; a.mask_st[1] = d->mask_st[1];
  a.bias_b_mul = d->bias_st[0] != 0 ? 1 : 0; a.err = err;
  a.row_chunks = 1;
  const int qblocks = (d->n_res + 127) / 128;
  CUtensorMap tq, tdo, tk, tv, tb;

  // ---- dK / dV -------------------------------------------------------------------------------
  TRI_TRY(qkv_map_rows(&tq, q, d, d->q_st, 64));
  TRI_TRY(qkv_map_rows(&tdo, d_o, d, d->do_st, 64));
  TRI_TRY(qkv_map_rows(&tk, k, d, d->k_st, 128));
  TRI_TRY(qkv_map_rows(&tv, v, d, d->v_st, 128));
  if (bias) {   // the dK/dV pass (thread = key) reads a transposed copy of the bias: [b][h][key][query]
    const int nb = d->bias_st[0] != 0 ? d->B : 1;
    transpose_bias_kernel<<<dim3(cdiv(d->n_res, 64), cdiv(d->n_res, 64), nb * d->H), dim3(32, 8), 0, st>>>(
        static_cast<const uint16_t*>(bias), d->bias_st[0], d->bias_st[1], d->bias_st[2], d->n_res, d->H,
        static_cast<uint16_t*>(bias_t));
    TRI_LAUNCH_OK();
    const uint64_t dims[4] = {(uint64_t)d->n_res, (uint64_t)d->n_res, (uint64_t)d->H, (uint64_t)nb};
    const uint64_t str[3] = {(uint64_t)d->n_res, (uint64_t)d->n_res * d->n_res, nb > 1 ? (uint64_t)d->H * d->n_res * d->n_res : 0};
    const uint32_t box[4] = {64, 128, 1, 1};
    TRI_TRY(make_tmap(&tb, bias_t, d->dtype, 4, dims, str, box, 128));
  } else {
    tb = tq;
  }
  a.out0 = dk; a.out1 = dv;
  for (int i = 0; i < 4; ++i) { a.out0_st[i] = d->dk_st[i]; a.out1_st[i] = d->dv_st[i]; }
  a.idesc_a = make_idesc(kind, 128, 64, false, false);
  a.idesc_b = make_idesc(kind, 128, HD, false, true);
  a.idesc_c = make_idesc(kind, 128, HD, true, true);
  // Head dim 32: dK, dV and dQ come from one pass (dQ as per-key-block partials, summed below); head dim 64 has no
  // TMEM columns to spare for the dQ accumulator and keeps the separate dQ pass.
  constexpr bool kMerge = HD == 32;
  const long long dq_plane = (long long)d->B * d->n_seq * d->n_res * d->H * d->D;
  a.dq_part = dq_part; a.dq_part_plane = dq_plane;
  {
    auto kern = bias ? attn_bwd_dkdv_kernel<T, HD, true, kMerge> : attn_bwd_dkdv_kernel<T, HD, false, kMerge>;
    TRI_TRY(set_dyn_smem(kern, GeoC<HD>::SMEM));   // per-device attribute: set on every launch
    KernelTimer kt(kMerge ? "tc_attn_bwd_dkdvdq" : "tc_attn_bwd_dkdv", st, (kMerge ? 10.0 : 8.0) * pairs * d->D,
                   (kMerge ? 7.0 : 6.0) * tensor_bytes);
    kern<<<(unsigned)((long long)qblocks * d->B * d->n_seq * d->H), 320, GeoC<HD>::SMEM, st>>>(tq, tdo, tk, tv, tb, a);
    TRI_LAUNCH_OK();
  }
  if (kMerge) {
    KernelTimer kt("tc_attn_dq_sum", st, 0.0, (qblocks + 1.0) * tensor_bytes);
    attn_dq_sum_kernel<T><<<cdiv(dq_plane / 8, 256), 256, 0, st>>>(static_cast<const T*>(dq_part), qblocks, dq_plane, *d,
                                                               static_cast<T*>(dq));
    TRI_LAUNCH_OK();
  }
  // ---- dQ ------------------------------------------------------------------------------------
  TRI_TRY(qkv_map_rows(&tq, q, d, d->q_st, 128));
  TRI_TRY(qkv_map_rows(&tdo, d_o, d, d->do_st, 128));
  TRI_TRY(qkv_map_rows(&tk, k, d, d->k_st, 64));
  TRI_TRY(qkv_map_rows(&tv, v, d, d->v_st, 64));
  if (bias) TRI_TRY(bias_map(&tb, bias, d, 128));
  a.out0 = dq; a.out1 = nullptr;
  for (int i = 0; i < 4; ++i) a.out0_st[i] = d->dq_st[i];
  a.idesc_a = make_idesc(kind, 128, 64, false, false);
  a.idesc_b = make_idesc(kind, 128, HD, false, true);
  if (!kMerge) {
    auto kern = bias ? attn_bwd_dq_kernel<T, HD, true> : attn_bwd_dq_kernel<T, HD, false>;
    TRI_TRY(set_dyn_smem(kern, GeoQ<HD>::SMEM));
    KernelTimer kt("tc_attn_bwd_dq", st, 2.0 * pairs * d->D, 5.0 * tensor_bytes);
    kern<<<(unsigned)((long long)qblocks * d->B * d->n_seq * d->H), 320, GeoQ<HD>::SMEM, st>>>(tq, tdo, tk, tv, tb, a);
    TRI_LAUNCH_OK();
  }
  // ---- dbias ---------------------------------------------------------------------------------
  if (dbias != nullptr) {
    // Row chunks only as far as they are needed to fill the GPU (two CTAs per SM): with enough (batch, head, query
    // block, key block) combinations one CTA sums all rows and no partial sums are written or added.
    const long long combos = (long long)qblocks * ((d->n_res + 63) / 64) * d->B * d->H, slots = 2LL * sm_count();
    int chunks = 1;
    if (combos * 10 < slots * 9) chunks = (int)std::min<long long>(kDbiasRowChunks, (slots + combos - 1) / combos);
    chunks = std::max(1, std::min(chunks, d->n_seq / 2));
    const long long nb = (long long)d->B * d->H * d->n_res * d->n_res;
    const int kblocks = (d->n_res + 63) / 64;
    a.row_chunks = chunks;
    a.out0 = chunks > 1 ? dbias_partial : dbias;
    a.idesc_a = make_idesc(kind, 128, 64, false, false);
    auto kern = attn_bwd_dbias_kernel<T, HD>;   // (K / V maps with 64-key boxes and the bias map are those of the dQ pass)
    TRI_TRY(set_dyn_smem(kern, GeoB<HD>::SMEM));
    KernelTimer kt("tc_attn_bwd_dbias", st, 0.0, 4.0 * tensor_bytes);
    kern<<<(unsigned)((long long)qblocks * kblocks * d->B * d->H * chunks), 320, GeoB<HD>::SMEM, st>>>(tq, tdo, tk, tv, tb, a);
    TRI_LAUNCH_OK();
    if (chunks > 1) {   // fixed-order sum of the row-chunk partials
      sum_partials_kernel<<<cdiv(nb, 256), 256, 0, st>>>(dbias_partial, chunks, nb, dbias);
      TRI_LAUNCH_OK();
    }
  }
  return 0;
}

bool forced_simt() {
  const char* e = getenv("TRI_B200_FORCE_SIMT");
  return e != nullptr && e[0] == '1';
}

// A tensor map needs strides that are non-zero multiples of 16 bytes on every axis with more than one entry; a
// broadcast (zero-stride) view therefore goes to the CUDA-core kernels, which take any stride.
bool strides_ok(const TriAttnDesc* d, const int64_t* st) {
  const int extent[4] = {d->B, d->n_seq, d->n_res, d->H};
  for (int i = 0; i < 4; ++i) {
    if (st[i] % 8 != 0) return false;
    if (st[i] == 0 && extent[i] > 1) return false;
  }
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
               const uint8_t* mask, void* o, float* stats, int* err, float* mask_terms, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tb;
  TRI_TRY(qkv_map(&tq, q, d, d->q_st));
  TRI_TRY(qkv_map(&tk, k, d, d->k_st));
  TRI_TRY(qkv_map(&tv, v, d, d->v_st));
  AttnArgs a;
  a.B = d->B; a.S = d->n_seq; a.N = d->n_res; a.H = d->H; a.scale = d->scale;
  a.o = o; for (int i = 0; i < 4; ++i) a.o_st[i] = d->o_st[i];
  a.stats = stats; a.mask_terms = mask_terms; a.npad = (d->n_res + 127) / 128 * 128;
  a.bias_b_mul = d->bias_st[0] != 0 ? 1 : 0;
  {
    const long long n = (long long)d->B * d->n_seq * a.npad;
    mask_terms_kernel<<<cdiv(n, 256), 256, 0, st>>>(mask, d->mask_st[0], d->mask_st[1], d->B, d->n_seq, d->n_res, a.npad, mask_terms);
    TRI_LAUNCH_OK();
  }
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
  const long long blocks = (long long)((d->n_res + 127) / 128) * d->B * d->n_seq * d->H;
  const double pairs = (double)d->B * d->n_seq * d->H * d->n_res * (double)d->n_res;
  KernelTimer kt("tc_attn_fwd", st, 4.0 * pairs * d->D, 2.0 * 4.0 * d->B * d->n_seq * (double)d->n_res * d->H * d->D);
  auto kern = bias != nullptr ? attn_fwd_tc_kernel<T, HD, true> : attn_fwd_tc_kernel<T, HD, false>;
  TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<HD>::SMEM));
  kern<<<(unsigned)std::min<long long>(blocks, 2LL * sm_count()), 320, Geo<HD>::SMEM, st>>>(tq, tk, tv, tb, a);
  TRI_LAUNCH_OK();
  return 0;
}

}  // namespace

bool attn_fwd_supported(const TriAttnDesc* d) {
  if (forced_simt()) return false;
  if (d->dtype != TRI_BF16 && d->dtype != TRI_F16) return false;
  if (d->D != 32 && d->D != 64) return false;
  if (d->n_res % 8 != 0 || d->n_res > 16384) return false;
  if (!strides_ok(d, d->q_st) || !strides_ok(d, d->k_st) || !strides_ok(d, d->v_st) || !strides_ok(d, d->o_st)) return false;
  if (d->bias_st[1] % 8 != 0 || d->bias_st[2] % 8 != 0 || d->bias_st[0] % 8 != 0) return false;
  if ((long long)((d->n_res + 127) / 128) * d->B * d->n_seq * d->H > 2147483647LL) return false;
  return true;
}

bool attn_bwd_supported(const TriAttnDesc* d) {
  return attn_fwd_supported(d) && strides_ok(d, d->do_st) && strides_ok(d, d->dq_st) && strides_ok(d, d->dk_st) &&
         strides_ok(d, d->dv_st) && d->n_seq <= 65535;
}

static size_t attn_npad(const TriAttnDesc* d) { return ((size_t)d->n_res + 127) / 128 * 128; }
// partial dQ of the merged dK/dV + dQ pass (head dim 32 only): one 16-bit tensor of q's size per 128-key block
static size_t attn_dq_part_bytes(const TriAttnDesc* d) {
  if (d->D != 32) return 0;
  return align_up(attn_npad(d) / 128 * (size_t)d->B * d->n_seq * d->n_res * d->H * d->D * 2);
}

size_t attn_ws_bytes(const TriAttnDesc* d, int is_bwd) {
  if (!is_bwd) return 512 + align_up((size_t)d->B * d->n_seq * attn_npad(d) * sizeof(float));   // additive key-mask terms
  return 512 + align_up((size_t)d->B * d->n_seq * d->H * d->n_res * sizeof(float)) +
         align_up((size_t)kDbiasRowChunks * d->B * d->H * d->n_res * d->n_res * sizeof(float)) +
         align_up((size_t)d->B * d->H * d->n_res * d->n_res * 2) +   // transposed 16-bit copy of the bias
         align_up(3 * (size_t)d->B * d->n_seq * d->H * attn_npad(d) * sizeof(float)) +   // padded per-row constants
         align_up((size_t)d->B * d->n_seq * attn_npad(d) * sizeof(float)) +              // additive key-mask terms
         attn_dq_part_bytes(d);                                                          // merged pass: dQ per key block
}

int attn_forward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                 const uint8_t* mask, void* o, float* lse, void* ws, size_t ws_size, cudaStream_t st) {
  if (ws == nullptr || ws_size < attn_ws_bytes(d, 0)) return fail(TRI_ERR_WORKSPACE, "attention forward workspace too small");
  TRI_CUDA_OK(cudaMemsetAsync(ws, 0, 256, st));
  int* err = static_cast<int*>(ws);
  float* mt = reinterpret_cast<float*>(static_cast<char*>(ws) + 512);
  if (d->dtype == TRI_BF16) {
    if (d->D == 32) return fwd_launch<__nv_bfloat16, 32>(d, q, k, v, bias, mask, o, lse, err, mt, st);
    return fwd_launch<__nv_bfloat16, 64>(d, q, k, v, bias, mask, o, lse, err, mt, st);
  }
  if (d->D == 32) return fwd_launch<__half, 32>(d, q, k, v, bias, mask, o, lse, err, mt, st);
  return fwd_launch<__half, 64>(d, q, k, v, bias, mask, o, lse, err, mt, st);
}

int attn_backward(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                  const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                  void* dv, float* dbias, void* ws, size_t ws_size, cudaStream_t st) {
  if (ws == nullptr || ws_size < attn_ws_bytes(d, 1)) return fail(TRI_ERR_WORKSPACE, "attention backward workspace too small");
  TRI_CUDA_OK(cudaMemsetAsync(ws, 0, 256, st));
  int* err = static_cast<int*>(ws);
  float* delta = reinterpret_cast<float*>(static_cast<char*>(ws) + 512);
  float* part = reinterpret_cast<float*>(static_cast<char*>(ws) + 512 +
                                         align_up((size_t)d->B * d->n_seq * d->H * d->n_res * sizeof(float)));
  void* bias_t = reinterpret_cast<char*>(part) + align_up((size_t)kDbiasRowChunks * d->B * d->H * d->n_res * d->n_res * sizeof(float));
  float* prep = reinterpret_cast<float*>(static_cast<char*>(bias_t) + align_up((size_t)d->B * d->H * d->n_res * d->n_res * 2));
  float* mterms = reinterpret_cast<float*>(reinterpret_cast<char*>(prep) + align_up(3 * (size_t)d->B * d->n_seq * d->H * attn_npad(d) * sizeof(float)));
  void* dq_part = reinterpret_cast<char*>(mterms) + align_up((size_t)d->B * d->n_seq * attn_npad(d) * sizeof(float));
  if (d->dtype == TRI_BF16) {
    if (d->D == 32) return bwd_launch<__nv_bfloat16, 32>(d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, err, delta, part, bias_t, prep, mterms, dq_part, st);
    return bwd_launch<__nv_bfloat16, 64>(d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, err, delta, part, bias_t, prep, mterms, dq_part, st);
  }
  if (d->D == 32) return bwd_launch<__half, 32>(d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, err, delta, part, bias_t, prep, mterms, dq_part, st);
  return bwd_launch<__half, 64>(d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, err, delta, part, bias_t, prep, mterms, dq_part, st);
}

}  // namespace tc
}  // namespace tri
