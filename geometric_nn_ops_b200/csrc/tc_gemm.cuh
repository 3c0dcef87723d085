// Persistent, warp-specialised tcgen05 GEMM:  D[m, n] = sum_k A(m, k) * B(n, k), fp32 accumulation in TMEM.
//
//   warp 0      TMA producer: fills a ring of shared-memory stages (128-byte swizzle) with operand tiles
//   warp 1      MMA issuer:   tcgen05.mma from the stages into one of two TMEM accumulators
//   warps 2..9  epilogue:     two groups of four warps (each group covers the 128 TMEM lanes and takes half
//                             of the accumulator columns): tcgen05.ld, fused epilogue, 16/32-byte stores
//
// A tile is 128 (M) x BN (N); K advances 128 bytes per stage (64 bf16/fp16 or 32 fp32 elements).  Each
// operand may be K-major (K contiguous in global memory) or MN-major (M or N contiguous); the second form
// is what the transposed contractions and the weight-gradient GEMMs need, and costs nothing: only the TMA
// box shape and the MMA descriptors differ.  Two K "segments" with their own tensor maps can feed the
// same tile, either into the same accumulator columns (a sum of two products) or into the second half
// of them (two products side by side); the fused gate epilogues use that.  With split_k the batch index
// selects a K range instead of a batch entry (weight gradients over all pixels).
//
// The input-gate GEMMs run TRANSPOSED (weights are the M operand, pixels the N operand), so that a thread
// owns one channel and its registers hold consecutive pixels: the channel-major a / b / dPG tensors are
// then written and read with plain contiguous vector accesses instead of 2-byte scatters.
//
// All waits are bounded (see tc_common.cuh); a timeout lands in *args.err and the kernel drains.
#pragma once

#include "tc_common.cuh"

namespace tri {
namespace tc {

enum Epilogue {
  EPI_STORE = 0,         // out0[batch][m][n] = acc (+ bias0[n])
  EPI_GATE_IN = 1,       // transposed: rows = channels of one half (tile_m = a or b), cols [P(128 px) | G(128 px)]:
                         //   half-plane[c][px] = (P+bp)*sigmoid(G+bg)*mask[px]
  EPI_GATE_OUT = 2,      // rows = pixels, cols [y(128) | g(128)]: out0[m][c] = (y+b)*sigmoid(g+b)
  EPI_GATE_OUT_BWD = 3,  // same cols, aux = d_out: out0 = d_out*sig, out1 = d_out*(y+b)*sig*(1-sig)
  EPI_GATE_IN_BWD = 4    // transposed like GATE_IN; aux2/aux3 = channel-major d(a), d(b); aux = mask;
                         //   d = d(half)[c][px]*mask;  out0 is channel-major [512][M]:
                         //   row half*256+c = d*sig(G),  row half*256+128+c = d*P*sig*(1-sig)
};

constexpr int kBM = 128;
constexpr int kStageA = kBM * 128;  // bytes
// warp 0 producer, warp 1 MMA, then the epilogue warps: 16 for the gate-in, gate-out and gate-out backward
// epilogues, whose per-element arithmetic (sigmoid, products) is latency-bound with fewer warps per scheduler; 8 for
// the plain store and for gate-in backward (which spends its registers on a tile-ahead prefetch instead)
constexpr int gemm_epi_warps(int epi) { return (epi == 0 || epi == 4) ? 8 : 16; }
constexpr int gemm_threads(int epi) { return 64 + 32 * gemm_epi_warps(epi); }

struct GemmArgs {
  int M, N;                  // output extent of one batch entry
  int kblocks0, kblocks1;    // K blocks (of 128 bytes) in segment 0 / segment 1 (0 = no second segment)
  int seg1_col;              // accumulator column where segment 1 lands (0 = add to segment 0's columns)
  int seg1_n;                // N extent of segment 1's MMA (columns), segment 0 uses bn0
  int bn0;                   // N extent of segment 0's MMA
  int batches, tiles_m, tiles_n;
  int split_k;               // batch index selects K range [batch*kblocks0, ...) instead of a batch entry
  int a_tile_batch;          // the M-tile index is A's batch coordinate (rows 0..127 of plane tile_m)
  int a_mn[2], b_mn[2];      // per segment: operand is MN-major
  uint32_t idesc[2];
  // epilogue
  void* out0;
  void* out1;
  long long ld_out, batch_out;   // elements
  const float* bias0;            // per output column (EPI_STORE) / per accumulator column or row (gates)
  const void* aux;               // mask (GATE_IN*) or d_out (GATE_OUT_BWD), in the input dtype
  const void* aux2;              // GATE_IN_BWD: channel-major gradient of the a half
  const void* aux3;              //              ... of the b half
  long long plane;               // GATE_IN(_BWD): pixels per batch entry; channel-major plane stride
  // GATE_IN with peer_world > 0: channel c of half tm goes to GPU c / peer_cs, into its buffer
  // [2 * peer_batches][peer_cs][peer_world][plane] at (tm * peer_batches + batch, c % peer_cs, peer_rank)
  void* peer_out[16];
  int peer_world, peer_rank, peer_cs, peer_batches;
  int* err;
};

template <typename T> struct ElemTraits;
template <> struct ElemTraits<__nv_bfloat16> { static constexpr int kind = KIND_BF16; };
template <> struct ElemTraits<__half> { static constexpr int kind = KIND_F16; };
template <> struct ElemTraits<float> { static constexpr int kind = KIND_TF32; };

__device__ __forceinline__ float fast_sigmoid(float x) {
  return __fdividef(1.0f, 1.0f + ex2_approx(-1.4426950408889634f * x));
}

// sigmoid of two values with packed fp32x2 arithmetic around the two MUFU pairs (the gate epilogues are bound by
// instruction issue, and a packed instruction does the work of two)
__device__ __forceinline__ float2 sigmoid2(float2 x) {
  const float2 t = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  const float2 den = __fadd2_rn(make_float2(ex2_approx(t.x), ex2_approx(t.y)), make_float2(1.0f, 1.0f));
  return make_float2(__fdividef(1.0f, den.x), __fdividef(1.0f, den.y));
}

// 8 consecutive elements <-> registers, with 16-byte (16-bit types) or 2 x 16-byte (fp32) accesses
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    union { uint4 u; T h[8]; } pk;
    pk.u = *reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32(pk.h[i]);
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* v) {
  if constexpr (sizeof(T) == 4) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    union { uint4 u; T h[8]; } pk;
#pragma unroll
    for (int i = 0; i < 8; ++i) pk.h[i] = from_f32<T>(v[i]);
    *reinterpret_cast<uint4*>(p) = pk.u;
  }
}

// The same 8 elements as raw 16-byte words: issued early, converted when used, so that a tile's global loads
// are all in flight before its arithmetic (the epilogue warps are too few to hide one load after another).
template <typename T> struct Raw8 { uint4 w[sizeof(T) == 4 ? 2 : 1]; };
template <typename T> __device__ __forceinline__ Raw8<T> ldraw8(const T* p) {
  Raw8<T> r;
  r.w[0] = __ldg(reinterpret_cast<const uint4*>(p));
  if constexpr (sizeof(T) == 4) r.w[1] = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  return r;
}
template <typename T> __device__ __forceinline__ void cvtraw8(const Raw8<T>& r, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    v[0] = __uint_as_float(r.w[0].x); v[1] = __uint_as_float(r.w[0].y); v[2] = __uint_as_float(r.w[0].z); v[3] = __uint_as_float(r.w[0].w);
    v[4] = __uint_as_float(r.w[1].x); v[5] = __uint_as_float(r.w[1].y); v[6] = __uint_as_float(r.w[1].z); v[7] = __uint_as_float(r.w[1].w);
  } else {
    union { uint4 u; T h[8]; } pk;
    pk.u = r.w[0];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32(pk.h[i]);
  }
}

// 32-byte accesses (16 values of a 16-bit type) for the channel-major tensors of the transposed gate GEMMs: a lane
// then reads or writes whole 32-byte sectors of its channel row instead of two half sectors in two requests.
template <typename T> __device__ __forceinline__ void ldraw16(const T* p, Raw8<T>& lo, Raw8<T>& hi) {
  static_assert(sizeof(T) == 2, "16-bit types");
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(lo.w[0].x), "=r"(lo.w[0].y), "=r"(lo.w[0].z), "=r"(lo.w[0].w), "=r"(hi.w[0].x), "=r"(hi.w[0].y),
                 "=r"(hi.w[0].z), "=r"(hi.w[0].w)
               : "l"(p));
}
template <typename T> __device__ __forceinline__ void store16(T* p, const float* v) {
  static_assert(sizeof(T) == 2, "16-bit types");
  union { uint4 u[2]; T h[16]; } pk;
#pragma unroll
  for (int i = 0; i < 16; ++i) pk.h[i] = from_f32<T>(v[i]);
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(pk.u[0].x), "r"(pk.u[0].y), "r"(pk.u[0].z),
               "r"(pk.u[0].w), "r"(pk.u[1].x), "r"(pk.u[1].y), "r"(pk.u[1].z), "r"(pk.u[1].w)
               : "memory");
}

template <typename TOUT>
__device__ __forceinline__ void store_row32(TOUT* dst, const float (&v)[32], int valid, bool vec_ok) {
  if (valid >= 32 && vec_ok) {
    if constexpr (sizeof(TOUT) == 2) {
      if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {   // whole 32-byte sectors per request
        store16<TOUT>(dst, &v[0]);
        store16<TOUT>(dst + 16, &v[16]);
        return;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) store8<TOUT>(dst + 8 * i, &v[8 * i]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = from_f32<TOUT>(v[i]);
  }
}

// two 32-column loads (columns c0.. and c1..) with one wait
__device__ __forceinline__ void ld32x2_f(uint32_t t0, uint32_t t1, float (&a)[32], float (&b)[32]) {
  uint32_t ra[32], rb[32];
  tmem_ld_32x32(t0, ra);
  tmem_ld_32x32(t1, rb);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) { a[i] = __uint_as_float(ra[i]); b[i] = __uint_as_float(rb[i]); }
}
// two 16-column loads with one wait
__device__ __forceinline__ void ld16x2_f(uint32_t t0, uint32_t t1, float (&a)[16], float (&b)[16]) {
  uint32_t ra[16], rb[16];
  tmem_ld_32x16(t0, ra);
  tmem_ld_32x16(t1, rb);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) { a[i] = __uint_as_float(ra[i]); b[i] = __uint_as_float(rb[i]); }
}
__device__ __forceinline__ void ld32_f(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// where the gate-in epilogue writes channel `row` of half `tm`, batch entry `bb`, pixel `pix`: this GPU's
// channel-major output, or (row-sharded runs) the exchange buffer of the GPU that owns the channel
template <typename TOUT>
__device__ __forceinline__ TOUT* gate_in_dst(const GemmArgs& g, int tm, long long bb, int row, long long pix) {
  if (g.peer_world > 0) {
    const int w = row / g.peer_cs, cl = row - w * g.peer_cs;
    return reinterpret_cast<TOUT*>(g.peer_out[w]) +
           ((((long long)tm * g.peer_batches + bb) * g.peer_cs + cl) * g.peer_world + g.peer_rank) * g.plane + pix;
  }
  return reinterpret_cast<TOUT*>(tm == 0 ? g.out0 : g.out1) + (bb * 128 + row) * g.plane + pix;
}

template <typename TIN, typename TOUT, int BN, int EPI, int STAGES>
__global__ void __launch_bounds__(gemm_threads(EPI), 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
               const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1, const GemmArgs g) {
  constexpr int ES = sizeof(TIN);
  constexpr int BKE = 128 / ES;        // K elements per stage
  constexpr int UK = 32 / ES;          // K elements per MMA
  constexpr int CE = 128 / ES;         // MN elements per 128-byte chunk (MN-major operands)
  constexpr int STAGE_B = BN * 128;
  // MN-major tiles: 16-bit types use the plain 128-byte swizzle (8-k groups of 1024 bytes); 32-bit
  // types only exist with the 32-byte-atom swizzle (4-k groups of 512 bytes, layout code 1).
  constexpr uint32_t MN_SBO = ES == 4 ? 512 : 1024;
  constexpr uint32_t MN_LAYOUT = ES == 4 ? 1 : 2;
  constexpr int KIND = ElemTraits<TIN>::kind == KIND_TF32 ? KIND_TF32 : KIND_F16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * kStageA;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + STAGES * STAGE_B);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], gemm_epi_warps(EPI)); }
    mbar_fence_init();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmB0);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total = g.batches * g.tiles_m * g.tiles_n;
  const int kb_total = g.kblocks0 + g.kblocks1;
  // tile -> (batch, tile_m, tile_n); with a_tile_batch the M tiles (weight blocks) of one pixel tile are
  // adjacent in the schedule so the shared activation tile is still in L2 for the second one
  auto decode = [&](int tile, int& tm, int& tn, int& bz) {
    if (g.a_tile_batch) { tm = tile % g.tiles_m; tn = (tile / g.tiles_m) % g.tiles_n; }
    else { tn = tile % g.tiles_n; tm = (tile / g.tiles_n) % g.tiles_m; }
    bz = tile / (g.tiles_n * g.tiles_m);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    const bool leader = elect_one();
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        int tm, tn, bz;
        decode(tile, tm, tn, bz);
        const int n0 = tn * (g.seg1_col ? g.bn0 : BN);
        const int zc = g.split_k ? 0 : bz;
        const int koff = g.split_k ? bz * g.kblocks0 * BKE : 0;
        const int am = g.a_tile_batch ? 0 : tm * kBM, az = g.a_tile_batch ? tm : zc;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, g.err, 1)) { ok = false; break; }
          const int seg = kb >= g.kblocks0 ? 1 : 0;
          const int kk = (seg ? kb - g.kblocks0 : kb) * BKE + koff;
          const CUtensorMap* ma = seg ? &tmA1 : &tmA0;
          const CUtensorMap* mb = seg ? &tmB1 : &tmB0;
          const int bn = seg ? g.seg1_n : g.bn0;
          mbar_expect_tx(&full[stage], kStageA + bn * 128);
          uint8_t* a_dst = sA + stage * kStageA;
          uint8_t* b_dst = sB + stage * STAGE_B;
          if (!g.a_mn[seg]) {
            tma_load_3d(a_dst, ma, &full[stage], kk, am, az);
          } else {
            for (int c = 0; c < kBM / CE; ++c) tma_load_3d(a_dst + c * (BKE * 128), ma, &full[stage], am + c * CE, kk, az);
          }
          if (!g.b_mn[seg]) {
            tma_load_3d(b_dst, mb, &full[stage], kk, n0, zc);
          } else {
            for (int c = 0; c < bn / CE; ++c) tma_load_3d(b_dst + c * (BKE * 128), mb, &full[stage], n0 + c * CE, kk, zc);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const bool leader = elect_one();
    if (leader) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      const uint32_t a_base = smem_u32(sA), b_base = smem_u32(sB);
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, g.err, 2)) break;
        tc_fence_after_sync();
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full[stage], phase, g.err, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const int seg = kb >= g.kblocks0 ? 1 : 0;
          const int kin = seg ? kb - g.kblocks0 : kb;
          const uint32_t d_addr = tmem_base + acc * BN + (seg ? g.seg1_col : 0);
          const bool fresh = kin == 0 && !(seg == 1 && g.seg1_col == 0);  // first product into these columns
          const uint32_t a_stage = a_base + stage * kStageA, b_stage = b_base + stage * STAGE_B;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = g.a_mn[seg] ? make_smem_desc(a_stage + ks * UK * 128, BKE * 128, MN_SBO, MN_LAYOUT)
                                            : make_smem_desc(a_stage + ks * 32, 16, 1024);
            const uint64_t bd = g.b_mn[seg] ? make_smem_desc(b_stage + ks * UK * 128, BKE * 128, MN_SBO, MN_LAYOUT)
                                            : make_smem_desc(b_stage + ks * 32, 16, 1024);
            umma<KIND>(d_addr, ad, bd, g.idesc[seg], (fresh && ks == 0) ? 0u : 1u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue: groups of 4 warps
    const int quarter = warp & 3;            // the TMEM lane quarter this warp may read
    const int grp = (warp - 2) >> 2;         // column share this warp's group takes (2 or 4 groups)
    constexpr int NGRP = gemm_epi_warps(EPI) / 4;
    constexpr int CPG = 4 / NGRP;            // gate epilogues: 32-pixel (or channel) chunks per group
    const int row = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    // The backward gate epilogues read a gradient tile from global memory.  Gate-in backward fetches it a whole tile
    // ahead (the loads of tile t+1 are issued before tile t's arithmetic): its warps are too few to hide a load
    // issued just before its use.
    constexpr bool kGradTile = EPI == EPI_GATE_IN_BWD || EPI == EPI_GATE_OUT_BWD;
    auto fetch_grad = [&](int t, Raw8<TIN> (&dst)[CPG][4]) {
      int tm, tn, bz;
      decode(t, tm, tn, bz);
      if constexpr (EPI == EPI_GATE_IN_BWD) {
        const TIN* dplane = reinterpret_cast<const TIN*>(tm == 0 ? g.aux2 : g.aux3);
        const long long t0 = (long long)tn * 128, tb0 = t0 / g.plane, tp0 = t0 - tb0 * g.plane;   // one division per tile
        const bool wide = sizeof(TIN) == 2 && (g.plane & 15) == 0 && (g.N & 15) == 0;   // 16-pixel groups: aligned, never split
#pragma unroll
        for (int jj = 0; jj < CPG; ++jj)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int off = (grp * CPG + jj) * 32 + u * 8;
            if (t0 + off < g.N) {
              long long bb = tb0, pix = tp0 + off;
              while (pix >= g.plane) { pix -= g.plane; ++bb; }
              const TIN* src = dplane + (bb * 128 + row) * g.plane + pix;
              if constexpr (sizeof(TIN) == 2) {
                if (wide) { if ((u & 1) == 0) ldraw16<TIN>(src, dst[jj][u], dst[jj][u + 1]); }
                else dst[jj][u] = ldraw8<TIN>(src);
              } else {
                dst[jj][u] = ldraw8<TIN>(src);
              }
            }
          }
      } else if constexpr (EPI == EPI_GATE_OUT_BWD) {
        const int m = tm * kBM + row;
        const TIN* dout = reinterpret_cast<const TIN*>(g.aux) + (long long)m * 128;
        if (m < g.M) {
#pragma unroll
          for (int jj = 0; jj < CPG; ++jj)
#pragma unroll
            for (int u = 0; u < 4; u += 2) {
              if constexpr (sizeof(TIN) == 2) {   // rows of 256 bytes: 32-byte loads are aligned
                ldraw16<TIN>(dout + (grp * CPG + jj) * 32 + u * 8, dst[jj][u], dst[jj][u + 1]);
              } else {
                dst[jj][u] = ldraw8<TIN>(dout + (grp * CPG + jj) * 32 + u * 8);
                dst[jj][u + 1] = ldraw8<TIN>(dout + (grp * CPG + jj) * 32 + u * 8 + 8);
              }
            }
        }
      }
    };
    // (gate-in backward: 8 epilogue warps with registers to spare; gate-out backward, on 16 warps and already at 70 %
    // of HBM bandwidth, fetches its tile just before waiting for the product)
    constexpr bool kAhead = EPI == EPI_GATE_IN_BWD && sizeof(TIN) == 2;   // (fp32 tiles would not fit the registers twice)
    Raw8<TIN> dnext[kAhead ? CPG : 1][4];
    if constexpr (kAhead) {
      if ((int)blockIdx.x < total) fetch_grad(blockIdx.x, dnext);
    }
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      int tm, tn, bz;
      decode(tile, tm, tn, bz);
      Raw8<TIN> dpre[CPG][4];
      if constexpr (kAhead) {
#pragma unroll
        for (int jj = 0; jj < CPG; ++jj)
#pragma unroll
          for (int u = 0; u < 4; ++u) dpre[jj][u] = dnext[jj][u];
        if (tile + (int)gridDim.x < total) fetch_grad(tile + gridDim.x, dnext);
      } else if constexpr (kGradTile) {
        fetch_grad(tile, dpre);
      }
      if (!mbar_wait(&tfull[acc], acc_phase, g.err, 4)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      if constexpr (EPI == EPI_STORE) {
        const int m = tm * kBM + row, n0 = tn * BN;
        TOUT* out = reinterpret_cast<TOUT*>(g.out0) + bz * g.batch_out + (long long)m * g.ld_out;
        const bool vec_ok = (g.ld_out * sizeof(TOUT)) % 16 == 0 && (g.batch_out * sizeof(TOUT)) % 16 == 0;
        constexpr int CH = BN / 32 / NGRP;  // 32-column chunks per group
#pragma unroll 1
        for (int jj = 0; jj < CH; ++jj) {
          const int j = grp * CH + jj;
          float v[32];
          ld32_f(t_row + j * 32, v);
          const int n = n0 + j * 32;
          if (g.bias0 != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (n + i < g.N) v[i] += g.bias0[n + i];
          }
          if (m < g.M && n < g.N) store_row32<TOUT>(out + n, v, g.N - n, vec_ok);
        }
      } else if constexpr (EPI == EPI_GATE_IN || EPI == EPI_GATE_IN_BWD) {
        // row = channel of half tm; columns: P for pixels n0..n0+127, then G for the same pixels
        const long long n0 = (long long)tn * 128;
        const long long nb0 = n0 / g.plane, np0 = n0 - nb0 * g.plane;   // one division per tile
        const bool wide16 = sizeof(TOUT) == 2 && (g.plane & 15) == 0 && (g.N & 15) == 0 && (g.ld_out & 15) == 0;
        const TIN* mask = reinterpret_cast<const TIN*>(g.aux);
        float bp = 0.f, bg = 0.f;
        if (g.bias0 != nullptr) { bp = g.bias0[tm * 256 + row]; bg = g.bias0[tm * 256 + 128 + row]; }
#pragma unroll
        for (int jj = 0; jj < CPG; ++jj) {
          const int j = grp * CPG + jj;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {   // 16 pixels at a time keeps the registers of 576 threads within budget
            float p[16], gt[16];
            ld16x2_f(t_row + j * 32 + hf * 16, t_row + 128 + j * 32 + hf * 16, p, gt);
            float o0[16], o1[16];   // GATE_IN: gated value; GATE_IN_BWD: dP and dG
            long long bb16 = 0, pix16 = 0;
#pragma unroll
            for (int uu = 0; uu < 2; ++uu) {
              const int u = hf * 2 + uu;
              const long long m8 = n0 + j * 32 + u * 8;   // 8 pixels: same batch entry, all valid or none
              if (m8 >= g.N) continue;
              long long bb = nb0, pix = np0 + j * 32 + u * 8;
              while (pix >= g.plane) { pix -= g.plane; ++bb; }
              if (uu == 0) { bb16 = bb; pix16 = pix; }
              float mk[8];
              if (mask != nullptr) load8<TIN>(mask + m8, mk);
              const float2 bp2 = make_float2(bp, bp), bg2 = make_float2(bg, bg);
              if constexpr (EPI == EPI_GATE_IN) {
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                  const float2 pv = __fadd2_rn(make_float2(p[uu * 8 + i], p[uu * 8 + i + 1]), bp2);
                  const float2 sg = sigmoid2(__fadd2_rn(make_float2(gt[uu * 8 + i], gt[uu * 8 + i + 1]), bg2));
                  float2 r = __fmul2_rn(pv, sg);
                  if (mask != nullptr) r = __fmul2_rn(r, make_float2(mk[i], mk[i + 1]));
                  o0[uu * 8 + i] = r.x;
                  o0[uu * 8 + i + 1] = r.y;
                }
                if (!wide16) store8<TOUT>(gate_in_dst<TOUT>(g, tm, bb, row, pix), &o0[uu * 8]);
              } else {
                float d[8];
                cvtraw8<TIN>(dpre[jj][u], d);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                  float2 dd = make_float2(d[i], d[i + 1]);
                  if (mask != nullptr) dd = __fmul2_rn(dd, make_float2(mk[i], mk[i + 1]));
                  const float2 sg = sigmoid2(__fadd2_rn(make_float2(gt[uu * 8 + i], gt[uu * 8 + i + 1]), bg2));
                  const float2 pv = __fadd2_rn(make_float2(p[uu * 8 + i], p[uu * 8 + i + 1]), bp2);
                  const float2 dp = __fmul2_rn(dd, sg);                                           // d * sig
                  const float2 oms = __ffma2_rn(sg, make_float2(-1.0f, -1.0f), make_float2(1.0f, 1.0f));
                  const float2 dg = __fmul2_rn(__fmul2_rn(dp, pv), oms);                          // d * P * sig * (1 - sig)
                  o0[uu * 8 + i] = dp.x; o0[uu * 8 + i + 1] = dp.y;
                  o1[uu * 8 + i] = dg.x; o1[uu * 8 + i + 1] = dg.y;
                }
                if (!wide16) {
                  TOUT* o = reinterpret_cast<TOUT*>(g.out0);
                  store8<TOUT>(o + (long long)(tm * 256 + row) * g.ld_out + m8, &o0[uu * 8]);
                  store8<TOUT>(o + (long long)(tm * 256 + 128 + row) * g.ld_out + m8, &o1[uu * 8]);
                }
              }
            }
            if constexpr (sizeof(TOUT) == 2) {
              const long long m16 = n0 + j * 32 + hf * 16;
              if (wide16 && m16 < g.N) {   // one 32-byte store per output row
                if constexpr (EPI == EPI_GATE_IN) {
                  store16<TOUT>(gate_in_dst<TOUT>(g, tm, bb16, row, pix16), o0);
                } else {
                  TOUT* o = reinterpret_cast<TOUT*>(g.out0);
                  store16<TOUT>(o + (long long)(tm * 256 + row) * g.ld_out + m16, o0);
                  store16<TOUT>(o + (long long)(tm * 256 + 128 + row) * g.ld_out + m16, o1);
                }
              }
            }
          }
        }
      } else {
        // EPI_GATE_OUT / EPI_GATE_OUT_BWD: row = pixel; cols [0,128) = y, [128,256) = gate pre-activation
        const int m = tm * kBM + row;
        TOUT* o0 = reinterpret_cast<TOUT*>(g.out0) + (long long)m * 128;
        TOUT* o1 = reinterpret_cast<TOUT*>(g.out1) + (long long)m * 128;
#pragma unroll
        for (int jj = 0; jj < CPG; ++jj) {
          const int j = grp * CPG + jj;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            float y[16], gt[16];
            ld16x2_f(t_row + j * 32 + hf * 16, t_row + 128 + j * 32 + hf * 16, y, gt);
            if (m < g.M) {
              float r0[16], r1[16];
#pragma unroll
              for (int uu = 0; uu < 2; ++uu) {
                const int u = hf * 2 + uu;
                float d[8];
                if constexpr (EPI == EPI_GATE_OUT_BWD) cvtraw8<TIN>(dpre[jj][u], d);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const int c = j * 32 + u * 8 + i;
                  float yv = y[uu * 8 + i], gv = gt[uu * 8 + i];
                  if (g.bias0 != nullptr) { yv += g.bias0[c]; gv += g.bias0[128 + c]; }
                  const float sg = fast_sigmoid(gv);
                  if constexpr (EPI == EPI_GATE_OUT) {
                    r0[uu * 8 + i] = yv * sg;
                  } else {
                    r0[uu * 8 + i] = d[i] * sg;
                    r1[uu * 8 + i] = d[i] * yv * sg * (1.0f - sg);
                  }
                }
              }
              // 16 channels of this pixel: one 32-byte store for 16-bit outputs (rows are 256 bytes, so it is aligned)
              if constexpr (sizeof(TOUT) == 2) {
                store16<TOUT>(o0 + j * 32 + hf * 16, r0);
                if constexpr (EPI == EPI_GATE_OUT_BWD) store16<TOUT>(o1 + j * 32 + hf * 16, r1);
              } else {
                store8<TOUT>(o0 + j * 32 + hf * 16, r0);
                store8<TOUT>(o0 + j * 32 + hf * 16 + 8, r0 + 8);
                if constexpr (EPI == EPI_GATE_OUT_BWD) {
                  store8<TOUT>(o1 + j * 32 + hf * 16, r1);
                  store8<TOUT>(o1 + j * 32 + hf * 16 + 8, r1 + 8);
                }
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
// One GEMM operand: a rank-3 tensor (inner, outer, batch); inner is contiguous.  K-major: inner = K,
// outer = rows (M or N).  MN-major: inner = rows, outer = K.
struct Operand {
  const void* ptr = nullptr;
  bool mn_major = false;
  uint64_t inner = 0, outer = 0, batch = 1;
  uint64_t st_outer = 0, st_batch = 0;  // elements
};

struct GemmPlan {
  Operand a[2], b[2];
  int M = 0, N = 0;
  int K0 = 0, K1 = 0;        // K extent per segment (per split when split_k)
  int seg1_col = 0;
  int batches = 1;
  int split_k = 0;
  int a_tiles = 0;           // > 0: A's batch dimension enumerates this many 128-row M tiles (gate-in GEMMs)
  void* out0 = nullptr;
  void* out1 = nullptr;
  long long ld_out = 0, batch_out = 0;
  const float* bias0 = nullptr;
  const void* aux = nullptr;
  const void* aux2 = nullptr;
  const void* aux3 = nullptr;
  long long plane = 0;
  void* const* peer_out = nullptr;   // GATE_IN: per-rank exchange buffers (see GemmArgs)
  int peer_world = 0, peer_rank = 0, peer_batches = 0;
  const char* name = "tc_gemm";
  double flops = 0, bytes = 0;
};

// dtype: TRI_F32 (tf32 MMA), TRI_BF16, TRI_F16.  out_f32: EPI_STORE writes fp32 instead of the input dtype.
int launch_gemm(cudaStream_t st, int dtype, int epi, int bn, bool out_f32, const GemmPlan& p, int* err);

}  // namespace tc
}  // namespace tri
