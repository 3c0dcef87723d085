// LayerNorm fused into the two projection kernels of the triangle multiplicative update (see tc_lngemm.cuh).
//
// ln_gate_in.  One persistent CTA per SM, 704 threads:
//   warp 0       TMA: the concatenated weights once (128 KB, resident), then one 128-pixel x tile per step into one of
//                two 32 KB buffers
//   warp 1       tcgen05.mma: per tile and half (a, b) the P and G products, M = the half's 128 channels, N = 128
//                pixels, into one of two 256-column accumulators (the halves alternate, so the epilogue of one half
//                runs under the products of the other)
//   warps 2-5    LayerNorm: thread = pixel row; normalises the row in place (two passes over it in shared memory:
//                statistics, result), writes the statistics, releases the tile to the MMA warp and
//                stores it as z with one TMA store per 64-channel half.  (With two warps owning two rows each the
//                kernel ran at the pace of this role: 9.4 us per tile against 5.4 for the two gate epilogues.)
//   warps 6-21   gate epilogue, thread = channel holding consecutive pixels (the order of the channel-major a / b)
//
// Against the two-kernel form (LayerNorm kernel, then the gate GEMM reading z once per half) x is read once, z is
// written from shared memory and never read back here, and the weights stay in shared memory.  The gate epilogue is
// bound by instruction issue, and the LayerNorm role's instructions compete with it for the same schedulers, so the
// kernel is slower than the gate GEMM alone (0.21 against 0.165 ms per launch at 768 x 768 pixels) but faster than
// the pair (0.24).
// Every mbarrier wait is bounded; a timeout lands in *err and all roles drain.
#include "tc_lngemm.cuh"

#include "tc_gemm.cuh"

namespace tri {
namespace tc {

namespace {

constexpr int kThreads = 704;
constexpr int kSub = 16384;                 // one [128 rows x 128 bytes] swizzled sub-tile
constexpr uint32_t kWBytes = 8 * kSub;      // (Pa, Ga, Pb, Gb) x (k 0..63, k 64..127)
constexpr uint32_t kXBytes = 2 * kSub;      // one pixel tile: two 64-channel halves
constexpr int kXBufs = 2;                 // (a third buffer, which still fits, changed nothing)

struct Args {
  long long M, plane;
  int tiles;
  float eps;
  const void* gamma;
  const void* beta;
  const float* bias;
  const void* mask;
  void* a_cm;
  void* b_cm;
  float* mean;
  float* rstd;
  int* err;
};

template <typename T> __device__ __forceinline__ void unpack8(const uint4& w, float (&v)[8]) {
  union { uint4 u; T h[8]; } pk;
  pk.u = w;
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = to_f32(pk.h[i]);
}
template <typename T> __device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  union { uint4 u; T h[8]; } pk;
#pragma unroll
  for (int i = 0; i < 8; ++i) pk.h[i] = from_f32<T>(v[i]);
  return pk.u;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
ln_gate_in_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                  const __grid_constant__ CUtensorMap tmZ, const Args g) {
  constexpr int KIND = ElemTraits<T>::kind;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;
  uint8_t* sX = smem + kWBytes;
  float* s_gamma = reinterpret_cast<float*>(sX + kXBufs * kXBytes);
  float* s_beta = s_gamma + 128;
  uint64_t* wfull = reinterpret_cast<uint64_t*>(s_beta + 128);
  uint64_t* xfull = wfull + 1;            // [kXBufs] tile landed (TMA bytes)
  uint64_t* xnorm = xfull + kXBufs;       // [kXBufs] tile normalised (one arrival per LayerNorm warp)
  uint64_t* xempty = xnorm + kXBufs;      // [kXBufs] tile consumed: the products (commit) and the z store (its reads) are done
  uint64_t* tfull = xempty + kXBufs;      // [2] accumulator of half h complete
  uint64_t* tempty = tfull + 2;     // [2] accumulator of half h read by all 16 epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(wfull, 1);
    for (int b = 0; b < kXBufs; ++b) { mbar_init(&xfull[b], 1); mbar_init(&xnorm[b], 4); mbar_init(&xempty[b], 2); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 16); }
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmZ);
  }
  if (threadIdx.x < 128) {
    s_gamma[threadIdx.x] = g.gamma ? to_f32(reinterpret_cast<const T*>(g.gamma)[threadIdx.x]) : 1.f;
    s_beta[threadIdx.x] = g.beta ? to_f32(reinterpret_cast<const T*>(g.beta)[threadIdx.x]) : 0.f;
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(wfull, kWBytes);
      for (int blk = 0; blk < 4; ++blk)
        for (int kb = 0; kb < 2; ++kb) tma_load_3d(sW + (blk * 2 + kb) * kSub, &tmW, wfull, kb * 64, blk * 128, 0);
      int i = 0;
      for (int tile = blockIdx.x; tile < g.tiles; tile += gridDim.x, ++i) {
        const int b = i % kXBufs;
        if (!mbar_wait(&xempty[b], ((i / kXBufs) & 1) ^ 1, g.err, 10)) break;
        mbar_expect_tx(&xfull[b], kXBytes);
        for (int kb = 0; kb < 2; ++kb) tma_load_3d(sX + b * kXBytes + kb * kSub, &tmX, &xfull[b], kb * 64, tile * 128, 0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc(KIND, 128, 128, false, false);
      const uint32_t w_base = smem_u32(sW), x_base = smem_u32(sX);
      bool ok = mbar_wait(wfull, 0, g.err, 11);
      int i = 0;
      for (int tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x, ++i) {
        const int b = i % kXBufs;
        if (!mbar_wait(&xnorm[b], (i / kXBufs) & 1, g.err, 12)) break;
        tc_fence_after_sync();
        for (int half = 0; half < 2 && ok; ++half) {
          if (!mbar_wait(&tempty[half], (i & 1) ^ 1, g.err, 13)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int pg = 0; pg < 2; ++pg) {   // P block, G block of this half
            const uint32_t d_addr = tmem_base + half * 256 + pg * 128;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb)
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = make_smem_desc(w_base + ((half * 2 + pg) * 2 + kb) * kSub + ks * 32, 16, 1024);
                const uint64_t bd = make_smem_desc(x_base + b * kXBytes + kb * kSub + ks * 32, 16, 1024);
                umma<KIND>(d_addr, ad, bd, idesc, (kb == 0 && ks == 0) ? 0u : 1u);
              }
          }
          umma_commit(&tfull[half]);
        }
        if (ok) umma_commit(&xempty[b]);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------------ LayerNorm: thread = pixel row of the tile
    const int r0 = threadIdx.x - 64;
    const uint32_t sw = (uint32_t)(r0 & 7) << 4;
    int i = 0;
    for (int tile = blockIdx.x; tile < g.tiles; tile += gridDim.x, ++i) {
      const int b = i % kXBufs;
      const bool landed = mbar_wait(&xfull[b], (i / kXBufs) & 1, g.err, 14);
      if (!__all_sync(0xffffffffu, landed)) break;
      const int r = r0;
      uint8_t* rowp = sX + b * kXBytes + r * 128;
      // Statistics in one pass over the row, shifted by its first element K: sums of (x - K) and (x - K)^2.  K is one
      // of the 128 samples, so (mean - K)^2 <= 128 var and the subtraction below loses at most seven bits of fp32.
      // Packed fp32x2 arithmetic and two accumulators each: the pass is a chain of dependent additions.
      float2 s0 = make_float2(0.f, 0.f), s1 = s0, q0 = s0, q1 = s0;
      float2 nk;
      {
        float v[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(rowp + sw), v);
        nk = make_float2(-v[0], -v[0]);
      }
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        float v[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(rowp + (c >> 3) * kSub + (((c & 7) << 4) ^ sw)), v);
        const float2 d0 = __fadd2_rn(make_float2(v[0], v[1]), nk), d1 = __fadd2_rn(make_float2(v[2], v[3]), nk);
        const float2 d2 = __fadd2_rn(make_float2(v[4], v[5]), nk), d3 = __fadd2_rn(make_float2(v[6], v[7]), nk);
        s0 = __fadd2_rn(s0, d0); q0 = __ffma2_rn(d0, d0, q0);
        s1 = __fadd2_rn(s1, d1); q1 = __ffma2_rn(d1, d1, q1);
        s0 = __fadd2_rn(s0, d2); q0 = __ffma2_rn(d2, d2, q0);
        s1 = __fadd2_rn(s1, d3); q1 = __ffma2_rn(d3, d3, q1);
      }
      const float ms = ((s0.x + s0.y) + (s1.x + s1.y)) * (1.0f / 128);          // mean - K
      const float mu = ms - nk.x;
      const float var = fmaxf(((q0.x + q0.y) + (q1.x + q1.y)) * (1.0f / 128) - ms * ms, 0.f);
      const float rs = 1.0f / sqrtf(var + g.eps);
      const float2 nmu = make_float2(-mu, -mu);
      const float2 rs2 = make_float2(rs, rs);
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        uint4* p = reinterpret_cast<uint4*>(rowp + (c >> 3) * kSub + (((c & 7) << 4) ^ sw));
        float v[8];
        unpack8<T>(*p, v);
        const float4 g0 = *reinterpret_cast<const float4*>(s_gamma + c * 8), g1 = *reinterpret_cast<const float4*>(s_gamma + c * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(s_beta + c * 8), b1 = *reinterpret_cast<const float4*>(s_beta + c * 8 + 4);
        const float2 o0 = __ffma2_rn(__fadd2_rn(make_float2(v[0], v[1]), nmu), __fmul2_rn(rs2, make_float2(g0.x, g0.y)), make_float2(b0.x, b0.y));
        const float2 o1 = __ffma2_rn(__fadd2_rn(make_float2(v[2], v[3]), nmu), __fmul2_rn(rs2, make_float2(g0.z, g0.w)), make_float2(b0.z, b0.w));
        const float2 o2 = __ffma2_rn(__fadd2_rn(make_float2(v[4], v[5]), nmu), __fmul2_rn(rs2, make_float2(g1.x, g1.y)), make_float2(b1.x, b1.y));
        const float2 o3 = __ffma2_rn(__fadd2_rn(make_float2(v[6], v[7]), nmu), __fmul2_rn(rs2, make_float2(g1.z, g1.w)), make_float2(b1.z, b1.w));
        const float o[8] = {o0.x, o0.y, o1.x, o1.y, o2.x, o2.y, o3.x, o3.y};
        *p = pack8<T>(o);
      }
      const long long m = (long long)tile * 128 + r;
      if (m < g.M) { g.mean[m] = mu; g.rstd[m] = rs; }
      fence_proxy_async_smem();   // the tile is read next by tcgen05.mma and by the TMA store
      __syncwarp();
      if (lane == 0) mbar_arrive(&xnorm[b]);
      if (r0 == 0) {
        // every row is normalised once all four warps have arrived; then z leaves from shared memory
        if (mbar_wait(&xnorm[b], (i / kXBufs) & 1, g.err, 15)) {
          tma_store_3d(&tmZ, sX + b * kXBytes, 0, tile * 128, 0);
          tma_store_3d(&tmZ, sX + b * kXBytes + kSub, 64, tile * 128, 0);
          bulk_commit_group();
          bulk_wait_group_read0();
          mbar_arrive(&xempty[b]);
        }
      }
      __syncwarp();
    }
    if (r0 == 0) bulk_wait_group0();
  } else {
    // ------------------------------------------------------------------ gate epilogue: thread = channel of the half
    const int quarter = warp & 3, j = (warp - 6) >> 2;   // TMEM lane quarter; 32-pixel chunk of the tile
    const int row = quarter * 32 + lane;
    const bool wide16 = (g.plane & 15) == 0 && (g.M & 15) == 0;
    const T* mask = reinterpret_cast<const T*>(g.mask);
    int i = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x, ++i) {
      const long long n0 = (long long)tile * 128;
      const long long nb0 = n0 / g.plane, np0 = n0 - nb0 * g.plane;   // one division per tile
      for (int half = 0; half < 2; ++half) {
        const bool done = mbar_wait(&tfull[half], i & 1, g.err, 16);
        if (!__all_sync(0xffffffffu, done)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 256;
        float bp = 0.f, bg = 0.f;
        if (g.bias != nullptr) { bp = g.bias[half * 256 + row]; bg = g.bias[half * 256 + 128 + row]; }
        const float2 bp2 = make_float2(bp, bp), bg2 = make_float2(bg, bg);
        T* dplane = reinterpret_cast<T*>(half == 0 ? g.a_cm : g.b_cm);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          float p[16], gt[16], o[16];
          ld16x2_f(t_row + j * 32 + hf * 16, t_row + 128 + j * 32 + hf * 16, p, gt);
          long long bb16 = 0, pix16 = 0;
#pragma unroll
          for (int uu = 0; uu < 2; ++uu) {
            const int off = j * 32 + hf * 16 + uu * 8;
            const long long m8 = n0 + off;   // 8 pixels: same batch entry, all valid or none
            if (m8 >= g.M) continue;
            long long bb = nb0, pix = np0 + off;
            while (pix >= g.plane) { pix -= g.plane; ++bb; }
            if (uu == 0) { bb16 = bb; pix16 = pix; }
            float mk[8];
            if (mask != nullptr) load8<T>(mask + m8, mk);
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              const float2 pv = __fadd2_rn(make_float2(p[uu * 8 + e], p[uu * 8 + e + 1]), bp2);
              const float2 sg = sigmoid2(__fadd2_rn(make_float2(gt[uu * 8 + e], gt[uu * 8 + e + 1]), bg2));
              float2 rr = __fmul2_rn(pv, sg);
              if (mask != nullptr) rr = __fmul2_rn(rr, make_float2(mk[e], mk[e + 1]));
              o[uu * 8 + e] = rr.x;
              o[uu * 8 + e + 1] = rr.y;
            }
            if (!wide16) store8<T>(dplane + (bb * 128 + row) * g.plane + pix, &o[uu * 8]);
          }
          if (wide16 && n0 + j * 32 + hf * 16 < g.M) store16<T>(dplane + (bb16 * 128 + row) * g.plane + pix16, o);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[half]);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T>
int launch(cudaStream_t st, const LnGateIn& p) {
  const uint64_t M = (uint64_t)p.M;
  CUtensorMap tmX, tmW, tmZ;
  const uint64_t xd[3] = {128, M, 1}, xs[2] = {128, 128 * M};
  const uint64_t wd[3] = {128, 512, 1}, wsd[2] = {128, 128 * 512};
  const uint32_t box[3] = {64, 128, 1};
  const bool f16 = p.dtype == TRI_F16;
  TRI_TRY(make_tmap_3d(&tmX, p.x, 2, f16, xd, xs, box, false));
  TRI_TRY(make_tmap_3d(&tmW, p.wcat, 2, f16, wd, wsd, box, false));
  TRI_TRY(make_tmap_3d(&tmZ, p.z, 2, f16, xd, xs, box, false));
  Args a;
  a.M = p.M; a.plane = p.plane; a.tiles = (int)((p.M + 127) / 128); a.eps = p.eps;
  a.gamma = p.gamma; a.beta = p.beta; a.bias = p.bias_cat; a.mask = p.mask;
  a.a_cm = p.a_cm; a.b_cm = p.b_cm; a.mean = p.mean; a.rstd = p.rstd; a.err = p.err;
  constexpr size_t smem = 1024 + kWBytes + kXBufs * kXBytes + 2 * 128 * sizeof(float) + (1 + 3 * kXBufs + 4) * 8 + 16;
  static_assert(smem <= 232448, "shared memory of one CTA");
  auto kern = ln_gate_in_kernel<T>;
  TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = std::min(a.tiles, sm_count());
  KernelTimer kt("tc_ln_gate_in", st, 2.0 * p.M * 128 * 512, 4.0 * p.M * 128 * 2);
  kern<<<grid, kThreads, smem, st>>>(tmX, tmW, tmZ, a);
  TRI_LAUNCH_OK();
  return 0;
}


// =================================================================================================================
// ln_gate_out: LayerNorm over the channels of channel-major t, fused into the output projection and gate
// =================================================================================================================
// 704 threads as above.  A tile is 128 pixels.  Its t part arrives as the MN-major A operand of the product
// y = u Wo^T: per 64-channel half, two chunks of [64 channel rows x 128 bytes = 64 pixels] (128-byte swizzle), which
// is how the contraction's output lies in memory -- nothing is transposed.  The LayerNorm role normalises every
// pixel's 128 channels in place: a thread owns 8 pixels (one 16-byte piece of a row) and 16 of the 128 channels;
// the eight partial (mean, M2) pairs of a pixel are combined through shared memory (Chan's formula), then each
// thread rewrites its pieces and, for training, stores them to the channel-major u the backward pass reads.
// The z part (K-major) feeds the gate product unchanged.  Output weights and gate weights stay in shared memory.
constexpr uint32_t kOWBytes = 4 * kSub;     // (Wo, Wgo) x (k 0..63, k 64..127)
constexpr uint32_t kOTile = 4 * kSub;       // t: 2 halves x [2 chunks x 8 KB]; z: 2 halves x 16 KB
constexpr int kOBufs = 2;

struct OutArgs {
  long long M;
  int tiles;
  float eps;
  const void* gamma;
  const void* beta;
  const float* bias;
  void* u_cm;
  float* mean;
  float* rstd;
  void* out;
  int* err;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
ln_gate_out_kernel(const __grid_constant__ CUtensorMap tmT, const __grid_constant__ CUtensorMap tmZ,
                   const __grid_constant__ CUtensorMap tmWo, const __grid_constant__ CUtensorMap tmWg, const OutArgs g) {
  constexpr int KIND = ElemTraits<T>::kind;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;
  uint8_t* sT = smem + kOWBytes;
  float* s_pm = reinterpret_cast<float*>(sT + kOBufs * kOTile);   // [8][128] partial means
  float* s_pq = s_pm + 8 * 128;                                   // [8][128] partial sums of squared deviations
  float* s_mean = s_pq + 8 * 128;
  float* s_rstd = s_mean + 128;
  float* s_gamma = s_rstd + 128;
  float* s_beta = s_gamma + 128;
  uint64_t* wfull = reinterpret_cast<uint64_t*>(s_beta + 128);
  uint64_t* bfull = wfull + 1;            // [kOBufs] tile landed
  uint64_t* bnorm = bfull + kOBufs;       // [kOBufs] t part normalised (one arrival per LayerNorm warp)
  uint64_t* bempty = bnorm + kOBufs;      // [kOBufs] both products of the tile are done
  uint64_t* tfull = bempty + kOBufs;      // [2] accumulator complete
  uint64_t* tempty = tfull + 2;           // [2] accumulator read by all 16 epilogue warps
  uint64_t* nsync = tempty + 2;           // [2] the two meeting points of the 128 LayerNorm threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(nsync + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(wfull, 1);
    for (int b = 0; b < kOBufs; ++b) { mbar_init(&bfull[b], 1); mbar_init(&bnorm[b], 4); mbar_init(&bempty[b], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 16); mbar_init(&nsync[b], 128); }
    mbar_fence_init();
    tma_prefetch_desc(&tmT);
    tma_prefetch_desc(&tmZ);
    tma_prefetch_desc(&tmWo);
    tma_prefetch_desc(&tmWg);
  }
  if (threadIdx.x < 128) {
    s_gamma[threadIdx.x] = g.gamma ? to_f32(reinterpret_cast<const T*>(g.gamma)[threadIdx.x]) : 1.f;
    s_beta[threadIdx.x] = g.beta ? to_f32(reinterpret_cast<const T*>(g.beta)[threadIdx.x]) : 0.f;
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(wfull, kOWBytes);
      for (int kb = 0; kb < 2; ++kb) {
        tma_load_3d(sW + kb * kSub, &tmWo, wfull, kb * 64, 0, 0);
        tma_load_3d(sW + (2 + kb) * kSub, &tmWg, wfull, kb * 64, 0, 0);
      }
      int i = 0;
      for (int tile = blockIdx.x; tile < g.tiles; tile += gridDim.x, ++i) {
        const int b = i % kOBufs;
        if (!mbar_wait(&bempty[b], ((i / kOBufs) & 1) ^ 1, g.err, 20)) break;
        uint8_t* buf = sT + b * kOTile;
        mbar_expect_tx(&bfull[b], kOTile);
        for (int kb = 0; kb < 2; ++kb) {
          for (int c = 0; c < 2; ++c) tma_load_3d(buf + kb * kSub + c * (kSub / 2), &tmT, &bfull[b], tile * 128 + c * 64, kb * 64, 0);
          tma_load_3d(buf + 2 * kSub + kb * kSub, &tmZ, &bfull[b], kb * 64, tile * 128, 0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_y = make_idesc(KIND, 128, 128, true, false);    // A = u tile, pixels contiguous
      const uint32_t idesc_g = make_idesc(KIND, 128, 128, false, false);   // A = z tile, channels contiguous
      const uint32_t w_base = smem_u32(sW), t_base = smem_u32(sT);
      bool ok = mbar_wait(wfull, 0, g.err, 21);
      int i = 0;
      for (int tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x, ++i) {
        const int b = i % kOBufs, acc = i & 1;
        if (!mbar_wait(&bnorm[b], (i / kOBufs) & 1, g.err, 22)) break;
        if (!mbar_wait(&tempty[acc], ((i >> 1) & 1) ^ 1, g.err, 23)) break;
        tc_fence_after_sync();
        const uint32_t buf = t_base + b * kOTile, d_addr = tmem_base + acc * 256;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            // 16 channel rows per MMA; the second 64-pixel chunk of the half lies 8 KB further
            const uint64_t ad = make_smem_desc(buf + kb * kSub + ks * 16 * 128, kSub / 2, 1024);
            const uint64_t bd = make_smem_desc(w_base + kb * kSub + ks * 32, 16, 1024);
            umma<KIND>(d_addr, ad, bd, idesc_y, (kb == 0 && ks == 0) ? 0u : 1u);
          }
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = make_smem_desc(buf + (2 + kb) * kSub + ks * 32, 16, 1024);
            const uint64_t bd = make_smem_desc(w_base + (2 + kb) * kSub + ks * 32, 16, 1024);
            umma<KIND>(d_addr + 128, ad, bd, idesc_g, (kb == 0 && ks == 0) ? 0u : 1u);
          }
        umma_commit(&tfull[acc]);
        umma_commit(&bempty[b]);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------------ LayerNorm over channels
    const int tid = threadIdx.x - 64;
    const int pg = tid & 15, kp = tid >> 4;       // 8-pixel group of the tile; 16-channel part
    const int gg = pg & 7;                        // 16-byte piece within the 128-byte row of its 64-pixel chunk
    const uint32_t part_off = (kp >> 2) * kSub + (pg >> 3) * (kSub / 2) + (kp & 3) * 16 * 128;
    T* u_cm = reinterpret_cast<T*>(g.u_cm);
    int i = 0;
    for (int tile = blockIdx.x; tile < g.tiles; tile += gridDim.x, ++i) {
      const int b = i % kOBufs;
      const bool landed = mbar_wait(&bfull[b], (i / kOBufs) & 1, g.err, 24);
      if (!__all_sync(0xffffffffu, landed)) break;
      uint8_t* part = sT + b * kOTile + part_off;   // rows kp*16 .. kp*16+15 of this thread's chunk
      // partial statistics of 8 pixels over 16 channels, shifted by the first channel's values
      float2 nk[4], s[4], q[4];
      {
        float v[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(part + (gg << 4)), v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          nk[e] = make_float2(-v[2 * e], -v[2 * e + 1]);
          s[e] = make_float2(0.f, 0.f);
          q[e] = s[e];
        }
      }
#pragma unroll 4
      for (int r = 0; r < 16; ++r) {
        float v[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(part + r * 128 + ((gg ^ (r & 7)) << 4)), v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 d = __fadd2_rn(make_float2(v[2 * e], v[2 * e + 1]), nk[e]);
          s[e] = __fadd2_rn(s[e], d);
          q[e] = __ffma2_rn(d, d, q[e]);
        }
      }
      {
        float pm[8], pq[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float sx = s[e].x * (1.0f / 16), sy = s[e].y * (1.0f / 16);
          pm[2 * e] = sx - nk[e].x;                       // mean of the 16 samples
          pm[2 * e + 1] = sy - nk[e].y;
          pq[2 * e] = fmaxf(q[e].x - s[e].x * sx, 0.f);   // their sum of squared deviations
          pq[2 * e + 1] = fmaxf(q[e].y - s[e].y * sy, 0.f);
        }
        float4* dm = reinterpret_cast<float4*>(s_pm + kp * 128 + pg * 8);
        float4* dq = reinterpret_cast<float4*>(s_pq + kp * 128 + pg * 8);
        dm[0] = make_float4(pm[0], pm[1], pm[2], pm[3]); dm[1] = make_float4(pm[4], pm[5], pm[6], pm[7]);
        dq[0] = make_float4(pq[0], pq[1], pq[2], pq[3]); dq[1] = make_float4(pq[4], pq[5], pq[6], pq[7]);
      }
      mbar_arrive(&nsync[0]);
      const bool met0 = mbar_wait(&nsync[0], i & 1, g.err, 25);
      if (!__all_sync(0xffffffffu, met0)) break;
      {
        // thread = pixel: combine the eight partials (equal counts): M2 = sum M2_k + 16 sum (mean_k - mean)^2
        float pm[8], m = 0.f, m2 = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) { pm[k] = s_pm[k * 128 + tid]; m += pm[k]; m2 += s_pq[k * 128 + tid]; }
        m *= (1.0f / 8);
        float dev = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) dev = fmaf(pm[k] - m, pm[k] - m, dev);
        const float rs = 1.0f / sqrtf((m2 + 16.f * dev) * (1.0f / 128) + g.eps);
        s_mean[tid] = m;
        s_rstd[tid] = rs;
        const long long px = (long long)tile * 128 + tid;
        if (px < g.M) { g.mean[px] = m; g.rstd[px] = rs; }
      }
      mbar_arrive(&nsync[1]);
      const bool met1 = mbar_wait(&nsync[1], i & 1, g.err, 26);
      if (!__all_sync(0xffffffffu, met1)) break;
      {
        const float4 m0 = *reinterpret_cast<const float4*>(s_mean + pg * 8), m1 = *reinterpret_cast<const float4*>(s_mean + pg * 8 + 4);
        const float4 r0 = *reinterpret_cast<const float4*>(s_rstd + pg * 8), r1 = *reinterpret_cast<const float4*>(s_rstd + pg * 8 + 4);
        const float2 nm[4] = {make_float2(-m0.x, -m0.y), make_float2(-m0.z, -m0.w), make_float2(-m1.x, -m1.y), make_float2(-m1.z, -m1.w)};
        const float2 rr[4] = {make_float2(r0.x, r0.y), make_float2(r0.z, r0.w), make_float2(r1.x, r1.y), make_float2(r1.z, r1.w)};
        const long long px0 = (long long)tile * 128 + pg * 8;   // 8 pixels: all inside the tensor or none
        T* udst = (u_cm != nullptr && px0 < g.M) ? u_cm + (long long)(kp * 16) * g.M + px0 : nullptr;
#pragma unroll 4
        for (int r = 0; r < 16; ++r) {
          uint4* p = reinterpret_cast<uint4*>(part + r * 128 + ((gg ^ (r & 7)) << 4));
          float v[8], o[8];
          unpack8<T>(*p, v);
          const float gm = s_gamma[kp * 16 + r], bt = s_beta[kp * 16 + r];
          const float2 gm2 = make_float2(gm, gm), bt2 = make_float2(bt, bt);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 y = __ffma2_rn(__fadd2_rn(make_float2(v[2 * e], v[2 * e + 1]), nm[e]), __fmul2_rn(rr[e], gm2), bt2);
            o[2 * e] = y.x;
            o[2 * e + 1] = y.y;
          }
          const uint4 w = pack8<T>(o);
          *p = w;
          if (udst != nullptr) *reinterpret_cast<uint4*>(udst + (long long)r * g.M) = w;
        }
      }
      fence_proxy_async_smem();   // the tile is read next by tcgen05.mma
      __syncwarp();
      if (lane == 0) mbar_arrive(&bnorm[b]);
    }
  } else {
    // ------------------------------------------------------------------ gate epilogue: thread = pixel
    const int quarter = warp & 3, j = (warp - 6) >> 2;   // TMEM lane quarter; 32-channel chunk of the output row
    const int row = quarter * 32 + lane;
    int i = 0;
    for (int tile = blockIdx.x; tile < g.tiles; tile += gridDim.x, ++i) {
      const int acc = i & 1;
      const bool done = mbar_wait(&tfull[acc], (i >> 1) & 1, g.err, 27);
      if (!__all_sync(0xffffffffu, done)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
      const long long m = (long long)tile * 128 + row;
      T* orow = reinterpret_cast<T*>(g.out) + m * 128;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float y[16], gt[16];
        ld16x2_f(t_row + j * 32 + hf * 16, t_row + 128 + j * 32 + hf * 16, y, gt);
        if (m < g.M) {
          float o[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int c = j * 32 + hf * 16 + e;
            float yv = y[e], gv = gt[e];
            if (g.bias != nullptr) { yv += g.bias[c]; gv += g.bias[128 + c]; }
            o[e] = yv * fast_sigmoid(gv);
          }
          store16<T>(orow + j * 32 + hf * 16, o);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T>
int launch_out(cudaStream_t st, const LnGateOut& p) {
  const uint64_t M = (uint64_t)p.M;
  CUtensorMap tmT, tmZ, tmWo, tmWg;
  const bool f16 = p.dtype == TRI_F16;
  const uint64_t td[3] = {M, 128, 1}, ts[2] = {M, 128 * M};
  const uint32_t tbox[3] = {64, 64, 1};
  const uint64_t zd[3] = {128, M, 1}, zs[2] = {128, 128 * M};
  const uint64_t wd[3] = {128, 128, 1}, wsd[2] = {128, 128 * 128};
  const uint32_t box[3] = {64, 128, 1};
  TRI_TRY(make_tmap_3d(&tmT, p.t_cm, 2, f16, td, ts, tbox, false));
  TRI_TRY(make_tmap_3d(&tmZ, p.z, 2, f16, zd, zs, box, false));
  TRI_TRY(make_tmap_3d(&tmWo, p.w_out, 2, f16, wd, wsd, box, false));
  TRI_TRY(make_tmap_3d(&tmWg, p.w_gate, 2, f16, wd, wsd, box, false));
  OutArgs a;
  a.M = p.M; a.tiles = (int)((p.M + 127) / 128); a.eps = p.eps; a.gamma = p.gamma; a.beta = p.beta;
  a.bias = p.bias_out; a.u_cm = p.u_cm; a.mean = p.mean; a.rstd = p.rstd; a.out = p.out; a.err = p.err;
  constexpr size_t smem = 1024 + kOWBytes + kOBufs * kOTile + (2 * 8 * 128 + 4 * 128) * sizeof(float) + (1 + 3 * kOBufs + 6) * 8 + 16;
  static_assert(smem <= 232448, "shared memory of one CTA");
  auto kern = ln_gate_out_kernel<T>;
  TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = std::min(a.tiles, sm_count());
  KernelTimer kt("tc_ln_gate_out", st, 2.0 * p.M * 128 * 256, (p.u_cm ? 4.0 : 3.0) * p.M * 128 * 2);
  kern<<<grid, kThreads, smem, st>>>(tmT, tmZ, tmWo, tmWg, a);
  TRI_LAUNCH_OK();
  return 0;
}

}  // namespace

bool ln_gate_in_supported(int dtype, long long M, long long plane) {
  return (dtype == TRI_BF16 || dtype == TRI_F16) && M > 0 && plane > 0 && plane % 8 == 0 && M % plane == 0 &&
         M < (1LL << 31) - 128;
}

int ln_gate_in(cudaStream_t st, const LnGateIn& p) {
  if (!ln_gate_in_supported(p.dtype, p.M, p.plane)) return fail(TRI_ERR_ARG, "ln_gate_in: unsupported shape or dtype");
  return p.dtype == TRI_BF16 ? launch<__nv_bfloat16>(st, p) : launch<__half>(st, p);
}

bool ln_gate_out_supported(int dtype, long long M, long long plane) {
  return (dtype == TRI_BF16 || dtype == TRI_F16) && M > 0 && M == plane && M % 8 == 0 && M < (1LL << 31) - 128;
}

int ln_gate_out(cudaStream_t st, const LnGateOut& p) {
  if (!ln_gate_out_supported(p.dtype, p.M, p.M)) return fail(TRI_ERR_ARG, "ln_gate_out: unsupported shape or dtype");
  return p.dtype == TRI_BF16 ? launch_out<__nv_bfloat16>(st, p) : launch_out<__half>(st, p);
}

}  // namespace tc
}  // namespace tri
