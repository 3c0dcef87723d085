// LayerNorm fused into the input projection of the triangle multiplicative update (see tc_lngemm.cuh).
//
// One persistent CTA per SM, 704 threads:
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

}  // namespace

bool ln_gate_in_supported(int dtype, long long M, long long plane) {
  return (dtype == TRI_BF16 || dtype == TRI_F16) && M > 0 && plane > 0 && plane % 8 == 0 && M % plane == 0 &&
         M < (1LL << 31) - 128;
}

int ln_gate_in(cudaStream_t st, const LnGateIn& p) {
  if (!ln_gate_in_supported(p.dtype, p.M, p.plane)) return fail(TRI_ERR_ARG, "ln_gate_in: unsupported shape or dtype");
  return p.dtype == TRI_BF16 ? launch<__nv_bfloat16>(st, p) : launch<__half>(st, p);
}

}  // namespace tc
}  // namespace tri
