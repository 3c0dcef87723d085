// extern "C" surface of libtri_b200.so: argument checks and dispatch between the
// tensor-core (tcgen05) kernels and the exact-fp32 CUDA-core kernels.
#include <algorithm>
#include <atomic>
#include <cstring>
#include <initializer_list>
#include <mutex>
#include <map>
#include <string>
#include <vector>

#include "attn_simt.cuh"
#include "common.cuh"
#include "tc_gemm.cuh"
#include "tc_paths.cuh"
#include "trimul_simt.cuh"

namespace tri {
namespace {
thread_local char g_err[512] = "";
std::atomic<const char*> g_path{"none"};  // process-wide: the backward runs on autograd's thread
// Launch counter and timing records are process-wide: autograd runs the backward on its own thread.
std::atomic<long long> g_launches{0};

struct ProfRecord { const char* name; cudaEvent_t beg, end; double flops, bytes; };
std::atomic<bool> g_prof_on{false};
std::mutex g_prof_mu;
std::vector<ProfRecord>* g_prof = nullptr;
}  // namespace

KernelTimer::KernelTimer(const char* name, cudaStream_t stream, double flops, double bytes) : slot(-1), st(stream) {
  if (!g_prof_on.load()) return;
  std::lock_guard<std::mutex> lock(g_prof_mu);
  if (g_prof == nullptr) g_prof = new std::vector<ProfRecord>();
  ProfRecord r{name, nullptr, nullptr, flops, bytes};
  if (cudaEventCreate(&r.beg) != cudaSuccess || cudaEventCreate(&r.end) != cudaSuccess) return;
  cudaEventRecord(r.beg, st);
  g_prof->push_back(r);
  slot = (int)g_prof->size() - 1;
}
KernelTimer::~KernelTimer() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lock(g_prof_mu);
  if (g_prof != nullptr && slot < (int)g_prof->size()) cudaEventRecord((*g_prof)[slot].end, st);
}

int sm_count() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cache[kMaxDevices];   // zero-initialised; 0 = not queried yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < kMaxDevices) {
    const int n = cache[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev >= 0 && dev < kMaxDevices) cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

char* last_error_buf() { return g_err; }
void set_path(const char* name) { g_path.store(name); }
void count_launch(int n) { g_launches += n; }

static int check_attn(const TriAttnDesc* d) {
  if (d == nullptr) return fail(TRI_ERR_ARG, "descriptor is null");
  if (d->B <= 0 || d->n_seq <= 0 || d->n_res <= 0 || d->H <= 0 || d->D <= 0)
    return fail(TRI_ERR_ARG, "attention sizes must be positive (B=%d n_seq=%d n_res=%d H=%d D=%d)", d->B,
                d->n_seq, d->n_res, d->H, d->D);
  if (d->D > 128) return fail(TRI_ERR_UNSUPPORTED, "head dim %d > 128 is not supported", d->D);
  if (d->dtype < TRI_F32 || d->dtype > TRI_F16) return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
  if (d->precision != TRI_PREC_IEEE && d->precision != TRI_PREC_TF32)
    return fail(TRI_ERR_ARG, "bad precision %d", d->precision);
  if ((long long)d->B * d->n_seq * d->H > 2147483647LL / 4) return fail(TRI_ERR_UNSUPPORTED, "too many rows");
  return 0;
}

static int check_mul(const TriMulDesc* d) {
  if (d == nullptr) return fail(TRI_ERR_ARG, "descriptor is null");
  if (d->B <= 0 || d->N <= 0 || d->C <= 0 || d->Ch <= 0)
    return fail(TRI_ERR_ARG, "trimul sizes must be positive (B=%d N=%d C=%d Ch=%d)", d->B, d->N, d->C, d->Ch);
  if (d->C > 1024 || d->Ch > 1024) return fail(TRI_ERR_UNSUPPORTED, "channel width above 1024 is not supported");
  if (d->dtype < TRI_F32 || d->dtype > TRI_F16) return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
  if (d->precision != TRI_PREC_IEEE && d->precision != TRI_PREC_TF32)
    return fail(TRI_ERR_ARG, "bad precision %d", d->precision);
  if (d->direction != TRI_OUTGOING && d->direction != TRI_INCOMING)
    return fail(TRI_ERR_ARG, "bad direction %d", d->direction);
  if ((long long)d->B * d->N * d->N * 2 * std::max(d->C, d->Ch) > 2147483647LL * 8)
    return fail(TRI_ERR_UNSUPPORTED, "pair tensor too large");
  return 0;
}

// What the tensor-core attention kernels need beyond the descriptor: every tensor they reach through a tensor map
// starts on a 16-byte boundary, and a bias that is present is not a broadcast view over heads or queries (its batch
// stride may be zero).  Anything else runs on the CUDA-core kernels, which take any pointer and stride.
static bool attn_operands_fit_tma(const TriAttnDesc* d, const void* bias, std::initializer_list<const void*> ptrs) {
  for (const void* p : ptrs)
    if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
  if (bias != nullptr) {
    if ((reinterpret_cast<uintptr_t>(bias) & 15) != 0) return false;
    if (d->bias_st[1] == 0 && d->H > 1) return false;
    if (d->bias_st[2] == 0 && d->n_res > 1) return false;
  }
  return true;
}

}  // namespace tri

using namespace tri;

extern "C" {

int tri_abi_version(void) { return 1; }
const char* tri_last_error(void) { return last_error_buf(); }
const char* tri_last_path(void) { return g_path.load(); }
long long tri_launch_count(void) { return g_launches.load(); }
void tri_reset_launch_count(void) { g_launches = 0; }

void tri_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(g_prof_mu);
  if (g_prof != nullptr) {
    for (auto& r : *g_prof) { cudaEventDestroy(r.beg); cudaEventDestroy(r.end); }
    g_prof->clear();
  }
  g_prof_on = on != 0;
}

int tri_profile_summary(char* buf, size_t cap) {
  if (buf == nullptr || cap == 0) return fail(TRI_ERR_ARG, "buffer is null");
  buf[0] = 0;
  std::lock_guard<std::mutex> lock(g_prof_mu);
  if (g_prof == nullptr) return 0;
  struct Agg { int n = 0; double ms = 0, flops = 0, bytes = 0; };
  std::map<std::string, Agg> agg;
  for (auto& r : *g_prof) {
    TRI_CUDA_OK(cudaEventSynchronize(r.end));
    float ms = 0.f;
    TRI_CUDA_OK(cudaEventElapsedTime(&ms, r.beg, r.end));
    auto& a = agg[r.name];
    a.n += 1;
    a.ms += ms;
    a.flops += r.flops;
    a.bytes += r.bytes;
  }
  size_t off = 0;
  for (auto& kv : agg) {
    int n = snprintf(buf + off, cap - off, "%s %d %.6f %.6e %.6e\n", kv.first.c_str(), kv.second.n, kv.second.ms,
                     kv.second.flops, kv.second.bytes);
    if (n < 0 || (size_t)n >= cap - off) return fail(TRI_ERR_ARG, "buffer too small");
    off += (size_t)n;
  }
  return 0;
}

size_t tri_attn_ws_bytes(const TriAttnDesc* d, int is_bwd) {
  if (check_attn(d) != 0) return 0;
  return std::max(tc::attn_ws_bytes(d, is_bwd), simt::attn_ws_bytes(d, is_bwd));
}

int tri_attn_fwd(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                 const uint8_t* mask, void* o, float* lse, void* ws, size_t ws_bytes, tri_stream_t stream) {
  TRI_TRY(check_attn(d));
  if (!q || !k || !v || !o || !lse) return fail(TRI_ERR_ARG, "q, k, v, o and lse must not be null");
  if (tc::attn_fwd_supported(d) && attn_operands_fit_tma(d, bias, {q, k, v})) {
    set_path("tcgen05");
    return tc::attn_forward(d, q, k, v, bias, mask, o, lse, ws, ws_bytes, (cudaStream_t)stream);
  }
  set_path("simt");
  return simt::attn_forward(d, q, k, v, bias, mask, o, lse, (cudaStream_t)stream);
}

int tri_attn_bwd(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                 const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                 void* dv, float* dbias, void* ws, size_t ws_bytes, tri_stream_t stream) {
  TRI_TRY(check_attn(d));
  if (!q || !k || !v || !o || !lse || !d_o || !dq || !dk || !dv || !ws)
    return fail(TRI_ERR_ARG, "q, k, v, o, lse, d_o, dq, dk, dv and ws must not be null");
  if (tc::attn_bwd_supported(d) && attn_operands_fit_tma(d, bias, {q, k, v, d_o})) {
    set_path("tcgen05");
    return tc::attn_backward(d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, ws, ws_bytes,
                             (cudaStream_t)stream);
  }
  set_path("simt");
  return simt::attn_backward(d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, ws, ws_bytes,
                             (cudaStream_t)stream);
}

int tri_attn_bwd_noalloc(const TriAttnDesc* d, const void* q, const void* k, const void* v, const void* bias,
                         const uint8_t* mask, const void* o, const float* lse, const void* d_o, void* dq, void* dk,
                         void* dv, float* dbias, tri_stream_t stream) {
  TRI_TRY(check_attn(d));
  if (!q || !k || !v || !o || !lse || !d_o || !dq || !dk || !dv)
    return fail(TRI_ERR_ARG, "q, k, v, o, lse, d_o, dq, dk and dv must not be null");
  return simt::attn_backward_static(d, q, k, v, bias, mask, o, lse, d_o, dq, dk, dv, dbias, (cudaStream_t)stream);
}

static int check_project(const TriAttnProjDesc* d) {
  if (d == nullptr) return fail(TRI_ERR_ARG, "descriptor is null");
  if (d->dtype < TRI_F32 || d->dtype > TRI_F16) return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
  if (!tc::attn_project_supported(d))
    return fail(TRI_ERR_UNSUPPORTED, "the fused projection needs C = 128, 1 <= H <= 8, H*D a multiple of 8, and bf16 / fp16 or fp32-tf32");
  return 0;
}

size_t tri_attn_project_ws_bytes(const TriAttnProjDesc* d) {
  return check_project(d) != 0 ? 0 : tc::attn_project_ws_bytes(d);
}

int tri_attn_project(const TriAttnProjDesc* d, const void* z, const void* ln_w, const void* ln_b, const void* w_qkv,
                     const void* w_bias, void* qkv, void* bias, void* ws, size_t ws_bytes, tri_stream_t stream) {
  TRI_TRY(check_project(d));
  if (!z || !w_qkv || !w_bias || !qkv || !bias || !ws) return fail(TRI_ERR_ARG, "z, w_qkv, w_bias, qkv, bias and ws must not be null");
  set_path("tcgen05");
  return tc::attn_project(d, z, ln_w, ln_b, w_qkv, w_bias, qkv, bias, ws, ws_bytes, (cudaStream_t)stream);
}

size_t tri_mul_saved_bytes(const TriMulDesc* d) {
  if (check_mul(d) != 0) return 0;
  return tc::mul_supported(d) ? tc::mul_saved_bytes(d) : simt::saved_bytes(d);
}

size_t tri_mul_ws_bytes(const TriMulDesc* d, int is_bwd) {
  if (check_mul(d) != 0) return 0;
  return tc::mul_supported(d) ? tc::mul_ws_bytes(d, is_bwd) : simt::ws_bytes(d, is_bwd);
}

static int check_mul_weights(const TriMulWeights* w) {
  if (w == nullptr || !w->p_in_w || !w->g_in_w || !w->p_out_w || !w->g_out_w)
    return fail(TRI_ERR_ARG, "p_in, g_in, p_out and g_out weights are required");
  return 0;
}

int tri_mul_fwd(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, void* out,
                void* saved, void* ws, size_t ws_bytes, tri_stream_t stream) {
  TRI_TRY(check_mul(d));
  TRI_TRY(check_mul_weights(w));
  if (!x || !out || !ws) return fail(TRI_ERR_ARG, "x, out and ws must not be null");
  if (tc::mul_supported(d)) {
    set_path("tcgen05");
    return tc::mul_forward(d, x, mask, w, out, saved, ws, ws_bytes, (cudaStream_t)stream);
  }
  set_path("simt");
  return simt::forward(d, x, mask, w, out, saved, ws, ws_bytes, (cudaStream_t)stream);
}

int tri_mul_bwd(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w, const void* saved,
                const void* d_out, void* dx, const TriMulWeightGrads* g, void* ws, size_t ws_bytes,
                tri_stream_t stream) {
  TRI_TRY(check_mul(d));
  TRI_TRY(check_mul_weights(w));
  if (!x || !saved || !d_out || !dx || !g || !ws)
    return fail(TRI_ERR_ARG, "x, saved, d_out, dx, grads and ws must not be null");
  if (tc::mul_supported(d)) {
    set_path("tcgen05");
    return tc::mul_backward(d, x, mask, w, saved, d_out, dx, g, ws, ws_bytes, (cudaStream_t)stream);
  }
  set_path("simt");
  return simt::backward(d, x, mask, w, saved, d_out, dx, g, ws, ws_bytes, (cudaStream_t)stream);
}

static int check_shard(const TriMulShardDesc* d) {
  if (d == nullptr) return fail(TRI_ERR_ARG, "descriptor is null");
  if (d->B <= 0 || d->rows <= 0 || d->N <= 0) return fail(TRI_ERR_ARG, "shard sizes must be positive");
  if (d->dtype < TRI_F32 || d->dtype > TRI_F16) return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
  if (!tc::mul_shard_supported(d))
    return fail(TRI_ERR_UNSUPPORTED, "sharded trimul needs C = Ch = 128, N %% 8 == 0 and bf16/fp16 or fp32-tf32");
  return 0;
}

size_t tri_mul_shard_saved_bytes(const TriMulShardDesc* d) {
  return check_shard(d) != 0 ? 0 : tc::mul_shard_saved_bytes(d);
}

size_t tri_mul_shard_ws_bytes(const TriMulShardDesc* d, int phase) {
  return check_shard(d) != 0 ? 0 : tc::mul_shard_ws_bytes(d, phase);
}

size_t tri_mul_shard_prep_bytes(const TriMulShardDesc* d) {
  return check_shard(d) != 0 ? 0 : tc::mul_shard_prep_bytes(d);
}

int tri_mul_shard_phase(const TriMulShardDesc* d, int phase, const TriMulShardBufs* bufs, void* ws, size_t ws_bytes,
                        tri_stream_t stream) {
  TRI_TRY(check_shard(d));
  if (!bufs || !bufs->w || !bufs->saved || !ws) return fail(TRI_ERR_ARG, "bufs, weights, saved and ws must not be null");
  TRI_TRY(check_mul_weights(bufs->w));
  set_path("tcgen05");
  return tc::mul_shard_phase(d, phase, bufs, ws, ws_bytes, (cudaStream_t)stream);
}

// one block row per (outer index, slice of the run): 16-byte copies, source and destination both contiguous per run
static __global__ void permute_runs_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long d0, long long d1,
                                    long long d2, int p0, int p1, int p2, long long run_v) {
  const long long outer = blockIdx.y;   // destination outer index, dimensions (d[p0], d[p1], d[p2])
  const long long dd[3] = {d0, d1, d2};
  const long long e2 = dd[p2], e1 = dd[p1];
  long long idx[3];
  idx[p2] = outer % e2;
  idx[p1] = (outer / e2) % e1;
  idx[p0] = outer / (e2 * e1);
  const uint4* s = src + ((idx[0] * d1 + idx[1]) * d2 + idx[2]) * run_v;
  uint4* d = dst + outer * run_v;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; i + 3 * stride < run_v; i += 4 * stride) {   // four loads in flight per thread
    const uint4 a = __ldg(s + i), b = __ldg(s + i + stride), c = __ldg(s + i + 2 * stride), e = __ldg(s + i + 3 * stride);
    d[i] = a; d[i + stride] = b; d[i + 2 * stride] = c; d[i + 3 * stride] = e;
  }
  for (; i < run_v; i += stride) d[i] = __ldg(s + i);
}

int tri_permute_runs(const void* src, void* dst, const int64_t dims[3], const int32_t perm[3], int64_t run_bytes,
                     tri_stream_t stream) {
  if (src == nullptr || dst == nullptr) return fail(TRI_ERR_ARG, "tri_permute_runs: null pointer");
  if (run_bytes <= 0 || run_bytes % 16 != 0 || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15))
    return fail(TRI_ERR_ARG, "tri_permute_runs: runs must be 16-byte aligned multiples of 16 bytes");
  int seen = 0;
  for (int i = 0; i < 3; ++i) {
    if (perm[i] < 0 || perm[i] > 2 || dims[i] <= 0) return fail(TRI_ERR_ARG, "tri_permute_runs: bad permutation or extent");
    seen |= 1 << perm[i];
  }
  if (seen != 7) return fail(TRI_ERR_ARG, "tri_permute_runs: perm is not a permutation");
  const long long outer = dims[0] * dims[1] * dims[2];
  if (outer > 65535) return fail(TRI_ERR_ARG, "tri_permute_runs: more than 65535 runs");
  const long long run_v = run_bytes / 16;
  const int bx = (int)std::max<long long>(1, std::min<long long>(32, (run_v + 2047) / 2048));
  KernelTimer kt("tri_permute_runs", (cudaStream_t)stream, 0.0, 2.0 * outer * run_bytes);
  permute_runs_kernel<<<dim3(bx, (unsigned)outer), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), dims[0], dims[1], dims[2], perm[0], perm[1], perm[2], run_v);
  TRI_LAUNCH_OK();
  return 0;
}

struct ScatterPtrs { uint4* p[16]; };

static __global__ void scatter_runs_kernel(const uint4* __restrict__ src, ScatterPtrs dst, long long d1, long long d2,
                                           long long s0, long long s1, long long s2, long long base, int peer_dim,
                                           long long run_v) {
  const long long outer = blockIdx.y;   // source run index (i0, i1, i2)
  const long long i2 = outer % d2, i1 = (outer / d2) % d1, i0 = outer / (d2 * d1);
  const long long peer = peer_dim == 0 ? i0 : (peer_dim == 1 ? i1 : i2);
  const uint4* s = src + outer * run_v;
  uint4* d = dst.p[peer] + (base + i0 * s0 + i1 * s1 + i2 * s2) * run_v;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; i + 3 * stride < run_v; i += 4 * stride) {
    const uint4 a = __ldg(s + i), b = __ldg(s + i + stride), c = __ldg(s + i + 2 * stride), e = __ldg(s + i + 3 * stride);
    d[i] = a; d[i + stride] = b; d[i + 2 * stride] = c; d[i + 3 * stride] = e;
  }
  for (; i < run_v; i += stride) d[i] = __ldg(s + i);
}

int tri_scatter_runs(const TriScatterDesc* d, const void* src, void* const* dst_ptrs, tri_stream_t stream) {
  if (d == nullptr || src == nullptr || dst_ptrs == nullptr) return fail(TRI_ERR_ARG, "tri_scatter_runs: null pointer");
  if (d->run_bytes <= 0 || d->run_bytes % 16 != 0 || ((uintptr_t)src & 15))
    return fail(TRI_ERR_ARG, "tri_scatter_runs: runs must be 16-byte aligned multiples of 16 bytes");
  if (d->peer_dim < 0 || d->peer_dim > 2 || d->n_peers < 1 || d->n_peers > 16 || d->dims[d->peer_dim] != d->n_peers)
    return fail(TRI_ERR_ARG, "tri_scatter_runs: bad peer dimension");
  ScatterPtrs ptrs = {};
  for (int i = 0; i < d->n_peers; ++i) {
    if (dst_ptrs[i] == nullptr || ((uintptr_t)dst_ptrs[i] & 15)) return fail(TRI_ERR_ARG, "tri_scatter_runs: bad destination pointer");
    ptrs.p[i] = static_cast<uint4*>(dst_ptrs[i]);
  }
  const long long outer = d->dims[0] * d->dims[1] * d->dims[2];
  if (outer <= 0 || outer > 65535) return fail(TRI_ERR_ARG, "tri_scatter_runs: between 1 and 65535 runs");
  const long long run_v = d->run_bytes / 16;
  const int bx = (int)std::max<long long>(1, std::min<long long>(32, (run_v + 2047) / 2048));
  KernelTimer kt("tri_scatter_runs", (cudaStream_t)stream, 0.0, 2.0 * outer * d->run_bytes);
  scatter_runs_kernel<<<dim3(bx, (unsigned)outer), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const uint4*>(src), ptrs, d->dims[1], d->dims[2], d->dst_stride[0], d->dst_stride[1], d->dst_stride[2],
      d->dst_base_run, d->peer_dim, run_v);
  TRI_LAUNCH_OK();
  return 0;
}

int tri_scatter_runs_dma(const TriScatterDesc* d, const void* src, void* const* dst_ptrs, tri_stream_t stream) {
  if (d == nullptr || src == nullptr || dst_ptrs == nullptr) return fail(TRI_ERR_ARG, "tri_scatter_runs_dma: null pointer");
  if (d->run_bytes <= 0 || d->run_bytes % 16 != 0 || ((uintptr_t)src & 15))
    return fail(TRI_ERR_ARG, "tri_scatter_runs_dma: runs must be 16-byte aligned multiples of 16 bytes");
  if (d->peer_dim < 0 || d->peer_dim > 2 || d->n_peers < 1 || d->n_peers > 16 || d->dims[d->peer_dim] != d->n_peers)
    return fail(TRI_ERR_ARG, "tri_scatter_runs_dma: bad peer dimension");
  for (int i = 0; i < d->n_peers; ++i)
    if (dst_ptrs[i] == nullptr || ((uintptr_t)dst_ptrs[i] & 15)) return fail(TRI_ERR_ARG, "tri_scatter_runs_dma: bad destination pointer");
  const long long outer = d->dims[0] * d->dims[1] * d->dims[2];
  if (outer <= 0) return fail(TRI_ERR_ARG, "tri_scatter_runs_dma: empty exchange");
  // source strides in runs (the source is contiguous); rows of a 2-D copy walk the longer of the two other dimensions
  const long long ss[3] = {d->dims[1] * d->dims[2], d->dims[2], 1};
  const int p = d->peer_dim, o0 = p == 0 ? 1 : 0, o1 = p == 2 ? 1 : 2;
  const int b = d->dims[o0] >= d->dims[o1] ? o0 : o1, a = b == o0 ? o1 : o0;
  const long long run = d->run_bytes;
  const long long spitch = std::max<long long>(ss[b], 1) * run, dpitch = std::max<long long>(d->dst_stride[b], 1) * run;
  if (d->dims[b] > 1 && (d->dst_stride[b] < 1 || spitch > 2147483647LL || dpitch > 2147483647LL))
    return fail(TRI_ERR_UNSUPPORTED, "tri_scatter_runs_dma: pitch beyond a two-dimensional copy");
  KernelTimer kt("tri_scatter_dma", (cudaStream_t)stream, 0.0, 2.0 * outer * run);
  for (long long w = 0; w < d->n_peers; ++w)
    for (long long ia = 0; ia < d->dims[a]; ++ia) {
      const char* s = static_cast<const char*>(src) + (w * ss[p] + ia * ss[a]) * run;
      char* t = static_cast<char*>(dst_ptrs[w]) + (d->dst_base_run + w * d->dst_stride[p] + ia * d->dst_stride[a]) * run;
      TRI_CUDA_OK(cudaMemcpy2DAsync(t, (size_t)dpitch, s, (size_t)spitch, (size_t)run, (size_t)d->dims[b],
                                    cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    }
  return 0;
}

// ---- arrival flags for the peer-store exchange -------------------------------------------------------------------
// state[0] = number of barriers this rank has entered, state[3] = status of the last wait (0 = ok).  Both live in this
// GPU's memory and are advanced by the kernel itself, so a captured graph can be replayed without changing an argument.
struct SignalPtrs { uint32_t* flags[16]; };

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One block, one thread per peer.  Thread w tells peer w "everything this rank queued before barrier number e has
// been stored" (slot `rank` of that peer's flag array := e, release at system scope; the copy kernel ahead of this
// one on the stream has completed, so its stores are performed), then waits until peer w has said the same here.
// The wait is bounded: when the limit runs out state[3] records which peer was missing and the kernel returns, so
// a rank that never arrives shows up as an error status instead of a hung GPU.
static __global__ void peer_barrier_kernel(SignalPtrs sig, int rank, int n_peers, uint32_t* state, long long limit_cycles) {
  __shared__ uint32_t epoch;
  if (threadIdx.x == 0) { epoch = state[0] + 1; state[0] = epoch; }
  __syncthreads();
  const int w = threadIdx.x;
  if (w < n_peers) {
    store_release_sys(sig.flags[w] + rank, epoch);
    const uint32_t* mine = sig.flags[rank] + w;
    const long long t0 = clock64();
    bool ok = false;
    for (;;) {
      if ((int32_t)(load_acquire_sys(mine) - epoch) >= 0) { ok = true; break; }
      if (clock64() - t0 > limit_cycles) break;
    }
    if (!ok) atomicCAS(&state[3], 0u, 100u + w);
  }
}

int tri_peer_barrier(const TriPeerSignal* sig, int64_t limit_cycles, tri_stream_t stream) {
  if (sig == nullptr || sig->flag_ptrs == nullptr || sig->state == nullptr || sig->n_peers < 1 || sig->n_peers > 16 ||
      sig->rank < 0 || sig->rank >= sig->n_peers)
    return fail(TRI_ERR_ARG, "tri_peer_barrier: bad signal descriptor");
  SignalPtrs sp = {};
  for (int i = 0; i < sig->n_peers; ++i) {
    if (sig->flag_ptrs[i] == nullptr) return fail(TRI_ERR_ARG, "tri_peer_barrier: null flag pointer");
    sp.flags[i] = static_cast<uint32_t*>(sig->flag_ptrs[i]);
  }
  if (limit_cycles <= 0) limit_cycles = 10000000000LL;   // about five seconds of SM clocks: ranks may be skewed by a
                                                          // first-call set-up (module load, buffer rendezvous)
  KernelTimer kt("tri_peer_barrier", (cudaStream_t)stream, 0.0, 0.0);
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(sp, sig->rank, sig->n_peers, sig->state, limit_cycles);
  TRI_LAUNCH_OK();
  return 0;
}

int tri_ws_status(const void* ws, tri_stream_t stream) {
  if (ws == nullptr) return fail(TRI_ERR_ARG, "ws is null");
  int code = 0;
  TRI_CUDA_OK(cudaMemcpyAsync(&code, ws, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  TRI_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  if (code != 0) return fail(TRI_ERR_DEVICE, "a tensor-core kernel gave up waiting (code %d)", code);
  return 0;
}

int tri_bgemm(const TriGemmDesc* d, const void* a, const void* b, void* c, void* ws, size_t ws_bytes,
              tri_stream_t stream) {
  if (!d || !a || !b || !c || !ws) return fail(TRI_ERR_ARG, "null argument");
  if (ws_bytes < 256) return fail(TRI_ERR_WORKSPACE, "tri_bgemm needs a 256-byte workspace");
  if (d->M <= 0 || d->N <= 0 || d->K <= 0 || d->batch <= 0) return fail(TRI_ERR_ARG, "sizes must be positive");
  if (d->dtype < TRI_F32 || d->dtype > TRI_F16) return fail(TRI_ERR_ARG, "bad dtype %d", d->dtype);
  cudaStream_t st = (cudaStream_t)stream;
  TRI_CUDA_OK(cudaMemsetAsync(ws, 0, 256, st));
  tc::GemmPlan p;
  p.a[0].ptr = a; p.a[0].mn_major = d->a_mn_major != 0;
  p.a[0].inner = d->a_mn_major ? d->M : d->K; p.a[0].outer = d->a_mn_major ? d->K : d->M;
  p.a[0].batch = d->batch; p.a[0].st_outer = d->lda; p.a[0].st_batch = d->batch_a;
  p.b[0].ptr = b; p.b[0].mn_major = d->b_mn_major != 0;
  p.b[0].inner = d->b_mn_major ? d->N : d->K; p.b[0].outer = d->b_mn_major ? d->K : d->N;
  p.b[0].batch = d->batch; p.b[0].st_outer = d->ldb; p.b[0].st_batch = d->batch_b;
  p.M = d->M; p.N = d->N; p.K0 = d->K; p.batches = d->batch;
  p.out0 = c; p.ld_out = d->ldc; p.batch_out = d->batch_c;
  p.name = "tc_bgemm";
  p.flops = 2.0 * d->batch * d->M * (double)d->N * d->K;
  const double es = d->dtype == TRI_F32 ? 4.0 : 2.0;
  p.bytes = d->batch * (es * ((double)d->M * d->K + (double)d->N * d->K) + (d->out_f32 ? 4.0 : es) * d->M * d->N);
  set_path("tcgen05");
  return tc::launch_gemm(st, d->dtype, tc::EPI_STORE, d->N > 128 ? 256 : 128, d->out_f32 != 0, p, (int*)ws);
}

}  // extern "C"
