/*
 * tri_b200.h -- C ABI of libtri_b200.so: triangle attention and triangle
 * multiplicative update for NVIDIA B200 (sm_100a).
 *
 * The reference project (AMDResearch/geometric-nn-ops) is pure Python and has
 * no FFI; the seam these entry points replace is its private kernel package
 * (geometric_nn_ops_torch/triangle/_kernels/__init__.py:4-8 declares it
 * swappable).  Each function below names the reference kernel-layer function
 * whose work it takes over.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless it points to a descriptor struct.
 *  - The caller owns all memory, including workspaces; query the size first.
 *    No entry point here allocates, frees or synchronises; all work is queued
 *    on the given stream.
 *  - Return value: 0 = ok, <0 = bad argument (TRI_ERR_*), >0 = cudaError_t.
 *    tri_last_error() returns a thread-local message for the last failure.
 *  - Strides are in ELEMENTS.  The innermost (head-dim / channel) axis is
 *    always contiguous.
 */
#ifndef TRI_B200_H_
#define TRI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tri_stream_t; /* == cudaStream_t */

enum { TRI_F32 = 0, TRI_BF16 = 1, TRI_F16 = 2 };
/* fp32 matmul precision, as read from torch.backends.cuda.matmul.fp32_precision
 * (geometric_nn_ops_torch/_precision.py:34-44).  Ignored for 16-bit dtypes. */
enum { TRI_PREC_IEEE = 0, TRI_PREC_TF32 = 1 };
enum { TRI_OUTGOING = 0, TRI_INCOMING = 1 };
enum {
  TRI_ERR_ARG = -1,        /* null pointer / bad enum / bad size */
  TRI_ERR_WORKSPACE = -2,  /* workspace too small */
  TRI_ERR_UNSUPPORTED = -3,/* shape not supported by any kernel */
  TRI_ERR_DEVICE = -4      /* a kernel reported a failure (e.g. a bounded wait ran out) */
};

int tri_abi_version(void);
const char* tri_last_error(void);
/* Name of the kernel family the most recent forward/backward (on any thread) ran on:
 * "simt" (CUDA-core fp32 path) or "tcgen05" (tensor-core path). */
const char* tri_last_path(void);
/* Number of kernel launches issued by this library (all threads) since the
 * last call to tri_reset_launch_count(). */
long long tri_launch_count(void);
void tri_reset_launch_count(void);

/* Per-kernel timing for benchmarks (no counterpart in the reference, which uses torch.profiler in
 * benchmarks/profile_trimul.py:73-87).  While enabled, every kernel launch (any thread) is bracketed
 * by CUDA events on its stream.  tri_profile_summary waits for them and writes one line per kernel,
 * "name launches total_ms flops bytes", the last two being the ALGORITHMIC work the launches did.  Enabling (or disabling) drops earlier records. */
void tri_profile_enable(int on);
int tri_profile_summary(char* buf, size_t cap);

/* ------------------------------------------------------------------------ */
/* Triangle attention                                                       */
/* ------------------------------------------------------------------------ */
/* q, k, v, o, dO, dq, dk, dv: logical [B, n_seq, n_res, H, D], strides for
 * (batch, row, residue, head), D contiguous -- both the reference's native
 * layout and the cuequivariance (B, N, H, S, D) layout are plain stride
 * choices.  bias: [B, H, n_res, n_res] with strides (batch, head, query), key
 * contiguous; batch stride may be 0.  mask: bytes (bool), [B, n_seq, n_res]
 * with strides (batch, row), key contiguous; nonzero = keep.
 * lse: fp32 [2, B, n_seq, H, n_res] contiguous softmax statistics: plane 0 is the row maximum m of
 * the logits, plane 1 is log(sum_j exp(logit_j - m)); the log-sum-exp is their sum.  They are kept
 * apart because a fully masked row has m = -1e9, where adding the second term would round it away.
 * dbias: fp32 [B, H, n_res, n_res]
 * contiguous, summed over rows. */
typedef struct TriAttnDesc {
  int32_t B, n_seq, n_res, H, D;
  int32_t dtype;      /* TRI_F32 / TRI_BF16 / TRI_F16 */
  int32_t precision;  /* TRI_PREC_* */
  float scale;
  int64_t q_st[4], k_st[4], v_st[4], o_st[4];
  int64_t do_st[4], dq_st[4], dk_st[4], dv_st[4];
  int64_t bias_st[3];
  int64_t mask_st[2];
} TriAttnDesc;

/* Replaces EvoformerAttention.forward + _attn_fwd
 * (geometric_nn_ops_torch/triangle/_kernels/triangle_attention.py:1090-1276, 183-365). */
int tri_attn_fwd(const TriAttnDesc* d, const void* q, const void* k, const void* v,
                 const void* bias /*nullable*/, const uint8_t* mask /*nullable*/,
                 void* o, float* lse, void* ws, size_t ws_bytes, tri_stream_t stream);

/* Replaces EvoformerAttention.backward + _attn_bwd_preprocess / _attn_bwd_dk_dv /
 * _attn_bwd_dbias_dq (same file :1278-1442, 548-1087). */
int tri_attn_bwd(const TriAttnDesc* d, const void* q, const void* k, const void* v,
                 const void* bias, const uint8_t* mask, const void* o, const float* lse,
                 const void* d_o, void* dq, void* dk, void* dv, float* dbias /*nullable*/,
                 void* ws, size_t ws_bytes, tri_stream_t stream);

size_t tri_attn_ws_bytes(const TriAttnDesc* d, int is_bwd);

/* Attention backward for callers that cannot provide a workspace.  (No counterpart in the reference,
 * which always allocates through torch.)  Meant for hosts where device allocation is off limits at call
 * time: a serving loop running on a frozen memory pool, an operator plugin whose host exposes no
 * allocator, a process pinned at its memory budget.  Same arguments and results as tri_attn_bwd minus
 * the workspace: the per-row scratch (one float per (batch, row, head, query)) lives in a 4 MiB array
 * built into the library image, resident on every GPU that loads the library until the process exits.
 *  - Limit: B * n_seq * H * n_res <= 1048576; larger problems are refused with TRI_ERR_UNSUPPORTED.
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on each device
 *    resolves the array's device address (cudaGetSymbolAddress, with that device current); make that
 *    first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's contents.  Nothing in it
 *    has to start at zero (each call rewrites what it reads), but two calls whose kernels overlap on the
 *    GPU (different streams) race on it: serialise them.
 *  - Always runs the CUDA-core kernels, in every dtype. */
int tri_attn_bwd_noalloc(const TriAttnDesc* d, const void* q, const void* k, const void* v,
                         const void* bias, const uint8_t* mask, const void* o, const float* lse,
                         const void* d_o, void* dq, void* dk, void* dv, float* dbias /*nullable*/,
                         tri_stream_t stream);

/* Fused input projection of triangle attention inside a pair stack: zn = LayerNorm(z) over the 128 channels, then
 *   qkv[m][0 : 3*H*D] = zn[m] Wqkv^T   (one [M, 3*H*D] buffer: columns [0, H*D) are q, then k, then v, each read by
 *                                       tri_attn_fwd as [.., H, D] with a residue stride of 3*H*D elements)
 *   bias[h][m]        = zn[m] . Wb[h]  (head-major: with M = B*N*N pixels this is the [B, H, N, N] pair bias for B = 1)
 * No counterpart in the reference, whose attention takes pre-projected tensors
 * (geometric_nn_ops_torch/triangle/_triattn.py:36-44); callers there run a LayerNorm, four linears and a permute.
 * z: [M, C] contiguous, C = 128; ln_w / ln_b: [C] or NULL; w_qkv: [3*H*D, C]; w_bias: [H, C], H <= 8; everything in
 * `dtype` (fp32 needs precision tf32: tensor-core path only).  Forward only. */
typedef struct TriAttnProjDesc {
  int64_t M;
  int32_t C, H, D;
  int32_t dtype, precision;
  float eps;
} TriAttnProjDesc;

size_t tri_attn_project_ws_bytes(const TriAttnProjDesc* d);
int tri_attn_project(const TriAttnProjDesc* d, const void* z, const void* ln_w /*nullable*/, const void* ln_b /*nullable*/,
                     const void* w_qkv, const void* w_bias, void* qkv, void* bias, void* ws, size_t ws_bytes,
                     tri_stream_t stream);

/* ------------------------------------------------------------------------ */
/* Triangle multiplicative update                                           */
/* ------------------------------------------------------------------------ */
/* x, out, d_out, dx: [B, N, N, C] contiguous in `dtype`.  mask: [B, N, N]
 * contiguous in `dtype` (1 = keep), nullable.  Weights are contiguous in
 * `dtype`; p_in / g_in are the concatenated [a; b] projections [2*Ch, C]. */
typedef struct TriMulDesc {
  int32_t B, N, C, Ch;
  int32_t dtype, precision, direction;
  float eps;
} TriMulDesc;

typedef struct TriMulWeights {
  const void *norm_in_w, *norm_in_b;   /* [C]      nullable */
  const void *p_in_w, *p_in_b;         /* [2Ch,C], [2Ch] (bias nullable) */
  const void *g_in_w, *g_in_b;         /* [2Ch,C], [2Ch] */
  const void *norm_out_w, *norm_out_b; /* [Ch]     nullable */
  const void *p_out_w, *p_out_b;       /* [C,Ch],  [C] */
  const void *g_out_w, *g_out_b;       /* [C,C],   [C] */
} TriMulWeights;

/* fp32 outputs, same shapes as the weights; a null member is skipped. */
typedef struct TriMulWeightGrads {
  float *norm_in_w, *norm_in_b, *p_in_w, *p_in_b, *g_in_w, *g_in_b;
  float *norm_out_w, *norm_out_b, *p_out_w, *p_out_b, *g_out_w, *g_out_b;
} TriMulWeightGrads;

/* Bytes of the opaque block the forward fills for the backward. */
size_t tri_mul_saved_bytes(const TriMulDesc* d);
size_t tri_mul_ws_bytes(const TriMulDesc* d, int is_bwd);

/* Replaces trimul_triton (geometric_nn_ops_torch/triangle/_kernels/trimul.py:404-448)
 * and, for grad-requiring calls, the torch path trimul_torch
 * (geometric_nn_ops_torch/triangle/_reference/trimul.py:57-97).
 * saved == NULL means inference (nothing kept). */
int tri_mul_fwd(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w,
                void* out, void* saved /*nullable*/, void* ws, size_t ws_bytes,
                tri_stream_t stream);

/* Backward of the above.  The reference has no kernel for it: it differentiates
 * trimul_torch with autograd (geometric_nn_ops_torch/triangle/_trimul.py:31-36). */
int tri_mul_bwd(const TriMulDesc* d, const void* x, const void* mask, const TriMulWeights* w,
                const void* saved, const void* d_out, void* dx, const TriMulWeightGrads* g,
                void* ws, size_t ws_bytes, tri_stream_t stream);

/* ------------------------------------------------------------------------ */
/* Row-sharded triangle multiplicative update (one GPU per shard of rows)   */
/* ------------------------------------------------------------------------ */
/* No counterpart in the reference, which is single-device.  The pair tensor is sharded over its first
 * pair axis: this rank holds x[:, i0:i0+rows, :, :].  Everything except the contraction is pixel-wise, so
 * the op splits into phases around two exchanges that the caller performs (NCCL all-to-all):
 *   PROJECT      x -> a_cm, b_cm  [B, Ch, rows, N]   (channel-major gated projections of the local rows)
 *   ... exchange rows -> channels; contraction per channel with tri_bgemm; exchange channels -> rows ...
 *   OUTPUT       t_cm [B, Ch, rows, N] -> out [B, rows, N, C]
 *   OUTPUT_BWD   d_out, t_cm -> dt_cm, gradients of norm_out / p_out / g_out (this rank's partial sums)
 *   ... the two backward contractions between the same exchanges ...
 *   PROJECT_BWD  gradients da, db passed in a_cm, b_cm -> dx, gradients of norm_in / p_in / g_in (partial)
 * `saved` (tri_mul_shard_saved_bytes) carries z, u, dgo and the LayerNorm statistics between phases.
 * Weight gradients are per-rank partial sums: all-reduce them.  Tensor-core path only
 * (C = Ch = 128, N % 8 == 0, bf16 / fp16, or fp32 with precision tf32). */
typedef struct TriMulShardDesc {
  int32_t B, rows, N, C, Ch;
  int32_t dtype, precision;
  float eps;
} TriMulShardDesc;

typedef struct TriMulShardBufs {
  const void* x;            /* [B, rows, N, C] */
  const void* mask;         /* [B, rows, N], nullable */
  const TriMulWeights* w;
  void* saved;
  void* a_cm;               /* PROJECT: out a;  PROJECT_BWD: in da */
  void* b_cm;               /* PROJECT: out b;  PROJECT_BWD: in db */
  const void* t_cm;         /* OUTPUT, OUTPUT_BWD: in */
  void* out;                /* OUTPUT: out */
  const void* d_out;        /* OUTPUT_BWD: in */
  void* dt_cm;              /* OUTPUT_BWD: out */
  void* dx;                 /* PROJECT_BWD: out */
  const TriMulWeightGrads* g;
  /* PROJECT with peer_world > 1: the gate-in GEMM's epilogue stores a and b straight into every rank's exchange
   * buffer instead of a_cm / b_cm (compute and the row -> channel exchange in one kernel).  peer_ab[w] is rank w's
   * buffer, laid out [2*B, C_hidden/peer_world, peer_world*rows, N] (a for the first B entries, then b), as a
   * pointer valid on this GPU; channel c goes to rank c / (C_hidden/peer_world).  The caller provides the barrier
   * afterwards, as for tri_scatter_runs.  NULL / 0 keeps the plain outputs. */
  void* const* peer_ab;
  int32_t peer_world, peer_rank;
  /* Optional: a buffer of tri_mul_shard_prep_bytes() that carries the prepared weights (the concatenated, reordered
   * input projections and the fp32 bias vectors) from phase to phase.  Every phase needs them; with prep == NULL each
   * phase prepares them again in its workspace.  Pass prep_ready = 0 to the first phase that sees a set of weights
   * (it fills the buffer) and 1 to later phases of the same forward + backward. */
  void* prep;
  int32_t prep_ready;
} TriMulShardBufs;

enum { TRI_PHASE_PROJECT = 0, TRI_PHASE_OUTPUT = 1, TRI_PHASE_OUTPUT_BWD = 2, TRI_PHASE_PROJECT_BWD = 3 };

size_t tri_mul_shard_saved_bytes(const TriMulShardDesc* d);
size_t tri_mul_shard_ws_bytes(const TriMulShardDesc* d, int phase);
size_t tri_mul_shard_prep_bytes(const TriMulShardDesc* d);
int tri_mul_shard_phase(const TriMulShardDesc* d, int phase, const TriMulShardBufs* bufs, void* ws,
                        size_t ws_bytes, tri_stream_t stream);

/* ------------------------------------------------------------------------ */
/* Batched tensor-core GEMM (building block of the trimul contraction)      */
/* ------------------------------------------------------------------------ */
/* C[b][m][n] = sum_k A[b](m,k) * B[b](n,k), fp32 accumulation on tcgen05.  This is the per-channel
 * N x N x N "combine" step, which the reference runs as a torch.einsum over permuted views
 * (geometric_nn_ops_torch/triangle/_reference/trimul.py:44-54); exported for tests and benchmarks.
 * An operand is K-major ([rows][K], ld = row stride) or MN-major ([K][rows], ld = stride between k).
 * dtype TRI_F32 computes in tf32.  All strides in elements and multiples of 16 bytes. */
typedef struct TriGemmDesc {
  int32_t M, N, K, batch;
  int32_t dtype;
  int32_t a_mn_major, b_mn_major;
  int32_t out_f32;           /* store fp32 instead of `dtype` */
  int64_t lda, ldb, ldc;
  int64_t batch_a, batch_b, batch_c;
} TriGemmDesc;

int tri_bgemm(const TriGemmDesc* d, const void* a, const void* b, void* c, void* ws, size_t ws_bytes,
              tri_stream_t stream);

/* Layout change around the row <-> channel exchanges of the sharded multiplicative update (tri_mul_shard_phase):
 * dst[i_p0][i_p1][i_p2][run] = src[i0][i1][i2][run], where (p0, p1, p2) = perm is a permutation of the three
 * outer dimensions (dst dimension k is src dimension perm[k]) and `run_bytes` contiguous bytes move together
 * (a multiple of 16; both pointers 16-byte aligned).  It replaces torch's permute().contiguous() on the packing
 * and unpacking sides of the all-to-all, which ran at a quarter of HBM bandwidth.  No counterpart in the
 * reference (single device). */
int tri_permute_runs(const void* src, void* dst, const int64_t dims[3], const int32_t perm[3], int64_t run_bytes,
                     tri_stream_t stream);

/* The same run copy with the destination on other GPUs: an all-to-all with the layout change folded in, done by
 * plain stores into peer-mapped memory over NVLink (one pass over the data, against pack + NCCL all-to-all +
 * unpack).  Run (i0, i1, i2) of src goes to GPU i_{peer_dim}, at run index
 *   dst_base_run + i0*dst_stride[0] + i1*dst_stride[1] + i2*dst_stride[2]
 * of that GPU's buffer dst_ptrs[i_{peer_dim}] (device pointers valid on this GPU, e.g. from symmetric memory; the
 * entry of this rank is its own buffer).  The caller orders the exchange: every rank's copy must have finished
 * before any rank reads its buffer (a barrier or a tiny all-reduce on the same stream does), and a buffer must
 * not be rewritten while a peer still reads it.  The kernel only stores to peers; it never loads from them. */
typedef struct TriScatterDesc {
  int64_t dims[3];
  int64_t dst_stride[3];   /* in runs */
  int64_t dst_base_run;
  int64_t run_bytes;       /* multiple of 16 */
  int32_t peer_dim;        /* which of the three indices selects the destination GPU */
  int32_t n_peers;         /* = dims[peer_dim], at most 16 */
} TriScatterDesc;

int tri_scatter_runs(const TriScatterDesc* d, const void* src, void* const* dst_ptrs, tri_stream_t stream);

/* The same exchange issued to the copy engines instead of a kernel: one strided two-dimensional device-to-device
 * copy per (destination GPU, index of the shorter of the two other dimensions), each moving dims[longer] runs.  It
 * occupies no SM, so the step's other kernels keep the whole GPU while the slabs cross NVLink; the copies of one call
 * run one after the other, which costs more latency than the kernel once there are many destinations (measured on
 * B200: better than the kernel at 2 GPUs, worse at 8).  Same contract as
 * tri_scatter_runs (ordering by the caller; capturable into a CUDA graph as copy nodes).  Returns
 * TRI_ERR_UNSUPPORTED when a pitch exceeds what a two-dimensional copy takes (2 GiB); use the kernel then. */
int tri_scatter_runs_dma(const TriScatterDesc* d, const void* src, void* const* dst_ptrs, tri_stream_t stream);
/* Arrival flags for the peer-store exchange, in place of a collective as the barrier after tri_scatter_runs.
 * No counterpart in the reference (single device).  Every rank owns an array of 16 uint32 arrival flags in memory
 * that all peers can store to (symmetric memory), zeroed before first use; flag_ptrs[w] is rank w's array as mapped
 * on this GPU.  `state` is 4 uint32 in this GPU's own memory, zero-initialised once: state[0] counts the barriers this
 * rank has entered, state[3] is the status of the last wait.
 * tri_peer_barrier queues a one-block kernel that (1) stores this rank's barrier number into slot `rank` of every
 * peer's flag array (release at system scope: whatever this rank queued on the stream before it, e.g. the copy kernel
 * of tri_scatter_runs, has completed and is visible), then (2) waits until all n_peers slots of this rank's own array
 * have reached that number; kernels queued behind it then read the exchanged data.  The wait is BOUNDED: after
 * limit_cycles SM clocks (<= 0: about five seconds) it gives up, stores 100 + the missing peer in state[3] and returns,
 * so a missing rank becomes an error the host can read, never a hung GPU.  The barrier number advances on the
 * device, so a captured CUDA graph replays without changed arguments.  Every rank must enter the same barriers in
 * the same order.  A receive buffer may be rewritten by a later exchange once this rank has passed a barrier of a
 * LATER exchange with the same peers: their copy kernel for that one is ordered, on their stream, behind whatever
 * read the earlier data. */
typedef struct TriPeerSignal {
  void* const* flag_ptrs;  /* [n_peers] */
  uint32_t* state;         /* 4 words, this GPU */
  int32_t rank, n_peers;
} TriPeerSignal;

int tri_peer_barrier(const TriPeerSignal* sig, int64_t limit_cycles, tri_stream_t stream);

/* The tensor-core kernels bound every wait; if one runs out, the kernel records a code in the first
 * word of the workspace it was given and drains instead of hanging.  This call copies that word back
 * (it synchronises the stream) and returns it: 0 = no failure. */
int tri_ws_status(const void* ws, tri_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TRI_B200_H_ */
