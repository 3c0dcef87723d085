// Host driver of the tcgen05 GEMM: tensor-map construction and template dispatch.
#include "tc_gemm.cuh"

#include <cstring>

namespace tri {
namespace tc {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

}  // namespace

int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, bool is_f16, const uint64_t dims[3],
                 const uint64_t strides_elems[2], const uint32_t box[3], bool atom_32b) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return fail(TRI_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(TRI_ERR_ARG, "TMA base address must be 16-byte aligned");
  cuuint64_t gdim[3] = {dims[0], dims[1], dims[2]};
  cuuint64_t gstr[2] = {strides_elems[0] * elem_bytes, strides_elems[1] * elem_bytes};
  // a batch of one may carry any stride; give it a legal one
  if (dims[2] == 1) gstr[1] = gstr[0] * dims[1];
  if (dims[1] == 1 && gstr[0] == 0) gstr[0] = dims[0] * elem_bytes;
  if (gstr[0] % 16 != 0 || gstr[1] % 16 != 0) return fail(TRI_ERR_ARG, "TMA strides must be multiples of 16 bytes");
  cuuint32_t bdim[3] = {box[0], box[1], box[2]};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                           : (is_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom_32b ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(TRI_ERR_ARG, "cuTensorMapEncodeTiled failed (%d): dims %llu %llu %llu strides %llu %llu box %u %u %u",
                (int)r, (unsigned long long)gdim[0], (unsigned long long)gdim[1], (unsigned long long)gdim[2],
                (unsigned long long)gstr[0], (unsigned long long)gstr[1], bdim[0], bdim[1], bdim[2]);
  return 0;
}

int make_tmap(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
              const uint64_t* strides_elems, const uint32_t* box, int swizzle_bytes) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return fail(TRI_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");
  if (rank < 2 || rank > 5) return fail(TRI_ERR_ARG, "tensor map rank %d out of range", rank);
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(TRI_ERR_ARG, "TMA base address must be 16-byte aligned");
  const int es = dtype == TRI_F32 ? 4 : 2;
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bdim[5], estr[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bdim[i] = box[i]; estr[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) {
    gstr[i] = strides_elems[i] * es;
    // a dimension of extent one may carry any stride (even zero): give it a legal one
    if (dims[i + 1] == 1 && (gstr[i] == 0 || gstr[i] % 16 != 0)) gstr[i] = (i == 0 ? dims[0] * es : gstr[i - 1] * dims[i]);
    if (gstr[i] % 16 != 0 || gstr[i] == 0)
      return fail(TRI_ERR_ARG, "TMA stride %d is %llu bytes: must be a non-zero multiple of 16", i, (unsigned long long)gstr[i]);
  }
  CUtensorMapDataType dt = dtype == TRI_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : (dtype == TRI_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TRI_ERR_ARG, "cuTensorMapEncodeTiled failed (%d) for a rank-%d map", (int)r, rank);
  return 0;
}

static int operand_map(CUtensorMap* out, const Operand& o, int dtype, int rows_box) {
  const int es = dtype == TRI_F32 ? 4 : 2;
  const uint32_t span = 128 / es;  // elements in 128 bytes
  uint64_t dims[3] = {o.inner, o.outer, o.batch};
  uint64_t str[2] = {o.st_outer, o.st_batch};
  uint32_t box[3];
  if (!o.mn_major) { box[0] = span; box[1] = (uint32_t)rows_box; box[2] = 1; }
  else { box[0] = span; box[1] = span; box[2] = 1; }  // [128-byte chunk of rows] x [one stage of K]
  return make_tmap_3d(out, o.ptr, es, dtype == TRI_F16, dims, str, box, o.mn_major && es == 4);
}

template <typename TIN, typename TOUT, int BN, int EPI>
static int launch_t(cudaStream_t st, const CUtensorMap* maps, const GemmArgs& g, const GemmPlan& p) {
  constexpr int STAGES = BN == 256 ? 4 : 6;
  constexpr size_t smem = 1024 + (size_t)STAGES * (kStageA + BN * 128) + (2 * STAGES + 4) * 8 + 16;
  auto kern = tc_gemm_kernel<TIN, TOUT, BN, EPI, STAGES>;
  // The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute: set it on every launch
  // (a host-side call of about a microsecond) instead of remembering it process-wide.
  TRI_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int total = g.batches * g.tiles_m * g.tiles_n;
  const int grid = std::min(total, sm_count());
  KernelTimer kt(p.name, st, p.flops, p.bytes);
  kern<<<grid, gemm_threads(EPI), smem, st>>>(maps[0], maps[1], maps[2], maps[3], g);
  TRI_LAUNCH_OK();
  return 0;
}

template <typename TIN>
static int launch_in(cudaStream_t st, int epi, int bn, bool out_f32, const CUtensorMap* maps, const GemmArgs& g,
                     const GemmPlan& p) {
  if (epi == EPI_STORE) {
    if (out_f32 || sizeof(TIN) == 4) {
      if (bn == 256) return launch_t<TIN, float, 256, EPI_STORE>(st, maps, g, p);
      return launch_t<TIN, float, 128, EPI_STORE>(st, maps, g, p);
    }
    if (bn == 256) return launch_t<TIN, TIN, 256, EPI_STORE>(st, maps, g, p);
    return launch_t<TIN, TIN, 128, EPI_STORE>(st, maps, g, p);
  }
  if (bn != 256) return fail(TRI_ERR_ARG, "gate epilogues need 256-column tiles");
  if (epi == EPI_GATE_IN) return launch_t<TIN, TIN, 256, EPI_GATE_IN>(st, maps, g, p);
  if (epi == EPI_GATE_OUT) return launch_t<TIN, TIN, 256, EPI_GATE_OUT>(st, maps, g, p);
  if (epi == EPI_GATE_OUT_BWD) return launch_t<TIN, TIN, 256, EPI_GATE_OUT_BWD>(st, maps, g, p);
  if (epi == EPI_GATE_IN_BWD) return launch_t<TIN, TIN, 256, EPI_GATE_IN_BWD>(st, maps, g, p);
  return fail(TRI_ERR_ARG, "unknown epilogue %d", epi);
}

int launch_gemm(cudaStream_t st, int dtype, int epi, int bn, bool out_f32, const GemmPlan& p, int* err) {
  const int es = dtype == TRI_F32 ? 4 : 2;
  const int bke = 128 / es;
  const bool two = p.K1 > 0;
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = p.M; g.N = p.N;
  g.kblocks0 = (p.K0 + bke - 1) / bke;
  g.kblocks1 = two ? (p.K1 + bke - 1) / bke : 0;
  g.seg1_col = p.seg1_col;
  const bool side_by_side = two && p.seg1_col != 0;
  g.bn0 = side_by_side ? 128 : bn;
  g.seg1_n = two ? (side_by_side ? 128 : bn) : 0;
  g.batches = p.batches;
  g.a_tile_batch = p.a_tiles > 0;
  g.tiles_m = p.a_tiles > 0 ? p.a_tiles : (p.M + kBM - 1) / kBM;
  g.tiles_n = side_by_side ? (p.N + 127) / 128 : (p.N + bn - 1) / bn;
  g.split_k = p.split_k;
  const int kind = dtype == TRI_F32 ? KIND_TF32 : (dtype == TRI_BF16 ? KIND_BF16 : KIND_F16);
  for (int s = 0; s < 2; ++s) {
    const int src = (s == 1 && !two) ? 0 : s;
    g.a_mn[s] = p.a[src].mn_major;
    g.b_mn[s] = p.b[src].mn_major;
    g.idesc[s] = make_idesc(kind, kBM, s == 0 ? g.bn0 : (two ? g.seg1_n : g.bn0), p.a[src].mn_major, p.b[src].mn_major);
  }
  g.out0 = p.out0; g.out1 = p.out1; g.ld_out = p.ld_out; g.batch_out = p.batch_out;
  g.bias0 = p.bias0; g.aux = p.aux; g.aux2 = p.aux2; g.aux3 = p.aux3; g.plane = p.plane; g.err = err;
  g.peer_world = 0; g.peer_rank = 0; g.peer_cs = 128; g.peer_batches = 0;
  for (int i = 0; i < 16; ++i) g.peer_out[i] = nullptr;
  if (p.peer_out != nullptr && p.peer_world > 1) {
    if (epi != EPI_GATE_IN || p.peer_world > 16 || 128 % p.peer_world != 0)
      return fail(TRI_ERR_ARG, "peer outputs need the gate-in epilogue and a rank count that divides 128 (at most 16)");
    g.peer_world = p.peer_world; g.peer_rank = p.peer_rank; g.peer_cs = 128 / p.peer_world; g.peer_batches = p.peer_batches;
    for (int i = 0; i < p.peer_world; ++i) {
      if (p.peer_out[i] == nullptr) return fail(TRI_ERR_ARG, "null peer output buffer");
      g.peer_out[i] = p.peer_out[i];
    }
  }

  CUtensorMap maps[4];
  TRI_TRY(operand_map(&maps[0], p.a[0], dtype, kBM));
  TRI_TRY(operand_map(&maps[1], p.b[0], dtype, g.bn0));
  if (two) {
    TRI_TRY(operand_map(&maps[2], p.a[1], dtype, kBM));
    TRI_TRY(operand_map(&maps[3], p.b[1], dtype, g.seg1_n));
  } else {
    maps[2] = maps[0];
    maps[3] = maps[1];
  }
  switch (dtype) {
    case TRI_F32: return launch_in<float>(st, epi, bn, out_f32, maps, g, p);
    case TRI_BF16: return launch_in<__nv_bfloat16>(st, epi, bn, out_f32, maps, g, p);
    case TRI_F16: return launch_in<__half>(st, epi, bn, out_f32, maps, g, p);
  }
  return fail(TRI_ERR_ARG, "bad dtype %d", dtype);
}

}  // namespace tc
}  // namespace tri
