// Tensor-core paths: dispatch predicates and host drivers.
#include "tc_paths.cuh"

#include <cstdlib>

namespace tri {
namespace tc {

static bool forced_simt() {
  const char* e = getenv("TRI_B200_FORCE_SIMT");
  return e != nullptr && e[0] == '1';
}

bool attn_supported(const TriAttnDesc* d) { (void)d; return false; }
size_t attn_ws_bytes(const TriAttnDesc*, int) { return 0; }
int attn_forward(const TriAttnDesc*, const void*, const void*, const void*, const void*, const uint8_t*, void*,
                 float*, void*, size_t, cudaStream_t) {
  return fail(TRI_ERR_UNSUPPORTED, "no tensor-core attention kernel for this problem");
}
int attn_backward(const TriAttnDesc*, const void*, const void*, const void*, const void*, const uint8_t*,
                  const void*, const float*, const void*, void*, void*, void*, float*, void*, size_t, cudaStream_t) {
  return fail(TRI_ERR_UNSUPPORTED, "no tensor-core attention kernel for this problem");
}

bool mul_supported(const TriMulDesc* d) { (void)d; (void)forced_simt; return false; }
size_t mul_saved_bytes(const TriMulDesc*) { return 0; }
size_t mul_ws_bytes(const TriMulDesc*, int) { return 0; }
int mul_forward(const TriMulDesc*, const void*, const void*, const TriMulWeights*, void*, void*, void*, size_t,
                cudaStream_t) {
  return fail(TRI_ERR_UNSUPPORTED, "no tensor-core trimul kernel for this problem");
}
int mul_backward(const TriMulDesc*, const void*, const void*, const TriMulWeights*, const void*, const void*, void*,
                 const TriMulWeightGrads*, void*, size_t, cudaStream_t) {
  return fail(TRI_ERR_UNSUPPORTED, "no tensor-core trimul kernel for this problem");
}

}  // namespace tc
}  // namespace tri
