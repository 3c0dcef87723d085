// Tensor-core attention path: dispatch predicate and host drivers (trimul lives in tc_trimul.cu).
#include "tc_paths.cuh"

#include <cstdlib>

namespace tri {
namespace tc {

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

}  // namespace tc
}  // namespace tri
