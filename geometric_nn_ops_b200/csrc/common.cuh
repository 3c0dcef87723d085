// Shared helpers for every translation unit of libtri_b200.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/tri_b200.h"

namespace tri {

// ---- thread-local status ---------------------------------------------------
char* last_error_buf();            // 512 bytes, thread local
void set_path(const char* name);   // "simt" / "tcgen05"
void count_launch(int n = 1);

// Optional per-kernel timing: when enabled (tri_profile_enable), every launch site is bracketed by a
// pair of CUDA events on the launching stream; tri_profile_summary sums them per kernel name.
// `flops` and `bytes` are the ALGORITHMIC work of the launch (not measured traffic).
struct KernelTimer {
  int slot;
  cudaStream_t st;
  KernelTimer(const char* name, cudaStream_t stream, double flops = 0.0, double bytes = 0.0);
  ~KernelTimer();
};

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define TRI_CUDA_OK(expr)                                                          \
  do {                                                                             \
    cudaError_t e_ = (expr);                                                       \
    if (e_ != cudaSuccess)                                                         \
      return ::tri::fail((int)e_, "%s failed: %s (%s:%d)", #expr,                  \
                         cudaGetErrorString(e_), __FILE__, __LINE__);              \
  } while (0)

#define TRI_LAUNCH_OK()                                                            \
  do {                                                                             \
    ::tri::count_launch();                                                         \
    cudaError_t e_ = cudaGetLastError();                                           \
    if (e_ != cudaSuccess)                                                         \
      return ::tri::fail((int)e_, "kernel launch failed: %s (%s:%d)",              \
                         cudaGetErrorString(e_), __FILE__, __LINE__);              \
  } while (0)

#define TRI_TRY(expr)                                                              \
  do {                                                                             \
    int r_ = (expr);                                                               \
    if (r_ != 0) return r_;                                                        \
  } while (0)

// ---- element types -----------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Round an fp32 value to the tf32 grid (10 explicit mantissa bits, round to nearest).
__device__ __forceinline__ float round_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

__device__ __forceinline__ float sigmoidf_acc(float v) { return 1.0f / (1.0f + expf(-v)); }

// Multiprocessors of the CURRENT device.  Cached per device: one process may drive several GPUs (one thread each,
// or autograd's backward thread), so neither this nor any launch attribute may be remembered process-wide.
int sm_count();

inline size_t dtype_size(int dtype) { return dtype == TRI_F32 ? 4 : 2; }
inline size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }
inline int cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }

// Bump allocator over a caller-provided workspace.
struct Arena {
  char* base;
  size_t cap, off;
  Arena(void* p, size_t bytes) : base((char*)p), cap(bytes), off(0) {}
  template <typename T> T* take(size_t n) {
    size_t bytes = align_up(n * sizeof(T));
    T* r = (T*)(base + off);
    off += bytes;
    return r;
  }
  bool ok() const { return off <= cap; }
};

}  // namespace tri
