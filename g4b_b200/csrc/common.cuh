// Shared host/device helpers of libg4b_attn.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/g4b_attn.h"

namespace g4b {

// ---------------------------------------------------------------------------------------
// host: error reporting
// ---------------------------------------------------------------------------------------
char* last_error_buffer();  // thread-local, 512 bytes (api.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define G4B_CUDA_CHECK(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return ::g4b::fail(G4B_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));   \
  } while (0)

inline int dtype_size(int dt) {
  switch (dt) {
    case G4B_F32: case G4B_I32: return 4;
    case G4B_F16: case G4B_BF16: return 2;
    case G4B_I64: return 8;
    case G4B_U8: case G4B_FP8_E4M3: return 1;
  }
  return 0;
}

inline bool is_float_dtype(int dt) { return dt == G4B_F32 || dt == G4B_F16 || dt == G4B_BF16; }

// Row-major contiguity of the trailing dims [from, ndim).
inline bool contiguous_from(const G4bTensor& t, int from) {
  int64_t expect = 1;
  for (int i = t.ndim - 1; i >= from; --i) {
    if (t.shape[i] != 1 && t.stride[i] != expect) return false;
    expect *= t.shape[i];
  }
  return true;
}

// True while the calling thread is in validate-only mode: a launcher that has finished its
// argument checks returns G4B_VALIDATED instead of touching the CUDA runtime.
bool validate_only_mode();  // api.cu
#define G4B_STOP_IF_VALIDATE_ONLY() do { if (::g4b::validate_only_mode()) return G4B_VALIDATED; } while (0)

// Device status word: 0, or the code of the first bounded wait that gave up.
int32_t* device_status_ptr();  // address of the __device__ word on the current device (api.cu)

// kernels' launchers (one per .cu file)
int launch_kv_append(const G4bAppendArgs& a, cudaStream_t st);
int launch_advance(const G4bAdvanceArgs& a, cudaStream_t st);
int launch_combine(const G4bCombineArgs& a, cudaStream_t st);
int launch_decode(const G4bAttnArgs& a, int num_splits, cudaStream_t st);            // register-streaming kernel (head dim 256)
bool decode_stream_supports(const G4bAttnArgs& a);                                    // shapes the TMA-fed kernel takes
int launch_decode_stream(const G4bAttnArgs& a, int num_splits, const G4bDecodeStepArgs* step, cudaStream_t st,
                         const G4bTensor* k_scales = nullptr, const G4bTensor* v_scales = nullptr);
int launch_kv_append_fp8(const G4bFp8AppendArgs& a, cudaStream_t st);
int launch_kv_dequant_fp8(const G4bFp8DequantArgs& a, cudaStream_t st);
int launch_prefill(const G4bAttnArgs& a, cudaStream_t st);

// ---------------------------------------------------------------------------------------
// device: scalar conversions
// ---------------------------------------------------------------------------------------
template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  static constexpr int kDtype = G4B_F32;
  __device__ static float to_float(float v) { return v; }
  __device__ static float from_float(float v) { return v; }
};
template <> struct ElemTraits<__half> {
  static constexpr int kDtype = G4B_F16;
  __device__ static float to_float(__half v) { return __half2float(v); }
  __device__ static __half from_float(float v) { return __float2half_rn(v); }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int kDtype = G4B_BF16;
  __device__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// Runs `body` with `T` bound to the C++ type of a float dtype enum.
#define G4B_DISPATCH_FLOAT(DT, T, ...)                                      \
  switch (DT) {                                                             \
    case G4B_F32:  { using T = float;          __VA_ARGS__; break; }        \
    case G4B_F16:  { using T = __half;         __VA_ARGS__; break; }        \
    case G4B_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; }        \
    default: break;                                                         \
  }

}  // namespace g4b
