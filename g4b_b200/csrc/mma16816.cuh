// Warp-level m16n8k16 tensor instructions (f16 / bf16 operands, f32 accumulate) and the small
// conversions around them, shared by the Tq == 1 kernels.
#pragma once

#include "common.cuh"

namespace g4b {

template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
  static constexpr bool kSplitP = true;
  __device__ static __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
  // sum of the two rounded values a packed register holds
  __device__ static __forceinline__ float sum2(uint32_t v) {
    return __uint_as_float(v << 16) + __uint_as_float(v & 0xffff0000u);
  }
};
template <> struct Mma<__half> {
  static constexpr bool kSplitP = false;
  __device__ static __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
  __device__ static __forceinline__ float sum2(uint32_t v) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    return f.x + f.y;
  }
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ float load_as_float(const void* base, int64_t i, int dt) {
  if (dt == G4B_F32) return ((const float*)base)[i];
  if (dt == G4B_F16) return __half2float(((const __half*)base)[i]);
  return __bfloat162float(((const __nv_bfloat16*)base)[i]);
}

__device__ __forceinline__ void store_from_float(void* base, int64_t i, int dt, float v) {
  if (dt == G4B_F32) ((float*)base)[i] = v;
  else if (dt == G4B_F16) ((__half*)base)[i] = __float2half_rn(v);
  else ((__nv_bfloat16*)base)[i] = __float2bfloat16_rn(v);
}

}  // namespace g4b
