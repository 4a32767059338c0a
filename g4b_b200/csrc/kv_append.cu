// KV-cache append and decode-state advance.
//
// Replaces g4b/kernels/add_kv_to_cache.py:83-159 (ring scatter with optional weight-less
// RMS norm and cast on store) and g4b/kernels/advance_decode_state.py:31-63. Adds the paged
// destination (16-token pages addressed through a block table), which the reference does
// not have.
//
// Both kernels are launch-bound at decode sizes (512 rows of 512 B) and pure streaming at
// prefill sizes: one warp per four consecutive tokens of a (slot, kv head), 16-byte accesses.
#include "common.cuh"
#include <type_traits>

namespace g4b {

struct AppendParams {
  const void* x;
  void* cache;
  const void* cache_offsets;
  const float* x_rsos;
  const uint8_t* user_phase;
  const int32_t* block_tables;
  int64_t xs0, xs1, xs2;        // x strides (elements)
  int64_t rs0, rs1, rs2;        // x_rsos strides
  int64_t off_stride, phase_stride;
  int64_t bt_stride0, bt_stride1;
  int B, G, Tq, D;
  int T;                        // ring length (ring mode)
  int page_size, page_shift;    // paged mode
  int num_pages, max_pages;
  int offsets_are_i64;
  int phase;
  float eps;
  int32_t* status;
};

template <typename T> __device__ __forceinline__ float ld_f(const T* p) {
  return ElemTraits<T>::to_float(*p);
}

constexpr int kAppendRows = 4;   // consecutive tokens of one (slot, kv head) per warp

// One warp per block, kAppendRows consecutive tokens of one (slot, kv head) per warp: what
// depends on the warp alone derives from blockIdx (uniform registers, 32-bit arithmetic; the
// host bounds the grid), the ring's modulo is taken once, and the loads of all the rows go out
// before any is converted, so that a lane has up to eight 16-byte loads in flight.
template <typename TX, typename TC, bool kSameBits>
__global__ void __launch_bounds__(32) kv_append_kernel(AppendParams p) {
  const int lane = threadIdx.x;
  const uint32_t groups = (uint32_t)(p.Tq + kAppendRows - 1) / kAppendRows;   // row groups per (slot, head)
  const uint32_t bg = blockIdx.x / groups;
  const int t0 = (int)(blockIdx.x - bg * groups) * kAppendRows;
  const int b = (int)(bg / (uint32_t)p.G), g = (int)(bg - (uint32_t)b * (uint32_t)p.G);
  const int n = min(kAppendRows, p.Tq - t0);

  if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) return;

  int64_t off;
  if (p.offsets_are_i64) off = ((const int64_t*)p.cache_offsets)[b * p.off_stride];
  else off = ((const int32_t*)p.cache_offsets)[b * p.off_stride];
  const int64_t pos0 = off + t0;

  // destination rows; nullptr after recording why not
  TC* dst[kAppendRows];
  if (p.block_tables != nullptr) {
#pragma unroll
    for (int i = 0; i < kAppendRows; ++i) {
      dst[i] = nullptr;
      if (i >= n) continue;
      const int64_t pos = pos0 + i;
      const int64_t pg = pos >> p.page_shift;
      if (pos < 0 || pg >= p.max_pages) {  // refuse to write outside the block table
        if (lane == 0) atomicCAS(p.status, 0, 0x100 | 1);
        continue;
      }
      const int32_t page = p.block_tables[b * p.bt_stride0 + pg * p.bt_stride1];
      if (page < 0 || page >= p.num_pages) {
        if (lane == 0) atomicCAS(p.status, 0, 0x100 | 2);
        continue;
      }
      const int r = (int)(pos & (p.page_size - 1));
      dst[i] = (TC*)p.cache + (((int64_t)page * p.G + g) * p.page_size + r) * p.D;
    }
  } else {
    int64_t r;
    if ((uint64_t)pos0 <= 0x7fffffffull) {
      r = (uint32_t)pos0 % (uint32_t)p.T;        // the usual case, without a 64-bit division
    } else {
      r = pos0 % p.T;
      if (r < 0) r += p.T;
    }
    TC* const slot = (TC*)p.cache + ((int64_t)b * p.G + g) * p.T * p.D;
#pragma unroll
    for (int i = 0; i < kAppendRows; ++i) {
      int64_t ri = r + i;
      if (ri >= p.T) ri -= p.T;                  // Tq <= T, so one wrap at most
      dst[i] = i < n ? slot + ri * p.D : nullptr;
    }
  }
  const TX* const src0 = (const TX*)p.x + b * p.xs0 + g * p.xs1 + (int64_t)t0 * p.xs2;
  const bool norm = p.x_rsos != nullptr;

  if constexpr (kSameBits) {
    // same element type, no norm: move bits untouched
    if (!norm) {
      constexpr int V = 16 / sizeof(TX);
      bool aligned = (p.D % V) == 0 && ((uintptr_t)src0 & 15) == 0 && (p.xs2 % V) == 0;
#pragma unroll
      for (int i = 0; i < kAppendRows; ++i) aligned = aligned && ((uintptr_t)dst[i] & 15) == 0;
      if (aligned) {
        for (int d = lane * V; d < p.D; d += 32 * V) {
          uint4 v[kAppendRows];
#pragma unroll
          for (int i = 0; i < kAppendRows; ++i)
            if (i < n) v[i] = *(const uint4*)(src0 + i * p.xs2 + d);
#pragma unroll
          for (int i = 0; i < kAppendRows; ++i)
            if (dst[i] != nullptr) *(uint4*)(dst[i] + d) = v[i];
        }
      } else {
        for (int i = 0; i < n; ++i)
          if (dst[i] != nullptr)
            for (int d = lane; d < p.D; d += 32) dst[i][d] = (TC)src0[i * p.xs2 + d];
      }
      return;
    }
  }
  float scale[kAppendRows];
#pragma unroll
  for (int i = 0; i < kAppendRows; ++i) {
    scale[i] = 1.0f;
    if (norm && i < n) scale[i] = rsqrtf(p.x_rsos[b * p.rs0 + g * p.rs1 + (t0 + i) * p.rs2] / (float)p.D + p.eps);
  }
  bool vec_ok = (p.D % 8) == 0 && ((uintptr_t)src0 & (8 * sizeof(TX) - 1)) == 0 && (p.xs2 % 8) == 0;
#pragma unroll
  for (int i = 0; i < kAppendRows; ++i) vec_ok = vec_ok && ((uintptr_t)dst[i] & (8 * sizeof(TC) - 1)) == 0;
  if (vec_ok) {
    // 8 elements per lane per pass: 16- or 32-byte loads, 16- or 32-byte stores
    for (int d = lane * 8; d < p.D; d += 256) {
      alignas(32) TX in[kAppendRows][8];
#pragma unroll
      for (int i = 0; i < kAppendRows; ++i) {
        if (i >= n) continue;
        const TX* src = src0 + i * p.xs2 + d;
        *(uint4*)&in[i][0] = *(const uint4*)src;
        if constexpr (sizeof(TX) == 4) *(uint4*)&in[i][4] = *(const uint4*)(src + 4);
      }
#pragma unroll
      for (int i = 0; i < kAppendRows; ++i) {
        if (dst[i] == nullptr) continue;
        alignas(32) TC out[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float v = ElemTraits<TX>::to_float(in[i][e]);
          if (norm) v *= scale[i];
          out[e] = ElemTraits<TC>::from_float(v);
        }
        *(uint4*)(dst[i] + d) = *(const uint4*)&out[0];
        if constexpr (sizeof(TC) == 4) *(uint4*)(dst[i] + d + 4) = *(const uint4*)&out[4];
      }
    }
    return;
  }
  for (int i = 0; i < n; ++i) {
    if (dst[i] == nullptr) continue;
    for (int d = lane; d < p.D; d += 32) {
      float v = ld_f(src0 + i * p.xs2 + d);
      if (norm) v *= scale[i];
      dst[i][d] = ElemTraits<TC>::from_float(v);
    }
  }
}

template <typename TX, typename TC>
static int launch_typed(const AppendParams& p, cudaStream_t st) {
  const int64_t groups = (p.Tq + kAppendRows - 1) / kAppendRows;
  const int64_t blocks = (int64_t)p.B * p.G * groups;
  if (blocks == 0) return G4B_OK;
  if (blocks > 0x7fffffffLL) return fail(G4B_ERR_UNSUPPORTED, "kv_append: too many rows");
  constexpr bool same = std::is_same<TX, TC>::value;
  kv_append_kernel<TX, TC, same><<<(unsigned)blocks, 32, 0, st>>>(p);
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

int launch_kv_append(const G4bAppendArgs& a, cudaStream_t st) {
  AppendParams p{};
  p.x = a.x.ptr; p.cache = a.cache.ptr; p.cache_offsets = a.cache_offsets.ptr;
  p.x_rsos = (const float*)a.x_rsos.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr;
  p.block_tables = (const int32_t*)a.block_tables.ptr;
  p.xs0 = a.x.stride[0]; p.xs1 = a.x.stride[1]; p.xs2 = a.x.stride[2];
  p.rs0 = a.x_rsos.stride[0]; p.rs1 = a.x_rsos.stride[1]; p.rs2 = a.x_rsos.stride[2];
  p.off_stride = a.cache_offsets.stride[0];
  p.phase_stride = a.user_phase.stride[0];
  p.bt_stride0 = a.block_tables.stride[0]; p.bt_stride1 = a.block_tables.stride[1];
  p.B = (int)a.x.shape[0]; p.G = (int)a.x.shape[1]; p.Tq = (int)a.x.shape[2]; p.D = (int)a.x.shape[3];
  p.offsets_are_i64 = a.cache_offsets.dtype == G4B_I64;
  p.phase = a.phase; p.eps = a.rmsnorm_eps;
  G4B_STOP_IF_VALIDATE_ONLY();
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;
  if (p.block_tables != nullptr) {
    p.page_size = a.page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < a.page_size) ++p.page_shift;
    p.num_pages = (int)a.cache.shape[0];
    p.max_pages = (int)a.block_tables.shape[1];
    p.T = 0;
  } else {
    p.T = (int)a.cache.shape[2];
  }
  int rc = G4B_ERR_BAD_DTYPE;
  G4B_DISPATCH_FLOAT(a.x.dtype, TX,
    G4B_DISPATCH_FLOAT(a.cache.dtype, TC, rc = launch_typed<TX, TC>(p, st)));
  if (rc == G4B_ERR_BAD_DTYPE) return fail(rc, "kv_append: x/cache dtypes must be f32, f16 or bf16");
  return rc;
}

// ---------------------------------------------------------------------------------------
// append into an e4m3 pool with one scale per (page, kv head)
// ---------------------------------------------------------------------------------------
struct Fp8AppendParams {
  const void* x; uint8_t* cache; float* scales; const void* cache_offsets; const float* x_rsos;
  const uint8_t* user_phase; const int32_t* block_tables;
  int64_t xs0, xs1, xs2, rs0, rs1, rs2, ss0, ss1, off_stride, phase_stride, bt_s0, bt_s1;
  int B, G, Tq, D, page_shift, num_pages, max_pages, phase, x_dtype;
  bool offsets_are_i64;
  float eps, headroom;
  int32_t* status;
};

__device__ __forceinline__ float ld_any(const void* base, int64_t i, int dt) {
  if (dt == G4B_F32) return ((const float*)base)[i];
  if (dt == G4B_F16) return __half2float(((const __half*)base)[i]);
  return __bfloat162float(((const __nv_bfloat16*)base)[i]);
}

// One warp per (slot, kv head, token).  The page's scale comes from the page's first row: from
// x when that row is part of this call (every row of the page then computes the same value;
// the first row's warp stores it), else from the scale tensor.
__global__ void __launch_bounds__(32) kv_append_fp8_kernel(Fp8AppendParams p) {
  const int lane = threadIdx.x;
  const uint32_t idx = blockIdx.x;
  const int t = (int)(idx % (uint32_t)p.Tq);
  const int g = (int)((idx / (uint32_t)p.Tq) % (uint32_t)p.G);
  const int b = (int)(idx / ((uint32_t)p.Tq * (uint32_t)p.G));
  if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) return;
  const int64_t off = p.offsets_are_i64 ? ((const int64_t*)p.cache_offsets)[b * p.off_stride]
                                        : (int64_t)((const int32_t*)p.cache_offsets)[b * p.off_stride];
  const int64_t pos = off + t;
  const int page_size = 1 << p.page_shift;
  const int64_t pg = pos >> p.page_shift;
  const int row = (int)(pos & (page_size - 1));
  int page = pg < p.max_pages ? p.block_tables[b * p.bt_s0 + pg * p.bt_s1] : -1;
  if (page < 0 || page >= p.num_pages) {     // never follow a bad table entry
    if (lane == 0) atomicCAS(p.status, 0, 0x100 | 3);
    return;
  }
  auto row_scale = [&](int tt) -> float {    // V norm factor of token tt
    if (p.x_rsos == nullptr) return 1.f;
    return rsqrtf(p.x_rsos[b * p.rs0 + g * p.rs1 + tt * p.rs2] / (float)p.D + p.eps);
  };
  const int64_t xrow = b * p.xs0 + g * p.xs1;
  const int t0 = t - row;                    // token that is the page's first row (may lie before this call)
  float scale;
  if (t0 >= 0) {
    const float r0 = row_scale(t0);
    float amax = 0.f;
    for (int d = lane; d < p.D; d += 32) amax = fmaxf(amax, fabsf(ld_any(p.x, xrow + t0 * p.xs2 + d, p.x_dtype) * r0));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    scale = fmaxf(amax * p.headroom / 448.f, 5.9604644775390625e-8f);
    if (row == 0 && lane == 0) p.scales[page * p.ss0 + g * p.ss1] = scale;
  } else {
    scale = p.scales[page * p.ss0 + g * p.ss1];
  }
  const float r = row_scale(t);
  uint8_t* dst = p.cache + ((((int64_t)page * p.G + g) << p.page_shift) + row) * p.D;
  for (int d = 2 * lane; d < p.D; d += 64) {
    const float a = ld_any(p.x, xrow + t * p.xs2 + d, p.x_dtype) * r / scale;
    const float c = d + 1 < p.D ? ld_any(p.x, xrow + t * p.xs2 + d + 1, p.x_dtype) * r / scale : 0.f;
    uint16_t two;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(two) : "f"(c), "f"(a));   // high byte <- first source
    dst[d] = (uint8_t)(two & 0xff);
    if (d + 1 < p.D) dst[d + 1] = (uint8_t)(two >> 8);
  }
}

int launch_kv_append_fp8(const G4bFp8AppendArgs& a, cudaStream_t st) {
  Fp8AppendParams p{};
  p.x = a.x.ptr; p.cache = (uint8_t*)a.cache.ptr; p.scales = (float*)a.scales.ptr;
  p.cache_offsets = a.cache_offsets.ptr; p.x_rsos = (const float*)a.x_rsos.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr; p.block_tables = (const int32_t*)a.block_tables.ptr;
  p.xs0 = a.x.stride[0]; p.xs1 = a.x.stride[1]; p.xs2 = a.x.stride[2];
  p.rs0 = a.x_rsos.stride[0]; p.rs1 = a.x_rsos.stride[1]; p.rs2 = a.x_rsos.stride[2];
  p.ss0 = a.scales.stride[0]; p.ss1 = a.scales.stride[1];
  p.off_stride = a.cache_offsets.stride[0]; p.phase_stride = a.user_phase.stride[0];
  p.bt_s0 = a.block_tables.stride[0]; p.bt_s1 = a.block_tables.stride[1];
  p.B = (int)a.x.shape[0]; p.G = (int)a.x.shape[1]; p.Tq = (int)a.x.shape[2]; p.D = (int)a.x.shape[3];
  while ((1 << p.page_shift) < a.page_size) ++p.page_shift;
  p.num_pages = (int)a.cache.shape[0]; p.max_pages = (int)a.block_tables.shape[1];
  p.phase = a.phase; p.x_dtype = a.x.dtype;
  p.offsets_are_i64 = a.cache_offsets.dtype == G4B_I64;
  p.eps = a.rmsnorm_eps; p.headroom = a.headroom;
  const int64_t blocks = (int64_t)p.B * p.G * p.Tq;
  if (blocks == 0) return G4B_OK;
  if (blocks > 0x7fffffffLL) return fail(G4B_ERR_UNSUPPORTED, "kv_append_fp8: too many rows");
  G4B_STOP_IF_VALIDATE_ONLY();
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;
  kv_append_fp8_kernel<<<(unsigned)blocks, 32, 0, st>>>(p);
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

// ---------------------------------------------------------------------------------------
// 8-bit pool -> 16-bit pool (for prefill chunks over an 8-bit cache)
// ---------------------------------------------------------------------------------------
struct Fp8DequantParams {
  const uint8_t* cache; const float* scales; void* out;
  const int32_t* block_tables; const int32_t* time_dim_sizes; const uint8_t* user_phase;
  int64_t ss0, ss1, bt_s0, bt_s1, time_stride, phase_stride;
  int G, num_pages, max_pages, page_shift, phase;
  int64_t run_bytes;          // page_size x D: bytes of one (page, kv head) run of the 8-bit pool
  int32_t* status;
};

// One block per (page, kv head) run: with block tables the grid is (max_pages * G, B) and a
// block finds its page in the table (or leaves: past the slot's length, slot off phase, bad
// entry); without them it is (num_pages * G, 1).  A thread turns 16 bytes into 16 values:
// e4m3 -> f16 is exact, the product with the scale is taken in f32 and rounded once.
template <typename T>
__global__ void __launch_bounds__(256) kv_dequant_fp8_kernel(Fp8DequantParams p) {
  const int g = (int)(blockIdx.x % (uint32_t)p.G);
  int page = (int)(blockIdx.x / (uint32_t)p.G);
  if (p.block_tables != nullptr) {
    const int b = blockIdx.y, pg = page;
    if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) return;
    const int time = p.time_dim_sizes[b * p.time_stride];
    if (((int64_t)pg << p.page_shift) >= time) return;
    page = p.block_tables[b * p.bt_s0 + pg * p.bt_s1];
    if (page < 0 || page >= p.num_pages) {     // never follow a bad table entry
      if (threadIdx.x == 0) atomicCAS(p.status, 0, 0x100 | 3);
      return;
    }
  }
  const float scale = p.scales[page * p.ss0 + g * p.ss1];
  const int64_t run = ((int64_t)page * p.G + g) * p.run_bytes;
  const uint8_t* src = p.cache + run;
  T* dst = (T*)p.out + run;
  for (int64_t i = 16 * (int64_t)threadIdx.x; i < p.run_bytes; i += 16 * 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t two;
        const uint16_t pair = (uint16_t)(h ? (w[j] >> 16) : (w[j] & 0xffffu));
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(two) : "h"(pair));
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&two));
        if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) {
          const __half2 r = __floats2half2_rn(f.x * scale, f.y * scale);
          o[2 * j + h] = *reinterpret_cast<const uint32_t*>(&r);
        } else {
          const __nv_bfloat162 r = __floats2bfloat162_rn(f.x * scale, f.y * scale);
          o[2 * j + h] = *reinterpret_cast<const uint32_t*>(&r);
        }
      }
    }
    *reinterpret_cast<uint4*>(dst + i) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(dst + i + 8) = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

int launch_kv_dequant_fp8(const G4bFp8DequantArgs& a, cudaStream_t st) {
  Fp8DequantParams p{};
  p.cache = (const uint8_t*)a.cache.ptr; p.scales = (const float*)a.scales.ptr; p.out = a.out.ptr;
  p.block_tables = (const int32_t*)a.block_tables.ptr; p.time_dim_sizes = (const int32_t*)a.time_dim_sizes.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr;
  p.ss0 = a.scales.stride[0]; p.ss1 = a.scales.stride[1];
  p.bt_s0 = a.block_tables.stride[0]; p.bt_s1 = a.block_tables.stride[1];
  p.time_stride = a.time_dim_sizes.stride[0]; p.phase_stride = a.user_phase.stride[0];
  p.G = (int)a.cache.shape[1]; p.num_pages = (int)a.cache.shape[0];
  p.max_pages = p.block_tables != nullptr ? (int)a.block_tables.shape[1] : 0;
  while ((1 << p.page_shift) < a.page_size) ++p.page_shift;
  p.phase = a.phase;
  p.run_bytes = a.cache.shape[2] * a.cache.shape[3];
  const int64_t B = p.block_tables != nullptr ? a.block_tables.shape[0] : 1;
  const int64_t runs = (p.block_tables != nullptr ? (int64_t)p.max_pages : (int64_t)p.num_pages) * p.G;
  if (runs == 0 || B == 0) return G4B_OK;
  if (runs > 0x7fffffffLL || B > 65535) return fail(G4B_ERR_TOO_LARGE, "dequant: too many pages or slots for one launch");
  G4B_STOP_IF_VALIDATE_ONLY();
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;
  const dim3 grid((unsigned)runs, (unsigned)B, 1);
  if (a.out.dtype == G4B_F16) kv_dequant_fp8_kernel<__half><<<grid, 256, 0, st>>>(p);
  else kv_dequant_fp8_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

// ---------------------------------------------------------------------------------------
// advance_decode_state
// ---------------------------------------------------------------------------------------
__global__ void advance_kernel(int32_t* in_tok, const int32_t* out_tok, int32_t* cache_offsets,
                               int32_t* time_dim_sizes, const uint8_t* user_phase, int B,
                               int64_t in_s1, int64_t out_s0, int64_t off_s, int64_t time_s,
                               int64_t phase_s) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (user_phase[b * phase_s] != (uint8_t)G4B_PHASE_DECODE) return;
  in_tok[b * in_s1] = out_tok[b * out_s0];
  cache_offsets[b * off_s] += 1;
  time_dim_sizes[b * time_s] += 1;
}

int launch_advance(const G4bAdvanceArgs& a, cudaStream_t st) {
  const int B = (int)a.input_token_ids.shape[1];
  if (B == 0) return G4B_OK;
  G4B_STOP_IF_VALIDATE_ONLY();
  advance_kernel<<<(B + 255) / 256, 256, 0, st>>>(
      (int32_t*)a.input_token_ids.ptr, (const int32_t*)a.out_token_ids.ptr,
      (int32_t*)a.cache_offsets.ptr, (int32_t*)a.time_dim_sizes.ptr,
      (const uint8_t*)a.user_phase.ptr, B, a.input_token_ids.stride[1], a.out_token_ids.stride[0],
      a.cache_offsets.stride[0], a.time_dim_sizes.stride[0], a.user_phase.stride[0]);
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

}  // namespace g4b
