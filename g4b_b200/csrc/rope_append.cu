// Per-head RMS norm + rotary embedding of q and k, V norm, and the KV-cache append, in one
// launch.
//
// Replaces the three launches the reference makes between the q/k/v projections and the
// attention call (g4b/models/gemma4e.py:564-592): apply_rope (g4b/kernels/rope.py:8-39,
// 123-211) and two add_kv_to_cache calls (g4b/kernels/add_kv_to_cache.py:83-159).  The
// reference writes the rotated k back to its scratchpad and reads it again to append it;
// here the row goes from registers to the cache, and q can leave in the 16-bit type the
// prefill kernel wants.
//
// Pure streaming: a one-warp block per (slot, token, head) row at decode sizes, per token with
// all its heads at prefill sizes (the sines and cosines of a token are shared by its heads),
// 16-byte accesses.  A lane holds the elements [4l, 4l+4) and [D/2 + 4l, D/2 + 4l + 4) of the
// row, i.e. complete rotation pairs.  The kernel is bound by instruction issue before HBM, so
// the per-row instruction count is what the structure below is about.
#include "common.cuh"

namespace g4b {
namespace {


struct RopeParams {
  const void* q; const void* k; const void* v;
  void* q_out; void* k_out;
  const float* freqs;
  const void* cache_offsets;
  const float* q_rsos; const float* k_rsos; const float* v_rsos;
  const float* q_w; const float* k_w;
  void* k_cache; void* v_cache;
  const uint8_t* user_phase;
  const int32_t* block_tables;
  int64_t qs[3], ks[3], vs[3], qos[3], kos[3];     // strides (elements) of dims 0..2
  int64_t qrs[3], krs[3], vrs[3];
  int64_t off_stride, phase_stride, bt_s0, bt_s1, freq_stride, qw_stride, kw_stride;
  int in_dtype, q_out_dtype, k_out_dtype, cache_dtype;
  int B, H, G, Tq, D;
  int n_heads;                  // H + G (+ G with v)
  int heads_per_warp;
  uint32_t n_slots;             // warps per token = ceil(n_heads / heads_per_warp)
  uint32_t rows;                // B * Tq
  int T;                        // ring length
  int page_size, page_shift, num_pages, max_pages;
  int offsets_are_i64, phase, norm_qk, norm_v;
  int q_untouched;              // no norm, no rotation, no q_out: q rows are left alone
  float eps;
  float inv_d;                  // 1 / D when D is a power of two, else 0
  int32_t* status;
};

__device__ __forceinline__ float4 load4(const void* base, int dtype, int64_t idx) {
  if (dtype == G4B_F32) return *reinterpret_cast<const float4*>((const float*)base + idx);
  const uint2 raw = *reinterpret_cast<const uint2*>((const uint16_t*)base + idx);
  float4 r;
  if (dtype == G4B_F16) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    r = make_float4(a.x, a.y, b.x, b.y);
  } else {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    r = make_float4(a.x, a.y, b.x, b.y);
  }
  return r;
}

__device__ __forceinline__ void store4(void* base, int dtype, int64_t idx, float4 v) {
  if (dtype == G4B_F32) {
    *reinterpret_cast<float4*>((float*)base + idx) = v;
    return;
  }
  uint2 raw;
  if (dtype == G4B_F16) {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
  } else {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
  }
  *reinterpret_cast<uint2*>((uint16_t*)base + idx) = raw;
}

__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 scale4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float dot4(float4 a) { return a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w; }

// Where position `pos` of slot b lands in the caches: row of kv head g = base + g * head_stride.
// Worked out once per warp (the ring's modulo and the block-table look-up do not depend on the
// head).  base < 0 after recording why not, or when the warp appends nothing.
struct CachePos { int64_t base; int64_t head_stride; };

__device__ __forceinline__ CachePos cache_pos(const RopeParams& p, int b, int64_t pos, int lane) {
  CachePos c{-1, 0};
  if (p.block_tables != nullptr) {
    const int64_t pg = pos >> p.page_shift;
    if (pos < 0 || pg >= p.max_pages) {
      if (lane == 0) atomicCAS(p.status, 0, 0x100 | 1);
      return c;
    }
    const int32_t page = p.block_tables[b * p.bt_s0 + pg * p.bt_s1];
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) atomicCAS(p.status, 0, 0x100 | 2);
      return c;
    }
    c.base = (int64_t)page * p.G * p.page_size + (pos & (p.page_size - 1));
    c.head_stride = p.page_size;
    return c;
  }
  int64_t r;
  if ((uint64_t)pos <= 0x7fffffffull) {
    r = (uint32_t)pos % (uint32_t)p.T;          // the usual case, without a 64-bit division
  } else {
    r = pos % p.T;
    if (r < 0) r += p.T;
  }
  c.base = (int64_t)b * p.G * p.T + r;
  c.head_stride = p.T;
  return c;
}

// One tensor's heads of one token (KIND 0 q, 1 k, 2 v, a compile-time constant so that the
// source / destination choices cost nothing at run time), four rows at a time: the loads of
// all four rows go out before anything is computed, so that a lane has eight 16-byte loads
// in flight (one row at a time left HBM at a quarter of its bandwidth).
template <int KIND, int ITERS, bool kExact, int kOut>
__device__ __forceinline__ void rows_of_kind(const RopeParams& p, int h_begin, int h_end, int b, int t, CachePos cpos,
                                             int lane, const float4 (&sn)[ITERS], const float4 (&cs)[ITERS]) {
  constexpr int kBatch = 4;
  // kOut != 0 is the engine's own configuration (see the kernel): which options are on is
  // then known at compile time, and the per-row tests of them disappear.
  constexpr bool kEngine = kOut != 0;
  const int half = p.D >> 1;
  const void* src = KIND == 0 ? p.q : (KIND == 1 ? p.k : p.v);
  const int64_t* ss = KIND == 0 ? p.qs : (KIND == 1 ? p.ks : p.vs);
  const int64_t src_row = b * ss[0] + t * ss[2];
  const int64_t src_hs = ss[1];
  // destinations
  void* cache = KIND == 1 ? p.k_cache : (KIND == 2 ? p.v_cache : nullptr);
  const bool to_cache = (kEngine ? KIND != 0 : cache != nullptr) && cpos.base >= 0;
  void* out = nullptr;
  int64_t out_row = 0, out_hs = 0;
  const int in_dtype = kOut != 0 ? (int)G4B_F32 : p.in_dtype;
  const int cache_dtype = kOut != 0 ? kOut : p.cache_dtype;
  int out_dtype = in_dtype;
  if (kEngine) {
    if (KIND == 0) { out = p.q_out; out_row = b * p.qos[0] + t * p.qos[2]; out_hs = p.qos[1]; }
  } else if (KIND == 0) {
    if (p.q_out != nullptr) { out = p.q_out; out_dtype = p.q_out_dtype; out_row = b * p.qos[0] + t * p.qos[2]; out_hs = p.qos[1]; }
    else if (!p.q_untouched) { out = const_cast<void*>(p.q); out_row = src_row; out_hs = src_hs; }
  } else if (KIND == 1) {
    if (p.k_out != nullptr) { out = p.k_out; out_dtype = p.k_out_dtype; out_row = b * p.kos[0] + t * p.kos[2]; out_hs = p.kos[1]; }
    else if (p.k_cache == nullptr) { out = const_cast<void*>(p.k); out_row = src_row; out_hs = src_hs; }
  }
  const bool has_out = kEngine ? KIND == 0 : out != nullptr;
  if (!has_out && !to_cache) return;     // nothing to write (warp-uniform)
  const bool norm = KIND == 2 ? p.norm_v != 0 : (kEngine || p.norm_qk != 0);
  const float* rsos = kEngine ? nullptr : (KIND == 0 ? p.q_rsos : (KIND == 1 ? p.k_rsos : p.v_rsos));
  const int64_t* rs = KIND == 0 ? p.qrs : (KIND == 1 ? p.krs : p.vrs);
  const float* w = KIND == 0 ? p.q_w : (KIND == 1 ? p.k_w : nullptr);
  const int64_t ws = kEngine ? 1 : (KIND == 0 ? p.qw_stride : p.kw_stride);
  const bool has_w = kEngine ? KIND != 2 : w != nullptr;
  // norm weights of this lane's elements (the same for every head of the tensor)
  float4 w1[ITERS], w2[ITERS];
  if (norm && has_w) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int d1 = it * 128 + lane * 4;
      if (kExact || d1 < half) {
        if (ws == 1) {
          w1[it] = *reinterpret_cast<const float4*>(w + d1);
          w2[it] = *reinterpret_cast<const float4*>(w + d1 + half);
        } else {
          w1[it] = make_float4(w[d1 * ws], w[(d1 + 1) * ws], w[(d1 + 2) * ws], w[(d1 + 3) * ws]);
          w2[it] = make_float4(w[(d1 + half) * ws], w[(d1 + half + 1) * ws], w[(d1 + half + 2) * ws], w[(d1 + half + 3) * ws]);
        }
      }
    }
  }
  const bool rotate = KIND != 2 && (kEngine || p.freqs != nullptr);

  for (int h0 = h_begin; h0 < h_end; h0 += kBatch) {
    float4 x1[kBatch][ITERS], x2[kBatch][ITERS];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      if (h0 + i < h_end) {
        const int64_t so = src_row + (h0 + i) * src_hs;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
          const int d1 = it * 128 + lane * 4;
          if (kExact || d1 < half) {
            x1[i][it] = load4(src, in_dtype, so + d1);
            x2[i][it] = load4(src, in_dtype, so + d1 + half);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int h = h0 + i;
      if (h >= h_end) continue;
      const int64_t crow = to_cache ? cpos.base + h * cpos.head_stride : -1;
      if (norm) {
        float sumsq = 0.f;
        if (!kEngine && rsos != nullptr) {
          sumsq = rsos[b * rs[0] + h * rs[1] + t * rs[2]];
        } else {
#pragma unroll
          for (int it = 0; it < ITERS; ++it)
            if (kExact || it * 128 + lane * 4 < half) sumsq += dot4(x1[i][it]) + dot4(x2[i][it]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
        }
        // a power-of-two D makes the product the same number as the quotient
        const float inv = rsqrtf((p.inv_d != 0.f ? sumsq * p.inv_d : sumsq / (float)p.D) + p.eps);
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
          if (kExact || it * 128 + lane * 4 < half) {
            if (has_w) {
              // x * (inv * w): the reference's grouping (rope.py:33-34)
              x1[i][it] = mul4(x1[i][it], scale4(w1[it], inv));
              x2[i][it] = mul4(x2[i][it], scale4(w2[it], inv));
            } else {
              x1[i][it] = scale4(x1[i][it], inv);
              x2[i][it] = scale4(x2[i][it], inv);
            }
          }
        }
      }
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int d1 = it * 128 + lane * 4;
        if (kExact || d1 < half) {
          float4 y1 = x1[i][it], y2 = x2[i][it];
          if (rotate) {
            const float4 a = x1[i][it], c = x2[i][it], s = sn[it], co = cs[it];
            y1 = make_float4(co.x * a.x - s.x * c.x, co.y * a.y - s.y * c.y, co.z * a.z - s.z * c.z, co.w * a.w - s.w * c.w);
            y2 = make_float4(co.x * c.x + s.x * a.x, co.y * c.y + s.y * a.y, co.z * c.z + s.z * a.z, co.w * c.w + s.w * a.w);
          }
          if (has_out) {
            const int64_t oo = out_row + h * out_hs + d1;
            store4(out, kOut != 0 ? kOut : out_dtype, oo, y1);
            store4(out, kOut != 0 ? kOut : out_dtype, oo + half, y2);
          }
          if (crow >= 0) {
            store4(cache, cache_dtype, crow * p.D + d1, y1);
            store4(cache, cache_dtype, crow * p.D + d1 + half, y2);
          }
        }
      }
    }
  }
}

// ITERS: passes of 32 lanes x 4 pairs over half the head dim (1 up to D = 256, 2 up to 512);
// kExact: D is exactly ITERS * 256, so no lane is ever past the row's end.
// A warp takes heads [h_begin, h_end) of one token out of the token's H + 2G (q heads, then k,
// then v): all of them at prefill sizes, so that the token's sines and cosines are computed
// once; one at decode sizes, for parallelism.  Index arithmetic that runs once per warp is
// 32-bit (the host bounds the warp count): 64-bit divisions cost a subroutine each.
// kOut: 0, or the 16-bit type of q_out and of the caches in the engine's own configuration
// (gemma4e.py:564-592: f32 q/k/v, q and k normed with weights and rotated, v normed without,
// q to q_out, k and v to the caches only, no precomputed sums of squares), so that neither
// loads and stores nor rows carry run-time switches.
template <int ITERS, bool kExact, int kOut>
__global__ void __launch_bounds__(32, ITERS == 1 ? (kOut != 0 ? 32 : 28) : 16) rope_norm_append_kernel(RopeParams p) {
  // One warp per block: everything that depends on the warp alone then derives from blockIdx,
  // which the compiler knows to be uniform (uniform registers and branches, no convergence
  // barriers around the per-head conditions).
  const int lane = threadIdx.x;
  const uint32_t warp = blockIdx.x;
  const uint32_t row = p.n_slots == 1 ? warp : warp / p.n_slots;
  if (row >= p.rows) return;
  const int slot = (int)(warp - row * p.n_slots);
  const int b = (int)(row / (uint32_t)p.Tq), t = (int)(row - (uint32_t)b * (uint32_t)p.Tq);
  const int half = p.D >> 1;

  int64_t off;
  if (p.offsets_are_i64) off = ((const int64_t*)p.cache_offsets)[b * p.off_stride];
  else off = ((const int32_t*)p.cache_offsets)[b * p.off_stride];
  const int64_t pos = off + t;
  const bool in_phase = p.user_phase == nullptr || p.user_phase[b * p.phase_stride] == (uint8_t)p.phase;

  const int h_begin = slot * p.heads_per_warp;
  const int h_end = min(h_begin + p.heads_per_warp, p.n_heads);

  // sines and cosines of this token, for the pairs this lane owns
  float4 sn[ITERS], cs[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int d1 = it * 128 + lane * 4;
    sn[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    cs[it] = make_float4(1.f, 1.f, 1.f, 1.f);
    if (p.freqs != nullptr && h_begin < p.H + p.G && (kExact || d1 < half)) {
      const float fp = (float)pos;
      // theta is the fp32 product, as in the reference (rope.py:171) and its torch oracle
      sincosf(fp * p.freqs[(d1 + 0) * p.freq_stride], &sn[it].x, &cs[it].x);
      sincosf(fp * p.freqs[(d1 + 1) * p.freq_stride], &sn[it].y, &cs[it].y);
      sincosf(fp * p.freqs[(d1 + 2) * p.freq_stride], &sn[it].z, &cs[it].z);
      sincosf(fp * p.freqs[(d1 + 3) * p.freq_stride], &sn[it].w, &cs[it].w);
    }
  }
  // the warp's head range, cut into its q, k and v parts
  const int q0 = min(h_begin, p.H), q1 = min(h_end, p.H);
  const int k0 = min(max(h_begin, p.H), p.H + p.G) - p.H, k1 = min(max(h_end, p.H), p.H + p.G) - p.H;
  const int v0 = max(h_begin, p.H + p.G) - p.H - p.G, v1 = max(h_end, p.H + p.G) - p.H - p.G;
  CachePos cpos{-1, 0};
  if (in_phase && h_end > p.H && (p.k_cache != nullptr || p.v_cache != nullptr)) cpos = cache_pos(p, b, pos, lane);
  if (q1 > q0) rows_of_kind<0, ITERS, kExact, kOut>(p, q0, q1, b, t, cpos, lane, sn, cs);
  if (k1 > k0) rows_of_kind<1, ITERS, kExact, kOut>(p, k0, k1, b, t, cpos, lane, sn, cs);
  if (v1 > v0) rows_of_kind<2, ITERS, kExact, kOut>(p, v0, v1, b, t, cpos, lane, sn, cs);
}

int check_view(const G4bTensor& t, const char* name, int ndim, int64_t d0, int64_t d1, int64_t d2, int64_t d3) {
  if (t.ptr == nullptr) return fail(G4B_ERR_BAD_ARG, "%s: null pointer", name);
  if (t.ndim != ndim) return fail(G4B_ERR_BAD_ARG, "%s: expected rank %d, got %d", name, ndim, t.ndim);
  const int64_t want[4] = {d0, d1, d2, d3};
  for (int i = 0; i < ndim; ++i)
    if (want[i] >= 0 && t.shape[i] != want[i])
      return fail(G4B_ERR_BAD_ARG, "%s: extent %d is %lld, expected %lld", name, i, (long long)t.shape[i], (long long)want[i]);
  return G4B_OK;
}

// A [.,.,.,D] row view the kernel can read or write 16 bytes at a time.
int check_rows(const G4bTensor& t, const char* name) {
  if (!is_float_dtype(t.dtype)) return fail(G4B_ERR_BAD_DTYPE, "%s must be f32, f16 or bf16", name);
  if (t.shape[3] > 1 && t.stride[3] != 1) return fail(G4B_ERR_BAD_STRIDE, "%s: innermost stride must be 1", name);
  if (((uintptr_t)t.ptr & 15) != 0) return fail(G4B_ERR_BAD_STRIDE, "%s: base must be 16-byte aligned", name);
  for (int i = 0; i < 3; ++i)
    if (t.shape[i] > 1 && (t.stride[i] % 4) != 0)
      return fail(G4B_ERR_BAD_STRIDE, "%s: strides must be multiples of 4 elements", name);
  return G4B_OK;
}

void copy3(int64_t* dst, const G4bTensor& t) { dst[0] = t.stride[0]; dst[1] = t.stride[1]; dst[2] = t.stride[2]; }

}  // namespace

int launch_rope_norm_append(const G4bRopeAppendArgs& a, cudaStream_t st) {
  int rc;
  if ((rc = check_view(a.q, "q", 4, -1, -1, -1, -1))) return rc;
  const int64_t B = a.q.shape[0], H = a.q.shape[1], Tq = a.q.shape[2], D = a.q.shape[3];
  if ((rc = check_view(a.k, "k", 4, B, -1, Tq, D))) return rc;
  const int64_t G = a.k.shape[1];
  if ((rc = check_rows(a.q, "q")) || (rc = check_rows(a.k, "k"))) return rc;
  if (a.k.dtype != a.q.dtype) return fail(G4B_ERR_BAD_DTYPE, "q and k must have one dtype");
  if (D % 8 != 0 || D < 8 || D > 512) return fail(G4B_ERR_UNSUPPORTED, "head dim must be a multiple of 8, at most 512");
  const bool has_v = a.v.ptr != nullptr;
  if (has_v) {
    if ((rc = check_view(a.v, "v", 4, B, G, Tq, D)) || (rc = check_rows(a.v, "v"))) return rc;
    if (a.v.dtype != a.q.dtype) return fail(G4B_ERR_BAD_DTYPE, "v must have the dtype of q and k");
    if (a.v_cache.ptr == nullptr) return fail(G4B_ERR_BAD_ARG, "v needs v_cache");
  } else if (a.v_cache.ptr != nullptr) {
    return fail(G4B_ERR_BAD_ARG, "v_cache needs v");
  }
  if (a.q_out.ptr != nullptr && ((rc = check_view(a.q_out, "q_out", 4, B, H, Tq, D)) || (rc = check_rows(a.q_out, "q_out")))) return rc;
  if (a.k_out.ptr != nullptr && ((rc = check_view(a.k_out, "k_out", 4, B, G, Tq, D)) || (rc = check_rows(a.k_out, "k_out")))) return rc;
  if (a.rope_freqs.ptr != nullptr) {
    if ((rc = check_view(a.rope_freqs, "rope_freqs", 1, D / 2, -1, -1, -1))) return rc;   // rope.py:147
    if (a.rope_freqs.dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "rope_freqs must be f32");
  }
  if ((rc = check_view(a.cache_offsets, "cache_offsets", 1, B, -1, -1, -1))) return rc;    // rope.py:148
  if (a.cache_offsets.dtype != G4B_I32 && a.cache_offsets.dtype != G4B_I64)
    return fail(G4B_ERR_BAD_DTYPE, "cache_offsets must be int32 or int64");
  const G4bTensor* rsos[3] = {&a.q_rsos, &a.k_rsos, &a.v_rsos};
  const char* rsos_name[3] = {"q_rsos", "k_rsos", "v_rsos"};
  for (int i = 0; i < 3; ++i) {
    if (rsos[i]->ptr == nullptr) continue;
    if ((rc = check_view(*rsos[i], rsos_name[i], 3, B, i == 0 ? H : G, Tq, -1))) return rc;  // rope.py:152-157
    if (rsos[i]->dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "%s must be f32", rsos_name[i]);
  }
  const G4bTensor* w[2] = {&a.q_norm_w, &a.k_norm_w};
  for (int i = 0; i < 2; ++i) {
    if (w[i]->ptr == nullptr) continue;
    if ((rc = check_view(*w[i], i == 0 ? "q_norm_w" : "k_norm_w", 1, D, -1, -1, -1))) return rc;  // rope.py:158-159
    if (w[i]->dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "norm weights must be f32");
    if (((uintptr_t)w[i]->ptr & 15) != 0) return fail(G4B_ERR_BAD_STRIDE, "norm weights must be 16-byte aligned");
  }
  const bool paged = a.block_tables.ptr != nullptr;
  const G4bTensor* caches[2] = {&a.k_cache, &a.v_cache};
  for (int i = 0; i < 2; ++i) {
    const G4bTensor& c = *caches[i];
    if (c.ptr == nullptr) continue;
    const char* nm = i == 0 ? "k_cache" : "v_cache";
    if ((rc = check_view(c, nm, 4, -1, G, -1, D))) return rc;
    if (!is_float_dtype(c.dtype)) return fail(G4B_ERR_BAD_DTYPE, "%s must be f32, f16 or bf16", nm);
    if (!contiguous_from(c, 0)) return fail(G4B_ERR_BAD_STRIDE, "%s must be contiguous", nm);
    if (((uintptr_t)c.ptr & 15) != 0) return fail(G4B_ERR_BAD_STRIDE, "%s must be 16-byte aligned", nm);
    if (paged) {
      if (c.shape[2] != a.page_size) return fail(G4B_ERR_BAD_ARG, "%s: pool dim 2 must equal page_size", nm);
    } else {
      if (c.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "%s: ring cache must have B slots", nm);
      if (Tq > c.shape[2]) return fail(G4B_ERR_BAD_ARG, "more new tokens than cache rows");   // add_kv_to_cache.py:123
    }
  }
  if (a.k_cache.ptr != nullptr && a.v_cache.ptr != nullptr) {
    if (a.k_cache.dtype != a.v_cache.dtype) return fail(G4B_ERR_BAD_DTYPE, "k_cache and v_cache must have one dtype");
    for (int i = 0; i < 4; ++i)
      if (a.k_cache.shape[i] != a.v_cache.shape[i]) return fail(G4B_ERR_BAD_ARG, "k_cache/v_cache shapes differ");
  }
  if (paged) {
    if ((rc = check_view(a.block_tables, "block_tables", 2, B, -1, -1, -1))) return rc;
    if (a.block_tables.dtype != G4B_I32) return fail(G4B_ERR_BAD_DTYPE, "block_tables must be int32");
    if (a.page_size <= 0 || (a.page_size & (a.page_size - 1)) != 0) return fail(G4B_ERR_BAD_ARG, "page_size must be a power of two");
    if (a.k_cache.ptr == nullptr) return fail(G4B_ERR_BAD_ARG, "block_tables without a cache");
  }
  if (a.user_phase.ptr != nullptr) {
    if ((rc = check_view(a.user_phase, "user_phase", 1, B, -1, -1, -1))) return rc;
    if (a.user_phase.dtype != G4B_U8) return fail(G4B_ERR_BAD_DTYPE, "user_phase must be uint8");
  }

  RopeParams p{};
  p.q = a.q.ptr; p.k = a.k.ptr; p.v = a.v.ptr; p.q_out = a.q_out.ptr; p.k_out = a.k_out.ptr;
  p.freqs = (const float*)a.rope_freqs.ptr; p.freq_stride = a.rope_freqs.stride[0];
  p.cache_offsets = a.cache_offsets.ptr; p.off_stride = a.cache_offsets.stride[0];
  p.offsets_are_i64 = a.cache_offsets.dtype == G4B_I64;
  p.q_rsos = (const float*)a.q_rsos.ptr; p.k_rsos = (const float*)a.k_rsos.ptr; p.v_rsos = (const float*)a.v_rsos.ptr;
  p.q_w = (const float*)a.q_norm_w.ptr; p.k_w = (const float*)a.k_norm_w.ptr;
  p.qw_stride = a.q_norm_w.stride[0]; p.kw_stride = a.k_norm_w.stride[0];
  p.k_cache = a.k_cache.ptr; p.v_cache = a.v_cache.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr; p.phase_stride = a.user_phase.stride[0];
  p.block_tables = (const int32_t*)a.block_tables.ptr;
  p.bt_s0 = a.block_tables.stride[0]; p.bt_s1 = a.block_tables.stride[1];
  copy3(p.qs, a.q); copy3(p.ks, a.k); copy3(p.vs, a.v); copy3(p.qos, a.q_out); copy3(p.kos, a.k_out);
  copy3(p.qrs, a.q_rsos); copy3(p.krs, a.k_rsos); copy3(p.vrs, a.v_rsos);
  p.in_dtype = a.q.dtype; p.q_out_dtype = a.q_out.dtype; p.k_out_dtype = a.k_out.dtype;
  p.cache_dtype = a.k_cache.ptr != nullptr ? a.k_cache.dtype : a.v_cache.dtype;
  p.B = (int)B; p.H = (int)H; p.G = (int)G; p.Tq = (int)Tq; p.D = (int)D;
  p.n_heads = (int)(H + G + (has_v ? G : 0));
  p.phase = a.phase; p.norm_qk = a.norm_qk; p.norm_v = a.norm_v; p.eps = a.rmsnorm_eps;
  p.q_untouched = a.norm_qk == 0 && a.rope_freqs.ptr == nullptr && a.q_out.ptr == nullptr;
  if (paged) {
    p.page_size = a.page_size;
    while ((1 << p.page_shift) < a.page_size) ++p.page_shift;
    p.num_pages = (int)a.k_cache.shape[0];
    p.max_pages = (int)a.block_tables.shape[1];
  } else if (a.k_cache.ptr != nullptr || a.v_cache.ptr != nullptr) {
    p.T = (int)(a.k_cache.ptr != nullptr ? a.k_cache.shape[2] : a.v_cache.shape[2]);
  } else {
    p.T = 1;
  }
  G4B_STOP_IF_VALIDATE_ONLY();
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;

  const int64_t rows = B * Tq;
  if (rows == 0 || p.n_heads == 0) return G4B_OK;
  // Few rows (decode): one head per warp, for parallelism.  Many (prefill): a warp takes all
  // heads of a token, four at a time, and computes the token's sines and cosines once.
  p.heads_per_warp = rows * p.n_heads >= 16384 ? p.n_heads : 1;
  const int64_t n_slots = (p.n_heads + p.heads_per_warp - 1) / p.heads_per_warp;
  const int64_t warps = rows * n_slots;
  const int64_t blocks = warps;
  if (warps > 0x7fffffffLL) return fail(G4B_ERR_UNSUPPORTED, "rope_norm_append: too many rows");
  p.inv_d = (D & (D - 1)) == 0 ? 1.f / (float)D : 0.f;
  p.n_slots = (uint32_t)n_slots;
  p.rows = (uint32_t)rows;
  const bool exact = D == 256 || D == 512;
  // the engine's own configuration gets the variants with everything decided at compile time
  int out16 = 0;
  if (a.q.dtype == G4B_F32 && a.q_out.ptr != nullptr && a.k_out.ptr == nullptr && a.k_cache.ptr != nullptr &&
      (a.q_out.dtype == G4B_F16 || a.q_out.dtype == G4B_BF16) && a.q_out.dtype == p.cache_dtype &&
      a.rope_freqs.ptr != nullptr && a.norm_qk != 0 && a.q_norm_w.ptr != nullptr && a.k_norm_w.ptr != nullptr &&
      p.qw_stride == 1 && p.kw_stride == 1 && a.q_rsos.ptr == nullptr && a.k_rsos.ptr == nullptr &&
      a.v_rsos.ptr == nullptr)
    out16 = a.q_out.dtype;
#define G4B_ROPE_LAUNCH(ITERS_, EXACT_)                                                                   \
  do {                                                                                                    \
    if (out16 == G4B_F16) rope_norm_append_kernel<ITERS_, EXACT_, G4B_F16><<<(unsigned)blocks, 32, 0, st>>>(p);        \
    else if (out16 == G4B_BF16) rope_norm_append_kernel<ITERS_, EXACT_, G4B_BF16><<<(unsigned)blocks, 32, 0, st>>>(p); \
    else rope_norm_append_kernel<ITERS_, EXACT_, 0><<<(unsigned)blocks, 32, 0, st>>>(p);                 \
  } while (0)
  if (D <= 256) {
    if (exact) G4B_ROPE_LAUNCH(1, true); else G4B_ROPE_LAUNCH(1, false);
  } else {
    if (exact) G4B_ROPE_LAUNCH(2, true); else G4B_ROPE_LAUNCH(2, false);
  }
#undef G4B_ROPE_LAUNCH
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

}  // namespace g4b

extern "C" int g4b_rope_norm_append(const G4bRopeAppendArgs* args, void* cuda_stream) {
  if (args == nullptr) return g4b::fail(G4B_ERR_BAD_ARG, "args is null");
  return g4b::launch_rope_norm_append(*args, (cudaStream_t)cuda_stream);
}
