// C ABI of libg4b_attn.so: argument validation, dispatch, status handling.
//
// Mirrors the host wrappers of the reference: flash_attention (g4b/kernels/fa2.py:634-715),
// add_kv_to_cache (g4b/kernels/add_kv_to_cache.py:162-186) and advance_decode_state
// (g4b/kernels/advance_decode_state.py:66-80).  What the reference checks with Triton
// static_asserts at compile time (fa2.py:289-320, add_kv_to_cache.py:113-128) is checked
// here per call and reported as an error code.
#include "common.cuh"

namespace g4b {

static thread_local char tls_error[512] = {0};
char* last_error_buffer() { return tls_error; }

// Validate-only mode of the calling thread (g4b_set_validate_only): launchers stop after
// their argument checks, before the first CUDA call, and return G4B_VALIDATED.
static thread_local bool tls_validate_only = false;
bool validate_only_mode() { return tls_validate_only; }

// One status word per device, in static device memory (nothing is allocated).
__device__ int32_t g_device_status = 0;

int32_t* device_status_ptr() {
  constexpr int kMaxDev = 64;
  // Filled without a lock: two threads that race on an entry both store the same address, and
  // an aligned pointer store is not torn.
  static int32_t* cache[kMaxDev] = {nullptr};
  int dev = 0;
  const cudaError_t ge = cudaGetDevice(&dev);
  if (ge != cudaSuccess) {
    fail(G4B_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(ge));
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDev) {
    fail(G4B_ERR_CUDA, "device index %d outside 0..%d", dev, kMaxDev - 1);
    return nullptr;
  }
  if (cache[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_device_status);
    if (e != cudaSuccess) {
      fail(G4B_ERR_CUDA, "cudaGetSymbolAddress(status) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = (int32_t*)ptr;
  }
  return cache[dev];
}

static int check_tensor(const G4bTensor& t, const char* name, int ndim, bool inner_unit) {
  if (t.ptr == nullptr) return fail(G4B_ERR_BAD_ARG, "%s: null pointer", name);
  if (t.ndim != ndim) return fail(G4B_ERR_BAD_ARG, "%s: expected rank %d, got %d", name, ndim, t.ndim);
  for (int i = 0; i < ndim; ++i)
    if (t.shape[i] < 0) return fail(G4B_ERR_BAD_ARG, "%s: negative extent", name);
  if (inner_unit && t.shape[ndim - 1] > 1 && t.stride[ndim - 1] != 1)
    return fail(G4B_ERR_BAD_STRIDE, "%s: innermost stride must be 1", name);
  return G4B_OK;
}

static bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// Shape rules shared by prefill and decode (fa2.py:289-320).
static int validate_attn(const G4bAttnArgs& a, bool need_partials, int splits, bool tq1 = false) {
  int rc;
  if ((rc = check_tensor(a.q, "q", 4, true))) return rc;
  if ((rc = check_tensor(a.o, "o", 4, true))) return rc;
  if ((rc = check_tensor(a.k_cache, "k_cache", 4, true))) return rc;
  if ((rc = check_tensor(a.v_cache, "v_cache", 4, true))) return rc;
  if ((rc = check_tensor(a.time_dim_sizes, "time_dim_sizes", 1, false))) return rc;
  if (a.time_dim_sizes.dtype != G4B_I32) return fail(G4B_ERR_BAD_DTYPE, "time_dim_sizes must be int32");
  const int64_t B = a.q.shape[0], H = a.q.shape[1], Tq = a.q.shape[2], D = a.q.shape[3];
  for (int i = 0; i < 4; ++i)
    if (a.o.shape[i] != a.q.shape[i]) return fail(G4B_ERR_BAD_ARG, "o shape must equal q shape");
  if (a.time_dim_sizes.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "time_dim_sizes must have B entries");
  if (a.user_phase.ptr != nullptr) {
    if ((rc = check_tensor(a.user_phase, "user_phase", 1, false))) return rc;
    if (a.user_phase.dtype != G4B_U8) return fail(G4B_ERR_BAD_DTYPE, "user_phase must be uint8");
    if (a.user_phase.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "user_phase must have B entries");
  }
  if (!is_float_dtype(a.q.dtype) || !is_float_dtype(a.o.dtype))
    return fail(G4B_ERR_BAD_DTYPE, "q/o must be f32, f16 or bf16");
  if (a.k_cache.dtype != a.v_cache.dtype || (a.k_cache.dtype != G4B_F16 && a.k_cache.dtype != G4B_BF16))
    return fail(G4B_ERR_BAD_DTYPE, "k_cache/v_cache must both be f16 or both bf16");
  for (int i = 0; i < 4; ++i)
    if (a.k_cache.shape[i] != a.v_cache.shape[i]) return fail(G4B_ERR_BAD_ARG, "k_cache/v_cache shapes differ");
  if (!contiguous_from(a.k_cache, 0) || !contiguous_from(a.v_cache, 0))
    return fail(G4B_ERR_BAD_STRIDE, "k_cache/v_cache must be contiguous");
  if (a.k_cache.shape[3] != D) return fail(G4B_ERR_BAD_ARG, "head dim of q and cache differ");
  const int64_t G = a.k_cache.shape[1];
  if (G <= 0 || H % G != 0) return fail(G4B_ERR_BAD_ARG, "query heads must be a multiple of kv heads");
  if (D != 256 && D != 128 && !(tq1 && D == 512))
    return fail(G4B_ERR_UNSUPPORTED, "head dim %lld not supported (Tq == 1: 128, 256, 512; Tq > 1: 128, 256)", (long long)D);
  if ((((uintptr_t)a.k_cache.ptr) | ((uintptr_t)a.v_cache.ptr)) & 15)
    return fail(G4B_ERR_BAD_STRIDE, "k_cache/v_cache must be 16-byte aligned");
  if (a.stage != G4B_STAGE_CAUSAL && a.stage != G4B_STAGE_FULL)
    return fail(G4B_ERR_BAD_ARG, "stage must be STAGE_FULL (1) or STAGE_CAUSAL (3)");
  if (a.sliding_window < 0) return fail(G4B_ERR_BAD_ARG, "sliding_window must be >= 0");
  if (a.ctx_window_size <= 0) return fail(G4B_ERR_BAD_ARG, "ctx_window_size must be positive");
  if (a.block_tables.ptr != nullptr) {
    if ((rc = check_tensor(a.block_tables, "block_tables", 2, false))) return rc;
    if (a.block_tables.dtype != G4B_I32) return fail(G4B_ERR_BAD_DTYPE, "block_tables must be int32");
    if (a.block_tables.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "block_tables must have B rows");
    if (!is_pow2(a.page_size) || a.page_size < 16)
      return fail(G4B_ERR_BAD_ARG, "page_size must be a power of two >= 16");
    if (a.k_cache.shape[2] != a.page_size) return fail(G4B_ERR_BAD_ARG, "pool dim 2 must equal page_size");
    if ((int64_t)a.ctx_window_size > a.block_tables.shape[1] * (int64_t)a.page_size)
      return fail(G4B_ERR_BAD_ARG, "ctx_window_size exceeds block table capacity");
  } else {
    if (a.k_cache.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "ring cache must have B slots");
    if (a.ctx_window_size > a.k_cache.shape[2])  // fa2.py:298
      return fail(G4B_ERR_BAD_ARG, "ctx_window_size exceeds cache length");
  }
  if (need_partials) {
    if (a.partial_o.ptr == nullptr || a.partial_l.ptr == nullptr || a.partial_m.ptr == nullptr)
      return fail(G4B_ERR_BAD_ARG, "partial_o, partial_l, and partial_m must be provided together");
    if ((rc = check_tensor(a.partial_o, "partial_o", 5, true))) return rc;
    if ((rc = check_tensor(a.partial_l, "partial_l", 4, false))) return rc;
    if ((rc = check_tensor(a.partial_m, "partial_m", 4, false))) return rc;
    if (!is_float_dtype(a.partial_o.dtype)) return fail(G4B_ERR_BAD_DTYPE, "partial_o must be f32, f16 or bf16");
    if (a.partial_l.dtype != G4B_F32 || a.partial_m.dtype != G4B_F32)
      return fail(G4B_ERR_BAD_DTYPE, "partial_l/partial_m must be f32");
    if (a.partial_o.shape[0] < splits || a.partial_l.shape[0] < splits || a.partial_m.shape[0] < splits)
      return fail(G4B_ERR_BAD_ARG, "partial buffers hold fewer than %d splits", splits);  // fa2.py:299-311
    for (int i = 0; i < 4; ++i)
      if (a.partial_o.shape[i + 1] != a.o.shape[i]) return fail(G4B_ERR_BAD_ARG, "partial_o shape must be [S,B,H,Tq,D]");
    for (int i = 0; i < 3; ++i)
      if (a.partial_l.shape[i + 1] != a.o.shape[i] || a.partial_m.shape[i + 1] != a.o.shape[i])
        return fail(G4B_ERR_BAD_ARG, "partial_l/partial_m shape must be [S,B,H,Tq]");
  }
  (void)Tq;
  return G4B_OK;
}

static int max_partial_splits(const G4bAttnArgs& a) {
  if (a.partial_o.ptr == nullptr || a.partial_l.ptr == nullptr || a.partial_m.ptr == nullptr) return 1;
  int64_t s = a.partial_o.shape[0];
  if (a.partial_l.shape[0] < s) s = a.partial_l.shape[0];
  if (a.partial_m.shape[0] < s) s = a.partial_m.shape[0];
  return (int)(s < 1 ? 1 : s);
}

static int resolve_splits(const G4bAttnArgs& a) {
  const int max_splits = max_partial_splits(a);
  if (a.num_kv_splits > 0) return a.num_kv_splits < max_splits ? a.num_kv_splits : max_splits;
  int s = g4b_select_kv_splits(a.ctx_window_size, max_splits, a.phase, (int)a.q.shape[2]);
  // The reference's table only looks at the context length (fa2.py:201-212).  A decode CTA is
  // one (slot, kv head, split) and this GPU holds 2 x 148 of them: with few slots the table
  // leaves most SMs idle (8 slots x 4 kv heads at 4096 keys: 32 CTAs).  Where the caller's
  // workspace has room, split further, down to 256 keys per split.  Static in the shapes, like
  // the reference's choice, so the launch geometry stays capturable.
  if (a.q.shape[2] == 1 && s < max_splits && a.q.ndim == 4 && a.k_cache.ndim == 4) {
    const int64_t units = a.q.shape[0] * a.k_cache.shape[1];
    if (units > 0 && units * s < 296) {
      int64_t want = (296 + units - 1) / units;
      const int64_t by_len = a.ctx_window_size / 256;
      if (want > by_len) want = by_len;
      if (want > max_splits) want = max_splits;
      if (want > s) s = (int)want;
    }
  }
  return s;
}

}  // namespace g4b

using namespace g4b;

extern "C" {

int g4b_abi_version(void) { return G4B_ABI_VERSION; }

void g4b_set_validate_only(int on) { tls_validate_only = on != 0; }

const char* g4b_last_error_string(void) { return last_error_buffer(); }

int g4b_select_kv_splits(int ctx_window_size, int max_kv_splits, int phase, int tq) {
  // _prune_invalid_configs, fa2.py:201-212
  if (phase != G4B_PHASE_DECODE || tq != 1) return 1;
  int target;
  if (max_kv_splits <= 1 || ctx_window_size <= 4096) target = 1;
  else if (ctx_window_size < 8192) target = 4;
  else if (ctx_window_size < 32768) target = 8;
  else target = 16;
  return target < max_kv_splits ? target : (max_kv_splits < 1 ? 1 : max_kv_splits);
}

int g4b_attn_decode(const G4bAttnArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  const G4bAttnArgs& a = *args;
  const int splits = a.num_kv_splits > 0 ? a.num_kv_splits : 1;
  const bool tq1 = a.q.ndim == 4 && a.q.shape[2] == 1;
  int rc = validate_attn(a, splits > 1, splits, tq1);
  if (rc) return rc;
  if (a.q.shape[2] != 1) return fail(G4B_ERR_UNSUPPORTED, "decode kernel needs Tq == 1");
  if (a.q.shape[1] / a.k_cache.shape[1] > 8)
    return fail(G4B_ERR_UNSUPPORTED, "decode kernel supports at most 8 query heads per kv head");
  if (decode_stream_supports(a)) return launch_decode_stream(a, splits, nullptr, (cudaStream_t)cuda_stream);
  if (a.q.shape[3] != 256) return fail(G4B_ERR_UNSUPPORTED, "decode: ring caches shorter than 16 rows need head dim 256");
  return launch_decode(a, splits, (cudaStream_t)cuda_stream);
}

int g4b_decode_step(const G4bDecodeStepArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  G4bAttnArgs a = args->attn;
  if (a.q.ndim != 4 || a.q.shape[2] != 1) return fail(G4B_ERR_UNSUPPORTED, "decode step needs q of shape [B,H,1,D]");
  if (a.k_cache.ndim != 4) return fail(G4B_ERR_BAD_ARG, "k_cache: expected rank 4");
  const int splits = resolve_splits(a);
  a.num_kv_splits = splits;
  int rc = validate_attn(a, true, splits, true);
  if (rc) return rc;
  if (a.q.shape[1] / a.k_cache.shape[1] > 8)
    return fail(G4B_ERR_UNSUPPORTED, "decode step supports at most 8 query heads per kv head");
  if (!decode_stream_supports(a))
    return fail(G4B_ERR_UNSUPPORTED, "decode step needs pages or a ring of at least 16 rows");
  G4bDecodeStepArgs s = *args;
  s.attn = a;
  rc = launch_decode_stream(a, splits, &s, (cudaStream_t)cuda_stream);
  // without peers the splits are merged by a second launch, scheduled while the first drains
  if (rc != G4B_OK || s.world > 1 || (s.world == 1 && s.state != nullptr) || splits == 1) return rc;
  G4bCombineArgs c{};
  c.partial_o = a.partial_o; c.partial_l = a.partial_l; c.partial_m = a.partial_m; c.o = a.o;
  c.user_phase = a.user_phase; c.num_splits = splits; c.phase = a.phase;
  return g4b_attn_combine(&c, cuda_stream);
}

int g4b_attn_prefill(const G4bAttnArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  int rc = validate_attn(*args, false, 1);
  if (rc) return rc;
  return launch_prefill(*args, (cudaStream_t)cuda_stream);
}

int g4b_attn_combine(const G4bCombineArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  const G4bCombineArgs& a = *args;
  int rc;
  if ((rc = check_tensor(a.partial_o, "partial_o", 5, true))) return rc;
  if ((rc = check_tensor(a.partial_l, "partial_l", 4, false))) return rc;
  if ((rc = check_tensor(a.partial_m, "partial_m", 4, false))) return rc;
  if ((rc = check_tensor(a.o, "o", 4, true))) return rc;
  if (a.partial_l.dtype != G4B_F32 || a.partial_m.dtype != G4B_F32)
    return fail(G4B_ERR_BAD_DTYPE, "partial_l/partial_m must be f32");
  if (a.num_splits < 1 || a.num_splits > a.partial_o.shape[0] || a.num_splits > a.partial_l.shape[0] ||
      a.num_splits > a.partial_m.shape[0])
    return fail(G4B_ERR_BAD_ARG, "num_splits out of range of the partial buffers");
  for (int i = 0; i < 4; ++i)
    if (a.partial_o.shape[i + 1] != a.o.shape[i]) return fail(G4B_ERR_BAD_ARG, "partial_o shape must be [S,B,H,Tq,D]");
  for (int i = 0; i < 3; ++i)
    if (a.partial_l.shape[i + 1] != a.o.shape[i] || a.partial_m.shape[i + 1] != a.o.shape[i])
      return fail(G4B_ERR_BAD_ARG, "partial_l/partial_m shape must be [S,B,H,Tq]");
  if (a.user_phase.ptr != nullptr) {
    if ((rc = check_tensor(a.user_phase, "user_phase", 1, false))) return rc;
    if (a.user_phase.dtype != G4B_U8 || a.user_phase.shape[0] != a.o.shape[0])
      return fail(G4B_ERR_BAD_ARG, "user_phase must be uint8 [B]");
  }
  return launch_combine(a, (cudaStream_t)cuda_stream);
}

int g4b_flash_attention(const G4bAttnArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  G4bAttnArgs a = *args;
  // the partial triple must be complete or absent (fa2.py:656-657)
  const int given = (a.partial_o.ptr != nullptr) + (a.partial_l.ptr != nullptr) + (a.partial_m.ptr != nullptr);
  if (given != 0 && given != 3)
    return fail(G4B_ERR_BAD_ARG, "partial_o, partial_l, and partial_m must be provided together");
  if (a.q.ndim != 4) return fail(G4B_ERR_BAD_ARG, "q: expected rank 4");
  const bool decode_path = a.q.shape[2] == 1 && a.q.shape[1] / (a.k_cache.shape[1] > 0 ? a.k_cache.shape[1] : 1) <= 8;
  if (!decode_path) return g4b_attn_prefill(&a, cuda_stream);
  const int splits = resolve_splits(a);
  a.num_kv_splits = splits;
  int rc = g4b_attn_decode(&a, cuda_stream);
  if (rc || splits == 1) return rc;
  G4bCombineArgs c{};
  c.partial_o = a.partial_o; c.partial_l = a.partial_l; c.partial_m = a.partial_m; c.o = a.o;
  c.user_phase = a.user_phase; c.num_splits = splits; c.phase = a.phase;
  return g4b_attn_combine(&c, cuda_stream);
}

int g4b_kv_append(const G4bAppendArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  const G4bAppendArgs& a = *args;
  int rc;
  if ((rc = check_tensor(a.x, "x", 4, true))) return rc;
  if ((rc = check_tensor(a.cache, "cache", 4, true))) return rc;
  if ((rc = check_tensor(a.cache_offsets, "cache_offsets", 1, false))) return rc;
  if (a.cache_offsets.dtype != G4B_I32 && a.cache_offsets.dtype != G4B_I64)
    return fail(G4B_ERR_BAD_DTYPE, "cache_offsets must be int32 or int64");
  if (!is_float_dtype(a.x.dtype) || !is_float_dtype(a.cache.dtype))
    return fail(G4B_ERR_BAD_DTYPE, "x/cache must be f32, f16 or bf16");
  const int64_t B = a.x.shape[0], G = a.x.shape[1], Tq = a.x.shape[2], D = a.x.shape[3];
  if (a.cache_offsets.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "cache_offsets must have B entries");
  if (!contiguous_from(a.cache, 0)) return fail(G4B_ERR_BAD_STRIDE, "cache must be contiguous");
  if (a.cache.shape[1] != G || a.cache.shape[3] != D)
    return fail(G4B_ERR_BAD_ARG, "x and cache disagree on kv heads or head dim");  // add_kv_to_cache.py:113-115
  if (a.block_tables.ptr != nullptr) {
    if ((rc = check_tensor(a.block_tables, "block_tables", 2, false))) return rc;
    if (a.block_tables.dtype != G4B_I32) return fail(G4B_ERR_BAD_DTYPE, "block_tables must be int32");
    if (a.block_tables.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "block_tables must have B rows");
    if (!is_pow2(a.page_size)) return fail(G4B_ERR_BAD_ARG, "page_size must be a power of two");
    if (a.cache.shape[2] != a.page_size) return fail(G4B_ERR_BAD_ARG, "pool dim 2 must equal page_size");
  } else {
    if (a.cache.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "ring cache must have B slots");
    if (Tq > a.cache.shape[2])  // add_kv_to_cache.py:123
      return fail(G4B_ERR_BAD_ARG, "more new tokens than cache rows");
  }
  if (a.x_rsos.ptr != nullptr) {
    if ((rc = check_tensor(a.x_rsos, "x_rsos", 3, false))) return rc;
    if (a.x_rsos.dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "x_rsos must be f32");
    if (a.x_rsos.shape[0] != B || a.x_rsos.shape[1] != G || a.x_rsos.shape[2] != Tq)
      return fail(G4B_ERR_BAD_ARG, "x_rsos shape must be [B,G,Tq]");
  }
  if (a.user_phase.ptr != nullptr) {
    if ((rc = check_tensor(a.user_phase, "user_phase", 1, false))) return rc;
    if (a.user_phase.dtype != G4B_U8 || a.user_phase.shape[0] != B)
      return fail(G4B_ERR_BAD_ARG, "user_phase must be uint8 [B]");
  }
  return launch_kv_append(a, (cudaStream_t)cuda_stream);
}

static bool is_byte_dtype(int dt) { return dt == G4B_U8 || dt == G4B_FP8_E4M3; }

int g4b_kv_append_fp8(const G4bFp8AppendArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  const G4bFp8AppendArgs& a = *args;
  int rc;
  if ((rc = check_tensor(a.x, "x", 4, true))) return rc;
  if ((rc = check_tensor(a.cache, "cache", 4, true))) return rc;
  if ((rc = check_tensor(a.scales, "scales", 2, false))) return rc;
  if ((rc = check_tensor(a.cache_offsets, "cache_offsets", 1, false))) return rc;
  if ((rc = check_tensor(a.block_tables, "block_tables", 2, false))) return rc;
  if (!is_float_dtype(a.x.dtype)) return fail(G4B_ERR_BAD_DTYPE, "x must be f32, f16 or bf16");
  if (!is_byte_dtype(a.cache.dtype)) return fail(G4B_ERR_BAD_DTYPE, "cache must hold one byte per element (e4m3)");
  if (a.scales.dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "scales must be f32");
  if (a.cache_offsets.dtype != G4B_I32 && a.cache_offsets.dtype != G4B_I64)
    return fail(G4B_ERR_BAD_DTYPE, "cache_offsets must be int32 or int64");
  if (a.block_tables.dtype != G4B_I32) return fail(G4B_ERR_BAD_DTYPE, "block_tables must be int32");
  const int64_t B = a.x.shape[0], G = a.x.shape[1], Tq = a.x.shape[2], D = a.x.shape[3];
  if (a.cache_offsets.shape[0] != B || a.block_tables.shape[0] != B)
    return fail(G4B_ERR_BAD_ARG, "cache_offsets and block_tables must have B entries / rows");
  if (!contiguous_from(a.cache, 0)) return fail(G4B_ERR_BAD_STRIDE, "cache must be contiguous");
  if (a.cache.shape[1] != G || a.cache.shape[3] != D) return fail(G4B_ERR_BAD_ARG, "x and cache disagree on kv heads or head dim");
  if (!is_pow2(a.page_size) || a.cache.shape[2] != a.page_size) return fail(G4B_ERR_BAD_ARG, "pool dim 2 must equal page_size, a power of two");
  if (a.scales.shape[0] != a.cache.shape[0] || a.scales.shape[1] != G) return fail(G4B_ERR_BAD_ARG, "scales must be [num_pages, G]");
  if (!(a.headroom >= 1.f)) return fail(G4B_ERR_BAD_ARG, "headroom must be >= 1");
  if (a.x_rsos.ptr != nullptr) {
    if ((rc = check_tensor(a.x_rsos, "x_rsos", 3, false))) return rc;
    if (a.x_rsos.dtype != G4B_F32 || a.x_rsos.shape[0] != B || a.x_rsos.shape[1] != G || a.x_rsos.shape[2] != Tq)
      return fail(G4B_ERR_BAD_ARG, "x_rsos must be f32 [B,G,Tq]");
  }
  if (a.user_phase.ptr != nullptr) {
    if ((rc = check_tensor(a.user_phase, "user_phase", 1, false))) return rc;
    if (a.user_phase.dtype != G4B_U8 || a.user_phase.shape[0] != B) return fail(G4B_ERR_BAD_ARG, "user_phase must be uint8 [B]");
  }
  return launch_kv_append_fp8(a, (cudaStream_t)cuda_stream);
}

int g4b_kv_dequant_fp8(const G4bFp8DequantArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  const G4bFp8DequantArgs& a = *args;
  int rc;
  if ((rc = check_tensor(a.cache, "cache", 4, true))) return rc;
  if ((rc = check_tensor(a.scales, "scales", 2, false))) return rc;
  if ((rc = check_tensor(a.out, "out", 4, true))) return rc;
  if (!is_byte_dtype(a.cache.dtype)) return fail(G4B_ERR_BAD_DTYPE, "cache must hold one byte per element (e4m3)");
  if (a.scales.dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "scales must be f32");
  if (a.out.dtype != G4B_F16 && a.out.dtype != G4B_BF16) return fail(G4B_ERR_BAD_DTYPE, "out must be f16 or bf16");
  if (!contiguous_from(a.cache, 0) || !contiguous_from(a.out, 0)) return fail(G4B_ERR_BAD_STRIDE, "cache and out must be contiguous");
  for (int i = 0; i < 4; ++i)
    if (a.cache.shape[i] != a.out.shape[i]) return fail(G4B_ERR_BAD_ARG, "out must have the shape of cache");
  if (!is_pow2(a.page_size) || a.cache.shape[2] != a.page_size) return fail(G4B_ERR_BAD_ARG, "pool dim 2 must equal page_size, a power of two");
  if ((a.cache.shape[2] * a.cache.shape[3]) % 16 != 0) return fail(G4B_ERR_BAD_ARG, "page_size x D must be a multiple of 16");
  if ((((uintptr_t)a.cache.ptr) & 15) || (((uintptr_t)a.out.ptr) & 15)) return fail(G4B_ERR_BAD_STRIDE, "cache and out must be 16-byte aligned");
  if (a.scales.shape[0] != a.cache.shape[0] || a.scales.shape[1] != a.cache.shape[1]) return fail(G4B_ERR_BAD_ARG, "scales must be [num_pages, G]");
  if (a.block_tables.ptr != nullptr) {
    if ((rc = check_tensor(a.block_tables, "block_tables", 2, false))) return rc;
    if (a.block_tables.dtype != G4B_I32) return fail(G4B_ERR_BAD_DTYPE, "block_tables must be int32");
    if (a.time_dim_sizes.ptr == nullptr) return fail(G4B_ERR_BAD_ARG, "block_tables needs time_dim_sizes");
    if ((rc = check_tensor(a.time_dim_sizes, "time_dim_sizes", 1, false))) return rc;
    if (a.time_dim_sizes.dtype != G4B_I32 || a.time_dim_sizes.shape[0] != a.block_tables.shape[0])
      return fail(G4B_ERR_BAD_ARG, "time_dim_sizes must be int32 [B]");
    if (a.user_phase.ptr != nullptr) {
      if ((rc = check_tensor(a.user_phase, "user_phase", 1, false))) return rc;
      if (a.user_phase.dtype != G4B_U8 || a.user_phase.shape[0] != a.block_tables.shape[0]) return fail(G4B_ERR_BAD_ARG, "user_phase must be uint8 [B]");
    }
  } else if (a.time_dim_sizes.ptr != nullptr || a.user_phase.ptr != nullptr) {
    return fail(G4B_ERR_BAD_ARG, "time_dim_sizes and user_phase are only read with block_tables");
  }
  return launch_kv_dequant_fp8(a, (cudaStream_t)cuda_stream);
}

int g4b_flash_attention_fp8(const G4bAttnArgs* args, const G4bTensor* k_scales, const G4bTensor* v_scales,
                            void* cuda_stream) {
  if (args == nullptr || k_scales == nullptr || v_scales == nullptr) return fail(G4B_ERR_BAD_ARG, "args or scales null");
  G4bAttnArgs a = *args;
  const int given = (a.partial_o.ptr != nullptr) + (a.partial_l.ptr != nullptr) + (a.partial_m.ptr != nullptr);
  if (given != 0 && given != 3) return fail(G4B_ERR_BAD_ARG, "partial_o, partial_l, and partial_m must be provided together");
  if (a.q.ndim != 4 || a.q.shape[2] != 1) return fail(G4B_ERR_UNSUPPORTED, "e4m3 caches: Tq == 1 only");
  if (a.k_cache.ndim != 4 || a.v_cache.ndim != 4) return fail(G4B_ERR_BAD_ARG, "k_cache / v_cache: expected rank 4");
  if (!is_byte_dtype(a.k_cache.dtype) || !is_byte_dtype(a.v_cache.dtype))
    return fail(G4B_ERR_BAD_DTYPE, "e4m3 caches must hold one byte per element");
  if (a.block_tables.ptr == nullptr) return fail(G4B_ERR_UNSUPPORTED, "e4m3 caches: paged only");
  // the shape rules are those of the 16-bit path: check them on a copy that claims f16 caches
  G4bAttnArgs chk = a;
  chk.k_cache.dtype = chk.v_cache.dtype = G4B_F16;
  const int splits = resolve_splits(a);
  a.num_kv_splits = chk.num_kv_splits = splits;
  int rc = validate_attn(chk, splits > 1, splits, true);
  if (rc) return rc;
  if (a.q.shape[1] / a.k_cache.shape[1] > 8) return fail(G4B_ERR_UNSUPPORTED, "at most 8 query heads per kv head");
  const G4bTensor* sc[2] = {k_scales, v_scales};
  for (const G4bTensor* t : sc) {
    if (t->ptr == nullptr || t->ndim != 2 || t->dtype != G4B_F32 || t->shape[0] != a.k_cache.shape[0] || t->shape[1] != a.k_cache.shape[1])
      return fail(G4B_ERR_BAD_ARG, "k_scales / v_scales must be f32 [num_pages, G]");
  }
  rc = launch_decode_stream(a, splits, nullptr, (cudaStream_t)cuda_stream, k_scales, v_scales);
  if (rc || splits == 1) return rc;
  G4bCombineArgs c{};
  c.partial_o = a.partial_o; c.partial_l = a.partial_l; c.partial_m = a.partial_m; c.o = a.o;
  c.user_phase = a.user_phase; c.num_splits = splits; c.phase = a.phase;
  return g4b_attn_combine(&c, cuda_stream);
}

int g4b_advance_decode_state(const G4bAdvanceArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  const G4bAdvanceArgs& a = *args;
  int rc;
  if ((rc = check_tensor(a.input_token_ids, "input_token_ids", 2, false))) return rc;
  if ((rc = check_tensor(a.out_token_ids, "out_token_ids", 2, false))) return rc;
  if ((rc = check_tensor(a.cache_offsets, "cache_offsets", 1, false))) return rc;
  if ((rc = check_tensor(a.time_dim_sizes, "time_dim_sizes", 1, false))) return rc;
  if ((rc = check_tensor(a.user_phase, "user_phase", 1, false))) return rc;
  if (a.input_token_ids.dtype != G4B_I32 || a.out_token_ids.dtype != G4B_I32 ||
      a.cache_offsets.dtype != G4B_I32 || a.time_dim_sizes.dtype != G4B_I32 || a.user_phase.dtype != G4B_U8)
    return fail(G4B_ERR_BAD_DTYPE, "advance_decode_state: int32 vectors and a uint8 phase vector expected");
  const int64_t B = a.input_token_ids.shape[1];
  // advance_decode_state.py:46-51
  if (a.input_token_ids.shape[0] < 1 || a.out_token_ids.shape[1] < 1 || a.out_token_ids.shape[0] != B ||
      a.cache_offsets.shape[0] != B || a.time_dim_sizes.shape[0] != B || a.user_phase.shape[0] != B)
    return fail(G4B_ERR_BAD_ARG, "advance_decode_state: vectors must all have B entries");
  return launch_advance(a, (cudaStream_t)cuda_stream);
}

int g4b_device_status(void* cuda_stream, int32_t* status_out) {
  int32_t* dptr = device_status_ptr();
  if (dptr == nullptr) return G4B_ERR_CUDA;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  int32_t v = 0, zero = 0;
  G4B_CUDA_CHECK(cudaStreamSynchronize(st));
  G4B_CUDA_CHECK(cudaMemcpyAsync(&v, dptr, sizeof(v), cudaMemcpyDeviceToHost, st));
  G4B_CUDA_CHECK(cudaStreamSynchronize(st));
  if (status_out != nullptr) *status_out = v;
  if (v != 0) {
    G4B_CUDA_CHECK(cudaMemcpyAsync(dptr, &zero, sizeof(zero), cudaMemcpyHostToDevice, st));
    G4B_CUDA_CHECK(cudaStreamSynchronize(st));
    return fail(G4B_ERR_DEVICE_WAIT, "a kernel recorded status 0x%x (0x1xx / 0x2xx: bad block-table entry in an append / "
                "decode launch, 0x3xx: a bounded wait of the prefill kernel ran out, 0x4xx: a peer did not show up)", v);
  }
  return G4B_OK;
}

}  // extern "C"
