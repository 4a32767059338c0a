// Split-KV decode attention for callers that must not allocate device memory.
//
// The ordinary entry points take the split-KV workspace (partial_o / partial_l / partial_m)
// from the caller.  Some callers have nowhere to get one: a serving loop that fixed its
// memory budget at load time and forbids cudaMalloc afterwards, a plugin running inside a
// host engine that owns every allocation, code running where an allocation would stall the
// device.  This entry point keeps the workspace in a fixed array that is part of the
// library image instead.  It calls no cudaMalloc, no cudaFree and no allocating library
// routine; it reuses the existing decode and combine kernels unchanged.
#include "common.cuh"

namespace g4b {

// Capacity: one workspace row per (split, slot, query head); a row is the un-normalised
// accumulator (256 floats) plus the row sum and the row maximum.  8192 rows = 8.06 MiB,
// held by every GPU that loads the library until the process exits.
constexpr int kStaticRows = 8192;
constexpr int kStaticHeadDim = 256;
constexpr int kStaticRowFloats = kStaticHeadDim + 2;
constexpr int kStaticMaxSplits = 16;

static __device__ __align__(256) float g_decode_scratch[(size_t)kStaticRows * kStaticRowFloats];

// Device address of the array on the CURRENT device.  In host code the array's name is only
// a stand-in for the symbol: the address a kernel can use has to be asked for, per device,
// with that device current.
static float* decode_scratch_on_current_device() {
  constexpr int kMaxDev = 64;
  // Filled without a lock: threads that race on an entry all store the same address, and an
  // aligned pointer store is not torn.
  static float* cache[kMaxDev] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    fail(G4B_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDev) {
    fail(G4B_ERR_CUDA, "device index %d outside 0..%d", dev, kMaxDev - 1);
    return nullptr;
  }
  if (cache[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_decode_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fail(G4B_ERR_CUDA, "cudaGetSymbolAddress(decode scratch) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = ptr;
  }
  return cache[dev];
}

}  // namespace g4b

using namespace g4b;

extern "C" int g4b_attn_decode_static_scratch(const G4bAttnArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(G4B_ERR_BAD_ARG, "args is null");
  G4bAttnArgs a = *args;
  if (a.partial_o.ptr != nullptr || a.partial_l.ptr != nullptr || a.partial_m.ptr != nullptr)
    return fail(G4B_ERR_BAD_ARG, "g4b_attn_decode_static_scratch takes no partial buffers: it uses the library's own");
  if (a.q.ndim != 4 || a.q.shape[2] != 1)
    return fail(G4B_ERR_UNSUPPORTED, "g4b_attn_decode_static_scratch needs q of shape [B,H,1,D]");
  if (a.q.shape[3] != kStaticHeadDim)
    return fail(G4B_ERR_UNSUPPORTED, "g4b_attn_decode_static_scratch is built for head dim %d", kStaticHeadDim);
  const int64_t B = a.q.shape[0], H = a.q.shape[1];
  int splits = a.num_kv_splits;
  if (splits <= 0) {
    // no count asked for: the reference's table, cut down to what the array holds (one split
    // needs no workspace at all), so that large batches are served rather than refused
    splits = g4b_select_kv_splits(a.ctx_window_size, kStaticMaxSplits, a.phase, 1);
    const int64_t fit = B * H > 0 ? kStaticRows / (B * H) : kStaticMaxSplits;
    if (splits > fit) splits = (int)fit;
    if (splits < 1) splits = 1;
  }
  const int64_t rows = (int64_t)splits * B * H;
  if (splits > kStaticMaxSplits || (splits > 1 && rows > kStaticRows))
    return fail(G4B_ERR_TOO_LARGE,
                "static decode workspace too small: %d splits x %lld slots x %lld heads = %lld rows, the fixed "
                "maximum is %d splits and %d rows; pass your own partial buffers to g4b_flash_attention instead",
                splits, (long long)B, (long long)H, (long long)rows, kStaticMaxSplits, kStaticRows);
  a.num_kv_splits = splits;
  if (splits == 1) return g4b_attn_decode(&a, cuda_stream);   // no workspace needed at all
  G4B_STOP_IF_VALIDATE_ONLY();

  float* scratch = decode_scratch_on_current_device();
  if (scratch == nullptr) return G4B_ERR_CUDA;
  // rows laid out [split][slot][head][1][acc(256) | l | m]
  const int64_t rs = kStaticRowFloats;
  G4bTensor po{}, pl{}, pm{};
  po.ptr = scratch; po.ndim = 5; po.dtype = G4B_F32;
  po.shape[0] = splits; po.shape[1] = B; po.shape[2] = H; po.shape[3] = 1; po.shape[4] = kStaticHeadDim;
  po.stride[0] = B * H * rs; po.stride[1] = H * rs; po.stride[2] = rs; po.stride[3] = rs; po.stride[4] = 1;
  pl.ptr = scratch + kStaticHeadDim; pl.ndim = 4; pl.dtype = G4B_F32;
  pl.shape[0] = splits; pl.shape[1] = B; pl.shape[2] = H; pl.shape[3] = 1;
  pl.stride[0] = B * H * rs; pl.stride[1] = H * rs; pl.stride[2] = rs; pl.stride[3] = rs;
  pm = pl;
  pm.ptr = scratch + kStaticHeadDim + 1;
  a.partial_o = po; a.partial_l = pl; a.partial_m = pm;
  int rc = g4b_attn_decode(&a, cuda_stream);
  if (rc) return rc;
  G4bCombineArgs c{};
  c.partial_o = po; c.partial_l = pl; c.partial_m = pm; c.o = a.o;
  c.user_phase = a.user_phase; c.num_splits = splits; c.phase = a.phase;
  return g4b_attn_combine(&c, cuda_stream);
}
