// Split-KV combine: log-sum-exp merge of per-split partial results.
//
// Replaces _reduce_split_kv_kernel (g4b/kernels/fa2.py:546-631). Every split s holds an
// un-normalised accumulator acc_s, its row sum l_s and its row maximum m_s in log2 units
// (fa2.py:438-472). The merge is
//     m = max_s m_s;  o = (sum_s acc_s * 2^(m_s - m)) / (sum_s l_s * 2^(m_s - m))
// (fa2.py:618-626). Splits that saw no key carry m = -inf, l = 0 and are skipped.
// The same kernel merges partials that NCCL gathered from other GPUs: they are ordinary
// local memory by the time it runs.
#include "common.cuh"

namespace g4b {

struct CombineParams {
  const void* po; const float* pl; const float* pm; void* o;
  const uint8_t* user_phase;
  int64_t po_s[5], pl_s[4], pm_s[4], o_s[4];
  int64_t phase_stride;
  int S, B, H, Tq, D, phase;
  int groups;          // split groups per block (power of two, 1..32); the block covers 1024 / groups elements
};

constexpr int kCombineThreads = 256;
constexpr int kCombineMaxSplits = 1024;   // weights of one row live in shared memory


// 4 consecutive elements of a partial row.  vmode 2: one 16-byte (f32) or 8-byte (16-bit)
// load; 1: two 8-byte loads (f32 rows that start on odd multiples of 8 bytes, as in a packed
// [.., D + 2] buffer); 0: element by element, n_valid of them.
template <typename TP>
__device__ __forceinline__ float4 load4_partial(const TP* src, int vmode, int n_valid) {
  float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vmode == 2) {
    if constexpr (sizeof(TP) == 4) {
      r = *reinterpret_cast<const float4*>(src);
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(src);
      const TP* e = reinterpret_cast<const TP*>(&raw);
      r = make_float4(ElemTraits<TP>::to_float(e[0]), ElemTraits<TP>::to_float(e[1]),
                      ElemTraits<TP>::to_float(e[2]), ElemTraits<TP>::to_float(e[3]));
    }
  } else if (vmode == 1) {
    if constexpr (sizeof(TP) == 4) {
      const float2 a = *reinterpret_cast<const float2*>(src);
      const float2 b = *reinterpret_cast<const float2*>(src + 2);
      r = make_float4(a.x, a.y, b.x, b.y);
    }
  } else {
    if (n_valid > 0) r.x = ElemTraits<TP>::to_float(src[0]);
    if (n_valid > 1) r.y = ElemTraits<TP>::to_float(src[1]);
    if (n_valid > 2) r.z = ElemTraits<TP>::to_float(src[2]);
    if (n_valid > 3) r.w = ElemTraits<TP>::to_float(src[3]);
  }
  return r;
}

// One block per ((b, h, t) row, slice of the head dim).  Phase 1 (every block of the row
// repeats it: 2 S floats): the threads share out the splits, find the row maximum and turn
// every split's (m, l) into a weight 2^(m_s - m) and the row sum.  Phase 2: the block is
// `groups` split groups x (256 / groups) lanes of 4 elements; a thread adds up its
// S / groups splits with independent 16-byte loads, and the groups are summed through shared
// memory.  The launcher takes few groups (whole rows per block) when there are many rows, and
// up to 32 when there are few (one long sequence: 8 rows, 128 or more splits), so that the
// grid still has 8 blocks per row and no thread walks more than a handful of splits.
template <typename TP, typename TO>
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(CombineParams p) {
  __shared__ float s_w[kCombineMaxSplits];
  __shared__ float s_red[kCombineThreads / 32];
  __shared__ float4 s_acc[kCombineThreads];
  // 32-bit index arithmetic: the row count is a grid extent
  const uint32_t row = blockIdx.x, bh = row / (uint32_t)p.Tq;
  const int t = (int)(row - bh * (uint32_t)p.Tq);
  const int b = (int)(bh / (uint32_t)p.H);
  const int h = (int)(bh - (uint32_t)b * (uint32_t)p.H);
  if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // Launched with programmatic stream serialization: the grid may be resident before the
  // kernel that writes the partials has finished; nothing of theirs is read before this wait
  // (which returns at once when the launch before was an ordinary one).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t ml_off = b * p.pm_s[1] + h * p.pm_s[2] + t * p.pm_s[3];
  const int64_t l_off = b * p.pl_s[1] + h * p.pl_s[2] + t * p.pl_s[3];

  // Everything the block needs from memory is asked for first -- the (m, l) pairs of the
  // thread's splits and its first eight accumulator pieces, none of which depends on another --
  // so the block pays one trip to L2 where the two phases used to pay three or four.
  const TP* po = (const TP*)p.po + b * p.po_s[1] + h * p.po_s[2] + t * p.po_s[3];
  TO* o = (TO*)p.o + b * p.o_s[0] + h * p.o_s[1] + t * p.o_s[2];
  const int lanes = kCombineThreads / p.groups;               // threads per split group
  const int grp = tid / lanes;
  const int cols = lanes * 4;                                 // head-dim elements per block
  const int d = blockIdx.y * cols + (tid % lanes) * 4;        // this thread's 4 elements
  const int n_valid = p.D - d;                                // <= 0: past the head dim
  // vector loads need every split's row to start aligned like the first one
  int vmode = 0;
  if (n_valid >= 4) {
    const uintptr_t a0 = (uintptr_t)(po + d);
    if (a0 % (4 * sizeof(TP)) == 0 && p.po_s[0] % 4 == 0) vmode = 2;
    else if (sizeof(TP) == 4 && a0 % 8 == 0 && p.po_s[0] % 2 == 0) vmode = 1;
  }
  constexpr int kMl = kCombineMaxSplits / kCombineThreads;    // (m, l) pairs per thread
  constexpr int kPre = 8;                                     // accumulator pieces requested up front
  float ms[kMl], ls[kMl];
#pragma unroll
  for (int j = 0; j < kMl; ++j) {
    const int s = tid + j * kCombineThreads;
    ms[j] = -INFINITY; ls[j] = 0.f;
    if (s < p.S) { ms[j] = p.pm[s * p.pm_s[0] + ml_off]; ls[j] = p.pl[s * p.pl_s[0] + l_off]; }
  }
  float4 x[kPre];
  if (n_valid > 0) {
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      const int sj = grp + j * p.groups;
      x[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (sj < p.S) x[j] = load4_partial<TP>(po + (int64_t)sj * p.po_s[0] + d, vmode, n_valid);
    }
  }

  // ---- phase 1: weights 2^(m_s - m) and the row sum ----
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMl; ++j) m = fmaxf(m, ms[j]);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) s_red[warp] = m;
  __syncthreads();
  m = s_red[0];
  for (int w = 1; w < kCombineThreads / 32; ++w) m = fmaxf(m, s_red[w]);
  __syncthreads();
  float l = 0.f;
#pragma unroll
  for (int j = 0; j < kMl; ++j) {
    const int s = tid + j * kCombineThreads;
    const float w = (ms[j] == -INFINITY) ? 0.f : exp2f(ms[j] - m);
    if (s < p.S) s_w[s] = w;
    if (w != 0.f) l += ls[j] * w;
  }
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if (lane == 0) s_red[warp] = l;
  __syncthreads();
  l = 0.f;
  for (int w = 0; w < kCombineThreads / 32; ++w) l += s_red[w];
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;

  // ---- phase 2: weighted sum of the accumulators; a partial with weight 0 (a split that saw
  // no key) is loaded like the others and then left out, whatever its accumulator holds ----
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (n_valid > 0) {
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      const int s = grp + j * p.groups;
      const float w = s < p.S ? s_w[s] : 0.f;
      if (w == 0.f) continue;
      acc.x += x[j].x * w; acc.y += x[j].y * w; acc.z += x[j].z * w; acc.w += x[j].w * w;
    }
    for (int s0 = grp + kPre * p.groups; s0 < p.S; s0 += 4 * p.groups) {
      float4 y[4];
      float w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int s = s0 + j * p.groups;
        w[j] = s < p.S ? s_w[s] : 0.f;
        y[j] = load4_partial<TP>(po + (int64_t)min(s, p.S - 1) * p.po_s[0] + d, vmode, n_valid);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (w[j] == 0.f) continue;
        acc.x += y[j].x * w[j]; acc.y += y[j].y * w[j]; acc.z += y[j].z * w[j]; acc.w += y[j].w * w[j];
      }
    }
  }
  s_acc[tid] = acc;
  __syncthreads();
  for (int c = tid; c < cols; c += kCombineThreads) {
    // element c of the block's slice, summed over the groups
    const int c4 = c >> 2, ci = c & 3;
    float sum = 0.f;
    for (int g2 = 0; g2 < p.groups; ++g2) sum += reinterpret_cast<const float*>(&s_acc[g2 * lanes + c4])[ci];
    const int dd = blockIdx.y * cols + c;
    if (dd < p.D) o[dd] = ElemTraits<TO>::from_float(sum * inv_l);
  }
}

int launch_combine(const G4bCombineArgs& a, cudaStream_t st) {
  CombineParams p{};
  p.po = a.partial_o.ptr; p.pl = (const float*)a.partial_l.ptr; p.pm = (const float*)a.partial_m.ptr;
  p.o = a.o.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr;
  p.phase_stride = a.user_phase.stride[0];
  for (int i = 0; i < 5; ++i) p.po_s[i] = a.partial_o.stride[i];
  for (int i = 0; i < 4; ++i) { p.pl_s[i] = a.partial_l.stride[i]; p.pm_s[i] = a.partial_m.stride[i]; p.o_s[i] = a.o.stride[i]; }
  p.S = a.num_splits; p.B = (int)a.o.shape[0]; p.H = (int)a.o.shape[1]; p.Tq = (int)a.o.shape[2];
  p.D = (int)a.o.shape[3]; p.phase = a.phase;
  const int64_t rows = (int64_t)p.B * p.H * p.Tq;
  if (rows == 0) return G4B_OK;
  if (rows > 0x7fffffffLL) return fail(G4B_ERR_UNSUPPORTED, "combine: too many rows");
  if (p.S > kCombineMaxSplits) return fail(G4B_ERR_TOO_LARGE, "combine: at most %d splits", kCombineMaxSplits);
  G4B_STOP_IF_VALIDATE_ONLY();
  // Split groups per block: at least enough that the block's lanes do not reach past the head
  // dim, then more (narrower blocks, more of them) only while the grid is short of a few
  // waves -- every block repeats phase 1 and pays two block-wide reductions.
  int g_min = 1;
  while (g_min < 32 && kCombineThreads / g_min * 4 > p.D) g_min *= 2;
  p.groups = g_min;
  while (p.groups < 32 && p.groups < p.S &&
         rows * ((p.D + kCombineThreads / p.groups * 4 - 1) / (kCombineThreads / p.groups * 4)) < 592)
    p.groups *= 2;
  const int cols = kCombineThreads / p.groups * 4;
  const dim3 grid((unsigned)rows, (unsigned)((p.D + cols - 1) / cols), 1);
  // The merge always follows the kernel that wrote the partials on the same stream: let its
  // blocks be scheduled while that kernel drains (they wait inside before reading anything).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kCombineThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  bool launched = false;
  cudaError_t err = cudaSuccess;
  G4B_DISPATCH_FLOAT(a.partial_o.dtype, TP,
    G4B_DISPATCH_FLOAT(a.o.dtype, TO,
      err = cudaLaunchKernelEx(&cfg, combine_kernel<TP, TO>, p); launched = true));
  if (!launched) return fail(G4B_ERR_BAD_DTYPE, "combine: partial_o/o dtypes must be f32, f16 or bf16");
  G4B_CUDA_CHECK(err);
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

}  // namespace g4b
