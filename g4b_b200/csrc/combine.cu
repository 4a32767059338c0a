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
};

constexpr int kCombineThreads = 256;
constexpr int kCombineMaxSplits = 1024;   // weights of one row live in shared memory

// One block per (b, h, t) row.  Phase 1: the threads share out the splits, find the row
// maximum and turn every split's (m, l) into a weight 2^(m_s - m) and the row sum.  Phase 2:
// the block is (split group) x (pair of head-dim elements); each thread accumulates its
// splits with independent loads, and the groups are summed through shared memory.
template <typename TP, typename TO>
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(CombineParams p) {
  __shared__ float s_w[kCombineMaxSplits];
  __shared__ float s_red[kCombineThreads / 32];
  __shared__ float s_acc[kCombineThreads][2];
  int64_t row = blockIdx.x;
  const int t = (int)(row % p.Tq); row /= p.Tq;
  const int h = (int)(row % p.H);
  const int b = (int)(row / p.H);
  if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t ml_off = b * p.pm_s[1] + h * p.pm_s[2] + t * p.pm_s[3];
  const int64_t l_off = b * p.pl_s[1] + h * p.pl_s[2] + t * p.pl_s[3];

  // ---- phase 1 ----
  float m = -INFINITY;
  for (int s = tid; s < p.S; s += kCombineThreads) {
    const float ms = p.pm[s * p.pm_s[0] + ml_off];
    s_w[s] = ms;
    m = fmaxf(m, ms);
  }
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) s_red[warp] = m;
  __syncthreads();
  m = s_red[0];
  for (int w = 1; w < kCombineThreads / 32; ++w) m = fmaxf(m, s_red[w]);
  __syncthreads();
  float l = 0.f;
  for (int s = tid; s < p.S; s += kCombineThreads) {
    const float ms = s_w[s];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    s_w[s] = w;
    if (w != 0.f) l += p.pl[s * p.pl_s[0] + l_off] * w;
  }
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if (lane == 0) s_red[warp] = l;
  __syncthreads();
  l = 0.f;
  for (int w = 0; w < kCombineThreads / 32; ++w) l += s_red[w];
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;

  // ---- phase 2 ----
  const TP* po = (const TP*)p.po + b * p.po_s[1] + h * p.po_s[2] + t * p.po_s[3];
  TO* o = (TO*)p.o + b * p.o_s[0] + h * p.o_s[1] + t * p.o_s[2];
  const int pairs = (p.D + 1) / 2;
  // as many split groups as fit: pairs * groups <= threads (groups >= 1)
  int groups = kCombineThreads / pairs;
  if (groups < 1) groups = 1;
  if (groups > p.S) groups = p.S;
  for (int d0 = 0; d0 < pairs; d0 += kCombineThreads / groups) {
    const int per = kCombineThreads / groups;          // pairs handled per pass
    const int grp = tid / per, pi = d0 + tid % per;
    float a0 = 0.f, a1 = 0.f;
    if (grp < groups && pi < pairs) {
      const int d = 2 * pi;
      const bool two = d + 1 < p.D;
#pragma unroll 4
      for (int s = grp; s < p.S; s += groups) {
        const float w = s_w[s];
        if (w == 0.f) continue;
        const TP* src = po + s * p.po_s[0] + d;
        a0 += ElemTraits<TP>::to_float(src[0]) * w;
        if (two) a1 += ElemTraits<TP>::to_float(src[1]) * w;
      }
    }
    __syncthreads();
    s_acc[tid][0] = a0; s_acc[tid][1] = a1;
    __syncthreads();
    if (grp == 0 && pi < pairs) {
      for (int g2 = 1; g2 < groups; ++g2) { a0 += s_acc[g2 * per + tid][0]; a1 += s_acc[g2 * per + tid][1]; }
      const int d = 2 * pi;
      o[d] = ElemTraits<TO>::from_float(a0 * inv_l);
      if (d + 1 < p.D) o[d + 1] = ElemTraits<TO>::from_float(a1 * inv_l);
    }
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
  bool launched = false;
  G4B_DISPATCH_FLOAT(a.partial_o.dtype, TP,
    G4B_DISPATCH_FLOAT(a.o.dtype, TO,
      combine_kernel<TP, TO><<<(unsigned)rows, kCombineThreads, 0, st>>>(p); launched = true));
  if (!launched) return fail(G4B_ERR_BAD_DTYPE, "combine: partial_o/o dtypes must be f32, f16 or bf16");
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

}  // namespace g4b
