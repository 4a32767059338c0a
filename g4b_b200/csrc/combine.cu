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

template <typename TP, typename TO>
__global__ void __launch_bounds__(128) combine_kernel(CombineParams p) {
  // one block per (b, h, t) row; thread handles 2 consecutive d per pass
  int64_t row = blockIdx.x;
  const int t = (int)(row % p.Tq); row /= p.Tq;
  const int h = (int)(row % p.H);
  const int b = (int)(row / p.H);
  if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) return;

  float m = -INFINITY;
  for (int s = 0; s < p.S; ++s)
    m = fmaxf(m, p.pm[s * p.pm_s[0] + b * p.pm_s[1] + h * p.pm_s[2] + t * p.pm_s[3]]);
  float l = 0.f;
  for (int s = 0; s < p.S; ++s) {
    const float ms = p.pm[s * p.pm_s[0] + b * p.pm_s[1] + h * p.pm_s[2] + t * p.pm_s[3]];
    const float ls = p.pl[s * p.pl_s[0] + b * p.pl_s[1] + h * p.pl_s[2] + t * p.pl_s[3]];
    if (ms != -INFINITY) l += ls * exp2f(ms - m);
  }
  const float inv_l = l > 0.f ? 1.0f / l : 0.f;

  const TP* po = (const TP*)p.po + b * p.po_s[1] + h * p.po_s[2] + t * p.po_s[3];
  TO* o = (TO*)p.o + b * p.o_s[0] + h * p.o_s[1] + t * p.o_s[2];
  for (int d = threadIdx.x * 2; d < p.D; d += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int s = 0; s < p.S; ++s) {
      const float ms = p.pm[s * p.pm_s[0] + b * p.pm_s[1] + h * p.pm_s[2] + t * p.pm_s[3]];
      if (ms == -INFINITY) continue;
      const float w = exp2f(ms - m);
      const TP* src = po + s * p.po_s[0] + d;
      a0 += ElemTraits<TP>::to_float(src[0]) * w;
      if (d + 1 < p.D) a1 += ElemTraits<TP>::to_float(src[1]) * w;
    }
    o[d] = ElemTraits<TO>::from_float(a0 * inv_l);
    if (d + 1 < p.D) o[d + 1] = ElemTraits<TO>::from_float(a1 * inv_l);
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
  bool launched = false;
  G4B_DISPATCH_FLOAT(a.partial_o.dtype, TP,
    G4B_DISPATCH_FLOAT(a.o.dtype, TO,
      combine_kernel<TP, TO><<<(unsigned)rows, 128, 0, st>>>(p); launched = true));
  if (!launched) return fail(G4B_ERR_BAD_DTYPE, "combine: partial_o/o dtypes must be f32, f16 or bf16");
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

}  // namespace g4b
