// Single-token decode attention, register-streaming form: the K/V of one (slot, kv head,
// split) go global -> registers exactly once.  The TMA-fed kernel in decode_stream.cu has
// replaced it wherever its 16-row boxes fit; this one remains for ring caches shorter than
// 16 rows (head dim 256).
//
// Replaces _attn_kernel (g4b/kernels/fa2.py:256-480) for Tq == 1, in the reference's ring
// layout (fa2.py:52-55,75) and in the paged layout (16-token pages behind a block table).
//
// Design (HBM-bound; one K/V byte is read once and serves all query heads of its kv head):
//  * a CTA of 4 warps owns one (slot b, kv head g, split s); warps take 16-key blocks
//    round-robin, so a block is exactly one (page, head) run of 2 x 8 KB in paged mode;
//  * K and V rows go global -> registers with 128-bit loads laid out so that the loaded
//    registers ARE the operand fragments of warp-level m16n8k16 tensor instructions:
//      S[head, key]  = Q K^T   with the contraction index permuted identically in Q and K,
//      O^T[d, head]  = V^T P^T with V^T fragments assembled from two key rows by byte
//                               permutes and P^T taken straight from the S accumulators;
//    no shared memory, no barriers and no conversions on the streaming path;
//  * base-2 online softmax per head, row maxima by two warp shuffles; the O rescale is
//    skipped (warp vote) when no maximum moved;
//  * the 4 warps merge through shared memory; the CTA writes o (1 split) or the
//    (acc, l, m) partial of fa2.py:438-472 (m in log2 units).
#include "common.cuh"
#include "mma16816.cuh"

namespace g4b {

struct DecodeParams {
  const void* q; const void* k; const void* v; void* o;
  const int32_t* time_dim_sizes; const uint8_t* user_phase; const int32_t* block_tables;
  void* po; float* pl; float* pm;
  int64_t q_s0, q_s1;            // q strides for b, h (elements)
  int64_t o_s0, o_s1;
  int64_t po_s0, po_s1, po_s2;   // partial_o strides for s, b, h
  int64_t pl_s0, pl_s1, pl_s2, pm_s0, pm_s1, pm_s2;
  int64_t time_stride, phase_stride, bt_s0, bt_s1;
  int B, H, G, T;                // T: ring rows (ring mode)
  int page_shift, num_pages, max_pages;
  int ctx_window, sliding_window, phase, num_splits;
  int q_dtype, o_dtype, po_dtype;
  float scale_log2;              // scale * log2(e)
  int32_t* status;
};

constexpr int kDecodeWarps = 4;
constexpr int kD = 256;

// Per-warp running state of the online softmax and the O^T accumulators.
struct WarpState {
  float oacc[16][4];
  float m_run;   // running max of head gi (log2 units), identical in the 4 lanes of a row
  float l_run;   // this lane's share of the running sum
};

// One 16-key block.  krow[t]: row of key 8t + gi (+ 8c elements); vrow[kk]: row of key
// 2c + (kk&1) + 8(kk>>1) (+ 8gi elements); vok[kk]: that key is inside [lo_all, hi_all).
template <typename T>
__device__ __forceinline__ void block_step(WarpState& st, const uint32_t (&qf)[8][4],
                                           const T* const (&krow)[2], const T* const (&vrow)[4],
                                           const bool (&vok)[4], int j0, bool full, int lo_all,
                                           int hi_all, float scale_log2, int c) {
  uint4 kf[2][8];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int i = 0; i < 8; ++i) kf[t][i] = ld_stream(krow[t] + 32 * i);
  uint4 vf[4][4];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      vf[kk][i] = vok[kk] ? ld_stream(vrow[kk] + 64 * i) : make_uint4(0u, 0u, 0u, 0u);

  // ---------------- S = Q K^T ----------------
  float s[2][4];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      Mma<T>::run(s[t], qf[i][0], 0u, qf[i][1], 0u, kf[t][i].x, kf[t][i].y);
      Mma<T>::run(s[t], qf[i][2], 0u, qf[i][3], 0u, kf[t][i].z, kf[t][i].w);
    }
  }
  // ---------------- online softmax (head gi; keys 8t + 2c, 8t + 2c + 1) ----------------
  float sv[4];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int key = j0 + 8 * t + 2 * c + e;
      float x = s[t][e] * scale_log2;
      if (!full && (key < lo_all || key >= hi_all)) x = -INFINITY;
      sv[2 * t + e] = x;
    }
  float mb = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
  mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
  mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
  const float m_new = fmaxf(st.m_run, mb);
  const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
  const float alpha = exp2f(st.m_run - m_use);   // 0 on the first block
  const bool moved = m_new > st.m_run;
  st.m_run = m_new;
  float pr[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) pr[e] = exp2f(sv[e] - m_use);
  if (__any_sync(0xffffffffu, moved)) {
    // O^T columns are heads 2c, 2c+1: fetch their factors from the rows that own them
    const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * c) * 4);
    const float a1 = __shfl_sync(0xffffffffu, alpha, (2 * c + 1) * 4);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      st.oacc[i][0] *= a0; st.oacc[i][1] *= a1; st.oacc[i][2] *= a0; st.oacc[i][3] *= a1;
    }
  }
  const uint32_t pb0 = Mma<T>::pack(pr[0], pr[1]);
  const uint32_t pb1 = Mma<T>::pack(pr[2], pr[3]);
  // row sum over the ROUNDED probabilities the tensor instruction multiplies, so numerator
  // and denominator stay consistent (exact for a single visible key)
  st.l_run = st.l_run * alpha + Mma<T>::sum2(pb0) + Mma<T>::sum2(pb1);
  // bf16 keeps 8 significant bits of p: feed the rounding residue through a second product
  // (P = P_hi + P_lo) so the weights carry ~16 bits, like the f16 path's 11
  uint32_t pl0 = 0u, pl1 = 0u;
  if constexpr (Mma<T>::kSplitP) {
    pl0 = Mma<T>::pack(pr[0] - __uint_as_float(pb0 << 16), pr[1] - __uint_as_float(pb0 & 0xffff0000u));
    pl1 = Mma<T>::pack(pr[2] - __uint_as_float(pb1 << 16), pr[3] - __uint_as_float(pb1 & 0xffff0000u));
    st.l_run += Mma<T>::sum2(pl0) + Mma<T>::sum2(pl1);
  }
  // ---------------- O^T += V^T P^T ----------------
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t v0[4] = {vf[0][i].x, vf[0][i].y, vf[0][i].z, vf[0][i].w};
    const uint32_t v1[4] = {vf[1][i].x, vf[1][i].y, vf[1][i].z, vf[1][i].w};
    const uint32_t v2[4] = {vf[2][i].x, vf[2][i].y, vf[2][i].z, vf[2][i].w};
    const uint32_t v3[4] = {vf[3][i].x, vf[3][i].y, vf[3][i].z, vf[3][i].w};
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const uint32_t a0 = __byte_perm(v0[e2], v1[e2], 0x5410);
      const uint32_t a1 = __byte_perm(v0[e2], v1[e2], 0x7632);
      const uint32_t a2 = __byte_perm(v2[e2], v3[e2], 0x5410);
      const uint32_t a3 = __byte_perm(v2[e2], v3[e2], 0x7632);
      Mma<T>::run(st.oacc[i * 4 + e2], a0, a1, a2, a3, pb0, pb1);
      if constexpr (Mma<T>::kSplitP) Mma<T>::run(st.oacc[i * 4 + e2], a0, a1, a2, a3, pl0, pl1);
    }
  }
}

template <typename T, bool kPaged>
__global__ void __launch_bounds__(kDecodeWarps * 32, 2) decode_kernel(DecodeParams p) {
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gi = lane >> 2, c = lane & 3;   // mma fragment coordinates
  const int R = p.H / p.G;                  // query heads per kv head (<= 8)

  if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) return;

  __shared__ float sm_o[kDecodeWarps][8][kD];
  __shared__ float sm_m[kDecodeWarps][8];
  __shared__ float sm_l[kDecodeWarps][8];

  // ---- key range of this split (fa2.py:52-67, with block-aligned split boundaries) ----
  const int time = p.time_dim_sizes[b * p.time_stride];
  const int window = min(time, p.ctx_window);
  // Ring mode counts keys from the oldest one the cache exposes; a paged cache is addressed
  // by absolute position, so there the exposed window is just another lower bound.
  int lo_all = kPaged ? time - window : 0;
  const int hi_all = kPaged ? time : window;
  if (p.sliding_window > 0) lo_all = max(lo_all, hi_all - p.sliding_window);
  const int lo_al = lo_all & ~15;
  const int nblk = hi_all > lo_al ? (hi_all - lo_al + 15) >> 4 : 0;
  const int bps = (nblk + p.num_splits - 1) / p.num_splits;   // blocks per split
  const int blk_lo = split * bps;
  const int blk_hi = min(nblk, blk_lo + bps);

  // ---- Q fragments: head gi, the 16 bytes at d = 32 i + 8 c, i = 0..7 ----
  uint32_t qf[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) { qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u; }
  if (gi < R) {
    const int h = g * R + gi;
    const int64_t qoff = b * p.q_s0 + h * p.q_s1;
    const bool q_is_t = p.q_dtype == ElemTraits<T>::kDtype;
    if (q_is_t && ((reinterpret_cast<uintptr_t>((const T*)p.q + qoff) & 15) == 0)) {
      // same element type as the cache: the 16 bytes are the fragment registers as they are
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 w = *reinterpret_cast<const uint4*>((const T*)p.q + qoff + 32 * i + 8 * c);
        qf[i][0] = w.x; qf[i][1] = w.y; qf[i][2] = w.z; qf[i][3] = w.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = load_as_float(p.q, qoff + 32 * i + 8 * c + e, p.q_dtype);
#pragma unroll
        for (int e = 0; e < 4; ++e) qf[i][e] = Mma<T>::pack(f[2 * e], f[2 * e + 1]);
      }
    }
  }

  WarpState st;
#pragma unroll
  for (int i = 0; i < 16; ++i) { st.oacc[i][0] = st.oacc[i][1] = st.oacc[i][2] = st.oacc[i][3] = 0.f; }
  st.m_run = -INFINITY;
  st.l_run = 0.f;

  if constexpr (kPaged) {
    const int32_t* bt = p.block_tables + b * p.bt_s0;
    const int page_mask = (1 << p.page_shift) - 1;
    // page ids are fetched two blocks ahead of their use to keep the table off the critical path
    auto fetch = [&](int bl) -> int {
      if (bl >= blk_hi) return 0;
      const int pg = (lo_al + (bl << 4)) >> p.page_shift;
      int page = pg < p.max_pages ? bt[pg * p.bt_s1] : -1;
      if (page < 0 || page >= p.num_pages) {   // never follow a bad table entry
        atomicCAS(p.status, 0, 0x200 | 1);
        page = 0;
      }
      return page;
    };
    int blk = blk_lo + warp;
    int page_cur = fetch(blk);
    int page_nxt = fetch(blk + kDecodeWarps);
    for (; blk < blk_hi; blk += kDecodeWarps) {
      const int page_after = fetch(blk + 2 * kDecodeWarps);
      const int j0 = lo_al + (blk << 4);
      const bool full = (j0 >= lo_all) && (j0 + 16 <= hi_all);
      const int64_t base =
          ((((int64_t)page_cur * p.G + g) << p.page_shift) + (j0 & page_mask)) * kD;
      const T* kb = (const T*)p.k + base;
      const T* vb = (const T*)p.v + base;
      const T* krow[2] = {kb + (int64_t)gi * kD + 8 * c, kb + (int64_t)(8 + gi) * kD + 8 * c};
      const T* vrow[4];
      bool vok[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int key = 2 * c + (kk & 1) + 8 * (kk >> 1);
        vrow[kk] = vb + (int64_t)key * kD + 8 * gi;
        vok[kk] = full || (j0 + key >= lo_all && j0 + key < hi_all);
      }
      block_step<T>(st, qf, krow, vrow, vok, j0, full, lo_all, hi_all, p.scale_log2, c);
      page_cur = page_nxt; page_nxt = page_after;
    }
  } else {
    const int64_t bg = ((int64_t)b * p.G + g) * p.T * kD;
    const T* kb = (const T*)p.k + bg;
    const T* vb = (const T*)p.v + bg;
    const int ring_start = max(time - p.ctx_window, 0) % p.T;
    auto ring_row = [&](int j) -> int64_t {   // logical key -> element offset of its row
      int r = ring_start + min(j, hi_all - 1);   // keys past the window: any valid row, masked later
      if (r >= p.T) r -= p.T;
      return (int64_t)r * kD;
    };
    for (int blk = blk_lo + warp; blk < blk_hi; blk += kDecodeWarps) {
      const int j0 = lo_al + (blk << 4);
      const bool full = (j0 >= lo_all) && (j0 + 16 <= hi_all);
      const T* krow[2] = {kb + ring_row(j0 + gi) + 8 * c, kb + ring_row(j0 + 8 + gi) + 8 * c};
      const T* vrow[4];
      bool vok[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int key = j0 + 2 * c + (kk & 1) + 8 * (kk >> 1);
        vrow[kk] = vb + ring_row(key) + 8 * gi;
        vok[kk] = full || (key >= lo_all && key < hi_all);
      }
      block_step<T>(st, qf, krow, vrow, vok, j0, full, lo_all, hi_all, p.scale_log2, c);
    }
  }

  // ---- merge the warps ----
  float l_run = st.l_run;
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (c == 0) { sm_m[warp][gi] = st.m_run; sm_l[warp][gi] = l_run; }
  // oacc[i*4+e2]: rows d = 64 i + 8 gi + 2 e2 (+1 for regs 2,3), columns heads 2c, 2c+1
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const int d = 64 * i + 8 * gi + 2 * e2;
      const float* a = st.oacc[i * 4 + e2];
      *reinterpret_cast<float2*>(&sm_o[warp][2 * c][d]) = make_float2(a[0], a[2]);
      *reinterpret_cast<float2*>(&sm_o[warp][2 * c + 1][d]) = make_float2(a[1], a[3]);
    }
  __syncthreads();

  for (int idx = threadIdx.x; idx < R * kD; idx += kDecodeWarps * 32) {
    const int hh = idx / kD, d = idx % kD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) m = fmaxf(m, sm_m[w][hh]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float mw = sm_m[w][hh];
      if (mw == -INFINITY) continue;
      const float sc = exp2f(mw - m);
      acc += sm_o[w][hh][d] * sc;
      l += sm_l[w][hh] * sc;
    }
    const int h = g * R + hh;
    if (p.num_splits == 1) {
      const float outv = l > 0.f ? acc / l : 0.f;
      store_from_float(p.o, b * p.o_s0 + h * p.o_s1 + d, p.o_dtype, outv);
    } else {
      store_from_float(p.po, split * p.po_s0 + b * p.po_s1 + h * p.po_s2 + d, p.po_dtype, acc);
      if (d == 0) {
        p.pl[split * p.pl_s0 + b * p.pl_s1 + h * p.pl_s2] = l;
        p.pm[split * p.pm_s0 + b * p.pm_s1 + h * p.pm_s2] = m;
      }
    }
  }
}

int launch_decode(const G4bAttnArgs& a, int num_splits, cudaStream_t st) {
  DecodeParams p{};
  p.q = a.q.ptr; p.k = a.k_cache.ptr; p.v = a.v_cache.ptr; p.o = a.o.ptr;
  p.time_dim_sizes = (const int32_t*)a.time_dim_sizes.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr;
  p.block_tables = (const int32_t*)a.block_tables.ptr;
  p.po = a.partial_o.ptr; p.pl = (float*)a.partial_l.ptr; p.pm = (float*)a.partial_m.ptr;
  p.q_s0 = a.q.stride[0]; p.q_s1 = a.q.stride[1];
  p.o_s0 = a.o.stride[0]; p.o_s1 = a.o.stride[1];
  p.po_s0 = a.partial_o.stride[0]; p.po_s1 = a.partial_o.stride[1]; p.po_s2 = a.partial_o.stride[2];
  p.pl_s0 = a.partial_l.stride[0]; p.pl_s1 = a.partial_l.stride[1]; p.pl_s2 = a.partial_l.stride[2];
  p.pm_s0 = a.partial_m.stride[0]; p.pm_s1 = a.partial_m.stride[1]; p.pm_s2 = a.partial_m.stride[2];
  p.time_stride = a.time_dim_sizes.stride[0]; p.phase_stride = a.user_phase.stride[0];
  p.bt_s0 = a.block_tables.stride[0]; p.bt_s1 = a.block_tables.stride[1];
  p.B = (int)a.q.shape[0]; p.H = (int)a.q.shape[1]; p.G = (int)a.k_cache.shape[1];
  const bool paged = a.block_tables.ptr != nullptr;
  if (paged) {
    p.page_shift = 0;
    while ((1 << p.page_shift) < a.page_size) ++p.page_shift;
    p.num_pages = (int)a.k_cache.shape[0];
    p.max_pages = (int)a.block_tables.shape[1];
    p.T = 0;
  } else {
    p.T = (int)a.k_cache.shape[2];
  }
  p.ctx_window = a.ctx_window_size; p.sliding_window = a.sliding_window; p.phase = a.phase;
  p.num_splits = num_splits;
  p.q_dtype = a.q.dtype; p.o_dtype = a.o.dtype; p.po_dtype = a.partial_o.dtype;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  G4B_STOP_IF_VALIDATE_ONLY();
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;
  if (p.B == 0) return G4B_OK;
  dim3 grid((unsigned)num_splits, (unsigned)p.G, (unsigned)p.B);
  const int kv_dt = a.k_cache.dtype;
  if (kv_dt == G4B_BF16) {
    if (paged) decode_kernel<__nv_bfloat16, true><<<grid, kDecodeWarps * 32, 0, st>>>(p);
    else decode_kernel<__nv_bfloat16, false><<<grid, kDecodeWarps * 32, 0, st>>>(p);
  } else if (kv_dt == G4B_F16) {
    if (paged) decode_kernel<__half, true><<<grid, kDecodeWarps * 32, 0, st>>>(p);
    else decode_kernel<__half, false><<<grid, kDecodeWarps * 32, 0, st>>>(p);
  } else {
    return fail(G4B_ERR_BAD_DTYPE, "decode: KV cache must be f16 or bf16");
  }
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

}  // namespace g4b
