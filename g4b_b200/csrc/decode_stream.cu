// Single-token decode attention as a TMA-fed stream: K/V tiles go HBM -> shared memory through
// a ring of mbarrier-guarded stages that one producer warp keeps full, independent of the
// registers of the warps that compute.  The same launch can append the new token's K/V rows
// and, when one sequence's KV range is split over GPUs, merge the splits and exchange the
// merged partials with the peers.
//
// Replaces _attn_kernel (g4b/kernels/fa2.py:256-480) for Tq == 1 and, in the decode step,
// the two add_kv_to_cache launches before it (g4b/models/gemma4e.py:575-592) and (exchange
// form) _reduce_split_kv_kernel (fa2.py:546-631), in the reference's ring layout
// (fa2.py:52-55,75) and in the paged layout.  Head dims 128, 256, 512; f16 / bf16 caches, or
// e4m3 pages with a scale per (page, kv head).
//
// A CTA = one (slot b, kv head g, split s): 3 consumer warps + 1 producer warp.
//   producer   walks the split's 16-key blocks; per block one stage = a K tile and a V tile
//              [16 keys x D], each ONE 128-byte-swizzled TMA box: the descriptor describes a
//              row as slabs of 128 bytes (a slab dimension whose stride lies below the row
//              stride), so [128 bytes x 16 rows x slabs] lands slab-major, the layout ldmatrix
//              reads without bank conflicts.  Paged: a box is one (page, kv head) run.  Ring:
//              the block that crosses the end of the ring becomes two stages whose boxes start
//              past the end / before row 0 and read zeros there.  Every stage carries its key
//              range, so partial blocks (window edges, the wrap, a bad table entry) are masked
//              by the consumer, never computed with.
//   consumers  take the stages in order, whichever warp is free next (a shared counter), so
//              all stages of the ring are in flight or in work whatever the warps' pace;
//              S = Q K^T and O^T = V^T P^T with warp-level m16n8k16 instructions whose K / V
//              operand fragments come out of the swizzled tiles by ldmatrix (V transposed on
//              the way); base-2 online softmax per head; all (<= 8) query heads of the kv head
//              share every byte.  The warp that meets the stage of the new token's position
//              overwrites that row of its tiles with k_new / v_new and stores them to the cache.
// The 3 warps merge through shared memory; the CTA writes o (one split) or the (acc, l, m)
// partial of fa2.py:438-472, which a merge launch (combine.cu) picks up.
//
// Exchange form (one sequence's KV range split over GPUs; every CTA of the launch is resident
// at once, which the launcher checks).  After its partial is written a CTA arrives at a
// grid-wide count.  The first D / 8 CTAs of every (slot, kv head) then each own 8 columns of the
// head dim: they wait (bounded) for the count, merge all local partials for their columns (one
// trip to L2: every thread asks for the pieces of its splits before it uses one and merges
// with a running maximum), push the merged piece to every GPU as self-announcing 8-byte words {value, launch count}, poll
// (bounded) their own buffer for the peers' pieces and finish the merge -- the word format of
// combine_exchange.cu, in the same launch as the attention.
#include <type_traits>

#include "common.cuh"
#include "mma16816.cuh"
#include "sm100_ptx.cuh"

namespace g4b {
namespace {

constexpr int kConsumers = 3;   // + 1 producer = 4 warps: two CTAs are 8 warps, 2 per SM sub-partition, so 255 registers each
constexpr int kStreamThreads = (kConsumers + 1) * 32;
constexpr int kXCols = 8;                     // head-dim columns a merging CTA owns
constexpr int kXWords = kXCols + 2;           // its piece per query head: the columns, the row sum, the row maximum
constexpr int kMaxResidentSplits = 320;       // splits of one (slot, kv head) when every CTA is resident
constexpr long long kPeerWaitLimit = 1ll << 31;   // SM cycles (about a second)

enum : int32_t { kErrBadEntry = 0x201, kErrStageFull = 0x211, kErrStageEmpty = 0x212, kErrStageOrder = 0x213,
                 kErrAppendRow = 0x214, kErrGridWait = 0x215, kErrPeerWait = 0x401 };

// Grid-wide arrival counts of the exchange form: {arrivals of even turns, of odd turns, whose
// turn it is}.  A launch counts on its turn's word and, once full, zeroes the other one and
// hands the turn over, so nothing is counted or reset at the end of a launch.  One set per
// GPU, shared by every launch on it.
__device__ uint32_t g_step_sync[3];

template <int D, bool kFp8 = false> struct StreamCfg {
  static constexpr int kTileBytes = 16 * D * (kFp8 ? 1 : 2);   // 16 keys of K, or of V
  static constexpr int kStageBytes = 2 * kTileBytes;
  // 16-bit pools: 64 / 96 / 192 KB in flight per CTA.  e4m3 pools at head dim <= 256: three CTAs
  // per SM (nine consumer warps: at half the bytes per key the tensor work, not HBM, sets the pace)
  static constexpr int kStages = kFp8 ? (D == 512 ? 6 : 8) : (D == 128 ? 8 : 6);
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kCtasPerSm = kFp8 ? (D >= 512 ? 2 : 3) : (D >= 512 ? 1 : 2);
};

struct StreamParams {
  const void* q; void* o;
  const int32_t* time_dim_sizes; const uint8_t* user_phase; const int32_t* block_tables;
  void* po; float* pl; float* pm;
  int64_t q_s0, q_s1, o_s0, o_s1;
  int64_t po_s0, po_s1, po_s2, pl_s0, pl_s1, pl_s2, pm_s0, pm_s1, pm_s2;
  int64_t time_stride, phase_stride, bt_s0, bt_s1;
  int B, H, G, T;
  int page_shift, num_pages, max_pages;
  int ctx_window, sliding_window, phase, num_splits;
  int q_dtype, o_dtype, po_dtype;
  float scale_log2;
  int32_t* status;
  // e4m3 pools: one f32 scale per (page, kv head), value = stored byte's value x scale
  const float* k_scales; const float* v_scales;
  int64_t ks_s0, ks_s1, vs_s0, vs_s1;
  // decode step
  uint32_t* sync;              // {arrivals of even turns, of odd turns, turn} (exchange form), else null
  void* k_cache; void* v_cache;
  const void* k_new; const void* v_new;
  int64_t kn_s0, kn_s1, vn_s0, vn_s1;
  unsigned long long* xbuf[8];
  uint32_t* xstate;
  int world, rank;
};

template <int kStages> struct alignas(16) Ctl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int4 meta[kStages];          // x: logical key of tile row 0, y / z: valid rows [y, z), w: cache row of tile row 0
  float2 scl[kStages];         // e4m3 pools: the stage's page scales (K, V)
  float sm_m[kConsumers][8];
  float sm_l[kConsumers][8];
  uint32_t epoch;
  uint32_t turn;               // which of the two arrival counters this launch counts on
  int flag;
  int next_stage;              // next stage no consumer has claimed yet
  volatile int done[kStages];  // uses of a ring slot that have been consumed
  volatile int fail;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void st_word_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// two neighbouring words in one request; each 8-byte half arrives whole
__device__ __forceinline__ ulonglong2 ld_pair_sys(const ulonglong2* p) {
  ulonglong2 v;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}

// Byte offset, inside a [16 rows x D] tile of 128-byte-swizzled 64-element slabs, of the
// 16-byte chunk `chunk` (8 elements) of row `row`.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)((chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int D> struct WarpAcc {
  float oacc[D / 16][4];   // O^T: rows d = 16 i + gi (regs 0, 1) and + 8 (regs 2, 3), columns heads 2c, 2c + 1
  float m_run;             // running max of head gi (log2 units), identical in the 4 lanes of a row
  float l_run;             // this lane's share of the running sum
};

// One stage: 16 keys.  qa[ks]: A fragments (a0, a2) of Q for contraction step ks (head gi).
template <typename T, int D>
__device__ __forceinline__ void stage_step(WarpAcc<D>& st, const uint32_t (&qa)[D / 16][2], uint32_t k_tile,
                                           uint32_t v_tile, int vlo, int vhi, float scale_log2, int lane) {
  const int c = lane & 3;
  const bool full = vlo == 0 && vhi == 16;
  // ---------------- S = Q K^T: two groups of 8 keys, two accumulator chains each ----------------
  float s[2][4], s2[2][4];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
    s2[t][0] = s2[t][1] = s2[t][2] = s2[t][3] = 0.f;
  }
#pragma unroll
  for (int kk = 0; kk < D / 32; ++kk) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      // matrices: (keys 8t.., chunk 4kk), (.., 4kk+1), (.., 4kk+2), (.., 4kk+3)
      uint32_t r0, r1, r2, r3;
      ldsm_x4(k_tile + tile_off(8 * t + (lane & 7), 4 * kk + (lane >> 3)), r0, r1, r2, r3);
      Mma<T>::run(s[t], qa[2 * kk][0], 0u, qa[2 * kk][1], 0u, r0, r1);
      Mma<T>::run(s2[t], qa[2 * kk + 1][0], 0u, qa[2 * kk + 1][1], 0u, r2, r3);
    }
  }
  // ---------------- online softmax (head gi; keys 8t + 2c, 8t + 2c + 1) ----------------
  float sv[4];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int key = 8 * t + 2 * c + e;
      float x = (s[t][e] + s2[t][e]) * scale_log2;
      if (!full && (key < vlo || key >= vhi)) x = -INFINITY;
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
    for (int i = 0; i < D / 16; ++i) {
      st.oacc[i][0] *= a0; st.oacc[i][1] *= a1; st.oacc[i][2] *= a0; st.oacc[i][3] *= a1;
    }
  }
  const uint32_t pb0 = Mma<T>::pack(pr[0], pr[1]);
  const uint32_t pb1 = Mma<T>::pack(pr[2], pr[3]);
  // row sum over the ROUNDED probabilities the tensor instruction multiplies, so numerator
  // and denominator stay consistent (exact for a single visible key)
  st.l_run = st.l_run * alpha + Mma<T>::sum2(pb0) + Mma<T>::sum2(pb1);
  // bf16 keeps 8 significant bits of p: feed the rounding residue through a second product
  uint32_t pl0 = 0u, pl1 = 0u;
  if constexpr (Mma<T>::kSplitP) {
    pl0 = Mma<T>::pack(pr[0] - __uint_as_float(pb0 << 16), pr[1] - __uint_as_float(pb0 & 0xffff0000u));
    pl1 = Mma<T>::pack(pr[2] - __uint_as_float(pb1 << 16), pr[3] - __uint_as_float(pb1 & 0xffff0000u));
    st.l_run += Mma<T>::sum2(pl0) + Mma<T>::sum2(pl1);
  }
  // ---------------- O^T += V^T P^T ----------------
  // rows outside the stage's key range may hold anything (NaN included): clear their bits
  uint32_t m01 = 0xffffffffu, m23 = 0xffffffffu;
  if (!full) {
    auto ok = [&](int key) { return key >= vlo && key < vhi; };
    m01 = (ok(2 * c) ? 0x0000ffffu : 0u) | (ok(2 * c + 1) ? 0xffff0000u : 0u);
    m23 = (ok(2 * c + 8) ? 0x0000ffffu : 0u) | (ok(2 * c + 9) ? 0xffff0000u : 0u);
  }
#pragma unroll
  for (int i = 0; i < D / 16; ++i) {
    // matrices: (keys 0-7, chunk 2i), (keys 0-7, chunk 2i+1), (keys 8-15, chunk 2i), (keys 8-15, chunk 2i+1)
    uint32_t a0, a1, a2, a3;
    ldsm_x4_t(v_tile + tile_off((lane & 7) + 8 * (lane >> 4), 2 * i + ((lane >> 3) & 1)), a0, a1, a2, a3);
    if (!full) { a0 &= m01; a1 &= m01; a2 &= m23; a3 &= m23; }
    Mma<T>::run(st.oacc[i], a0, a1, a2, a3, pb0, pb1);
    if constexpr (Mma<T>::kSplitP) Mma<T>::run(st.oacc[i], a0, a1, a2, a3, pl0, pl1);
  }
}

// e4m3 pair -> f16 pair
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo;\n\tcvt.u16.u32 lo, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(r) : "r"(two_bytes));
  return r;
}

// One stage of an e4m3 pool: 16 keys, rows of D bytes.  The tensor instructions run on f16:
// an e4m3 value is exact in f16, q is rounded to f16, and the page's scales go into the
// scores (K) and into the probabilities handed to the second product (V).
//   K: an 8 x 8 "b16" ldmatrix tile is 8 keys x 16 bytes; a thread gets 4 consecutive bytes of
//      key gi, d = 16 ks + 4c .. + 3, which become the two B registers of contraction step ks.
//      q's A registers are loaded in the same order (qa[ks] = q[16 ks + 4c, +1], q[16 ks + 4c + 2, +3]).
//   V: the transposing ldmatrix hands a thread bytes (key 2c: d, d + 1 | key 2c + 1: d, d + 1),
//      d = 2 gi of a 16-byte chunk; the even bytes form the A registers of one product (output
//      rows d = 32 j + 2 gi and + 16), the odd bytes those of a second (rows + 1).
// oacc[2 j + par]: rows d = 32 j + 2 gi + par (regs 0, 1) and + 16 (regs 2, 3).
template <int D>
__device__ __forceinline__ void stage_step_fp8(WarpAcc<D>& st, const uint32_t (&qa)[D / 16][2], uint32_t k_tile,
                                               uint32_t v_tile, int vlo, int vhi, float scale_log2_k, float v_scale,
                                               int lane) {
  using M = Mma<__half>;
  const int c = lane & 3;
  const bool full = vlo == 0 && vhi == 16;
  float s[2][4], s2[2][4];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
    s2[t][0] = s2[t][1] = s2[t][2] = s2[t][3] = 0.f;
  }
#pragma unroll
  for (int kk = 0; kk < D / 64; ++kk) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      uint32_t r[4];
      ldsm_x4(k_tile + tile_off(8 * t + (lane & 7), 4 * kk + (lane >> 3)), r[0], r[1], r[2], r[3]);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int ks = 4 * kk + q4;
        const uint32_t b0 = e4m3x2_to_f16x2(r[q4] & 0xffffu), b1 = e4m3x2_to_f16x2(r[q4] >> 16);
        if (q4 & 1) M::run(s2[t], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
        else M::run(s[t], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
      }
    }
  }
  float sv[4];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int key = 8 * t + 2 * c + e;
      float x = (s[t][e] + s2[t][e]) * scale_log2_k;
      if (!full && (key < vlo || key >= vhi)) x = -INFINITY;
      sv[2 * t + e] = x;
    }
  float mb = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
  mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
  mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
  const float m_new = fmaxf(st.m_run, mb);
  const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
  const float alpha = exp2f(st.m_run - m_use);
  const bool moved = m_new > st.m_run;
  st.m_run = m_new;
  float pr[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) pr[e] = exp2f(sv[e] - m_use);
  if (__any_sync(0xffffffffu, moved)) {
    const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * c) * 4);
    const float a1 = __shfl_sync(0xffffffffu, alpha, (2 * c + 1) * 4);
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      st.oacc[i][0] *= a0; st.oacc[i][1] *= a1; st.oacc[i][2] *= a0; st.oacc[i][3] *= a1;
    }
  }
  st.l_run = st.l_run * alpha + (pr[0] + pr[1]) + (pr[2] + pr[3]);
  // the page's V scale rides on the probabilities: O += (p * scale) * v_bytes
  const uint32_t pb0 = M::pack(pr[0] * v_scale, pr[1] * v_scale);
  const uint32_t pb1 = M::pack(pr[2] * v_scale, pr[3] * v_scale);
  uint32_t m01 = 0xffffffffu, m23 = 0xffffffffu;
  if (!full) {
    auto ok = [&](int key) { return key >= vlo && key < vhi; };
    m01 = (ok(2 * c) ? 0x0000ffffu : 0u) | (ok(2 * c + 1) ? 0xffff0000u : 0u);
    m23 = (ok(2 * c + 8) ? 0x0000ffffu : 0u) | (ok(2 * c + 9) ? 0xffff0000u : 0u);
  }
#pragma unroll
  for (int j = 0; j < D / 32; ++j) {
    // matrices: (keys 0-7, chunk 2j), (keys 8-15, chunk 2j), (keys 0-7, chunk 2j+1), (keys 8-15, chunk 2j+1)
    uint32_t v[4];
    ldsm_x4_t(v_tile + tile_off((lane & 7) + 8 * ((lane >> 3) & 1), 2 * j + (lane >> 4)), v[0], v[1], v[2], v[3]);
#pragma unroll
    for (int par = 0; par < 2; ++par) {
      const uint32_t sel = par ? 0x4431u : 0x4420u;      // bytes (1, 3) or (0, 2) into the low half
      uint32_t a0 = e4m3x2_to_f16x2(__byte_perm(v[0], 0u, sel));
      uint32_t a1 = e4m3x2_to_f16x2(__byte_perm(v[2], 0u, sel));
      uint32_t a2 = e4m3x2_to_f16x2(__byte_perm(v[1], 0u, sel));
      uint32_t a3 = e4m3x2_to_f16x2(__byte_perm(v[3], 0u, sel));
      if (!full) { a0 &= m01; a1 &= m01; a2 &= m23; a3 &= m23; }
      M::run(st.oacc[2 * j + par], a0, a1, a2, a3, pb0, pb1);
    }
  }
}

// Word offset inside one rank's exchange buffer: [parity][source rank][row][slice of 8 columns][8 + 2].
__device__ __forceinline__ int64_t xword(const StreamParams& p, int D, int par, int src, int row, int slice) {
  return ((((int64_t)par * p.world + src) * ((int64_t)p.B * p.H) + row) * (D / kXCols) + slice) * kXWords;
}

template <typename T, int D, bool kPaged, bool kFp8>
__global__ void __launch_bounds__(kStreamThreads, StreamCfg<D, kFp8>::kCtasPerSm)
decode_stream_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                     StreamParams p) {
  using Cfg = StreamCfg<D, kFp8>;
  constexpr int kSt = Cfg::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gi = lane >> 2, c = lane & 3;   // mma fragment coordinates
  const int R = p.H / p.G;                  // query heads per kv head (<= 8)
  uint8_t* ring = smem_raw;
  Ctl<kSt>* ctl = reinterpret_cast<Ctl<kSt>*>(smem_raw + Cfg::kRingBytes);
  // after the stream the ring is scratch: the warps' accumulators, then the merging CTAs' reduction and the peers' pieces
  float* sm_o = reinterpret_cast<float*>(ring);                                   // [kConsumers][8][D + 4]

  // asked for before anything else: the split's key range, then its block-table entries, then
  // its first tiles each wait for the one before
  const int time = p.time_dim_sizes[b * p.time_stride];
  // a merge launch that follows may be scheduled as soon as SM resources free up (it waits for
  // this grid to finish before it reads the partials)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == 0) {
    for (int s = 0; s < kSt; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 1);
    }
    ptx::fence_barrier_init();
    ctl->fail = 0;
    ctl->flag = 0;
    ctl->next_stage = 0;
    for (int s = 0; s < kSt; ++s) ctl->done[s] = 0;
    ctl->epoch = p.xstate != nullptr ? p.xstate[0] + 1u : 0u;
    ctl->turn = p.sync != nullptr ? (p.sync[2] & 1u) : 0u;
    ptx::prefetch_tensormap(&k_map);
    ptx::prefetch_tensormap(&v_map);
  }
  __syncthreads();

  // Exchange form: every CTA of the launch, whatever it did, arrives once on the arrival
  // counter of this launch's turn (its partial, if it has one, is written by then).  Launches
  // take turns on two counters: once all have arrived, the launch's first CTA zeroes the OTHER
  // counter (the previous launch's, which nobody polls any more), hands the turn over and
  // advances the caller's launch count; a CTA that does not merge leaves as soon as it has
  // arrived and nothing is counted at the end of the launch.
  const uint32_t n_ctas = gridDim.x * gridDim.y * gridDim.z;
  const bool first_cta = (blockIdx.x | blockIdx.y | blockIdx.z) == 0;
  auto grid_arrive = [&]() {
    __syncthreads();
    // (a release after the barrier covers the stores of every thread of the CTA)
    if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync + ctl->turn) : "memory");
  };
  // every thread returns whether all CTAs arrived in time; the loads after it see their stores
  auto all_arrived = [&]() -> bool {
    if (tid == 0) {
      const long long t0 = clock64();
      int ok = 1;
      for (;;) {
        uint32_t n;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(n) : "l"(p.sync + ctl->turn) : "memory");
        if (n >= n_ctas) break;
        if (clock64() - t0 > ptx::kWaitLimitCycles) { atomicCAS(p.status, 0, kErrGridWait); ok = 0; break; }
      }
      ctl->flag = ok;
      if (first_cta) {
        p.sync[ctl->turn ^ 1u] = 0;
        p.sync[2] = ctl->turn ^ 1u;
        p.xstate[0] = ctl->epoch;
      }
    }
    __syncthreads();
    return ctl->flag != 0;
  };

  if (p.user_phase != nullptr && p.user_phase[b * p.phase_stride] != (uint8_t)p.phase) {
    if (p.sync != nullptr) {
      grid_arrive();
      if (first_cta) all_arrived();
    }
    return;
  }

  // ---- key range of this split (fa2.py:52-67, with block-aligned split boundaries) ----
  const int window = min(time, p.ctx_window);
  // Ring mode counts keys from the oldest one the cache exposes; a paged cache is addressed by
  // absolute position, so there the exposed window is just another lower bound.
  int lo_all = kPaged ? time - window : 0;
  const int hi_all = kPaged ? time : window;
  if (p.sliding_window > 0) lo_all = max(lo_all, hi_all - p.sliding_window);
  const int lo_al = lo_all & ~15;
  const int nblk = hi_all > lo_al ? (hi_all - lo_al + 15) >> 4 : 0;
  const int bps = (nblk + p.num_splits - 1) / p.num_splits;   // blocks per split
  const int blk_lo = min(nblk, split * bps);
  const int blk_hi = min(nblk, blk_lo + bps);
  // ring: logical key jw is the first one stored at row 0 again; the block that holds it in
  // its middle (if any, and if it is ours) becomes two stages
  int ring_start = 0, jw = 0x7fffffff, wrap_blk = -1;
  if constexpr (!kPaged) {
    ring_start = max(time - p.ctx_window, 0) % p.T;
    jw = p.T - ring_start;
    if (jw > lo_al && jw < hi_all && ((jw - lo_al) & 15) != 0) wrap_blk = (jw - lo_al) >> 4;
  }
  const bool has_wrap = wrap_blk >= blk_lo && wrap_blk < blk_hi;
  const int n_stages = (blk_hi - blk_lo) + (has_wrap ? 1 : 0);
  const int pnew = (p.k_new != nullptr) ? hi_all - 1 : -1;   // logical key of the appended token

  WarpAcc<D> acc;
  if (warp == kConsumers) {
    // =============================== producer ===============================
    const int32_t* bt = kPaged ? p.block_tables + b * p.bt_s0 : nullptr;
    const int page_mask = kPaged ? (1 << p.page_shift) - 1 : 0;
    // K / V rows are read once: they leave L2 first, so that the block tables, the partials and
    // the kernel's own instructions stay there while hundreds of megabytes stream through
    const uint64_t pol_stream = ptx::policy_evict_first();
    int my_page = 0;
    float my_ks = 1.f, my_vs = 1.f;
    for (int n = 0; n < n_stages; ++n) {
      const int stg = n % kSt;
      // every decision to leave the loop is taken by the whole warp
      if (__any_sync(0xffffffffu, ctl->fail != 0)) break;
      if (n >= kSt) {
        const bool ok = ptx::mbar_wait(ptx::smem_u32(&ctl->empty[stg]), (uint32_t)((n / kSt) - 1) & 1u);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) { atomicCAS(p.status, 0, kErrStageEmpty); ctl->fail = 1; }
          break;
        }
      }
      // stage n -> (block, part of the wrap block)
      int blk = blk_lo + n, part = 0;
      if (has_wrap) {
        const int w_off = wrap_blk - blk_lo;
        if (n == w_off) part = 1;
        else if (n == w_off + 1) { blk = wrap_blk; part = 2; }
        else if (n > w_off + 1) blk = blk_lo + n - 1;
      }
      const int j0 = lo_al + (blk << 4);
      int vlo = max(0, lo_all - j0), vhi = min(16, hi_all - j0);
      int row0;   // cache row (paged: row of the pool seen as [num_pages * G * page, D]) of tile row 0
      int page = 0;
      if constexpr (kPaged) {
        // page ids of the next 32 blocks, one per lane
        if ((n & 31) == 0) {
          const int bl = blk_lo + n + lane;
          my_page = 0;
          if (bl < blk_hi) {
            const int pg = (lo_al + (bl << 4)) >> p.page_shift;
            my_page = pg < p.max_pages ? bt[pg * p.bt_s1] : -1;
            if constexpr (kFp8) {
              if (my_page >= 0 && my_page < p.num_pages) {
                my_ks = p.k_scales[my_page * p.ks_s0 + g * p.ks_s1];
                my_vs = p.v_scales[my_page * p.vs_s0 + g * p.vs_s1];
              }
            }
          }
        }
        page = __shfl_sync(0xffffffffu, my_page, n & 31);
        if constexpr (kFp8) {
          const float ks = __shfl_sync(0xffffffffu, my_ks, n & 31), vs = __shfl_sync(0xffffffffu, my_vs, n & 31);
          if (lane == 0) ctl->scl[stg] = make_float2(ks, vs);
        }
        if (page < 0 || page >= p.num_pages) {   // never follow a bad table entry: the stage counts for nothing
          if (lane == 0) atomicCAS(p.status, 0, kErrBadEntry);
          page = 0; vlo = vhi = 0;
        }
        row0 = ((page * p.G + g) << p.page_shift) + (j0 & page_mask);
      } else {
        row0 = ring_start + j0;
        if (row0 >= p.T) row0 -= p.T;
        if (part == 1) vhi = min(vhi, jw - j0);                      // rows up to the end of the ring
        if (part == 2) { vlo = max(vlo, jw - j0); row0 -= p.T; }     // the rest, from row 0 on (box starts before it)
      }
      // One box per tile: the descriptor's third dimension walks the D / 64 column slabs of a
      // row (stride 128 bytes), so a box [64 elements x 16 rows x D / 64 slabs] lands as the
      // slab-major swizzled tile the consumers read.  Lane 0 fetches K, lane 1 fetches V.
      const uint32_t bar = ptx::smem_u32(&ctl->full[stg]);
      if (lane == 0) {
        ctl->meta[stg] = make_int4(j0, vlo, vhi, row0);
        ptx::mbar_arrive_expect_tx(bar, (uint32_t)Cfg::kStageBytes);
      }
      __syncwarp();
      if (lane < 2) {
        const uint32_t dst = ptx::smem_u32(ring + stg * Cfg::kStageBytes) + (lane ? Cfg::kTileBytes : 0);
        const CUtensorMap* map = lane ? &v_map : &k_map;
        if constexpr (kPaged) ptx::tma_load_5d_hint(dst, map, bar, 0, j0 & page_mask, 0, g, page, pol_stream);
        else ptx::tma_load_4d_hint(dst, map, bar, 0, row0, 0, b * p.G + g, pol_stream);
      }
      __syncwarp();
    }
  } else {
    // =============================== consumers ===============================
    // Q fragments of head gi: a0 = q[16 ks + 2c, +1], a2 = q[16 ks + 8 + 2c, +1]
    uint32_t qa[D / 16][2];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) qa[ks][0] = qa[ks][1] = 0u;
    if (kFp8 && gi < R) {
      // e4m3 pools: q as f16, in the byte order of the K tiles (4 consecutive d per thread and step)
      const int64_t qoff = b * p.q_s0 + (g * R + gi) * p.q_s1;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int64_t e = qoff + 16 * ks + 4 * c;
        qa[ks][0] = Mma<T>::pack(load_as_float(p.q, e, p.q_dtype), load_as_float(p.q, e + 1, p.q_dtype));
        qa[ks][1] = Mma<T>::pack(load_as_float(p.q, e + 2, p.q_dtype), load_as_float(p.q, e + 3, p.q_dtype));
      }
    } else if (gi < R) {
      const int h = g * R + gi;
      const int64_t qoff = b * p.q_s0 + h * p.q_s1;
      if (p.q_dtype == ElemTraits<T>::kDtype && ((reinterpret_cast<uintptr_t>((const T*)p.q + qoff) & 3) == 0)) {
        const uint32_t* qw = reinterpret_cast<const uint32_t*>((const T*)p.q + qoff);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) { qa[ks][0] = qw[8 * ks + c]; qa[ks][1] = qw[8 * ks + 4 + c]; }
      } else {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const int64_t e = qoff + 16 * ks + 2 * c;
          qa[ks][0] = Mma<T>::pack(load_as_float(p.q, e, p.q_dtype), load_as_float(p.q, e + 1, p.q_dtype));
          qa[ks][1] = Mma<T>::pack(load_as_float(p.q, e + 8, p.q_dtype), load_as_float(p.q, e + 9, p.q_dtype));
        }
      }
    }
#pragma unroll
    for (int i = 0; i < D / 16; ++i) { acc.oacc[i][0] = acc.oacc[i][1] = acc.oacc[i][2] = acc.oacc[i][3] = 0.f; }
    acc.m_run = -INFINITY;
    acc.l_run = 0.f;

    for (;;) {
      int n = 0;
      if (lane == 0) n = atomicAdd(&ctl->next_stage, 1);
      n = __shfl_sync(0xffffffffu, n, 0);
      if (n >= n_stages) break;
      const int stg = n % kSt, use = n / kSt;
      if (__any_sync(0xffffffffu, ctl->fail != 0)) break;
      {
        // A parity wait can only tell the current phase from the one before.  Warps claim
        // stages out of step with each other, so first make sure that the slot's previous use
        // has been consumed (by whichever warp had it): then the barrier is in this use's phase
        // or just past it, never one behind.
        bool ok = true;
        if (ctl->done[stg] < use) {
          const long long t0 = clock64();
          while (ctl->done[stg] < use) {
            if (clock64() - t0 > ptx::kWaitLimitCycles) { ok = false; break; }
          }
        }
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) { atomicCAS(p.status, 0, kErrStageOrder); ctl->fail = 1; }
          break;
        }
        ok = ptx::mbar_wait(ptx::smem_u32(&ctl->full[stg]), (uint32_t)use & 1u);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) { atomicCAS(p.status, 0, kErrStageFull); ctl->fail = 1; }
          break;
        }
      }
      const int4 meta = ctl->meta[stg];
      uint8_t* kt = ring + stg * Cfg::kStageBytes;
      uint8_t* vt = kt + Cfg::kTileBytes;
      if (!kFp8 && pnew >= 0 && pnew - meta.x >= meta.y && pnew - meta.x < meta.z) {
        // the appended token lives in this stage: its K / V rows come from k_new / v_new (into
        // the tile, in place of whatever the cache held) and go to the cache for later steps
        const int rr = pnew - meta.x;
        const T* kn = (const T*)p.k_new + b * p.kn_s0 + g * p.kn_s1;
        const T* vn = (const T*)p.v_new + b * p.vn_s0 + g * p.vn_s1;
        int64_t crow = (int64_t)meta.w + rr;
        if constexpr (!kPaged) crow += ((int64_t)b * p.G + g) * p.T;
        // the row must lie inside the cache: a row outside it is reported and not written
        const int64_t cache_rows = kPaged ? ((int64_t)p.num_pages * p.G) << p.page_shift : (int64_t)p.B * p.G * p.T;
        const bool row_ok = rr >= 0 && rr < 16 && crow >= 0 && crow < cache_rows;
        if (!row_ok && lane == 0) atomicCAS(p.status, 0, kErrAppendRow);
        for (int ch = lane; row_ok && ch < D / 8; ch += 32) {
          const uint4 kv = *reinterpret_cast<const uint4*>(kn + 8 * ch);
          const uint4 vv = *reinterpret_cast<const uint4*>(vn + 8 * ch);
          *reinterpret_cast<uint4*>(kt + tile_off(rr, ch)) = kv;
          *reinterpret_cast<uint4*>(vt + tile_off(rr, ch)) = vv;
          *reinterpret_cast<uint4*>((T*)p.k_cache + crow * D + 8 * ch) = kv;
          *reinterpret_cast<uint4*>((T*)p.v_cache + crow * D + 8 * ch) = vv;
        }
        __syncwarp();
      }
      if (meta.z > meta.y) {
        if constexpr (kFp8) {
          const float2 sc = ctl->scl[stg];
          stage_step_fp8<D>(acc, qa, ptx::smem_u32(kt), ptx::smem_u32(vt), meta.y, meta.z, p.scale_log2 * sc.x, sc.y, lane);
        } else {
          stage_step<T, D>(acc, qa, ptx::smem_u32(kt), ptx::smem_u32(vt), meta.y, meta.z, p.scale_log2, lane);
        }
      }
      __syncwarp();
      if (lane == 0) {
        ctl->done[stg] = use + 1;
        ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[stg]));   // (a release: the count above is visible with it)
      }
    }
  }
  __syncthreads();   // every stage has been consumed: the ring is scratch from here on

  // ---- merge the warps ----
  constexpr int kPitch = D + 4;
  if (warp < kConsumers) {
    float l_run = acc.l_run;
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (c == 0) { ctl->sm_m[warp][gi] = acc.m_run; ctl->sm_l[warp][gi] = l_run; }
    float* so = sm_o + warp * 8 * kPitch;
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      // rows of accumulator i: 16-bit pools d = 16 i + gi and + 8; e4m3 pools d = 32 (i / 2) + 2 gi + i % 2 and + 16
      const int d = kFp8 ? 32 * (i >> 1) + 2 * gi + (i & 1) : 16 * i + gi;
      const int d2 = d + (kFp8 ? 16 : 8);
      so[(2 * c) * kPitch + d] = acc.oacc[i][0];
      so[(2 * c + 1) * kPitch + d] = acc.oacc[i][1];
      so[(2 * c) * kPitch + d2] = acc.oacc[i][2];
      so[(2 * c + 1) * kPitch + d2] = acc.oacc[i][3];
    }
  }
  __syncthreads();

  const bool exchange = p.sync != nullptr;
  // The warps' accumulators become the split's partial (or, with one split and no exchange,
  // the output row).  Every load of an iteration is asked for before the first use and nothing
  // branches: at two warps per scheduler a chain of dependent shared-memory loads is what this
  // costs.  V columns per thread: as wide as the partial buffer's alignment lets one store be.
  const bool to_o = p.num_splits == 1 && !exchange;
  auto merge_warps = [&](auto vc) {
    constexpr int V = decltype(vc)::value;
    for (int idx = tid; idx < R * (D / V); idx += kStreamThreads) {
      const int hh = idx / (D / V), d = V * (idx - hh * (D / V));
      float mw[kConsumers], lw[kConsumers], x[kConsumers][V];
#pragma unroll
      for (int w = 0; w < kConsumers; ++w) {
        mw[w] = ctl->sm_m[w][hh];
        lw[w] = ctl->sm_l[w][hh];
        const float* src = sm_o + (w * 8 + hh) * kPitch + d;
        if constexpr (V == 4) {
          const float4 t = *reinterpret_cast<const float4*>(src);
          x[w][0] = t.x; x[w][1] = t.y; x[w][2] = t.z; x[w][3] = t.w;
        } else if constexpr (V == 2) {
          const float2 t = *reinterpret_cast<const float2*>(src);
          x[w][0] = t.x; x[w][1] = t.y;
        } else {
          x[w][0] = src[0];
        }
      }
      float m = mw[0];
#pragma unroll
      for (int w = 1; w < kConsumers; ++w) m = fmaxf(m, mw[w]);
      float a[V], l = 0.f;
#pragma unroll
      for (int v = 0; v < V; ++v) a[v] = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumers; ++w) {
        const float sc = mw[w] == -INFINITY ? 0.f : exp2f(mw[w] - m);   // (a warp that saw no key holds zeros)
        l += lw[w] * sc;
#pragma unroll
        for (int v = 0; v < V; ++v) a[v] += x[w][v] * sc;
      }
      const int h = g * R + hh;
      if (to_o) {
#pragma unroll
        for (int v = 0; v < V; ++v)
          store_from_float(p.o, b * p.o_s0 + h * p.o_s1 + d + v, p.o_dtype, l > 0.f ? a[v] / l : 0.f);
        continue;
      }
      const int64_t off = split * p.po_s0 + b * p.po_s1 + h * p.po_s2 + d;
      if (p.po_dtype == G4B_F32) {
        float* dst = (float*)p.po + off;
        if constexpr (V == 4) *reinterpret_cast<float4*>(dst) = make_float4(a[0], a[1], a[2], a[3]);
        else if constexpr (V == 2) *reinterpret_cast<float2*>(dst) = make_float2(a[0], a[1]);
        else dst[0] = a[0];
      } else {
#pragma unroll
        for (int v = 0; v < V; ++v) store_from_float(p.po, off + v, p.po_dtype, a[v]);
      }
      if (d == 0) {
        p.pl[split * p.pl_s0 + b * p.pl_s1 + h * p.pl_s2] = l;
        p.pm[split * p.pm_s0 + b * p.pm_s1 + h * p.pm_s2] = m;
      }
    }
  };
  {
    const int64_t strides = p.po_s0 | p.po_s1 | p.po_s2;
    const uintptr_t base = (uintptr_t)p.po;
    const bool f32 = p.po_dtype == G4B_F32;
    if (to_o || !f32 || ((strides & 3) == 0 && (base & 15) == 0)) merge_warps(std::integral_constant<int, 4>{});
    else if ((strides & 1) == 0 && (base & 7) == 0) merge_warps(std::integral_constant<int, 2>{});
    else merge_warps(std::integral_constant<int, 1>{});
  }
  if (!exchange) return;   // the caller merges in a second launch

  // =============================== merge + exchange ===============================
  grid_arrive();
  constexpr int kSlices = D / kXCols;
  if (split >= kSlices) return;          // (the launch's first CTA, split 0, always merges)
  // a merging CTA: wait until every CTA of the launch has arrived (all are resident)
  const bool arrived = all_arrived();
  if (!arrived) return;

  const int S = p.num_splits;
  float4* s_red = reinterpret_cast<float4*>(ring);                              // [groups][pairs]: acc.x, acc.y, l, m
  float* x_own = reinterpret_cast<float*>(s_red + kStreamThreads);             // [R][kXWords]
  float* x_all = x_own + 8 * kXWords;                                           // [world][R][kXWords]
  const float* pof = (const float*)p.po;
  // threads = (group of splits) x (pair of columns of one head); R * 4 pairs, padded to 16 or 32
  const int pairs = R * (kXCols / 2);
  const int pad = pairs > 16 ? 32 : 16;
  const int n_grp = kStreamThreads / pad;
  const int pi = tid % pad, sg = tid / pad;
  const uint32_t epoch = ctl->epoch;
  const int par = (int)(epoch & 1u);
  for (int sl = split; sl < kSlices; sl += S) {
    // ---- this GPU's merged accumulator for columns [8 sl, 8 sl + 8) of the R heads ----
    // A thread merges every n_grp-th split of its column pair with a running maximum; the
    // (acc, l, m) of up to kJ splits are all asked for before the first is used, so that a merge
    // of 128 splits costs one trip to L2.
    constexpr int kJ = 16;
    float2 acc = make_float2(0.f, 0.f);
    float run_l = 0.f, run_m = -INFINITY;
    if (pi < pairs) {
      const int hh = pi / (kXCols / 2), d = sl * kXCols + 2 * (pi % (kXCols / 2));
      const int h = g * R + hh;
      const float* src = pof + b * p.po_s1 + h * p.po_s2 + d;
      const float* srcm = p.pm + b * p.pm_s1 + h * p.pm_s2;
      const float* srcl = p.pl + b * p.pl_s1 + h * p.pl_s2;
      for (int i0 = sg; i0 < S; i0 += kJ * n_grp) {
        float2 x[kJ];
        float mi[kJ], li[kJ];
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
          const int i = min(i0 + j * n_grp, S - 1);
          x[j] = __ldcg(reinterpret_cast<const float2*>(src + (int64_t)i * p.po_s0));
          mi[j] = __ldcg(srcm + (int64_t)i * p.pm_s0);
          li[j] = __ldcg(srcl + (int64_t)i * p.pl_s0);
        }
        float m_new = run_m;
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
          if (i0 + j * n_grp >= S) mi[j] = -INFINITY;
          m_new = fmaxf(m_new, mi[j]);
        }
        const float keep = run_m == -INFINITY ? 0.f : exp2f(run_m - m_new);
        acc.x *= keep; acc.y *= keep; run_l *= keep;
#pragma unroll
        for (int j = 0; j < kJ; ++j) {
          const float w = mi[j] == -INFINITY ? 0.f : exp2f(mi[j] - m_new);
          acc.x += x[j].x * w; acc.y += x[j].y * w;
          run_l += li[j] * w;
        }
        run_m = m_new;
      }
    }
    s_red[sg * pad + pi] = make_float4(acc.x, acc.y, run_l, run_m);
    __syncthreads();
    if (tid < pairs) {
      float4 v[8];                                  // n_grp is 4 or 8
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = s_red[min(q, n_grp - 1) * pad + tid];
      float m = -INFINITY;
#pragma unroll
      for (int q = 0; q < 8; ++q) m = fmaxf(m, v[q].w);
      float2 sum = make_float2(0.f, 0.f);
      float l = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float w = (q >= n_grp || v[q].w == -INFINITY) ? 0.f : exp2f(v[q].w - m);
        sum.x += v[q].x * w; sum.y += v[q].y * w; l += v[q].z * w;
      }
      const int hh = tid / (kXCols / 2), cp = tid % (kXCols / 2);
      x_own[hh * kXWords + 2 * cp] = sum.x;
      x_own[hh * kXWords + 2 * cp + 1] = sum.y;
      if (cp == 0) { x_own[hh * kXWords + kXCols] = l; x_own[hh * kXWords + kXCols + 1] = m; }
    }
    __syncthreads();
    // ---- push the piece to every GPU (own copy included) ----
    for (int idx = tid; idx < R * kXWords; idx += kStreamThreads) {
      const int hh = idx / kXWords, e = idx - hh * kXWords;
      const int64_t off = xword(p, D, par, p.rank, b * p.H + g * R + hh, sl) + e;
      const unsigned long long word = ((unsigned long long)epoch << 32) | __float_as_uint(x_own[idx]);
      for (int r = 0; r < p.world; ++r)
        if (r != p.rank) st_word_sys(p.xbuf[r] + off, word);
      x_all[(p.rank * R + hh) * kXWords + e] = x_own[idx];      // this GPU's own piece needs no trip
    }
    // ---- wait for every GPU's piece: a word has arrived once it carries this launch's count ----
    const long long t0 = clock64();
    const int n_pairs = p.world * R * (kXWords / 2);
    for (int base = tid; base < n_pairs; base += 4 * kStreamThreads) {
      const ulonglong2* src[4];
      bool have[4];
      int where[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int pr = base + j * kStreamThreads;
        have[j] = pr >= n_pairs;
        const int pc = min(pr, n_pairs - 1);
        const int r = pc / (R * (kXWords / 2)), rem = pc - r * (R * (kXWords / 2));
        const int hh = rem / (kXWords / 2), e = 2 * (rem - hh * (kXWords / 2));
        have[j] = have[j] || r == p.rank;
        where[j] = (r * R + hh) * kXWords + e;
        src[j] = reinterpret_cast<const ulonglong2*>(p.xbuf[p.rank] + xword(p, D, par, r, b * p.H + g * R + hh, sl) + e);
      }
      for (;;) {
        ulonglong2 w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (!have[j]) w[j] = ld_pair_sys(src[j]);
        bool all = true;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (have[j]) continue;
          if ((uint32_t)(w[j].x >> 32) == epoch && (uint32_t)(w[j].y >> 32) == epoch) {
            x_all[where[j]] = __uint_as_float((uint32_t)w[j].x);
            x_all[where[j] + 1] = __uint_as_float((uint32_t)w[j].y);
            have[j] = true;
          } else {
            all = false;
          }
        }
        if (all) break;
        if (ctl->fail || clock64() - t0 > kPeerWaitLimit) { atomicCAS(p.status, 0, kErrPeerWait); ctl->fail = 1; break; }
      }
    }
    __syncthreads();
    if (ctl->fail) break;
    // ---- final merge of the GPUs' pieces ----
    if (tid < R * kXCols) {
      const int hh = tid / kXCols, col = tid - hh * kXCols;
      float mm = -INFINITY;
      for (int r = 0; r < p.world; ++r) mm = fmaxf(mm, x_all[(r * R + hh) * kXWords + kXCols + 1]);
      float num = 0.f, den = 0.f;
      for (int r = 0; r < p.world; ++r) {
        const float* row = x_all + (r * R + hh) * kXWords;
        const float w = (row[kXCols + 1] == -INFINITY) ? 0.f : exp2f(row[kXCols + 1] - mm);
        num += row[col] * w;
        den += row[kXCols] * w;
      }
      store_from_float(p.o, b * p.o_s0 + (g * R + hh) * p.o_s1 + sl * kXCols + col, p.o_dtype, den > 0.f ? num / den : 0.f);
    }
    __syncthreads();
  }
}

template <typename T, int D, bool kPaged, bool kFp8 = false>
int launch_variant(const CUtensorMap& km, const CUtensorMap& vm, const StreamParams& p, dim3 grid, cudaStream_t st) {
  using Cfg = StreamCfg<D, kFp8>;
  constexpr int kSmem = Cfg::kRingBytes + (int)sizeof(Ctl<Cfg::kStages>);
  static bool attr_set[64] = {false};
  int dev = 0;
  G4B_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    G4B_CUDA_CHECK(cudaFuncSetAttribute(decode_stream_kernel<T, D, kPaged, kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    attr_set[dev] = true;
  }
  decode_stream_kernel<T, D, kPaged, kFp8><<<grid, kStreamThreads, kSmem, st>>>(km, vm, p);
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

template <typename T, int D>
int launch_layout(bool paged, const CUtensorMap& km, const CUtensorMap& vm, const StreamParams& p, dim3 grid, cudaStream_t st) {
  return paged ? launch_variant<T, D, true>(km, vm, p, grid, st) : launch_variant<T, D, false>(km, vm, p, grid, st);
}

template <typename T>
int launch_dim(int D, bool paged, const CUtensorMap& km, const CUtensorMap& vm, const StreamParams& p, dim3 grid, cudaStream_t st) {
  switch (D) {
    case 128: return launch_layout<T, 128>(paged, km, vm, p, grid, st);
    case 256: return launch_layout<T, 256>(paged, km, vm, p, grid, st);
    case 512: return launch_layout<T, 512>(paged, km, vm, p, grid, st);
  }
  return fail(G4B_ERR_UNSUPPORTED, "decode: head dim %d not supported (128, 256 or 512)", D);
}

// Device address of the grid counters on the current device (looked up once per device).
int step_sync_ptr(uint32_t** out) {
  constexpr int kMaxDev = 64;
  // Filled without a lock: threads that race on an entry all store the same address.
  static uint32_t* cache[kMaxDev] = {nullptr};
  int dev = 0;
  G4B_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDev) return fail(G4B_ERR_CUDA, "device index %d outside 0..%d", dev, kMaxDev - 1);
  if (cache[dev] == nullptr) {
    void* a = nullptr;
    G4B_CUDA_CHECK(cudaGetSymbolAddress(&a, g_step_sync));
    cache[dev] = (uint32_t*)a;
  }
  *out = cache[dev];
  return G4B_OK;
}

}  // namespace

bool decode_stream_supports(const G4bAttnArgs& a) {
  const int64_t D = a.q.shape[3];
  if (D != 128 && D != 256 && D != 512) return false;
  if (a.q.shape[1] / a.k_cache.shape[1] > 8) return false;
  if (a.block_tables.ptr != nullptr) return a.page_size >= 16;
  return a.k_cache.shape[2] >= 16;
}

// `step` == nullptr: plain decode (o for one split, partials otherwise).  Otherwise the decode
// step: merge in the launch, optional append and exchange.
int launch_decode_stream(const G4bAttnArgs& a, int num_splits, const G4bDecodeStepArgs* step, cudaStream_t st,
                         const G4bTensor* k_scales, const G4bTensor* v_scales) {
  const bool paged = a.block_tables.ptr != nullptr;
  const bool fp8 = k_scales != nullptr;
  const int64_t B = a.q.shape[0], H = a.q.shape[1], D = a.q.shape[3], G = a.k_cache.shape[1];
  StreamParams p{};
  p.q = a.q.ptr; p.o = a.o.ptr;
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
  p.B = (int)B; p.H = (int)H; p.G = (int)G;
  p.ctx_window = a.ctx_window_size; p.sliding_window = a.sliding_window; p.phase = a.phase;
  p.num_splits = num_splits;
  p.q_dtype = a.q.dtype; p.o_dtype = a.o.dtype; p.po_dtype = a.partial_o.dtype;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.world = 1;
  if (paged) {
    while ((1 << p.page_shift) < a.page_size) ++p.page_shift;
    p.num_pages = (int)a.k_cache.shape[0];
    p.max_pages = (int)a.block_tables.shape[1];
    if ((int64_t)p.num_pages * G * a.page_size > 0x7fffffffLL) return fail(G4B_ERR_TOO_LARGE, "decode: page pool beyond 2^31 rows");
  } else {
    p.T = (int)a.k_cache.shape[2];
  }
  if (fp8) {
    if (!paged || step != nullptr) return fail(G4B_ERR_UNSUPPORTED, "e4m3 caches: paged decode only");
    p.k_scales = (const float*)k_scales->ptr; p.v_scales = (const float*)v_scales->ptr;
    p.ks_s0 = k_scales->stride[0]; p.ks_s1 = k_scales->stride[1];
    p.vs_s0 = v_scales->stride[0]; p.vs_s1 = v_scales->stride[1];
  }
  const bool fused = step != nullptr;
  if (fused) {
    if (a.partial_o.dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "decode step: partial_o must be f32");
    if ((((uintptr_t)a.partial_o.ptr) & 7) || (a.partial_o.stride[0] | a.partial_o.stride[1] | a.partial_o.stride[2]) % 2 != 0)
      return fail(G4B_ERR_BAD_STRIDE, "decode step: partial_o rows must start on 8-byte boundaries");
    if (step->k_new.ptr != nullptr || step->v_new.ptr != nullptr) {
      const G4bTensor* nt[2] = {&step->k_new, &step->v_new};
      for (const G4bTensor* t : nt) {
        if (t->ptr == nullptr) return fail(G4B_ERR_BAD_ARG, "decode step: k_new and v_new must be given together");
        if (t->ndim != 4 || t->shape[0] != B || t->shape[1] != G || t->shape[2] != 1 || t->shape[3] != D)
          return fail(G4B_ERR_BAD_ARG, "decode step: k_new / v_new must be [B,G,1,D]");
        if (t->dtype != a.k_cache.dtype) return fail(G4B_ERR_BAD_DTYPE, "decode step: k_new / v_new must have the cache dtype");
        if (t->stride[3] != 1 || (((uintptr_t)t->ptr) & 15) || (t->stride[0] % 8) || (t->stride[1] % 8))
          return fail(G4B_ERR_BAD_STRIDE, "decode step: k_new / v_new rows must be contiguous and 16-byte aligned");
      }
      p.k_new = step->k_new.ptr; p.v_new = step->v_new.ptr;
      p.kn_s0 = step->k_new.stride[0]; p.kn_s1 = step->k_new.stride[1];
      p.vn_s0 = step->v_new.stride[0]; p.vn_s1 = step->v_new.stride[1];
      p.k_cache = a.k_cache.ptr; p.v_cache = a.v_cache.ptr;
    }
    // the exchange form: with peers, or (world == 1 with a state given) alone, pushing to itself
    if (step->world > 1 || (step->world == 1 && step->state != nullptr)) {
      if (step->world > 8 || step->rank < 0 || step->rank >= step->world) return fail(G4B_ERR_BAD_ARG, "decode step: bad world / rank");
      if (step->state == nullptr) return fail(G4B_ERR_BAD_ARG, "decode step: state is null");
      if (num_splits > kMaxResidentSplits) return fail(G4B_ERR_TOO_LARGE, "decode step with peers: at most %d splits", kMaxResidentSplits);
      const int64_t need = 2ll * step->world * B * H * (D / kXCols) * kXWords * 8;
      if (step->xbuf_bytes < need) return fail(G4B_ERR_BAD_ARG, "decode step: exchange buffers too small (need %lld bytes per rank)", (long long)need);
      for (int r = 0; r < step->world; ++r) {
        if (step->xbuf[r] == nullptr || (((uintptr_t)step->xbuf[r]) & 15))
          return fail(G4B_ERR_BAD_ARG, "decode step: exchange buffer of rank %d missing or not 16-byte aligned", r);
        p.xbuf[r] = (unsigned long long*)step->xbuf[r];
      }
      // a CTA that waits for a peer holds its SM slot: every CTA of the launch must be resident
      // at once on every GPU, or two GPUs could each wait for a group the other has not started
      int dev = 0, sms = 0;
      G4B_STOP_IF_VALIDATE_ONLY();
      G4B_CUDA_CHECK(cudaGetDevice(&dev));
      G4B_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      const int64_t resident = (int64_t)sms * (D >= 512 ? 1 : 2);
      if ((int64_t)num_splits * G * B > resident)
        return fail(G4B_ERR_TOO_LARGE, "decode step with peers: %lld CTAs do not fit the GPU at once (%lld); use fewer splits",
                    (long long)((int64_t)num_splits * G * B), (long long)resident);
      p.xstate = (uint32_t*)step->state; p.world = step->world; p.rank = step->rank;
    }
  }
  G4B_STOP_IF_VALIDATE_ONLY();
  if (p.xstate != nullptr) {
    int rc = step_sync_ptr(&p.sync);
    if (rc) return rc;
  }
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;
  if (B == 0) return G4B_OK;
  CUtensorMap km, vm;
  int rc;
  const int esz = fp8 ? 1 : 2;
  // A row of D elements is described as slabs of 128 bytes: dims (element in slab, row, slab,
  // ...), the slab stride (128 bytes) below the row stride, so that one box holds a whole tile.
  const uint64_t per_slab = 128 / esz;
  const uint64_t slabs = (uint64_t)D / per_slab;
  if (paged) {
    const uint64_t P = (uint64_t)a.k_cache.shape[2], NP = (uint64_t)a.k_cache.shape[0];
    const uint64_t dims[5] = {per_slab, P, slabs, (uint64_t)G, NP};
    const uint64_t strides[4] = {(uint64_t)D * esz, 128, P * D * esz, (uint64_t)G * P * D * esz};
    const uint32_t box[5] = {(uint32_t)per_slab, 16, (uint32_t)slabs, 1, 1};
    if ((rc = encode_map(&km, a.k_cache.dtype, 5, a.k_cache.ptr, dims, strides, box, "k pool"))) return rc;
    if ((rc = encode_map(&vm, a.v_cache.dtype, 5, a.v_cache.ptr, dims, strides, box, "v pool"))) return rc;
  } else {
    const uint64_t dims[4] = {64, (uint64_t)p.T, slabs, (uint64_t)(B * G)};
    const uint64_t strides[3] = {(uint64_t)D * esz, 64 * esz, (uint64_t)p.T * D * esz};
    const uint32_t box[4] = {64, 16, (uint32_t)slabs, 1};
    if ((rc = encode_map(&km, a.k_cache.dtype, 4, a.k_cache.ptr, dims, strides, box, "k_cache"))) return rc;
    if ((rc = encode_map(&vm, a.v_cache.dtype, 4, a.v_cache.ptr, dims, strides, box, "v_cache"))) return rc;
  }
  dim3 grid((unsigned)num_splits, (unsigned)G, (unsigned)B);
  if (fp8) {
    switch ((int)D) {
      case 128: return launch_variant<__half, 128, true, true>(km, vm, p, grid, st);
      case 256: return launch_variant<__half, 256, true, true>(km, vm, p, grid, st);
      case 512: return launch_variant<__half, 512, true, true>(km, vm, p, grid, st);
    }
    return fail(G4B_ERR_UNSUPPORTED, "decode: head dim %d not supported (128, 256 or 512)", (int)D);
  }
  if (a.k_cache.dtype == G4B_BF16) return launch_dim<__nv_bfloat16>((int)D, paged, km, vm, p, grid, st);
  if (a.k_cache.dtype == G4B_F16) return launch_dim<__half>((int)D, paged, km, vm, p, grid, st);
  return fail(G4B_ERR_BAD_DTYPE, "decode: KV cache must be f16 or bf16");
}

}  // namespace g4b
