// Flash-attention forward for Tq > 1 (prefill chunks), head dim 256 (and 128, on tiles whose
// upper half is the TMA's zero fill: the time of head dim 256), f16 / bf16, on the
// 5th-generation tensor cores: tcgen05.mma with accumulators in tensor memory, operands
// staged in shared memory by TMA, online softmax in registers.
//
// Replaces _attn_kernel / _attn_inner of the reference (g4b/kernels/fa2.py:37-136, 256-480)
// for the prefill phase: ring-buffer KV cache (fa2.py:52-55,75), GQA (fa2.py:337), causal
// and full stages (fa2.py:354-435), per-slot phase skip (fa2.py:333-335); adds the softmax
// scale and the per-query sliding window of scripts/reference_impl.py:437-443.
//
// A work item = 128 query rows of one query head.  The grid is persistent: one CTA (or, when
// the head counts allow it, one cluster of two CTAs that take two heads of one kv head and
// share every K / V tile through cta_group::2 MMAs) per SM walks a static list of items,
// heaviest first.  Ten warps:
//   warp 0      producer: TMA loads of Q (once per item) and of K / V chunks into a 5-slot ring
//   warp 1      one thread issues every tcgen05.mma; the warp owns the TMEM allocation
//   warps 2..9  softmax, two warpgroups: a thread owns query row r (TMEM lane r) for one
//               half of a tile's 128 keys, so row max / row sum need no shuffles, only one
//               shared-memory exchange with the partner warp; they also rescale O when a
//               maximum moved and write the output (each half of the head dim)
//
// TMEM (512 columns x 128 lanes x 32 bit):  O[128 x 256] f32 in columns 0..255,
// S0 / S1 [128 x 128] f32 in columns 256..383 / 384..511.  P (f16/bf16) overwrites the
// first 64 columns of its S buffer and is the A operand of the P.V product from TMEM.
//
// Per 128-key tile j:   S(j) = Q K(j)^T  (16 MMAs 128x128x16, A and B from smem, K-major)
//                        O  += P(j) V(j)  ( 8 MMAs 128x256x16, A from TMEM, B MN-major smem)
// issued in the order QK(0) QK(1) PV(0) QK(2) PV(1) ... so the tensor pipe works on
// QK(j+1) / PV(j-1) while the softmax warps turn S(j) into P(j).
//
// Shared memory: Q 64 KB (4 slabs of [128 rows x 64 d], 128-byte swizzle) + 5 x 32 KB ring.
// One-CTA form: a K chunk is half the head dim of a tile ([128 keys x 128 d], 2 slabs), a V
// chunk half the keys ([64 keys x 256 d], 4 slabs).  Pair form: each CTA stages half of every
// tile, K as its 64 keys x 256 d, V as 128 keys x its 128 head-dim columns.
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <cudaTypedefs.h>

namespace g4b {

namespace {

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 128;          // keys per S tile
constexpr int kHD = 256;          // head dim
constexpr int kStages = 5;          // 32 KB ring slots in shared memory
constexpr int kChunkBytes = 32768;
constexpr int kQBytes = kBM * kHD * 2;
constexpr int kThreads = 320;      // producer warp, MMA warp, 2 softmax warpgroups
constexpr int kXchgBytes = 2 * 2 * kBM * 4;   // row maxima: [tile parity][column half][row]
constexpr int kSmemBytes = kQBytes + kStages * kChunkBytes + 256 /*barriers*/ + kXchgBytes;

constexpr uint32_t kColO = 0, kColS0 = 256, kColS1 = 384;

enum : int32_t {
  kErrQFull = 0x301, kErrKvEmpty = 0x302, kErrKvFull = 0x303, kErrSFull = 0x304,
  kErrPFull = 0x305, kErrPvDone = 0x306, kErrSmemAlign = 0x307, kErrPair = 0x308, kErrBadPage = 0x309, kErrQEmpty = 0x30a, kErrOFree = 0x30b, kErrStageFree = 0x30c,
};

// Division of a non-negative 31-bit value by a launch constant as multiply-high + shift: the
// item geometry holds half a dozen divisions, each a ~100-cycle dependent chain in a warp
// that nothing overlaps with, paid by every role at every item switch.
struct FastDiv {
  uint32_t mul, shift, d;
  __host__ void set(uint32_t div) {
    d = div < 1 ? 1 : div;
    if (d == 1) { mul = 0; shift = 0; return; }
    uint32_t lg = 0;
    while ((1ull << lg) < d) ++lg;
    const uint32_t pw = 31 + lg;
    mul = (uint32_t)(((1ull << pw) + d - 1) / d);
    shift = pw - 32;
  }
  __device__ __forceinline__ int div(int x) const { return d == 1 ? x : (int)(__umulhi((uint32_t)x, mul) >> shift); }
  __device__ __forceinline__ int mod(int x) const { return x - div(x) * (int)d; }
};

struct PrefillParams {
  void* o;
  const void* k; const void* v;              // raw cache pointers (manual fallback loads)
  const int32_t* time_dim_sizes; const uint8_t* user_phase;
  const int32_t* block_tables;               // paged mode: [B, max_pages]; else null
  int64_t o_s0, o_s1, o_s2;
  int64_t time_stride, phase_stride, bt_s0, bt_s1;
  int page_shift, num_pages, max_pages;      // paged mode
  int B, H, G, Tq, T;
  int D;                                     // head dim in memory: 256, or 128 (the upper half of every tile is then zero fill)
  // split-KV for chunks that would leave most SMs idle: work items are (item, key range),
  // un-normalised (acc, l, m) go to the caller's partial buffers and a merge launch follows
  float* po; float* pl; float* pm;
  int64_t po_s[4], pl_s[4], pm_s[4];         // strides of s, b, h, t (elements; d stride 1)
  int n_splits;
  FastDiv by_splits;
  const float* q_f32;                        // q given as f32 (the engine's scratchpad type): converted on load
  int64_t q_s0, q_s1, q_s2;                  // its strides for b, h, t (elements)
  int n_q_tiles;                             // ceil(Tq / 128)
  FastDiv by_units, by_H, by_HperG, by_T;    // units per query tile, H, H / G, ring length
  int ctx_window, sliding_window, phase, causal;
  int o_dtype;
  float scale_log2;
  int32_t* status;
};

struct Barriers {
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_a[2];          // first quarter-pairs of P(j) written (keys 0..31 and 64..95)
  uint64_t p_b[2];          // the rest of P(j) written
  uint64_t pv_done;
  uint64_t q_empty;        // last Q.K^T of a work item done: the Q buffer may be refilled
  uint64_t o_free;         // the softmax warps have read O out of tensor memory
  uint64_t stage_free;     // the softmax warps are done with the ring slot they borrowed for the output
  uint64_t pair[4];        // one per softmax warp pair (64 arrivals): shared-memory exchanges
  uint32_t tmem_base;
  int32_t abort_flag;
};

__device__ __forceinline__ void record(int32_t* status, int32_t code) { atomicCAS(status, 0, code); }

// Geometry of one work item = 128 query rows of one head (fa2.py:52-64).  Ring mode counts
// keys from the oldest one the cache exposes (fa2.py:52-56).  A paged cache is addressed by
// absolute position: all `time` keys are addressable (so 128-key tiles start on page
// boundaries) and the exposed window is just another lower bound.  Items are ordered with
// the latest (heaviest) query tiles first; in a CTA pair the two CTAs take heads 2u and 2u+1.
// The slot's length and phase (geo_time, geo_active) come from G4B_ITEM_LOOP_HEAD, which reads
// them one item ahead: fetched at the item switch itself, their two dependent global loads
// held up the MMA issuer and the softmax warps for thousands of cycles per item.
#define G4B_ITEM_LOOP_PROLOGUE()                                                                     \
  int time_nx_ = 0;                                                                                   \
  bool act_nx_ = false;                                                                               \
  fetch_item(item_of_round(0), time_nx_, act_nx_)
#define G4B_ITEM_LOOP_HEAD(round)                                                                    \
  const int item = item_of_round(round);                                                              \
  const int geo_time = time_nx_;                                                                      \
  const bool geo_active = act_nx_;                                                                    \
  fetch_item(((round) + 1) * n_workers < n_items ? item_of_round((round) + 1) : -1, time_nx_, act_nx_)
#define G4B_ITEM_GEOMETRY(item)                                                                      \
  const int item_ = kSplit ? p.by_splits.div(item) : (item);                                          \
  const int split_ = kSplit ? (item) - item_ * p.n_splits : 0;                                        \
  const int level_ = p.by_units.div(item_);                                                           \
  const int unit_ = item_ - level_ * units_per_level;                                                 \
  const int q_tile = p.n_q_tiles - 1 - level_;                                                        \
  const int bh = kPair ? 2 * unit_ + (int)rank : unit_;                                               \
  const int b = p.by_H.div(bh), h = bh - b * p.H;                                                     \
  const int g = p.by_HperG.div(h);                                                                    \
  const int m0 = q_tile * kBM;                                                                        \
  const bool active = geo_active;                                                                     \
  const bool paged = p.block_tables != nullptr;                                                       \
  const int time = geo_time;                                                                          \
  const int window = paged ? time : min(time, p.ctx_window);                                          \
  const int win_lo = paged ? max(0, time - p.ctx_window) : 0;                                         \
  const int ring_start = paged ? 0 : p.by_T.mod(max(time - p.ctx_window, 0));                         \
  const int q_t_base = window - p.Tq; /* logical position of query row 0 */                           \
  const int rows_valid = min(kBM, p.Tq - m0);                                                         \
  const int qpos_min = q_t_base + m0;                                                                 \
  const int qpos_max = q_t_base + m0 + rows_valid - 1;                                                \
  const int key_hi = p.causal ? min(window, qpos_max + 1) : window;                                   \
  const int key_lo = p.sliding_window > 0 ? max(win_lo, qpos_min - p.sliding_window + 1) : win_lo;    \
  /* uniform over the item: some row may see fewer than 64 keys in all */                             \
  const bool few_keys = qpos_min - win_lo < 64 || (p.sliding_window > 0 && p.sliding_window < 64);    \
  const bool precise = PackT<T>::kSplitP && few_keys;                                                 \
  const int tile_lo_all_ = key_lo / kBN;                                                              \
  const int n_tiles_all_ = (active && key_hi > key_lo) ? (key_hi + kBN - 1) / kBN - tile_lo_all_ : 0; \
  /* this split's share of the item's key tiles */                                                    \
  const int tps_ = kSplit ? p.by_splits.div(n_tiles_all_ + p.n_splits - 1) : n_tiles_all_;            \
  const int tile_lo = tile_lo_all_ + split_ * tps_;                                                   \
  const int n_tiles = max(0, min(tps_, n_tiles_all_ - split_ * tps_));                                \
  (void)ring_start; (void)precise; (void)few_keys; (void)g; (void)h; (void)tile_lo; (void)qpos_max; (void)split_

// Where logical key `key` of this (slot, kv head) lives, or null if it is outside the
// context (ring buffer or page pool).
template <typename T>
struct KeySource {
  const T* base;            // ring: start of (b, g); paged: start of the pool
  const int32_t* bt;        // paged: block table row of slot b
  int64_t bt_s1;
  int ring_start, Trows;    // ring
  int G, g, page_shift, num_pages, max_pages;   // paged
  int window;               // keys [0, window) exist
  int D;                    // elements per row in memory
  bool paged;
  __device__ __forceinline__ const T* row(int key) const {
    if (key < 0 || key >= window) return nullptr;
    if (!paged) {
      int pr = ring_start + key;
      if (pr >= Trows) pr -= Trows;
      return base + (int64_t)pr * D;
    }
    const int pg = key >> page_shift;
    if (pg >= max_pages) return nullptr;
    const int page = bt[pg * bt_s1];
    if (page < 0 || page >= num_pages) return nullptr;
    return base + ((((int64_t)page * G + g) << page_shift) + (key & ((1 << page_shift) - 1))) * D;
  }
};

// Copies `nrows` rows of a chunk with ordinary loads, applying the 128-byte swizzle by hand;
// rows whose key is outside the context are written as zeros.  Used for the tile that crosses
// the end of the ring buffer and for V rows past the context (which may hold anything, and
// 0 x NaN would poison the accumulator).
//   slab_rows: rows per slab (128 for K chunks, 64 for V chunks); d0: first head-dim element;
//   nslabs: 64-element slabs in the chunk.
template <typename T>
__device__ __forceinline__ void manual_chunk(uint8_t* dst, const KeySource<T>& src, int key0, int nrows, int d0,
                                             int nslabs, int slab_rows, int lane) {
  const int chunks_per_row = nslabs * 8;   // 16-byte pieces per row
  for (int idx = lane; idx < nrows * chunks_per_row; idx += 32) {
    const int r = idx / chunks_per_row, ch = idx % chunks_per_row;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    const T* rp = src.row(key0 + r);
    if (rp != nullptr && d0 + ch * 8 < src.D) val = *reinterpret_cast<const uint4*>(rp + d0 + ch * 8);   // (columns past the head dim: zero, like the TMA fill)
    const int slab = ch >> 3, c16 = ch & 7;
    uint8_t* p = dst + slab * (slab_rows * 128) + r * 128 + ((c16 ^ (r & 7)) << 4);
    *reinterpret_cast<uint4*>(p) = val;
  }
}

template <typename T> struct PackT;
template <> struct PackT<__nv_bfloat16> {
  static constexpr uint32_t kFmt = 1;
  // 8 significant bits: rows that see only a few keys get their probabilities as a
  // (rounded + residue) pair, multiplied by two MMAs
  static constexpr bool kSplitP = true;
  __device__ static __forceinline__ float lo_val(uint32_t v) { return __uint_as_float(v << 16); }
  __device__ static __forceinline__ float hi_val(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
  // sum of the two rounded values a packed register holds
  __device__ static __forceinline__ float sum2(uint32_t v) {
    return __uint_as_float(v << 16) + __uint_as_float(v & 0xffff0000u);
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
};
template <> struct PackT<__half> {
  static constexpr uint32_t kFmt = 0;
  static constexpr bool kSplitP = false;
  __device__ static __forceinline__ float lo_val(uint32_t v) { return __low2float(*reinterpret_cast<const __half2*>(&v)); }
  __device__ static __forceinline__ float hi_val(uint32_t v) { return __high2float(*reinterpret_cast<const __half2*>(&v)); }
  __device__ static __forceinline__ float sum2(uint32_t v) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    return f.x + f.y;
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
};

// kPair = false: one CTA per 128 query rows (cta_group::1).
// kPair = true : a cluster of two CTAs works on two query heads of the same kv head at the
//   same query tile (rows 0..127 = the even head in CTA 0, rows 128..255 = the odd head in
//   CTA 1) with cta_group::2 MMAs issued by CTA 0.  Both heads read the same K/V tiles, and
//   each CTA stages only half of every tile (K: half the keys, V: half the head dim), so the
//   ring covers twice the time and Q.K^T reads 96 instead of 128 bytes of shared memory per
//   cycle -- the two things that starve the single-CTA form.
template <typename T, bool kPair, bool kStageOut, bool kShortItems, bool kSplit, bool kNarrow>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
               const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap o_map, PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // head dim in memory: 256, or (kNarrow) 128 -- the tiles stay 256 wide, their upper half is
  // the TMA's zero fill and the accumulator's upper half is never stored
  constexpr int kD = kNarrow ? 128 : kHD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // kStageOut: the epilogue turns the output block through shared memory to store whole
  // 128-byte row segments.  It borrows the ring slot of the item's last V chunk: that slot is
  // the last one the item frees and the one the producer refills last (with a chunk the next
  // item needs only for its second P.V product), so the producer just waits for stage_free
  // before that one refill and the ring keeps all five slots in the steady state.
  constexpr int kSt = kStages;
  const uint32_t rank = kPair ? ptx::cluster_ctarank() : 0u;   // 0 = the CTA that issues the MMAs
  const bool leader = rank == 0;

  // Persistent: a worker (a CTA, or a CTA pair) walks a static list of work items, so barrier
  // set-up, the tensor-memory allocation and the launch gap are paid once, and the producer
  // runs ahead into the next item while the current one drains.  Round r hands item
  // r * workers + w to worker w, alternating the direction so heavy and light items pair up.
  const int units_per_level = kPair ? (p.B * p.H) / 2 : p.B * p.H;   // (slot, head[s]) units per query tile
  const int n_items = p.n_q_tiles * units_per_level * (kSplit ? p.n_splits : 1);
  const int n_workers = kPair ? (int)gridDim.x / 2 : (int)gridDim.x;
  const int worker = kPair ? (int)blockIdx.x / 2 : (int)blockIdx.x;
  auto item_of_round = [&](int round) -> int {
    const int pos = (round & 1) ? n_workers - 1 - worker : worker;
    const int item = round * n_workers + pos;
    return item < n_items ? item : -1;
  };
  auto fetch_item = [&](int item, int& time_o, bool& act_o) {
    if (item < 0) { time_o = 0; act_o = false; return; }
    const int item_ = kSplit ? p.by_splits.div(item) : item;
    const int unit_ = p.by_units.mod(item_);
    const int b_ = p.by_H.div(kPair ? 2 * unit_ + (int)rank : unit_);
    act_o = p.user_phase == nullptr || p.user_phase[b_ * p.phase_stride] == (uint8_t)p.phase;
    time_o = p.time_dim_sizes[b_ * p.time_stride];
  };
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sRing = smem + kQBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kQBytes + kStages * kChunkBytes);
  float* xchg = reinterpret_cast<float*>(smem + kQBytes + kStages * kChunkBytes + 256);
  const uint32_t bar_q = ptx::smem_u32(&bars->q_full);
  const uint32_t bar_pv = ptx::smem_u32(&bars->pv_done);
  if (threadIdx.x == 0) {
    // In a pair, the barriers the MMA issuer waits on live in CTA 0 and count both CTAs.
    constexpr uint32_t kN = kPair ? 2u : 1u;
    ptx::mbar_init(bar_q, kN);
    for (int s = 0; s < kSt; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->kv_full[s]), kN);
      ptx::mbar_init(ptx::smem_u32(&bars->kv_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->s_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->p_a[s]), 8 * kN);   // one arrival per softmax warp
      ptx::mbar_init(ptx::smem_u32(&bars->p_b[s]), 8 * kN);
    }
    ptx::mbar_init(bar_pv, 1);
    ptx::mbar_init(ptx::smem_u32(&bars->q_empty), 1);
    ptx::mbar_init(ptx::smem_u32(&bars->o_free), 8 * kN);
    ptx::mbar_init(ptx::smem_u32(&bars->stage_free), 8);     // this CTA's softmax warps
    for (int s = 0; s < 4; ++s) ptx::mbar_init(ptx::smem_u32(&bars->pair[s]), 2);   // one arrival per warp of the pair
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&q_map);
    ptx::prefetch_tensormap(&k_map);
    ptx::prefetch_tensormap(&v_map);
    if constexpr (kStageOut) ptx::prefetch_tensormap(&o_map);
    // An earlier CTA gave up on a wait: drain the grid.  One thread reads so all agree (in a
    // pair: CTA 0 decides for both).  The swizzled tiles need the buffer on a 1024-byte
    // boundary: refuse to run otherwise.
    if (leader) {
      int32_t a = *reinterpret_cast<volatile int32_t*>(p.status);
      // only a wait of this kernel that ran out (0x3xx) drains it: a bad block-table entry that
      // an append, decode or earlier prefill launch reported must not turn later launches into
      // no-ops
      if ((a & 0xf00) != 0x300 || a == kErrBadPage) a = 0;
      if (a == 0 && (ptx::smem_u32(smem_raw) & 1023u) != 0) { record(p.status, kErrSmemAlign); a = kErrSmemAlign; }
      bars->abort_flag = a;
      if constexpr (kPair) ptx::st_cluster_u32(ptx::map_to_cta(ptx::smem_u32(&bars->abort_flag), 1), (uint32_t)a);
    }
  }
  if constexpr (kPair) ptx::cluster_sync_all(); else __syncthreads();
  if (*reinterpret_cast<volatile int32_t*>(&bars->abort_flag) != 0) return;

  if (warp == 1) {
    if constexpr (kPair) {
      ptx::tmem_alloc_pair(ptx::smem_u32(&bars->tmem_base), 512);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), 512);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  // where this CTA's arrivals for the MMA issuer go (CTA 0's copy of the barrier)
  auto issuer_bar = [&](uint64_t* local) -> uint32_t {
    const uint32_t a = ptx::smem_u32(local);
    if constexpr (kPair) return ptx::map_to_cta(a, 0);
    else return a;
  };
  // one arrival per warp: every lane has finished (and fenced) its own tensor-memory stores,
  // the warp converges, one lane signals
  auto arrive_issuer = [&](uint32_t bar) {
    __syncwarp();
    if (lane == 0) {
      // P lives in tensor memory (ordered by tcgen05.wait::st + tcgen05.fence above), so the
      // cross-CTA arrival needs no memory ordering of its own
      if constexpr (kPair) ptx::mbar_arrive_cluster_relaxed(bar);
      else ptx::mbar_arrive(bar);
    }
  };

  if (warp == 0) {
    // =============================== producer ===============================
    // K/V tiles are re-read by every query tile of 4 heads: keep them in L2; Q is read once
    const uint64_t pol_kv = ptx::policy_evict_last();
    const uint64_t pol_q = ptx::policy_evict_first();
    uint32_t cc = 0;   // chunk counter over the ring (runs on across work items)
    int n_done = 0;    // work items this worker has gone through
    bool ok = true;
    G4B_ITEM_LOOP_PROLOGUE();
    for (int round = 0; round * n_workers < n_items && ok; ++round) {
    G4B_ITEM_LOOP_HEAD(round);
    if (item < 0) continue;
    G4B_ITEM_GEOMETRY(item);
    if (n_tiles <= 0) continue;
    KeySource<T> ksrc, vsrc;
    ksrc.paged = paged; ksrc.window = window; ksrc.ring_start = ring_start; ksrc.Trows = p.T; ksrc.D = kD;
    ksrc.G = p.G; ksrc.g = g; ksrc.page_shift = p.page_shift; ksrc.num_pages = p.num_pages;
    ksrc.max_pages = p.max_pages; ksrc.bt = paged ? p.block_tables + b * p.bt_s0 : nullptr; ksrc.bt_s1 = p.bt_s1;
    ksrc.base = paged ? (const T*)p.k : (const T*)p.k + ((int64_t)b * p.G + g) * p.T * kD;
    vsrc = ksrc;
    vsrc.base = paged ? (const T*)p.v : (const T*)p.v + ((int64_t)b * p.G + g) * p.T * kD;
    const int bg = b * p.G + g;
    // The previous item's epilogue borrows the slot of its last V chunk (chunk cc - 1), which
    // chunk cc + 4 refills.  stage_free completes once per item, so it must also be waited for
    // before this item can complete it again: at the latest before this item's last chunk.
    bool stage_pending = kStageOut && n_done > 0;
    const uint32_t stage_cc = cc + (uint32_t)min(4, 2 * n_tiles - 1);
    auto wait_stage = [&]() -> bool {
      if (!stage_pending || cc != stage_cc) return true;
      stage_pending = false;
      int w = 1;
      if (lane == 0) w = ptx::mbar_wait(ptx::smem_u32(&bars->stage_free), (n_done - 1) & 1) ? 1 : 0;
      w = __shfl_sync(0xffffffffu, w, 0);
      if (!w) { if (lane == 0) record(p.status, kErrStageFree); ok = false; }
      return w != 0;
    };
    {
      // the Q buffer is free once the last Q.K^T of the previous item has run
      int w = 1;
      if (lane == 0 && n_done > 0) w = ptx::mbar_wait(ptx::smem_u32(&bars->q_empty), (n_done - 1) & 1) ? 1 : 0;
      w = __shfl_sync(0xffffffffu, w, 0);
      if (!w) { if (lane == 0) record(p.status, kErrQEmpty); ok = false; break; }
    }
    if (p.q_f32 != nullptr) {
      // f32 q: the warp reads one row (1 KB) per pass, rounds it to the cache type and writes
      // the four 128-byte-swizzled slabs the TMA load would have produced; rows past Tq are
      // zero like the out-of-bounds fill
      const float* q0 = p.q_f32 + b * p.q_s0 + h * p.q_s1;
      const int slab = lane >> 3, c16 = lane & 7;
#pragma unroll 4
      for (int r = 0; r < kBM; ++r) {
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (m0 + r < p.Tq && lane * 8 < kD) {
          const float4* src = reinterpret_cast<const float4*>(q0 + (int64_t)(m0 + r) * p.q_s2 + lane * 8);
          const float4 a = src[0], c = src[1];
          w = make_uint4(PackT<T>::pack(a.x, a.y), PackT<T>::pack(a.z, a.w), PackT<T>::pack(c.x, c.y), PackT<T>::pack(c.z, c.w));
        }
        *reinterpret_cast<uint4*>(sQ + slab * 16384 + r * 128 + ((c16 ^ (r & 7)) << 4)) = w;
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) ptx::mbar_arrive_cluster(issuer_bar(&bars->q_full));
        else ptx::mbar_arrive(bar_q);
      }
    } else if (lane == 0) {
      if constexpr (kPair) {
        const uint32_t qb = issuer_bar(&bars->q_full);
        ptx::mbar_arrive_expect_tx_cluster(qb, kQBytes);
        for (int s = 0; s < 4; ++s)
          ptx::tma_load_4d_pair(ptx::smem_u32(sQ + s * 16384), &q_map, qb, s * 64, m0, h, b, pol_q);
      } else {
        ptx::mbar_arrive_expect_tx(bar_q, kQBytes);
        for (int s = 0; s < 4; ++s)
          ptx::tma_load_4d_hint(ptx::smem_u32(sQ + s * 16384), &q_map, bar_q, s * 64, m0, h, b, pol_q);
      }
    }
    // lane 0 waits for the stage to drain; the outcome is shared so the warp stays converged
    auto wait_empty = [&](int st, uint32_t c) -> bool {
      int w = 1;
      if (lane == 0) w = ptx::mbar_wait(ptx::smem_u32(&bars->kv_empty[st]), ((c / kSt) & 1) ^ 1) ? 1 : 0;
      w = __shfl_sync(0xffffffffu, w, 0);
      if (!w) { if (lane == 0) record(p.status, kErrKvEmpty); ok = false; }
      return w != 0;
    };
    // Paged mode: page ids of the 16-key groups [key0, key0 + 16 n), one per lane; -1 marks a
    // group that must not be fetched by TMA (outside the table / the pool).
    auto page_ids = [&](int key0, int n) -> int {
      int id = -1;
      if (lane < n) {
        const int key = key0 + 16 * lane;
        const int pg = key >> p.page_shift;
        if (key < window && pg < p.max_pages) {
          id = ksrc.bt[pg * p.bt_s1];
          if (id < 0 || id >= p.num_pages) { record(p.status, kErrBadPage); id = -1; }
        }
      }
      return id;
    };
    const int page_mask = (1 << p.page_shift) - 1;
    // chunk order = MMA consumption order: K(0) K(1) V(0) K(2) V(1) ... K(n-1) V(n-2) V(n-1)
    auto load_k = [&](int j) {
      const int key0 = (tile_lo + j) * kBN;
      int pr0 = ring_start + key0;
      if (pr0 >= p.T) pr0 -= p.T;
      const int live = min(kBN, window - key0);          // keys of this tile inside the context
      bool manual;
      int my_page = -1;
      if (paged) {
        my_page = page_ids(key0, 8);
        // every 16-key group that holds live keys needs a page; K rows past the context are
        // masked later, so their groups may come from any valid page (page 0)
        const bool bad = lane < 8 && key0 + 16 * lane < window && my_page < 0;
        manual = __any_sync(0xffffffffu, bad);
        if (my_page < 0) my_page = 0;
      } else {
        manual = pr0 + live > p.T;                       // the tile crosses the end of the ring
      }
      for (int kc = 0; kc < 2 && ok; ++kc, ++cc) {
        const int st = cc % kSt;
        const uint32_t full = ptx::smem_u32(&bars->kv_full[st]);
        if (!wait_empty(st, cc)) break;
        uint8_t* dst = sRing + st * kChunkBytes;
        if (!manual) {
          if (lane == 0) ptx::mbar_arrive_expect_tx(full, kChunkBytes);
          __syncwarp();
          if (!paged) {
            if (lane == 0)
              for (int s = 0; s < 2; ++s)
                ptx::tma_load_3d_hint(ptx::smem_u32(dst + s * 16384), &k_map, full, kc * 128 + s * 64, pr0, bg, pol_kv);
          } else if (lane < 8) {
            // lane i fetches its own 16-key group: 2 slabs of [16 rows x 64 d]
            const int row = (key0 + 16 * lane) & page_mask;
            for (int s = 0; s < 2; ++s)
              ptx::tma_load_4d_hint(ptx::smem_u32(dst + s * 16384 + lane * 2048), &k_map, full, kc * 128 + s * 64, row,
                                    g, my_page, pol_kv);
          }
        } else {
          manual_chunk<T>(dst, ksrc, key0, kBN, kc * 128, 2, 128, lane);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(full);
        }
        __syncwarp();
      }
    };
    auto load_v = [&](int j) {
      const int key0t = (tile_lo + j) * kBN;
      for (int vc = 0; vc < 2 && ok; ++vc, ++cc) {
        const int key0 = key0t + vc * 64;
        int pr0 = ring_start + key0;
        if (pr0 >= p.T) pr0 -= p.T;
        const int live = min(64, window - key0);
        // rows past the context must read as zero; rows past the ring end must wrap
        bool manual = live < 64 || (!paged && pr0 + 64 > p.T);
        int my_page = -1;
        if (paged && !manual) {
          my_page = page_ids(key0, 4);
          manual = __any_sync(0xffffffffu, lane < 4 && my_page < 0);
        }
        const int st = cc % kSt;
        const uint32_t full = ptx::smem_u32(&bars->kv_full[st]);
        if (!wait_empty(st, cc)) break;
        uint8_t* dst = sRing + st * kChunkBytes;
        if (!manual) {
          if (lane == 0) ptx::mbar_arrive_expect_tx(full, kChunkBytes);
          __syncwarp();
          if (!paged) {
            if (lane == 0)
              for (int s = 0; s < 4; ++s)
                ptx::tma_load_3d_hint(ptx::smem_u32(dst + s * 8192), &v_map, full, s * 64, pr0, bg, pol_kv);
          } else if (lane < 4) {
            const int row = (key0 + 16 * lane) & page_mask;
            for (int s = 0; s < 4; ++s)
              ptx::tma_load_4d_hint(ptx::smem_u32(dst + s * 8192 + lane * 2048), &v_map, full, s * 64, row, g, my_page,
                                    pol_kv);
          }
        } else {
          manual_chunk<T>(dst, vsrc, key0, 64, 0, 4, 64, lane);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(full);
        }
        __syncwarp();
      }
    };
    // ---- pair form: one 32 KB chunk per tile and operand.  K chunk = this CTA's 64 keys of
    // the tile x 256 d (4 slabs of [64 rows x 64 d]); V chunk = all 128 keys x this CTA's 128
    // head-dim columns (2 slabs of [128 rows x 64 d]).  Every CTA accounts for its own bytes
    // on CTA 0's barrier (2 arrivals per phase).
    auto load_k_pair = [&](int j) {
      const int key0 = (tile_lo + j) * kBN + 64 * (int)rank;
      int pr0 = ring_start + key0;
      if (pr0 >= p.T) pr0 -= p.T;
      const int live = min(64, window - key0);
      bool manual;
      int my_page = -1;
      if (paged) {
        my_page = page_ids(key0, 4);
        manual = __any_sync(0xffffffffu, lane < 4 && key0 + 16 * lane < window && my_page < 0);
        if (my_page < 0) my_page = 0;
      } else {
        manual = live > 0 && pr0 + live > p.T;
      }
      const int st = cc % kSt;
      const uint32_t full = issuer_bar(&bars->kv_full[st]);
      if (!wait_empty(st, cc) || !wait_stage()) return;
      uint8_t* dst = sRing + st * kChunkBytes;
      if (!manual) {
        if (lane == 0) ptx::mbar_arrive_expect_tx_cluster(full, kChunkBytes);
        __syncwarp();
        if (!paged) {
          if (lane == 0)
            for (int s = 0; s < 4; ++s)
              ptx::tma_load_3d_pair(ptx::smem_u32(dst + s * 8192), &k_map, full, s * 64, pr0, bg, pol_kv);
        } else if (lane < 4) {
          const int row = (key0 + 16 * lane) & page_mask;
          for (int s = 0; s < 4; ++s)
            ptx::tma_load_4d_pair(ptx::smem_u32(dst + s * 8192 + lane * 2048), &k_map, full, s * 64, row, g, my_page,
                                  pol_kv);
        }
      } else {
        manual_chunk<T>(dst, ksrc, key0, 64, 0, 4, 64, lane);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(full);
      }
      __syncwarp();
      ++cc;
    };
    auto load_v_pair = [&](int j) {
      const int key0 = (tile_lo + j) * kBN;
      const int d0 = 128 * (int)rank;
      int pr0 = ring_start + key0;
      if (pr0 >= p.T) pr0 -= p.T;
      const int live = min(kBN, window - key0);
      bool manual = live < kBN || (!paged && pr0 + kBN > p.T);
      int my_page = -1;
      if (paged && !manual) {
        my_page = page_ids(key0, 8);
        manual = __any_sync(0xffffffffu, lane < 8 && my_page < 0);
      }
      const int st = cc % kSt;
      const uint32_t full = issuer_bar(&bars->kv_full[st]);
      if (!wait_empty(st, cc) || !wait_stage()) return;
      uint8_t* dst = sRing + st * kChunkBytes;
      if (!manual) {
        if (lane == 0) ptx::mbar_arrive_expect_tx_cluster(full, kChunkBytes);
        __syncwarp();
        if (!paged) {
          if (lane == 0)
            for (int s = 0; s < 2; ++s)
              ptx::tma_load_3d_pair(ptx::smem_u32(dst + s * 16384), &v_map, full, d0 + s * 64, pr0, bg, pol_kv);
        } else if (lane < 8) {
          const int row = (key0 + 16 * lane) & page_mask;
          for (int s = 0; s < 2; ++s)
            ptx::tma_load_4d_pair(ptx::smem_u32(dst + s * 16384 + lane * 2048), &v_map, full, d0 + s * 64, row, g,
                                  my_page, pol_kv);
        }
      } else {
        manual_chunk<T>(dst, vsrc, key0, kBN, d0, 2, 128, lane);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(full);
      }
      __syncwarp();
      ++cc;
    };
    if constexpr (kPair) {
      load_k_pair(0);
      if (n_tiles > 1 && ok) load_k_pair(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        load_v_pair(j);
        if (ok && j + 2 < n_tiles) load_k_pair(j + 2);
      }
    } else {
      load_k(0);
      if (n_tiles > 1) load_k(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        load_v(j);
        if (j + 2 < n_tiles) load_k(j + 2);
      }
    }
    ++n_done;
    }   // work items
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    if constexpr (kPair) {
      // Pair form: only CTA 0 issues.  One MMA spans both CTAs: rows 0..127 of the 256-row
      // tile (A operand, accumulator, P) are CTA 0's, rows 128..255 CTA 1's; the B operand is
      // split between the two shared memories (K: keys 0..63 | 64..127, V: d 0..127 | 128..255)
      // at the same offsets.  Completion is signalled to the barriers of both CTAs.
      if (leader) {
        constexpr uint32_t idesc_qk = ptx::make_idesc_f16(PackT<T>::kFmt, 256, 128, 0, 0);
        constexpr uint32_t idesc_pv = ptx::make_idesc_f16(PackT<T>::kFmt, 256, 256, 0, 1);
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024 B, version 1, SWIZZLE_128B
        constexpr uint32_t kLoKMajor = 1u << 16;
        constexpr uint32_t kLoVMajor = (16384u >> 4) << 16;   // LBO: 64-wide slabs of 128 rows are 16 KB apart
        const uint32_t q_lo = (ptx::smem_u32(sQ) >> 4) | kLoKMajor;
        const uint32_t ring_lo = ptx::smem_u32(sRing) >> 4;
        auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {
          return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity));
        };
        auto commit_both = [&](uint64_t* local) {   // same barrier in CTA 0 and CTA 1
          const uint32_t a = ptx::smem_u32(local);
          ptx::tc_commit_pair(ptx::map_to_cta(a, 0));
          ptx::tc_commit_pair(ptx::map_to_cta(a, 1));
        };
        bool ok = true;
        uint32_t cc = 0;
        int tg = 0;       // tiles issued so far: S buffer and barrier phases run on across items
        int n_done = 0;
        G4B_ITEM_LOOP_PROLOGUE();
        for (int round = 0; round * n_workers < n_items && ok; ++round) {
        G4B_ITEM_LOOP_HEAD(round);
        if (item < 0) continue;
        G4B_ITEM_GEOMETRY(item);
        if (n_tiles <= 0) continue;
        ok = wait_all(bar_q, n_done & 1);
        if (!ok) { if (lane == 0) record(p.status, kErrQFull); break; }
        ptx::tc_fence_after();
        auto issue_qk = [&](int j) {
          const int t = tg + j;
          const uint32_t d_tmem = tmem + ((t & 1) ? kColS1 : kColS0);
          const int st = cc % kSt;
          if (!wait_all(ptx::smem_u32(&bars->kv_full[st]), (cc / kSt) & 1)) {
            if (lane == 0) record(p.status, kErrKvFull);
            ok = false; return;
          }
          ptx::tc_fence_after();
          const uint32_t k_lo = (ring_lo + st * (kChunkBytes >> 4)) | kLoKMajor;
          if (ptx::elect_one()) {
#pragma unroll
            for (int k16 = 0; k16 < 16; ++k16) {
              const uint32_t aoff = ((k16 >> 2) * 16384 + (k16 & 3) * 32) >> 4;   // Q: slabs of 128 rows
              const uint32_t boff = ((k16 >> 2) * 8192 + (k16 & 3) * 32) >> 4;    // K: slabs of 64 rows
              ptx::mma_ss_pair(d_tmem, ptx::desc64(q_lo + aoff, kDescHi), ptx::desc64(k_lo + boff, kDescHi), idesc_qk,
                               k16 != 0);
            }
            commit_both(&bars->kv_empty[st]);
            commit_both(&bars->s_full[t & 1]);
            if (j == n_tiles - 1) commit_both(&bars->q_empty);   // last use of this item's Q
          }
          __syncwarp();
          ++cc;
        };
        auto issue_pv = [&](int j) {
          const int st = cc % kSt;
          if (!wait_all(ptx::smem_u32(&bars->kv_full[st]), (cc / kSt) & 1)) {
            if (lane == 0) record(p.status, kErrKvFull);
            ok = false; return;
          }
          const int t = tg + j;
          const uint32_t v_lo = (ring_lo + st * (kChunkBytes >> 4)) | kLoVMajor;
          const uint32_t p_tmem = tmem + ((t & 1) ? kColS1 : kColS0);
          if (j == 0 && n_done > 0) {
            // the first product of an item overwrites O: the previous item's O must have been read
            if (!wait_all(ptx::smem_u32(&bars->o_free), (n_done - 1) & 1)) {
              if (lane == 0) record(p.status, kErrOFree);
              ok = false; return;
            }
            ptx::tc_fence_after();
          }
          for (int part = 0; part < 2 && ok; ++part) {
            const uint32_t bar = ptx::smem_u32(part == 0 ? &bars->p_a[t & 1] : &bars->p_b[t & 1]);
            if (!wait_all(bar, (t >> 1) & 1)) {
              if (lane == 0) record(p.status, kErrPFull);
              ok = false; return;
            }
            ptx::tc_fence_after();
            if (ptx::elect_one()) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                // part 0: keys 0..31 and 64..95 (k16 = 0,1,4,5); part 1: the rest
                const int k16 = (i >> 1) * 4 + part * 2 + (i & 1);
                const uint64_t vdesc = ptx::desc64(v_lo + (k16 * 2048 >> 4), kDescHi);
                ptx::mma_ts_pair(tmem + kColO, p_tmem + k16 * 8, vdesc, idesc_pv, (j | part | i) != 0);
                if (precise) ptx::mma_ts_pair(tmem + kColO, p_tmem + 64 + k16 * 8, vdesc, idesc_pv, 1u);
              }
              if (part == 1) {
                commit_both(&bars->kv_empty[st]);
                commit_both(&bars->pv_done);
              }
            }
            __syncwarp();
          }
          ++cc;
        };
        if (ok) issue_qk(0);
        if (ok && n_tiles > 1) issue_qk(1);
        for (int j = 0; j < n_tiles && ok; ++j) {
          issue_pv(j);
          if (ok && j + 2 < n_tiles) issue_qk(j + 2);
        }
        tg += n_tiles;
        ++n_done;
        }   // work items
      }
      __syncwarp();
    } else {
    // The whole warp walks the loop (uniform control flow keeps addresses and descriptors in
    // uniform registers); one elected lane issues each tcgen05 instruction.  Descriptors are
    // a constant upper word plus a lower word that is a base and a compile-time offset.
    constexpr uint32_t idesc_qk = ptx::make_idesc_f16(PackT<T>::kFmt, 128, 128, 0, 0);
    constexpr uint32_t idesc_pv = ptx::make_idesc_f16(PackT<T>::kFmt, 128, 256, 0, 1);
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024 B, version 1, SWIZZLE_128B
    constexpr uint32_t kLoKMajor = 1u << 16;                                // LBO field unused (1)
    constexpr uint32_t kLoVMajor = (8192u >> 4) << 16;                      // LBO 8192 B between 64-wide slabs
    const uint32_t q_lo = (ptx::smem_u32(sQ) >> 4) | kLoKMajor;
    const uint32_t ring_lo = ptx::smem_u32(sRing) >> 4;
    auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {
      return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity));
    };
    bool ok = true;
    uint32_t cc = 0;
    int tg = 0;       // tiles issued so far: S buffer and barrier phases run on across items
    int n_done = 0;
    G4B_ITEM_LOOP_PROLOGUE();
    for (int round = 0; round * n_workers < n_items && ok; ++round) {
    G4B_ITEM_LOOP_HEAD(round);
    if (item < 0) continue;
    G4B_ITEM_GEOMETRY(item);
    if (n_tiles <= 0) continue;
    ok = wait_all(bar_q, n_done & 1);
    if (!ok) { if (lane == 0) record(p.status, kErrQFull); break; }
    ptx::tc_fence_after();
    auto issue_qk = [&](int j) {
      const int t = tg + j;
      const uint32_t d_tmem = tmem + ((t & 1) ? kColS1 : kColS0);
      for (int kc = 0; kc < 2 && ok; ++kc, ++cc) {
        const int st = cc % kSt;
        if (!wait_all(ptx::smem_u32(&bars->kv_full[st]), (cc / kSt) & 1)) {
          if (lane == 0) record(p.status, kErrKvFull);
          ok = false; break;
        }
        ptx::tc_fence_after();
        const uint32_t k_lo = (ring_lo + st * (kChunkBytes >> 4)) | kLoKMajor;
        const uint32_t a_lo = q_lo + kc * (2 * 16384 >> 4);
        if (ptx::elect_one()) {
#pragma unroll
          for (int k16 = 0; k16 < 8; ++k16) {
            const uint32_t off = ((k16 >> 2) * 16384 + (k16 & 3) * 32) >> 4;
            ptx::mma_ss(d_tmem, ptx::desc64(a_lo + off, kDescHi), ptx::desc64(k_lo + off, kDescHi), idesc_qk,
                        (kc | k16) != 0);
          }
          ptx::tc_commit(ptx::smem_u32(&bars->kv_empty[st]));
        }
        __syncwarp();
      }
      if (ok && ptx::elect_one()) {
        ptx::tc_commit(ptx::smem_u32(&bars->s_full[t & 1]));
        if (j == n_tiles - 1) ptx::tc_commit(ptx::smem_u32(&bars->q_empty));   // last use of this item's Q
      }
      __syncwarp();
    };
    auto issue_pv = [&](int j) {
      // both V chunks first (they landed long ago), then P in the order the softmax warps
      // finish it: keys 0..31 and 64..95, then 32..63 and 96..127
      uint32_t v_lo[2];
      int st2[2];
      for (int vc = 0; vc < 2 && ok; ++vc, ++cc) {
        st2[vc] = cc % kSt;
        if (!wait_all(ptx::smem_u32(&bars->kv_full[st2[vc]]), (cc / kSt) & 1)) {
          if (lane == 0) record(p.status, kErrKvFull);
          ok = false; return;
        }
        v_lo[vc] = (ring_lo + st2[vc] * (kChunkBytes >> 4)) | kLoVMajor;
      }
      const int t = tg + j;
      const uint32_t p_tmem = tmem + ((t & 1) ? kColS1 : kColS0);
      if (j == 0 && n_done > 0) {
        // the first product of an item overwrites O: the previous item's O must have been read
        if (!wait_all(ptx::smem_u32(&bars->o_free), (n_done - 1) & 1)) {
          if (lane == 0) record(p.status, kErrOFree);
          ok = false; return;
        }
        ptx::tc_fence_after();
      }
      for (int part = 0; part < 2 && ok; ++part) {
        const uint32_t bar = ptx::smem_u32(part == 0 ? &bars->p_a[t & 1] : &bars->p_b[t & 1]);
        if (!wait_all(bar, (t >> 1) & 1)) {
          if (lane == 0) record(p.status, kErrPFull);
          ok = false; return;
        }
        ptx::tc_fence_after();
        if (ptx::elect_one()) {
#pragma unroll
          for (int vc = 0; vc < 2; ++vc) {
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              const int k16 = part * 2 + kk;
              // 16 keys = 8 packed columns of P; 16 rows of every V slab = 2048 bytes
              const uint64_t vdesc = ptx::desc64(v_lo[vc] + (k16 * 2048 >> 4), kDescHi);
              ptx::mma_ts(tmem + kColO, p_tmem + vc * 32 + k16 * 8, vdesc, idesc_pv, (j | part | vc | kk) != 0);
              if (precise)   // residue of the probabilities, in the upper half of the S buffer
                ptx::mma_ts(tmem + kColO, p_tmem + 64 + vc * 32 + k16 * 8, vdesc, idesc_pv, 1u);
            }
          }
          if (part == 1) {
            ptx::tc_commit(ptx::smem_u32(&bars->kv_empty[st2[0]]));
            ptx::tc_commit(ptx::smem_u32(&bars->kv_empty[st2[1]]));
            ptx::tc_commit(bar_pv);
          }
        }
        __syncwarp();
      }
    };
    if (ok) issue_qk(0);
    if (ok && n_tiles > 1) issue_qk(1);
    for (int j = 0; j < n_tiles && ok; ++j) {
      issue_pv(j);
      if (ok && j + 2 < n_tiles) issue_qk(j + 2);
    }
    tg += n_tiles;
    ++n_done;
    }   // work items
    __syncwarp();
    }
  } else {
    // =============================== softmax / epilogue ===============================
    // Two warpgroups share every row: warps 2..5 own the first 64 keys of a tile (and O
    // columns 0..127), warps 6..9 the other 64 (O columns 128..255).  A warp and its partner
    // (warp + 4, same TMEM lanes) trade row maxima through shared memory.
    const int half = (warp - 2) >> 2;
    const int lane_base = (warp & 3) * 32;
    const int r = lane_base + lane;                       // query row = TMEM lane
    const uint32_t trow = tmem + ((uint32_t)lane_base << 16);
    const uint32_t pair_bar = ptx::smem_u32(&bars->pair[warp & 3]);   // barrier of the warp pair
    uint32_t pair_phase = 0;
    // bounded rendezvous of the two warps that share these rows (a named barrier would have
    // no time limit); false when the partner never arrived
    auto pair_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(pair_bar);
      const bool w = __all_sync(0xffffffffu, ptx::mbar_wait(pair_bar, pair_phase & 1));
      ++pair_phase;
      return w;
    };
    bool ok = true;
    int tg = 0;       // tiles seen so far: S buffer and barrier phases run on across items
    int n_done = 0;
    // The ring slot borrowed for the last item's output goes back to the producer once the copy
    // engine has read the boxes out of it.  Called a tile into the next item (the producer needs
    // the slot for that item's fifth chunk at the earliest, or for its second if it has one
    // tile), when the read has long ended, instead of waiting for it in the epilogue.  (Giving
    // the slot back before the first tile instead cost 1.5 % on long items: the wait sits in
    // front of the tile that the tensor pipe is waiting for.)
    // The reference maximum a row ended the last item with is the first guess for
    // the same row of the next one (another head or query tile of similar scores).  A guess
    // at most 2^8 below or 2^4 above the first maximum the row really sees is kept -- any
    // reference in that range is as good as the maximum itself -- so the first tile of an item can take the
    // optimistic path too instead of waiting for the partner's maximum before the first exp.
    float m_carry = -INFINITY;
    bool stage_held = false;
    auto release_stage = [&]() {
      if (!stage_held) return;
      stage_held = false;
      if (lane == 0) {
        ptx::bulk_wait_read_all();
        ptx::mbar_arrive(ptx::smem_u32(&bars->stage_free));
      }
      __syncwarp();
    };
    G4B_ITEM_LOOP_PROLOGUE();
    for (int round = 0; round * n_workers < n_items && ok; ++round) {
    G4B_ITEM_LOOP_HEAD(round);
    if (item < 0) continue;
    G4B_ITEM_GEOMETRY(item);
    if (n_tiles <= 0) {
      release_stage();
      if constexpr (kSplit) {
        // an empty key range: the merge skips a partial with m = -inf, l = 0 (fa2.py:466-472)
        if (active && half == 0 && r < rows_valid) {
          p.pl[split_ * p.pl_s[0] + b * p.pl_s[1] + h * p.pl_s[2] + (int64_t)(m0 + r) * p.pl_s[3]] = 0.f;
          p.pm[split_ * p.pm_s[0] + b * p.pm_s[1] + h * p.pm_s[2] + (int64_t)(m0 + r) * p.pm_s[3]] = -INFINITY;
        }
        continue;
      }
      // no visible key for any row of this tile: the output rows are defined as zero
      if (active && half == 0 && r < rows_valid) {
        const int64_t off = b * p.o_s0 + h * p.o_s1 + (int64_t)(m0 + r) * p.o_s2;
        for (int d = 0; d < kD; ++d) {
          if (p.o_dtype == G4B_F32) ((float*)p.o)[off + d] = 0.f;
          else ((uint16_t*)p.o)[off + d] = 0;
        }
      }
      continue;
    }
    const int qpos = q_t_base + m0 + r;
    const int hi_r = p.causal ? min(window, qpos + 1) : window;
    const int lo_r = p.sliding_window > 0 ? max(win_lo, qpos - p.sliding_window + 1) : win_lo;
    float m_used = !few_keys ? m_carry : -INFINITY;   // reference maximum the accumulated O and l are scaled by
    bool anchored = false;      // m_used has been checked against a key this row sees
    float l_run = 0.f;          // this thread's half of the row sum

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int t = tg + j;
      const uint32_t s_col = (t & 1) ? kColS1 : kColS0;
      if (j == 1) release_stage();
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&bars->s_full[t & 1]), (t >> 1) & 1))) {
        record(p.status, kErrSFull); ok = false; break;
      }
      ptx::tc_fence_after();
      const int kbase = (tile_lo + j) * kBN;
      // warp-uniform: does any row of this CTA need element masks in this tile?
      const bool need_mask = (p.causal && kbase + kBN - 1 > qpos_min) || (kbase + kBN > window) ||
                             (kbase < key_lo) ||
                             (p.sliding_window > 0 && kbase < qpos_max - p.sliding_window + 1);
      uint32_t sraw[2][32];
      ptx::tmem_ld32(trow + s_col + half * 64, sraw[0]);
      ptx::tmem_ld32(trow + s_col + half * 64 + 32, sraw[1]);
      ptx::tc_wait_ld();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
        // the keys this row sees are one range [nlo, nhi) of the thread's 64: as one bit per key,
        // so that an element costs a bit test and a select instead of two compares and a select
        const int nlo = lo_r - kbase - half * 64, nhi = hi_r - kbase - half * 64;
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          const int lo = min(max(nlo - 32 * q2, 0), 32), hi = min(max(nhi - 32 * q2, 0), 32);
          const uint32_t below_hi = hi >= 32 ? 0xffffffffu : ((1u << hi) - 1u);
          const uint32_t below_lo = lo >= 32 ? 0xffffffffu : ((1u << lo) - 1u);
          const uint32_t bits = below_hi & ~below_lo;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = __uint_as_float(sraw[q2][i]);
            x = (bits & (1u << i)) ? x : -INFINITY;
            sraw[q2][i] = __float_as_uint(x);
            mx4[i & 3] = fmaxf(mx4[i & 3], x);
          }
        }
      } else {
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sraw[q2][i]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // publish the half-row maximum for the partner warp; collect the partner's later
      // exchange buffers alternate with every rendezvous of the pair (also across items), so a
      // write can never overtake the partner's read of the exchange before last
      float* xm = xchg + (pair_phase & 1) * (2 * kBM);
      xm[half * kBM + r] = mx;
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(pair_bar);

      const uint32_t bar_pa = issuer_bar(&bars->p_a[t & 1]);   // in a pair: CTA 0's barrier
      const uint32_t bar_pb = issuer_bar(&bars->p_b[t & 1]);
      uint32_t pk[32];
      // Optimistic path: the reference maximum rarely moves (it only has to stay within 2^8
      // of the true one), so start exponentiating against the current one while the maxima
      // are still being traded, and fall back only if the new maximum is out of range.
      bool fast = !few_keys && __all_sync(0xffffffffu, m_used != -INFINITY);
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      if (fast) {
        const float neg_m = -m_used;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[0][i]), p.scale_log2, neg_m));
          const float p1 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[0][i + 1]), p.scale_log2, neg_m));
          sum4[(i >> 1) & 3] += p0 + p1;
          pk[i >> 1] = PackT<T>::pack(p0, p1);
        }
      }
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(pair_bar, pair_phase & 1))) {
        record(p.status, kErrPair); ok = false; break;
      }
      ++pair_phase;
      mx = fmaxf(mx, xm[(half ^ 1) * kBM + r]);
      const float m_blk = mx * p.scale_log2;
      bool exceed = m_blk > m_used + 8.f;
      bool first_seen = false;
      if (!few_keys && !anchored && m_blk != -INFINITY) {
        // the row's first visible key: a guess that lies too far ABOVE is replaced as well
        // (nothing has been accumulated against it yet, so nothing is rescaled)
        first_seen = anchored = true;
        exceed = exceed || m_blk < m_used - 4.f;   // (f16 probabilities: keep them well above the subnormals)
      }
      if (fast && __any_sync(0xffffffffu, exceed)) fast = false;   // same outcome in the partner warp

      if (fast) {
        // first 32 keys of this half are final: let the P.V product start on them
        ptx::tmem_st16(trow + s_col + half * 32, pk);
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        arrive_issuer(bar_pa);
        const float neg_m = -m_used;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[1][i]), p.scale_log2, neg_m));
          const float p1 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[1][i + 1]), p.scale_log2, neg_m));
          sum4[(i >> 1) & 3] += p0 + p1;
          pk[16 + (i >> 1)] = PackT<T>::pack(p0, p1);
        }
        ptx::tmem_st16(trow + s_col + half * 32 + 16, pk + 16);
        l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        arrive_issuer(bar_pb);
        // keep the PV-done phase bookkeeping in step (no stall: PV(j-1) ended long ago)
        if (j > 0 && !__all_sync(0xffffffffu, ptx::mbar_wait(bar_pv, (t - 1) & 1))) {
          record(p.status, kErrPvDone); ok = false;
        }
        continue;
      }

      if (kShortItems && !few_keys) {
        // Variant for short work items (sliding windows), where the first tile is a fifth of
        // the item; with long items the extra code only disturbs the steady state (-2 %).
        // The reference maximum moves (first tile of an item, or a jump of more than 2^8: lazy
        // rescale -- p stays <= 256, exact enough in f32 sums and representable in f16/bf16).
        // Same two-part hand-over as above, after O and l have been rescaled.
        float alpha = 1.f;
        bool rescale = false;
        if (exceed) {
          rescale = (m_used != -INFINITY) && !first_seen;
          alpha = rescale ? ptx::ex2_approx(m_used - m_blk) : 1.f;
          m_used = m_blk;
        }
        l_run *= alpha;
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        sum4[0] = sum4[1] = sum4[2] = sum4[3] = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[0][i]), p.scale_log2, neg_m));
          const float p1 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[0][i + 1]), p.scale_log2, neg_m));
          sum4[(i >> 1) & 3] += p0 + p1;
          pk[i >> 1] = PackT<T>::pack(p0, p1);
        }
        // O may only be touched once PV(j-1) has drained, and must be rescaled before P.V(j)
        // adds to it, i.e. before any part of P is published
        if (j > 0) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar_pv, (t - 1) & 1))) { record(p.status, kErrPvDone); ok = false; break; }
          ptx::tc_fence_after();
          if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t ov[32];
              ptx::tmem_ld32(trow + kColO + half * 128 + c4 * 32, ov);
              ptx::tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              ptx::tmem_st32(trow + kColO + half * 128 + c4 * 32, ov);
            }
          }
        }
        ptx::tmem_st16(trow + s_col + half * 32, pk);
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        arrive_issuer(bar_pa);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[1][i]), p.scale_log2, neg_m));
          const float p1 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[1][i + 1]), p.scale_log2, neg_m));
          sum4[(i >> 1) & 3] += p0 + p1;
          pk[16 + (i >> 1)] = PackT<T>::pack(p0, p1);
        }
        ptx::tmem_st16(trow + s_col + half * 32 + 16, pk + 16);
        l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        arrive_issuer(bar_pb);
        continue;
      }

      // ---- precise path: items in which some row sees fewer than 64 keys ----
      float alpha = 1.f;
      bool rescale = false;
      if (exceed) {
        rescale = (m_used != -INFINITY) && !first_seen;
        alpha = rescale ? ptx::ex2_approx(m_used - m_blk) : 1.f;
        m_used = m_blk;
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      sum4[0] = sum4[1] = sum4[2] = sum4[3] = 0.f;
      uint32_t plo[32];
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[q2][i]), p.scale_log2, neg_m));
          const float p1 = ptx::ex2_approx(fmaf(__uint_as_float(sraw[q2][i + 1]), p.scale_log2, neg_m));
          const uint32_t packed = PackT<T>::pack(p0, p1);
          pk[q2 * 16 + (i >> 1)] = packed;
          if (few_keys) {
            // rows that see only a few keys: sum the ROUNDED probabilities the tensor core
            // multiplies, so numerator and denominator agree (exact for one visible key) ...
            sum4[(i >> 1) & 3] += PackT<T>::sum2(packed);
            if constexpr (PackT<T>::kSplitP) {
              // ... and give bf16 its rounding residue back through a second product
              const uint32_t lo = PackT<T>::pack(p0 - PackT<T>::lo_val(packed), p1 - PackT<T>::hi_val(packed));
              sum4[(i >> 1) & 3] += PackT<T>::sum2(lo);
              plo[q2 * 16 + (i >> 1)] = lo;
            }
          } else {
            sum4[(i >> 1) & 3] += p0 + p1;
          }
        }
      l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      ptx::tmem_st32(trow + s_col + half * 32, pk);
      if constexpr (PackT<T>::kSplitP) {
        if (few_keys) ptx::tmem_st32(trow + s_col + 64 + half * 32, plo);
      }
      // O may only be touched once PV(j-1) has drained
      if (j > 0) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar_pv, (t - 1) & 1))) { record(p.status, kErrPvDone); ok = false; }
        ptx::tc_fence_after();
        if (ok && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t ov[32];
            ptx::tmem_ld32(trow + kColO + half * 128 + c4 * 32, ov);
            ptx::tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            ptx::tmem_st32(trow + kColO + half * 128 + c4 * 32, ov);
          }
        }
      }
      ptx::tc_wait_st();
      ptx::tc_fence_before();
      arrive_issuer(bar_pa);
      arrive_issuer(bar_pb);
    }

    if (!few_keys && m_used != -INFINITY) m_carry = m_used;
    // ---- epilogue: O / l -> global ----
    release_stage();   // (an item of one tile: its only V chunk may be the one that waits for the slot)
    if (ok) {
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar_pv, (tg + n_tiles - 1) & 1))) { record(p.status, kErrPvDone); ok = false; }
      ptx::tc_fence_after();
    }
    // the row sum is the sum of both halves (both scaled by the same m_used)
    if (ok) {
      float* xl = xchg + (pair_phase & 1) * (2 * kBM);
      xl[half * kBM + r] = l_run;
      if (!pair_sync()) { record(p.status, kErrPair); ok = false; }
      l_run += xl[(half ^ 1) * kBM + r];
    }
    if (ok) {
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      // (head dim 128: the accumulator's columns 128..255 are zeros nobody stores)
      const bool row_ok = r < rows_valid && half * 128 < kD;
      const uint64_t pol_o = ptx::policy_evict_first();   // the output is not read again here
      const int64_t off = b * p.o_s0 + h * p.o_s1 + (int64_t)(m0 + r) * p.o_s2 + half * 128;
      if constexpr (kSplit) {
        // split-KV: the un-normalised accumulator, the row sum and the reference maximum (log2
        // units) in the reference's partial format (fa2.py:438-472)
        float* dst_row = p.po + split_ * p.po_s[0] + b * p.po_s[1] + h * p.po_s[2] + (int64_t)(m0 + r) * p.po_s[3] + half * 128;
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t ov[32];
          ptx::tmem_ld32(trow + kColO + half * 128 + c4 * 32, ov);
          ptx::tc_wait_ld();
          if (row_ok) {
            float4* dst = reinterpret_cast<float4*>(dst_row + c4 * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_float4(__uint_as_float(ov[4 * i]), __uint_as_float(ov[4 * i + 1]),
                                                             __uint_as_float(ov[4 * i + 2]), __uint_as_float(ov[4 * i + 3]));
          }
        }
        ptx::tc_fence_before();
        arrive_issuer(issuer_bar(&bars->o_free));
        if (row_ok && half == 0) {
          p.pl[split_ * p.pl_s[0] + b * p.pl_s[1] + h * p.pl_s[2] + (int64_t)(m0 + r) * p.pl_s[3]] = l_run;
          p.pm[split_ * p.pm_s[0] + b * p.pm_s[1] + h * p.pm_s[2] + (int64_t)(m0 + r) * p.pm_s[3]] = m_used;
        }
      } else if (p.o_dtype == G4B_F32) {
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t ov[32];
          ptx::tmem_ld32(trow + kColO + half * 128 + c4 * 32, ov);
          ptx::tc_wait_ld();
          if (row_ok) {
            float4* dst = reinterpret_cast<float4*>((float*)p.o + off + c4 * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              ptx::st_global_v4_hint(dst + i, make_uint4(__float_as_uint(__uint_as_float(ov[4 * i]) * inv_l),
                                                         __float_as_uint(__uint_as_float(ov[4 * i + 1]) * inv_l),
                                                         __float_as_uint(__uint_as_float(ov[4 * i + 2]) * inv_l),
                                                         __float_as_uint(__uint_as_float(ov[4 * i + 3]) * inv_l)), pol_o);
          }
        }
        ptx::tc_fence_before();
        arrive_issuer(issuer_bar(&bars->o_free));
      } else {
        if constexpr (kStageOut) {
          // A lane owns a row, and rows are kilobytes apart in memory: stored directly, every
          // 16-byte store touches its own line, and 64 KB of stores per item queue up in front
          // of the warps that should be exponentiating the next item's scores.  Instead the warp
          // writes its [32 rows x 64 columns] block into shared memory in the 128-byte-swizzled
          // layout of a TMA box (4 KB per warp, twice) and one lane hands it to the copy engine,
          // which stores whole rows while the warp moves on (rows past Tq are clipped by the
          // box).  The second half is pulled out of tensor memory while the engine reads the
          // first; the wait for the second, and the hand-back of the slot, are left to
          // release_stage() a tile later.
          // (2 chunks per tile in the pair form: the item's last V chunk is chunk 2 (tg + n_tiles) - 1)
          const int stage_slot = (2 * (tg + n_tiles) - 1) % kStages;
          uint8_t* stage = sRing + stage_slot * kChunkBytes + (warp - 2) * 4096;
#pragma unroll
          for (int cp = 0; cp < 2; ++cp) {
            uint32_t pk[2][16];
#pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
              uint32_t ov[32];
              ptx::tmem_ld32(trow + kColO + half * 128 + (2 * cp + c2) * 32, ov);
              ptx::tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i)
                pk[c2][i] = PackT<T>::pack(__uint_as_float(ov[2 * i]) * inv_l, __uint_as_float(ov[2 * i + 1]) * inv_l);
            }
            if (cp == 1) {
              // O is out of tensor memory: the next item's first P.V may overwrite it
              ptx::tc_fence_before();
              arrive_issuer(issuer_bar(&bars->o_free));
              // the first box must have been read out of the stage before it is overwritten
              if (lane == 0) ptx::bulk_wait_read_all();
              __syncwarp();
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint32_t* src = &pk[c >> 2][(c & 3) * 4];
              *reinterpret_cast<uint4*>(stage + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_uint4(src[0], src[1], src[2], src[3]);
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && lane_base < rows_valid && half * 128 < kD) {   // (a box wholly past Tq or the head dim is not issued at all)
              ptx::tma_store_4d_hint(&o_map, ptx::smem_u32(stage), half * 128 + cp * 64, m0 + lane_base, h, b, pol_o);
              ptx::bulk_commit();
            }
          }
          stage_held = true;
        } else {
        // pull this thread's 128 accumulator columns out (normalised and packed: 64 registers),
        // hand O back to the MMA issuer -- the next item's first P.V overwrites it -- then store
        uint32_t pk[4][16];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t ov[32];
          ptx::tmem_ld32(trow + kColO + half * 128 + c4 * 32, ov);
          ptx::tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            pk[c4][i] = PackT<T>::pack(__uint_as_float(ov[2 * i]) * inv_l, __uint_as_float(ov[2 * i + 1]) * inv_l);
        }
        ptx::tc_fence_before();
        arrive_issuer(issuer_bar(&bars->o_free));
        if (row_ok) {

#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint4* dst = reinterpret_cast<uint4*>((T*)p.o + off + c4 * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              ptx::st_global_v4_hint(dst + i, make_uint4(pk[c4][4 * i], pk[c4][4 * i + 1], pk[c4][4 * i + 2], pk[c4][4 * i + 3]),
                                     pol_o);
          }
        }
        }
      }
    }
    tg += n_tiles;
    ++n_done;
    }   // work items
    release_stage();
  }

  // ---- teardown: every thread arrives here, on success and after a failed wait ----
  if constexpr (kStageOut) {
    if (warp >= 2 && lane == 0) ptx::bulk_wait_all();   // the output boxes handed to the copy engine are stored
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kPair) {
    // CTA 0's MMAs read this CTA's shared and tensor memory: leave together
    ptx::cluster_sync_all();
    if (warp == 1) {
      ptx::tc_fence_after();
      ptx::tmem_dealloc_pair(tmem, 512);
    }
  } else if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------
// host side: tensor maps + launch
// ---------------------------------------------------------------------------------------
template <typename T, bool kPair, bool kStageOut, bool kShortItems, bool kSplit, bool kNarrow>
static int launch_variant(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const CUtensorMap& om,
                          const PrefillParams& p, dim3 grid, cudaStream_t st) {
  static bool attr_set[64] = {false};
  int dev = 0;
  G4B_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    G4B_CUDA_CHECK(cudaFuncSetAttribute(prefill_kernel<T, kPair, kStageOut, kShortItems, kSplit, kNarrow>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  G4B_CUDA_CHECK(cudaLaunchKernelEx(&cfg, prefill_kernel<T, kPair, kStageOut, kShortItems, kSplit, kNarrow>, qm, km, vm, om, p));
  return G4B_OK;
}

template <typename T, bool kNarrow>
static int launch_width(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const CUtensorMap& om,
                        const PrefillParams& p, dim3 grid, bool pair, bool stage_out, bool short_items, bool split,
                        cudaStream_t st) {
  if (split) {
    if (pair) return launch_variant<T, true, false, false, true, kNarrow>(qm, km, vm, om, p, grid, st);
    return launch_variant<T, false, false, false, true, kNarrow>(qm, km, vm, om, p, grid, st);
  }
  if (pair && stage_out && short_items) return launch_variant<T, true, true, true, false, kNarrow>(qm, km, vm, om, p, grid, st);
  if (pair && stage_out) return launch_variant<T, true, true, false, false, kNarrow>(qm, km, vm, om, p, grid, st);
  if (pair) return launch_variant<T, true, false, false, false, kNarrow>(qm, km, vm, om, p, grid, st);
  return launch_variant<T, false, false, false, false, kNarrow>(qm, km, vm, om, p, grid, st);
}

template <typename T>
static int launch_typed(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const CUtensorMap& om,
                        const PrefillParams& p, dim3 grid, bool pair, bool stage_out, bool short_items, bool split,
                        cudaStream_t st) {
  if (p.D == 128) return launch_width<T, true>(qm, km, vm, om, p, grid, pair, stage_out, short_items, split, st);
  return launch_width<T, false>(qm, km, vm, om, p, grid, pair, stage_out, short_items, split, st);
}

}  // namespace

int launch_prefill(const G4bAttnArgs& a, cudaStream_t st) {
  const bool paged = a.block_tables.ptr != nullptr;
  const bool q_f32 = a.q.dtype == G4B_F32;
  if (!q_f32 && a.q.dtype != a.k_cache.dtype)
    return fail(G4B_ERR_BAD_DTYPE, "prefill: q must have the cache dtype (f16 or bf16) or be f32");
  if (a.o.dtype != a.k_cache.dtype && a.o.dtype != G4B_F32)
    return fail(G4B_ERR_BAD_DTYPE, "prefill: o must have the cache dtype or be f32");
  const int64_t B = a.q.shape[0], H = a.q.shape[1], Tq = a.q.shape[2], D = a.q.shape[3];
  const int64_t G = a.k_cache.shape[1], T = a.k_cache.shape[2];
  if (B == 0 || Tq == 0) return G4B_OK;
  const int esz = 2;
  for (int i = 0; i < 3; ++i) {
    if ((a.q.stride[i] * (q_f32 ? 4 : esz)) % 16 != 0) return fail(G4B_ERR_BAD_STRIDE, "prefill: q strides must be multiples of 16 bytes");
  }
  if (((uintptr_t)a.q.ptr) & 15) return fail(G4B_ERR_BAD_STRIDE, "prefill: q must be 16-byte aligned");
  const int osz = dtype_size(a.o.dtype);
  for (int i = 0; i < 3; ++i)
    if ((a.o.stride[i] * osz) % 16 != 0) return fail(G4B_ERR_BAD_STRIDE, "prefill: o strides must be multiples of 16 bytes");
  if (((uintptr_t)a.o.ptr) & 15) return fail(G4B_ERR_BAD_STRIDE, "prefill: o must be 16-byte aligned");
  const int64_t n_q_tiles = (Tq + kBM - 1) / kBM;
  if (B * H * n_q_tiles > 0x7fffffffLL) return fail(G4B_ERR_UNSUPPORTED, "prefill: too many work items");

  // Two heads of one kv head per CTA pair when the head counts allow it.
  const bool pair = (H % 2 == 0) && ((H / G) % 2 == 0);
  G4B_STOP_IF_VALIDATE_ONLY();
  CUtensorMap qm, km, vm;
  int rc;
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)Tq, (uint64_t)H, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)a.q.stride[2] * esz, (uint64_t)a.q.stride[1] * esz, (uint64_t)a.q.stride[0] * esz};
    const uint32_t box[4] = {64, (uint32_t)kBM, 1, 1};
    if (!q_f32 && (rc = encode_map(&qm, a.q.dtype, 4, a.q.ptr, dims, strides, box, "q"))) return rc;
  }
  if (!paged) {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)T, (uint64_t)(B * G)};
    const uint64_t strides[2] = {(uint64_t)D * esz, (uint64_t)T * D * esz};
    // one CTA: K boxes of a whole tile (128 keys), V boxes of half a tile; a pair: K boxes of
    // this CTA's 64 keys, V boxes of all 128 keys (of this CTA's half of the head dim)
    const uint32_t boxk[3] = {64, pair ? 64u : (uint32_t)kBN, 1};
    const uint32_t boxv[3] = {64, pair ? (uint32_t)kBN : 64u, 1};
    if ((rc = encode_map(&km, a.k_cache.dtype, 3, a.k_cache.ptr, dims, strides, boxk, "k_cache"))) return rc;
    if ((rc = encode_map(&vm, a.v_cache.dtype, 3, a.v_cache.ptr, dims, strides, boxv, "v_cache"))) return rc;
  } else {
    // pool [num_pages, G, page, D]: one box = 16 rows of one (page, kv head), 64 elements wide
    const uint64_t P = (uint64_t)a.k_cache.shape[2], NP = (uint64_t)a.k_cache.shape[0];
    const uint64_t dims[4] = {(uint64_t)D, P, (uint64_t)G, NP};
    const uint64_t strides[3] = {(uint64_t)D * esz, P * D * esz, (uint64_t)G * P * D * esz};
    const uint32_t box[4] = {64, 16, 1, 1};
    if ((rc = encode_map(&km, a.k_cache.dtype, 4, a.k_cache.ptr, dims, strides, box, "k pool"))) return rc;
    if ((rc = encode_map(&vm, a.v_cache.dtype, 4, a.v_cache.ptr, dims, strides, box, "v pool"))) return rc;
  }
  PrefillParams p{};
  p.o = a.o.ptr; p.k = a.k_cache.ptr; p.v = a.v_cache.ptr;
  p.time_dim_sizes = (const int32_t*)a.time_dim_sizes.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr;
  p.o_s0 = a.o.stride[0]; p.o_s1 = a.o.stride[1]; p.o_s2 = a.o.stride[2];
  p.time_stride = a.time_dim_sizes.stride[0]; p.phase_stride = a.user_phase.stride[0];
  p.B = (int)B; p.H = (int)H; p.G = (int)G; p.Tq = (int)Tq; p.T = paged ? 1 : (int)T;
  p.D = (int)D;
  p.n_q_tiles = (int)n_q_tiles;
  p.by_units.set((uint32_t)(pair ? B * H / 2 : B * H));
  p.by_H.set((uint32_t)H);
  p.by_HperG.set((uint32_t)(H / G));
  p.by_T.set((uint32_t)(paged ? 1 : T));
  const bool stage_out = pair && a.o.dtype != G4B_F32;
  // tiles per work item, from what the host knows (context lengths live on the device)
  const int64_t est_tiles = a.sliding_window > 0 ? (a.sliding_window + 127) / 128 + 1 : (int64_t)a.ctx_window_size / 256 + 1;
  const bool short_items = est_tiles <= 12;
  if (paged) {
    p.block_tables = (const int32_t*)a.block_tables.ptr;
    p.bt_s0 = a.block_tables.stride[0]; p.bt_s1 = a.block_tables.stride[1];
    p.page_shift = 0;
    while ((1 << p.page_shift) < a.page_size) ++p.page_shift;
    p.num_pages = (int)a.k_cache.shape[0];
    p.max_pages = (int)a.block_tables.shape[1];
  }
  p.ctx_window = a.ctx_window_size; p.sliding_window = a.sliding_window; p.phase = a.phase;
  p.causal = a.stage == G4B_STAGE_CAUSAL;
  p.o_dtype = a.o.dtype;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;
  // persistent launch: one worker (CTA or CTA pair) per SM (pair of SMs), or fewer if there
  // are fewer work items
  static int sm_count[64] = {0};
  int dev = 0;
  G4B_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(G4B_ERR_CUDA, "device index out of range");
  if (sm_count[dev] == 0) G4B_CUDA_CHECK(cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
  const int64_t base_items = n_q_tiles * (pair ? (B * H) / 2 : B * H);
  int64_t workers = pair ? sm_count[dev] / 2 : sm_count[dev];
  if (workers < 1) workers = 1;
  // Split-KV: a chunk of a few hundred query rows is a handful of work items however long the
  // context is (B1 H16 Tq256 over 65536 keys: 16 CTA pairs busy for 512 tiles each, 58 idle).
  // With the caller's partial buffers at hand the key range of every item is cut into as many
  // pieces as it takes to occupy the workers, at least four tiles each; a merge launch follows.
  p.n_splits = 1;
  const bool have_partials = a.partial_o.ptr != nullptr && a.partial_l.ptr != nullptr && a.partial_m.ptr != nullptr;
  if (have_partials) {
    int64_t want = a.num_kv_splits > 0 ? a.num_kv_splits : (base_items * 2 <= workers ? workers / base_items : 1);
    const int64_t keys_bound = a.sliding_window > 0 ? a.sliding_window + kBM : a.ctx_window_size;
    const int64_t tiles_bound = (keys_bound + kBN - 1) / kBN;
    if (a.num_kv_splits <= 0 && want > tiles_bound / 4) want = tiles_bound / 4;
    if (want > a.partial_o.shape[0]) want = a.partial_o.shape[0];
    if (want > a.partial_l.shape[0]) want = a.partial_l.shape[0];
    if (want > a.partial_m.shape[0]) want = a.partial_m.shape[0];
    if (want > 1024) want = 1024;
    // buffers of another type (the engine's decode workspace is f16) are simply not used,
    // unless the caller asked for a split count
    const bool f32_partials = a.partial_o.dtype == G4B_F32 && a.partial_l.dtype == G4B_F32 && a.partial_m.dtype == G4B_F32;
    if (!f32_partials && a.num_kv_splits <= 0) want = 1;
    if (want > 1) {
      if (!f32_partials) return fail(G4B_ERR_BAD_DTYPE, "prefill: split-KV partials must be f32");
      if (a.partial_o.ndim != 5 || a.partial_l.ndim != 4 || a.partial_m.ndim != 4)
        return fail(G4B_ERR_BAD_ARG, "prefill: partial_o must be [S,B,H,Tq,D], partial_l/m [S,B,H,Tq]");
      for (int i = 0; i < 4; ++i) {
        if (a.partial_o.shape[i + 1] != a.q.shape[i]) return fail(G4B_ERR_BAD_ARG, "prefill: partial_o shape must be [S,B,H,Tq,D]");
        if (i < 3 && (a.partial_l.shape[i + 1] != a.q.shape[i] || a.partial_m.shape[i + 1] != a.q.shape[i]))
          return fail(G4B_ERR_BAD_ARG, "prefill: partial_l/partial_m shape must be [S,B,H,Tq]");
        if (a.partial_o.stride[i] % 4 != 0) return fail(G4B_ERR_BAD_STRIDE, "prefill: partial_o strides must be multiples of 16 bytes");
      }
      if (a.partial_o.stride[4] != 1 || (((uintptr_t)a.partial_o.ptr) & 15))
        return fail(G4B_ERR_BAD_STRIDE, "prefill: partial_o rows must be contiguous and 16-byte aligned");
      p.n_splits = (int)want;
      p.by_splits.set((uint32_t)want);
      p.po = (float*)a.partial_o.ptr; p.pl = (float*)a.partial_l.ptr; p.pm = (float*)a.partial_m.ptr;
      for (int i = 0; i < 4; ++i) { p.po_s[i] = a.partial_o.stride[i]; p.pl_s[i] = a.partial_l.stride[i]; p.pm_s[i] = a.partial_m.stride[i]; }
    }
  }
  const int64_t n_items = base_items * p.n_splits;
  if (n_items > 0x7fffffffLL) return fail(G4B_ERR_UNSUPPORTED, "prefill: too many work items");
  if (workers > n_items) workers = n_items;
  dim3 grid((unsigned)(pair ? 2 * workers : workers), 1, 1);
  bool stage = stage_out && p.n_splits == 1;   // partials are stored directly
  if (q_f32) {
    qm = km;   // never used by the kernel: q is converted on load
    p.q_f32 = (const float*)a.q.ptr;
    p.q_s0 = a.q.stride[0]; p.q_s1 = a.q.stride[1]; p.q_s2 = a.q.stride[2];
  }
  // the output as the copy engine stores it: boxes of 32 rows x 64 columns of one (slot, head)
  CUtensorMap om = km;   // (never used when the output is not staged)
  if (stage) {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)Tq, (uint64_t)H, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)a.o.stride[2] * esz, (uint64_t)a.o.stride[1] * esz, (uint64_t)a.o.stride[0] * esz};
    const uint32_t box[4] = {64, 32, 1, 1};
    // an output layout the descriptor cannot express (the driver refuses it) is stored directly
    if (encode_map(&om, a.o.dtype, 4, a.o.ptr, dims, strides, box, "o") != G4B_OK) { om = km; stage = false; }
  }
  if (a.k_cache.dtype == G4B_BF16) rc = launch_typed<__nv_bfloat16>(qm, km, vm, om, p, grid, pair, stage, short_items, p.n_splits > 1, st);
  else rc = launch_typed<__half>(qm, km, vm, om, p, grid, pair, stage, short_items, p.n_splits > 1, st);
  if (rc != G4B_OK || p.n_splits == 1) return rc;
  G4bCombineArgs c{};
  c.partial_o = a.partial_o; c.partial_l = a.partial_l; c.partial_m = a.partial_m; c.o = a.o;
  c.user_phase = a.user_phase; c.num_splits = p.n_splits; c.phase = a.phase;
  return launch_combine(c, st);
}

}  // namespace g4b
