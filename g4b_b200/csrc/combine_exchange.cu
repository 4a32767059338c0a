// Split-KV combine across GPUs in one kernel: local merge, exchange over peer memory, final
// merge.
//
// One sequence whose KV pages are split over W GPUs ends, on every GPU, with S local partials
// per (slot, head) in the reference's split-KV format (un-normalised accumulator, row sum,
// row maximum in log2 units: g4b/kernels/fa2.py:438-472).  The merge is associative
// (fa2.py:618-626), so each GPU first merges its own S partials into one, then the W merged
// partials are exchanged and merged again.  The exchange is not a library collective: each
// block stores its piece of the merged partial straight into every peer's exchange buffer
// (plain stores to peer-mapped memory travel over NVLink), waits for the same piece from every
// peer in its own memory, and finishes the merge.  16 KB per GPU pair cross the links; there
// is no second launch and no host round trip.
//
// Every value travels as one 8-byte word {value, launch count}: an aligned 8-byte store is
// seen whole or not at all, so the word is its own arrival flag.  The receiver polls the words
// themselves until they carry this launch's count.  No fence and no separate flag write sit
// between the data and its announcement, which is what the latency of so small an exchange is
// made of (data, system fence, flag, each a trip over the link: 20 us per launch with a flag
// per piece against 5 us for the same merge without peers).
//
// Blocks wait only for blocks of OTHER GPUs (same index there), never for blocks of their own
// grid.  (With more blocks than a GPU holds at once, a block can only be served if the peer
// gets to the same block; shapes that large may end in the time-out code below.)  Every wait is bounded; on a timeout
// the block records a code in the device status word and gives up.  Buffers are double
// buffered by launch parity: a peer can be at most one launch ahead, because its next launch
// cannot finish without this GPU's next contribution; a word of the same parity therefore
// still holds the count of two launches ago, never this one's.
#include "common.cuh"

namespace g4b {
namespace {

constexpr int kXThreads = 256;
constexpr int kXCols = 32;            // head-dim elements per block
constexpr int kXMaxSplits = 1024;
constexpr int kXMaxWorld = 8;
constexpr long long kXWaitLimit = 1ll << 31;   // SM cycles (about a second)

enum : int32_t { kErrPeerWait = 0x401 };

struct ExchangeParams {
  const void* po; const float* pl; const float* pm; void* o;
  const uint8_t* user_phase;
  int64_t po_s[5], pl_s[4], pm_s[4], o_s[4];
  int64_t phase_stride;
  unsigned long long* xbuf[kXMaxWorld];   // exchange buffer of every rank (own entry: local memory)
  uint32_t* state;                // local: {launches completed, blocks done in this launch}
  int32_t* status;
  int S, B, H, Tq, D, phase, world, rank;
  int rows, slices;
};

__device__ __forceinline__ void st_word_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Word offset inside one rank's exchange buffer.
__device__ __forceinline__ int64_t xbuf_off(const ExchangeParams& p, int par, int src, int row, int slice) {
  return ((((int64_t)par * p.world + src) * p.rows + row) * p.slices + slice) * (kXCols + 2);
}

template <typename TP, typename TO>
__global__ void __launch_bounds__(kXThreads) combine_exchange_kernel(ExchangeParams p) {
  __shared__ float s_w[kXMaxSplits];
  __shared__ float s_red[kXThreads / 32];
  __shared__ float s_acc[kXThreads];
  __shared__ float s_part[kXMaxWorld][kXCols + 2];
  __shared__ uint32_t s_epoch;
  __shared__ int s_fail;
  const int row = blockIdx.x, slice = blockIdx.y;
  const int t = row % p.Tq, h = (row / p.Tq) % p.H, b = row / (p.Tq * p.H);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { s_epoch = p.state[0] + 1; s_fail = 0; }
  const bool live = p.user_phase == nullptr || p.user_phase[b * p.phase_stride] == (uint8_t)p.phase;

  if (live) {
    // ---- local merge, phase 1: weights of the S local splits ----
    const int64_t ml_off = b * p.pm_s[1] + h * p.pm_s[2] + t * p.pm_s[3];
    const int64_t l_off = b * p.pl_s[1] + h * p.pl_s[2] + t * p.pl_s[3];
    float m = -INFINITY;
    for (int s = tid; s < p.S; s += kXThreads) {
      const float ms = p.pm[s * p.pm_s[0] + ml_off];
      s_w[s] = ms;
      m = fmaxf(m, ms);
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = s_red[0];
    for (int w = 1; w < kXThreads / 32; ++w) m = fmaxf(m, s_red[w]);
    __syncthreads();
    float l = 0.f;
    for (int s = tid; s < p.S; s += kXThreads) {
      const float ms = s_w[s];
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
      s_w[s] = w;
      if (w != 0.f) l += p.pl[s * p.pl_s[0] + l_off] * w;
    }
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) s_red[warp] = l;
    __syncthreads();
    l = 0.f;
    for (int w = 0; w < kXThreads / 32; ++w) l += s_red[w];

    // ---- phase 2: 8 split groups x 32 elements, summed through shared memory ----
    const TP* po = (const TP*)p.po + b * p.po_s[1] + h * p.po_s[2] + t * p.po_s[3];
    const int c = tid & (kXCols - 1), grp = tid / kXCols;
    const int d = slice * kXCols + c;
    float acc = 0.f;
    if (d < p.D) {
#pragma unroll 4
      for (int s = grp; s < p.S; s += kXThreads / kXCols) {
        const float w = s_w[s];
        if (w != 0.f) acc += ElemTraits<TP>::to_float(po[s * p.po_s[0] + d]) * w;
      }
    }
    s_acc[tid] = acc;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int par = (int)(epoch & 1u);
    if (tid < kXCols + 2) {
      float v;
      if (tid < kXCols) {
        v = 0.f;
        for (int g2 = 0; g2 < kXThreads / kXCols; ++g2) v += s_acc[g2 * kXCols + tid];
      } else {
        v = tid == kXCols ? l : m;
      }
      // ---- push this rank's merged piece to every rank (own copy included) ----
      const int64_t off = xbuf_off(p, par, p.rank, row, slice) + tid;
      const unsigned long long word = ((unsigned long long)epoch << 32) | __float_as_uint(v);
      for (int r = 0; r < p.world; ++r) st_word_sys(p.xbuf[r] + off, word);
    }
    // ---- wait for every rank's piece: a word has arrived once it carries this launch's count ----
    const long long t0 = clock64();
    for (int i = tid; i < p.world * (kXCols + 2); i += kXThreads) {
      const int r = i / (kXCols + 2), e = i % (kXCols + 2);
      const unsigned long long* src = p.xbuf[p.rank] + xbuf_off(p, par, r, row, slice) + e;
      unsigned long long w = ld_word_sys(src);
      while ((uint32_t)(w >> 32) != epoch) {
        if (s_fail || clock64() - t0 > kXWaitLimit) { atomicCAS(p.status, 0, kErrPeerWait); s_fail = 1; break; }
        w = ld_word_sys(src);
      }
      s_part[r][e] = __uint_as_float((uint32_t)w);
    }
    __syncthreads();
    if (!s_fail) {
      // ---- final merge of the W pieces ----
      if (tid < kXCols && d < p.D) {
        float mm = -INFINITY;
        for (int r = 0; r < p.world; ++r) mm = fmaxf(mm, s_part[r][kXCols + 1]);
        float num = 0.f, den = 0.f;
        for (int r = 0; r < p.world; ++r) {
          const float mr = s_part[r][kXCols + 1];
          const float w = (mr == -INFINITY) ? 0.f : exp2f(mr - mm);
          num += s_part[r][tid] * w;
          den += s_part[r][kXCols] * w;
        }
        TO* o = (TO*)p.o + b * p.o_s[0] + h * p.o_s[1] + t * p.o_s[2];
        o[d] = ElemTraits<TO>::from_float(den > 0.f ? num / den : 0.f);
      }
    }
  }
  // ---- the last block of the launch advances the launch count ----
  __syncthreads();
  if (tid == 0) {
    const uint32_t n_blocks = gridDim.x * gridDim.y;
    __threadfence();
    if (atomicAdd(&p.state[1], 1u) == n_blocks - 1) {
      p.state[1] = 0;
      __threadfence();
      p.state[0] = s_epoch;
    }
  }
}

}  // namespace

int launch_combine_exchange(const G4bExchangeArgs& a, cudaStream_t st) {
  if (a.world < 1 || a.world > kXMaxWorld) return fail(G4B_ERR_BAD_ARG, "exchange: world must be 1..%d", kXMaxWorld);
  if (a.rank < 0 || a.rank >= a.world) return fail(G4B_ERR_BAD_ARG, "exchange: rank outside the world");
  if (a.num_splits < 1 || a.num_splits > kXMaxSplits) return fail(G4B_ERR_TOO_LARGE, "exchange: 1..%d splits", kXMaxSplits);
  if (a.partial_o.ptr == nullptr || a.partial_l.ptr == nullptr || a.partial_m.ptr == nullptr || a.o.ptr == nullptr)
    return fail(G4B_ERR_BAD_ARG, "exchange: partial_o/l/m and o are required");
  if (a.partial_o.ndim != 5 || a.partial_l.ndim != 4 || a.partial_m.ndim != 4 || a.o.ndim != 4)
    return fail(G4B_ERR_BAD_ARG, "exchange: ranks must be 5/4/4/4");
  if (a.partial_l.dtype != G4B_F32 || a.partial_m.dtype != G4B_F32) return fail(G4B_ERR_BAD_DTYPE, "exchange: partial_l/m must be f32");
  if (a.partial_o.shape[0] < a.num_splits || a.partial_l.shape[0] < a.num_splits || a.partial_m.shape[0] < a.num_splits)
    return fail(G4B_ERR_BAD_ARG, "exchange: fewer partials than splits");
  for (int i = 0; i < 4; ++i)
    if (a.partial_o.shape[i + 1] != a.o.shape[i]) return fail(G4B_ERR_BAD_ARG, "exchange: partial_o and o disagree");
  if (a.state == nullptr) return fail(G4B_ERR_BAD_ARG, "exchange: state is null");
  ExchangeParams p{};
  for (int r = 0; r < a.world; ++r) {
    if (a.xbuf[r] == nullptr) return fail(G4B_ERR_BAD_ARG, "exchange: buffer of rank %d missing", r);
    if (((uintptr_t)a.xbuf[r] & 7) != 0) return fail(G4B_ERR_BAD_STRIDE, "exchange: buffers must be 8-byte aligned");
    p.xbuf[r] = (unsigned long long*)a.xbuf[r];
  }
  p.po = a.partial_o.ptr; p.pl = (const float*)a.partial_l.ptr; p.pm = (const float*)a.partial_m.ptr; p.o = a.o.ptr;
  p.user_phase = (const uint8_t*)a.user_phase.ptr; p.phase_stride = a.user_phase.stride[0];
  for (int i = 0; i < 5; ++i) p.po_s[i] = a.partial_o.stride[i];
  for (int i = 0; i < 4; ++i) { p.pl_s[i] = a.partial_l.stride[i]; p.pm_s[i] = a.partial_m.stride[i]; p.o_s[i] = a.o.stride[i]; }
  p.S = a.num_splits; p.B = (int)a.o.shape[0]; p.H = (int)a.o.shape[1]; p.Tq = (int)a.o.shape[2]; p.D = (int)a.o.shape[3];
  p.phase = a.phase; p.world = a.world; p.rank = a.rank;
  p.state = (uint32_t*)a.state;
  const int64_t rows = (int64_t)p.B * p.H * p.Tq;
  if (rows == 0) return G4B_OK;
  p.rows = (int)rows; p.slices = (p.D + kXCols - 1) / kXCols;
  if (rows > 65535 || p.slices > 65535) return fail(G4B_ERR_TOO_LARGE, "exchange: too many rows");
  const int64_t need_x = 2ll * a.world * rows * p.slices * (kXCols + 2) * 8;
  if (a.xbuf_bytes < need_x)
    return fail(G4B_ERR_BAD_ARG, "exchange: buffers too small (need %lld bytes per rank)", (long long)need_x);
  G4B_STOP_IF_VALIDATE_ONLY();
  p.status = device_status_ptr();
  if (p.status == nullptr) return G4B_ERR_CUDA;
  const dim3 grid((unsigned)rows, (unsigned)p.slices, 1);
  bool launched = false;
  G4B_DISPATCH_FLOAT(a.partial_o.dtype, TP,
    G4B_DISPATCH_FLOAT(a.o.dtype, TO,
      combine_exchange_kernel<TP, TO><<<grid, kXThreads, 0, st>>>(p); launched = true));
  if (!launched) return fail(G4B_ERR_BAD_DTYPE, "exchange: partial_o/o dtypes must be f32, f16 or bf16");
  G4B_CUDA_CHECK(cudaGetLastError());
  return G4B_OK;
}

}  // namespace g4b

extern "C" int g4b_attn_combine_exchange(const G4bExchangeArgs* args, void* cuda_stream) {
  if (args == nullptr) return g4b::fail(G4B_ERR_BAD_ARG, "args is null");
  return g4b::launch_combine_exchange(*args, (cudaStream_t)cuda_stream);
}

extern "C" int64_t g4b_exchange_buffer_bytes(int world, int64_t rows, int head_dim) {
  // large enough for either entry point: g4b_attn_combine_exchange moves pieces of 32 columns
  // (+ l, m), g4b_decode_step pieces of 8 columns (+ l, m)
  const int64_t slices = (head_dim + g4b::kXCols - 1) / g4b::kXCols;
  const int64_t a = 2ll * world * rows * slices * (g4b::kXCols + 2) * 8;
  const int64_t b = 2ll * world * rows * ((head_dim + 7) / 8) * 10 * 8;
  return a > b ? a : b;
}
