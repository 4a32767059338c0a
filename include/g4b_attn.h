/*
 * g4b_attn.h -- C ABI of libg4b_attn.so: the attention hot path of the g4b Gemma
 * inference engine (flash-attention prefill, paged / ring KV-cache append, single-token
 * split-KV decode with log-sum-exp combine) as hand-written CUDA for sm_100a.
 *
 * Every entry point takes plain structs of pointers, sizes and element strides, launches
 * on the stream it is given, allocates nothing on the device, never synchronises the
 * host, never aborts, and returns 0 or a negative G4B_ERR_* code. The message for the
 * last failure on the calling thread is available from g4b_last_error_string().
 *
 * Each declaration cites the interface of the reference (barnii77/g4b) that it replaces.
 */
#ifndef G4B_ATTN_H_
#define G4B_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define G4B_ABI_VERSION 2

/* element types (g4b/tensor.py dtypes that reach this path) */
enum G4bDtype {
  G4B_F32 = 0,
  G4B_F16 = 1,
  G4B_BF16 = 2,
  G4B_I32 = 3,
  G4B_I64 = 4,
  G4B_U8 = 5,
  G4B_FP8_E4M3 = 6 /* one byte per element; caches only (g4b_kv_append_fp8, g4b_flash_attention_fp8) */
};

/* per-slot phase encoding, g4b/kernels/fa2.py:26-31 */
enum G4bPhase { G4B_PHASE_UNALLOCATED = 0, G4B_PHASE_PREFILL = 1, G4B_PHASE_DECODE = 2 };

/* masking stage, g4b/kernels/fa2.py:14-16 */
enum G4bStage { G4B_STAGE_FULL = 1, G4B_STAGE_CAUSAL = 3 };

enum G4bStatus {
  G4B_OK = 0,
  G4B_VALIDATED = 1,         /* validate-only mode: every argument check passed, nothing launched */
  G4B_ERR_BAD_ARG = -1,      /* null pointer, bad rank, inconsistent shapes            */
  G4B_ERR_BAD_DTYPE = -2,    /* dtype combination no kernel is built for               */
  G4B_ERR_BAD_STRIDE = -3,   /* innermost stride != 1, non-contiguous cache, alignment */
  G4B_ERR_UNSUPPORTED = -4,  /* shape outside what the kernels cover (e.g. head dim)   */
  G4B_ERR_CUDA = -5,         /* a CUDA runtime / driver call failed                    */
  G4B_ERR_DEVICE_WAIT = -6,  /* g4b_device_status found a code that a kernel recorded      */
  G4B_ERR_TOO_LARGE = -7     /* size beyond a stated fixed maximum                     */
};

/*
 * A strided view, the C form of what g4b/kernels/utils.py:113-122 unpacks from any
 * object with .shape/.stride/.dtype/.data_ptr(): base pointer, shape and strides in
 * ELEMENTS, rank <= 5.  ptr == NULL means "argument not given".
 */
typedef struct G4bTensor {
  void* ptr;
  int64_t shape[5];
  int64_t stride[5];
  int32_t ndim;
  int32_t dtype; /* enum G4bDtype */
} G4bTensor;

/*
 * Arguments of one attention call; the C form of
 *   flash_attention(q, k_cache, v_cache, o, time_dim_sizes, user_phase, ctx_window_size,
 *                   phase, partial_o, partial_l, partial_m, *, stage)
 * (g4b/kernels/fa2.py:634-652).
 *
 *  q, o          [B, H, Tq, D] views, last stride 1 (fa2.py:312-314)
 *  ring mode     k_cache, v_cache [B, G, T, D] contiguous (fa2.py:315-320); logical key j
 *                of slot b lives in row (ring_start + j) % T (fa2.py:52-55,75)
 *  paged mode    block_tables.ptr != NULL: k_cache, v_cache are page pools
 *                [num_pages, G, page_size, D] contiguous, block_tables int32 [B, max_pages];
 *                logical key j lives in page block_tables[b, j / page_size], row
 *                j % page_size (not in the reference, which has a ring buffer only)
 *  time_dim_sizes int32 [B]: context length of slot b including this step's tokens
 *  user_phase    uint8 [B] or absent: slot b is skipped unless user_phase[b] == phase
 *                (fa2.py:333-335)
 *  ctx_window_size  number of most recent keys the cache exposes (fa2.py:53-54)
 *  sliding_window   0, or W: query at absolute position p also ignores keys at positions
 *                <= p - W (scripts/reference_impl.py:440-441).  0 keeps the reference
 *                kernel's chunk-shared lower bound only (fa2.py:58-64).
 *  scale         multiplies q.k before the softmax; the reference uses 1.0 (fa2.py:89)
 *  partial_*     split-KV workspace [S, B, H, Tq, D] / [S, B, H, Tq] (fa2.py:438-472);
 *                partial_o f32/f16/bf16, partial_l and partial_m f32, m in log2 units
 *  num_kv_splits 0 = the reference's static policy (fa2.py:201-212), else forced
 */
typedef struct G4bAttnArgs {
  G4bTensor q, k_cache, v_cache, o;
  G4bTensor time_dim_sizes, user_phase;
  G4bTensor partial_o, partial_l, partial_m;
  G4bTensor block_tables;
  int32_t ctx_window_size;
  int32_t phase;
  int32_t stage;
  int32_t page_size;
  int32_t sliding_window;
  int32_t num_kv_splits;
  float scale;
  int32_t reserved;
} G4bAttnArgs;

/* Head dims: the Tq == 1 path (g4b_attn_decode, g4b_decode_step, g4b_attn_combine, and
 * g4b_flash_attention when Tq == 1 with at most 8 query heads per kv head) takes 128, 256 and
 * 512; the Tq > 1 kernel (g4b_attn_prefill) takes 256 and 128 (128 on the 256-wide tiles, so at
 * the time of 256). */

/* replaces flash_attention() as a whole (fa2.py:634-715): picks the prefill or the
 * decode kernel, the split count, and runs the combine when splits > 1. */
int g4b_flash_attention(const G4bAttnArgs* args, void* cuda_stream);

/* replaces the launch of _attn_kernel for Tq > 1 (fa2.py:256-480, 672-690):
 * tcgen05 / TMEM / TMA flash-attention forward, head dim 256 or 128, f16 or bf16 caches, q and o in
 * the cache dtype or f32.  If the partial triple is given (f32, [S,B,H,Tq,D] / [S,B,H,Tq]) and
 * the chunk has too few (slot, head, 128-row tile) units to occupy the GPU, every unit's key
 * range is split over up to S pieces (num_kv_splits forces a count) and merged by a second
 * launch; the reference splits in the decode phase only (fa2.py:201-212). */
int g4b_attn_prefill(const G4bAttnArgs* args, void* cuda_stream);

/* replaces the launch of _attn_kernel for Tq == 1 (fa2.py:256-480 with
 * NUM_KV_SPLITS >= 1): streams K/V once from HBM; writes o when the split count is 1,
 * else un-normalised partials (fa2.py:438-472) and leaves the merge to the caller. */
int g4b_attn_decode(const G4bAttnArgs* args, void* cuda_stream);

/*
 * The decode step of one attention layer; replaces, for Tq == 1, the two add_kv_to_cache
 * launches, the _attn_kernel launch and the _reduce_split_kv_kernel launch of the reference's
 * decode phase (g4b/models/gemma4e.py:575-607, fa2.py:702-714) by two launches (attention
 * with the append inside it, then the merge, scheduled while the first drains) or, when the
 * KV range of one sequence is split over GPUs, by ONE launch that also exchanges and merges.
 *
 *   attn            as for g4b_attn_decode; partial_* (f32, rows on 8-byte boundaries) are the
 *                   split workspace; num_kv_splits > 0 forces the split count, 0 picks it as
 *                   g4b_flash_attention does
 *   k_new, v_new    optional, together: [B, G, 1, D] rows in the cache dtype.  For every slot in
 *                   phase they are written to the cache at position time_dim_sizes[b] - 1
 *                   (ring row (time - 1) % T, or the page the block table names) and used as
 *                   that position's K / V, whatever the cache held there before
 *   world > 1       one sequence's KV range is split over `world` GPUs (one process each, the
 *                   same call sequence and shapes on every rank): the local splits are merged,
 *                   the merged (acc, l, m) travel to every rank's exchange buffer as 8-byte
 *                   words {value, launch count} through peer-mapped memory, and every rank
 *                   finishes the merge, all inside the attention launch.  xbuf / state /
 *                   xbuf_bytes as for g4b_attn_combine_exchange (same size; a buffer must not be
 *                   shared between the two entry points).  Every CTA of the launch must be
 *                   resident at once (splits * G * B <= 2 x the SM count; 1 x at head dim 512)
 *                   and splits <= 320, else G4B_ERR_TOO_LARGE.  A peer that does not show up
 *                   within about a second leaves 0x401 in the status word; after that the
 *                   buffers and `state` must be zeroed again on every rank before the next call.
 *                   The launch counts its CTAs in three words inside the library (one set per
 *                   GPU: two arrival counts used in turns, and the turn): two such launches
 *                   that overlap on one GPU would share them -- keep them on one stream or
 *                   order them.
 */
typedef struct G4bDecodeStepArgs {
  G4bAttnArgs attn;
  G4bTensor k_new, v_new;
  void* xbuf[8];
  void* state;
  int64_t xbuf_bytes;
  int32_t world;
  int32_t rank;
} G4bDecodeStepArgs;
int g4b_decode_step(const G4bDecodeStepArgs* args, void* cuda_stream);

/* replaces _reduce_split_kv_kernel (fa2.py:546-631): log-sum-exp merge of the first
 * num_splits partials into o.  Also merges partials gathered from other GPUs. */
typedef struct G4bCombineArgs {
  G4bTensor partial_o, partial_l, partial_m, o;
  G4bTensor user_phase; /* optional uint8 [B]: rows of slots with user_phase[b] != phase keep o */
  int32_t num_splits;
  int32_t phase;
} G4bCombineArgs;
int g4b_attn_combine(const G4bCombineArgs* args, void* cuda_stream);

/* The split count g4b_flash_attention would use; the reference's policy in
 * _prune_invalid_configs (fa2.py:186-225). */
int g4b_select_kv_splits(int ctx_window_size, int max_kv_splits, int phase, int tq);

/*
 * replaces add_kv_to_cache(x, cache, cache_offsets, rmsnorm_eps, x_rsos, user_phase,
 * phase) (g4b/kernels/add_kv_to_cache.py:162-186):
 *   cache[b, g, (cache_offsets[b] + t) % T, :] = cast(x[b, g, t, :] * r)
 * with r = rsqrt(x_rsos[b,g,t] / D + eps) when x_rsos is given, else 1
 * (add_kv_to_cache.py:148-158).  Paged mode (block_tables given): row cache_offsets[b]+t
 * of the sequence goes to page block_tables[b, p / page_size], row p % page_size.
 * cache_offsets may be int32 or int64.  Slots with user_phase[b] != phase are skipped.
 */
typedef struct G4bAppendArgs {
  G4bTensor x;             /* [B, G, Tq, D] view, last stride 1; f32, f16 or bf16 */
  G4bTensor cache;         /* ring [B, G, T, D] or pool [num_pages, G, page_size, D] */
  G4bTensor cache_offsets; /* [B] int32 or int64 */
  G4bTensor x_rsos;        /* optional [B, G, Tq] f32 view */
  G4bTensor user_phase;    /* optional uint8 [B] */
  G4bTensor block_tables;  /* optional int32 [B, max_pages] */
  float rmsnorm_eps;
  int32_t phase;
  int32_t page_size;
  int32_t reserved;
} G4bAppendArgs;
int g4b_kv_append(const G4bAppendArgs* args, void* cuda_stream);

/*
 * replaces advance_decode_state(input_token_ids, out_token_ids, cache_offsets,
 * time_dim_sizes, user_phase) (g4b/kernels/advance_decode_state.py:31-80): for every slot
 * in the decode phase, input_token_ids[0,b] = out_token_ids[b,0], cache_offsets[b] += 1,
 * time_dim_sizes[b] += 1.
 */
typedef struct G4bAdvanceArgs {
  G4bTensor input_token_ids; /* int32 [>=1, B] */
  G4bTensor out_token_ids;   /* int32 [B, >=1] */
  G4bTensor cache_offsets;   /* int32 [B] */
  G4bTensor time_dim_sizes;  /* int32 [B] */
  G4bTensor user_phase;      /* uint8 [B] */
} G4bAdvanceArgs;
int g4b_advance_decode_state(const G4bAdvanceArgs* args, void* cuda_stream);

/*
 * KV cache in 8 bits (e4m3), paged.  No counterpart in the reference, whose caches are f16
 * (g4b/models/gemma4e.py:32,866-870); the arithmetic is the reference's attention on the
 * de-quantised values.  A pool is [num_pages, G, page_size, D] bytes with one f32 scale per
 * (page, kv head) beside it, [num_pages, G]: value = e4m3(byte) x scale.
 *
 * g4b_kv_append_fp8: as g4b_kv_append in paged mode (same index arithmetic, same optional V
 * norm and phase gate), then quantised.  The scale of a (page, kv head) is fixed by the FIRST
 * row of the page, whichever call appends it and however the rows are chunked:
 *     scale = max(max_d |row[d]| x headroom / 448, 2^-24)
 * and every row of the page is stored as round-to-nearest-even, saturating e4m3 of
 * row[d] / scale.  `headroom` (>= 1, e.g. 2) leaves later rows of the page room above the first
 * row's maximum before they saturate.  A call that appends rows to a page whose first row an
 * earlier call wrote reads the scale that call left.
 *
 * g4b_flash_attention_fp8: Tq == 1 attention over such pools (head dims 128, 256, 512; at most
 * 8 query heads per kv head), split-KV and merge as g4b_flash_attention.  q / o may be f32, f16
 * or bf16; products run in f16 with f32 accumulation.
 *
 * g4b_kv_dequant_fp8: for prefill chunks (Tq > 1) over such a cache.  Writes
 * round-to-nearest(e4m3(byte) x scale) into a caller-owned f16 / bf16 pool of the same geometry,
 * page p of the 8-bit pool into page p of `out`, so the same block tables address both and
 * g4b_flash_attention runs over `out`.  With block_tables and time_dim_sizes only the pages that
 * hold the first time_dim_sizes[b] tokens of the slots (of the slots in `phase`, when
 * user_phase is given) are converted and every other page of `out` is left as it is; without
 * them every page is.  A table entry outside the pool is skipped and reported (0x103 in the
 * device status word).
 */
typedef struct G4bFp8AppendArgs {
  G4bTensor x;             /* [B, G, Tq, D] view, last stride 1; f32, f16 or bf16 */
  G4bTensor cache;         /* pool [num_pages, G, page_size, D], 1 byte per element */
  G4bTensor scales;        /* f32 [num_pages, G] */
  G4bTensor cache_offsets; /* [B] int32 or int64 */
  G4bTensor x_rsos;        /* optional [B, G, Tq] f32 view */
  G4bTensor user_phase;    /* optional uint8 [B] */
  G4bTensor block_tables;  /* int32 [B, max_pages] */
  float rmsnorm_eps;
  float headroom;
  int32_t phase;
  int32_t page_size;
} G4bFp8AppendArgs;
int g4b_kv_append_fp8(const G4bFp8AppendArgs* args, void* cuda_stream);
typedef struct G4bFp8DequantArgs {
  G4bTensor cache;          /* pool [num_pages, G, page_size, D], 1 byte per element */
  G4bTensor scales;         /* f32 [num_pages, G] */
  G4bTensor out;            /* pool [num_pages, G, page_size, D], f16 or bf16, contiguous */
  G4bTensor block_tables;   /* optional int32 [B, max_pages] (then time_dim_sizes is required) */
  G4bTensor time_dim_sizes; /* optional int32 [B] */
  G4bTensor user_phase;     /* optional uint8 [B] (only with block_tables) */
  int32_t phase;
  int32_t page_size;
} G4bFp8DequantArgs;
int g4b_kv_dequant_fp8(const G4bFp8DequantArgs* args, void* cuda_stream);
int g4b_flash_attention_fp8(const G4bAttnArgs* args, const G4bTensor* k_scales, const G4bTensor* v_scales,
                            void* cuda_stream);

/*
 * Tq == 1 attention with split-KV and merge, for callers that cannot allocate device memory
 * (a serving loop whose memory was fixed at load time, a plugin inside an engine that owns
 * every allocation).  It has no counterpart in the reference, whose caller always brings the
 * partial buffers (g4b/models/gemma4e.py:819-821).  Same arguments as g4b_flash_attention,
 * except that partial_o / partial_l / partial_m must be absent: the split-KV workspace is a
 * fixed array inside the library (8192 rows of 258 floats, 8.06 MiB per GPU, held until the
 * process exits).  Limits: head dim 256, at most 16 splits, splits * B * H <= 8192; anything
 * larger returns G4B_ERR_TOO_LARGE when the split count was asked for (num_kv_splits > 0); with
 * num_kv_splits == 0 the count of g4b_select_kv_splits is cut down to what the array holds.
 * Allocates nothing.  The first call on each device looks
 * up the array's device address (cudaGetSymbolAddress) and should therefore be made once
 * before any stream capture on that device.  All calls share the one array, which keeps the
 * previous call's contents: nothing needs clearing (every entry the merge reads is written
 * first by the same call), but two calls that overlap on the GPU race on it -- keep them on
 * one stream or order them.
 */
int g4b_attn_decode_static_scratch(const G4bAttnArgs* args, void* cuda_stream);

/*
 * One launch for the three the reference issues between the q/k/v projections and the
 * attention call (g4b/models/gemma4e.py:564-592): apply_rope on q and k
 * (g4b/kernels/rope.py:8-39,123-211: per-head RMS norm with weight, then rotation of the
 * element pairs (i, i + D/2) by theta = (cache_offsets[b] + t) * rope_freqs[i], in fp32),
 * add_kv_to_cache of the rotated k, and add_kv_to_cache of v with the weight-less V norm
 * (g4b/kernels/add_kv_to_cache.py:148-159).
 *
 * Where the rows go:
 *   q  -> q_out if given (any float dtype: this is how an f32 scratchpad becomes the 16-bit
 *         Q that the prefill kernel reads), else back into q (what apply_rope does);
 *   k  -> k_cache (ring or paged, only slots with user_phase[b] == phase) and/or k_out; with
 *         neither, back into k (what apply_rope does);
 *   v  -> v_cache (same gate); v and v_cache may be absent together.
 * The rotation is not gated by phase (the reference's is not either).
 *
 * Norms: q and k are normalised iff norm_qk != 0, v iff norm_v != 0.  A row's sum of squares
 * comes from *_rsos if given (the reference's matmul epilogue produces it), else the kernel
 * computes it from the row.  q_norm_w / k_norm_w [D] are optional (absent = ones).
 * rope_freqs absent = no rotation (norm and append only).
 */
typedef struct G4bRopeAppendArgs {
  G4bTensor q;             /* [B, H, Tq, D] view, last stride 1; f32, f16 or bf16 */
  G4bTensor k;             /* [B, G, Tq, D] view */
  G4bTensor v;             /* optional [B, G, Tq, D] view */
  G4bTensor q_out;         /* optional [B, H, Tq, D] view */
  G4bTensor k_out;         /* optional [B, G, Tq, D] view */
  G4bTensor rope_freqs;    /* optional f32 [D/2] */
  G4bTensor cache_offsets; /* [B] int32 or int64: position of token 0 of each slot */
  G4bTensor q_rsos;        /* optional f32 [B, H, Tq] view */
  G4bTensor k_rsos;        /* optional f32 [B, G, Tq] view */
  G4bTensor v_rsos;        /* optional f32 [B, G, Tq] view */
  G4bTensor q_norm_w;      /* optional f32 [D] */
  G4bTensor k_norm_w;      /* optional f32 [D] */
  G4bTensor k_cache;       /* optional ring [B, G, T, D] or pool [num_pages, G, page_size, D] */
  G4bTensor v_cache;       /* optional, same form as k_cache */
  G4bTensor user_phase;    /* optional uint8 [B] */
  G4bTensor block_tables;  /* optional int32 [B, max_pages]: caches are page pools */
  float rmsnorm_eps;
  int32_t phase;
  int32_t page_size;
  int32_t norm_qk;
  int32_t norm_v;
  int32_t reserved;
} G4bRopeAppendArgs;
int g4b_rope_norm_append(const G4bRopeAppendArgs* args, void* cuda_stream);

/*
 * Split-KV merge across GPUs in one launch, for one sequence whose KV range is split over
 * `world` GPUs (one process per GPU).  No counterpart in the reference, which is single-GPU;
 * the arithmetic is the reference's merge (g4b/kernels/fa2.py:618-626) applied twice: the
 * `num_splits` local partials are merged into one, the merged partials of all ranks are
 * exchanged through peer-mapped memory (every rank stores its piece into every rank's
 * exchange buffer as 8-byte words {value, launch count}, so a word announces itself), and
 * merged again into `o`.  Every rank must make the same sequence of calls with the same
 * shapes, and a slot must be in `phase` on all ranks or on none.
 *
 * xbuf[r]: address, in this process, of rank r's exchange buffer (own entry: ordinary local
 * memory; others: peer mappings), 8-byte aligned.  Size per rank from
 * g4b_exchange_buffer_bytes(); it must start zeroed and be used for nothing else.  state:
 * two zero-initialised uint32 in local memory.  A peer that does not show up within about a
 * second leaves code 0x401 in the device status word; after that the buffers and `state` must
 * be zeroed again on every rank (and the ranks brought back in step) before the next call: a
 * rank that gave up may otherwise run ahead and overwrite words of the same parity that a peer
 * has not read.  Block (row, slice) of this launch waits for the same block of every peer; with
 * more blocks (rows x ceil(D / 32)) than one GPU holds at once this relies on every GPU getting
 * to the same blocks, which CUDA does not promise -- such shapes can end in 0x401 too.
 * g4b_decode_step's exchange form checks residency on the host instead.
 */
typedef struct G4bExchangeArgs {
  G4bTensor partial_o;     /* local [S, B, H, Tq, D] f32/f16/bf16 */
  G4bTensor partial_l;     /* local [S, B, H, Tq] f32 */
  G4bTensor partial_m;     /* local [S, B, H, Tq] f32, log2 units */
  G4bTensor o;             /* [B, H, Tq, D] */
  G4bTensor user_phase;    /* optional uint8 [B] */
  void* xbuf[8];
  void* state;
  int64_t xbuf_bytes;      /* size of every rank's exchange buffer */
  int32_t num_splits;
  int32_t phase;
  int32_t world;
  int32_t rank;
} G4bExchangeArgs;
int g4b_attn_combine_exchange(const G4bExchangeArgs* args, void* cuda_stream);
/* Bytes of one rank's exchange buffer for `rows` = B * H * Tq rows of `head_dim` elements. */
int64_t g4b_exchange_buffer_bytes(int world, int64_t rows, int head_dim);

/* Message of the last failing call on this thread ("" if none). No reference counterpart:
 * the reference raises Python exceptions from its wrappers (fa2.py:656-657). */
const char* g4b_last_error_string(void);

/* ABI version of the loaded library (G4B_ABI_VERSION). */
int g4b_abi_version(void);

/*
 * Reads (and clears) the device-side status word of the current device after
 * synchronising the given stream.  Kernels never trap: one that meets a block-table entry
 * outside the pool skips it and records 0x1xx (append) / 0x201 (decode) / 0x309 (prefill); a
 * bounded wait that runs out makes the kernel return early and record 0x21x (decode), 0x3xx
 * (prefill) or 0x4xx (a peer GPU that did not show up).  The word keeps the FIRST code until this call
 * clears it.  While it holds a 0x3xx wait code every later prefill launch returns at once
 * without computing (the tensor pipe may be in an unknown state); codes of other kernels do
 * not stop any launch.  Returns G4B_OK with *status_out = 0, or G4B_ERR_DEVICE_WAIT with the
 * code in *status_out.  No reference counterpart.
 */
int g4b_device_status(void* cuda_stream, int32_t* status_out);

/*
 * Validate-only mode for the calling thread (0 = off, the default).  While it is on, every
 * entry point above runs its argument checks and returns G4B_VALIDATED (or the error) without
 * making a CUDA call or launching anything; pointers are never dereferenced.  For tests of
 * the argument checks on machines without a GPU.  No reference counterpart.
 */
void g4b_set_validate_only(int on);

#ifdef __cplusplus
}
#endif
#endif /* G4B_ATTN_H_ */
