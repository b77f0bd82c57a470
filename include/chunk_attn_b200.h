/*
 * chunk_attn_b200.h — C ABI of the B200 (sm_100a) ChunkAttention decode kernels.
 *
 * This is the boundary between the C++ host (prefix tree, chunk pool bookkeeping, the
 * `Attention` class and its pybind11 surface) and the hand-written CUDA underneath.  It
 * replaces, function for function, the free functions the reference's host calls in
 * cpp/chunk_attn/kernel_cuda.h:57-69 and the `KernelContext` they share (kernel_cuda.h:9-55).
 * Only plain pointers, integers and a CUDA stream cross it: no torch types, no C++ types,
 * no exceptions.  Every function returns CA_OK (0) or a negative CA_ERR_* code;
 * ca_last_error() gives the message of the calling thread's last failure.
 *
 * There is no CPU implementation behind this ABI.  A function that needs the GPU fails with
 * CA_ERR_CUDA when no device is usable; nothing falls back to the host.
 *
 * Threading: a context is driven by one thread at a time (the reference's `Attention` has the
 * same contract, src/chunk_attn/models/model_host.py:82-123).  All device work is ordered on
 * the stream passed to each call.
 */
#ifndef CHUNK_ATTN_B200_H_
#define CHUNK_ATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CA_API __attribute__((visibility("default")))

/* ---- status codes ------------------------------------------------------------------------ */
#define CA_OK 0
#define CA_ERR_INVALID (-1)      /* bad argument (null pointer, range, unsupported shape)      */
#define CA_ERR_CUDA (-2)         /* a CUDA runtime call failed; see ca_last_error()            */
#define CA_ERR_STATE (-3)        /* call order: work list not refreshed, tail slot overflow    */
#define CA_ERR_DEVICE_STATUS (-4) /* a kernel reported a bounded wait that ran out            */

/* element types of q/k/v/out and of the chunk pool */
#define CA_DTYPE_F16 0
#define CA_DTYPE_F32 1

/* `partition` of ca_attention, the reference's meaning (cpp/chunk_attn/attention.h:46):
 * 0 auto, 1 chunk-first then sequence-first, 2 sequence-first only. */
#define CA_PARTITION_AUTO 0
#define CA_PARTITION_CHUNK_FIRST 1
#define CA_PARTITION_SEQ_FIRST 2

typedef struct ca_context ca_context;
typedef struct ca_plan ca_plan;
typedef void* ca_stream; /* cudaStream_t */

/* One entry of the per-step work list the host hands down: a live, non-root chunk of the
 * prefix tree and the contiguous range of sequence rows whose context contains it.
 * Replaces GPT::ChunkInfo (cpp/chunk_attn/chunk_info.h:7-15); the chunk is named by its
 * slot in the pool instead of by pointer, and carries its token count. */
typedef struct ca_chunk_info {
    int32_t chunk_id;  /* slot in the pool, 0 <= chunk_id < max_chunks */
    int32_t n_tokens;  /* tokens currently stored, 0..chunk_size        */
    int32_t seq_begin; /* first row (inclusive)                         */
    int32_t seq_end;   /* last row (exclusive)                          */
} ca_chunk_info;

/* ---- library ------------------------------------------------------------------------------ */
CA_API const char* ca_last_error(void);
CA_API int ca_version(void);

/* ---- pool geometry -------------------------------------------------------------------------
 * The pool is ONE device allocation made by the caller:
 *     [max_chunks][n_heads][2 (K then V)][chunk_size][d_head] elements.
 * A (chunk, head) pair therefore owns one contiguous K tile immediately followed by its V tile,
 * which is what one bulk copy into shared memory fetches.  When a token row is a multiple of 128 bytes, a tile is
 * stored as panels, [row_bytes / 128][chunk_size][128 bytes]: panel p holds bytes [128 p, 128 p + 128) of every
 * token row, and inside a token's 128-byte line the 16-byte granule c sits at position c ^ (token & 7) -- the
 * canonical 128-byte-swizzled operand layout of the tcgen05 tensor cores, so a staged tile is handed to
 * tcgen05.mma by descriptor, and the same layout keeps the ldmatrix loads of the mma.sync path bank-conflict free.
 * Other row sizes are stored row-major.  The layout is
 * private to this library (the reference exposes no K/V tensors to Python either,
 * cpp/chunk_attn/python_exports.cpp:16-21); ca_tile_elem_offset() is its definition.
 * Replaces the [n_heads, chunk_size, d_head] views of cpp/chunk_attn/chunk_allocator.cpp:43-55. */
CA_API int64_t ca_chunk_bytes(int n_heads, int d_head, int chunk_size, int dtype);
CA_API int64_t ca_tile_elem_offset(int d_head, int chunk_size, int dtype, int token, int elem);

/* ---- context --------------------------------------------------------------------------------
 * Replaces GPT::KernelContext (cpp/chunk_attn/kernel_cuda.h:9-55).  Owns the device work lists
 * and the partial-result scratch; borrows the pool.  `pool` must be 256-byte aligned. */
CA_API int ca_context_create(ca_context** out, int device, int n_heads, int d_head, int chunk_size,
                             int dtype, void* pool, int64_t max_chunks, int tpp_threshold);
CA_API void ca_context_destroy(ca_context* ctx);

/* 0: one launch walks shared runs and private tails together (default);
 * 1: the chunk-first items and the sequence-first items are launched as two kernels. */
#define CA_OPT_SPLIT_PHASES 1
/* number of persistent CTAs; 0 = two per SM */
#define CA_OPT_NUM_CTAS 2
/* how a sequence's private tail (one query row) is walked: 1 (default) on tensor cores, 16 tokens
 * per warp; 0 on CUDA cores with 128-bit shared-memory loads and warp-shuffle reductions */
#define CA_OPT_SEQ_FIRST_TENSOR 3
/* 1: the attention kernel records per-CTA nanosecond timestamps, read with ca_context_read_trace;
 * 2: as 1, but the tcgen05 kernel for wide runs accounts for the cycles of its two serial roles instead
 * (see ca_context_read_trace) */
#define CA_OPT_TRACE 4
/* programmatic dependent launches: bit 0, the merge kernel is set up while the attention kernel
 * drains; bit 1, the attention kernel is set up while the kernel before it in the stream finishes
 * (it waits for that kernel's completion before it touches global memory).  Default 3. */
#define CA_OPT_DEPENDENT_LAUNCH 5
/* Shared runs on the tcgen05 / TMEM kernel (tensor memory accumulators, tcgen05.mma fed by descriptor from the
 * staged tiles): 0 never, 1 (default) when walking the step's wide runs (more than 32 rows) with mma.sync would
 * take longer than half of what its unique K/V needs at HBM rate, 2 every shared run. */
#define CA_OPT_WIDE_RUNS 6
/* SM cycles a kernel may wait on one of its internal barriers before it gives up, records a status code
 * (ca_status_read) and returns; default 4e9, about two seconds.  The waits exist so that a lost copy or a
 * damaged work list ends in an error code instead of a hung GPU. */
#define CA_OPT_WAIT_LIMIT_CYCLES 7
/* 1: when a step has both wide shared runs and short private tails, their two kernels (independent work, one bound
 * by the tensor pipes, one by memory) run side by side on two streams; 0 (default): one after the other -- measured
 * on B200 the two orders take the same time within 3 %, the wide kernel's CTAs leave little room beside them. */
#define CA_OPT_OVERLAP_KERNELS 9
/* 1 (default): when EVERY row of the batch has a short private tail (the serving shape: many requests with short
 * suffixes over shared prompts), the tails are not all empty and the batch has at most 32 768 (row, head) pairs --
 * or the output goes to host memory (ca_attention_host) --, the short-tails kernel runs last in ca_attention / ca_attention_host /
 * ca_attention_to_peers, keeps each tail's partial in registers, combines it with the row's other partials and
 * stores the output rows itself: no merge launch, and the tails' partials never travel through memory.
 * 0: the tails are written as partial rows and the merge kernel combines them. */
#define CA_OPT_FINISH_IN_TAILS 10
/* Failure-path tests only: the CTA that draws item `value` of the next launches stops feeding its consumer
 * warps, whose bounded wait then runs out (status 1).  -1 (default) switches it off. */
#define CA_OPT_TEST_WITHHOLD_ITEM 8
CA_API int ca_context_set_option(ca_context* ctx, int option, int64_t value);

/* Rebuild and upload the work lists after the tree changed.
 * Replaces GPT::refresh_kernel_context (cpp/chunk_attn/kernel_cuda.h:67-69,
 * kernel_cuda.cu:1331-1445).  `infos` is a host array in the order the host's depth-first walk
 * produced it (parents before children); resets the appended-token counter to 0. */
CA_API int ca_refresh_kernel_context(ca_context* ctx, const ca_chunk_info* infos, int n_infos,
                                     int n_seqs, ca_stream stream);

/* Write one new K row and one new V row per sequence into that sequence's tail chunk, at slot
 * (tokens at last refresh + tokens appended since), then count the append.
 * k, v: device, [n_seqs, n_heads, d_head] contiguous.
 * Replaces GPT::append_kv (cpp/chunk_attn/kernel_cuda.h:65, kernel_cuda.cu:1273-1318) and the
 * `delta_tokens += 1` of cpp/chunk_attn/attention.cpp:112. */
CA_API int ca_append_kv(ca_context* ctx, const void* k, const void* v, int n_seqs, ca_stream stream);
CA_API int ca_context_delta_tokens(const ca_context* ctx);

/* Decode attention for the current batch: out[s, h, :] = softmax(q[s, h, :] K_s^T / sqrt(d)) V_s
 * over the context of row s.  q, out: device, [n_seqs, n_heads, d_head] contiguous.
 * Replaces GPT::attention (cpp/chunk_attn/kernel_cuda.h:57-61, kernel_cuda.cu:1320-1329). */
CA_API int ca_attention(ca_context* ctx, const void* q, void* out, int n_seqs, int partition,
                        ca_stream stream);

/* The same step for a caller whose queries and result live in HOST memory: copies q to the device,
 * runs ca_attention, has the last kernel store the result rows directly into `out_host` and waits
 * for the stream.  Page-locked buffers (cudaHostAlloc / cudaHostRegister / torch pin_memory) are
 * used in place; pageable ones are staged through pinned buffers of the context.  On return
 * out_host holds the result.  No counterpart in the reference, whose forward takes device tensors
 * (cpp/chunk_attn/attention.cpp:374-397); a caller with host data would wrap it in two copies. */
CA_API int ca_attention_host(ca_context* ctx, const void* q_host, void* out_host, int n_seqs, int partition,
                             ca_stream stream);

/* Head-sharded variant of ca_attention (one process per GPU, this context holds n_heads of
 * total_heads, starting at head_offset): the last kernel of the step (the merge kernel, or the short-tails
 * kernel when it finishes the rows, CA_OPT_FINISH_IN_TAILS) writes every output row straight into
 * each rank's full-width buffer peer_out[i], fp16 [n_seqs, total_heads, d_head], with plain stores
 * to peer memory over NVLink — compute and gather in one kernel, no collective library call.
 * peer_out is a HOST array of n_peers (<= 8) device pointers that this GPU can address (the rank's
 * own buffer included), 16-byte aligned; the caller orders the ranks before anyone reads (ca_peer_barrier on the
 * stream).  multicast_out, when not NULL, is a multicast address that maps the same buffer on every rank
 * (NVLink SHARP / NVLS, e.g. the multicast pointer of a torch symmetric-memory allocation): every row segment is
 * then written with ONE multimem.st that the switch replicates, instead of n_peers unicast stores.
 * No counterpart in the reference, which is single-device. */
CA_API int ca_attention_to_peers(ca_context* ctx, const void* q, void* const* peer_out, int n_peers,
                                 void* multicast_out, int total_heads, int head_offset, int n_seqs, ca_stream stream);

/* Barrier among the n_peers ranks of a node, on the stream: flag_arrays is a HOST array of device pointers,
 * flag_arrays[i] = rank i's array of n_peers 32-bit words in memory every rank can address (zero at the start).
 * Rank `rank` stores `epoch` (1, 2, 3, ... one more per barrier) into word `rank` of every array and waits until
 * all words of its own array have reached it.  The wait is bounded: after timeout_ns a rank gives up, stores 6
 * into *status (optional device word) and the kernel returns -- a peer that never arrives costs the time limit,
 * never a hung GPU.  Replaces the device-side barrier of the collective library for the fused gather; no
 * counterpart in the reference. */
CA_API int ca_peer_barrier(void* const* flag_arrays, int n_peers, int rank, uint32_t epoch, int64_t timeout_ns,
                           int32_t* status, ca_stream stream);

/* The two halves of ca_attention, separately launchable (profiling, tests):
 * ca_attn_partials = chunk-first over shared runs + sequence-first over private tails, emitting
 * per-piece partial outputs with their running max and sum-of-exponentials
 * (replaces attn_chunks_first / attn_seqs_first, cpp/chunk_attn/kernel_cuda.h:63-64);
 * ca_attn_merge = online-softmax combination of the partials of every (row, head)
 * (replaces the merge inlined in kernel_cuda.cu:962-984,1042-1085).
 * `phases`: 1 chunk-first items only, 2 sequence-first items only, 3 both. */
CA_API int ca_attn_partials(ca_context* ctx, const void* q, int n_seqs, int phases, ca_stream stream);
CA_API int ca_attn_merge(ca_context* ctx, void* out, int n_seqs, ca_stream stream);

/* Prefill ingestion: copy tokens [first_token, first_token + n_tokens) of a sequence's K and V
 * into freshly allocated chunks; token first_token + i goes to chunk_ids[i / chunk_size], row
 * i % chunk_size.  k, v: device, element strides (stride_token, stride_head, 1).
 * chunk_ids: HOST array of ceil(n_tokens / chunk_size) pool slots.
 * Replaces Chunk::append_tokens (cpp/chunk_attn/chunk.cpp:63-81) as driven by
 * Attention::add_seq (cpp/chunk_attn/attention.cpp:176-180). */
CA_API int ca_scatter_prefill(ca_context* ctx, const void* k, const void* v, int64_t stride_token,
                              int64_t stride_head, int first_token, int n_tokens,
                              const int32_t* chunk_ids, ca_stream stream);

/* Write single token rows: token i of k / v goes to row rows[i] of chunk chunk_ids[i] (HOST
 * arrays of n_tokens entries).  Used when a sequence forks into beams, each continuing with its
 * own token in its own copy of the tail.  Invalidates the context's work list (the tails' fill
 * counts changed unevenly): call ca_refresh_kernel_context before the next ca_attention.
 * Replaces Chunk::append_tokens as driven by Attention::append_completion
 * (cpp/chunk_attn/attention.cpp:227-261, chunk.cpp:63-81). */
CA_API int ca_scatter_rows(ca_context* ctx, const void* k, const void* v, int64_t stride_token,
                           int64_t stride_head, int n_tokens, const int32_t* chunk_ids, const int32_t* rows,
                           ca_stream stream);

/* Copy-on-write: clone whole chunks (all heads, K and V) src_ids[i] -> dst_ids[i].
 * src_ids, dst_ids: HOST arrays.  Replaces Chunk::deep_copy (cpp/chunk_attn/chunk.cpp:93-107). */
CA_API int ca_copy_chunks(ca_context* ctx, const int32_t* src_ids, const int32_t* dst_ids, int n,
                          ca_stream stream);

/* Read back chunk rows in the logical [n_heads][n_tokens][d_head] order (tests, debugging). */
CA_API int ca_read_chunk(ca_context* ctx, int chunk_id, int n_tokens, void* k_out, void* v_out,
                         ca_stream stream);

/* Device status word (0 = clean; first failure wins): 1 a consumer warp gave up waiting for a tile, 2 the
 * producer gave up waiting for a free stage, 3 copies still in flight at kernel exit, 4 an item or merge
 * entry of the work list named a slot, row, head or chunk out of range and was skipped (every index is
 * checked on the device against the sizes the context knows).  Synchronises the stream; returns
 * CA_ERR_DEVICE_STATUS when the word is not 0.  ca_status_clear zeroes it (stream-ordered) so that the
 * context can be used again after a reported failure. */
CA_API int ca_status_read(ca_context* ctx, ca_stream stream, int32_t* status);
CA_API int ca_status_clear(ca_context* ctx, ca_stream stream);

/* Per-CTA timestamps of the last attention launch when CA_OPT_TRACE is on (diagnostics): for CTA i,
 * out[8i..8i+3] = start, producer warp end, first consumer warp end, last consumer warp end, in ns
 * of the GPU's global timer; out[8i+4..8i+7] = SM cycles: first consumer warp waiting for tiles, the
 * same warp combining warps / storing partials, producer waiting for free stages, first consumer
 * warp in total.  `out` is a HOST array of 8 * max_ctas; returns the CTA count through n_ctas.
 * Synchronises the stream.
 * When the step's wide runs went to the tcgen05 kernel and nothing was left for the persistent kernel, the
 * trace is that kernel's: out[8i..8i+6] = entry, set-up done, first score tile ready, last P written, O
 * complete, partial rows stored, exit (ns).  With CA_OPT_TRACE = 2 entries 1-5 and 7 are SM cycles summed over
 * the CTA's tiles instead: the MMA thread issuing [1] the P V and [2] the Q K^T tcgen05.mma with their
 * commits, [3] that thread waiting for P and the V tile, [4] the first softmax thread waiting for a score
 * tile, [5] that thread from scores ready to P handed over, [7] bits 0-47 the MMA thread waiting for the K
 * tile, bits 48-63 the SM the CTA ran on. */
CA_API int ca_context_read_trace(ca_context* ctx, uint64_t* out, int max_ctas, int* n_ctas, ca_stream stream);

/* Per-step counters of the current work list (the roofline metric is computed from them). */
typedef struct ca_plan_stats {
    int64_t unique_kv_bytes;   /* sum over live chunks of n_tokens * n_heads * d_head * 2 * sizeof */
    int32_t n_chunks;          /* live non-root chunks, empty tails included                      */
    int32_t n_shared_chunks;   /* chunks walked by the chunk-first phase                          */
    int32_t n_runs;            /* maximal chains of shared chunks with identical sharers          */
    int32_t n_items;           /* pieces of work, (item, head) pairs (at most 9 tiles each); the item
                                  array itself holds n_items / n_heads entries                    */
    int32_t n_slots;           /* partial rows, all heads                                         */
    int32_t n_ctas;            /* persistent CTAs launched                                        */
    int32_t fast_path;         /* 1 when the tensor-core/TMA kernels serve this geometry          */
    int32_t kernels_per_step;  /* launches one ca_attention call makes (from ca_context_stats: as the
                                  context would launch them now, options and appended tokens included) */
    int32_t n_items_cf;        /* how many items are chunk-first items (they come first)          */
    int32_t n_items_short;     /* how many items, after the persistent kernel's, are short private tails
                                  walked by the half-warp-per-item kernel instead of the persistent one */
    int32_t n_items_wide;      /* how many items, at the end of the list, are pieces of wide shared runs
                                  for the tcgen05 / TMEM kernel                                       */
} ca_plan_stats;
CA_API int ca_context_stats(const ca_context* ctx, ca_plan_stats* out);

/* ---- element-wise companions (`chunk_attn.ops`) ----------------------------------------------------
 * The three kernels the reference's model code imports from the same extension module
 * (cpp/chunk_attn/python_exports_ops.cpp:11-19).  fp16 or fp32, device pointers, rows contiguous.
 *
 * ca_rms_norm: out[t, :] = round(input[t, :] * rsqrt(mean(input[t, :]^2) + epsilon)) * weight
 *   (replaces vllm::rms_norm, cpp/chunk_attn/layernorm_kernels.cu:83-105).
 * ca_fused_add_rms_norm: residual += input (rounded), then input = rms_norm(residual) * weight, in place
 *   (replaces vllm::fused_add_rms_norm, layernorm_kernels.cu:107-129).
 * ca_rotary_embedding: rotates the first rot_dim elements of every head of query and key in place by the
 *   angle of the token's position; cos_sin_cache is [max_position, rot_dim] = [cos | sin] per position;
 *   query_stride / key_stride are the element strides between tokens; is_neox pairs (i, i + rot_dim/2),
 *   otherwise (2i, 2i + 1) (replaces vllm::rotary_embedding, cpp/chunk_attn/pos_encoding_kernels.cu:94-139).
 *   max_position is the number of rows of cos_sin_cache: a token whose position lies outside [0, max_position)
 *   is left unrotated and, when `status` (an optional device word, first failure wins) is given, 5 is
 *   stored there; the reference reads past its table in that case.  max_position <= 0 switches the check off. */
CA_API int ca_rms_norm(void* out, const void* input, const void* weight, float epsilon, int64_t num_tokens,
                       int hidden_size, int dtype, ca_stream stream);
CA_API int ca_fused_add_rms_norm(void* input, void* residual, const void* weight, float epsilon,
                                 int64_t num_tokens, int hidden_size, int dtype, ca_stream stream);
CA_API int ca_rotary_embedding(const int64_t* positions, void* query, void* key, const void* cos_sin_cache,
                               int rot_dim, int64_t query_stride, int64_t key_stride, int num_heads,
                               int num_kv_heads, int head_size, int64_t num_tokens, int is_neox, int dtype,
                               int64_t max_position, int32_t* status, ca_stream stream);

/* ---- allocation-free decode step ---------------------------------------------------------------
 * No counterpart in the reference: this entry point exists for callers that cannot allocate device
 * memory when they reach the decode step, for instance a plugin inside a serving process whose
 * framework reserved the whole GPU for its own arena at start-up (a raw cudaMalloc then fails or
 * is forbidden), or a latency-critical loop that cannot take the device-wide synchronisation that
 * cudaMalloc / cudaFree imply.  ca_attention keeps its partial results in scratch that
 * ca_refresh_kernel_context grows with cudaMalloc; ca_attention_static keeps them in a fixed
 * __device__ array inside the library (CA_STATIC_MAX_SLOTS partial rows of 520 bytes, about
 * 8.1 MiB, resident on every GPU that loads the library until the process exits) and allocates
 * nothing: no cudaMalloc, no cudaFree, no allocating library routine.
 *
 * Same computation and geometry as the tensor-core path of ca_attention (fp16, d_head 128,
 * chunk_size 64).  The caller passes inputs and outputs only, all in device memory it owns, on the
 * calling thread's current device:
 *   pool            the chunk pool (layout above), 256-byte aligned
 *   q, out          [n_seqs, n_heads, 128] fp16, contiguous
 *   items, merge_off, merge_slots   the work list: the arrays ca_plan_build produces with wide_runs = 0
 *                   (this entry point launches the persistent kernel only)
 *                   (CA_PLAN_ITEMS with n_items entries of 16 ints -- the array holds every item once for all
 *                   heads, so n_items = ca_plan_stats.n_items / n_heads --, CA_PLAN_MERGE_OFF,
 *                   CA_PLAN_MERGE_SLOTS), copied to the device by the caller
 *   n_ctas          persistent CTAs to launch (ca_plan_stats.n_ctas)
 *   n_slots         ca_plan_stats.n_slots of that plan; above CA_STATIC_MAX_SLOTS the call is refused
 *                   with CA_ERR_INVALID and a message naming both numbers
 *   delta_tokens    tokens appended to every tail since the plan was built
 *   status          optional device word for the kernels' status (0 = clean, codes as for ca_status_read);
 *                   NULL selects a word inside the library, read back with ca_attention_static_status.
 *                   It is cleared at the start of each call.
 *
 * The work list is read from device memory the host cannot inspect, so the kernels check it: an item or merge
 * entry that names a partial row >= n_slots, a row >= n_seqs or a head >= n_heads is skipped and status 4 is
 * recorded (the output rows concerned are then wrong, but nothing outside the scratch, q or out is touched).
 * Chunk numbers cannot be checked here, because the pool's size is not an argument: a work list built for
 * another pool is the caller's responsibility.
 *
 * The first call on a device looks up the device address of the scratch (cudaGetSymbolAddress)
 * and sets the kernel's shared-memory attribute; make that first call before any stream capture, and, since the
 * library image with its 8.1 MiB array is mapped onto the device when the library's first kernel or symbol is
 * touched (CUDA loads modules lazily), before the host framework has taken all of the GPU's memory.
 * All calls on a device share the one scratch array, which still holds the previous call's
 * partial rows when the next call starts (none of them needs clearing: every row a merge list names
 * is rewritten first; the status word and the item counter of the self-scheduling kernel do, and every call
 * clears them on its stream before its kernels run, so a call does not depend on how the previous one ended).
 * delta_tokens is an argument of the launch: a recorded call replays with the value it was recorded with.
 * Two calls that overlap on the GPU (different streams, or different threads)
 * therefore race on it: keep calls on one device stream-ordered. */
#define CA_STATIC_MAX_SLOTS 16384
CA_API int ca_attention_static(const void* pool, int n_heads, const void* q, void* out, int n_seqs,
                               const int32_t* items, int n_items, int n_ctas, const int32_t* merge_off,
                               const int32_t* merge_slots, int n_slots, int delta_tokens,
                               int32_t* status, ca_stream stream);
/* The library's own status word of ca_attention_static calls made with status = NULL on the current device
 * (synchronises the stream).  No counterpart in the reference. */
CA_API int ca_attention_static_status(int32_t* status, ca_stream stream);

/* ---- host-only planner (no GPU needed) -------------------------------------------------------
 * The work-list builder used by ca_refresh_kernel_context, exposed so that it can be checked on
 * a machine without a GPU.  Arrays are owned by the plan. */
#define CA_PLAN_ITEMS 0          /* int32[][16], every item ONCE for all heads (the kernels expand: piece v is
                                    item v / n_heads for head v % n_heads): n_tiles, 0, row_begin, n_rows,
                                    slot_base (head h's partial rows start at slot_base * n_heads + h, stride
                                    n_heads), flags (bit 0: last tile is a tail; bit 1: an item of the tcgen05
                                    kernel; bits 8..: token splits, 0 = CUDA-core walk), last_tokens, pool slots
                                    of up to 9 tiles (wide item: offset into CA_PLAN_WIDE_CHUNKS)                */
#define CA_PLAN_MERGE_OFF 3      /* int32[n_seqs + 1]: one list per ROW, shared by the row's heads               */
#define CA_PLAN_MERGE_SLOTS 4    /* int32[]: partial rows as numbered per item; head h's is entry * n_heads + h  */
#define CA_PLAN_PATH_OFF 5       /* int32[n_seqs + 1]   (sequence-first-only path lists)         */
#define CA_PLAN_PATH_CHUNKS 6    /* int32[]: pool slots root -> leaf                             */
#define CA_PLAN_PATH_TOKENS 7    /* int32[]: tokens in that chunk at refresh                     */
#define CA_PLAN_TAIL_CHUNK 8     /* int32[n_seqs]                                                */
#define CA_PLAN_TAIL_TOKENS 9    /* int32[n_seqs]                                                */
#define CA_PLAN_WIDE_CHUNKS 10   /* int32[]: chunk lists of the wide items (an item's first chunk entry
                                    is its offset here); empty when wide_runs is 0               */
/* wide_runs: the meaning of CA_OPT_WIDE_RUNS (0 never, 1 by cost, 2 every shared run) */
CA_API int ca_plan_build(ca_plan** out, const ca_chunk_info* infos, int n_infos, int n_seqs,
                         int n_heads, int chunk_size, int tpp_threshold, int n_ctas,
                         int64_t max_chunks, int split_phases, int seq_first_tensor, int wide_runs);
CA_API int ca_plan_array(const ca_plan* plan, int which, const int32_t** data, int64_t* count);
CA_API int ca_plan_stats_get(const ca_plan* plan, ca_plan_stats* out);
/* One work list for several contexts.  The caches of a model's layers see the same tree at every step, so
 * their work lists are identical: build the list once with the parameters of one context (geometry,
 * options, CTA count) and upload it into each of them.  ca_refresh_from_plan is ca_refresh_kernel_context
 * without the planning; it refuses a plan built for another geometry, pool size or set of options.  The plan
 * may be destroyed as soon as the call returns.  *out == NULL makes a new plan; otherwise the plan *out points
 * to is rebuilt in place (its buffers are reused; after a failed rebuild its contents are unspecified).  No counterpart in the reference, which rebuilds per layer
 * (src/chunk_attn/models/llama_hf/modeling_llama.py:101-106). */
CA_API int ca_plan_build_for_context(const ca_context* ctx, ca_plan** out, const ca_chunk_info* infos, int n_infos,
                                     int n_seqs);
CA_API int ca_refresh_from_plan(ca_context* ctx, const ca_plan* plan, ca_stream stream);
CA_API void ca_plan_destroy(ca_plan* plan);

#ifdef __cplusplus
}
#endif
#endif /* CHUNK_ATTN_B200_H_ */
