/*
 * C ABI of the B200 (sm_100a) paged FP8-e4m3 KV-cache GQA decode-attention library
 * (libpaged_fp8_decode.so).
 *
 * Plain pointers and sizes only: no torch types.  Every entry point is asynchronous on
 * the CUDA stream it is given, allocates nothing unless stated, returns 0 on success or a
 * negative PFD_ERR_* code, and records a message readable with pfd_last_error().
 *
 * File/line citations name the interface of the reference project
 * (Kevin-Li-2025/single-gpu-inference-lab) that each entry point replaces.
 */
#ifndef PAGED_FP8_DECODE_H_
#define PAGED_FP8_DECODE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PFD_ABI_VERSION 4

/* element types of query / output / partial_output */
#define PFD_DTYPE_F32 0
#define PFD_DTYPE_F16 1
#define PFD_DTYPE_BF16 2

#define PFD_OK 0
#define PFD_ERR_INVALID (-1)     /* bad argument; nothing was launched            */
#define PFD_ERR_UNSUPPORTED (-2) /* geometry outside what the kernels implement   */
#define PFD_ERR_CUDA (-3)        /* a CUDA runtime / driver call failed           */
#define PFD_ERR_DEVICE (-4)      /* a kernel recorded an error status             */

/* flags */
#define PFD_FLAG_NO_TMA 1u        /* stream K/V with plain 16-byte global loads instead of TMA */
#define PFD_FLAG_NO_DIRECT_OUT 2u /* always go through the partial workspace + merge kernel    */
#define PFD_FLAG_PARTIAL_ONLY 4u  /* launch the split-KV partial kernel only (kernel timing)   */
#define PFD_FLAG_FIXED_SPLITS 8u  /* always use the fixed-split grid + merge kernel             */
#define PFD_FLAG_EARLY_METADATA 32u /* the caller vouches that the kernel preceding this call in
                                     the stream writes neither seq_lens, block_table nor the plan
                                     (true for every layer of a model step, whose metadata is
                                     built once; not true for a call enqueued right behind
                                     pfd_plan_decode): the kernels may then read them while that
                                     kernel drains                                               */
#define PFD_FLAG_SINGLE_LAUNCH 64u /* with `plan`: the balanced kernel also combines the pieces of cut
                                     sequences (the warp whose piece arrives last does it), so the
                                     step is one launch and no merge kernel follows; measured slower
                                     on B200 than the two launches, for callers that want one node  */
#define PFD_FLAG_ALL_IN_GROUPS 128u /* grouped shared-prefix decode: the caller has read word 4 of the
                                     groups buffer and it equals the batch, i.e. no request is outside
                                     the groups.  The split-KV pass over the short suffixes may then
                                     run as small CTAs beside the dense prefix pass instead of behind
                                     it.  Only a hint about speed: with a request in no group after
                                     all the result is the same, that request's share just takes
                                     longer                                                         */
#define PFD_FLAG_EARLY_KV 256u /* with PFD_FLAG_EARLY_METADATA and a plan: the caller also vouches that the
                                kernel preceding this call in the stream writes K/V only into the LAST page of
                                each sequence (a decode step's cache append writes one token, at position
                                seq_len - 1) and nothing of the workspace: the balanced kernel then starts
                                streaming every other page while that kernel drains and fetches the page pairs
                                that end a sequence, and the queries, after it has completed                   */
/*
 * Kernel selection.  For head_dim 128, at most 8 query heads per kv head, a TMA-describable
 * cache and a dense f32 workspace of at least pfd_balanced_workspace_rows() rows the balanced
 * persistent kernel + its merge kernel run (split_size then only sizes the workspace); with `plan`
 * set both read their work split instead of deriving it.  Anything else, or
 * PFD_FLAG_FIXED_SPLITS, runs the fixed-split grid + merge kernel.
 */

/*
 * Stream order.  Every kernel of a call is launched with programmatic stream serialisation: it may
 * become resident while the kernel in front of it in the stream drains, but it reads and writes
 * nothing before that kernel has completed -- except, under PFD_FLAG_EARLY_METADATA, seq_lens,
 * block_table and the plan.  The last kernel of a call completes only after every kernel of the
 * call has (whatever rows it had to merge itself), so whoever enqueues work behind a call, with or
 * without programmatic launch attributes, finds the call's output complete.  Nothing is allocated,
 * nothing synchronises with the host; the entry points that take a workspace are captured in CUDA
 * graphs by this repository's tests.
 */

/*
 * Operands of one decode-attention layer-step.
 *
 * Replaces the argument list of
 *   l20_paged_decode_fp8_e4m3_split_out_cuda(query, key_cache, value_cache, block_table,
 *       seq_lens, partial_output, partial_max, partial_sum, output, k_scale, v_scale,
 *       max_seq_len, split_size)      integrations/vllm/cuda/l20_paged_decode.cu:651-664
 * and of the Triton launcher l20_paged_split_kv_attention_fp8
 *                                      integrations/vllm/l20_paged_split_kv.py:597-695
 * (which, unlike the CUDA launcher, honours cache strides: :665-668).
 *
 * Layouts (all device pointers):
 *   query, output   [batch, num_q_heads, head_dim]   f16 or bf16, innermost contiguous
 *   key/value_cache [pages, page_size=16, num_kv_heads, head_dim] e4m3 bytes addressed by
 *                   (page, token, head) byte strides; head_dim bytes contiguous.  NHD (the
 *                   reference op's layout) and HND are both just strides.
 *   block_table     [batch, >= ceil(max_seq_len/16)] int32 physical page ids
 *   seq_lens        [batch] int32
 *   partial_output  [batch, num_q_heads, workspace_splits, head_dim] (partial_dtype),
 *   partial_max/sum [batch, num_q_heads, workspace_splits] f32; workspace_splits >=
 *                   ceil((max_seq_len - kv_start) / split_size).  May be NULL when that
 *                   quotient is 1.
 * Split s of sequence b covers tokens [kv_start + s*split_size, kv_start + (s+1)*split_size)
 * clipped to [0, seq_lens[b]).  partial_max is in natural-log units, partial_output is the
 * un-normalised sum of p*v (v already scaled), as in the reference kernels.
 */
/*
 * KV-range exchange between the GPUs of one node (no counterpart in the reference, which is
 * single-GPU).  Every rank holds a KV range of every sequence; its decode call yields packed
 * (o, m, l) rows for that range, which every rank needs for the final merge.  With `exchange`
 * set in pfd_decode_args the kernels that finish those rows store them straight into slot
 * `rank` of EVERY rank's receive buffer (plain stores through peer mappings over NVLink).  Each
 * 8-byte word of a row holds an f32 value in its low half and the step's tag in its high half
 * and arrives whole, so the receiver needs no flag: pfd_exchange_merge() polls (bounded) the
 * words of this rank's own buffer, row by row, until they carry the tag, and merges them.  No
 * collective call, no fence, no remote load.
 *
 *   recv[p]   rank p's receive buffer, 8-byte words [2][world][batch * num_q_heads][PFD_XCH_ROW]
 *             (a row: o[head_dim], m, l), as mapped in THIS process (recv[rank] is local memory,
 *             the others peer memory); zero before the first step
 *   control   two local 32-bit words, zero before the first step: steps completed, merge CTAs done
 * The step's tag lives on the device (control[0] + 1, wrapping), so that a step captured in a
 * CUDA graph can be replayed: pfd_exchange_merge()'s kernel advances it, succeed or not, and
 * every rank must therefore run exactly one decode call (at most) and one pfd_exchange_merge()
 * per step.  The tag's lowest bit selects the half of the buffer, so that a rank one step ahead
 * never overwrites what a slower rank still merges; no rank can get further ahead than that,
 * because its next merge waits for the slower rank's rows.
 * Allocate with pfd_exchange_alloc() / map the peers' with pfd_exchange_open() (or any other way
 * that yields peer-accessible device memory).  Needs the balanced kernel + merge kernel (head_dim
 * 128, FP8 caches, at most 8 query heads per kv head, no PFD_FLAG_SINGLE_LAUNCH / FIXED_SPLITS);
 * other calls are refused.  world <= 8.
 */
#define PFD_XCH_ROW 130
typedef struct pfd_exchange {
  int32_t world, rank;
  void* recv[8];
  void* control;
} pfd_exchange;

typedef struct pfd_decode_args {
  uint32_t struct_size; /* sizeof(pfd_decode_args): lets the library reject a stale caller */
  uint32_t flags;

  int32_t batch;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_dim;  /* 64 or 128 */
  int32_t page_size; /* 16 */
  int32_t max_seq_len;
  int32_t split_size; /* multiple of 16, >= 16 */
  int32_t kv_start;   /* first token attended (0 for a normal decode step) */
  int32_t query_dtype;   /* PFD_DTYPE_F16 | PFD_DTYPE_BF16; output uses the same */
  int32_t partial_dtype; /* PFD_DTYPE_F32 | F16 | BF16 */
  float sm_scale;        /* softmax scale; 0 selects head_dim^-0.5 */
  float k_scale;         /* used when k_scale_per_head == NULL */
  float v_scale;         /* used when v_scale_per_head == NULL */
  int32_t workspace_splits;

  const void* query;
  int64_t q_stride_b, q_stride_h; /* elements */
  const void* key_cache;
  const void* value_cache;
  int64_t num_pages;
  int64_t k_stride_page, k_stride_token, k_stride_head; /* bytes */
  int64_t v_stride_page, v_stride_token, v_stride_head; /* bytes */
  const int32_t* block_table;
  int64_t bt_stride_b; /* elements */
  const int32_t* seq_lens;
  const float* k_scale_per_head; /* [num_kv_heads] device floats, or NULL */
  const float* v_scale_per_head;

  void* partial_output;
  float* partial_max;
  float* partial_sum;
  int64_t partial_stride_b, partial_stride_h, partial_stride_s; /* elements, of partial_max */

  void* output; /* [batch, num_q_heads, head_dim], may be NULL if packed_output is set */
  int64_t o_stride_b, o_stride_h; /* elements */
  /* optional [batch, num_q_heads, head_dim + 2] f32: merged (o un-normalised, m, l) of the
   * attended range, the exchange format for a KV range split across GPUs */
  float* packed_output;

  void* stream; /* cudaStream_t */

  /* Optional [batch + 1] int32: with it, block_table is a flat list of page ids and the pages of
   * sequence b are block_table[page_indptr[b] ...] (FlashInfer's indptr / indices addressing,
   * l20_paged_decode_split_indices_out_cuda, integrations/vllm/cuda/l20_paged_decode.cu:600-649);
   * bt_stride_b is ignored.  Only the balanced persistent kernel reads it: a call that would
   * run on the fixed-split grid or the shared-prefix pass is refused with PFD_ERR_UNSUPPORTED. */
  const int32_t* page_indptr;

  /* Optional device buffer written by pfd_plan_decode() for the same batch, lengths, block table,
   * kv_start, head counts and workspace: the balanced persistent kernel and its merge kernel then
   * read their work split from it (and PFD_FLAG_SINGLE_LAUNCH becomes available).  NULL, or a
   * call that does not run the balanced kernel: ignored. */
  void* plan;

  /* Optional: push the packed (o, m, l) rows of this call to every rank (see pfd_exchange).
   * packed_output and output are then ignored; the result comes from pfd_exchange_merge(). */
  const pfd_exchange* exchange;
} pfd_decode_args;

/*
 * One decode-attention layer-step: split-KV partial kernel + LSE merge kernel.
 * Replaces l20_paged_decode_fp8_e4m3_split_out_cuda
 * (integrations/vllm/cuda/l20_paged_decode.cu:651-725) and the two Triton launches of
 * l20_paged_split_kv_attention_fp8 (integrations/vllm/l20_paged_split_kv.py:652-694).
 */
int pfd_paged_decode_fp8_e4m3_split_out(const pfd_decode_args* args);

/*
 * The non-quantised sibling: one decode-attention layer-step over K/V caches stored in the
 * query's own 16-bit type (fp16 or bf16), head_dim 128, at most 8 query heads per KV head.
 * Replaces l20_paged_decode_split_out_cuda (integrations/vllm/cuda/l20_paged_decode.cu:549-600;
 * op schema l20_paged_decode.cpp:121-127).  Same struct; k_stride_* / v_stride_* count
 * elements of the cache type, k_scale / v_scale and the per-head scale pointers are ignored.
 * It always runs the balanced persistent kernel.  The workspace (f32, f16 or bf16 partials,
 * dense [batch, num_q_heads, workspace_splits]) is used as a flat list of rows; any workspace of
 * at least 2 * num_q_heads rows works, one of pfd_balanced_workspace_rows() rows or more lets
 * every SM take part.
 */
int pfd_paged_decode_kv16_split_out(const pfd_decode_args* args);

/*
 * Plan of a model step's decode-attention calls: everything the balanced persistent kernel
 * derives from seq_lens and block_table alone (pair prefix sum, every warp group's range and
 * first page ids, arrival counters for the pieces of cut sequences), computed once by a small
 * kernel on args->stream and then shared by the calls of all layers, which pass it as
 * args->plan.  `cache_elem_bytes` is 1 for pfd_paged_decode_fp8_e4m3_split_out and 2 for
 * pfd_paged_decode_kv16_split_out (they run different warp counts).  Reads of `args`: batch,
 * head counts, head_dim, kv_start, the workspace fields, seq_lens, block_table / page_indptr,
 * stream.  Returns PFD_ERR_UNSUPPORTED (nothing launched) when the call would not run the
 * balanced kernel.  A plan stays valid while those inputs do not change; using it with other
 * values makes the kernel set device status 2 and write nothing.  Calls that share a plan must
 * not overlap on the GPU (same stream, or ordered by events).  The reference has no counterpart:
 * its kernels take one CTA per (query head, split, sequence) and need no work split.
 */
int64_t pfd_plan_bytes(int32_t batch, int32_t num_kv_heads);
int pfd_plan_decode(const pfd_decode_args* args, int32_t cache_elem_bytes, void* plan, int64_t plan_bytes);

/*
 * Rows of (o, m, l) the workspace must hold for the balanced persistent kernel on the current device:
 * batch * num_q_heads * workspace_splits >= this.  The balanced kernel gives every group of
 * num_kv_heads warps two slots of num_q_heads rows.  Negative on error.  No counterpart in the
 * reference, whose workspace is always [B, Hq, splits].
 */
int64_t pfd_balanced_workspace_rows(int32_t num_q_heads, int32_t num_kv_heads);

/*
 * Allocation-free variant of pfd_paged_decode_fp8_e4m3_split_out.  It has no counterpart in
 * the reference project, whose launcher always takes the partial workspace from its caller.
 *
 * Some hosts of this library cannot provide that workspace: an inference engine that measured
 * free HBM at start-up and handed all of it to its KV-cache pool has nothing left for a later
 * cudaMalloc (and cudaMalloc would stall the whole device while it runs), and a host written
 * in C, Go or Rust has no tensor allocator to borrow from.  For them the split-KV partials
 * (partial_output, partial_max, partial_sum of `args`, which are ignored here) live in a fixed
 * array of PFD_NOALLOC_SCRATCH_BYTES inside the library image; every GPU that loads the
 * library carries that array until the process exits.  Inputs and outputs are still the
 * caller's.  The call is refused with PFD_ERR_UNSUPPORTED when
 *   batch * num_q_heads * ceil((max_seq_len - kv_start) / split_size) * (head_dim + 2) * 4
 * exceeds the array (a larger split_size shrinks the need; a request whose longest sequence fits
 * one split writes its rows directly, touches no scratch and is never refused for size).  It
 * always runs the fixed-split grid, so it takes a block table only (page_indptr is refused) and
 * ignores `plan`; PFD_FLAG_PARTIAL_ONLY is refused, since the partials would stay inside the
 * library.  No cudaMalloc, cudaFree or other allocating routine is called, on the first call or
 * later.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress)
 * with the caller's current device, which must be the device of `args->stream`; make that
 * first call before any stream capture begins.  All calls on a device share the one array and
 * nothing in it needs clearing between calls (every live split is written before it is read),
 * but two calls whose kernels overlap on the GPU (different streams, or different host threads
 * on different streams) would overwrite each other's partials: serialise them.
 */
#define PFD_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)
int pfd_paged_decode_fp8_e4m3_split_out_noalloc(const pfd_decode_args* args);

/*
 * Decode step of a batch whose requests ALL share one paged prefix: block_table[b][0 ..
 * prefix_len/16) names the same physical pages for every b (the caller checks that, e.g. with
 * the grouping of find_l20_shared_prefix_groups,
 * integrations/vllm/l20_shared_prefix_decode_dispatch.py:52-76).  Three kernels:
 *   1. dense prefix pass on tcgen05 tensor cores: 128 (request, q head) rows x 256 prefix tokens
 *      per CTA, K/V converted e4m3 -> f16 on the way into shared memory, accumulators in TMEM;
 *      replaces _shared_paged_prefix_gqa_partial_kernel
 *      (src/l20_stack/ops/triton_decode_attention.py:704-813);
 *   2. suffix pass: the split-KV partial kernel with kv_start = prefix_len
 *      (replaces _paged_suffix_gqa_partial_kernel, :815-912);
 *   3. the LSE merge over prefix chunks and suffix splits
 *      (replaces _prefix_suffix_gqa_reduce_kernel, :652-702).
 * Needs head_dim 128, prefix_len a multiple of 16, an f32 workspace with
 * workspace_splits >= ceil(prefix_len / 256) + ceil((max_seq_len - prefix_len) / split_size),
 * and 16-byte aligned query rows.  kv_start must be 0.
 */
int pfd_shared_prefix_decode_fp8_e4m3(const pfd_decode_args* args, int32_t prefix_len);

/*
 * LSE merge of `num_parts` packed partials [num_parts, rows, head_dim + 2] f32
 * (o un-normalised, m natural-log, l) into output [rows, head_dim] of `out_dtype`.
 * Same maths as _paged_split_kv_reduce (integrations/vllm/l20_paged_split_kv.py:459-488)
 * and paged_decode_merge_kernel (integrations/vllm/cuda/l20_paged_decode.cu:424-463), with
 * no limit on the number of parts.  Used after the all-gather of a KV-range split.
 */
int pfd_merge_packed(const float* packed, int32_t num_parts, int64_t rows, int32_t head_dim,
                     void* output, int32_t out_dtype, void* stream);

/*
 * Receiving side of a KV-range exchange step: one kernel on `stream` (enqueue it behind the decode
 * call of the same step), one warp per row, that waits until the words of all `world` ranks' copies
 * of the row in this rank's receive buffer carry the step's tag -- at most the wait limit
 * (pfd_set_wait_limit_ns); on expiry device status 4 is set and the row is left alone -- and then
 * LSE-merges the `world` packed partials of the row into output [rows, head_dim] of `out_dtype`.
 * Same maths as pfd_merge_packed.
 */
int pfd_exchange_merge(const pfd_exchange* exchange, int64_t rows, int32_t head_dim, void* output,
                       int32_t out_dtype, void* stream);

/*
 * Memory for one rank's side of the exchange: cudaMalloc of `bytes` (zero-filled), with the
 * 64-byte CUDA IPC handle that the other ranks' processes turn into a peer mapping with
 * pfd_exchange_open().  pfd_exchange_bytes() is what the receive buffer + control words of one
 * rank need; the control words start at pfd_exchange_control_offset() bytes.
 * These four allocate / map / free device memory (the decode entry points never do).
 */
typedef struct pfd_ipc_handle { unsigned char bytes[64]; } pfd_ipc_handle;
int64_t pfd_exchange_bytes(int32_t world, int64_t rows, int32_t head_dim);
int64_t pfd_exchange_control_offset(int32_t world, int64_t rows, int32_t head_dim);
int pfd_exchange_alloc(int64_t bytes, void** ptr, pfd_ipc_handle* handle);
int pfd_exchange_open(const pfd_ipc_handle* handle, void** peer_ptr);
int pfd_exchange_close(void* peer_ptr);
int pfd_exchange_free(void* ptr);

/*
 * Shared-prefix groups of a decode batch, found on the device (three small kernels on `stream`,
 * no host copy): requests whose first `prefix length` tokens sit in the same pages.  Same key and
 * the same filters as the reference's host-side find_l20_shared_prefix_groups
 * (integrations/vllm/l20_shared_prefix_decode_dispatch.py:41-76): (prefix length, chain of the
 * prefix's block ids); prefixes shorter than min_prefix_len and groups of fewer than min_batch
 * requests are dropped; groups are numbered by their first member, members ascend.  The prefix
 * length of row b is prefix_lengths[b] (device int32), or uniform_prefix_len when that is NULL
 * and this positive.  With neither, the prefixes are DISCOVERED from the table and seq_lens: rows
 * are keyed on their first ceil(min_prefix_len / 16) pages, and a group's prefix is as long as all
 * its members agree with its first member, in whole pages that every member has filled.  (The
 * reference's trace_l20_shared_prefix_decode_candidate, :245-315, tries the one candidate
 * floor(min(seq_lens) / 16) * 16, which finds nothing once the requests have private suffixes of
 * a page or more.)  Unlike the reference, which dispatches only when one group spans the batch,
 * any number of groups (up to max_groups; later ones are left out) plus requests in no group come
 * out.
 *
 * `groups` (device, pfd_prefix_groups_bytes() bytes) as int32 words: [0] magic, [1] batch,
 * [2] max_groups, [3] number of groups, [4] rows in groups, [5..7] 0, then row_prefix_len[batch]
 * (0 = in no group), row_group[batch] (-1 = none), group_offsets[max_groups + 1],
 * group_prefix_len[max_groups], group_rows[batch] (group g's requests are
 * group_rows[group_offsets[g] .. group_offsets[g + 1])), then scratch.  batch <= 2048.
 */
int64_t pfd_prefix_groups_bytes(int32_t batch, int32_t max_groups);
int pfd_group_shared_prefixes(const int32_t* block_table, int64_t bt_stride_b, int32_t bt_cols,
                              const int32_t* prefix_lengths, int32_t uniform_prefix_len, const int32_t* seq_lens,
                              int32_t batch, int32_t min_batch, int32_t min_prefix_len, int32_t max_groups,
                              void* groups, int64_t groups_bytes, void* stream);

/*
 * Decode step of a batch with any number of shared-prefix groups (and requests in none), all
 * decided on the device: `groups` is the buffer pfd_group_shared_prefixes() filled for this batch
 * (same batch size, same max_groups; made once per model step, read by every layer's call).  The
 * dense tensor-core pass runs per group over the group's request list, the split-KV pass covers
 * every request from the end of its group's prefix (from token 0 for a request in no group), one
 * merge.  A prefix is used up to a multiple of 16 tokens and up to min(max_prefix_len,
 * max_seq_len); what lies beyond goes through the split-KV pass, so any bound is safe and a
 * tight one saves idle CTAs.  Every member of a group must be at least as long as the group's
 * prefix.  max_suffix_len bounds what a request IN a group has behind its prefix (0 = unknown: the
 * whole context); the split-KV grid is sized for it, ceil(max_suffix_len / split_size) splits, and
 * a request in no group covers its whole context with as many, longer, splits.  A member whose
 * suffix exceeds the bound would be attended only up to it (device status 5 reports it): give a true bound (max_seq_len minus
 * the smallest prefix a group can have, i.e. the min_prefix_len of the grouping call).  The
 * workspace needs ceil(min(max_prefix_len, max_seq_len) / 256) +
 * ceil(min(max_suffix_len or max_seq_len, max_seq_len) / split_size) slots on its split axis.  The reference has no counterpart: its
 * dispatch stops at one group spanning the batch
 * (integrations/vllm/l20_shared_prefix_decode_dispatch.py:122-159).
 */
int pfd_shared_prefix_decode_grouped_fp8_e4m3(const pfd_decode_args* args, const void* groups, int32_t max_groups,
                                              int32_t max_prefix_len, int32_t max_suffix_len);

/*
 * Debug / parity entry: writes, for every (sequence, token < max_seq_len), the cache slot
 * index page*16 + token%16 that the kernels' address function resolves (-1 beyond the
 * sequence) into slots[batch, max_seq_len] (int64).  Counterpart of the gather
 * `physical = table[b, t // 16]; offsets = t % 16`
 * (scripts/smoke_cuda_paged_fp8_decode_op.py:29-33).
 */
int pfd_resolve_slots(const int32_t* block_table, int64_t bt_stride_b, const int32_t* seq_lens,
                      int32_t batch, int32_t max_seq_len, int64_t* slots, void* stream);

/*
 * Synchronises with the current device and reads (then clears) the error word the kernels set
 * when a bounded wait gave up: 0 = none, 1 = a TMA copy did not complete in time (the step's
 * output is then undefined), 2 = args->plan was made for other inputs (nothing was written),
 * 3 = the tensor cores of the dense shared-prefix pass did not complete in time (output undefined),
 * 4 = a rank's rows of a KV-range exchange step did not arrive in time (those rows were not merged),
 * 5 = grouped shared-prefix decode: a request's suffix is longer than max_suffix_len (its output is wrong).
 * The kernels never trap and never spin without a limit.
 */
int pfd_device_status(int32_t* status);

/*
 * Every device-side wait (for a TMA copy, for the tensor cores) gives up after this many
 * nanoseconds, sets the error word and lets the kernel finish.  Default 200 ms: a decode step
 * lasts well under one.  Process-wide, read at launch.
 */
int pfd_set_wait_limit_ns(uint64_t limit_ns);

/*
 * Tuning: which form the split-KV pass of the shared-prefix entry points takes.  -1 (default):
 * chosen per call -- two-warp CTAs that run on the same SMs WHILE the dense prefix pass runs when
 * the SMs that pass leaves free could not absorb the suffix work meanwhile (and, with a groups
 * table, PFD_FLAG_ALL_IN_GROUPS is set), else the ordinary four-warp CTAs, which start on those
 * free SMs and take the rest after the pass; 0: always the latter; 1: always the former.
 * Process-wide, read at launch; results do not depend on it.
 */
int pfd_set_suffix_form(int32_t form);

/*
 * Self-test of that mechanism (it allocates one pinned host word while it runs): a one-warp
 * kernel arms a barrier for bytes that no copy will deliver and waits for them with the given
 * limit.  Returns after the kernel has finished; pfd_device_status() then reads 1, and
 * *waited_ns (optional) holds how long the wait lasted on the device.  Nothing traps, faults
 * or stays in flight.
 */
int pfd_selftest_bounded_wait(uint64_t limit_ns, uint64_t* waited_ns, void* stream);

/* Which kernels the calling thread's last decode call launched. */
#define PFD_PATH_FIXED_LDG 1 /* fixed-split grid, plain 16-byte loads, + merge kernel */
#define PFD_PATH_FIXED_TMA 2 /* fixed-split grid, TMA pipeline, + merge kernel         */
#define PFD_PATH_BALANCED 3  /* balanced persistent kernel + its merge kernel            */
#define PFD_PATH_BALANCED_KV16 4 /* the same for 16-bit caches (pfd_paged_decode_kv16_split_out) */
#define PFD_PATH_FUSED 5       /* balanced persistent kernel alone (PFD_FLAG_SINGLE_LAUNCH)   */
#define PFD_PATH_FUSED_KV16 6  /* the same for 16-bit caches                                  */
int pfd_last_path(void);

/*
 * The producer step: rotary embedding of the new tokens' query and key (in place) and append of
 * key / value to the paged cache, optionally quantised to FP8-e4m3 with per-kv-head scales.
 * Replaces l20_rope_and_cache (integrations/vllm/l20_rope_kv.py:256-328), which handles fp16 /
 * bf16 caches only ("quantized KV cache is not supported", :273-274).
 * Strides count elements.  cos_sin_cache is [max_position, rotary_dim]: cos of the rotary_dim / 2
 * frequencies, then sin (vLLM's layout), float32 or the query's type.  slot_mapping[t] =
 * block * block_size + offset, negative = do not store that token.  cache_dtype: PFD_DTYPE_F16 /
 * PFD_DTYPE_BF16 (must equal query_dtype) or PFD_DTYPE_E4M3; scales are read for E4M3 only.
 */
#define PFD_DTYPE_E4M3 3
typedef struct pfd_rope_args {
  uint32_t struct_size; /* sizeof(pfd_rope_args) */
  int32_t num_tokens, num_q_heads, num_kv_heads, head_dim, rotary_dim, block_size;
  int32_t is_neox;       /* 1: pairs (i, i + rotary_dim / 2); 0: pairs (2i, 2i + 1) */
  int32_t query_dtype;   /* of query, key, value */
  int32_t cos_sin_dtype; /* PFD_DTYPE_F32 or query_dtype */
  int32_t cache_dtype;
  void* query;           /* [tokens, num_q_heads, head_dim], rotated in place */
  int64_t q_stride_t, q_stride_h;
  void* key;             /* [tokens, num_kv_heads, head_dim], rotated in place */
  int64_t k_stride_t, k_stride_h;
  const void* value;
  int64_t v_stride_t, v_stride_h;
  const int64_t* positions;
  const void* cos_sin_cache;
  int64_t cos_sin_stride;
  const int64_t* slot_mapping;
  void* key_cache;       /* logical [blocks, block_size, num_kv_heads, head_dim] */
  int64_t kc_stride_block, kc_stride_token, kc_stride_head;
  void* value_cache;
  int64_t vc_stride_block, vc_stride_token, vc_stride_head;
  float k_scale, v_scale;
  const float* k_scale_per_head; /* optional [num_kv_heads], overrides k_scale */
  const float* v_scale_per_head;
  void* stream;
} pfd_rope_args;
int pfd_rope_quant_append(const pfd_rope_args* args);

/* Number of kernels this library has launched in this process (for launch accounting). */
int64_t pfd_launch_count(void);

/* Message of the last failing call on this thread ("" if none). */
const char* pfd_last_error(void);

int pfd_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PAGED_FP8_DECODE_H_ */
