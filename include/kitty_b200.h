/*
 * kitty_b200 — C ABI of the B200 (sm_100a) implementation of Kitty's quantized
 * KV-cache hot path: quantize-and-append, flush, fused dequant decode attention.
 *
 * Every entry point takes plain pointers and sizes, launches on the CUDA stream
 * it is given, never synchronises the host with the device, never allocates or
 * frees device memory (unless its comment says otherwise) and returns an int:
 * 0 on success, a negative kitty_status otherwise.  Nothing throws.
 *
 * File:line citations name the reference interface (paths inside the Kitty
 * project, src/kitty/...) that the entry point replaces.
 *
 * Geometry is fixed to what the reference hard-codes (kvcache/kitty.py:43-47):
 * page = 128 tokens, head_dim = 128, 32 boosted channels, sink = 32 tokens.
 * Anything else is rejected with KITTY_E_BADSHAPE.
 */
#ifndef KITTY_B200_H
#define KITTY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  KITTY_OK = 0,
  KITTY_E_BADARG = -1,    /* null / misaligned pointer, bad enum, negative count        */
  KITTY_E_BADSHAPE = -2,  /* geometry other than page 128 / D 128 / 32 boosted / G > 16 */
  KITTY_E_WORKSPACE = -3, /* caller's workspace too small                               */
  KITTY_E_CUDA = -4,      /* a CUDA runtime call failed (see cudaGetLastError)          */
  KITTY_E_TIMEOUT = -5,   /* a bounded device-side wait ran out                         */
  KITTY_E_STATIC_LIMIT = -6 /* problem needs more scratch than kitty_decode_attn_static has */
} kitty_status;

typedef enum { KITTY_F16 = 0, KITTY_BF16 = 1, KITTY_F32 = 2 } kitty_dtype;

/* How the 32 boosted key channels of a page are chosen. */
typedef enum {
  /* In-kernel: score = mean|x| over the page rounded once to the input dtype,
     descending, equal scores ordered by ascending channel number; slot = rank.
     (kernels/kitty_quant_pack.py:280-288 with a defined tie order.) */
  KITTY_SELECT_FUSED = 0,
  /* The caller supplies the dense->sparse index bytes, as the reference's kernel
     receives them (kernels/kitty_quant_pack.py:19-20, 65-71). */
  KITTY_SELECT_SUPPLIED = 1
} kitty_select_mode;

/* fp32 division used for (x - min) / scale. */
typedef enum {
  KITTY_DIV_IEEE = 0, /* correctly rounded; equals the reference run on a host    */
  KITTY_DIV_FULL = 1  /* PTX div.full.f32 (2 ulp)                                 */
} kitty_div_mode;

/* Device buffers of one layer, with the names, shapes and dtypes of the
 * reference's KVCache_Layer (kvcache/utils_kv_per_layer.py:18-83).  All tensors
 * are contiguous; strides that may differ are explicit. */
typedef struct {
  int32_t max_bs, max_page, h_kv, head_dim, d_boost, page_size, sink_size, reserved;
  uint8_t *KeyCache;            /* u8  [max_bs*max_page, h_kv*5248]        */
  void *KeyCache_metadata;      /* f16 [max_bs*max_page, h_kv, 128, 2]     */
  uint8_t *ValueCache;          /* u8  [max_bs*max_page, h_kv*4096]        */
  void *ValueCache_metadata;    /* f16 [max_bs*max_page, h_kv, 128, 2]     */
  const int64_t *PageTable_K;   /* i64 [max_bs, max_page]                  */
  const int64_t *PageTable_V;   /* i64 [max_bs, max_page]                  */
  void *Sink_Buffer_K;          /* f16 [max_bs, h_kv, 32, 128]             */
  void *Sink_Buffer_V;
  void *Q_Buffer_K;             /* f16 [max_bs, h_kv, 128, 128]            */
  void *Q_Buffer_V;
  void *Local_Buffer_V;         /* f16 [max_bs, h_kv, 128, 128] ring       */
} kitty_layer;

/* The reference keeps these as Python ints on the layer object
 * (utils_kv_per_layer.py:53-80) and passes them to its kernels as scalars. */
typedef struct {
  int32_t PageCount_K, PageCount_V, Sink_Count, Q_Buffer_Count_K, Q_Buffer_Count_V, Local_Count_V,
      Write_Offset_Local_V, reserved;
} kitty_counts;

int kitty_version(void);
const char *kitty_strerror(int status);

/* quantize_pack_k (kernels/kitty_quant_pack.py:253-312 and the kernel at :13-152).
 * key: [B, H, T, 128] of `dtype`, element strides (stride_b, stride_h, stride_t), unit
 * stride over channels, every row 16-byte aligned.  Quantizes tokens
 * [t_offset, t_offset + 128*pages) of every (b, h) into pages
 * page_table[b, page_offset + p].  idx_io: u8 [B, H, pages, 128], read when
 * select == KITTY_SELECT_SUPPLIED, written (if non-null) with the chosen bytes
 * otherwise.  One pass over the keys: score, top-32 rank, min/max, codes, pack. */
int kitty_quant_pack_k(const void *key, int dtype, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                       int32_t B, int32_t H, int64_t t_offset, int32_t pages, const int64_t *page_table,
                       int64_t page_table_stride_b, int32_t page_offset, uint8_t *cache,
                       int64_t cache_stride_page, void *cache_meta, uint8_t *idx_io, int select, int div_mode,
                       void *stream);

/* quantize_pack_v (kernels/kitty_quant_pack.py:315-356, kernel at :155-249). */
int kitty_quant_pack_v(const void *value, int dtype, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                       int32_t B, int32_t H, int64_t t_offset, int32_t pages, const int64_t *page_table,
                       int64_t page_table_stride_b, int32_t page_offset, uint8_t *cache,
                       int64_t cache_stride_page, void *cache_meta, int div_mode, void *stream);

/* quantize_pack_k and quantize_pack_v of one prompt in ONE launch: the pair of calls the reference's prefill always
 * issues back to back (kvcache/kitty.py:126-192: keys at :143, values at :175).  Arguments as in the two
 * functions above, the key ones prefixed k_, the value ones v_; both halves are validated before anything is
 * launched.  With 16-bit input and KITTY_DIV_IEEE the key tiles are dispatched first and the value tiles fill the
 * SMs that the last wave of key tiles leaves free; otherwise this is the two launches.  Results are bit-identical to
 * the two separate calls. */
int kitty_quant_pack_kv(const void *key, const void *value, int dtype, int64_t k_stride_b, int64_t k_stride_h,
                        int64_t k_stride_t, int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t, int32_t B,
                        int32_t H, int64_t k_t_offset, int32_t k_pages, const int64_t *k_page_table,
                        int64_t k_page_table_stride_b, int32_t k_page_offset, uint8_t *k_cache,
                        int64_t k_cache_stride_page, void *k_cache_meta, uint8_t *idx_io, int select,
                        int64_t v_t_offset, int32_t v_pages, const int64_t *v_page_table,
                        int64_t v_page_table_stride_b, int32_t v_page_offset, uint8_t *v_cache,
                        int64_t v_cache_stride_page, void *v_cache_meta, int div_mode, void *stream);

/* The full-precision copies of KittyCache.quantize_prefill (kvcache/kitty.py:137-141,
 * 164-172) in one launch: the first `sink` tokens into the sink buffers, the last
 * qbuf_k keys into Q_Buffer_K, the last local_v values into Local_Buffer_V and the
 * qbuf_v values before those into Q_Buffer_V, all cast to fp16.  key/value:
 * [B, H, L, 128] with the given element strides. */
int kitty_prefill_tails(const kitty_layer *layer, const void *key, const void *value, int dtype,
                        int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t, int64_t v_stride_b,
                        int64_t v_stride_h, int64_t v_stride_t, int32_t B, int64_t L, int32_t sink,
                        int32_t qbuf_k, int32_t local_v, int32_t qbuf_v, void *stream);

/* Rotary position embedding of one decode token: q [B, h_q, 128] and k [B, h_kv, 128] (contiguous) to q_out /
 * k_out of the same shape and type, out = x*cos + rotate_half(x)*sin with every product and the sum rounded to
 * the data type — bit-identical to the element-wise sequence of the model's attention forward
 * (models/qwen3/modeling_qwen3.py:222-232), in one launch.  cos / sin: [B or 1, 128] of the same type, rows
 * cos_stride_b elements apart (0 when all rows share one position). */
int kitty_rope_qk(const void *q, const void *k, const void *cos, const void *sin, void *q_out, void *k_out, int dtype,
                  int32_t B, int32_t h_q, int32_t h_kv, int64_t cos_stride_b, void *stream);

/* Decode branch of KittyCache.update (kvcache/kitty.py:101-123): one token per
 * (b, h) goes to the sink, or to Q_Buffer_K and the value ring (the ring's oldest
 * token moving to Q_Buffer_V when the ring is full).  `counts` is the state
 * BEFORE the append; the caller advances its counters exactly as kitty.py does.
 * key/value: [B, H, 1, 128] with element strides (stride_b, stride_h). */
int kitty_append(const kitty_layer *layer, const kitty_counts *counts, const void *key, const void *value,
                 int dtype, int64_t k_stride_b, int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_h,
                 int32_t B, void *stream);

/* KittyCache.quantize_decode (kvcache/kitty.py:194-236): Q_Buffer_K becomes key
 * page PageCount_K when flush_k != 0 and Q_Buffer_V becomes value page
 * PageCount_V when flush_v != 0 — both in one launch. */
int kitty_flush(const kitty_layer *layer, const kitty_counts *counts, int32_t B, int flush_k, int flush_v,
                int select, int div_mode, void *stream);

/* Bytes of scratch kitty_decode_attn needs for this problem size (negative
 * kitty_status on bad arguments).  The workspace is caller-owned device memory,
 * 256-byte aligned, ZERO-FILLED ONCE before its first use: its first word is a
 * sticky status that a kernel sets when a bounded wait runs out, its second word
 * the counter the streaming kernel hands work items out with (left at zero by
 * every completed call).  Calls that
 * share a workspace must not overlap on the device.  The reference allocates its
 * scratch (the logits tensor) inside the call (kernels/kitty_attention.py:426-430). */
int64_t kitty_decode_workspace_bytes(int32_t B, int32_t h_kv, int32_t h_q, int32_t max_pages);

/* Copies the workspace's status word to *host_status and SYNCHRONISES the stream
 * (the one entry point that does).  Returns KITTY_E_TIMEOUT when it is set. */
int kitty_workspace_status(const void *workspace, int32_t *host_status, void *stream);

/* kitty_attention_forward (kernels/kitty_attention.py:403-526: qk_kernel, softmax,
 * sv_kernel) as one fused pass: split over the sequence, online softmax, packed
 * pages streamed with bulk async copies and unpacked in registers.
 * query: [B, h_q, 1, 128] contiguous of q_dtype (F16 or BF16, F32 accepted).
 * out:   [B, 1, h_q, 128] contiguous of out_dtype.
 * page_begin/page_end restrict the packed pages visited (sequence split across
 * GPUs); pass 0 and -1 for all pages.  flags: bit0 include the sink tokens, bit1
 * include everything after the last common packed page (extra key pages,
 * Q-buffers, value ring); pass 3 on a single GPU.
 * If partial_out is non-null the un-normalised result is written there instead
 * of `out`, as fp32 [B, h_q, 130] = (acc[128], running max, running sum) in the
 * base-2 domain, for kitty_lse_merge.
 * impl: 0 = default kernels (int8 tensor-core streaming kernel for groups of up
 * to 4 query heads per KV head, fp16 tensor-core streaming kernel otherwise);
 * 2 = the fp16 streaming kernel for every group size; 1 = the plain CUDA-core
 * kernel for every tile (slow; kept as an in-library cross-check). */
int kitty_decode_attn(const kitty_layer *layer, const kitty_counts *counts, const void *query, int q_dtype,
                      int32_t B, int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                      int64_t workspace_bytes, int32_t page_begin, int32_t page_end, int32_t flags,
                      float *partial_out, int impl, void *stream);

/* ---- Ragged batches: one set of counters per batch row -------------------------------------
 * The reference keeps ONE set of counters for the whole batch (utils_kv_per_layer.py:53-80), so every sequence of a
 * batch has to have the same length and a prompt can only be given in one piece (kvcache/kitty.py:89-95).  These
 * entry points take a kitty_counts per batch row instead — the same structure twice: row_counts_host (host memory,
 * B entries: argument checks and the work plan) and row_counts_dev (device memory, B entries, the same values: read
 * by the kernels).  The caller advances every row's counters as kvcache/kitty.py:102-123 and :201-234 do for the
 * batch.  Rows may then differ in length, and a prompt can arrive in several pieces (token by token through
 * kitty_append_rows / kitty_flush_rows).
 *
 * kitty_append_rows: kitty_append per row; a row whose `reserved` field is non-zero takes no token in this call.
 * kitty_flush_rows:  kitty_flush per row: a row's Q_Buffer_K / Q_Buffer_V becomes its page PageCount_K / PageCount_V
 *                    when its Q_Buffer_Count_K / Q_Buffer_Count_V is 128; other rows are left alone.
 * kitty_decode_attn_rows: kitty_decode_attn over the whole sequence of every row. */
int kitty_append_rows(const kitty_layer *layer, const kitty_counts *row_counts_host, const kitty_counts *row_counts_dev,
                      const void *key, const void *value, int dtype, int64_t k_stride_b, int64_t k_stride_h,
                      int64_t v_stride_b, int64_t v_stride_h, int32_t B, void *stream);
int kitty_flush_rows(const kitty_layer *layer, const kitty_counts *row_counts_host, const kitty_counts *row_counts_dev,
                     int32_t B, int select, int div_mode, void *stream);
int kitty_decode_attn_rows(const kitty_layer *layer, const kitty_counts *row_counts_host,
                           const kitty_counts *row_counts_dev, const void *query, int q_dtype, int32_t B, int32_t h_q,
                           float scaling, void *out, int out_dtype, void *workspace, int64_t workspace_bytes, int impl,
                           void *stream);

/* ---- Decode step with device-resident state (CUDA-graph friendly) ------------------------
 * The reference passes its counters to every kernel as Python ints
 * (kernels/kitty_attention.py:458-460, 510-514), which bakes them into a captured graph.  Here the
 * per-step state lives in a small device block that every kernel of the step reads; a captured
 * graph stays valid for the life of the cache because no launch argument or launch dimension
 * depends on the step.  All layers of a cache share the block (their counters are identical).
 *
 *   host, once per token:   kitty_plan_step(...) fills a kitty_step_state on the host and
 *                           writes it to the device block (one small launch on the stream: the
 *                           168 bytes travel as a kernel argument, so no host buffer has to
 *                           stay untouched until the copy runs).
 *   per layer (capturable): kitty_decode_step(...) = append + attention + merge + flush-if-due.
 *   host, after the token:  advance the counters as kvcache/kitty.py:102-123, 201-234 does
 *                           (kitty_plan_step returns the new counters in state->next).
 * Limits: in-kernel channel selection.  kitty_plan_step / kitty_decode_step cover the whole sequence on one
 * GPU; the _split / _exchange forms below cover this rank's part of a sequence split over GPUs. */
typedef struct {
  kitty_counts before;   /* state before this step's append                                        */
  kitty_counts after;    /* after the append: what the attention kernels see                       */
  kitty_counts next;     /* after the step's flushes: `before` of the next step (host use)         */
  int32_t pb, pe, ch, nchunk, has_sink, has_tail, n_slots, n_tiles, chunk_slot0, edge_slot;
  int32_t n_items, n_edge, flush_k, flush_v;
  int32_t edge_parts, edge_part_tok;
  int32_t xchg_seq, reserved;      /* sequence-split steps: exchange sequence number of the step's first layer */
} kitty_step_state;      /* 168 bytes */

/* Fills *state (host memory) for one decode step of a cache whose counters are *before and, when
 * device_state is not null, stores the same 160 bytes there in stream order. */
int kitty_plan_step(const kitty_layer *layer, const kitty_counts *before, int32_t B, int32_t h_q,
                    kitty_step_state *state, kitty_step_state *device_state, void *stream);

/* kitty_plan_step for one rank of a sequence split over GPUs: the attention of the step visits the common packed
 * pages [page_begin, page_end) only, flags as for kitty_decode_attn (bit0 sink, bit1 tail), and xchg_seq is the
 * exchange sequence number of the step's first layer (see kitty_decode_step_exchange).  The append and the flushes
 * are planned as in kitty_plan_step: every rank keeps the counters (and, cheaply, the fp16 buffers) up to date. */
int kitty_plan_step_split(const kitty_layer *layer, const kitty_counts *before, int32_t B, int32_t h_q,
                          int32_t page_begin, int32_t page_end, int32_t flags, int32_t xchg_seq,
                          kitty_step_state *state, kitty_step_state *device_state, void *stream);

/* One layer's decode step from the device-resident state: kitty_append, kitty_decode_attn
 * (impl 0, whole sequence) and kitty_flush in four launches whose arguments do not depend on the
 * step (streaming, merge and flush kernels are launched as programmatic dependents of the kernel
 * before them, so their launch latencies overlap).  key/value: [B, H, 1, 128] (element strides as for kitty_append); query [B, h_q, 1, 128]
 * contiguous; out [B, 1, h_q, 128] contiguous; workspace as for kitty_decode_attn. */
int kitty_decode_step(const kitty_layer *layer, const kitty_step_state *device_state, const void *key,
                      const void *value, int kv_dtype, int64_t k_stride_b, int64_t k_stride_h, int64_t v_stride_b,
                      int64_t v_stride_h, const void *query, int q_dtype, int32_t B, int32_t h_q, float scaling,
                      void *out, int out_dtype, void *workspace, int64_t workspace_bytes, int div_mode, void *stream);

/* kitty_decode_step for one rank of a sequence split: the merge step of the attention exchanges this rank's partial
 * with the other ranks over peer memory and writes the complete result, as kitty_decode_attn_exchange does (same
 * exchange buffers, same bounded waits).  The sequence number of the exchange is device_state->xchg_seq +
 * seq_offset, so that the launch arguments do not change from token to token: give every layer of a model its own
 * seq_offset (0, 1, 2, ...) and let xchg_seq grow by the number of layers per token, starting at 1. */
int kitty_decode_step_exchange(const kitty_layer *layer, const kitty_step_state *device_state, const void *key,
                               const void *value, int kv_dtype, int64_t k_stride_b, int64_t k_stride_h,
                               int64_t v_stride_b, int64_t v_stride_h, const void *query, int q_dtype, int32_t B,
                               int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                               int64_t workspace_bytes, int div_mode, void *const *peer_buffers, int32_t rank,
                               int32_t world, int32_t seq_offset, int32_t *status, int64_t wait_ns, void *stream);

/* Size in bytes of the scratch array built into the library for kitty_decode_attn_static. */
#define KITTY_STATIC_SCRATCH_BYTES (8u << 20)

/* kitty_decode_attn for callers that must not allocate device memory and have no
 * buffer to lend as a workspace.  (No counterpart in the reference: its decode
 * path allocates its scratch tensors inside every call.)
 *
 * Who needs it: a host that has handed all free device memory to another
 * allocator (a framework's caching pool, a serving engine's KV arena), so that a
 * raw cudaMalloc would fail or fragment that pool; code on a latency-critical
 * path, where cudaMalloc/cudaFree take a driver-wide lock and may synchronise the
 * device; and embedders that are only allowed to pass through the tensors they
 * were given.  For them the split-KV partial results live in a fixed
 * `static __device__` array of KITTY_STATIC_SCRATCH_BYTES inside the library;
 * every GPU that loads the library carries that array until the process exits.
 *
 * Arguments are those of kitty_decode_attn without workspace/workspace_bytes,
 * plus status_out: a DEVICE pointer to an int32 (or null) that receives the
 * bounded-wait status word of this call (0 = fine) when the call's work on the
 * stream completes.  The entry point calls no cudaMalloc/cudaFree and no
 * allocating library routine.  The first call on a device looks the array's
 * address up (cudaGetSymbolAddress, with that device current) and opts the
 * kernels into large shared memory; make that first call outside any stream
 * capture.  A problem whose partials do not fit returns KITTY_E_STATIC_LIMIT
 * before any kernel is launched.  All calls on a device share the one array: the status
 * word and the item hand-out counter are cleared at the start of each call,
 * everything else is overwritten before it is read, and two calls that overlap on
 * the GPU (different streams) race — serialise them. */
int kitty_decode_attn_static(const kitty_layer *layer, const kitty_counts *counts, const void *query, int q_dtype,
                             int32_t B, int32_t h_q, float scaling, void *out, int out_dtype, int32_t page_begin,
                             int32_t page_end, int32_t flags, float *partial_out, int impl, int32_t *status_out,
                             void *stream);

/* Log-sum-exp combination of n_parts partial results (fp32 [n_parts, rows, 130],
 * the layout partial_out uses; rows = B*h_q) into out [rows, 128] of out_dtype.
 * Used after the all-gather of a sequence-split decode step.  The reference has
 * no multi-GPU path (utils_kv_per_layer.py:16 "To Do: Multi-GPU Inference"). */
int kitty_lse_merge(const float *partials, int32_t n_parts, int64_t rows, void *out, int out_dtype,
                    void *stream);

/* Sequence-split combine without a collective: the log-sum-exp merge of kitty_lse_merge with the
 * exchange of the partials done by the kernel itself over peer memory (NVLink).  No counterpart in the
 * reference (single GPU only).
 *
 * Every rank owns an exchange buffer of kitty_lse_exchange_bytes(rows, world, &flag_offset) bytes that all
 * ranks can address (CUDA IPC / VMM peer mapping, e.g. torch symmetric memory), zero-filled once before
 * the first call.  peer_buffers is a DEVICE array of `world` pointers: entry r is rank r's buffer as
 * mapped in this process.  All ranks call with the same rows/world and the same seq, which starts at 1
 * and grows by one per call.  The kernel stores this rank's partial (fp32 [rows, 130], the partial_out
 * layout) into every rank's buffer, raises a per-row flag, waits at most wait_ns nanoseconds (0: the default
 * of one second) for the other ranks' flags and writes out [rows, 128].  A wait that runs out sets *status
 * (device int32, may be null) to 1 and leaves the row unwritten; the kernel returns normally and the context
 * stays usable (the host reports it as KITTY_E_TIMEOUT once it has read the word).  rows <=
 * KITTY_EXCHANGE_MAX_ROWS so that every block of the launch is resident (a block waits only for the same row
 * on other GPUs). */
#define KITTY_EXCHANGE_MAX_ROWS 1024
/* kitty_decode_attn of this rank's part of the sequence (page_begin/page_end/flags as there) whose final merge
 * kernel also does the exchange above: one call and one launch fewer per layer than kitty_decode_attn with
 * partial_out followed by kitty_lse_exchange_merge.  B*h_q <= KITTY_EXCHANGE_MAX_ROWS.  A rank whose part is
 * empty still has to call (it contributes an empty partial). */
int kitty_decode_attn_exchange(const kitty_layer *layer, const kitty_counts *counts, const void *query, int q_dtype,
                               int32_t B, int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                               int64_t workspace_bytes, int32_t page_begin, int32_t page_end, int32_t flags, int impl,
                               void *const *peer_buffers, int32_t rank, int32_t world, int32_t seq, int32_t *status,
                               int64_t wait_ns, void *stream);
int64_t kitty_lse_exchange_bytes(int64_t rows, int32_t world, int64_t *flag_offset);
int kitty_lse_exchange_merge(const float *local_partial, int64_t rows, void *const *peer_buffers, int32_t rank,
                             int32_t world, int32_t seq, void *out, int out_dtype, int32_t *status, int64_t wait_ns,
                             void *stream);

#ifdef __cplusplus
}
#endif
#endif /* KITTY_B200_H */
