// Work decomposition shared by the decode-attention kernels.
//
// Token order of one (batch, kv-head) sequence (kernels/kitty_attention.py:88-207,
// 269-386 of the reference):
//   keys   = sink | packed key pages   | Q_Buffer_K
//   values = sink | packed value pages | Q_Buffer_V | ring (oldest first)
// "Tile" u = 0 is the sink; tile u >= 1 covers positions [(u-1)*128, u*128) after
// the sink.  Tiles 1..PageCount_V hold a packed key page AND a packed value page
// ("common pages", the streaming hot loop); later tiles pair extra key pages or
// Q_Buffer_K with fp16 values ("tail").
//
// A decode call is cut into items; each item reduces a run of tiles for one
// (batch, kv-head) to a partial result (acc[128], max, sum) per query head in
// the workspace, and a merge kernel combines the slots.
#pragma once

#include "common.cuh"

namespace kitty {

struct DecodePlan {
  int32_t B, H, G, h_q;
  int32_t pb, pe;        // common pages visited: [pb, pe), pe <= PageCount_V
  int32_t ch;            // pages per chunk
  int32_t nchunk;        // chunks per (b, h)
  int32_t has_sink;      // slot 0 is the sink tile
  int32_t has_tail;      // last slot is the tail
  int32_t n_slots;       // has_sink + nchunk + has_tail
  int32_t n_tiles;       // total tiles of the sequence (sink tile included)
  int32_t fast_chunks;   // 1: chunks are reduced by the streaming kernel, 0: by the plain kernel
  int32_t chunk_slot0;   // slot of chunk 0
  int32_t edge_slot;     // first slot written by the edge reduction (sink + tail), when it runs
  int32_t edge_parts;    // the edge of one (b, h) is reduced in this many parts (slots edge_slot ...)
  int32_t edge_part_tok; // edge tokens per part (a multiple of 64; sink tokens first, then the tail)
};

struct DecodeArgs {
  kitty_layer L;
  kitty_counts C;
  DecodePlan P;
  const void *q;         // [B, h_q, 1, 128]
  int32_t q_dtype;
  float scale_log2;      // scaling * log2(e): logits live in the base-2 domain
  float *partials;       // [B*H, n_slots, G, PART]
  int32_t *status;       // workspace header: [0] set non-zero when a bounded wait ran out, [1] item hand-out counter
  const kitty_step_state *dyn;   // or null.  Non-null: plan, counters and item counts are read from it on the device
  const kitty_counts *rows;      // or null.  Non-null: one set of counters per batch row (ragged batch); C and the
                                 // plan then hold the largest values over the rows, and a row stops where its own
                                 // counters say
};

// Counters of batch row b: the row's own when the call carries per-row counters, the call's otherwise.
__device__ __forceinline__ kitty_counts row_counts(const DecodeArgs &a, const kitty_counts &C, int b) {
  return a.rows != nullptr ? a.rows[b] : C;
}

// Merge n partials per row.  Row r's partial s lives at
//   base + ((r / gm) * ns * gm + r % gm) * PART + s * stride_part   (floats).
// Peer-memory exchange of the merged partials (sequence split over GPUs); peers == nullptr: none.
struct XchgDesc {
  float *const *peers;       // device array [world]: base address of every rank's exchange buffer
  int64_t flag_offset;       // byte offset of the flag area inside an exchange buffer
  int32_t rank, world, seq;
  int32_t *status;           // or null: set non-zero when a wait ran out
  unsigned long long wait_ns;   // how long a block waits for the other ranks' partials of its row
};

constexpr unsigned long long XCHG_WAIT_NS_DEFAULT = 1000000000ull;   // 1 s: far beyond any healthy exchange

struct MergeArgs {
  const float *partials;
  int64_t rows, stride_part;
  int32_t n, gm, ns;
  void *out;          // [rows, 128] of out_dtype, or null
  int32_t out_dtype;
  float *partial_out; // [rows, PART] or null: merged but un-normalised
  int32_t *work_counter;  // or null: word the streaming kernel used to hand out items; reset to 0 here
  const kitty_step_state *dyn;   // or null.  Non-null: the number of slots is read from it on the device
  XchgDesc x;                    // x.peers non-null: exchange the row's partial with the other ranks before writing out
};

int launch_decode_plain(const DecodeArgs &a, int items_per_bh, cudaStream_t s);
int launch_decode_paged(const DecodeArgs &a, int n_items, int n_gt, int n_edge, int grid, cudaStream_t s,
                        bool dependent = false);
int launch_decode_paged_i8(const DecodeArgs &a, int n_items, int n_edge, int grid, cudaStream_t s,
                           bool dependent = false);   // dependent: programmatic dependent of the kernel before it
int launch_append_dyn(const kitty_layer &L, const kitty_step_state *dyn, const void *key, const void *value, int dtype,
                      int64_t ksb, int64_t ksh, int64_t vsb, int64_t vsh, int32_t B, cudaStream_t s);
int launch_flush_dyn(const kitty_layer &L, const kitty_step_state *dyn, int32_t B, int div_mode, cudaStream_t s);
int launch_merge(const MergeArgs &m, cudaStream_t s);
int sm_count();        // multiprocessors of the current device (cached per device)
int i8_blocks_per_sm(int G);   // resident blocks per multiprocessor of the integer streaming kernel for groups of G heads

__device__ __forceinline__ float load_q(const void *q, int dtype, int64_t i) {
  if (dtype == KITTY_F16) return __half2float(static_cast<const __half *>(q)[i]);
  if (dtype == KITTY_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(q)[i]);
  return static_cast<const float *>(q)[i];
}

}  // namespace kitty
