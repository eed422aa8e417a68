// Host side of the decode-attention entry points: argument checks, the split of
// a call into items (chunks of common pages, the sink tile, the tail) and the
// launches.  No allocation, no host/device synchronisation.
#include <algorithm>

#include "decode.cuh"

namespace kitty {

constexpr int64_t WS_HEADER = 256;   // bytes at the start of the workspace: sticky status word, item hand-out counter
constexpr int PG_WARPS_HOST = 4;     // warps per block of the streaming kernel (pages per chunk come in multiples)
constexpr int MAX_CHUNKS = 128;      // chunks per (batch, kv-head): with few rows, one page per warp fills the GPU

}  // namespace kitty

int kitty::sm_count() {
  static std::atomic<int> cached[MAX_DEVICES];       // zero-initialised; any thread may fill an entry (same value)
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

namespace kitty {

static int chunk_cap(int64_t bh_gt, int grid_max) {
  const int64_t cap = (16LL * grid_max) / std::max<int64_t>(1, bh_gt);
  return static_cast<int>(std::min<int64_t>(MAX_CHUNKS, std::max<int64_t>(1, cap)));
}

// Pick pages-per-chunk so that the items fill `grid_max` resident blocks in whole waves.
static void plan_chunks(int n_pages, int64_t bh_gt, int grid_max, bool dynamic, int *ch_out, int *nchunk_out) {
  if (n_pages <= 0) {
    *ch_out = PG_WARPS_HOST;
    *nchunk_out = 0;
    return;
  }
  const int cap = std::min(chunk_cap(bh_gt, grid_max), (n_pages + PG_WARPS_HOST - 1) / PG_WARPS_HOST);
  double best = 1e30;
  int best_ch = n_pages, best_n = 1;
  for (int want = 1; want <= cap; ++want) {
    int ch = (n_pages + want - 1) / want;
    ch = (ch + PG_WARPS_HOST - 1) / PG_WARPS_HOST * PG_WARPS_HOST;
    const int n = (n_pages + ch - 1) / ch;
    const int64_t items = bh_gt * n;
    const int64_t waves = (items + grid_max - 1) / grid_max;
    // per item: its pages (one per warp at a time) plus a fixed part worth about 2.5 pages — the table look-up, the
    // first copy's flight, the block's merge
    const double item_cost = ch / PG_WARPS_HOST + 2.5;
    // static round-robin: whole waves.  Dynamic hand-out: the average load plus one item of tail — except for a
    // small call (latency-bound: every item has a block of its own and a warp walks at most four pages), which
    // takes one item's time
    const bool one_wave = items <= grid_max && ch <= 4 * PG_WARPS_HOST;
    const double cost = !dynamic ? static_cast<double>(waves) * item_cost
                        : (one_wave ? item_cost : static_cast<double>(items) * item_cost / grid_max + item_cost);
    if (cost < best - 1e-9) {
      best = cost;
      best_ch = ch;
      best_n = n;
    }
  }
  *ch_out = best_ch;
  *nchunk_out = best_n;
}

// Edge (sink + tail) of one (b, h): in how many parts it is reduced.  With few (b, h) rows a single
// block per row would leave most of the GPU waiting on one latency-bound reduction of up to 416 tokens,
// so the edge is cut into 64- or 128-token parts (one work item and one partial slot each).
constexpr int EDGE_PARTS_MAX = 7;                 // ceil((32 + 3 * 128) / 64)
static void plan_edge(int has_sink, int has_tail, const kitty_counts &C, int64_t bh, bool split, int *parts, int *part_tok) {
  const int ne = (has_sink ? C.Sink_Count : 0) +
                 (has_tail ? (C.PageCount_K - C.PageCount_V) * PAGE + C.Q_Buffer_Count_K : 0);
  int tok = 64 * EDGE_PARTS_MAX;                  // one part holds any edge
  if (split) {
    const int sms = sm_count();
    if (2 * bh <= sms) tok = 64;                  // measured: pays up to about half a row per SM; beyond one row
    else if (bh <= sms) tok = 128;                // per SM the streamed pages hide a whole edge and parts only add work
  }
  *part_tok = tok;
  *parts = ne > 0 ? (ne + tok - 1) / tok : 0;
}

}  // namespace kitty

using namespace kitty;

extern "C" int64_t kitty_decode_workspace_bytes(int32_t B, int32_t h_kv, int32_t h_q, int32_t max_pages) {
  if (B <= 0 || h_kv <= 0 || h_q <= 0 || h_q % h_kv != 0 || max_pages < 0) return KITTY_E_BADARG;
  const int G = h_q / h_kv;
  if (G > MAX_GROUP) return KITTY_E_BADSHAPE;
  const int64_t grid_max = 4 * sm_count();                    // the larger of the two streaming kernels' resident grids
  const int64_t bh = static_cast<int64_t>(B) * h_kv;
  // chunk slots of a call with bh' <= bh rows: bh' * min(chunk_cap(bh'), pages / 4) <= the expression below, which
  // never decreases with bh — a workspace sized for the largest batch serves every smaller one
  const int64_t cap_pages = std::min<int64_t>(MAX_CHUNKS, std::max(1, (max_pages + PG_WARPS_HOST - 1) / PG_WARPS_HOST));
  const int64_t chunk_slots = std::min(bh * cap_pages, std::max(bh, 16 * grid_max));
  return WS_HEADER + (chunk_slots + bh * EDGE_PARTS_MAX) * G * PART * static_cast<int64_t>(sizeof(float));
}

static bool counts_ok(const kitty_layer *layer, const kitty_counts &C) {
  if (C.PageCount_K < 0 || C.PageCount_V < 0 || C.PageCount_K > layer->max_page || C.PageCount_V > layer->max_page ||
      C.Sink_Count < 0 || C.Sink_Count > SINK || C.Q_Buffer_Count_K < 0 || C.Q_Buffer_Count_K > PAGE ||
      C.Q_Buffer_Count_V < 0 || C.Q_Buffer_Count_V > PAGE || C.Local_Count_V < 0 || C.Local_Count_V > PAGE ||
      C.Write_Offset_Local_V < 0 || C.Write_Offset_Local_V >= PAGE)
    return false;
  const int64_t tk = static_cast<int64_t>(C.PageCount_K) * PAGE + C.Q_Buffer_Count_K;
  const int64_t tv = static_cast<int64_t>(C.PageCount_V) * PAGE + C.Q_Buffer_Count_V + C.Local_Count_V;
  return tk == tv && C.PageCount_V <= C.PageCount_K && !(C.Sink_Count < SINK && tk != 0);
}

// rows_host / rows_dev: null, or one set of counters per batch row (ragged batch; host copy for the checks and the
// plan, device copy for the kernels).  `counts` is then ignored: the plan is made for the largest values over the rows
// and every row stops where its own counters say.
static int decode_attn_core(const kitty_layer *layer, const kitty_counts *counts, const void *query, int q_dtype,
                            int32_t B, int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                            int64_t workspace_bytes, int32_t page_begin, int32_t page_end, int32_t flags,
                            float *partial_out, int impl, const XchgDesc *xchg, void *stream,
                            const kitty_counts *rows_host = nullptr, const kitty_counts *rows_dev = nullptr) {
  if (!layer || (!counts && !rows_host) || !query || !workspace) return KITTY_E_BADARG;
  if ((rows_host != nullptr) != (rows_dev != nullptr)) return KITTY_E_BADARG;
  if (!out && !partial_out) return KITTY_E_BADARG;
  if (layer->head_dim != HD || layer->page_size != PAGE || layer->d_boost != DB || layer->sink_size != SINK)
    return KITTY_E_BADSHAPE;
  const int H = layer->h_kv;
  if (B <= 0 || B > layer->max_bs || H <= 0 || h_q <= 0 || h_q % H != 0) return KITTY_E_BADARG;
  const int G = h_q / H;
  if (G > MAX_GROUP) return KITTY_E_BADSHAPE;
  if (q_dtype < KITTY_F16 || q_dtype > KITTY_F32 || out_dtype < KITTY_F16 || out_dtype > KITTY_F32) return KITTY_E_BADARG;
  if (impl < 0 || impl > 2) return KITTY_E_BADARG;
  if (B > 65535 || H > 65535) return KITTY_E_BADARG;
  // C: the counters the plan is made for.  Uniform batch: the call's.  Ragged batch: a stand-in holding the largest
  // number of common pages, the longest sink and the longest tail over the rows.
  kitty_counts C;
  int64_t tk;
  if (rows_host == nullptr) {
    C = *counts;
    if (!counts_ok(layer, C)) return KITTY_E_BADARG;              // includes utils_kv_per_layer.py:94 (K and V lengths agree)
    tk = static_cast<int64_t>(C.PageCount_K) * PAGE + C.Q_Buffer_Count_K;
  } else {
    int pv = 0, sink = 0, tail = 0;
    for (int b = 0; b < B; ++b) {
      const kitty_counts &r = rows_host[b];
      if (!counts_ok(layer, r)) return KITTY_E_BADARG;
      pv = std::max(pv, r.PageCount_V);
      sink = std::max(sink, r.Sink_Count);
      tail = std::max(tail, (r.PageCount_K - r.PageCount_V) * PAGE + r.Q_Buffer_Count_K);
    }
    C = kitty_counts{};
    C.PageCount_V = pv;
    C.PageCount_K = pv + tail / PAGE;
    C.Q_Buffer_Count_K = tail % PAGE;
    C.Sink_Count = sink;
    tk = static_cast<int64_t>(C.PageCount_K) * PAGE + C.Q_Buffer_Count_K;
  }
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return KITTY_E_BADARG;

  DecodeArgs a;
  a.L = *layer;
  a.C = C;
  DecodePlan &P = a.P;
  P.B = B; P.H = H; P.G = G; P.h_q = h_q;
  const int pv = C.PageCount_V;
  P.pb = std::min(std::max(page_begin, 0), pv);
  P.pe = page_end < 0 ? pv : std::min(std::max(page_end, P.pb), pv);
  P.n_tiles = 1 + static_cast<int>((tk + PAGE - 1) / PAGE);
  P.has_sink = ((flags & 1) && C.Sink_Count > 0) ? 1 : 0;
  P.has_tail = ((flags & 2) && (P.n_tiles - 1 - pv) > 0) ? 1 : 0;
  const bool use_i8 = (impl == 0 && G <= 8);       // integer tensor-core kernel: one or two operand groups of 4 heads
  const int n_gt = use_i8 ? 1 : (G + 7) / 8;
  const int grid_max = (use_i8 ? i8_blocks_per_sm(G) : 2) * sm_count();   // resident blocks per SM of the streaming kernel
  P.fast_chunks = (impl != 1) ? 1 : 0;
  plan_edge(P.has_sink, P.has_tail, C, static_cast<int64_t>(B) * H, P.fast_chunks != 0, &P.edge_parts, &P.edge_part_tok);
  // static item assignment (fp16 kernel): leave blocks for the edge parts so that a small call is one wave
  const int64_t edge_blocks = use_i8 ? 0 : std::min<int64_t>(static_cast<int64_t>(B) * H * P.edge_parts, grid_max / 2);
  plan_chunks(P.pe - P.pb, static_cast<int64_t>(B) * H * n_gt, grid_max - static_cast<int>(edge_blocks), use_i8, &P.ch,
              &P.nchunk);
  const int has_edge = P.edge_parts > 0 ? 1 : 0;
  if (P.fast_chunks) {            // slots: [edge parts][chunks]
    P.n_slots = P.edge_parts + P.nchunk;
    P.chunk_slot0 = P.edge_parts;
    P.edge_slot = 0;
  } else {                        // slots: [sink?][chunks][tail?]
    P.n_slots = P.has_sink + P.nchunk + P.has_tail;
    P.chunk_slot0 = P.has_sink;
    P.edge_slot = 0;
  }
  if (P.n_slots == 0 && !partial_out && !xchg) return KITTY_E_BADARG;             // nothing to attend to

  const int64_t need = WS_HEADER + static_cast<int64_t>(B) * H * P.n_slots * G * PART * static_cast<int64_t>(sizeof(float));
  if (workspace_bytes < need) return KITTY_E_WORKSPACE;
  a.q = query;
  a.q_dtype = q_dtype;
  a.scale_log2 = scaling * 1.4426950408889634f;
  a.status = static_cast<int32_t *>(workspace);
  a.dyn = nullptr;
  a.rows = rows_dev;
  a.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + WS_HEADER);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (use_i8) {
    // the int8 streaming kernel also reduces the edge (sink + tail) inside its own grid
    const int64_t items = static_cast<int64_t>(B) * H * P.nchunk;
    const int64_t n_edge = static_cast<int64_t>(B) * H * P.edge_parts;
    if (items + n_edge > 0) {
      const int grid = static_cast<int>(std::min<int64_t>(items + n_edge, grid_max));
      // launched as a programmatic dependent of whatever precedes it in the stream (the kernel waits for that work
      // before it reads anything): behind kitty_append, whose blocks release their dependents at once, the launch
      // latency of this kernel is hidden
      if (int rc = launch_decode_paged_i8(a, static_cast<int>(items), static_cast<int>(n_edge), grid, s, true)) return rc;
    }
  } else if (P.fast_chunks) {
    // the fp16 streaming kernel reduces the edge parts in its own grid too, after a block's page items
    const int64_t items = static_cast<int64_t>(B) * H * n_gt * P.nchunk;
    const int64_t n_edge = static_cast<int64_t>(B) * H * P.edge_parts;
    if (items + n_edge > 0) {
      const int grid = static_cast<int>(std::min<int64_t>(items + n_edge, grid_max));
      if (int rc = launch_decode_paged(a, static_cast<int>(items), n_gt, static_cast<int>(n_edge), grid, s)) return rc;
    }
  } else {
    const int plain_items = P.has_sink + P.nchunk + P.has_tail;
    if (plain_items > 0)
      if (int rc = launch_decode_plain(a, plain_items, s)) return rc;
  }

  MergeArgs m;
  m.partials = a.partials;
  m.rows = static_cast<int64_t>(B) * h_q;
  m.stride_part = static_cast<int64_t>(G) * PART;
  m.n = P.n_slots;
  m.gm = G;
  m.ns = P.n_slots;
  m.out = out;
  m.out_dtype = out_dtype;
  m.partial_out = partial_out;
  m.work_counter = a.status + 1;
  m.dyn = nullptr;
  m.x = xchg ? *xchg : XchgDesc{};
  const int rc = launch_merge(m, s);
  // The merge kernel is what leaves the item hand-out counter at zero for the next call.  If it could not be
  // launched, zero the counter in stream order so that a failed call cannot poison the workspace.
  if (rc != KITTY_OK) cudaMemsetAsync(a.status + 1, 0, sizeof(int32_t), s);
  return rc;
}

extern "C" int kitty_decode_attn(const kitty_layer *layer, const kitty_counts *counts, const void *query, int q_dtype,
                                 int32_t B, int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                                 int64_t workspace_bytes, int32_t page_begin, int32_t page_end, int32_t flags,
                                 float *partial_out, int impl, void *stream) {
  return decode_attn_core(layer, counts, query, q_dtype, B, h_q, scaling, out, out_dtype, workspace, workspace_bytes,
                          page_begin, page_end, flags, partial_out, impl, nullptr, stream);
}

extern "C" int kitty_decode_attn_rows(const kitty_layer *layer, const kitty_counts *row_counts_host,
                                      const kitty_counts *row_counts_dev, const void *query, int q_dtype, int32_t B,
                                      int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                                      int64_t workspace_bytes, int impl, void *stream) {
  if (!row_counts_host || !row_counts_dev || !out) return KITTY_E_BADARG;
  return decode_attn_core(layer, nullptr, query, q_dtype, B, h_q, scaling, out, out_dtype, workspace, workspace_bytes, 0, -1,
                          3, nullptr, impl, nullptr, stream, row_counts_host, row_counts_dev);
}

extern "C" int kitty_decode_attn_exchange(const kitty_layer *layer, const kitty_counts *counts, const void *query,
                                          int q_dtype, int32_t B, int32_t h_q, float scaling, void *out, int out_dtype,
                                          void *workspace, int64_t workspace_bytes, int32_t page_begin, int32_t page_end,
                                          int32_t flags, int impl, void *const *peer_buffers, int32_t rank,
                                          int32_t world, int32_t seq, int32_t *status, int64_t wait_ns,
                                          void *stream) {
  if (!out || !peer_buffers || world <= 0 || world > 128 || rank < 0 || rank >= world || seq <= 0 || wait_ns < 0)
    return KITTY_E_BADARG;
  const int64_t rows = static_cast<int64_t>(B) * h_q;
  if (rows <= 0 || rows > KITTY_EXCHANGE_MAX_ROWS) return KITTY_E_BADARG;
  XchgDesc x;
  x.peers = reinterpret_cast<float *const *>(peer_buffers);
  kitty_lse_exchange_bytes(rows, world, &x.flag_offset);
  x.rank = rank;
  x.world = world;
  x.seq = seq;
  x.status = status;
  x.wait_ns = wait_ns > 0 ? static_cast<unsigned long long>(wait_ns) : XCHG_WAIT_NS_DEFAULT;
  return decode_attn_core(layer, counts, query, q_dtype, B, h_q, scaling, out, out_dtype, workspace, workspace_bytes,
                          page_begin, page_end, flags, nullptr, impl, &x, stream);
}

extern "C" int kitty_lse_merge(const float *partials, int32_t n_parts, int64_t rows, void *out, int out_dtype,
                               void *stream) {
  if (!partials || !out || n_parts <= 0 || rows < 0) return KITTY_E_BADARG;
  if (out_dtype < KITTY_F16 || out_dtype > KITTY_F32) return KITTY_E_BADARG;
  MergeArgs m;
  m.partials = partials;
  m.rows = rows;
  m.stride_part = rows * PART;
  m.n = n_parts;
  m.gm = 1;
  m.ns = 1;
  m.out = out;
  m.out_dtype = out_dtype;
  m.partial_out = nullptr;
  m.work_counter = nullptr;
  m.dyn = nullptr;
  m.x = XchgDesc{};
  return launch_merge(m, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------- //
// Decode step with device-resident state
// ------------------------------------------------------------------------- //
__global__ void store_step_state_kernel(kitty_step_state st, kitty_step_state *dst) {
  const int32_t *src = reinterpret_cast<const int32_t *>(&st);
  const int n = static_cast<int>(sizeof(kitty_step_state) / sizeof(int32_t));
  if (threadIdx.x < n) reinterpret_cast<int32_t *>(dst)[threadIdx.x] = src[threadIdx.x];
}

extern "C" int kitty_plan_step(const kitty_layer *layer, const kitty_counts *before, int32_t B, int32_t h_q,
                               kitty_step_state *state, kitty_step_state *device_state, void *stream) {
  return kitty_plan_step_split(layer, before, B, h_q, 0, -1, 3, 0, state, device_state, stream);
}

extern "C" int kitty_plan_step_split(const kitty_layer *layer, const kitty_counts *before, int32_t B, int32_t h_q,
                                     int32_t page_begin, int32_t page_end, int32_t flags, int32_t xchg_seq,
                                     kitty_step_state *state, kitty_step_state *device_state, void *stream) {
  if (!layer || !before || !state || xchg_seq < 0) return KITTY_E_BADARG;
  if (layer->head_dim != HD || layer->page_size != PAGE || layer->d_boost != DB || layer->sink_size != SINK)
    return KITTY_E_BADSHAPE;
  const int H = layer->h_kv;
  if (B <= 0 || B > layer->max_bs || H <= 0 || h_q <= 0 || h_q % H != 0) return KITTY_E_BADARG;
  const int G = h_q / H;
  if (G > MAX_GROUP) return KITTY_E_BADSHAPE;
  if (!counts_ok(layer, *before)) return KITTY_E_BADARG;
  kitty_step_state &st = *state;
  st = kitty_step_state{};
  st.before = *before;
  // append (kvcache/kitty.py:102-123)
  kitty_counts c = *before;
  if (c.Sink_Count < SINK) {
    c.Sink_Count += 1;
  } else {
    if (c.Q_Buffer_Count_K >= PAGE) return KITTY_E_BADARG;
    c.Q_Buffer_Count_K += 1;
    if (c.Local_Count_V < PAGE) {
      c.Local_Count_V += 1;
    } else {
      if (c.Q_Buffer_Count_V >= PAGE) return KITTY_E_BADARG;
      c.Q_Buffer_Count_V += 1;
      c.Write_Offset_Local_V = (c.Write_Offset_Local_V + 1) % PAGE;
    }
  }
  st.after = c;
  // flush (kvcache/kitty.py:201-234)
  st.flush_k = (c.Q_Buffer_Count_K == PAGE) ? 1 : 0;
  st.flush_v = (c.Q_Buffer_Count_V == PAGE) ? 1 : 0;
  if ((st.flush_k && c.PageCount_K >= layer->max_page) || (st.flush_v && c.PageCount_V >= layer->max_page))
    return KITTY_E_BADARG;
  kitty_counts n = c;
  if (st.flush_k) { n.PageCount_K += 1; n.Q_Buffer_Count_K = 0; }
  if (st.flush_v) { n.PageCount_V += 1; n.Q_Buffer_Count_V = 0; }
  st.next = n;
  // plan of the attention call (whole sequence, int8 streaming kernel)
  const int pv = c.PageCount_V;
  const int64_t tk = static_cast<int64_t>(c.PageCount_K) * PAGE + c.Q_Buffer_Count_K;
  st.pb = std::min(std::max(page_begin, 0), pv);
  st.pe = page_end < 0 ? pv : std::min(std::max(page_end, st.pb), pv);
  st.n_tiles = 1 + static_cast<int>((tk + PAGE - 1) / PAGE);
  st.has_sink = ((flags & 1) && c.Sink_Count > 0) ? 1 : 0;
  st.has_tail = ((flags & 2) && (st.n_tiles - 1 - pv) > 0) ? 1 : 0;
  st.xchg_seq = xchg_seq;
  // the same plan kitty_decode_attn makes for these counters: int8 kernel for groups of up to 8 heads, fp16 kernel above
  const bool use_i8 = G <= 8;
  const int n_gt = use_i8 ? 1 : (G + 7) / 8;
  const int grid_max = (use_i8 ? i8_blocks_per_sm(G) : 2) * sm_count();
  plan_edge(st.has_sink, st.has_tail, c, static_cast<int64_t>(B) * H, true, &st.edge_parts, &st.edge_part_tok);
  const int64_t edge_blocks = use_i8 ? 0 : std::min<int64_t>(static_cast<int64_t>(B) * H * st.edge_parts, grid_max / 2);
  plan_chunks(st.pe - st.pb, static_cast<int64_t>(B) * H * n_gt, grid_max - static_cast<int>(edge_blocks), use_i8, &st.ch, &st.nchunk);
  st.n_slots = st.edge_parts + st.nchunk;
  st.chunk_slot0 = st.edge_parts;
  st.edge_slot = 0;
  st.n_items = B * H * n_gt * st.nchunk;
  st.n_edge = B * H * st.edge_parts;
  if (device_state != nullptr) {
    if ((reinterpret_cast<uintptr_t>(device_state) & 15u) != 0) return KITTY_E_BADARG;
    store_step_state_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(st, device_state);
    if (cudaGetLastError() != cudaSuccess) return KITTY_E_CUDA;
  }
  return KITTY_OK;
}

static int decode_step_core(const kitty_layer *layer, const kitty_step_state *device_state, const void *key,
                            const void *value, int kv_dtype, int64_t k_stride_b, int64_t k_stride_h,
                            int64_t v_stride_b, int64_t v_stride_h, const void *query, int q_dtype, int32_t B,
                            int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                            int64_t workspace_bytes, int div_mode, const XchgDesc *xchg, void *stream) {
  if (!layer || !device_state || !key || !value || !query || !out || !workspace) return KITTY_E_BADARG;
  if (layer->head_dim != HD || layer->page_size != PAGE || layer->d_boost != DB || layer->sink_size != SINK)
    return KITTY_E_BADSHAPE;
  const int H = layer->h_kv;
  if (B <= 0 || B > layer->max_bs || B > 65535 || H <= 0 || H > 65535 || h_q <= 0 || h_q % H != 0) return KITTY_E_BADARG;
  const int G = h_q / H;
  if (G > MAX_GROUP) return KITTY_E_BADSHAPE;
  if (kv_dtype < KITTY_F16 || kv_dtype > KITTY_F32 || q_dtype < KITTY_F16 || q_dtype > KITTY_F32 ||
      out_dtype < KITTY_F16 || out_dtype > KITTY_F32)
    return KITTY_E_BADARG;
  if (div_mode != KITTY_DIV_IEEE && div_mode != KITTY_DIV_FULL) return KITTY_E_BADARG;
  const int64_t q16 = 16 / (kv_dtype == KITTY_F32 ? 4 : 2);
  if ((reinterpret_cast<uintptr_t>(key) & 15u) || (reinterpret_cast<uintptr_t>(value) & 15u) || k_stride_b % q16 ||
      k_stride_h % q16 || v_stride_b % q16 || v_stride_h % q16)
    return KITTY_E_BADARG;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return KITTY_E_BADARG;
  if (workspace_bytes < kitty_decode_workspace_bytes(B, H, h_q, layer->max_page)) return KITTY_E_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (int rc = launch_append_dyn(*layer, device_state, key, value, kv_dtype, k_stride_b, k_stride_h, v_stride_b,
                                 v_stride_h, B, s))
    return rc;
  DecodeArgs a;
  a.L = *layer;
  a.C = kitty_counts{};
  a.P = DecodePlan{};
  a.P.B = B; a.P.H = H; a.P.G = G; a.P.h_q = h_q;
  a.P.fast_chunks = 1;
  a.q = query;
  a.q_dtype = q_dtype;
  a.scale_log2 = scaling * 1.4426950408889634f;
  a.status = static_cast<int32_t *>(workspace);
  a.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + WS_HEADER);
  a.dyn = device_state;
  a.rows = nullptr;
  // fixed grids: the item counts are read on the device
  if (G <= 8) {
    if (int rc = launch_decode_paged_i8(a, 0, 0, i8_blocks_per_sm(G) * sm_count(), s, true)) return rc;
  } else {
    if (int rc = launch_decode_paged(a, 0, (G + 7) / 8, 0, 2 * sm_count(), s, true)) return rc;
  }
  MergeArgs m;
  m.partials = a.partials;
  m.rows = static_cast<int64_t>(B) * h_q;
  m.stride_part = static_cast<int64_t>(G) * PART;
  m.n = 0;
  m.gm = G;
  m.ns = 0;
  m.out = out;
  m.out_dtype = out_dtype;
  m.partial_out = nullptr;
  m.work_counter = a.status + 1;
  m.dyn = device_state;
  m.x = xchg ? *xchg : XchgDesc{};      // with an exchange, x.seq is the layer's offset to the state's sequence number
  if (int rc = launch_merge(m, s)) {
    cudaMemsetAsync(a.status + 1, 0, sizeof(int32_t), s);      // see decode_attn_core
    return rc;
  }
  return launch_flush_dyn(*layer, device_state, B, div_mode, s);
}

extern "C" int kitty_decode_step(const kitty_layer *layer, const kitty_step_state *device_state, const void *key,
                                 const void *value, int kv_dtype, int64_t k_stride_b, int64_t k_stride_h,
                                 int64_t v_stride_b, int64_t v_stride_h, const void *query, int q_dtype, int32_t B,
                                 int32_t h_q, float scaling, void *out, int out_dtype, void *workspace,
                                 int64_t workspace_bytes, int div_mode, void *stream) {
  return decode_step_core(layer, device_state, key, value, kv_dtype, k_stride_b, k_stride_h, v_stride_b, v_stride_h, query,
                          q_dtype, B, h_q, scaling, out, out_dtype, workspace, workspace_bytes, div_mode, nullptr, stream);
}

extern "C" int kitty_decode_step_exchange(const kitty_layer *layer, const kitty_step_state *device_state, const void *key,
                                          const void *value, int kv_dtype, int64_t k_stride_b, int64_t k_stride_h,
                                          int64_t v_stride_b, int64_t v_stride_h, const void *query, int q_dtype,
                                          int32_t B, int32_t h_q, float scaling, void *out, int out_dtype,
                                          void *workspace, int64_t workspace_bytes, int div_mode,
                                          void *const *peer_buffers, int32_t rank, int32_t world, int32_t seq_offset,
                                          int32_t *status, int64_t wait_ns, void *stream) {
  if (!peer_buffers || world <= 0 || world > 128 || rank < 0 || rank >= world || seq_offset < 0 || wait_ns < 0)
    return KITTY_E_BADARG;
  const int64_t rows = static_cast<int64_t>(B) * h_q;
  if (rows <= 0 || rows > KITTY_EXCHANGE_MAX_ROWS) return KITTY_E_BADARG;
  XchgDesc x;
  x.peers = reinterpret_cast<float *const *>(peer_buffers);
  kitty_lse_exchange_bytes(rows, world, &x.flag_offset);
  x.rank = rank;
  x.world = world;
  x.seq = seq_offset;
  x.status = status;
  x.wait_ns = wait_ns > 0 ? static_cast<unsigned long long>(wait_ns) : XCHG_WAIT_NS_DEFAULT;
  return decode_step_core(layer, device_state, key, value, kv_dtype, k_stride_b, k_stride_h, v_stride_b, v_stride_h, query,
                          q_dtype, B, h_q, scaling, out, out_dtype, workspace, workspace_bytes, div_mode, &x, stream);
}

extern "C" int kitty_workspace_status(const void *workspace, int32_t *host_status, void *stream) {
  if (!workspace || !host_status) return KITTY_E_BADARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(host_status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess) return KITTY_E_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return KITTY_E_CUDA;
  return *host_status ? KITTY_E_TIMEOUT : KITTY_OK;
}

extern "C" int kitty_version(void) { return 100; }

extern "C" const char *kitty_strerror(int status) {
  switch (status) {
    case KITTY_OK: return "ok";
    case KITTY_E_BADARG: return "bad argument (null or misaligned pointer, bad enum, inconsistent counters)";
    case KITTY_E_BADSHAPE: return "unsupported geometry (need page 128, head_dim 128, 32 boosted channels, sink 32, group <= 16)";
    case KITTY_E_WORKSPACE: return "workspace too small (see kitty_decode_workspace_bytes)";
    case KITTY_E_CUDA: return "CUDA runtime error";
    case KITTY_E_TIMEOUT: return "a bounded device-side wait ran out";
    case KITTY_E_STATIC_LIMIT:
      return "the problem needs more scratch than the built-in array of kitty_decode_attn_static "
             "(KITTY_STATIC_SCRATCH_BYTES); use kitty_decode_attn with a caller-owned workspace";
    default: return "unknown status";
  }
}

// ------------------------------------------------------------------------- //
// Decode attention without any caller-provided or allocated scratch.
// ------------------------------------------------------------------------- //
// The split-KV partials of kitty_decode_attn_static live here.  In host code the
// name `g_static_scratch` is only a handle for the runtime's symbol table, not a
// device address: the address is looked up per device below and that pointer is
// what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[KITTY_STATIC_SCRATCH_BYTES];

static void *static_scratch_ptr(int *rc) {
  static std::atomic<void *> cached[MAX_DEVICES];    // zero-initialised; any thread may fill an entry (same value)
  int dev = 0;
  *rc = KITTY_OK;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    *rc = KITTY_E_CUDA;
    return nullptr;
  }
  void *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
      *rc = KITTY_E_CUDA;
      return nullptr;
    }
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

extern "C" int kitty_decode_attn_static(const kitty_layer *layer, const kitty_counts *counts, const void *query,
                                        int q_dtype, int32_t B, int32_t h_q, float scaling, void *out, int out_dtype,
                                        int32_t page_begin, int32_t page_end, int32_t flags, float *partial_out,
                                        int impl, int32_t *status_out, void *stream) {
  int rc = KITTY_OK;
  void *ws = static_scratch_ptr(&rc);
  if (rc != KITTY_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Two words have to start at zero: the status word and the item hand-out counter behind it (an earlier call on
  // this device that failed half-way may have left the counter dirty, and no caller can reach the array to
  // repair it).  The partial slots are written before they are read.
  if (cudaMemsetAsync(ws, 0, 2 * sizeof(int32_t), s) != cudaSuccess) return KITTY_E_CUDA;
  rc = kitty_decode_attn(layer, counts, query, q_dtype, B, h_q, scaling, out, out_dtype, ws,
                         static_cast<int64_t>(KITTY_STATIC_SCRATCH_BYTES), page_begin, page_end, flags, partial_out, impl,
                         stream);
  if (rc == KITTY_E_WORKSPACE) return KITTY_E_STATIC_LIMIT;      // checked before anything is launched
  if (rc != KITTY_OK) return rc;
  if (status_out != nullptr &&
      cudaMemcpyAsync(status_out, ws, sizeof(int32_t), cudaMemcpyDeviceToDevice, s) != cudaSuccess)
    return KITTY_E_CUDA;
  return KITTY_OK;
}
