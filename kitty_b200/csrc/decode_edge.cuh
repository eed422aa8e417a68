// Edge reduction: the part of a decode-attention call that is not a pair of packed
// pages — the fp16 sink tokens and the tail of the sequence (key pages that have
// no packed value page yet, Q_Buffer_K, Q_Buffer_V, the rotated value ring;
// kernels/kitty_attention.py:88-113, 183-207, 269-289, 336-386 of the reference).
// At most 32 + 384 tokens per (batch, kv-head), ~100 KB of fp16 rows.
//
// One call per (batch, kv-head), by all warps of a block:
//   1. logits of every edge token into shared memory — fp16 key rows go through
//      mma.sync with A fragments loaded straight from global memory (each lane
//      reads 64 contiguous bytes of a row), packed key pages through the same
//      code path as the streaming kernel;
//   2. softmax statistics over the (small) edge, probabilities in place;
//   3. P.V on the CUDA cores, each lane owns 4 channels of a row, then a fixed-order cross-warp
//      reduction.  Two ways to fetch the value rows: straight from global memory (sixteen rows
//      in flight per warp), or — when the caller provides a row buffer and an mbarrier — in
//      waves of up to RB_ROWS rows brought by bulk async copies.  The first wave is requested
//      before the logits are computed, so it lands for free, and a wave keeps ~28 KB in flight
//      where register loads keep 16 KB; this roughly halves the time of an edge inside the
//      streaming kernel, where the edge is latency-bound.
//   4. one partial (acc, max, sum) per query head into the workspace slot.
#pragma once

#include "paged_core.cuh"

namespace kitty {

constexpr int EDGE_MAX_TOK = SINK + 3 * PAGE;   // sink + at most two key pages + Q_Buffer_K
constexpr int S_ROW = EDGE_MAX_TOK + 4;

// NG: query heads per KV head the buffers are sized for (4, or MAX_GROUP); NW: warps of the block;
// RB_ROWS: value rows of the bulk-copy row buffer (0: rows are loaded straight from global memory).
template <int NG, int NW, int RB_ROWS = 0>
struct EdgeSmem {
  static constexpr int SR = (NG <= 4) ? 4 : (NG <= 8) ? 8 : MAX_GROUP;   // rows of S / red (query heads)
  static constexpr int QR = (NG <= 8) ? 8 : MAX_GROUP;          // staged query rows (mma tiles of 8 heads)
  static constexpr int ROWS = RB_ROWS;
  float S[SR][S_ROW];                        // logits, then probabilities
  float red[SR][HD];                         // cross-warp reduction of the output
  __align__(16) __half qs[QR][QS_ROW];
  __align__(16) uint8_t krec[2][K_HEAD];
  __align__(16) uint32_t kmeta[2][HD];
  float mx[SR], sum[SR];
  uint8_t inv[NW][DB];
  __align__(128) uint8_t rows[RB_ROWS > 0 ? RB_ROWS * HD * 2 : 16];   // value rows of the current wave (fp16)
};

// Reduces part `part` of the edge of one (batch b, kv-head h) with the NW warps of the calling block and
// writes the partial into the workspace slot P.edge_slot + part.  The edge tokens are numbered sink first,
// then the tail; part i covers tokens [i * P.edge_part_tok, (i + 1) * P.edge_part_tok).  Part boundaries are
// multiples of 64 and the tail starts at token 0 or 32, so a 16-token key tile is never split.  With few
// (b, h) rows the host asks for several small parts so that the latency-bound edge spreads over more blocks.
// Every thread of the block must call it.
// bar / phase: with a row buffer, the shared-memory address of an mbarrier (initialised with count 1, used by
// nobody else) and the block-uniform count of its completed phases, carried from call to call.
template <int NG, int NW, typename Smem>
__device__ __forceinline__ void edge_item(const DecodeArgs &a, const DecodePlan &P, const kitty_counts &C,
                                          Smem &sm, int b, int h, int part, uint32_t bar = 0, uint32_t *phase = nullptr) {
  constexpr int EDGE_WARPS = NW;
  constexpr int SR = Smem::SR;
  constexpr int RB = Smem::ROWS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
  const int H = P.H, G = P.G;
  const int64_t bh = static_cast<int64_t>(b) * H + h;
  const int n_gt = (G + 7) >> 3;

  const int sink_n = P.has_sink ? C.Sink_Count : 0;
  const int npk = P.has_tail ? (C.PageCount_K - C.PageCount_V) : 0;     // key pages without a packed value page
  const int qk_n = P.has_tail ? C.Q_Buffer_Count_K : 0;
  const int tail_n = npk * PAGE + qk_n;
  const int ne_all = sink_n + tail_n;
  const int lo = part * P.edge_part_tok;                       // this part: edge tokens [lo, ne)
  const int ne = min(ne_all, lo + P.edge_part_tok);

  // value rows of edge token e: sink rows, then Q_Buffer_V rows, then the ring in logical order
  const __half *sinkv = static_cast<const __half *>(a.L.Sink_Buffer_V) + bh * SINK * HD;
  const __half *qbufv = static_cast<const __half *>(a.L.Q_Buffer_V) + bh * PAGE * HD;
  const __half *ringv = static_cast<const __half *>(a.L.Local_Buffer_V) + bh * PAGE * HD;
  const int qv_n = P.has_tail ? C.Q_Buffer_Count_V : 0;
  // Bulk copies of the rows of tokens [e0, e1) into the row buffer, row e at (e - e0) * 256 (one thread).
  auto issue_wave = [&](int e0, int e1) {
    const uint32_t dst0 = smem_u32(&sm.rows[0]);
    mbar_expect_tx(bar, static_cast<uint32_t>(e1 - e0) * HD * 2);
    auto piece = [&](int ea, int eb, const __half *src) {          // tokens [ea, eb) from contiguous rows at src
      if (ea < eb) bulk_g2s(dst0 + (ea - e0) * HD * 2, src, static_cast<uint32_t>(eb - ea) * HD * 2, bar);
    };
    int ea = e0, eb = min(e1, sink_n);
    piece(ea, eb, sinkv + ea * HD);
    ea = max(e0, sink_n); eb = min(e1, sink_n + qv_n);
    piece(ea, eb, qbufv + (ea - sink_n) * HD);
    ea = max(e0, sink_n + qv_n); eb = e1;
    if (ea < eb) {                                                  // ring rows j = e - sink_n - qv_n, physical (j + W) mod 128
      const int j0 = ea - sink_n - qv_n, j1 = eb - sink_n - qv_n;
      const int p0 = (j0 + C.Write_Offset_Local_V) & (PAGE - 1);
      const int n0 = min(j1 - j0, PAGE - p0);                       // rows before the wrap
      piece(ea, ea + n0, ringv + p0 * HD);
      piece(ea + n0, eb, ringv);
    }
  };
  if (RB > 0) {
    if (tid == 0 && lo < ne) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the buffer may have been written by plain stores
      issue_wave(lo, min(ne, lo + RB));
    }
  }

  // ---- stage the query and the tail's packed key pages ---- //
  for (int i = tid; i < n_gt * 8 * HD; i += EDGE_WARPS * 32) {
    const int g = i >> 7, d = i & (HD - 1);
    float v = 0.f;
    if (g < G) v = load_q(a.q, a.q_dtype, (static_cast<int64_t>(b) * P.h_q + h * G + g) * HD + d) * a.scale_log2;
    sm.qs[g][d] = __float2half_rn(v);
  }
  if (tid < EDGE_WARPS * DB) sm.inv[tid / DB][tid % DB] = 0;
  for (int p = 0; p < npk; ++p) {
    if (sink_n + p * PAGE >= ne || sink_n + (p + 1) * PAGE <= lo) continue;     // page outside this part
    const int64_t pid = a.L.PageTable_K[static_cast<int64_t>(b) * a.L.max_page + C.PageCount_V + p];
    const uint4 *src = reinterpret_cast<const uint4 *>(a.L.KeyCache + pid * (static_cast<int64_t>(H) * K_HEAD) + h * K_HEAD);
    for (int i = tid; i < K_HEAD / 16; i += EDGE_WARPS * 32) reinterpret_cast<uint4 *>(sm.krec[p])[i] = src[i];
    const uint4 *ms = reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(a.L.KeyCache_metadata) + (pid * H + h) * META_HEAD);
    if (tid < META_HEAD / 16) reinterpret_cast<uint4 *>(sm.kmeta[p])[tid] = ms[tid];
  }
  __syncthreads();

  // ---- 1a. packed key pages of the tail: one (page, group of 8 heads) per warp ---- //
  if (warp < npk * n_gt && sink_n + (warp / n_gt) * PAGE < ne && sink_n + (warp / n_gt + 1) * PAGE > lo) {
    const int p = warp / n_gt, gt = warp % n_gt;
    uint32_t q2[8][2];
    load_q_frags(&sm.qs[gt * 8], gid, tig, q2);
    float cl[8][4];
    qk_packed_page(sm.krec[p], sm.kmeta[p], &sm.qs[gt * 8], q2, sm.inv[warp], lane, cl);
    const int e0 = sink_n + p * PAGE + 16 * gid;
    if (gt * 8 + 2 * tig < SR) {
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        sm.S[gt * 8 + 2 * tig][e0 + m] = cl[m][0];
        sm.S[gt * 8 + 2 * tig + 1][e0 + m] = cl[m][1];
        sm.S[gt * 8 + 2 * tig][e0 + 8 + m] = cl[m][2];
        sm.S[gt * 8 + 2 * tig + 1][e0 + 8 + m] = cl[m][3];
      }
    }
  }
  // ---- 1b. fp16 key rows (sink, Q_Buffer_K): 16-token tiles ---- //
  {
    const int ns_t = (sink_n + 15) >> 4, nq_t = (qk_n + 15) >> 4;
    for (int j = warp; j < ns_t + nq_t; j += EDGE_WARPS) {
      const __half *base;
      int row0, nrows, e0;
      if (j < ns_t) {
        base = static_cast<const __half *>(a.L.Sink_Buffer_K) + bh * SINK * HD;
        row0 = 16 * j; nrows = sink_n; e0 = row0;
      } else {
        base = static_cast<const __half *>(a.L.Q_Buffer_K) + bh * PAGE * HD;
        row0 = 16 * (j - ns_t); nrows = qk_n; e0 = sink_n + npk * PAGE + row0;
      }
      if (e0 < lo || e0 >= ne) continue;                        // tile outside this part (warp-uniform)
      // lane (gid, tig): rows row0+gid and row0+gid+8, channels [32*tig, 32*tig+32)
      uint4 ra[4], rb[4];
      const int rA = row0 + gid, rB = row0 + gid + 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ra[i] = (rA < nrows) ? *reinterpret_cast<const uint4 *>(base + rA * HD + 32 * tig + 8 * i) : make_uint4(0, 0, 0, 0);
        rb[i] = (rB < nrows) ? *reinterpret_cast<const uint4 *>(base + rB * HD + 32 * tig + 8 * i) : make_uint4(0, 0, 0, 0);
      }
      const uint32_t *wa = reinterpret_cast<const uint32_t *>(ra), *wb = reinterpret_cast<const uint32_t *>(rb);
      for (int gt = 0; gt < n_gt; ++gt) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        // contraction index k = 2*tig, 2*tig+1 <-> channels 32*tig + 4*ks + {0,1}; k = 2*tig+8, +9 <-> + {2,3}
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint2 qq = *reinterpret_cast<const uint2 *>(&sm.qs[gt * 8 + gid][32 * tig + 4 * ks]);
          mma16816(c, wa[2 * ks], wb[2 * ks], wa[2 * ks + 1], wb[2 * ks + 1], qq.x, qq.y);
        }
        const int g0 = gt * 8 + 2 * tig;
        if (g0 >= SR) continue;
        if (rA < nrows) {
          sm.S[g0][e0 + gid] = c[0];
          sm.S[g0 + 1][e0 + gid] = c[1];
        }
        if (rB < nrows) {
          sm.S[g0][e0 + gid + 8] = c[2];
          sm.S[g0 + 1][e0 + gid + 8] = c[3];
        }
      }
    }
  }
  __syncthreads();

  // ---- 2. softmax statistics per query head; probabilities replace the logits ---- //
  for (int g = warp; g < G; g += EDGE_WARPS) {
    float mx = -INFINITY;
    for (int e = lo + lane; e < ne; e += 32) mx = fmaxf(mx, sm.S[g][e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
    for (int e = lo + lane; e < ne; e += 32) {
      const float p = ex2(sm.S[g][e] - mx);
      sm.S[g][e] = p;
      s += p;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
      sm.mx[g] = mx;
      sm.sum[g] = s;
    }
  }
  __syncthreads();

  // ---- 3. P.V: warp walks tokens warp, warp + NW, ...; lane owns channels 4*lane..4*lane+3 ---- //
  float acc[NG][4];
#pragma unroll
  for (int g = 0; g < NG; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  auto fma_row = [&](int e, uint2 raw) {
    const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    const float2 v23 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const float p = sm.S[g < SR ? g : 0][e];      // rows g >= G hold stale data; their results are never written
      acc[g][0] = fmaf(p, v01.x, acc[g][0]);
      acc[g][1] = fmaf(p, v01.y, acc[g][1]);
      acc[g][2] = fmaf(p, v23.x, acc[g][2]);
      acc[g][3] = fmaf(p, v23.y, acc[g][3]);
    }
  };
  if (RB > 0) {
    // waves of RB rows through the row buffer; the first one was requested at the top of the call
    bool ok = true;
    for (int w0 = lo; w0 < ne; w0 += RB) {
      const int w1 = min(ne, w0 + RB);
      if (ok) ok = mbar_wait(bar, *phase & 1u);
      ok = __syncthreads_and(ok) != 0;             // block-uniform: a wait that ran out ends the reduction for everyone
      if (!ok) {
        // Give the wave still in flight one more bounded chance to land: the row buffer is then not overwritten
        // under it, and the barrier's phase count stays in step for the block's next edge item.
        if (__syncthreads_and(mbar_wait(bar, *phase & 1u)) != 0) *phase += 1;
        break;
      }
      *phase += 1;
      constexpr int UNR = 8;
      for (int e0 = w0 + warp; e0 < w1; e0 += UNR * EDGE_WARPS) {
        uint2 raw[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int e = e0 + u * EDGE_WARPS;
          raw[u] = (e < w1) ? *reinterpret_cast<const uint2 *>(&sm.rows[(e - w0) * HD * 2 + 8 * lane]) : make_uint2(0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int e = e0 + u * EDGE_WARPS;
          if (e < w1) fma_row(e, raw[u]);
        }
      }
      if (w1 < ne) {
        __syncthreads();                             // every warp has read the wave: the buffer can be refilled
        if (tid == 0) issue_wave(w1, min(ne, w1 + RB));
      }
    }
    if (!ok && tid == 0) atomicExch(a.status, 1);    // result invalid; a copy still in flight may land later
  } else {
    auto row_of = [&](int e) -> const __half * {
      if (e < sink_n) return sinkv + e * HD;
      const int r = e - sink_n;
      if (r < qv_n) return qbufv + r * HD;
      return ringv + ((r - qv_n + C.Write_Offset_Local_V) & (PAGE - 1)) * HD;
    };
    constexpr int UNR = 16;
    for (int e0 = lo + warp; e0 < ne; e0 += UNR * EDGE_WARPS) {
      uint2 raw[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int e = e0 + u * EDGE_WARPS;
        raw[u] = (e < ne) ? *reinterpret_cast<const uint2 *>(row_of(e) + 4 * lane) : make_uint2(0, 0);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int e = e0 + u * EDGE_WARPS;
        if (e < ne) fma_row(e, raw[u]);
      }
    }
  }
  for (int w = 0; w < EDGE_WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int g = 0; g < NG && g < SR; ++g) {
        float4 *dst = reinterpret_cast<float4 *>(&sm.red[g][4 * lane]);
        float4 v = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        if (w > 0) {
          const float4 o = *dst;
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        *dst = v;
      }
    }
    __syncthreads();
  }

  // ---- 4. partial result ---- //
  float *dst = a.partials + ((bh * P.n_slots + P.edge_slot + part) * G) * PART;
  if (tid < HD)
    for (int g = 0; g < G; ++g) dst[g * PART + tid] = sm.red[g][tid];
  if (tid < G) {
    dst[tid * PART + HD] = (ne > lo) ? sm.mx[tid] : -INFINITY;
    dst[tid * PART + HD + 1] = (ne > lo) ? sm.sum[tid] : 0.f;
  }
}

}  // namespace kitty
