// Streaming decode attention over the common packed pages (key page i and
// value page i of one (batch, kv-head)), the hot loop of the decode step.
//
// Data path.  Each warp owns a private ring of shared-memory stages.  One lane
// issues four bulk async copies (cp.async.bulk, completion counted on an
// mbarrier) per page pair: key record 5248 B, key metadata 512 B, value record
// 4096 B, value metadata 512 B — the 10368 algorithmic bytes of the pair, each
// fetched from HBM exactly once.  While a pair is being reduced the next one is
// in flight.
//
// Arithmetic.  The 2-bit fields are never expanded one by one.  A 32-bit word of
// the record holds 16 tokens (keys) or 16 channels (values); two such words are
// byte-permuted into a register whose 16-bit halves hold the same field
// positions of two contraction indices, and `word & (3 << 2f)` IS an fp16x2
// operand: an fp16 subnormal whose value is code * 4^f * 2^-24.  mma.sync
// m16n8k16 (tokens or channels on M, the grouped query heads on N = 8) consumes
// it directly; the power-of-two row factor is applied to the fp32 accumulators.
// Scales are folded into the small operand (q*scale per page for keys, p*scale
// per token for values); the `+ min` terms are rank-1 and are produced by one
// extra mma chain each (rows of min / zero-point against q / p), the value
// chain also yielding the softmax denominator from a row of ones.
//
// Per (page pair, warp): 160 mma.sync and ~1450 other instructions, about 1000 of them on the
// integer/logic pipe, which is what bounds this kernel.  It serves query groups of 5..16 heads;
// groups of up to 4 heads use the int8 kernel (decode_paged_i8.cu).
#include "decode_edge.cuh"

namespace kitty {

constexpr int PG_WARPS = 4;
constexpr int PG_STAGES = 2;
constexpr int OFF_KREC = 0;
constexpr int OFF_KMETA = K_HEAD;                   // 5248
constexpr int OFF_VREC = OFF_KMETA + META_HEAD;     // 5760
constexpr int OFF_VMETA = OFF_VREC + V_HEAD;        // 9856
constexpr int STAGE_BYTES = OFF_VMETA + META_HEAD;  // 10368
constexpr int PB_ROW = 68;                          // words per query-head row of the probability buffer (64 + pad)
constexpr int PB_WORDS = 8 * PB_ROW;

struct PagedSmem {
  __align__(128) uint8_t stage[PG_WARPS][PG_STAGES][STAGE_BYTES];
  __align__(16) uint32_t pbuf[PG_WARPS][PB_WORDS];
  __align__(16) __half qs[8][QS_ROW];
  __align__(8) unsigned long long bar[PG_WARPS][PG_STAGES];
  uint8_t inv[PG_WARPS][DB];
  // copy of the device-resident step state (plan, counters, item counts) when the launch carries one
  DecodePlan dyn_plan;
  kitty_counts dyn_counts;
  int dyn_items, dyn_edge;
};
static_assert(PG_WARPS * 8 * PART * 4 <= PG_WARPS * PG_STAGES * STAGE_BYTES, "merge buffer overlays the stages");

struct PairSrc {
  const uint8_t *krec, *kmeta, *vrec, *vmeta;
};

__device__ __forceinline__ PairSrc pair_src(const DecodeArgs &a, int b, int h, int page) {
  const int H = a.P.H;
  const int64_t pk = a.L.PageTable_K[static_cast<int64_t>(b) * a.L.max_page + page];
  const int64_t pv = a.L.PageTable_V[static_cast<int64_t>(b) * a.L.max_page + page];
  PairSrc s;
  s.krec = a.L.KeyCache + pk * (static_cast<int64_t>(H) * K_HEAD) + static_cast<int64_t>(h) * K_HEAD;
  s.kmeta = static_cast<const uint8_t *>(a.L.KeyCache_metadata) + (pk * H + h) * META_HEAD;
  s.vrec = a.L.ValueCache + pv * (static_cast<int64_t>(H) * V_HEAD) + static_cast<int64_t>(h) * V_HEAD;
  s.vmeta = static_cast<const uint8_t *>(a.L.ValueCache_metadata) + (pv * H + h) * META_HEAD;
  return s;
}

// Edge items (sink + tail parts) run in the same grid after a block's page items; their buffers overlay the
// stages.  NGE: query heads per KV head the edge accumulators are sized for (8 or 16).
using PagedEdge = EdgeSmem<MAX_GROUP, PG_WARPS, 0>;
static_assert(sizeof(PagedEdge) <= PG_WARPS * PG_STAGES * STAGE_BYTES, "the edge buffers overlay the stages only");

// kDyn: the plan, the counters and the item counts come from the device block a.dyn (copied to shared memory once
// per block) instead of the launch arguments.
template <int NGE, bool kDyn>
__global__ void __launch_bounds__(PG_WARPS * 32) decode_paged_kernel(DecodeArgs a, int n_items_arg, int n_gt, int n_edge_arg) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  PagedSmem &sm = *reinterpret_cast<PagedSmem *>(smem_raw);
  dep_wait();          // step-state chain: launched behind the append kernel, whose rows the edge items read
  if (kDyn && threadIdx.x == 0) {
    const kitty_step_state &d = *a.dyn;
    DecodePlan p = a.P;
    p.pb = d.pb; p.pe = d.pe; p.ch = d.ch; p.nchunk = d.nchunk; p.has_sink = d.has_sink; p.has_tail = d.has_tail;
    p.n_slots = d.n_slots; p.n_tiles = d.n_tiles; p.chunk_slot0 = d.chunk_slot0; p.edge_slot = d.edge_slot;
    p.edge_parts = d.edge_parts; p.edge_part_tok = d.edge_part_tok;
    sm.dyn_plan = p;
    sm.dyn_counts = d.after;
    sm.dyn_items = d.n_items;
    sm.dyn_edge = d.n_edge;
  }
  if (kDyn) __syncthreads();
  const DecodePlan &P = kDyn ? sm.dyn_plan : a.P;
  const kitty_counts &C = kDyn ? sm.dyn_counts : a.C;
  const int n_items = kDyn ? sm.dyn_items : n_items_arg;
  const int n_edge = kDyn ? sm.dyn_edge : n_edge_arg;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int H = P.H, G = P.G;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < PG_STAGES; ++s) mbar_init(smem_u32(&sm.bar[warp][s]), 1);
  }
  if (lane < DB) sm.inv[warp][lane] = 0;
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();
  dep_release();       // the merge kernel that follows may be scheduled now; it waits for this grid to complete

  uint32_t seq = 0;          // page pairs consumed by this warp so far (ring position and parity)
  bool dead = false;         // a bounded wait ran out: stop consuming, keep the barriers uniform
  uint32_t inflight = 0;     // bit s: stage s has a copy in flight (lane 0's view, kept warp-uniform)

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int c = item % P.nchunk;
    const int gt = (item / P.nchunk) % n_gt;
    const int bh = item / (P.nchunk * n_gt);
    const int h = bh % H, b = bh / H;
    const int p0 = P.pb + c * P.ch;
    const int p1 = min(a.rows != nullptr ? min(P.pe, a.rows[b].PageCount_V) : P.pe, p0 + P.ch);
    const int g_valid = min(8, G - gt * 8);

    __syncthreads();   // previous item's merge buffer (overlaying the stages) and query are no longer read
    for (int i = tid; i < 8 * HD; i += PG_WARPS * 32) {
      const int g = i >> 7, d = i & (HD - 1);
      float v = 0.f;
      if (g < g_valid) v = load_q(a.q, a.q_dtype, (static_cast<int64_t>(b) * P.h_q + h * G + gt * 8 + g) * HD + d) * a.scale_log2;
      sm.qs[g][d] = __float2half_rn(v);
    }
    // first copies of this warp: pages p0 + warp, p0 + warp + PG_WARPS, ...
    const int first = p0 + warp;
    if (lane == 0 && !dead) {
      // the stages were last written through the generic proxy (merge buffer); order that before the bulk copies
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#pragma unroll
      for (int s = 0; s < PG_STAGES; ++s) {
        const int pg = first + s * PG_WARPS;
        if (pg < p1) {
          const uint32_t st = (seq + s) % PG_STAGES;
          const uint32_t bar = smem_u32(&sm.bar[warp][st]);
          const uint32_t dst = smem_u32(&sm.stage[warp][st][0]);
          const PairSrc src = pair_src(a, b, h, pg);
          mbar_expect_tx(bar, STAGE_BYTES);
          bulk_g2s(dst + OFF_KREC, src.krec, K_HEAD, bar);
          bulk_g2s(dst + OFF_KMETA, src.kmeta, META_HEAD, bar);
          bulk_g2s(dst + OFF_VREC, src.vrec, V_HEAD, bar);
          bulk_g2s(dst + OFF_VMETA, src.vmeta, META_HEAD, bar);
          inflight |= 1u << st;
        }
      }
    }
    inflight = __shfl_sync(0xffffffffu, inflight, 0);
    __syncthreads();   // staged query visible

    uint32_t q2[8][2];
    load_q_frags(sm.qs, gid, tig, q2);

    float acc[8][4];       // out[channel 16*gid + m (+8)][head 2*tig (+1)], still carrying the field weight
    float cz[4] = {0.f, 0.f, 0.f, 0.f};   // [0,1]: sum p*zero-point, [2,3]: sum p, heads 2*tig, 2*tig+1
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    float m_run0 = -INFINITY, m_run1 = -INFINITY;

    for (int pg = first; pg < p1; pg += PG_WARPS) {
      if (dead) break;
      const uint32_t st = seq % PG_STAGES, parity = (seq / PG_STAGES) & 1u;
      const uint32_t bar = smem_u32(&sm.bar[warp][st]);
      if (!mbar_wait(bar, parity)) {
        dead = true;
        if (lane == 0) atomicExch(a.status, 1);
        break;
      }
      inflight &= ~(1u << st);
      const uint8_t *stg = sm.stage[warp][st];
      const uint32_t *vw = reinterpret_cast<const uint32_t *>(stg + OFF_VREC);
      const uint32_t *vm = reinterpret_cast<const uint32_t *>(stg + OFF_VMETA);

      // ================= Q K^T ================= //
      float cl[8][4];    // logits[token 16*gid + m (+8)][head 2*tig (+1)]
      qk_packed_page(stg + OFF_KREC, reinterpret_cast<const uint32_t *>(stg + OFF_KMETA), sm.qs, q2, sm.inv[warp], lane, cl);

      // ================= online softmax ================= //
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        mx0 = fmaxf(mx0, fmaxf(cl[m][0], cl[m][2]));
        mx1 = fmaxf(mx1, fmaxf(cl[m][1], cl[m][3]));
      }
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
      }
      const float mn0 = fmaxf(m_run0, mx0), mn1 = fmaxf(m_run1, mx1);
      if (__any_sync(0xffffffffu, (mn0 > m_run0) || (mn1 > m_run1))) {
        const float a0 = (m_run0 == -INFINITY) ? 0.f : ex2(m_run0 - mn0);
        const float a1 = (m_run1 == -INFINITY) ? 0.f : ex2(m_run1 - mn1);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          acc[m][0] *= a0; acc[m][1] *= a1; acc[m][2] *= a0; acc[m][3] *= a1;
        }
        cz[0] *= a0; cz[1] *= a1; cz[2] *= a0; cz[3] *= a1;
        m_run0 = mn0;
        m_run1 = mn1;
      }
      // probabilities, as fp16 pairs (token 16*gid + m, token 16*gid + 8 + m), into the warp's buffer
      {
        uint32_t pw[2][8];
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const int pos = (m & 3) * 2 + (m >> 2);
          pw[0][pos] = pack_h2(ex2(cl[m][0] - m_run0), ex2(cl[m][2] - m_run0));
          pw[1][pos] = pack_h2(ex2(cl[m][1] - m_run1), ex2(cl[m][3] - m_run1));
        }
        uint32_t *pb = sm.pbuf[warp];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint4 *dst = reinterpret_cast<uint4 *>(pb + (2 * tig + j) * PB_ROW + gid * 8);
          dst[0] = make_uint4(pw[j][0], pw[j][1], pw[j][2], pw[j][3]);
          dst[1] = make_uint4(pw[j][4], pw[j][5], pw[j][6], pw[j][7]);
        }
      }
      __syncwarp();

      // ================= P V ================= //
      // contraction index k = 2*tig, 2*tig+1, 2*tig+8, 2*tig+9  <->  tokens 16*ks + tig + {0, 8, 4, 12}
      const uint32_t ones = 0x3c003c00u;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint2 pp = *reinterpret_cast<const uint2 *>(sm.pbuf[warp] + gid * PB_ROW + ks * 8 + 2 * tig);
        const int t = 16 * ks + tig;
        const uint32_t m0 = vm[t], m1 = vm[t + 8], m2 = vm[t + 4], m3 = vm[t + 12];       // (scale | zero << 16)
        const uint32_t b0 = hmul2_u(pp.x, __byte_perm(m0, m1, 0x5410));
        const uint32_t b1 = hmul2_u(pp.y, __byte_perm(m2, m3, 0x5410));
        mma16816(cz, __byte_perm(m0, m1, 0x7632), ones, __byte_perm(m2, m3, 0x7632), ones, pp.x, pp.y);
        const uint32_t w0 = vw[t * 8 + gid], w1 = vw[(t + 8) * 8 + gid], w2 = vw[(t + 4) * 8 + gid],
                       w3 = vw[(t + 12) * 8 + gid];
        const uint32_t xab = __byte_perm(w0, w1, 0x5410), yab = __byte_perm(w0, w1, 0x7632);
        const uint32_t xcd = __byte_perm(w2, w3, 0x5410), ycd = __byte_perm(w2, w3, 0x7632);
        const uint32_t xabs = xab >> 10, yabs = yab >> 10, xcds = xcd >> 10, ycds = ycd >> 10;
#pragma unroll
        for (int m = 0; m < 8; ++m)
          mma16816(acc[m], field(xab, xabs, m), field(yab, yabs, m), field(xcd, xcds, m), field(ycd, ycds, m), b0, b1);
      }
      __syncwarp();      // every lane is done with this stage and with the probability buffer
      ++seq;
      const int nxt = pg + PG_STAGES * PG_WARPS;
      if (nxt < p1) {
        if (lane == 0) {
          const uint32_t dst = smem_u32(&sm.stage[warp][st][0]);
          const PairSrc src = pair_src(a, b, h, nxt);
          mbar_expect_tx(bar, STAGE_BYTES);
          bulk_g2s(dst + OFF_KREC, src.krec, K_HEAD, bar);
          bulk_g2s(dst + OFF_KMETA, src.kmeta, META_HEAD, bar);
          bulk_g2s(dst + OFF_VREC, src.vrec, V_HEAD, bar);
          bulk_g2s(dst + OFF_VMETA, src.vmeta, META_HEAD, bar);
        }
        inflight |= 1u << st;
      }
    }

    if (dead) {
      // give copies still in flight a bounded time to land before the stages are reused or the block exits
      for (int s = 0; s < PG_STAGES; ++s)
        if (inflight & (1u << s)) {
          mbar_wait(smem_u32(&sm.bar[warp][s]), ((seq + ((s + PG_STAGES - seq % PG_STAGES) % PG_STAGES)) / PG_STAGES) & 1u);
          inflight &= ~(1u << s);
        }
    }
    __syncthreads();     // all warps have consumed every copy they issued: the stages can be overlaid

    // ---- warp result -> merge buffer [warp][head][PART] ---- //
    float *mb = reinterpret_cast<float *>(&sm.stage[0][0][0]);
    {
      float *w = mb + warp * 8 * PART;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const float u = field_unscale(m);
        w[(2 * tig) * PART + 16 * gid + m] = fmaf(acc[m][0], u, cz[0]);
        w[(2 * tig + 1) * PART + 16 * gid + m] = fmaf(acc[m][1], u, cz[1]);
        w[(2 * tig) * PART + 16 * gid + 8 + m] = fmaf(acc[m][2], u, cz[0]);
        w[(2 * tig + 1) * PART + 16 * gid + 8 + m] = fmaf(acc[m][3], u, cz[1]);
      }
      if (gid == 0) {
        w[(2 * tig) * PART + HD] = m_run0;
        w[(2 * tig) * PART + HD + 1] = cz[2];
        w[(2 * tig + 1) * PART + HD] = m_run1;
        w[(2 * tig + 1) * PART + HD + 1] = cz[3];
      }
    }
    __syncthreads();
    {
      float *dst = a.partials + ((static_cast<int64_t>(bh) * P.n_slots + (P.chunk_slot0 + c)) * G + gt * 8) * PART;
      for (int g = 0; g < g_valid; ++g) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < PG_WARPS; ++w) M = fmaxf(M, mb[(w * 8 + g) * PART + HD]);
        float A = 0.f, Ls = 0.f;
#pragma unroll
        for (int w = 0; w < PG_WARPS; ++w) {
          const float mw = mb[(w * 8 + g) * PART + HD];
          const float wt = (mw == -INFINITY) ? 0.f : ex2(mw - M);
          A = fmaf(mb[(w * 8 + g) * PART + tid], wt, A);
          Ls = fmaf(mb[(w * 8 + g) * PART + HD + 1], wt, Ls);
        }
        dst[g * PART + tid] = A;
        if (tid == 0) {
          dst[g * PART + HD] = M;
          dst[g * PART + HD + 1] = Ls;
        }
      }
    }
  }

  // ---- edge items, handed out from the last block backwards (those blocks have the fewest page items) ---- //
  PagedEdge &es = *reinterpret_cast<PagedEdge *>(smem_raw);
  for (int e = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x); e < n_edge; e += gridDim.x) {
    __syncthreads();     // the previous item's merge buffer / edge buffers are no longer read
    const int ebh = e / P.edge_parts, part = e % P.edge_parts;
    edge_item<NGE, PG_WARPS>(a, P, row_counts(a, C, ebh / H), es, ebh / H, ebh % H, part);
  }
}

int launch_decode_paged(const DecodeArgs &a, int n_items, int n_gt, int n_edge, int grid, cudaStream_t s, bool dependent) {
  static PerDeviceOnce once;      // opt-in to > 48 KB dynamic shared memory, once per device
  if (int rc = per_device_once(once, [] {
        const int smem = static_cast<int>(sizeof(PagedSmem));
        return (cudaFuncSetAttribute(decode_paged_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                cudaFuncSetAttribute(decode_paged_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                cudaFuncSetAttribute(decode_paged_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                cudaFuncSetAttribute(decode_paged_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess)
                   ? KITTY_OK : KITTY_E_CUDA;
      }))
    return rc;
  const dim3 g(grid), b(PG_WARPS * 32);
  const size_t sh = sizeof(PagedSmem);
  if (dependent && a.dyn != nullptr) {
    const cudaError_t e = (a.P.G <= 8) ? launch_after(decode_paged_kernel<8, true>, g, b, sh, s, a, n_items, n_gt, n_edge)
                                       : launch_after(decode_paged_kernel<16, true>, g, b, sh, s, a, n_items, n_gt, n_edge);
    return (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? KITTY_OK : KITTY_E_CUDA;
  }
  if (a.dyn != nullptr) {
    if (a.P.G <= 8) decode_paged_kernel<8, true><<<g, b, sh, s>>>(a, n_items, n_gt, n_edge);
    else decode_paged_kernel<16, true><<<g, b, sh, s>>>(a, n_items, n_gt, n_edge);
  } else {
    if (a.P.G <= 8) decode_paged_kernel<8, false><<<g, b, sh, s>>>(a, n_items, n_gt, n_edge);
    else decode_paged_kernel<16, false><<<g, b, sh, s>>>(a, n_items, n_gt, n_edge);
  }
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}

int paged_smem_bytes() { return static_cast<int>(sizeof(PagedSmem)); }

}  // namespace kitty
