// Streaming decode attention over the common packed pages for query groups of up
// to 8 heads per KV head — the integer tensor-core variant of the hot loop.
// (NG = 1: up to 4 heads; NG = 2: 5..8 heads as two operand groups of 4 that share
// every masked code fragment, so the unpacking work is done once per page.)
//
// Data path.  Each warp owns one shared-memory stage with a key part (record
// 5248 B + metadata 512 B) and a value part (4096 B + 512 B), each filled by bulk
// async copies (cp.async.bulk) that complete on the part's own mbarrier.  As soon
// as the warp has consumed the key part of page i it requests the key part of its
// next page, which lands while the warp does softmax and P V; the value part is
// re-requested after P V and lands during the next Q K^T.  One stage per warp keeps
// shared memory at ~13 KB per warp, so 16 warps (4 blocks) are resident per SM.
// The 10368 bytes of a page pair are fetched from HBM exactly once.
//
// Arithmetic: mma.sync.m16n8k32 on 8-bit integers.
//  * A operand = the packed codes themselves.  A record is a matrix of 32-byte
//    rows (one row per channel for keys, per token for values) whose bytes hold 4
//    fields.  `ldmatrix.m16n16.x2.trans.b8` reads 32 rows x 16 byte columns
//    transposed and hands every lane exactly the A fragment of m16n8k32 (rows =
//    byte columns, contraction index = record row); `reg & (0x03030303 << 2r)` is
//    then the u8 operand code * 4^r of field r — four fields per logic
//    instruction, no shifts and no byte permutes.  Tile (half hf, field r) row m
//    is token (or channel) 64*hf + 4*m + r.
//  * B operand = the small vector (q*scale for keys, p*scale for values) in
//    16-bit fixed point, split into a high and a low 8-bit limb.  The 8 columns
//    of the tile are (head, limb) for 4 heads, so one mma covers both limbs and
//    every tensor-core column does useful work; hi*256 + lo is recombined in the
//    fp32 epilogue together with the power-of-two weight 4^-r and the page's
//    fixed-point scale.  Conversion to fixed point is a fused multiply-add with
//    the magic constant 1.5*2^23 (the integer lands in the mantissa).
//  * The rank-1 terms (sum q*min, sum p*zero, sum p) are a few fp32 FMAs per lane.
// Per page pair and warp: 72 mma.sync, 18 ldmatrix and roughly 800 other instructions.
//
// Every wait on an mbarrier is bounded; when one runs out the warp sets the
// workspace's status word, stops consuming and the call's result is invalid.
#include "decode_edge.cuh"

namespace kitty {

constexpr int I8_WARPS = 4;
constexpr int I8_KPART = K_HEAD + META_HEAD;              // 5760
constexpr int I8_VPART = V_HEAD + META_HEAD;              // 4608
constexpr int PB_RS = 36;                                 // words per (head, limb) row of the probability buffer (32 + pad)
constexpr int QROW = HD + 4;                              // floats per row of the arranged query (pad against bank conflicts)
constexpr int I8_OFF_KREC = 0;
constexpr int I8_OFF_KMETA = K_HEAD;                      // 5248
constexpr int I8_OFF_VREC = I8_OFF_KMETA + META_HEAD;     // 5760
constexpr int I8_OFF_VMETA = I8_OFF_VREC + V_HEAD;        // 9856
constexpr int I8_STAGE_BYTES = I8_OFF_VMETA + META_HEAD;  // 10368
constexpr float KFIX = 8000.0f;     // |q^ * scale'| <= KFIX; the high plane uses 4x that, still inside int16
constexpr float VFIX = 60000.0f;    // p * scale' <= VFIX < 2^16 (unsigned limbs)
constexpr float MAGIC_S = 12582912.0f;   // 1.5 * 2^23: signed integers in the low mantissa bits
constexpr float MAGIC_U = 8388608.0f;    // 2^23: unsigned integers in the low mantissa bits

// The contraction index of a k-step is the record row itself: bytes 4*tg + i of the B registers
// <-> rows 32*ks + 4*tg + i (b0) and 32*ks + 16 + 4*tg + i (b1).
template <int NG>
struct I8Warp {
  __align__(128) uint8_t stage[I8_STAGE_BYTES];
  __align__(16) float sarr[HD];        // keys: scale' per channel; values: scale' per token
  __align__(16) float marr[HD];        // keys: min per channel;    values: zero-point per token
  __align__(16) uint32_t pb[NG][8 * PB_RS]; // probabilities * scale' as limb bytes: [group][head*2 + limb][token / 4] words
  uint8_t inv[DB];                     // slot -> its channel
};

template <int NG>
struct I8Main {
  I8Warp<NG> w[I8_WARPS];
  __align__(16) float qarr[4 * NG][QROW];   // query / qmax per head
  float qmax[4 * NG];
};

// Edge items bring their value rows in waves (28 KB / 26 KB) by bulk copies: what is left of the block's
// shared memory once the edge's own buffers are sized for the query heads.
template <int NG>
using I8Edge = EdgeSmem<4 * NG, I8_WARPS, (NG == 1) ? 112 : 104>;

// A block alternates between page-pair items and edge items (sink + tail of one (batch, kv-head)); the two
// kinds reuse the same shared memory.  The mbarriers live outside the shared region.
template <int NG>
struct I8Smem {
  union U {
    I8Main<NG> m;
    I8Edge<NG> e;
  } u;
  __align__(8) unsigned long long bar_k[I8_WARPS], bar_v[I8_WARPS], bar_e;
  int next_item;
  // copy of the device-resident step state (plan, counters, item counts) when the launch carries one
  DecodePlan dyn_plan;
  kitty_counts dyn_counts;
  int dyn_items, dyn_edge;
};
static_assert(I8_WARPS * 4 * PART * 4 <= sizeof(I8Warp<1>) * 2, "merge buffer overlays the first warps' buffers");
static_assert(I8_WARPS * 8 * PART * 4 <= sizeof(I8Warp<2>) * 2, "merge buffer overlays the first warps' buffers");
static_assert(sizeof(I8Smem<1>) <= 56 * 1024, "four blocks per SM");
static_assert(sizeof(I8Smem<2>) <= 75 * 1024, "three blocks per SM");
static_assert(sizeof(I8Edge<1>) <= sizeof(I8Main<1>) + 512, "the edge buffers should not grow the block's shared memory");
static_assert(sizeof(I8Edge<2>) <= sizeof(I8Main<2>) + 512, "the edge buffers should not grow the block's shared memory");

__device__ __forceinline__ void imma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_u8u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four fixed-point values -> one B register holding their limb bytes.  sel picks the byte
// (0x0040: byte 0 of both sources, 0x0051: byte 1 of both sources).
__device__ __forceinline__ uint32_t pack_limb(float y0, float y1, float y2, float y3, uint32_t sel) {
  const uint32_t p01 = __byte_perm(__float_as_uint(y0), __float_as_uint(y1), sel);
  const uint32_t p23 = __byte_perm(__float_as_uint(y2), __float_as_uint(y3), sel);
  return __byte_perm(p01, p23, 0x5410);
}

// One k-step of 32 contraction indices (record rows k0 .. k0+31) against the 128 byte-column x field rows, for NG
// small operands at once: the code fragments are loaded and masked once and fed to every group's accumulators.
// row_addr: shared-memory address of row k0 + lane of the record (32 bytes per row).  Tile 4*hf + r:
// fragment row m (gid, gid + 8) <-> byte column 16*hf + m, field r <-> index 64*hf + 4*m + r, weight 4^r.
template <bool kSignedB, int NG>
__device__ __forceinline__ void kstep32(uint32_t row_addr, const uint32_t (&b0)[NG], const uint32_t (&b1)[NG],
                                        int (&c)[NG][8][4]) {
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    uint32_t a0, a1, a2, a3;
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                 : "r"(row_addr + 16 * hf));
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const uint32_t msk = 0x03030303u << (2 * r);
      const uint32_t m0 = a0 & msk, m1 = a1 & msk, m2 = a2 & msk, m3 = a3 & msk;
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        if (kSignedB) imma_u8s8(c[g][4 * hf + r], m0, m1, m2, m3, b0[g], b1[g]);
        else imma_u8u8(c[g][4 * hf + r], m0, m1, m2, m3, b0[g], b1[g]);
      }
    }
    // field 3 needs no mask: the whole byte goes in, and fields 0..2 are subtracted once per page (finish_tiles)
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      if (kSignedB) imma_u8s8(c[g][4 * hf + 3], a0, a1, a2, a3, b0[g], b1[g]);
      else imma_u8u8(c[g][4 * hf + 3], a0, a1, a2, a3, b0[g], b1[g]);
    }
  }
}

// After the last k-step: tile 4*hf + 3 accumulated the whole bytes (all four fields); remove fields 0..2.
__device__ __forceinline__ void finish_tiles(int (&c)[8][4]) {
#pragma unroll
  for (int hf = 0; hf < 2; ++hf)
#pragma unroll
    for (int i = 0; i < 4; ++i) c[4 * hf + 3][i] -= c[4 * hf][i] + c[4 * hf + 1][i] + c[4 * hf + 2][i];
}

// pk / pv: the page's row in the cache (page-table entry), read by the caller well before the copy is
// issued so that the table lookup does not stall the warp.
__device__ __forceinline__ void i8_issue_k(const DecodeArgs &a, int h, int64_t pk, uint32_t dst, uint32_t bar) {
  const int H = a.P.H;
  mbar_expect_tx(bar, I8_KPART);
  bulk_g2s(dst + I8_OFF_KREC, a.L.KeyCache + pk * (static_cast<int64_t>(H) * K_HEAD) + static_cast<int64_t>(h) * K_HEAD, K_HEAD, bar);
  bulk_g2s(dst + I8_OFF_KMETA, static_cast<const uint8_t *>(a.L.KeyCache_metadata) + (pk * H + h) * META_HEAD, META_HEAD, bar);
}
__device__ __forceinline__ void i8_issue_v(const DecodeArgs &a, int h, int64_t pv, uint32_t dst, uint32_t bar) {
  const int H = a.P.H;
  mbar_expect_tx(bar, I8_VPART);
  bulk_g2s(dst + I8_OFF_VREC, a.L.ValueCache + pv * (static_cast<int64_t>(H) * V_HEAD) + static_cast<int64_t>(h) * V_HEAD, V_HEAD, bar);
  bulk_g2s(dst + I8_OFF_VMETA, static_cast<const uint8_t *>(a.L.ValueCache_metadata) + (pv * H + h) * META_HEAD, META_HEAD, bar);
}

// kDyn: the plan, the counters and the item counts come from the device block a.dyn (copied to shared
// memory once per block) instead of the launch arguments.  NG: operand groups of 4 query heads (1 or 2).
template <int NG, bool kDyn>
__global__ void __launch_bounds__(I8_WARPS * 32, NG == 1 ? 4 : 3) decode_paged_i8_kernel(DecodeArgs a, int n_items_arg, int n_edge_arg) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  I8Smem<NG> &smem = *reinterpret_cast<I8Smem<NG> *>(smem_raw);
  I8Main<NG> &sm = smem.u.m;
  dep_wait();          // step-state chain: launched behind the append kernel, whose rows the edge items read
  if (kDyn && threadIdx.x == 0) {
    const kitty_step_state &d = *a.dyn;
    DecodePlan p = a.P;
    p.pb = d.pb; p.pe = d.pe; p.ch = d.ch; p.nchunk = d.nchunk; p.has_sink = d.has_sink; p.has_tail = d.has_tail;
    p.n_slots = d.n_slots; p.n_tiles = d.n_tiles; p.chunk_slot0 = d.chunk_slot0; p.edge_slot = d.edge_slot;
    p.edge_parts = d.edge_parts; p.edge_part_tok = d.edge_part_tok;
    smem.dyn_plan = p;
    smem.dyn_counts = d.after;
    smem.dyn_items = d.n_items;
    smem.dyn_edge = d.n_edge;
  }
  if (kDyn) __syncthreads();
  const DecodePlan &P = kDyn ? smem.dyn_plan : a.P;
  const kitty_counts &C = kDyn ? smem.dyn_counts : a.C;
  const int n_items = kDyn ? smem.dyn_items : n_items_arg;
  const int n_edge = kDyn ? smem.dyn_edge : n_edge_arg;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int H = P.H, G = P.G;
  I8Warp<NG> &ws = sm.w[warp];
  const int colhead = gid >> 1;                                   // B column gid = (head of the group, limb)
  const bool hi_limb = (gid & 1) == 0;
  const uint32_t limb_sel = hi_limb ? 0x0051u : 0x0040u;
  const float kmagic = MAGIC_S + (hi_limb ? 128.0f : 0.0f);       // +128: rounds the low limb into the high one

  if (lane == 0) {
    mbar_init(smem_u32(&smem.bar_k[warp]), 1);
    mbar_init(smem_u32(&smem.bar_v[warp]), 1);
    if (warp == 0) mbar_init(smem_u32(&smem.bar_e), 1);
  }
  ws.inv[lane] = 0;
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();
  dep_release();       // the merge kernel that follows may be scheduled now; it waits for this grid to complete

  uint32_t kseq = 0, vseq = 0;   // key / value parts consumed by this warp so far (parity of each part's mbarrier)
  uint32_t edge_phase = 0;   // completed phases of the edge row barrier (block-uniform)
  bool dead = false;         // a bounded wait ran out: stop consuming, keep the block barriers uniform
  uint32_t inflight = 0;     // bit 0: a key-part copy is in flight, bit 1: a value-part copy (warp-uniform)
  const uint32_t bar_k = smem_u32(&smem.bar_k[warp]), bar_v = smem_u32(&smem.bar_v[warp]), stage_u32 = smem_u32(&ws.stage[0]);

  // Items are handed out dynamically (a work counter in the workspace header, zero on entry and reset by
  // the merge kernel that always follows), so blocks stay busy until the list is empty.  (Requesting the next
  // item ahead of time, to hide the atomic's round trip, measured slower: blocks then hold work they cannot start.)
  // The page-pair items come first and the edge items last: an edge item is the shorter of the two kinds, so the
  // tail of the launch is made of short items (spreading the edge items evenly through the list measured 2.5 %
  // slower at batch 128 and 5 % slower at batch 64; all edge items first measured like the even spread).
  const long long total = static_cast<long long>(n_items) + n_edge;
  for (;;) {
    __syncthreads();     // the previous item's merge buffer, query and work index are no longer read
    if (tid == 0) smem.next_item = atomicAdd(a.status + 1, 1);
    __syncthreads();
    const long long it = smem.next_item;
    if (it >= total) break;
    const int e_before = it < n_items ? 0 : static_cast<int>(it - n_items);
    const int e_after = it < n_items ? 0 : e_before + 1;
    const int item = static_cast<int>(it) - e_before;        // index among the page-pair items
    if (e_after > e_before) {
      // ---- edge item: one part of the sink + tail of one (batch, kv-head), by the whole block ---- //
      const int ebh = e_before / P.edge_parts, part = e_before % P.edge_parts;
      edge_item<4 * NG, I8_WARPS>(a, P, row_counts(a, C, ebh / H), smem.u.e, ebh / H, ebh % H, part,
                                  smem_u32(&smem.bar_e), &edge_phase);
      __syncthreads();
      ws.inv[lane] = 0;  // the slot table was overwritten: keep its entries valid positions
      continue;
    }
    const int c = item % P.nchunk;
    const int bh = item / P.nchunk;
    const int h = bh % H, b = bh / H;
    const int p0 = P.pb + c * P.ch;
    const int p1 = min(a.rows != nullptr ? min(P.pe, a.rows[b].PageCount_V) : P.pe, p0 + P.ch);

    // this warp's pages: p0 + warp, p0 + warp + I8_WARPS, ...  (requested first: the copies fly while the
    // query is staged)
    const int first = p0 + warp;
    if (!dead && first < p1) {
      if (lane == 0) {
        // the stage may have been written through the generic proxy (merge buffer): order that before the bulk copies
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        i8_issue_k(a, h, a.L.PageTable_K[static_cast<int64_t>(b) * a.L.max_page + first], stage_u32, bar_k);
        i8_issue_v(a, h, a.L.PageTable_V[static_cast<int64_t>(b) * a.L.max_page + first], stage_u32, bar_v);
      }
      inflight = 3u;
    }
    // ---- queries of heads warp, warp + 4, ...: maximum, then q / qmax ---- //
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const int hq = 4 * g + warp;
      float qv[4], mx = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int cch = 4 * lane + i;
        qv[i] = (hq < G) ? load_q(a.q, a.q_dtype, (static_cast<int64_t>(b) * P.h_q + h * G + hq) * HD + cch) * a.scale_log2 : 0.f;
        mx = fmaxf(mx, fabsf(qv[i]));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mx = fmaxf(mx, 1e-30f);
      const float inv_mx = 1.0f / mx;
      *reinterpret_cast<float4 *>(&sm.qarr[hq][4 * lane]) =
          make_float4(qv[0] * inv_mx, qv[1] * inv_mx, qv[2] * inv_mx, qv[3] * inv_mx);
      if (lane == 0) sm.qmax[hq] = mx;
    }
    __syncthreads();   // staged query visible

    // This lane's output heads are 4*g + tig (accumulator columns 2*tig, 2*tig+1 of group g = high and low limb).
    float qmax_t[NG];
    float acc[NG][8][2];   // out[channel 64*hf + 4*gid + r (+32)][head 4*g + tig], tile 4*hf + r
    float zsum[NG], lsum[NG];          // this lane's share of sum p*zero-point and sum p (its 16 tokens, head 4*g + tig)
    float m_run[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      qmax_t[g] = sm.qmax[4 * g + tig];
#pragma unroll
      for (int m = 0; m < 8; ++m) acc[g][m][0] = acc[g][m][1] = 0.f;
      zsum[g] = lsum[g] = 0.f;
      m_run[g] = -INFINITY;
    }

    for (int pg = first; pg < p1 && !dead; pg += I8_WARPS) {
      const int nxt = pg + I8_WARPS;
      // page-table entries of the next page: requested now, used after Q K^T / P V
      uint32_t pk_nxt = 0, pv_nxt = 0;
      if (nxt < p1) {
        pk_nxt = static_cast<uint32_t>(a.L.PageTable_K[static_cast<int64_t>(b) * a.L.max_page + nxt]);
        pv_nxt = static_cast<uint32_t>(a.L.PageTable_V[static_cast<int64_t>(b) * a.L.max_page + nxt]);
      }
      if (!mbar_wait(bar_k, kseq & 1u)) { dead = true; break; }
      ++kseq;
      inflight &= ~1u;
      const uint8_t *stg = ws.stage;
      const uint32_t *km = reinterpret_cast<const uint32_t *>(stg + I8_OFF_KMETA);
      const uint32_t *vm = reinterpret_cast<const uint32_t *>(stg + I8_OFF_VMETA);

      // ---- key pre-pass: slot table, scale' = scale * KFIX / max scale and min ---- //
      float k_unit;      // value of one fixed-point unit of q^ * scale
      {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(stg + I8_OFF_KREC + K_OFF_IDX + 4 * lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t s = (w >> (8 * i)) & 0xffu;
          if (s < DB) ws.inv[s] = static_cast<uint8_t>(4 * lane + i);
        }
        float sc[4], mn[4], smax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&km[4 * lane + i]));
          sc[i] = f.x;
          mn[i] = f.y;
          smax = fmaxf(smax, f.x);
        }
        // scales are positive, so their order is the order of their bit patterns: one integer warp reduction
        smax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(smax)));
        const float fix = KFIX * __frcp_rn(smax);          // scale >= 1e-6 by construction of the pages
        k_unit = smax * (1.0f / KFIX);
        *reinterpret_cast<float4 *>(&ws.sarr[4 * lane]) = make_float4(sc[0] * fix, sc[1] * fix, sc[2] * fix, sc[3] * fix);
        *reinterpret_cast<float4 *>(&ws.marr[4 * lane]) = make_float4(mn[0], mn[1], mn[2], mn[3]);
      }
      __syncwarp();

      // ================= Q K^T ================= //
      int cl[NG][8][4];  // [group][tile][hi row gid, lo row gid, hi row gid+8, lo row gid+8] of head 4*g + tig
#pragma unroll
      for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int m = 0; m < 8; ++m) cl[g][m][0] = cl[g][m][1] = cl[g][m][2] = cl[g][m][3] = 0;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const int pos = ks * 32 + tig * 4;
        const float4 sa = *reinterpret_cast<const float4 *>(&ws.sarr[pos]), sb = *reinterpret_cast<const float4 *>(&ws.sarr[pos + 16]);
        uint32_t b0[NG], b1[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const float *qrow = sm.qarr[4 * g + colhead];
          const float4 qa = *reinterpret_cast<const float4 *>(qrow + pos), qb = *reinterpret_cast<const float4 *>(qrow + pos + 16);
          b0[g] = pack_limb(fmaf(qa.x, sa.x, kmagic), fmaf(qa.y, sa.y, kmagic), fmaf(qa.z, sa.z, kmagic),
                            fmaf(qa.w, sa.w, kmagic), limb_sel);
          b1[g] = pack_limb(fmaf(qb.x, sb.x, kmagic), fmaf(qb.y, sb.y, kmagic), fmaf(qb.z, sb.z, kmagic),
                            fmaf(qb.w, sb.w, kmagic), limb_sel);
        }
        kstep32<true, NG>(stage_u32 + I8_OFF_KREC + (32 * ks + lane) * 32, b0, b1, cl);
      }
      // high plane: 32 slots = one k-step; bytes 4*tig + i <-> slot 4*tig + i, bytes 16 + 4*tig + i <-> slot 16 + 4*tig + i;
      // operand = 4 * q^ * scale' of the slot's channel
      {
        const uint32_t ia = *reinterpret_cast<const uint32_t *>(&ws.inv[4 * tig]);
        const uint32_t ib = *reinterpret_cast<const uint32_t *>(&ws.inv[16 + 4 * tig]);
        uint32_t b0[NG], b1[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const float *qrow = sm.qarr[4 * g + colhead];
          float ya[4], yb[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int pa = (ia >> (8 * i)) & 0xff, pb2 = (ib >> (8 * i)) & 0xff;
            ya[i] = fmaf(qrow[pa] * 4.0f, ws.sarr[pa], kmagic);
            yb[i] = fmaf(qrow[pb2] * 4.0f, ws.sarr[pb2], kmagic);
          }
          b0[g] = pack_limb(ya[0], ya[1], ya[2], ya[3], limb_sel);
          b1[g] = pack_limb(yb[0], yb[1], yb[2], yb[3], limb_sel);
        }
        kstep32<true, NG>(stage_u32 + I8_OFF_KREC + K_OFF_HI + lane * 32, b0, b1, cl);
      }
#pragma unroll
      for (int g = 0; g < NG; ++g) finish_tiles(cl[g]);
      __syncwarp();      // every lane is done with the key part: request the next page's
      if (nxt < p1) {
        if (lane == 0) i8_issue_k(a, h, pk_nxt, stage_u32, bar_k);
        inflight |= 1u;
      }
      // sum_c q*min for head 4*g + tig: this lane covers channels 16*gid .. 16*gid+15
      float bias[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float bs = 0.f;
        const float *qt = sm.qarr[4 * g + tig] + 16 * gid;
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const float4 qq = *reinterpret_cast<const float4 *>(qt + 4 * v4);
          const float4 mm = *reinterpret_cast<const float4 *>(&ws.marr[16 * gid + 4 * v4]);
          bs = fmaf(qq.x, mm.x, bs);
          bs = fmaf(qq.y, mm.y, bs);
          bs = fmaf(qq.z, mm.z, bs);
          bs = fmaf(qq.w, mm.w, bs);
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) bs += __shfl_xor_sync(0xffffffffu, bs, o);
        bias[g] = bs * qmax_t[g];
      }

      // ---- value pre-pass (plain token order): scale' = scale * VFIX / max scale, zero-point ---- //
      if (!mbar_wait(bar_v, vseq & 1u)) { dead = true; break; }
      ++vseq;
      inflight &= ~2u;
      float v_unit;
      {
        float sc[4], zp[4], smax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&vm[4 * lane + i]));
          sc[i] = f.x;
          zp[i] = f.y;
          smax = fmaxf(smax, f.x);
        }
        smax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(smax)));
        const float fix = VFIX * __frcp_rn(smax);
        v_unit = smax * (1.0f / VFIX);
        __syncwarp();                                      // every lane has read the key scales and mins
        *reinterpret_cast<float4 *>(&ws.sarr[4 * lane]) = make_float4(sc[0] * fix, sc[1] * fix, sc[2] * fix, sc[3] * fix);
        *reinterpret_cast<float4 *>(&ws.marr[4 * lane]) = make_float4(zp[0], zp[1], zp[2], zp[3]);
      }
      __syncwarp();      // value scales / zero-points visible

      // ================= online softmax: 16 tokens of head 4*g + tig per lane ================= //
      // e = 8*h8 + 4*hf + r  <->  cl[g][4*hf + r][2*h8 (hi), 2*h8 + 1 (lo)]  <->  token 64*hf + 32*h8 + 4*gid + r
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float lg[16];
        {
          const float u0 = k_unit * qmax_t[g];
          float mx = -INFINITY;
#pragma unroll
          for (int jj = 0; jj < 2; ++jj)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const float u = u0 * (1.0f / static_cast<float>(1 << (2 * r)));
#pragma unroll
              for (int h8 = 0; h8 < 2; ++h8) {
                const int d = cl[g][4 * jj + r][2 * h8] * 256 + cl[g][4 * jj + r][2 * h8 + 1];
                const float v = fmaf(static_cast<float>(d), u, bias[g]);
                lg[8 * h8 + 4 * jj + r] = v;
                mx = fmaxf(mx, v);
              }
            }
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          const float mnew = fmaxf(m_run[g], mx);
          const float alpha = (m_run[g] == -INFINITY) ? 0.f : ex2(m_run[g] - mnew);
          m_run[g] = mnew;
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            acc[g][m][0] *= alpha;
            acc[g][m][1] *= alpha;
          }
          zsum[g] *= alpha;
          lsum[g] *= alpha;
        }
        {
          // four consecutive tokens 64*hf + 32*h8 + 4*gid + {0..3} are one B word (k-step 2*hf + h8, word gid)
          uint32_t *dst = ws.pb[g] + (2 * tig) * PB_RS + gid;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf)
#pragma unroll
            for (int h8 = 0; h8 < 2; ++h8) {
              const int t0 = 64 * hf + 32 * h8 + 4 * gid;
              const float4 s4 = *reinterpret_cast<const float4 *>(&ws.sarr[t0]);
              const float4 z4 = *reinterpret_cast<const float4 *>(&ws.marr[t0]);
              const float sv[4] = {s4.x, s4.y, s4.z, s4.w}, zv[4] = {z4.x, z4.y, z4.z, z4.w};
              float y[4];
#pragma unroll
              for (int r = 0; r < 4; ++r) {
                const float p = ex2(lg[8 * h8 + 4 * hf + r] - m_run[g]);
                lsum[g] += p;
                zsum[g] = fmaf(p, zv[r], zsum[g]);
                y[r] = fmaf(p, sv[r], MAGIC_U);
              }
              // both limbs from one pair of PRMTs: (a.b0, b.b0, a.b1, b.b1)
              const uint32_t pab = __byte_perm(__float_as_uint(y[0]), __float_as_uint(y[1]), 0x5140);
              const uint32_t pcd = __byte_perm(__float_as_uint(y[2]), __float_as_uint(y[3]), 0x5140);
              dst[(2 * hf + h8) * 8] = __byte_perm(pab, pcd, 0x7632);               // high limbs
              dst[PB_RS + (2 * hf + h8) * 8] = __byte_perm(pab, pcd, 0x5410);       // low limbs
            }
        }
      }
      __syncwarp();

      // ================= P V ================= //
      // rows = channels; contraction bytes 4*tig + i <-> token 32*ks + 4*tig + i (b0), 32*ks + 16 + 4*tig + i (b1)
      int (&cv)[NG][8][4] = cl;      // the logit accumulators are dead: reuse their registers
#pragma unroll
      for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int m = 0; m < 8; ++m) cv[g][m][0] = cv[g][m][1] = cv[g][m][2] = cv[g][m][3] = 0;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t b0[NG], b1[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          b0[g] = ws.pb[g][gid * PB_RS + ks * 8 + tig];
          b1[g] = ws.pb[g][gid * PB_RS + ks * 8 + 4 + tig];
        }
        kstep32<false, NG>(stage_u32 + I8_OFF_VREC + (32 * ks + lane) * 32, b0, b1, cv);
      }
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        finish_tiles(cv[g]);
        const float u0 = v_unit;
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const float u = u0 * (1.0f / static_cast<float>(1 << (2 * r)));
            const int m = 4 * jj + r;
            acc[g][m][0] = fmaf(static_cast<float>(cv[g][m][0] * 256 + cv[g][m][1]), u, acc[g][m][0]);
            acc[g][m][1] = fmaf(static_cast<float>(cv[g][m][2] * 256 + cv[g][m][3]), u, acc[g][m][1]);
          }
      }
      __syncwarp();      // every lane is done with the value part and with the warp's buffers
      if (nxt < p1) {
        if (lane == 0) i8_issue_v(a, h, pv_nxt, stage_u32, bar_v);
        inflight |= 2u;
      }
    }

    if (dead) {
      if (lane == 0) atomicExch(a.status, 1);
      // give copies still in flight a bounded time to land before the stage is reused or the block exits: each
      // barrier is waited on with the parity of its own next phase
      if (inflight & 1u) mbar_wait(bar_k, kseq & 1u);
      if (inflight & 2u) mbar_wait(bar_v, vseq & 1u);
      inflight = 0;
    }
    // sum p*zero and sum p over all tokens of the warp's pages: add the 8 row groups
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        zsum[g] += __shfl_xor_sync(0xffffffffu, zsum[g], o);
        lsum[g] += __shfl_xor_sync(0xffffffffu, lsum[g], o);
      }
    __syncthreads();     // all warps have consumed every copy they issued: the first warps' buffers can be overlaid

    // ---- warp result -> merge buffer [warp][head][PART] ---- //
    constexpr int NH = 4 * NG;
    float *mb = reinterpret_cast<float *>(&sm.w[0].stage[0]);
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      float *w = mb + (warp * NH + 4 * g + tig) * PART;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          w[64 * jj + 4 * gid + r] = acc[g][4 * jj + r][0] + zsum[g];
          w[64 * jj + 32 + 4 * gid + r] = acc[g][4 * jj + r][1] + zsum[g];
        }
      if (gid == 0) {
        w[HD] = m_run[g];
        w[HD + 1] = lsum[g];
      }
    }
    __syncthreads();
    {
      float *dst = a.partials + ((static_cast<int64_t>(bh) * P.n_slots + (P.chunk_slot0 + c)) * G) * PART;
      for (int g = 0; g < G; ++g) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < I8_WARPS; ++w) M = fmaxf(M, mb[(w * NH + g) * PART + HD]);
        float A = 0.f, Ls = 0.f;
#pragma unroll
        for (int w = 0; w < I8_WARPS; ++w) {
          const float mw = mb[(w * NH + g) * PART + HD];
          const float wt = (mw == -INFINITY) ? 0.f : ex2(mw - M);
          A = fmaf(mb[(w * NH + g) * PART + tid], wt, A);
          Ls = fmaf(mb[(w * NH + g) * PART + HD + 1], wt, Ls);
        }
        dst[g * PART + tid] = A;
        if (tid == 0) {
          dst[g * PART + HD] = M;
          dst[g * PART + HD + 1] = Ls;
        }
      }
    }
  }
}

template <int NG>
static int launch_i8(const DecodeArgs &a, int n_items, int n_edge, int grid, cudaStream_t s, bool dependent) {
  static PerDeviceOnce once;      // opt-in to > 48 KB dynamic shared memory, once per device
  if (int rc = per_device_once(once, [] {
        const int smem = static_cast<int>(sizeof(I8Smem<NG>));
        return (cudaFuncSetAttribute(decode_paged_i8_kernel<NG, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                cudaFuncSetAttribute(decode_paged_i8_kernel<NG, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess)
                   ? KITTY_OK : KITTY_E_CUDA;
      }))
    return rc;
  const size_t sh = sizeof(I8Smem<NG>);
  if (dependent) {
    const cudaError_t e = (a.dyn != nullptr)
        ? launch_after(decode_paged_i8_kernel<NG, true>, dim3(grid), dim3(I8_WARPS * 32), sh, s, a, n_items, n_edge)
        : launch_after(decode_paged_i8_kernel<NG, false>, dim3(grid), dim3(I8_WARPS * 32), sh, s, a, n_items, n_edge);
    return (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? KITTY_OK : KITTY_E_CUDA;
  }
  if (a.dyn != nullptr)
    decode_paged_i8_kernel<NG, true><<<grid, I8_WARPS * 32, sh, s>>>(a, n_items, n_edge);
  else
    decode_paged_i8_kernel<NG, false><<<grid, I8_WARPS * 32, sh, s>>>(a, n_items, n_edge);
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}

// Groups of up to 4 query heads per KV head run with one operand group (4 blocks per multiprocessor), groups of 5..8
// with two (3 blocks).
int launch_decode_paged_i8(const DecodeArgs &a, int n_items, int n_edge, int grid, cudaStream_t s, bool dependent) {
  return a.P.G <= 4 ? launch_i8<1>(a, n_items, n_edge, grid, s, dependent) : launch_i8<2>(a, n_items, n_edge, grid, s, dependent);
}

int i8_blocks_per_sm(int G) { return G <= 4 ? 4 : 3; }

}  // namespace kitty
