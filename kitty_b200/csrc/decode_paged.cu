// Streaming decode attention over the common packed pages (key page i and
// value page i of one (batch, kv-head)), the hot loop of the decode step.
//
// Data path.  A block holds four warp pairs.  In a pair, the QK warp streams key
// records (5248 B + 512 B metadata) and the PV warp streams value records
// (4096 B + 512 B) through private two-slot shared-memory rings, each slot filled
// by bulk async copies (cp.async.bulk, completion counted on an mbarrier).  The
// 10368 algorithmic bytes of a page pair are fetched from HBM exactly once.
// The QK warp hands the page's probabilities (fp16) and the running-max
// correction to the PV warp through a two-slot buffer guarded by a full/empty
// mbarrier pair, so Q K^T of page i+1 overlaps P V of page i.
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
// Every wait on an mbarrier is bounded; when one runs out the warp sets the
// workspace's status word, stops consuming and the call's result is invalid.
#include "paged_core.cuh"

namespace kitty {

constexpr int PG_PAIRS = 4;
constexpr int PG_THREADS = PG_PAIRS * 64;
constexpr int RING = 2;
constexpr int KSLOT = K_HEAD + META_HEAD;           // 5760
constexpr int VSLOT = V_HEAD + META_HEAD;           // 4608
constexpr int PB_ROW = 68;                          // words per query-head row of the probability buffer (64 + pad)
constexpr int PB_WORDS = 8 * PB_ROW;
constexpr int PB_ALPHA = PB_WORDS;                  // 8 floats: factor that brings the previous pages to the new maximum
constexpr int PB_FLAG = PB_WORDS + 8;               // non-zero when any factor differs from 1
constexpr int PB_SLOT = PB_WORDS + 16;

struct PairSmem {
  __align__(128) uint8_t kst[RING][KSLOT];
  __align__(128) uint8_t vst[RING][VSLOT];
  __align__(16) uint32_t pb[RING][PB_SLOT];
  __align__(8) unsigned long long kbar[RING], vbar[RING], pfull[RING], pempty[RING];
  float mrun[8];             // QK warp's final running maxima of the item
  uint8_t inv[DB];
};

struct PagedSmem {
  PairSmem pair[PG_PAIRS];
  __align__(16) __half qs[8][QS_ROW];
};
static_assert(8 * PART * 4 <= RING * VSLOT, "a pair's result overlays its own value ring");

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void issue_k(const DecodeArgs &a, int b, int h, int page, uint32_t dst, uint32_t bar) {
  const int H = a.P.H;
  const int64_t pk = a.L.PageTable_K[static_cast<int64_t>(b) * a.L.max_page + page];
  mbar_expect_tx(bar, KSLOT);
  bulk_g2s(dst, a.L.KeyCache + pk * (static_cast<int64_t>(H) * K_HEAD) + static_cast<int64_t>(h) * K_HEAD, K_HEAD, bar);
  bulk_g2s(dst + K_HEAD, static_cast<const uint8_t *>(a.L.KeyCache_metadata) + (pk * H + h) * META_HEAD, META_HEAD, bar);
}
__device__ __forceinline__ void issue_v(const DecodeArgs &a, int b, int h, int page, uint32_t dst, uint32_t bar) {
  const int H = a.P.H;
  const int64_t pv = a.L.PageTable_V[static_cast<int64_t>(b) * a.L.max_page + page];
  mbar_expect_tx(bar, VSLOT);
  bulk_g2s(dst, a.L.ValueCache + pv * (static_cast<int64_t>(H) * V_HEAD) + static_cast<int64_t>(h) * V_HEAD, V_HEAD, bar);
  bulk_g2s(dst + V_HEAD, static_cast<const uint8_t *>(a.L.ValueCache_metadata) + (pv * H + h) * META_HEAD, META_HEAD, bar);
}

__global__ void __launch_bounds__(PG_THREADS, 2) decode_paged_kernel(DecodeArgs a, int n_items, int n_gt) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  PagedSmem &sm = *reinterpret_cast<PagedSmem *>(smem_raw);
  const DecodePlan &P = a.P;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pair = warp >> 1;
  const bool is_qk = (warp & 1) == 0;
  const int gid = lane >> 2, tig = lane & 3;
  const int H = P.H, G = P.G;
  PairSmem &ps = sm.pair[pair];

  if (is_qk && lane == 0) {
#pragma unroll
    for (int s = 0; s < RING; ++s) {
      mbar_init(smem_u32(&ps.kbar[s]), 1);
      mbar_init(smem_u32(&ps.vbar[s]), 1);
      mbar_init(smem_u32(&ps.pfull[s]), 1);
      mbar_init(smem_u32(&ps.pempty[s]), 1);
    }
  }
  if (is_qk) ps.inv[lane] = 0;
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();

  uint32_t seq = 0;          // pages consumed by this pair so far: ring slot = seq % RING, use = seq / RING
  bool dead = false;         // a bounded wait ran out: stop consuming, keep the block barriers uniform
  uint32_t inflight = 0;     // bit s: ring slot s of this warp has a copy in flight (warp-uniform)

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int c = item % P.nchunk;
    const int gt = (item / P.nchunk) % n_gt;
    const int bh = item / (P.nchunk * n_gt);
    const int h = bh % H, b = bh / H;
    const int p0 = P.pb + c * P.ch;
    const int p1 = min(P.pe, p0 + P.ch);
    const int g_valid = min(8, G - gt * 8);

    __syncthreads();   // the previous item's pair results (overlaying the value rings) and query are no longer read
    for (int i = tid; i < 8 * HD; i += PG_THREADS) {
      const int g = i >> 7, d = i & (HD - 1);
      float v = 0.f;
      if (g < g_valid) v = load_q(a.q, a.q_dtype, (static_cast<int64_t>(b) * P.h_q + h * G + gt * 8 + g) * HD + d) * a.scale_log2;
      sm.qs[g][d] = __float2half_rn(v);
    }
    // first copies of this pair: pages p0 + pair, p0 + pair + PG_PAIRS, ...
    const int first = p0 + pair;
    if (!dead) {
      if (lane == 0) {
        // the value rings were last written through the generic proxy (pair results): order that before the bulk copies
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#pragma unroll
        for (int s = 0; s < RING; ++s) {
          const int pg = first + s * PG_PAIRS;
          if (pg < p1) {
            const uint32_t st = (seq + s) % RING;
            if (is_qk) issue_k(a, b, h, pg, smem_u32(&ps.kst[st][0]), smem_u32(&ps.kbar[st]));
            else issue_v(a, b, h, pg, smem_u32(&ps.vst[st][0]), smem_u32(&ps.vbar[st]));
          }
        }
      }
#pragma unroll
      for (int s = 0; s < RING; ++s)
        if (first + s * PG_PAIRS < p1) inflight |= 1u << ((seq + s) % RING);
    }
    __syncthreads();   // staged query visible

    if (is_qk) {
      // =========================== QK warp =========================== //
      float m_run0 = -INFINITY, m_run1 = -INFINITY;    // running maxima of heads 2*tig, 2*tig+1
      uint32_t q2[8][2];
      load_q_frags(sm.qs, gid, tig, q2);
      for (int pg = first; pg < p1 && !dead; pg += PG_PAIRS) {
        const uint32_t st = seq % RING, use = seq / RING;
        const uint32_t kbar = smem_u32(&ps.kbar[st]);
        if (!mbar_wait(kbar, use & 1u)) { dead = true; break; }
        inflight &= ~(1u << st);
        const uint8_t *stg = ps.kst[st];
        float cl[8][4];    // logits[token 16*gid + m (+8)][head 2*tig (+1)]
        qk_packed_page(stg, reinterpret_cast<const uint32_t *>(stg + K_HEAD), sm.qs, q2, ps.inv, lane, cl);
        __syncwarp();      // every lane is done with the key slot
        const int nxt = pg + RING * PG_PAIRS;
        if (nxt < p1) {
          if (lane == 0) issue_k(a, b, h, nxt, smem_u32(&ps.kst[st][0]), kbar);
          inflight |= 1u << st;
        }

        // ---- online softmax ---- //
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
        const bool changed = __any_sync(0xffffffffu, (mn0 > m_run0) || (mn1 > m_run1));
        const float a0 = (m_run0 == -INFINITY) ? 0.f : ex2(m_run0 - mn0);
        const float a1 = (m_run1 == -INFINITY) ? 0.f : ex2(m_run1 - mn1);
        m_run0 = mn0;
        m_run1 = mn1;
        uint32_t pw[2][8];   // fp16 pairs (token 16*gid + m, token 16*gid + 8 + m)
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const int pos = (m & 3) * 2 + (m >> 2);
          pw[0][pos] = pack_h2(ex2(cl[m][0] - m_run0), ex2(cl[m][2] - m_run0));
          pw[1][pos] = pack_h2(ex2(cl[m][1] - m_run1), ex2(cl[m][3] - m_run1));
        }
        // ---- hand over to the PV warp ---- //
        if (!mbar_wait(smem_u32(&ps.pempty[st]), (use & 1u) ^ 1u)) { dead = true; break; }
        uint32_t *pb = ps.pb[st];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint4 *dst = reinterpret_cast<uint4 *>(pb + (2 * tig + j) * PB_ROW + gid * 8);
          dst[0] = make_uint4(pw[j][0], pw[j][1], pw[j][2], pw[j][3]);
          dst[1] = make_uint4(pw[j][4], pw[j][5], pw[j][6], pw[j][7]);
        }
        if (gid == 0) {
          reinterpret_cast<float *>(pb)[PB_ALPHA + 2 * tig] = a0;
          reinterpret_cast<float *>(pb)[PB_ALPHA + 2 * tig + 1] = a1;
        }
        if (lane == 0) pb[PB_FLAG] = changed ? 1u : 0u;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ps.pfull[st]));
        ++seq;
      }
      if (gid == 0) {
        ps.mrun[2 * tig] = m_run0;
        ps.mrun[2 * tig + 1] = m_run1;
      }
    } else {
      // =========================== PV warp =========================== //
      float acc[8][4];       // out[channel 16*gid + m (+8)][head 2*tig (+1)], still carrying the field weight
      float cz[4] = {0.f, 0.f, 0.f, 0.f};   // [0,1] sum p*zero-point, [2,3] sum p, heads 2*tig, 2*tig+1
#pragma unroll
      for (int m = 0; m < 8; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
      const uint32_t ones = 0x3c003c00u;
      for (int pg = first; pg < p1 && !dead; pg += PG_PAIRS) {
        const uint32_t st = seq % RING, use = seq / RING;
        const uint32_t vbar = smem_u32(&ps.vbar[st]);
        if (!mbar_wait(vbar, use & 1u)) { dead = true; break; }
        inflight &= ~(1u << st);
        if (!mbar_wait(smem_u32(&ps.pfull[st]), use & 1u)) { dead = true; break; }
        const uint8_t *stg = ps.vst[st];
        const uint32_t *vw = reinterpret_cast<const uint32_t *>(stg);
        const uint32_t *vm = reinterpret_cast<const uint32_t *>(stg + V_HEAD);
        const uint32_t *pb = ps.pb[st];
        if (pb[PB_FLAG]) {
          const float a0 = reinterpret_cast<const float *>(pb)[PB_ALPHA + 2 * tig];
          const float a1 = reinterpret_cast<const float *>(pb)[PB_ALPHA + 2 * tig + 1];
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            acc[m][0] *= a0; acc[m][1] *= a1; acc[m][2] *= a0; acc[m][3] *= a1;
          }
          cz[0] *= a0; cz[1] *= a1; cz[2] *= a0; cz[3] *= a1;
        }
        // contraction index k = 2*tig, 2*tig+1, 2*tig+8, 2*tig+9  <->  tokens 16*ks + tig + {0, 8, 4, 12}
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint2 pp = *reinterpret_cast<const uint2 *>(pb + gid * PB_ROW + ks * 8 + 2 * tig);
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
        __syncwarp();      // every lane is done with the value slot and the probability slot
        if (lane == 0) mbar_arrive(smem_u32(&ps.pempty[st]));
        const int nxt = pg + RING * PG_PAIRS;
        if (nxt < p1) {
          if (lane == 0) issue_v(a, b, h, nxt, smem_u32(&ps.vst[st][0]), vbar);
          inflight |= 1u << st;
        }
        ++seq;
      }
      // pair result [head][PART] into the pair's own value ring: every copy this warp issued has been consumed
      if (!dead) {
        float *w = reinterpret_cast<float *>(&ps.vst[0][0]);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const float u = field_unscale(m);
          w[(2 * tig) * PART + 16 * gid + m] = fmaf(acc[m][0], u, cz[0]);
          w[(2 * tig + 1) * PART + 16 * gid + m] = fmaf(acc[m][1], u, cz[1]);
          w[(2 * tig) * PART + 16 * gid + 8 + m] = fmaf(acc[m][2], u, cz[0]);
          w[(2 * tig + 1) * PART + 16 * gid + 8 + m] = fmaf(acc[m][3], u, cz[1]);
        }
        if (gid == 0) {
          w[(2 * tig) * PART + HD + 1] = cz[2];
          w[(2 * tig + 1) * PART + HD + 1] = cz[3];
        }
      }
    }

    if (dead) {
      if (lane == 0) atomicExch(a.status, 1);
      // give copies still in flight a bounded time to land before the rings are reused or the block exits
      for (int s = 0; s < RING; ++s)
        if (inflight & (1u << s)) {
          const uint32_t nseq = seq + ((s + RING - seq % RING) % RING);
          mbar_wait(smem_u32(is_qk ? &ps.kbar[s] : &ps.vbar[s]), (nseq / RING) & 1u);
          inflight &= ~(1u << s);
        }
    }
    __syncthreads();     // pair results are in place
    {
      float *dst = a.partials + ((static_cast<int64_t>(bh) * P.n_slots + (P.chunk_slot0 + c)) * G + gt * 8) * PART;
      const int ch = tid & (HD - 1);
      for (int g = tid >> 7; g < g_valid; g += PG_THREADS / HD) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < PG_PAIRS; ++w) M = fmaxf(M, sm.pair[w].mrun[g]);
        float A = 0.f, Ls = 0.f;
#pragma unroll
        for (int w = 0; w < PG_PAIRS; ++w) {
          const float *mb = reinterpret_cast<const float *>(&sm.pair[w].vst[0][0]);
          const float mw = sm.pair[w].mrun[g];
          const float wt = (mw == -INFINITY) ? 0.f : ex2(mw - M);
          A = fmaf(mb[g * PART + ch], wt, A);
          Ls = fmaf(mb[g * PART + HD + 1], wt, Ls);
        }
        dst[g * PART + ch] = A;
        if (ch == 0) {
          dst[g * PART + HD] = M;
          dst[g * PART + HD + 1] = Ls;
        }
      }
    }
  }
}

int launch_decode_paged(const DecodeArgs &a, int n_items, int n_gt, int grid, cudaStream_t s) {
  static int configured = -1;     // per-process opt-in to > 48 KB dynamic shared memory, done once per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return KITTY_E_CUDA;
  if (configured != dev) {
    if (cudaFuncSetAttribute(decode_paged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(PagedSmem))) != cudaSuccess)
      return KITTY_E_CUDA;
    configured = dev;
  }
  decode_paged_kernel<<<grid, PG_THREADS, sizeof(PagedSmem), s>>>(a, n_items, n_gt);
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}

}  // namespace kitty
