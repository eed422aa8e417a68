// Building blocks shared by the streaming decode kernels and the edge reduction:
// PTX wrappers (mbarrier, bulk async copy, mma.sync), the 2-bit-field-as-fp16-
// subnormal operand trick and the Q K^T product of one packed key page.
#pragma once

#include "decode.cuh"

namespace kitty {

constexpr int QS_ROW = HD + 8;   // halves per row of a staged query (row stride 272 B keeps rows 16-byte aligned)
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s: far beyond any healthy copy

// ---- PTX wrappers --------------------------------------------------------- //
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false when the phase did not complete within WAIT_LIMIT_NS.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
  return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 r = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&r);
}

// Field f (0..7) of both 16-bit halves of x as an fp16x2 operand: fp16
// subnormals worth code * 4^pos * 2^-24.  Fields 5..7 sit in the exponent bits,
// so they are taken from the copy shifted right by 10 (xs), where they are
// fields 0..2.  field_unscale(f) is the power of two that undoes the weight.
__device__ __forceinline__ uint32_t field(uint32_t x, uint32_t xs, int f) {
  return (f < 5) ? (x & (0x00030003u << (2 * f))) : (xs & (0x00030003u << (2 * (f - 5))));
}
__host__ __device__ constexpr float field_unscale(int f) {
  return 16777216.0f / static_cast<float>(1 << (2 * (f < 5 ? f : f - 5)));
}

// Query fragments of one lane: B-operand column n = gid (query head), contraction
// index k = 2*tig, 2*tig+1, 2*tig+8, 2*tig+9  <->  channels 16*ks + tig + {0, 4, 8, 12}.
// qs: staged query rows [8][QS_ROW] (fp16, already multiplied by scaling*log2 e).
__device__ __forceinline__ void load_q_frags(const __half (*qs)[QS_ROW], int gid, int tig, uint32_t (&q2)[8][2]) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const __half *qr = &qs[gid][16 * ks + tig];
    __half2 x = __halves2half2(qr[0], qr[4]);
    __half2 y = __halves2half2(qr[8], qr[12]);
    q2[ks][0] = *reinterpret_cast<uint32_t *>(&x);
    q2[ks][1] = *reinterpret_cast<uint32_t *>(&y);
  }
}

// Logits (base-2 domain) of the 128 tokens of one packed key page against the 8
// staged query heads, by one warp.
//   krec : the head's key record in shared memory (low plane | high plane | index bytes)
//   km   : its metadata as words (scale | min << 16), one per channel
//   inv  : 32-byte scratch of the warp (slot -> channel table)
// Result: cl[m][0..1] = token 16*gid + m, heads 2*tig, 2*tig+1; cl[m][2..3] = token 16*gid + 8 + m.
__device__ __forceinline__ void qk_packed_page(const uint8_t *krec, const uint32_t *km, const __half (*qs)[QS_ROW],
                                               const uint32_t (&q2)[8][2], uint8_t *inv, int lane, float (&cl)[8][4]) {
  const int gid = lane >> 2, tig = lane & 3;
  const uint32_t *kw = reinterpret_cast<const uint32_t *>(krec);
  const uint32_t *hw = reinterpret_cast<const uint32_t *>(krec + K_OFF_HI);
  {
    const uint32_t w = *reinterpret_cast<const uint32_t *>(krec + K_OFF_IDX + 4 * lane);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t s = (w >> (8 * i)) & 0xffu;
      if (s < DB) inv[s] = static_cast<uint8_t>(4 * lane + i);
    }
  }
  float cb[4] = {0.f, 0.f, 0.f, 0.f};   // sum_d q*min, identical in every row
#pragma unroll
  for (int m = 0; m < 8; ++m) cl[m][0] = cl[m][1] = cl[m][2] = cl[m][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int ch = 16 * ks + tig;
    const uint32_t m0 = km[ch], m1 = km[ch + 4], m2 = km[ch + 8], m3 = km[ch + 12];
    const uint32_t b0 = hmul2_u(q2[ks][0], __byte_perm(m0, m1, 0x5410));
    const uint32_t b1 = hmul2_u(q2[ks][1], __byte_perm(m2, m3, 0x5410));
    const uint32_t mnA = __byte_perm(m0, m1, 0x7632), mnB = __byte_perm(m2, m3, 0x7632);
    mma16816(cb, mnA, mnA, mnB, mnB, q2[ks][0], q2[ks][1]);
    const uint32_t w0 = kw[ch * 8 + gid], w1 = kw[(ch + 4) * 8 + gid], w2 = kw[(ch + 8) * 8 + gid],
                   w3 = kw[(ch + 12) * 8 + gid];
    const uint32_t xab = __byte_perm(w0, w1, 0x5410), yab = __byte_perm(w0, w1, 0x7632);
    const uint32_t xcd = __byte_perm(w2, w3, 0x5410), ycd = __byte_perm(w2, w3, 0x7632);
    const uint32_t xabs = xab >> 10, yabs = yab >> 10, xcds = xcd >> 10, ycds = ycd >> 10;
#pragma unroll
    for (int m = 0; m < 8; ++m)
      mma16816(cl[m], field(xab, xabs, m), field(yab, yabs, m), field(xcd, xcds, m), field(ycd, ycds, m), b0, b1);
  }
  __syncwarp();      // slot table complete
  // high plane: contraction over slots 16*hs + tig + {0,4,8,12}; operand = 4 * q * scale of the slot's channel
#pragma unroll
  for (int hs = 0; hs < 2; ++hs) {
    const int sl = 16 * hs + tig;
    uint32_t bq[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int ca = inv[sl + 8 * j], cc = inv[sl + 8 * j + 4];
      const __half2 qq = __halves2half2(qs[gid][ca], qs[gid][cc]);
      const __half2 ss = __halves2half2(__ushort_as_half(static_cast<unsigned short>(km[ca] & 0xffffu)),
                                        __ushort_as_half(static_cast<unsigned short>(km[cc] & 0xffffu)));
      const __half2 r = __hmul2(__hmul2(qq, ss), __float2half2_rn(4.0f));
      bq[j] = *reinterpret_cast<const uint32_t *>(&r);
    }
    const uint32_t w0 = hw[sl * 8 + gid], w1 = hw[(sl + 4) * 8 + gid], w2 = hw[(sl + 8) * 8 + gid],
                   w3 = hw[(sl + 12) * 8 + gid];
    const uint32_t xab = __byte_perm(w0, w1, 0x5410), yab = __byte_perm(w0, w1, 0x7632);
    const uint32_t xcd = __byte_perm(w2, w3, 0x5410), ycd = __byte_perm(w2, w3, 0x7632);
    const uint32_t xabs = xab >> 10, yabs = yab >> 10, xcds = xcd >> 10, ycds = ycd >> 10;
#pragma unroll
    for (int m = 0; m < 8; ++m)
      mma16816(cl[m], field(xab, xabs, m), field(yab, yabs, m), field(xcd, xcds, m), field(ycd, ycds, m), bq[0], bq[1]);
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const float u = field_unscale(m);
    cl[m][0] = fmaf(cl[m][0], u, cb[0]);
    cl[m][1] = fmaf(cl[m][1], u, cb[1]);
    cl[m][2] = fmaf(cl[m][2], u, cb[2]);
    cl[m][3] = fmaf(cl[m][3], u, cb[3]);
  }
}

}  // namespace kitty
