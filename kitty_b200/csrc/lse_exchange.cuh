// Exchange of per-row partials over peer memory and the merge that follows (device code shared by the
// stand-alone combine kernel and the merge kernel of a sequence-split attention call).
//
// Buffer of one rank (symmetric: same layout on every rank, `peers[r]` = base address of rank r's copy):
//   float  data [2][world][rows][PART]     partial of (parity, source rank, row)
//   int32  flag [2][world][rows]           sequence number of the call that wrote the partial
// `seq` grows by one per call (first call: 1; the buffer starts zeroed).  Two parities: a rank that is one
// call ahead writes the other half, and it cannot be two calls ahead because finishing a call needs every
// rank's flag of that call.  A block only waits for the block of the same row on the other GPUs, never for a
// block of its own GPU; the row count is capped so that every block of a launch is resident at once and no
// waiting block can keep a needed one from starting.  No multicast, no TMA: ordinary stores, a system-scope
// fence, volatile loads.  Every wait is bounded by time (XchgDesc::wait_ns) and reports through a status word.
#pragma once

#include "decode.cuh"

namespace kitty {


__device__ __forceinline__ unsigned long long xchg_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Called by the 128 threads (c = 0..127, one per channel) that hold row r's un-normalised partial: v = acc[c],
// m / l = running max / sum (same value in every thread).  Publishes it on every rank, waits for the other
// ranks' partials of the row and returns the merged numerator (per channel) and denominator.  The 128 threads
// synchronise on named barrier 1, so other threads of the block may have exited.  False: a wait ran out.
__device__ __forceinline__ bool xchg_row(const XchgDesc &x, int rows, int r, int c, float v, float m, float l,
                                         float &A_out, float &L_out) {
  __shared__ float xw_s[128];
  __shared__ int xok_s;
  const int par = x.seq & 1;
  const int64_t slot_me = (static_cast<int64_t>(par) * x.world + x.rank) * rows + r;
  for (int dst = 0; dst < x.world; ++dst) {
    float *p = x.peers[dst] + slot_me * PART;
    p[c] = v;
    if (c == 0) {
      p[HD] = m;
      p[HD + 1] = l;
    }
  }
  __threadfence_system();
  if (c == 0) xok_s = 1;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (c < x.world) {
    volatile int32_t *f = reinterpret_cast<volatile int32_t *>(reinterpret_cast<uint8_t *>(x.peers[c]) + x.flag_offset);
    f[slot_me] = x.seq;
    const volatile int32_t *mine =
        reinterpret_cast<const volatile int32_t *>(reinterpret_cast<const uint8_t *>(x.peers[x.rank]) + x.flag_offset);
    const int64_t slot = (static_cast<int64_t>(par) * x.world + c) * rows + r;
    const unsigned long long t0 = xchg_ns();
    while (mine[slot] != x.seq) {
      if (xchg_ns() - t0 > x.wait_ns) {
        xok_s = 0;
        if (x.status != nullptr) atomicExch(x.status, 1);
        break;
      }
    }
  }
  __threadfence_system();
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (!xok_s) return false;
  // merge the world partials of row r (read past L1: they were written by other GPUs)
  const float *buf = x.peers[x.rank] + (static_cast<int64_t>(par) * x.world * rows + r) * PART;
  const int64_t stride = static_cast<int64_t>(rows) * PART;
  float M = -INFINITY;
  for (int s = 0; s < x.world; ++s) M = fmaxf(M, __ldcg(buf + s * stride + HD));
  if (c < x.world) {
    const float ms = __ldcg(buf + c * stride + HD);
    xw_s[c] = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  float A = 0.f, L = 0.f;
  for (int s = 0; s < x.world; ++s) {
    const float w = xw_s[s];
    A = fmaf(__ldcg(buf + s * stride + c), w, A);
    L = fmaf(__ldcg(buf + s * stride + HD + 1), w, L);
  }
  A_out = A;
  L_out = L;
  return true;
}

__device__ __forceinline__ void store_out(void *out, int out_dtype, int64_t i, float v) {
  if (out_dtype == KITTY_F16) static_cast<__half *>(out)[i] = __float2half_rn(v);
  else if (out_dtype == KITTY_BF16) static_cast<__nv_bfloat16 *>(out)[i] = __float2bfloat16_rn(v);
  else static_cast<float *>(out)[i] = v;
}

}  // namespace kitty
