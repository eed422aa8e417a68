// Plain (CUDA-core) decode-attention kernel and the slot merge kernel.
//
// The plain kernel reduces any run of tiles — sink, packed pages, Q-buffers,
// the rotated value ring — with one thread per token (logits) and one thread
// per channel (output).  It is slow and simple on purpose: with impl=1 it
// computes a whole call and serves as an in-library cross-check of the streaming
// and the edge reduction.
//
// Dequantisation is `code * scale + min` evaluated in fp32 from the fp16
// metadata (kernels/kitty_attention.py:162-165, 317-320 of the reference do it in
// fp16; the difference is inside the stated attention tolerance).
#include <algorithm>

#include "lse_exchange.cuh"

namespace kitty {

struct PlainSmem {
  float q[MAX_GROUP][HD];          // query * scaling * log2(e)
  float sl[PAGE][MAX_GROUP + 1];   // logits, then probabilities
  __align__(16) uint8_t krec[K_HEAD];
  __align__(16) __half2 kmeta[HD];
  __align__(16) uint8_t vrec[V_HEAD];
  __align__(16) __half2 vmeta[PAGE];
  float m_run[MAX_GROUP], l_run[MAX_GROUP], alpha[MAX_GROUP];
};

__global__ void __launch_bounds__(128) decode_plain_kernel(DecodeArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  PlainSmem &sm = *reinterpret_cast<PlainSmem *>(smem_raw);
  const DecodePlan &P = a.P;
  const int tid = threadIdx.x;
  const int h = blockIdx.y, b = blockIdx.z, H = P.H, G = P.G;
  const kitty_counts C = row_counts(a, a.C, b);
  const int64_t bh = static_cast<int64_t>(b) * H + h;

  // ---- which tiles, which slot ---- //
  int u0, u1, slot;
  {
    int j = blockIdx.x;
    if (P.has_sink && j == 0) {
      u0 = 0; u1 = 1; slot = 0;
    } else {
      j -= P.has_sink;
      if (!P.fast_chunks && j < P.nchunk) {
        const int p0 = P.pb + j * P.ch;
        const int p1 = max(p0, min(min(P.pe, C.PageCount_V), p0 + P.ch));
        u0 = 1 + p0; u1 = 1 + p1; slot = P.has_sink + j;
      } else {
        // the tail of this row: its own number of tiles (P.n_tiles is the largest over the rows)
        u0 = C.PageCount_V + 1;
        u1 = 1 + (C.PageCount_K * PAGE + C.Q_Buffer_Count_K + PAGE - 1) / PAGE;
        slot = P.has_sink + P.nchunk;
      }
    }
  }
  const int t_pos = C.PageCount_K * PAGE + C.Q_Buffer_Count_K;   // tokens after the sink

  for (int i = tid; i < G * HD; i += 128) {
    const int g = i / HD, d = i % HD;
    sm.q[g][d] = load_q(a.q, a.q_dtype, (static_cast<int64_t>(b) * P.h_q + h * G + g) * HD + d) * a.scale_log2;
  }
  if (tid < MAX_GROUP) {
    sm.m_run[tid] = -INFINITY;
    sm.l_run[tid] = 0.f;
  }
  float out[MAX_GROUP];
#pragma unroll
  for (int g = 0; g < MAX_GROUP; ++g) out[g] = 0.f;
  __syncthreads();

  for (int u = u0; u < u1; ++u) {
    const int n = (u == 0) ? C.Sink_Count : min(PAGE, t_pos - (u - 1) * PAGE);
    if (n <= 0) continue;
    const bool k_packed = (u >= 1) && (u - 1 < C.PageCount_K);
    const bool v_packed = (u >= 1) && (u - 1 < C.PageCount_V);
    if (k_packed) {
      const int64_t pid = a.L.PageTable_K[static_cast<int64_t>(b) * a.L.max_page + (u - 1)];
      const uint4 *src = reinterpret_cast<const uint4 *>(a.L.KeyCache + pid * (static_cast<int64_t>(H) * K_HEAD) + h * K_HEAD);
      for (int i = tid; i < K_HEAD / 16; i += 128) reinterpret_cast<uint4 *>(sm.krec)[i] = src[i];
      const uint4 *ms = reinterpret_cast<const uint4 *>(static_cast<const __half2 *>(a.L.KeyCache_metadata) + (pid * H + h) * HD);
      if (tid < META_HEAD / 16) reinterpret_cast<uint4 *>(sm.kmeta)[tid] = ms[tid];
    }
    if (v_packed) {
      const int64_t pid = a.L.PageTable_V[static_cast<int64_t>(b) * a.L.max_page + (u - 1)];
      const uint4 *src = reinterpret_cast<const uint4 *>(a.L.ValueCache + pid * (static_cast<int64_t>(H) * V_HEAD) + h * V_HEAD);
      for (int i = tid; i < V_HEAD / 16; i += 128) reinterpret_cast<uint4 *>(sm.vrec)[i] = src[i];
      const uint4 *ms = reinterpret_cast<const uint4 *>(static_cast<const __half2 *>(a.L.ValueCache_metadata) + (pid * H + h) * PAGE);
      if (tid < META_HEAD / 16) reinterpret_cast<uint4 *>(sm.vmeta)[tid] = ms[tid];
    }
    __syncthreads();

    // ---- logits: thread = token ---- //
    if (tid < n) {
      float acc[MAX_GROUP];
#pragma unroll
      for (int g = 0; g < MAX_GROUP; ++g) acc[g] = 0.f;
      if (k_packed) {
        const int col = tid >> 2, sh = (tid & 3) * 2;
        for (int d = 0; d < HD; ++d) {
          uint32_t code = (sm.krec[d * K_ROW + col] >> sh) & 3u;
          const uint32_t s = sm.krec[K_OFF_IDX + d];
          if (s < DB) code |= ((sm.krec[K_OFF_HI + s * K_ROW + col] >> sh) & 3u) << 2;
          const float2 mt = __half22float2(sm.kmeta[d]);
          const float kv = static_cast<float>(code) * mt.x + mt.y;
#pragma unroll
          for (int g = 0; g < MAX_GROUP; ++g)
            if (g < G) acc[g] = fmaf(sm.q[g][d], kv, acc[g]);
        }
      } else {
        const __half *row;
        if (u == 0) row = static_cast<const __half *>(a.L.Sink_Buffer_K) + (bh * SINK + tid) * HD;
        else row = static_cast<const __half *>(a.L.Q_Buffer_K) + (bh * PAGE + ((u - 1 - C.PageCount_K) * PAGE + tid)) * HD;
        for (int d8 = 0; d8 < HD / 8; ++d8) {
          float kv[8];
          Vec8<__half>::load(row + 8 * d8, kv);
#pragma unroll
          for (int g = 0; g < MAX_GROUP; ++g)
            if (g < G) {
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[g] = fmaf(sm.q[g][8 * d8 + e], kv[e], acc[g]);
            }
        }
      }
#pragma unroll
      for (int g = 0; g < MAX_GROUP; ++g)
        if (g < G) sm.sl[tid][g] = acc[g];
    }
    __syncthreads();
    // ---- running max ---- //
    if (tid < G) {
      float mx = -INFINITY;
      for (int t = 0; t < n; ++t) mx = fmaxf(mx, sm.sl[t][tid]);
      const float mo = sm.m_run[tid], mn = fmaxf(mo, mx);
      sm.alpha[tid] = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
      sm.m_run[tid] = mn;
    }
    __syncthreads();
    if (tid < n) {
#pragma unroll
      for (int g = 0; g < MAX_GROUP; ++g)
        if (g < G) sm.sl[tid][g] = exp2f(sm.sl[tid][g] - sm.m_run[g]);
    }
    __syncthreads();
    if (tid < G) {
      float s = 0.f;
      for (int t = 0; t < n; ++t) s += sm.sl[t][tid];
      sm.l_run[tid] = sm.l_run[tid] * sm.alpha[tid] + s;
    }
    // ---- output: thread = channel ---- //
#pragma unroll
    for (int g = 0; g < MAX_GROUP; ++g)
      if (g < G) out[g] *= sm.alpha[g];
    if (v_packed) {
      const int col = tid >> 2, sh = (tid & 3) * 2;
      for (int t = 0; t < n; ++t) {
        const uint32_t code = (sm.vrec[t * V_ROW + col] >> sh) & 3u;
        const float2 mt = __half22float2(sm.vmeta[t]);
        const float v = static_cast<float>(code) * mt.x + mt.y;
#pragma unroll
        for (int g = 0; g < MAX_GROUP; ++g)
          if (g < G) out[g] = fmaf(sm.sl[t][g], v, out[g]);
      }
    } else {
      for (int t = 0; t < n; ++t) {
        const __half *row;
        if (u == 0) {
          row = static_cast<const __half *>(a.L.Sink_Buffer_V) + (bh * SINK + t) * HD;
        } else {
          const int r = (u - 1 - C.PageCount_V) * PAGE + t;       // position after the packed value pages
          if (r < C.Q_Buffer_Count_V) row = static_cast<const __half *>(a.L.Q_Buffer_V) + (bh * PAGE + r) * HD;
          else row = static_cast<const __half *>(a.L.Local_Buffer_V) + (bh * PAGE + ((r - C.Q_Buffer_Count_V + C.Write_Offset_Local_V) & (PAGE - 1))) * HD;
        }
        const float v = __half2float(row[tid]);
#pragma unroll
        for (int g = 0; g < MAX_GROUP; ++g)
          if (g < G) out[g] = fmaf(sm.sl[t][g], v, out[g]);
      }
    }
    __syncthreads();
  }

  float *dst = a.partials + ((bh * P.n_slots + slot) * G) * PART;
#pragma unroll
  for (int g = 0; g < MAX_GROUP; ++g)
    if (g < G) dst[g * PART + tid] = out[g];
  if (tid < G) {
    dst[tid * PART + HD] = sm.m_run[tid];
    dst[tid * PART + HD + 1] = sm.l_run[tid];
  }
}

// MERGE_GROUPS slot groups per row: thread (group, channel).  Four groups when a call has few rows (then every
// row has many slots and the launch is latency-bound), one when it has many rows of few slots.
template <int MERGE_GROUPS>
__global__ void __launch_bounds__(128 * MERGE_GROUPS) merge_kernel(MergeArgs a) {
  // One block per row (batch, query head); thread = (slot group, channel).  The slot weights are computed
  // once, in parallel (thread s <-> slot s), then every thread folds its channel over the slots of its
  // group with eight loads in flight, and the groups are added in a fixed order.
  __shared__ float w_s[128];
  __shared__ float red[4];
  __shared__ float part[MERGE_GROUPS][HD];
  const int64_t r = blockIdx.x;
  const int c = threadIdx.x & (HD - 1), grp = threadIdx.x >> 7;
  const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) & 3;
  dep_wait();          // launched while the kernel that writes the partials may still be running
  dep_release();       // a flush launched behind this kernel may be scheduled; it waits for this grid to complete
  if (a.dyn != nullptr) {
    a.n = a.ns = a.dyn->n_slots;
    a.x.seq += a.dyn->xchg_seq;        // device-resident step: x.seq holds the layer's offset
  }
  const float *base = a.partials + ((r / a.gm) * a.ns * a.gm + r % a.gm) * PART;
  float M = -INFINITY, A = 0.f, Lsum = 0.f;
  for (int s0 = 0; s0 < a.n; s0 += 128) {           // chunks of 128 slots (one chunk in practice)
    const int nn = min(128, a.n - s0);
    // every group computes the same weights (the loads hit L2); group 0 publishes them
    const float ms = (c < nn) ? base[(s0 + c) * a.stride_part + HD] : -INFINITY;
    const float ls = (c < nn) ? base[(s0 + c) * a.stride_part + HD + 1] : 0.f;
    float mx = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __syncthreads();                                 // previous chunk's w_s / red are no longer read
    if (grp == 0 && lane == 0) red[warp] = mx;
    __syncthreads();
    const float Mn = fmaxf(M, fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])));
    const float rescale = (M == -INFINITY) ? 0.f : exp2f(M - Mn);
    M = Mn;
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    if (grp == 0) w_s[c] = w;
    float lp = ls * w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lp += __shfl_xor_sync(0xffffffffu, lp, o);
    __syncthreads();                                 // red (max) consumed, w_s visible
    if (grp == 0 && lane == 0) red[warp] = lp;
    __syncthreads();
    Lsum = Lsum * rescale + ((red[0] + red[1]) + (red[2] + red[3]));
    A *= rescale;
    const float *p = base + static_cast<int64_t>(s0) * a.stride_part + c;
    constexpr int U = 8;
    for (int s = grp * U; s < nn; s += U * MERGE_GROUPS) {      // slots s .. s+U-1 of this group
      float v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = (s + u < nn) ? p[static_cast<int64_t>(s + u) * a.stride_part] : 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u) A = fmaf(v[u], (s + u < nn) ? w_s[s + u] : 0.f, A);
    }
  }
  if (MERGE_GROUPS > 1) {
    part[grp][c] = A;
    __syncthreads();
  }
  if (a.work_counter != nullptr && r == 0 && threadIdx.x == 0) *a.work_counter = 0;   // ready for the next call's item hand-out
  if (grp != 0) return;
  if (MERGE_GROUPS == 4) A = (part[0][c] + part[1][c]) + (part[2][c] + part[3][c]);
  if (a.x.peers != nullptr) {
    // sequence split: this row's partial goes to every rank, theirs come here, and the result is complete
    float Ax, Lx;
    if (!xchg_row(a.x, static_cast<int>(a.rows), static_cast<int>(r), c, A, M, Lsum, Ax, Lx)) return;
    store_out(a.out, a.out_dtype, r * HD + c, Ax / Lx);
    return;
  }
  if (a.partial_out) {
    float *o = a.partial_out + r * PART;
    o[c] = A;
    if (c == 0) {
      o[HD] = M;
      o[HD + 1] = Lsum;
    }
    return;
  }
  store_out(a.out, a.out_dtype, r * HD + c, A / Lsum);
}

int launch_decode_plain(const DecodeArgs &a, int items_per_bh, cudaStream_t s) {
  dim3 grid(items_per_bh, a.P.H, a.P.B);
  decode_plain_kernel<<<grid, 128, sizeof(PlainSmem), s>>>(a);
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}

int launch_merge(const MergeArgs &m, cudaStream_t s) {
  if (m.rows == 0) return KITTY_OK;
  cudaError_t e;
  // With a peer exchange every block waits for the block of the same row on the other GPUs, so all blocks of the
  // launch have to be resident at once: 512-thread blocks fit four per multiprocessor, 128-thread blocks sixteen.
  const int64_t wide_max = m.x.peers != nullptr ? std::min<int64_t>(1024, 4LL * sm_count()) : 1024;
  if (m.x.peers != nullptr && m.rows > 16LL * sm_count()) return KITTY_E_BADARG;
  if (m.rows <= wide_max) e = launch_after(merge_kernel<4>, dim3(static_cast<unsigned>(m.rows)), dim3(512), 0, s, m);
  else e = launch_after(merge_kernel<1>, dim3(static_cast<unsigned>(m.rows)), dim3(128), 0, s, m);
  return (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? KITTY_OK : KITTY_E_CUDA;
}

}  // namespace kitty
