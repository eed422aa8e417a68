// Sequence-split combine over peer memory: every rank stores its (acc[128], max, sum) partial of each
// query head straight into the exchange buffer of every rank (plain peer stores over NVLink), raises a
// per-row flag there, waits — bounded — for the other ranks' flags of the same row in its own buffer and
// merges.  One kernel replaces an all-gather collective plus a merge kernel; the exchange is 520 bytes per
// query head per rank, so the cost is one NVLink round trip instead of a collective's launch protocol.
//
// Buffer of one rank (symmetric: same layout on every rank, `peers[r]` = base address of rank r's copy):
//   float  data [2][world][rows][PART]     partial of (parity, source rank, row)
//   int32  flag [2][world][rows]           sequence number of the call that wrote the partial
// `seq` grows by one per call (first call: 1; the buffer starts zeroed).  Two parities: a rank that is one
// call ahead writes the other half, and it cannot be two calls ahead because finishing a call needs every
// rank's flag of that call.  A block only waits for the block of the same row on the other GPUs, never for a
// block of its own GPU; the row count is capped so that every block of a launch is resident at once and no
// waiting block can keep a needed one from starting.  No multicast, no TMA: ordinary stores, a system-scope
// fence, volatile loads.  Every wait is bounded by time and reports through a status word.
#include "decode.cuh"

namespace kitty {

constexpr unsigned long long XCHG_WAIT_NS = 1000000000ull;   // 1 s: far beyond any healthy exchange

struct XchgArgs {
  const float *local;        // [rows][PART] this rank's partial
  float *const *peers;       // device array [world]: base address of every rank's exchange buffer
  int64_t flag_offset;       // byte offset of the flag area inside an exchange buffer
  int32_t rank, world, rows, seq;
  void *out;                 // [rows][128] of out_dtype
  int32_t out_dtype;
  int32_t *status;           // or null: set non-zero when a wait ran out
};

__device__ __forceinline__ unsigned long long xchg_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(128) lse_exchange_merge_kernel(XchgArgs a) {
  __shared__ float w_s[128];
  __shared__ int ok_s;
  const int r = blockIdx.x, c = threadIdx.x;
  const int par = a.seq & 1;
  const int64_t slot_me = (static_cast<int64_t>(par) * a.world + a.rank) * a.rows + r;

  // ---- 1. publish this rank's partial of row r on every rank ---- //
  const float v = a.local[static_cast<int64_t>(r) * PART + c];
  const float ml = (c < 2) ? a.local[static_cast<int64_t>(r) * PART + HD + c] : 0.f;
  for (int dst = 0; dst < a.world; ++dst) {
    float *p = a.peers[dst] + slot_me * PART;
    p[c] = v;
    if (c < 2) p[HD + c] = ml;
  }
  __threadfence_system();
  __syncthreads();
  if (c < a.world) {
    volatile int32_t *f = reinterpret_cast<volatile int32_t *>(reinterpret_cast<uint8_t *>(a.peers[c]) + a.flag_offset);
    f[slot_me] = a.seq;
  }

  // ---- 2. wait for every rank's partial of this row (thread s <-> source rank s) ---- //
  if (c == 0) ok_s = 1;
  __syncthreads();
  if (c < a.world) {
    const volatile int32_t *f =
        reinterpret_cast<const volatile int32_t *>(reinterpret_cast<const uint8_t *>(a.peers[a.rank]) + a.flag_offset);
    const int64_t slot = (static_cast<int64_t>(par) * a.world + c) * a.rows + r;
    const unsigned long long t0 = xchg_ns();
    bool ok = true;
    while (f[slot] != a.seq) {
      if (xchg_ns() - t0 > XCHG_WAIT_NS) {
        ok = false;
        break;
      }
    }
    if (!ok) {
      ok_s = 0;
      if (a.status != nullptr) atomicExch(a.status, 1);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (!ok_s) return;          // block-uniform: the output of this row stays unwritten, the status word says why

  // ---- 3. merge the world partials of row r (read past L1: they were written by other GPUs) ---- //
  const float *mine = a.peers[a.rank] + (static_cast<int64_t>(par) * a.world * a.rows + r) * PART;
  const int64_t stride = static_cast<int64_t>(a.rows) * PART;
  float M = -INFINITY;
  for (int s = 0; s < a.world; ++s) M = fmaxf(M, __ldcg(mine + s * stride + HD));
  if (c < a.world) {
    const float ms = __ldcg(mine + c * stride + HD);
    w_s[c] = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
  }
  __syncthreads();
  float A = 0.f, L = 0.f;
  for (int s = 0; s < a.world; ++s) {
    const float w = w_s[s];
    A = fmaf(__ldcg(mine + s * stride + c), w, A);
    L = fmaf(__ldcg(mine + s * stride + HD + 1), w, L);
  }
  const float o = A / L;
  const int64_t oi = static_cast<int64_t>(r) * HD + c;
  if (a.out_dtype == KITTY_F16) static_cast<__half *>(a.out)[oi] = __float2half_rn(o);
  else if (a.out_dtype == KITTY_BF16) static_cast<__nv_bfloat16 *>(a.out)[oi] = __float2bfloat16_rn(o);
  else static_cast<float *>(a.out)[oi] = o;
}

}  // namespace kitty

using namespace kitty;

extern "C" int64_t kitty_lse_exchange_bytes(int64_t rows, int32_t world, int64_t *flag_offset) {
  if (rows <= 0 || world <= 0 || world > 128) return KITTY_E_BADARG;
  const int64_t data = 2 * static_cast<int64_t>(world) * rows * PART * static_cast<int64_t>(sizeof(float));
  const int64_t flags = 2 * static_cast<int64_t>(world) * rows * static_cast<int64_t>(sizeof(int32_t));
  if (flag_offset != nullptr) *flag_offset = data;
  return data + flags;
}

extern "C" int kitty_lse_exchange_merge(const float *local_partial, int64_t rows, void *const *peer_buffers,
                                        int32_t rank, int32_t world, int32_t seq, void *out, int out_dtype,
                                        int32_t *status, void *stream) {
  if (!local_partial || !peer_buffers || !out) return KITTY_E_BADARG;
  if (rows <= 0 || rows > KITTY_EXCHANGE_MAX_ROWS || world <= 0 || world > 128 || rank < 0 || rank >= world || seq <= 0)
    return KITTY_E_BADARG;
  if (out_dtype < KITTY_F16 || out_dtype > KITTY_F32) return KITTY_E_BADARG;
  XchgArgs a;
  a.local = local_partial;
  a.peers = reinterpret_cast<float *const *>(peer_buffers);
  kitty_lse_exchange_bytes(rows, world, &a.flag_offset);
  a.rank = rank;
  a.world = world;
  a.rows = static_cast<int32_t>(rows);
  a.seq = seq;
  a.out = out;
  a.out_dtype = out_dtype;
  a.status = status;
  lse_exchange_merge_kernel<<<static_cast<unsigned>(rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}
