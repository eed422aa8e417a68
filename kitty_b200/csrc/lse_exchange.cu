// Sequence-split combine over peer memory: every rank stores its (acc[128], max, sum) partial of each
// query head straight into the exchange buffer of every rank (plain peer stores over NVLink), raises a
// per-row flag there, waits — bounded — for the other ranks' flags of the same row in its own buffer and
// merges.  One kernel replaces an all-gather collective plus a merge kernel; the exchange is 520 bytes per
// query head per rank, so the cost is one NVLink round trip instead of a collective's launch protocol.
// The device code lives in lse_exchange.cuh (the merge kernel of a sequence-split attention call uses it too).
#include "lse_exchange.cuh"

namespace kitty {

struct XchgArgs {
  const float *local;        // [rows][PART] this rank's partial
  XchgDesc x;
  int32_t rows;
  void *out;                 // [rows][128] of out_dtype
  int32_t out_dtype;
};

__global__ void __launch_bounds__(128) lse_exchange_merge_kernel(XchgArgs a) {
  const int r = blockIdx.x, c = threadIdx.x;
  const float v = a.local[static_cast<int64_t>(r) * PART + c];
  const float m = a.local[static_cast<int64_t>(r) * PART + HD];
  const float l = a.local[static_cast<int64_t>(r) * PART + HD + 1];
  float A, L;
  if (!xchg_row(a.x, a.rows, r, c, v, m, l, A, L)) return;     // the row stays unwritten, the status word says why
  store_out(a.out, a.out_dtype, static_cast<int64_t>(r) * HD + c, A / L);
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
                                        int32_t *status, int64_t wait_ns, void *stream) {
  if (!local_partial || !peer_buffers || !out) return KITTY_E_BADARG;
  if (rows <= 0 || rows > KITTY_EXCHANGE_MAX_ROWS || world <= 0 || world > 128 || rank < 0 || rank >= world || seq <= 0)
    return KITTY_E_BADARG;
  if (out_dtype < KITTY_F16 || out_dtype > KITTY_F32 || wait_ns < 0) return KITTY_E_BADARG;
  XchgArgs a;
  a.local = local_partial;
  a.x.peers = reinterpret_cast<float *const *>(peer_buffers);
  kitty_lse_exchange_bytes(rows, world, &a.x.flag_offset);
  a.x.rank = rank;
  a.x.world = world;
  a.x.seq = seq;
  a.x.status = status;
  a.x.wait_ns = wait_ns > 0 ? static_cast<unsigned long long>(wait_ns) : XCHG_WAIT_NS_DEFAULT;
  a.rows = static_cast<int32_t>(rows);
  a.out = out;
  a.out_dtype = out_dtype;
  lse_exchange_merge_kernel<<<static_cast<unsigned>(rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}
