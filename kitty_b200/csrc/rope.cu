// Rotary position embedding of one decode token's query and key heads in one launch.
// The call site this replaces is the model's attention forward
// (models/qwen3/modeling_qwen3.py:222-232 apply_rotary_pos_emb: q*cos + rotate_half(q)*sin, eight
// element-wise launches plus the copies that make q and k contiguous for the cache).  Every product and
// the sum are rounded to the data type, as the element-wise kernels of the model do, so the result is
// bit-identical to that path.
#include "common.cuh"

namespace kitty {

struct RopeArgs {
  const void *q, *k, *cos, *sin;
  void *q_out, *k_out;
  int32_t B, h_q, h_kv;
  int64_t cs_b;       // element stride of cos / sin between batch rows (0: one position for all rows)
};

template <typename T>
__global__ void __launch_bounds__(256) rope_qk_kernel(RopeArgs a) {
  constexpr int HALF = HD / 2;
  const int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int rows_q = a.B * a.h_q, rows_k = a.B * a.h_kv;
  if (u >= static_cast<int64_t>(rows_q + rows_k) * HALF) return;
  const int d = static_cast<int>(u % HALF);
  int64_t row = u / HALF;
  const T *src;
  T *dst;
  int b;
  if (row < rows_q) {
    src = static_cast<const T *>(a.q) + row * HD;
    dst = static_cast<T *>(a.q_out) + row * HD;
    b = static_cast<int>(row / a.h_q);
  } else {
    row -= rows_q;
    src = static_cast<const T *>(a.k) + row * HD;
    dst = static_cast<T *>(a.k_out) + row * HD;
    b = static_cast<int>(row / a.h_kv);
  }
  const T *cs = static_cast<const T *>(a.cos) + b * a.cs_b, *sn = static_cast<const T *>(a.sin) + b * a.cs_b;
  const float x1 = to_f32<T>(src[d]), x2 = to_f32<T>(src[d + HALF]);
  const float c1 = to_f32<T>(cs[d]), c2 = to_f32<T>(cs[d + HALF]);
  const float s1 = to_f32<T>(sn[d]), s2 = to_f32<T>(sn[d + HALF]);
  auto R = [](float v) { return to_f32<T>(from_f32<T>(v)); };
  // rotate_half(x) = (-x2, x1)
  dst[d] = from_f32<T>(__fadd_rn(R(__fmul_rn(x1, c1)), R(__fmul_rn(-x2, s1))));
  dst[d + HALF] = from_f32<T>(__fadd_rn(R(__fmul_rn(x2, c2)), R(__fmul_rn(x1, s2))));
}

}  // namespace kitty

using namespace kitty;

extern "C" int kitty_rope_qk(const void *q, const void *k, const void *cos, const void *sin, void *q_out, void *k_out,
                             int dtype, int32_t B, int32_t h_q, int32_t h_kv, int64_t cos_stride_b, void *stream) {
  if (!q || !k || !cos || !sin || !q_out || !k_out) return KITTY_E_BADARG;
  if (B <= 0 || h_q <= 0 || h_kv <= 0 || cos_stride_b < 0) return KITTY_E_BADARG;
  if (dtype < KITTY_F16 || dtype > KITTY_F32) return KITTY_E_BADARG;
  RopeArgs a{q, k, cos, sin, q_out, k_out, B, h_q, h_kv, cos_stride_b};
  const int64_t n = static_cast<int64_t>(B) * (h_q + h_kv) * (HD / 2);
  const unsigned grid = static_cast<unsigned>((n + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == KITTY_F16) rope_qk_kernel<__half><<<grid, 256, 0, s>>>(a);
  else if (dtype == KITTY_BF16) rope_qk_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a);
  else rope_qk_kernel<float><<<grid, 256, 0, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}
