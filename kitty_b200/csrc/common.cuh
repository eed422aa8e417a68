// Shared constants and small device helpers for the kitty_b200 kernels (sm_100a).
#pragma once
#include <atomic>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kitty_b200.h"

namespace kitty {

// Fixed geometry (kvcache/kitty.py:43-47 of the reference).
constexpr int PAGE = 128;   // tokens per page
constexpr int HD = 128;     // head_dim
constexpr int DB = 32;      // boosted channels per page
constexpr int SINK = 32;    // full-precision sink tokens
// Key record of one head inside a page row (kernels/kitty_quant_pack.py:42-45).
constexpr int K_ROW = 32;                 // bytes per channel row (128 tokens x 2 bit)
constexpr int K_OFF_HI = K_ROW * HD;      // 4096: high plane, one row per slot
constexpr int K_OFF_IDX = K_ROW * (HD + DB);  // 5120: dense->sparse index bytes
constexpr int K_HEAD = K_OFF_IDX + HD;    // 5248
// Value record (kernels/kitty_quant_pack.py:180-181).
constexpr int V_ROW = 32;                 // bytes per token row (128 channels x 2 bit)
constexpr int V_HEAD = V_ROW * PAGE;      // 4096
constexpr int META_HEAD = PAGE * 2 * 2;   // 512 bytes: 128 x (scale, min) fp16

// Partial result of a slice of the sequence for one query head:
// acc[128], running max (base-2 logit domain), running sum.
constexpr int PART = HD + 2;

constexpr int MAX_GROUP = 16;  // query heads per KV head (kernels/kitty_attention.py:418)

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- once-per-device host set-up ------------------------------------------ //
// Entry points may be called from several host threads and on several devices.  Set-up that has to
// happen once per device (function-attribute opt-ins, attribute queries) goes through this helper:
// `setup` runs with the device current until it has succeeded once on that device.  It must be
// idempotent, because two threads that arrive together may both run it; nothing else is shared.
constexpr int MAX_DEVICES = 64;
struct PerDeviceOnce {
  std::atomic<int> done[MAX_DEVICES];
};
template <typename F>
inline int per_device_once(PerDeviceOnce &o, F &&setup) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return KITTY_E_CUDA;
  if (o.done[dev].load(std::memory_order_acquire)) return KITTY_OK;
  const int rc = setup();
  if (rc == KITTY_OK) o.done[dev].store(1, std::memory_order_release);
  return rc;
}

// ---- programmatic dependent launch ---------------------------------------- //
// A kernel launched with launch_after() may be scheduled while the kernel before it in the stream is still
// running, so that its launch latency is hidden; it must call dep_wait() before it touches anything the
// earlier kernel (or anything before that) wrote — dep_wait() returns once that kernel has completed and its
// writes are visible.  A kernel that is followed by such a launch calls dep_release() once its blocks are
// running, which lets the next launch be scheduled early.  Both are no-ops in an ordinary launch.
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- 8 consecutive channels -> fp32 --------------------------------------- //
template <typename T>
struct Vec8;

template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half *p, float (&o)[8]) { unpack(*reinterpret_cast<const uint4 *>(p), o); }
  static __device__ __forceinline__ void unpack(uint4 v, float (&o)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
  }
};

template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&o)[8]) { unpack(*reinterpret_cast<const uint4 *>(p), o); }
  static __device__ __forceinline__ void unpack(uint4 v, float (&o)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float *p, float (&o)[8]) {
    float4 a = *reinterpret_cast<const float4 *>(p);
    float4 b = *reinterpret_cast<const float4 *>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  }
};

// fp32 x8 -> fp16 x8 (round to nearest even), one 16-byte store.
__device__ __forceinline__ void store8_f16(__half *dst, const float (&v)[8]) {
  uint4 o;
  __half2 *h = reinterpret_cast<__half2 *>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4 *>(dst) = o;
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }

}  // namespace kitty
