// Stand-alone edge kernel: one block of 8 warps per (batch, kv-head).  Used with the fp16 streaming
// kernel; the int8 streaming kernel runs the same reduction inside its own grid.
#include "decode_edge.cuh"

namespace kitty {

constexpr int EDGE_KERNEL_WARPS = 8;
using EdgeKernelSmem = EdgeSmem<MAX_GROUP, EDGE_KERNEL_WARPS, 0>;

template <int NG>
__global__ void __launch_bounds__(EDGE_KERNEL_WARPS * 32) decode_edge_kernel(DecodeArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  EdgeKernelSmem &sm = *reinterpret_cast<EdgeKernelSmem *>(smem_raw);
  edge_item<NG, EDGE_KERNEL_WARPS>(a, a.P, a.C, sm, blockIdx.y, blockIdx.x, blockIdx.z);
}

int launch_decode_edge(const DecodeArgs &a, cudaStream_t s) {
  static int configured = -1;     // per-process opt-in to > 48 KB dynamic shared memory, once per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return KITTY_E_CUDA;
  const int smem = static_cast<int>(sizeof(EdgeKernelSmem));
  if (configured != dev) {
    if (cudaFuncSetAttribute(decode_edge_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaFuncSetAttribute(decode_edge_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaFuncSetAttribute(decode_edge_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return KITTY_E_CUDA;
    configured = dev;
  }
  dim3 grid(a.P.H, a.P.B, a.P.edge_parts);
  if (a.P.G <= 4) decode_edge_kernel<4><<<grid, EDGE_KERNEL_WARPS * 32, smem, s>>>(a);
  else if (a.P.G <= 8) decode_edge_kernel<8><<<grid, EDGE_KERNEL_WARPS * 32, smem, s>>>(a);
  else decode_edge_kernel<16><<<grid, EDGE_KERNEL_WARPS * 32, smem, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? KITTY_OK : KITTY_E_CUDA;
}

}  // namespace kitty
