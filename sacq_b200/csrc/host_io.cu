// Result hand-off to host memory for the host-buffer forward.
//
// A small result is cheaper to push to pinned host memory with coalesced 16-byte stores from
// a kernel than through the copy engine: on a stream that alternates kernels and copies each
// copy costs several microseconds of engine hand-over, more than a sub-megabyte transfer
// itself.  The kernel is launched with programmatic stream serialization, so its launch
// overlaps the tail of the GEMM in front of it.
#include "common.cuh"

namespace sacq {

namespace {

__global__ void __launch_bounds__(256) copy_to_host_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                           int64_t bytes) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // src is written by the previous kernel of the stream
  const int64_t n16 = bytes >> 4;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  const int64_t tail = n16 << 4;
  if (blockIdx.x == 0 && tail + threadIdx.x < bytes) dst[tail + threadIdx.x] = src[tail + threadIdx.x];
}

}  // namespace

// src (device) and dst (device alias of pinned host memory) must be 16-byte aligned.
int launch_copy_to_host(const void* src, void* dst, int64_t bytes, int num_sms, cudaStream_t s) {
  if (bytes <= 0) return SACQ_OK;
  int64_t blocks = (bytes / 16 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 2 * (int64_t)num_sms) blocks = 2 * (int64_t)num_sms;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SACQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, copy_to_host_kernel, static_cast<const uint8_t*>(src),
                                   static_cast<uint8_t*>(dst), bytes));
  count_launch();
  return SACQ_OK;
}

}  // namespace sacq
