// sacq_linear_a8_static_scratch: the split-K small-M forward for callers that cannot
// allocate device memory.
//
// Some hosts of this library run with a frozen device-memory budget: a robot-control
// loop that must not touch the allocator once it is live, an inference server whose
// arena owns every byte that is left, a plugin that is only handed input and output
// buffers.  For them the ordinary entry point's caller-provided workspace is a burden,
// so this variant keeps the split-K partial sums and arrival counters in a fixed array
// that is part of the library image.  Every GPU that loads the library holds the array
// (kStaticScratchBytes) until the process exits.
#include <string.h>

#include <atomic>

#include "common.cuh"

namespace sacq {

namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB, counters included

// Device storage.  In host code this name is only a handle for the runtime; the device
// address the kernel needs comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::atomic<void*> g_scratch_ptr[64] = {};   // per device; every writer stores the same address

int static_scratch_for_current_device(void** out) {
  int dev = -1;
  SACQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(SACQ_ERR_UNSUPPORTED, "device ordinal %d outside 0..63", dev);
  void* cached = g_scratch_ptr[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    if (ptr == nullptr) return set_error(SACQ_ERR_CUDA, "static scratch has no device address on device %d", dev);
    g_scratch_ptr[dev].store(ptr, std::memory_order_release);
    cached = ptr;
  }
  *out = cached;
  return SACQ_OK;
}

}  // namespace
}  // namespace sacq

using namespace sacq;

extern "C" {

SACQ_API int64_t sacq_static_scratch_bytes(void) { return (int64_t)kStaticScratchBytes; }

SACQ_API int sacq_linear_a8_static_scratch(const sacq_layer_t* L, const void* q, const float* scale, int64_t M,
                                           void* y_out, int64_t ldy, void* stream) {
  if (L == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "layer handle is null");
  if (M < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "M=%lld is negative", (long long)M);
  if (M == 0 || L->d.out_features == 0) return SACQ_OK;
  if (q == nullptr || scale == nullptr || y_out == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (ldy < L->d.out_features)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "ldy=%lld smaller than out_features=%lld", (long long)ldy,
                     (long long)L->d.out_features);
  if (!small_m_supported(L)) return set_error(SACQ_ERR_UNSUPPORTED, "layer geometry outside the small-M kernel");

  int prev = -1;
  SACQ_CUDA_TRY(cudaGetDevice(&prev));
  if (prev != L->d.device) SACQ_CUDA_TRY(cudaSetDevice(L->d.device));
  int rc = SACQ_OK;
  do {
    // the split-K CUDA-core variant is the one that needs scratch; run exactly that one
    sacq_layer view = *L;
    view.force_kernel = 3;
    // What the launch plan for (layer, M) uses, plus a bound that does not depend on the plan (how
    // far K is split depends on the device's SM count): one fp32 copy of the output must fit.
    int64_t need = 0, counters = 0;
    small_m_scratch_need(&view, M, &need, &counters);
    const int64_t one_split = sacq_workspace_counter_bytes() + M * L->d.out_features * (int64_t)sizeof(float);
    if (one_split > need) need = one_split;
    if (need > (int64_t)kStaticScratchBytes || counters * (int64_t)sizeof(int) > sacq_workspace_counter_bytes()) {
      rc = set_error(SACQ_ERR_WORKSPACE,
                     "this call (M=%lld, N=%lld) needs %lld bytes of scratch and %lld arrival counters, but the "
                     "built-in scratch holds %lld bytes and %lld counters; use sacq_linear_a8 with a "
                     "caller-provided workspace",
                     (long long)M, (long long)L->d.out_features, (long long)need, (long long)counters,
                     (long long)kStaticScratchBytes,
                     (long long)(sacq_workspace_counter_bytes() / (int64_t)sizeof(int)));
      break;
    }
    void* ptr = nullptr;
    rc = static_scratch_for_current_device(&ptr);
    if (rc != SACQ_OK) break;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left; the arrival counters must start at zero.
    const cudaError_t e = cudaMemsetAsync(ptr, 0, (size_t)sacq_workspace_counter_bytes(), s);
    if (e != cudaSuccess) {
      rc = cuda_fail(e, "clearing the arrival counters");
      break;
    }
    rc = launch_small_m(&view, q, scale, M, y_out, ldy, ptr, (int64_t)kStaticScratchBytes, s);
  } while (false);
  if (prev != L->d.device) cudaSetDevice(prev);
  return rc;
}

}  // extern "C"
