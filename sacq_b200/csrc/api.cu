// C ABI of libsacq_b200: layer handles, argument checking, kernel selection.
// The kernels live in dequant.cu, act_quant.cu, linear_small_m.cu, linear_large_m.cu.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "common.cuh"

static_assert(sizeof(sacq_layer_desc) == 88, "sacq_layer_desc layout is part of the ABI");

namespace sacq {

namespace {
thread_local char g_error[512] = "";
std::atomic<long long> g_launches{0};
constexpr int64_t kCounterBytes = 64 * 1024;  // 16384 row-block arrival counters
}  // namespace

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return set_error(SACQ_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

// Runs `fn` with the layer's device current, restoring the caller's device afterwards.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

int check_layer(const sacq_layer_t* L) {
  if (L == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "layer handle is null");
  return SACQ_OK;
}

// Rows per launch of the small-M kernel so that its arrival counters fit their region.
int64_t small_m_slab_rows(const sacq_layer* L) {
  const int64_t row_blocks = (L->d.out_features + 31) / 32;
  int64_t chunks = (kCounterBytes / (int64_t)sizeof(int)) / (row_blocks > 0 ? row_blocks : 1);
  if (chunks < 1) chunks = 1;
  return chunks * 16;
}

// Rows from which the grouped tensor-core kernel beats the index-unpacking warp-MMA kernel
// (which walks the weights once per 16-token chunk).  Measured crossovers: 33 rows on layers
// wide enough to give the tensor-core grid a CTA for most SMs (N = 6144), 48-64 rows at
// N = 2048, about 96 rows below that.
int64_t grouped_min_m(const sacq_layer* L) {
  if (L->d.out_features >= 32 * (int64_t)L->num_sms) return 33;
  return L->d.out_features >= 2048 ? 48 : 96;
}
constexpr int64_t kTmemMinM = 1024;
constexpr int64_t kTmemMinMBigCodebook = 128;
// INT8 activations have no FP8 warp-MMA path, so the tensor-core kernel takes over earlier.
constexpr int64_t kGroupedMinMInt8 = 48;

int pick_kernel(const sacq_layer* L, int64_t M) {
  if (L->force_kernel == 7) return large_m_grouped_supported(L) ? 3 : SACQ_ERR_UNSUPPORTED;
  if (L->force_kernel >= 12) return large_m_tmem_grouped_supported(L) ? 5 : SACQ_ERR_UNSUPPORTED;
  if (L->force_kernel >= 8) return large_m_tmem_supported(L) ? 4 : SACQ_ERR_UNSUPPORTED;
  if (L->force_kernel == 1 || L->force_kernel >= 3)
    return small_m_supported(L) ? 1 : SACQ_ERR_UNSUPPORTED;
  if (L->force_kernel == 2) return large_m_supported(L) ? 2 : SACQ_ERR_UNSUPPORTED;
  // A shape rule, not a backend switch.  From kTmemMinM rows the tensor-core kernel that keeps
  // the expanded weights in tensor memory wins on every layer shape (its 128-row tiles need that
  // many tokens to fill the device).  The threshold does not depend on the layer's width, so
  // the row shards of a split layer run the kernel the whole layer would, and reproduce it
  // bit for bit.  Layers whose codebook does not fit shared memory have no other tensor-core
  // kernel and switch earlier.
  if (large_m_tmem_supported(L) && (M >= kTmemMinM || (M >= kTmemMinMBigCodebook && !large_m_supported(L)))) return 4;
  // Above 64 rows the tcgen05 kernel always wins.
  // Between 17 and 64 rows the small-M kernel walks its row tiles once per 16-token chunk
  // while one tensor-core M tile covers them all; that pays off once the layer has enough
  // output rows to give the tensor-core grid a CTA for most SMs (measured: N = 6144 yes,
  // N <= 2048 no).
  if (large_m_supported(L)) {
    if (M > 64) return 2;
    if (M > 16 && L->d.out_features >= 32 * (int64_t)L->num_sms) return 2;   // 2048x6144 at M = 32: 14.1 us against 11.3 us
    // ... and from 49 rows on deep layers: four 16-token chunks of K = 6144 cost the warp-MMA
    // kernel 28.8 us, the tensor-core kernel 24.5 us (measured at N = 2048).
    if (M > 48 && L->d.in_features >= 4096) return 2;
    // ... and on layers of 2048 or more rows (2048 x 2048 at M = 64: 9.8 us against 8.9 us)
    if (M > 48 && L->d.out_features >= 2048) return 2;
  } else if (large_m_tmem_grouped_supported(L) && M >= large_m_tmem_grouped_min_m(L)) {
    return 5;                                          // grouped scales, odd index widths: weights in tensor memory
  } else if (M >= grouped_min_m(L) && large_m_grouped_supported(L)) {
    return 3;                                          // ... expanded weight tiles in shared memory
  }
  return small_m_supported(L) ? 1 : SACQ_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace sacq

using namespace sacq;

extern "C" {

SACQ_API int sacq_abi_version(void) { return SACQ_ABI_VERSION; }
SACQ_API const char* sacq_last_error(void) { return g_error; }
SACQ_API int64_t sacq_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }
SACQ_API int64_t sacq_workspace_counter_bytes(void) { return kCounterBytes; }

SACQ_API int sacq_layer_create(const sacq_layer_desc* desc, sacq_layer_t** out_layer) {
  if (desc == nullptr || out_layer == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  *out_layer = nullptr;
  if (desc->struct_size != sizeof(sacq_layer_desc))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "sacq_layer_desc.struct_size is %u, this library expects %zu",
                     desc->struct_size, sizeof(sacq_layer_desc));
  const sacq_layer_desc& d = *desc;
  if (d.out_features < 0 || d.in_features <= 0 || d.vector_dim <= 0 || d.group_size <= 0 || d.codebook_size <= 0)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "non-positive geometry (N=%lld K=%lld d=%d G=%d C=%d)",
                     (long long)d.out_features, (long long)d.in_features, d.vector_dim, d.group_size,
                     d.codebook_size);
  if (d.in_features % d.group_size != 0)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "in_features=%lld is not a multiple of group_size=%d",
                     (long long)d.in_features, d.group_size);
  if (d.group_size % d.vector_dim != 0)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "group_size=%d is not a multiple of vector_dim=%d", d.group_size,
                     d.vector_dim);
  if (d.index_bits < 1 || d.index_bits > 24)
    return set_error(SACQ_ERR_UNSUPPORTED, "index_bits=%d outside [1, 24]", d.index_bits);
  if (d.index_bits < 31 && (int64_t)d.codebook_size > (1LL << d.index_bits))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "codebook_size=%d does not fit index_bits=%d", d.codebook_size,
                     d.index_bits);
  if (d.in_features > (1 << 24) || d.out_features > (1 << 24))
    return set_error(SACQ_ERR_UNSUPPORTED, "features above 2^24 are not supported");
  const int64_t vpr = d.in_features / d.vector_dim;
  const int64_t expect = (d.out_features * vpr * d.index_bits + 7) / 8;
  if (d.packed_bytes != expect)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "packed stream has %lld bytes, expected %lld",
                     (long long)d.packed_bytes, (long long)expect);
  if (d.codebook == nullptr || d.scales == nullptr || (d.packed == nullptr && expect > 0))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null device pointer in layer description");
  if (reinterpret_cast<uintptr_t>(d.packed) % 16 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "packed stream must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(d.codebook) % 16 != 0 || reinterpret_cast<uintptr_t>(d.scales) % 2 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "codebook must be 16-byte aligned");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0)
    return set_error(SACQ_ERR_CUDA, "no CUDA device is available; this library has no CPU path");
  if (d.device < 0 || d.device >= ndev)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "device %d out of range (%d devices)", d.device, ndev);

  DeviceGuard guard(d.device);
  if (!guard.ok) return set_error(SACQ_ERR_CUDA, "cannot make device %d current", d.device);
  sacq_layer* L = new (std::nothrow) sacq_layer();
  if (L == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "out of host memory");
  memset(L, 0, sizeof(*L));
  L->d = d;
  L->vectors_per_row = vpr;
  L->num_groups = d.in_features / d.group_size;
  L->row_bits = vpr * d.index_bits;
  L->rows_16b_aligned = (L->row_bits % 128) == 0;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, d.device) != cudaSuccess) {
    delete L;
    return set_error(SACQ_ERR_CUDA, "cudaGetDeviceProperties failed");
  }
  if (prop.major != 10) {
    delete L;
    return set_error(SACQ_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", d.device,
                     prop.major, prop.minor);
  }
  L->num_sms = prop.multiProcessorCount;
  L->cb_entries = (d.codebook_size + 1) & ~1;
  const int64_t count = (int64_t)L->cb_entries * d.vector_dim;
  cudaError_t e = cudaMalloc(&L->cb_f16, (size_t)count * sizeof(__half));
  if (e == cudaSuccess) e = cudaMalloc(&L->cb_hilo, (size_t)count * 2);
  if (e == cudaSuccess) e = cudaMalloc(&L->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(L->d_status, 0, sizeof(int));
  if (e != cudaSuccess) {
    sacq_layer_destroy(L);
    return cuda_fail(e, "allocating derived codebook tables");
  }
  L->resident_bytes = count * 4 + (int64_t)sizeof(int);
  const int rc = launch_build_tables(L, nullptr);
  if (rc != SACQ_OK) {
    sacq_layer_destroy(L);
    return rc;
  }
  *out_layer = L;
  return SACQ_OK;
}

SACQ_API int sacq_layer_destroy(sacq_layer_t* L) {
  if (L == nullptr) return SACQ_OK;
  DeviceGuard guard(L->d.device);
  large_m_release(L);
  if (L->cb_f16) cudaFree(L->cb_f16);
  if (L->cb_hilo) cudaFree(L->cb_hilo);
  if (L->d_status) cudaFree(L->d_status);
  delete L;
  return SACQ_OK;
}

SACQ_API int64_t sacq_layer_resident_bytes(const sacq_layer_t* L) { return L ? L->resident_bytes : 0; }

SACQ_API int sacq_dequant_bf16(const sacq_layer_t* L, void* w_out, void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (w_out == nullptr && L->d.out_features > 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "w_out is null");
  DeviceGuard guard(L->d.device);
  return launch_dequant_bf16(L, w_out, static_cast<cudaStream_t>(stream));
}

SACQ_API int sacq_weight_row_scale(const sacq_layer_t* L, float* sw_out, void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (sw_out == nullptr && L->d.out_features > 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "sw_out is null");
  DeviceGuard guard(L->d.device);
  return launch_weight_row_scale(L, sw_out, static_cast<cudaStream_t>(stream));
}

SACQ_API int sacq_decode_weight_fp8(const sacq_layer_t* L, const float* sw, void* wq_out, void* stream) {
  if (int rc = check_layer(L)) return rc;
  if ((sw == nullptr || wq_out == nullptr) && L->d.out_features > 0)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(L->d.device);
  return launch_decode_weight_fp8(L, sw, wq_out, static_cast<cudaStream_t>(stream));
}

SACQ_API int sacq_quant_act_fp8(const void* x_bf16, int64_t x_pitch, int64_t M, int64_t K, void* q_out, float* scale_out,
                       void* stream) {
  if (M < 0 || K < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "negative size (M=%lld K=%lld)", (long long)M,
                                       (long long)K);
  if (M == 0) return SACQ_OK;
  if (x_pitch < K) return set_error(SACQ_ERR_INVALID_ARGUMENT, "row pitch %lld smaller than K=%lld",
                                    (long long)x_pitch, (long long)K);
  if (scale_out == nullptr || ((x_bf16 == nullptr || q_out == nullptr) && K > 0))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (K == 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "K must be positive");
  return launch_quant_act_fp8(x_bf16, x_pitch, M, K, q_out, scale_out, static_cast<cudaStream_t>(stream));
}

SACQ_API int sacq_act_quant_fp8(int kind, const void* a_bf16, int64_t a_pitch, const void* b_bf16, int64_t b_pitch,
                                int64_t M, int64_t K, void* q_out, float* scale_out, void* stream) {
  if (kind != SACQ_ACT_SILU_MUL && kind != SACQ_ACT_GELU)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "unknown activation kind %d", kind);
  if (M < 0 || K < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "negative size (M=%lld K=%lld)", (long long)M,
                                       (long long)K);
  if (M == 0) return SACQ_OK;
  if (K == 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "K must be positive");
  if (a_bf16 == nullptr || q_out == nullptr || scale_out == nullptr || (kind == SACQ_ACT_SILU_MUL && b_bf16 == nullptr))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (a_pitch < K || (kind == SACQ_ACT_SILU_MUL && b_pitch < K))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "row pitch smaller than K=%lld", (long long)K);
  return launch_act_quant_fp8(kind, a_bf16, a_pitch, b_bf16, b_pitch, nullptr, M, K, q_out, scale_out,
                              static_cast<cudaStream_t>(stream));
}

SACQ_API int sacq_layernorm_quant_fp8(const void* x_bf16, int64_t x_pitch, const void* gamma_bf16, const void* beta_bf16,
                                      float eps, const void* mod_scale_bf16, const void* mod_shift_bf16, int64_t M,
                                      int64_t K, void* y_out_bf16, int64_t y_pitch, void* q_out, float* scale_out,
                                      void* stream) {
  if (M < 0 || K < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "negative size (M=%lld K=%lld)", (long long)M,
                                       (long long)K);
  if (M == 0) return SACQ_OK;
  if (K == 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "K must be positive");
  if (x_bf16 == nullptr || q_out == nullptr || scale_out == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if ((mod_scale_bf16 == nullptr) != (mod_shift_bf16 == nullptr))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "modulation needs both its scale and its shift vector");
  if (x_pitch < K || (y_out_bf16 != nullptr && y_pitch < K))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "row pitch smaller than K=%lld", (long long)K);
  if (!(eps >= 0.f)) return set_error(SACQ_ERR_INVALID_ARGUMENT, "eps must be non-negative");
  return launch_layernorm_quant_fp8(x_bf16, x_pitch, gamma_bf16, beta_bf16, eps, mod_scale_bf16, mod_shift_bf16, M, K,
                                    y_out_bf16, y_pitch, q_out, scale_out, static_cast<cudaStream_t>(stream));
}

SACQ_API int sacq_modulate_quant_fp8(const void* x_bf16, int64_t x_pitch, const void* scale_vec_bf16,
                                     const void* shift_vec_bf16, int64_t M, int64_t K, void* q_out, float* scale_out,
                                     void* stream) {
  if (M < 0 || K < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "negative size (M=%lld K=%lld)", (long long)M,
                                       (long long)K);
  if (M == 0) return SACQ_OK;
  if (K == 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "K must be positive");
  if (x_bf16 == nullptr || scale_vec_bf16 == nullptr || shift_vec_bf16 == nullptr || q_out == nullptr ||
      scale_out == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (x_pitch < K) return set_error(SACQ_ERR_INVALID_ARGUMENT, "row pitch smaller than K=%lld", (long long)K);
  return launch_act_quant_fp8(2, x_bf16, x_pitch, scale_vec_bf16, 0, shift_vec_bf16, M, K, q_out, scale_out,
                              static_cast<cudaStream_t>(stream));
}

SACQ_API int sacq_layer_set_kernel(sacq_layer_t* L, int which) {
  if (int rc = check_layer(L)) return rc;
  if (which < 0 || which > 15) return set_error(SACQ_ERR_INVALID_ARGUMENT, "kernel selector %d not in 0..15", which);
  L->force_kernel = which;
  return SACQ_OK;
}

SACQ_API int sacq_layer_kernel_for(const sacq_layer_t* L, int64_t M) {
  if (int rc = check_layer(L)) return rc;
  const int k = pick_kernel(L, M);
  if (k < 0) return set_error(k, "no kernel can run this layer geometry");
  return k;
}

SACQ_API int64_t sacq_workspace_bytes(const sacq_layer_t* L, int64_t M) {
  if (L == nullptr || M < 0) return 0;
  if (pick_kernel(L, M) == 3) return kCounterBytes + large_m_grouped_workspace_bytes(L, M);
  if (pick_kernel(L, M) == 5) return kCounterBytes + large_m_tmem_grouped_workspace_bytes(L, M);
  const int64_t slab = small_m_slab_rows(L);
  return small_m_workspace_bytes(L, M < slab ? M : slab);
}

namespace {
// Common body of sacq_linear_a8 and sacq_linear_a8_residual.
int linear_a8_impl(const sacq_layer_t* L, const void* q, const float* scale, int64_t M, const void* residual,
                   int64_t ldr, void* y_out, int64_t ldy, void* workspace, int64_t workspace_bytes, void* stream,
                   const BcastDst* bc = nullptr) {
  if (int rc = check_layer(L)) return rc;
  if (M < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "M=%lld is negative", (long long)M);
  if (M == 0 || L->d.out_features == 0) return SACQ_OK;
  if (q == nullptr || scale == nullptr || y_out == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (ldy < L->d.out_features)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "ldy=%lld smaller than out_features=%lld", (long long)ldy,
                     (long long)L->d.out_features);
  if (residual != nullptr && ldr < L->d.out_features)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "ldr=%lld smaller than out_features=%lld", (long long)ldr,
                     (long long)L->d.out_features);
  DeviceGuard guard(L->d.device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k = pick_kernel(L, M);
  if (k < 0) return set_error(k, "no kernel can run this layer geometry");
  if (k == 2) return launch_large_m(L, q, scale, M, y_out, ldy, s, residual, ldr, bc);
  if (k == 4)
    return launch_large_m_tmem(L, q, scale, M, y_out, ldy, s, residual, ldr, bc,
                               L->force_kernel >= 9 ? L->force_kernel - 8 : 0);
  if (k == 3 || k == 5) {
    if (workspace == nullptr || workspace_bytes < kCounterBytes)
      return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given",
                       (long long)sacq_workspace_bytes(L, M), (long long)workspace_bytes);
    if (k == 5)
      return launch_large_m_tmem_grouped(L, q, scale, M, y_out, ldy, static_cast<uint8_t*>(workspace) + kCounterBytes,
                                         workspace_bytes - kCounterBytes, s, residual, ldr, 0, bc,
                                         L->force_kernel >= 13 ? L->force_kernel - 12 : 0);
    return launch_large_m_grouped(L, q, scale, M, y_out, ldy, static_cast<uint8_t*>(workspace) + kCounterBytes,
                                  workspace_bytes - kCounterBytes, s, residual, ldr, 0, bc);
  }
  const int64_t slab = small_m_slab_rows(L);
  for (int64_t m0 = 0; m0 < M; m0 += slab) {
    const int64_t rows = (M - m0) < slab ? (M - m0) : slab;
    BcastDst slab_bc{};
    if (bc != nullptr) {
      slab_bc.n = bc->n;
      for (int i = 0; i < bc->n; ++i) slab_bc.ptr[i] = static_cast<uint16_t*>(bc->ptr[i]) + m0 * ldy;
    }
    const int rc = launch_small_m(L, static_cast<const uint8_t*>(q) + m0 * L->d.in_features, scale + m0, rows,
                                  static_cast<uint16_t*>(y_out) + m0 * ldy, ldy, workspace, workspace_bytes, s,
                                  residual ? static_cast<const uint16_t*>(residual) + m0 * ldr : nullptr, ldr, 0,
                                  bc ? &slab_bc : nullptr);
    if (rc != SACQ_OK) return rc;
  }
  return SACQ_OK;
}
}  // namespace

namespace {
// INT8 activations run on the kernels that widen the activation bytes to fp16 themselves:
// the grouped tensor-core kernel (tcgen05 kind::f16) from kGroupedMinM rows, below that the
// fp16 warp-MMA kernel where the layer's geometry allows it, else the CUDA-core kernel.
int int8_small_selector(const sacq_layer* L) { return small_m_int8_selector(L); }
}  // namespace

SACQ_API int sacq_quant_act_int8(const void* x_bf16, int64_t x_pitch, int64_t M, int64_t K, void* q_out, float* scale_out,
                                 void* stream) {
  if (M < 0 || K < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "negative size (M=%lld K=%lld)", (long long)M,
                                       (long long)K);
  if (M == 0) return SACQ_OK;
  if (x_pitch < K) return set_error(SACQ_ERR_INVALID_ARGUMENT, "row pitch %lld smaller than K=%lld",
                                    (long long)x_pitch, (long long)K);
  if (scale_out == nullptr || ((x_bf16 == nullptr || q_out == nullptr) && K > 0))
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (K == 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "K must be positive");
  return launch_quant_act_int8(x_bf16, x_pitch, M, K, q_out, scale_out, static_cast<cudaStream_t>(stream));
}

SACQ_API int64_t sacq_workspace_bytes_int8(const sacq_layer_t* L, int64_t M) {
  if (L == nullptr || M < 0) return 0;
  if (large_m_tmem_grouped_supported(L) && M >= large_m_tmem_grouped_min_m(L))
    return kCounterBytes + large_m_tmem_grouped_workspace_bytes(L, M);
  if (M >= kGroupedMinMInt8 && large_m_grouped_supported(L)) return kCounterBytes + large_m_grouped_workspace_bytes(L, M);
  sacq_layer view = *L;
  view.force_kernel = int8_small_selector(L);
  const int64_t slab = small_m_slab_rows(L);
  return small_m_workspace_bytes(&view, M < slab ? M : slab);
}

SACQ_API int sacq_linear_a8i(const sacq_layer_t* L, const void* q_int8, const float* scale, int64_t M, void* y_out,
                             int64_t ldy, void* workspace, int64_t workspace_bytes, void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (M < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "M=%lld is negative", (long long)M);
  if (M == 0 || L->d.out_features == 0) return SACQ_OK;
  if (q_int8 == nullptr || scale == nullptr || y_out == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (ldy < L->d.out_features)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "ldy=%lld smaller than out_features=%lld", (long long)ldy,
                     (long long)L->d.out_features);
  DeviceGuard guard(L->d.device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (large_m_tmem_grouped_supported(L) && M >= large_m_tmem_grouped_min_m(L)) {
    if (workspace == nullptr || workspace_bytes < kCounterBytes)
      return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given",
                       (long long)sacq_workspace_bytes_int8(L, M), (long long)workspace_bytes);
    return launch_large_m_tmem_grouped(L, q_int8, scale, M, y_out, ldy, static_cast<uint8_t*>(workspace) + kCounterBytes,
                                       workspace_bytes - kCounterBytes, s, nullptr, 0, 1);
  }
  if (M >= kGroupedMinMInt8 && large_m_grouped_supported(L)) {
    if (workspace == nullptr || workspace_bytes < kCounterBytes)
      return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given",
                       (long long)sacq_workspace_bytes_int8(L, M), (long long)workspace_bytes);
    return launch_large_m_grouped(L, q_int8, scale, M, y_out, ldy, static_cast<uint8_t*>(workspace) + kCounterBytes,
                                  workspace_bytes - kCounterBytes, s, nullptr, 0, 1);
  }
  if (!small_m_supported(L)) return set_error(SACQ_ERR_UNSUPPORTED, "no kernel can run this layer geometry");
  sacq_layer view = *L;
  view.force_kernel = int8_small_selector(L);
  const int64_t slab = small_m_slab_rows(L);
  for (int64_t m0 = 0; m0 < M; m0 += slab) {
    const int64_t rows = (M - m0) < slab ? (M - m0) : slab;
    const int rc = launch_small_m(&view, static_cast<const uint8_t*>(q_int8) + m0 * L->d.in_features, scale + m0, rows,
                                  static_cast<uint16_t*>(y_out) + m0 * ldy, ldy, workspace, workspace_bytes, s, nullptr,
                                  0, 1);
    if (rc != SACQ_OK) return rc;
  }
  return SACQ_OK;
}

SACQ_API int sacq_weight_row_scale_int8(const sacq_layer_t* L, float* sw_out, void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (sw_out == nullptr && L->d.out_features > 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "sw_out is null");
  DeviceGuard guard(L->d.device);
  return launch_weight_row_scale(L, sw_out, static_cast<cudaStream_t>(stream), 127.0f);
}

SACQ_API int sacq_decode_weight_int8(const sacq_layer_t* L, const float* sw, void* wq_out, void* stream) {
  if (int rc = check_layer(L)) return rc;
  if ((sw == nullptr || wq_out == nullptr) && L->d.out_features > 0)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(L->d.device);
  return launch_decode_weight_int8(L, sw, wq_out, static_cast<cudaStream_t>(stream));
}

SACQ_API int64_t sacq_workspace_bytes_w8a8(const sacq_layer_t* L, int64_t M) {
  if (L == nullptr || M < 0) return 0;
  // the leading counter region of every workspace stays untouched (and zero) for the kernels that use it
  return kCounterBytes + ((L->d.out_features * L->d.in_features + 255) & ~(int64_t)255);
}

SACQ_API int sacq_linear_w8a8_int8(const sacq_layer_t* L, const void* q_int8, const float* act_scale, const float* w_scale,
                                   int64_t M, void* y_out, int64_t ldy, void* workspace, int64_t workspace_bytes,
                                   void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (M < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "M=%lld is negative", (long long)M);
  if (M == 0 || L->d.out_features == 0) return SACQ_OK;
  if (q_int8 == nullptr || act_scale == nullptr || w_scale == nullptr || y_out == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (ldy < L->d.out_features)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "ldy=%lld smaller than out_features=%lld", (long long)ldy,
                     (long long)L->d.out_features);
  if (!dense_i8_supported(L))
    return set_error(SACQ_ERR_UNSUPPORTED, "INT8 recipe needs in_features to be a multiple of 16");
  const int64_t need = sacq_workspace_bytes_w8a8(L, M);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given", (long long)need,
                     (long long)workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  DeviceGuard guard(L->d.device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // per call, as the reference does: packed stream -> int8 weight rows, then the dense integer GEMM
  void* wq = static_cast<uint8_t*>(workspace) + kCounterBytes;
  if (int rc = launch_decode_weight_int8(L, w_scale, wq, s)) return rc;
  return launch_dense_i8(L, q_int8, act_scale, wq, w_scale, M, y_out, ldy, s);
}

SACQ_API int sacq_linear_w8a8_fp8(const sacq_layer_t* L, const void* q_e4m3, const float* act_scale, const float* w_scale,
                                  int64_t M, void* y_out, int64_t ldy, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (M < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "M=%lld is negative", (long long)M);
  if (M == 0 || L->d.out_features == 0) return SACQ_OK;
  if (q_e4m3 == nullptr || act_scale == nullptr || w_scale == nullptr || y_out == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  if (ldy < L->d.out_features)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "ldy=%lld smaller than out_features=%lld", (long long)ldy,
                     (long long)L->d.out_features);
  if (!dense_i8_supported(L))
    return set_error(SACQ_ERR_UNSUPPORTED, "FP8 recipe needs in_features to be a multiple of 16");
  const int64_t need = sacq_workspace_bytes_w8a8(L, M);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given", (long long)need,
                     (long long)workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  DeviceGuard guard(L->d.device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // per call, as the reference does: packed stream -> e4m3 weight rows, then the dense FP8 GEMM
  void* wq = static_cast<uint8_t*>(workspace) + kCounterBytes;
  if (int rc = launch_decode_weight_fp8(L, w_scale, wq, s)) return rc;
  return launch_dense_i8(L, q_e4m3, act_scale, wq, w_scale, M, y_out, ldy, s, true);
}

SACQ_API int sacq_linear_a8(const sacq_layer_t* L, const void* q, const float* scale, int64_t M, void* y_out, int64_t ldy,
                   void* workspace, int64_t workspace_bytes, void* stream) {
  return linear_a8_impl(L, q, scale, M, nullptr, 0, y_out, ldy, workspace, workspace_bytes, stream);
}

SACQ_API int sacq_linear_a8_bcast(const sacq_layer_t* L, const void* q, const float* scale, int64_t M, void* y_out,
                                  void* const* peer_outs, int num_peers, int64_t ldy, void* workspace,
                                  int64_t workspace_bytes, void* stream) {
  if (num_peers < 0 || num_peers > kMaxBcast)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "num_peers=%d outside [0, %d]", num_peers, kMaxBcast);
  if (num_peers > 0 && peer_outs == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "peer_outs is null");
  BcastDst bc{};
  bc.n = num_peers;
  for (int i = 0; i < num_peers; ++i) {
    if (peer_outs[i] == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "peer output %d is null", i);
    bc.ptr[i] = peer_outs[i];
  }
  return linear_a8_impl(L, q, scale, M, nullptr, 0, y_out, ldy, workspace, workspace_bytes, stream, &bc);
}

// ---- buffers that other processes of the node can map (CUDA IPC) -------------------------
SACQ_API int sacq_peer_buffer_create(int device, int64_t bytes, void** dev_ptr, void* handle_out) {
  if (dev_ptr == nullptr || handle_out == nullptr || bytes <= 0)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument or non-positive size");
  DeviceGuard guard(device);
  if (!guard.ok) return set_error(SACQ_ERR_CUDA, "cannot make device %d current", device);
  void* p = nullptr;
  SACQ_CUDA_TRY(cudaMalloc(&p, (size_t)bytes));
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "cudaIpcGetMemHandle");
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == SACQ_PEER_HANDLE_BYTES, "handle size");
  memcpy(handle_out, &h, sizeof(h));
  *dev_ptr = p;
  return SACQ_OK;
}

SACQ_API int sacq_peer_buffer_open(int device, const void* handle, void** dev_ptr) {
  if (dev_ptr == nullptr || handle == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  DeviceGuard guard(device);
  if (!guard.ok) return set_error(SACQ_ERR_CUDA, "cannot make device %d current", device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  SACQ_CUDA_TRY(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return SACQ_OK;
}

SACQ_API int sacq_peer_buffer_close(int device, void* dev_ptr) {
  if (dev_ptr == nullptr) return SACQ_OK;
  DeviceGuard guard(device);
  SACQ_CUDA_TRY(cudaIpcCloseMemHandle(dev_ptr));
  return SACQ_OK;
}

SACQ_API int sacq_peer_buffer_destroy(int device, void* dev_ptr) {
  if (dev_ptr == nullptr) return SACQ_OK;
  DeviceGuard guard(device);
  SACQ_CUDA_TRY(cudaFree(dev_ptr));
  return SACQ_OK;
}

SACQ_API int sacq_linear_a8_residual(const sacq_layer_t* L, const void* q, const float* scale, int64_t M,
                                     const void* residual, int64_t ldr, void* y_out, int64_t ldy, void* workspace,
                                     int64_t workspace_bytes, void* stream) {
  if (residual == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "residual is null");
  return linear_a8_impl(L, q, scale, M, residual, ldr, y_out, ldy, workspace, workspace_bytes, stream);
}

SACQ_API int sacq_linear_a8_multi(const sacq_layer_t* const* layers, int num_layers, const void* q, const float* scale,
                                  int64_t M, void* const* y_outs, const int64_t* ldys, void* workspace,
                                  int64_t workspace_bytes, void* stream) {
  if (layers == nullptr || y_outs == nullptr || ldys == nullptr || num_layers <= 0)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument or no layers");
  for (int l = 0; l < num_layers; ++l) {
    if (int rc = check_layer(layers[l])) return rc;
    if (layers[l]->d.in_features != layers[0]->d.in_features)
      return set_error(SACQ_ERR_INVALID_ARGUMENT, "layers that share an input must have the same in_features");
    if (layers[l]->d.device != layers[0]->d.device)
      return set_error(SACQ_ERR_INVALID_ARGUMENT, "layers that share an input must be on one device");
    if (y_outs[l] == nullptr && layers[l]->d.out_features > 0 && M > 0)
      return set_error(SACQ_ERR_INVALID_ARGUMENT, "null output for layer %d", l);
    if (ldys[l] < layers[l]->d.out_features)
      return set_error(SACQ_ERR_INVALID_ARGUMENT, "ldy=%lld smaller than out_features=%lld", (long long)ldys[l],
                       (long long)layers[l]->d.out_features);
  }
  if (M < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "M=%lld is negative", (long long)M);
  if (M == 0) return SACQ_OK;
  if (q == nullptr || scale == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  {
    // one launch when every layer would use the staged small-M kernel on a common geometry
    bool small = num_layers >= 2;
    for (int l = 0; l < num_layers && small; ++l) small = pick_kernel(layers[l], M) == 1;
    if (small) {
      DeviceGuard guard(layers[0]->d.device);
      const int rc = launch_small_m_multi(layers, num_layers, q, scale, M, y_outs, ldys,
                                          static_cast<cudaStream_t>(stream));
      if (rc != SACQ_ERR_UNSUPPORTED) return rc;
    }
    // ... or the FP8 tensor-core kernel (blockIdx.z = layer)
    bool large = num_layers >= 2;
    for (int l = 0; l < num_layers && large; ++l) large = pick_kernel(layers[l], M) == 2;
    if (large) {
      DeviceGuard guard(layers[0]->d.device);
      const int rc = launch_large_m_multi(layers, num_layers, q, scale, M, y_outs, ldys,
                                          static_cast<cudaStream_t>(stream));
      if (rc != SACQ_ERR_UNSUPPORTED) return rc;
    }
  }
  for (int l = 0; l < num_layers; ++l) {
    const int rc = sacq_linear_a8(layers[l], q, scale, M, y_outs[l], ldys[l], workspace, workspace_bytes, stream);
    if (rc != SACQ_OK) return rc;
  }
  return SACQ_OK;
}

SACQ_API int sacq_linear_bf16(const sacq_layer_t* L, const void* x_bf16, int64_t x_pitch, int64_t M, void* q_scratch,
                     float* scale_scratch, void* y_out, int64_t ldy, void* workspace, int64_t workspace_bytes,
                     void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (M == 0) return SACQ_OK;
  int rc = sacq_quant_act_fp8(x_bf16, x_pitch, M, L->d.in_features, q_scratch, scale_scratch, stream);
  if (rc != SACQ_OK) return rc;
  return sacq_linear_a8(L, q_scratch, scale_scratch, M, y_out, ldy, workspace, workspace_bytes, stream);
}

// Layout of the device scratch of sacq_linear_bf16_host: workspace first (its counter
// region leads), then scale, x, q, y, each 256-byte aligned.
namespace {
struct HostForwardLayout {
  int64_t ws, scale, x, q, y, total;
};
HostForwardLayout host_forward_layout(const sacq_layer* L, int64_t M) {
  auto up = [](int64_t v) { return (v + 255) & ~(int64_t)255; };
  HostForwardLayout h;
  h.ws = 0;
  h.scale = up(sacq_workspace_bytes(L, M));
  h.x = h.scale + up(M * 4);
  h.q = h.x + up(M * L->d.in_features * 2);
  h.y = h.q + up(M * L->d.in_features);
  h.total = h.y + up(M * L->d.out_features * 2);
  return h;
}

// Transfers up to this size bypass the copy engine when the host buffer is pinned: the
// quantizer reads the activations straight from host memory and a copy kernel pushes the
// result back (each copy-engine hand-over on a stream costs more than the transfer itself).
constexpr int64_t kDirectHostIoBytes = 1 << 20;

// Device alias of a pinned (page-locked, mapped) host pointer, or null.
void* pinned_alias(const void* host) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, host) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}
}  // namespace

SACQ_API int64_t sacq_host_forward_scratch_bytes(const sacq_layer_t* L, int64_t M) {
  if (L == nullptr || M < 0) return 0;
  return host_forward_layout(L, M).total;
}

SACQ_API int sacq_linear_bf16_host(const sacq_layer_t* L, const void* x_host, int64_t M, void* y_host,
                                   void* dev_scratch, int64_t dev_scratch_bytes, void* stream) {
  if (int rc = check_layer(L)) return rc;
  if (M < 0) return set_error(SACQ_ERR_INVALID_ARGUMENT, "M=%lld is negative", (long long)M);
  if (M == 0 || L->d.out_features == 0) return SACQ_OK;
  if (x_host == nullptr || y_host == nullptr || dev_scratch == nullptr)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "null argument");
  const HostForwardLayout h = host_forward_layout(L, M);
  if (dev_scratch_bytes < h.total)
    return set_error(SACQ_ERR_WORKSPACE, "device scratch of %lld bytes needed, %lld given", (long long)h.total,
                     (long long)dev_scratch_bytes);
  if (reinterpret_cast<uintptr_t>(dev_scratch) % 256 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "device scratch must be 256-byte aligned");
  DeviceGuard guard(L->d.device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(dev_scratch);
  const int64_t K = L->d.in_features, N = L->d.out_features;
  const void* x_dev = base + h.x;
  void* x_alias = M * K * 2 <= kDirectHostIoBytes && reinterpret_cast<uintptr_t>(x_host) % 16 == 0
                      ? pinned_alias(x_host) : nullptr;
  if (x_alias != nullptr)
    x_dev = x_alias;                                   // the quantizer reads the pinned buffer itself
  else
    SACQ_CUDA_TRY(cudaMemcpyAsync(base + h.x, x_host, (size_t)(M * K * 2), cudaMemcpyHostToDevice, s));
  const int rc = sacq_linear_bf16(L, x_dev, K, M, base + h.q, reinterpret_cast<float*>(base + h.scale),
                                  base + h.y, N, base + h.ws, h.scale, stream);
  if (rc != SACQ_OK) return rc;
  void* y_alias = M * N * 2 <= kDirectHostIoBytes && reinterpret_cast<uintptr_t>(y_host) % 16 == 0
                      ? pinned_alias(y_host) : nullptr;
  if (y_alias != nullptr) return launch_copy_to_host(base + h.y, y_alias, M * N * 2, L->num_sms, s);
  SACQ_CUDA_TRY(cudaMemcpyAsync(y_host, base + h.y, (size_t)(M * N * 2), cudaMemcpyDeviceToHost, s));
  return SACQ_OK;
}

SACQ_API int sacq_layer_status(const sacq_layer_t* L, int* status_out) {
  if (int rc = check_layer(L)) return rc;
  if (status_out == nullptr) return set_error(SACQ_ERR_INVALID_ARGUMENT, "status_out is null");
  DeviceGuard guard(L->d.device);
  SACQ_CUDA_TRY(cudaMemcpy(status_out, L->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  return SACQ_OK;
}

}  // extern "C"
