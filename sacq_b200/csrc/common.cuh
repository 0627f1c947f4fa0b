// Shared device/host helpers for the sacq_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sacq_b200.h"

namespace sacq {

constexpr float kE4M3Max = 448.0f;
constexpr int kNumSMsB200 = 148;

// ----------------------------------------------------------------------------
// host side: the layer handle and error plumbing
// ----------------------------------------------------------------------------

struct LargeMPlan;  // built lazily by the large-M kernel's host code

}  // namespace sacq

struct sacq_layer {
  sacq_layer_desc d;
  int64_t vectors_per_row;   // K / d
  int64_t num_groups;        // K / G
  int64_t row_bits;          // (K/d) * b
  bool rows_16b_aligned;     // every row of the packed stream starts on a 16-byte boundary
  int num_sms;
  int force_kernel;          // 0 auto, 1 small-M, 2 large-M, 3..6 small-M variants, 7 grouped tensor-core
  int cb_entries;            // codebook entries rounded up to even: the derived tables are whole 16-byte units
  // derived device tables (owned)
  __half* cb_f16;            // [cb_entries, d] (zero padded) codebook * 2^cb_exp_shift as fp16 (small-M kernel)
  uint8_t* cb_hilo;          // [cb_entries][2][d] (zero padded) e4m3 high/low split of codebook * 2^cb8_exp_shift (large-M kernel)
  int cb_exp_shift;          // power-of-two normalisation folded back in the epilogue
  int cb8_exp_shift;
  int sc_exp_shift;          // max |scale| * 2^sc_exp_shift lies in [0.5, 1) (grouped tensor-core kernel)
  int* d_status;             // device status word, 0 = ok
  int64_t resident_bytes;
  sacq::LargeMPlan* large_plan;
};

namespace sacq {

// A non-zero shift (either sign of zero counts as none).  The fast kernels contract codewords and
// apply scale and shift afterwards; that drops the two bf16 roundings of the reference's
// reconstruction, which a shift larger than the weights makes visible.  Shifted layers therefore
// run on kernels that rebuild bf16(bf16(c * s) + shift) per weight.
inline bool has_shift(const sacq_layer* L) { return (L->d.shift_bf16 & 0x7fffu) != 0; }

int set_error(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
void count_launch(int n = 1);

#define SACQ_CUDA_TRY(expr)                                  \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return ::sacq::cuda_fail(_e, #expr); \
  } while (0)

// kernel entry points implemented in the other translation units
int launch_dequant_bf16(const sacq_layer* L, void* w_out, cudaStream_t s);
int launch_weight_row_scale(const sacq_layer* L, float* sw, cudaStream_t s, float limit = kE4M3Max);
int launch_decode_weight_fp8(const sacq_layer* L, const float* sw, void* wq, cudaStream_t s);
int launch_decode_weight_int8(const sacq_layer* L, const float* sw, void* wq, cudaStream_t s);
int launch_quant_act_fp8(const void* x, int64_t pitch, int64_t M, int64_t K, void* q, float* scale, cudaStream_t s);
int launch_quant_act_int8(const void* x, int64_t pitch, int64_t M, int64_t K, void* q, float* scale, cudaStream_t s);
int launch_act_quant_fp8(int kind, const void* a, int64_t a_pitch, const void* b, int64_t b_pitch, const void* c,
                         int64_t M, int64_t K, void* q, float* scale, cudaStream_t s);
int launch_layernorm_quant_fp8(const void* x, int64_t pitch, const void* gamma, const void* beta, float eps,
                               const void* mod_scale, const void* mod_shift, int64_t M, int64_t K, void* y_out,
                               int64_t y_pitch, void* q, float* scale, cudaStream_t s);
int launch_build_tables(sacq_layer* L, cudaStream_t s);
int launch_copy_to_host(const void* src, void* dst, int64_t bytes, int num_sms, cudaStream_t s);

bool small_m_supported(const sacq_layer* L);
// Kernel selector (5 = fp16 warp-MMA, 3 = CUDA-core) of the small-M variant that takes int8 activations.
int small_m_int8_selector(const sacq_layer* L);
int64_t small_m_workspace_bytes(const sacq_layer* L, int64_t M);
void small_m_scratch_need(const sacq_layer* L, int64_t M, int64_t* bytes, int64_t* counters);
// Further copies of a GEMM's output, written by the same epilogue: buffers of other GPUs of the
// node mapped into this process (plain peer stores over NVLink), same row pitch as y.
constexpr int kMaxBcast = 7;
struct BcastDst {
  void* ptr[kMaxBcast];
  int n;
};

// `residual` (bf16 [M, ldr], may be null) is added to the rounded output in every GEMM epilogue.
int launch_small_m(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                   void* ws, int64_t ws_bytes, cudaStream_t s, const void* residual = nullptr, int64_t ldr = 0,
                   int act_int8 = 0, const BcastDst* bc = nullptr);

int launch_small_m_multi(const sacq_layer* const* layers, int n, const void* q, const float* scale, int64_t M,
                         void* const* ys, const int64_t* ldys, cudaStream_t s);

bool large_m_supported(const sacq_layer* L);
int launch_large_m(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                   cudaStream_t s, const void* residual = nullptr, int64_t ldr = 0, const BcastDst* bc = nullptr);
int launch_large_m_multi(const sacq_layer* const* layers, int n, const void* q, const float* scale, int64_t M,
                         void* const* ys, const int64_t* ldys, cudaStream_t s);
void large_m_release(sacq_layer* L);

// Tensor-core kernel that keeps the expanded weights in tensor memory (linear_large_m_tmem.cu).
bool large_m_tmem_supported(const sacq_layer* L);
int large_m_tmem_pick_nt(const sacq_layer* L, int64_t M);
int launch_large_m_tmem(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                        cudaStream_t s, const void* residual = nullptr, int64_t ldr = 0, const BcastDst* bc = nullptr,
                        int nt_force = 0);

// Dense int8 x int8 -> int32 GEMM of the reference's deployed INT8 recipe (linear_dense_i8.cu).
bool dense_i8_supported(const sacq_layer* L);
int launch_dense_i8(const sacq_layer* L, const void* q, const float* act_scale, const void* wq, const float* w_scale,
                    int64_t M, void* y, int64_t ldy, cudaStream_t s, bool fp8 = false);

bool large_m_grouped_supported(const sacq_layer* L);
int64_t large_m_grouped_workspace_bytes(const sacq_layer* L, int64_t M);
int launch_large_m_grouped(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                           void* ws, int64_t ws_bytes, cudaStream_t s, const void* residual = nullptr,
                           int64_t ldr = 0, int act_int8 = 0, const BcastDst* bc = nullptr);

// Grouped-scale tensor-core kernel with the weights in tensor memory (linear_large_m_tmem_grouped.cu).
bool large_m_tmem_grouped_supported(const sacq_layer* L);
int64_t large_m_tmem_grouped_workspace_bytes(const sacq_layer* L, int64_t M);
int64_t large_m_tmem_grouped_min_m(const sacq_layer* L);
int launch_large_m_tmem_grouped(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                                void* ws, int64_t ws_bytes, cudaStream_t s, const void* residual = nullptr,
                                int64_t ldr = 0, int act_int8 = 0, const BcastDst* bc = nullptr, int nt_force = 0);

// ----------------------------------------------------------------------------
// device side
// ----------------------------------------------------------------------------

#ifdef SACQ_TRACE
// Profiling builds only (-DSACQ_TRACE): a timeline of kernel phases.  Block 0 of every traced kernel
// takes a slot (its launch order) and records %globaltimer at entry, after it has waited for its
// predecessor on the stream, when its staged operands have landed, and at exit.
struct TimelineEntry { long long kind, t_entry, t_dep, t_ready, t_exit, pad[3]; };
// (one buffer per translation unit: device symbols are not shared between them without
// relocatable device code; %globaltimer is, so the dumps merge by time)
static __device__ TimelineEntry g_timeline[512];
static __device__ unsigned g_timeline_count = 0;
#define SACQ_TL_DEFINE_DUMP(name)                                                                              \
  extern "C" SACQ_API int name(long long* out, int reset) {                                                    \
    unsigned n = 0;                                                                                            \
    if (cudaMemcpyFromSymbol(&n, g_timeline_count, sizeof(n)) != cudaSuccess) return -1;                       \
    if (out != nullptr && cudaMemcpyFromSymbol(out, g_timeline, sizeof(TimelineEntry) * 512) != cudaSuccess) return -1; \
    if (reset) { unsigned z = 0; cudaMemcpyToSymbol(g_timeline_count, &z, sizeof(z)); }                        \
    return (int)n;                                                                                             \
  }
__device__ __forceinline__ long long tl_now() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define SACQ_TL_BEGIN(kindv) int _tl = -1; if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) { _tl = (int)(atomicAdd(&g_timeline_count, 1u) & 511u); g_timeline[_tl].kind = (kindv); g_timeline[_tl].t_entry = tl_now(); }
#define SACQ_TL(field) do { if (_tl >= 0) g_timeline[_tl].field = tl_now(); } while (0)
#else
#define SACQ_TL_BEGIN(kindv) do { } while (0)
#define SACQ_TL(field) do { } while (0)
#endif

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// The reference reconstruction: bf16(bf16(c * s) + shift), two roundings
// (sacq/index_correction.py:104-106).  c*s is exact in fp32 (8-bit x 8-bit
// significands), so one RNE rounding gives torch's bf16 product.
__device__ __forceinline__ uint16_t reconstruct_bf16(uint32_t c_bits, float s, float shift) {
  float p = __bfloat162float(__float2bfloat16_rn(__fmul_rn(bf16_bits_to_float(c_bits), s)));
  return float_to_bf16_bits(__fadd_rn(p, shift));
}

// Two weights at once, packed (low half = first): the conversions are the paired instruction
// (cvt.rn.bf16x2.f32), which halves the load on the conversion pipe that bounds the reconstruction
// kernels.  Same bits as two reconstruct_bf16 calls.
__device__ __forceinline__ uint32_t reconstruct_bf16x2(uint32_t c0_bits, uint32_t c1_bits, float s, float shift) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(__fmul_rn(bf16_bits_to_float(c0_bits), s),
                                                 __fmul_rn(bf16_bits_to_float(c1_bits), s));
  const uint32_t pb = *reinterpret_cast<const uint32_t*>(&p);
  const __nv_bfloat162 w = __floats2bfloat162_rn(__fadd_rn(__uint_as_float(pb << 16), shift),
                                                 __fadd_rn(__uint_as_float(pb & 0xffff0000u), shift));
  return *reinterpret_cast<const uint32_t*>(&w);
}

// Two e4m3 bytes from two floats with RNE and saturation to +-448 (NaN stays NaN).
__device__ __forceinline__ uint32_t float2_to_e4m3x2(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}

// The reference's clamp(v, -448, 448) in front of an e4m3 conversion, where the conversion is
// float2_to_e4m3x2: cvt.rn.satfinite maps every |v| > 448 and both infinities to +-448 and keeps a NaN
// a NaN, exactly what the clamp followed by a plain conversion does, so nothing is left to compute
// (four instructions per element in kernels that are bound by instruction issue).
__device__ __forceinline__ float sat448(float v) { return v; }

// Running |v| maximum on bit patterns: among non-negative floats integer order is float order, infinity
// is above every finite value and every NaN above infinity, so a NaN (or an infinity) in a row survives
// the reduction the way it does in torch's amax, where fmaxf would drop it.
__device__ __forceinline__ uint32_t absmax_bits(uint32_t mx, float v) {
  const uint32_t b = __float_as_uint(v) & 0x7fffffffu;
  return b > mx ? b : mx;
}
__device__ __forceinline__ uint32_t warp_max_bits(uint32_t v) { return __reduce_max_sync(0xffffffffu, v); }

// Index `i` of a little-endian bit stream of `bits`-wide fields, read through
// aligned 32-bit words (bits <= 24).  `words` must be readable one word past
// the word holding the field's last bit.
__device__ __forceinline__ uint32_t extract_index(const uint32_t* __restrict__ words, int64_t i, int bits) {
  const int64_t p = i * bits;
  const int64_t w = p >> 5;
  const uint32_t off = (uint32_t)(p & 31);
  const uint32_t lo = __ldg(words + w);
  const uint32_t hi = __ldg(words + w + 1);
  return __funnelshift_r(lo, hi, off) & ((1u << bits) - 1u);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace sacq
