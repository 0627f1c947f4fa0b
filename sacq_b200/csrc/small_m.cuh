// Shared declarations of the small-M quantized-linear kernels (CUDA-core and mma variants).
#pragma once

#include <math.h>
#include <string.h>

#include <type_traits>

#include "common.cuh"

namespace sacq {
namespace smallm {

constexpr int kSpanIdx = 32;   // indices a lane consumes per span
constexpr int kMaxWarps = 8;

struct SmallMParams {
  const uint8_t* packed;
  const __half* cb_f16;        // [C, D] scaled by 2^cb_exp_shift
  const uint8_t* cb_hilo;      // [C][2][D] e4m3 high/low halves scaled by 2^cb8_exp_shift (staged warp-MMA kernel)
  const uint16_t* cb_bf16;     // [C, d] original (generic kernel)
  const uint16_t* scales;      // bf16 [N, num_groups]
  const uint16_t* bias;        // bf16 [N] or null
  const uint8_t* q;            // e4m3 [M, K]
  int* status;                 // layer status word (bounded waits report here)
  const float* act_scale;      // [M]
  uint16_t* y;                 // bf16 [M, ldy]
  const uint16_t* residual;    // bf16 [M, ldr] added to the rounded output, or null
  int64_t ldr;
  float* partial;              // [num_sg][M][N] (only when num_sg > 1)
  int* counters;               // [chunks * row_blocks]
  int64_t ldy;
  int64_t row_bytes;           // bytes per packed row (fast kernel)
  int N, K, M;
  int vpr;                     // vectors per row
  int d, bits;
  int num_groups, group_size;
  int C;
  int span_idx;                // generic kernel: vectors per span
  int spans_per_row;           // vpr / span
  int spans_per_item;          // consecutive spans one item covers
  int num_sg;                  // span groups per row = ceil(spans_per_row / spans_per_item)
  int row_blocks;              // ceil(N / 32)
  int chunks;                  // ceil(M / MT)
  int act_bufs;                // staged warp-MMA kernel: activation tile buffers (1 or 2)
  int64_t num_items;
  float out_mul;               // 2^-cb_exp_shift (fast) or 1 (generic)
  float shift;
  int act_int8;                // activations are int8 (the deployed recipe) instead of e4m3
  int n_bc;                    // further copies of the output (peer GPUs' buffers), same pitch as y
  uint16_t* ybc[kMaxBcast];
};

// Up to four layers sharing one set of quantized activations in a single launch of the staged
// warp-MMA kernel.  `base` carries everything the layers have in common.
constexpr int kMaxMulti = 4;
struct MultiParams {
  SmallMParams base;
  int n_layers;
  int cta_begin[kMaxMulti + 1];
  const uint8_t* packed[kMaxMulti];
  const uint8_t* cb_hilo[kMaxMulti];
  const uint16_t* scales[kMaxMulti];
  const uint16_t* bias[kMaxMulti];
  int* status[kMaxMulti];
  uint16_t* y[kMaxMulti];
  int64_t ldy[kMaxMulti];
  int N[kMaxMulti];
  int row_blocks[kMaxMulti];
  float out_mul[kMaxMulti];
  float shift[kMaxMulti];
};

// Output store shared by every small-M variant: y = bf16(v), or bf16(bf16(v) + residual) --
// the two roundings of `linear(x) + residual` computed as two bf16 tensor operations.
__device__ __forceinline__ void store_out(const SmallMParams& p, int64_t m, int64_t n, float v) {
  uint16_t o = float_to_bf16_bits(v);
  if (p.residual != nullptr)
    o = float_to_bf16_bits(__fadd_rn(bf16_bits_to_float(o), bf16_bits_to_float(__ldg(p.residual + m * p.ldr + n))));
  p.y[m * p.ldy + n] = o;
  for (int i = 0; i < p.n_bc; ++i) p.ybc[i][m * p.ldy + n] = o;
}

__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// e4m3 x4 (one 32-bit word) -> 2 x half2, exact.
__device__ __forceinline__ void e4m3x4_to_h2(uint32_t v, uint32_t& lo, uint32_t& hi) {
  const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xffff), __NV_E4M3);
  const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v >> 16), __NV_E4M3);
  lo = (uint32_t)a.x | ((uint32_t)a.y << 16);
  hi = (uint32_t)b.x | ((uint32_t)b.y << 16);
}

// int8 x4 (one 32-bit word) -> 2 x half2, exact.
__device__ __forceinline__ void s8x4_to_h2(uint32_t v, uint32_t& lo, uint32_t& hi) {
  const __half2 a = __halves2half2(__int2half_rn((int)(int8_t)(v & 0xff)), __int2half_rn((int)(int8_t)((v >> 8) & 0xff)));
  const __half2 b = __halves2half2(__int2half_rn((int)(int8_t)((v >> 16) & 0xff)), __int2half_rn((int)(int8_t)(v >> 24)));
  lo = *reinterpret_cast<const uint32_t*>(&a);
  hi = *reinterpret_cast<const uint32_t*>(&b);
}
// Four activation bytes of either format -> 2 x half2.
__device__ __forceinline__ void act4_to_h2(int act_int8, uint32_t v, uint32_t& lo, uint32_t& hi) {
  if (act_int8) s8x4_to_h2(v, lo, hi); else e4m3x4_to_h2(v, lo, hi);
}

// 8 consecutive fields of BITS bits held in BITS/4 words.
template <int BITS>
__device__ __forceinline__ uint32_t field8(const uint32_t (&w)[BITS / 4], int j) {
  const int bit = j * BITS;
  const int word = bit >> 5;
  const int off = bit & 31;
  if (off + BITS <= 32) return (w[word] >> off) & ((1u << BITS) - 1u);
  return __funnelshift_r(w[word], w[word + 1 < BITS / 4 ? word + 1 : word], off) & ((1u << BITS) - 1u);
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

// Host-side launch plan shared by the variants.
struct Plan {
  bool fast;
  bool mma;                  // warp-MMA variant (16 tokens per item) instead of the CUDA-core one
  int D, BITS;
  bool cb_smem;
  int MT;
  int span_idx, spans_per_row, spans_per_item, num_sg, row_blocks, chunks;
  int64_t num_items;
  int warps, grid;
  int r8;                    // warp-MMA variant: 8-row sub-blocks per tile (1, 2, 4; staged kernel also 6)
  bool staged;               // warp-MMA variant with bulk-copied tiles in shared memory
  int act_bufs;              // ... and how many activation tile buffers fit (1 or 2)
  bool unpacked;             // warp-MMA variant that unpacks indices to 16 bits in shared memory
  size_t smem;
};


constexpr size_t kSmemBudget = 227 * 1024;

// Launches one instantiation; the opt-in to large dynamic shared memory is per function
// and device, so it is set on first use and remembered.
template <auto Kern>
cudaError_t launch_kernel(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  Kern<<<pl.grid, pl.warps * 32, pl.smem, s>>>(p);
  return cudaGetLastError();
}

// Same, with programmatic dependent launch: the grid may start while the previous kernel
// of the stream is still running; the kernel must execute griddepcontrol.wait before it
// touches anything that kernel produces.
template <auto Kern>
cudaError_t launch_kernel_pdl(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)pl.grid);
  cfg.blockDim = dim3((unsigned)(pl.warps * 32));
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, Kern, p);
}

// linear_small_m_mma.cu
cudaError_t launch_small_m_mma(const Plan& pl, const SmallMParams& p, cudaStream_t s);
cudaError_t launch_small_m_mma_multi(const Plan& pl, const MultiParams& g, cudaStream_t s);
// Warps that share one 32-index span in the staged warp-MMA kernel, by tile height: tiles of 8, 16 and
// 48 rows run two lighter warps per span, the 32-row tile one.  The order in which an output's partial
// sums are added depends on this number and on nothing else of the tile.
inline int staged_halves(int r8) { return (r8 <= 2 || r8 == 6) ? 2 : 1; }

// Shared memory the staged warp-MMA kernel needs for (layer, r8); 0 if it cannot run it.
size_t small_m_mma_staged_smem(int C, int D, int K, int64_t row_bytes, int r8, int warps, int act_bufs);

// linear_small_m_unpacked.cu
cudaError_t launch_small_m_mma_unpacked(const Plan& pl, const SmallMParams& p, cudaStream_t s);
size_t small_m_mma_unpacked_smem(int C, int D, int K, int64_t row_bytes, int num_groups, int r8, int warps);

}  // namespace smallm
}  // namespace sacq
