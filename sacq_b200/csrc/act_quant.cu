// Fused per-token FP8 activation quantizer.
//
// Restates quantize_rows(x, 'fp8_e4m3fn') of the reference
// (inference_acceleration_2026_10_11/a8_accuracy_recovery_2026_10_20_r1/
// perrow_a8_candidate_r3.py:17-25; zero-scale rule a8_rtn_r2.py:29-30):
//   z = float(x); s = max|z| / 448 per row, 1 for an all-zero row;
//   q = e4m3( clamp(z / s, -448, 448) )   with IEEE division and RNE conversion.
// The reference spends five elementwise torch kernels on this; here one launch reads
// the bf16 row once from HBM (second pass from registers), so the algorithmic traffic
// is 2 bytes read + 1 byte written per element.
#include "common.cuh"

namespace sacq {

namespace {

constexpr int kThreads = 256;
constexpr int kMaxChunksPerThread = 4;  // 16-byte chunks a thread keeps in registers: K <= 8192 stays on chip

// Two encoded values of one row -> two bytes.  I8: round-half-to-even to int8 in [-127, 127]
// (quantize_rows(x, 'int8_symmetric'), perrow_a8_candidate_r3.py:17-25); else e4m3.
template <bool I8>
__device__ __forceinline__ uint32_t encode2(float z0, float z1, float s) {
  if constexpr (I8) {
    // round-half-even of the clamped quotient through the add of 1.5 * 2^23 (exact for |q| <= 127):
    // keeps the float -> int conversion off the special-function pipe the division already loads
    const float qa = fminf(fmaxf(__fdiv_rn(z0, s), -127.f), 127.f);
    const float qb = fminf(fmaxf(__fdiv_rn(z1, s), -127.f), 127.f);
    const uint32_t a = (uint32_t)(__float_as_int(__fadd_rn(qa, 12582912.0f)) - 0x4B400000) & 0xffu;
    const uint32_t b = (uint32_t)(__float_as_int(__fadd_rn(qb, 12582912.0f)) - 0x4B400000) & 0xffu;
    return a | (b << 8);
  } else {
    return float2_to_e4m3x2(sat448(__fdiv_rn(z0, s)), sat448(__fdiv_rn(z1, s)));
  }
}

// One CTA per row.  VEC: rows are 16-byte aligned and K % 8 == 0.
template <bool VEC, bool I8 = false>
__global__ void __launch_bounds__(kThreads)
quant_act_fp8_kernel(const uint16_t* __restrict__ x, int64_t pitch, int64_t K, uint8_t* __restrict__ q,
                     float* __restrict__ scale_out) {
  __shared__ uint32_t red[kThreads / 32];
  __shared__ float s_scale;
  SACQ_TL_BEGIN(1);
  // A GEMM launched with programmatic stream serialization may start its prologue now; it
  // waits for this grid to finish before it reads q or the scales.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // This grid is itself launched that way behind whatever precedes it on the stream (so its
  // launch latency overlaps that kernel's tail): wait for it before touching x, q or the scales
  // (the kernel in front may have produced x, or may still be reading q).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  SACQ_TL(t_dep);
  const int64_t m = blockIdx.x;
  const uint16_t* row = x + m * pitch;
  uint8_t* qrow = q + m * K;
  const int tid = threadIdx.x;

  uint32_t mx = 0u;                                  // bit pattern of the running |x| maximum (absmax_bits)
  uint4 keep[kMaxChunksPerThread];
  const int64_t chunks = VEC ? (K >> 3) : 0;
  if constexpr (VEC) {
#pragma unroll
    for (int c = 0; c < kMaxChunksPerThread; ++c) {
      const int64_t ch = tid + (int64_t)c * kThreads;
      keep[c] = make_uint4(0, 0, 0, 0);
      if (ch < chunks) keep[c] = __ldg(reinterpret_cast<const uint4*>(row) + ch);
      const uint32_t w[4] = {keep[c].x, keep[c].y, keep[c].z, keep[c].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mx = absmax_bits(mx, bf16_bits_to_float(w[j] & 0xffff));
        mx = absmax_bits(mx, bf16_bits_to_float(w[j] >> 16));
      }
    }
    for (int64_t ch = tid + (int64_t)kMaxChunksPerThread * kThreads; ch < chunks; ch += kThreads) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(row) + ch);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mx = absmax_bits(mx, bf16_bits_to_float(w[j] & 0xffff));
        mx = absmax_bits(mx, bf16_bits_to_float(w[j] >> 16));
      }
    }
  } else {
    for (int64_t k = tid; k < K; k += kThreads) mx = absmax_bits(mx, bf16_bits_to_float(__ldg(row + k)));
  }
  mx = warp_max_bits(mx);
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid < 32) {
    const float v = __uint_as_float(warp_max_bits(tid < kThreads / 32 ? red[tid] : 0u));
    if (tid == 0) {
      // a NaN maximum fails `> 0` like in the reference's torch.where: the row keeps scale 1 and its
      // NaN elements stay NaN; an infinite maximum gives an infinite scale
      const float s = v > 0.f ? __fdiv_rn(v, I8 ? 127.0f : kE4M3Max) : 1.0f;
      s_scale = s;
      scale_out[m] = s;
    }
  }
  __syncthreads();
  const float s = s_scale;

  if constexpr (VEC) {
    auto emit = [&](const uint4& v, int64_t ch) {
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t a = encode2<I8>(bf16_bits_to_float(w[2 * j] & 0xffff), bf16_bits_to_float(w[2 * j] >> 16), s);
        const uint32_t b = encode2<I8>(bf16_bits_to_float(w[2 * j + 1] & 0xffff),
                                       bf16_bits_to_float(w[2 * j + 1] >> 16), s);
        o[j] = a | (b << 16);
      }
      *(reinterpret_cast<uint2*>(qrow) + ch) = make_uint2(o[0], o[1]);
    };
#pragma unroll
    for (int c = 0; c < kMaxChunksPerThread; ++c) {
      const int64_t ch = tid + (int64_t)c * kThreads;
      if (ch < chunks) emit(keep[c], ch);
    }
    for (int64_t ch = tid + (int64_t)kMaxChunksPerThread * kThreads; ch < chunks; ch += kThreads)
      emit(__ldg(reinterpret_cast<const uint4*>(row) + ch), ch);
  } else {
    for (int64_t k = tid; k < K; k += kThreads) {
      const float z = bf16_bits_to_float(__ldg(row + k));
      qrow[k] = (uint8_t)(encode2<I8>(z, 0.f, s) & 0xff);
    }
  }
  SACQ_TL(t_exit);
}

// The same quantizer for many rows: one WARP per row, eight rows per CTA, no block-wide barrier.  With
// one CTA per row (above) a row's two phases are separated by two __syncthreads and 8,192 rows of
// K = 2048 take 24 us against 8 us of HBM traffic; here a lane keeps its 16-byte chunks of the row
// in registers across the warp reduction: 8 chunks of 8 elements per lane, i.e. rows of up to 2,048
// elements.  Longer rows stay on the kernel above: keeping 24 chunks per lane costs 240 registers
// and measured 77 us for 8,192 rows of 6,144 (re-reading the tail instead: 59 us) against 44 us
// there.  Same arithmetic, same bytes.  Rows are 16-byte aligned, K % 8 == 0.
constexpr int kRowsPerCta = 8;
constexpr int kKeepChunks = 8;

template <bool I8>
__global__ void __launch_bounds__(kRowsPerCta * 32)
quant_act_rows_kernel(const uint16_t* __restrict__ x, int64_t pitch, int64_t M, int64_t K, uint8_t* __restrict__ q,
                      float* __restrict__ scale_out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t m = (int64_t)blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
  if (m >= M) return;
  const uint4* row = reinterpret_cast<const uint4*>(x + m * pitch);
  uint2* qrow = reinterpret_cast<uint2*>(q + m * K);
  const int64_t chunks = K >> 3;
  auto chunk_max = [](uint32_t mx, const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mx = absmax_bits(mx, bf16_bits_to_float(w[j] & 0xffff));
      mx = absmax_bits(mx, bf16_bits_to_float(w[j] >> 16));
    }
    return mx;
  };
  uint32_t mx = 0u;
  uint4 keep[kKeepChunks];
#pragma unroll
  for (int c = 0; c < kKeepChunks; ++c) {
    const int64_t ch = lane + (int64_t)c * 32;
    keep[c] = make_uint4(0, 0, 0, 0);
    if (ch < chunks) keep[c] = __ldg(row + ch);
    mx = chunk_max(mx, keep[c]);
  }
  for (int64_t ch = lane + (int64_t)kKeepChunks * 32; ch < chunks; ch += 32) mx = chunk_max(mx, __ldg(row + ch));
  const float v = __uint_as_float(warp_max_bits(mx));
  const float s = v > 0.f ? __fdiv_rn(v, I8 ? 127.0f : kE4M3Max) : 1.0f;   // a NaN maximum keeps scale 1, as above
  if (lane == 0) scale_out[m] = s;
  auto emit = [&](const uint4& c, int64_t ch) {
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
    uint32_t o[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t a = encode2<I8>(bf16_bits_to_float(w[2 * j] & 0xffff), bf16_bits_to_float(w[2 * j] >> 16), s);
      const uint32_t b = encode2<I8>(bf16_bits_to_float(w[2 * j + 1] & 0xffff), bf16_bits_to_float(w[2 * j + 1] >> 16), s);
      o[j] = a | (b << 16);
    }
    qrow[ch] = make_uint2(o[0], o[1]);
  };
#pragma unroll
  for (int c = 0; c < kKeepChunks; ++c) {
    const int64_t ch = lane + (int64_t)c * 32;
    if (ch < chunks) emit(keep[c], ch);
  }
  for (int64_t ch = lane + (int64_t)kKeepChunks * 32; ch < chunks; ch += 32) emit(__ldg(row + ch), ch);
}

constexpr int64_t kRowsKernelMinM = 256;   // from here on the per-row CTAs outnumber what the device holds at once
constexpr int64_t kRowsKernelMaxK = 256 * kKeepChunks;   // rows the lanes hold entirely in registers

template <bool I8>
cudaError_t launch_rows(const cudaLaunchConfig_t& cfg, const uint16_t* x, int64_t pitch, int64_t M, int64_t K, uint8_t* q,
                        float* scale) {
  return cudaLaunchKernelEx(&cfg, quant_act_rows_kernel<I8>, x, pitch, M, K, q, scale);
}

}  // namespace

#ifdef SACQ_TRACE
SACQ_TL_DEFINE_DUMP(sacq_debug_timeline_quant)
#endif

int launch_quant_act_int8(const void* x, int64_t pitch, int64_t M, int64_t K, void* q, float* scale,
                          cudaStream_t s) {
  if (M == 0 || K == 0) return SACQ_OK;
  const bool vec = (K % 8 == 0) && (pitch % 8 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(q) % 8 == 0);
  if (M > 2147483647LL) return set_error(SACQ_ERR_UNSUPPORTED, "M=%lld exceeds the grid limit", (long long)M);
  if (vec && M >= kRowsKernelMinM && K <= kRowsKernelMaxK) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((M + kRowsPerCta - 1) / kRowsPerCta));
    cfg.blockDim = dim3(kRowsPerCta * 32);
    cfg.stream = s;
    SACQ_CUDA_TRY(launch_rows<true>(cfg, static_cast<const uint16_t*>(x), pitch, M, K, static_cast<uint8_t*>(q), scale));
  } else if (vec)
    quant_act_fp8_kernel<true, true><<<(unsigned)M, kThreads, 0, s>>>(static_cast<const uint16_t*>(x), pitch, K,
                                                                     static_cast<uint8_t*>(q), scale);
  else
    quant_act_fp8_kernel<false, true><<<(unsigned)M, kThreads, 0, s>>>(static_cast<const uint16_t*>(x), pitch, K,
                                                                      static_cast<uint8_t*>(q), scale);
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  return SACQ_OK;
}

int launch_quant_act_fp8(const void* x, int64_t pitch, int64_t M, int64_t K, void* q, float* scale,
                         cudaStream_t s) {
  if (M == 0 || K == 0) return SACQ_OK;
  const bool vec = (K % 8 == 0) && (pitch % 8 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(q) % 8 == 0);
  if (M > 2147483647LL) return set_error(SACQ_ERR_UNSUPPORTED, "M=%lld exceeds the grid limit", (long long)M);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)M);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
  if (vec && M >= kRowsKernelMinM && K <= kRowsKernelMaxK) {
    cfg.gridDim = dim3((unsigned)((M + kRowsPerCta - 1) / kRowsPerCta));
    cfg.blockDim = dim3(kRowsPerCta * 32);
    SACQ_CUDA_TRY(launch_rows<false>(cfg, xp, pitch, M, K, qp, scale));
  } else if (vec)
    SACQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quant_act_fp8_kernel<true, false>, xp, pitch, K, qp, scale));
  else
    SACQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quant_act_fp8_kernel<false, false>, xp, pitch, K, qp, scale));
  count_launch();
  return SACQ_OK;
}

}  // namespace sacq

// ----------------------------------------------------------------------------
// Activation function fused into the quantizer.
//
// The MLP of a transformer block feeds its down projection with act(gate) * up (gated) or
// act(x); run as separate tensor operations that is two or three elementwise kernels and a
// round trip of the [M, K] intermediate before the quantizer reads it again.  Here one launch
// produces the e4m3 row and its scale directly; the intermediate is never written.  The
// arithmetic follows the tensor operations it replaces, rounding to bf16 where they do, so the
// bytes equal quantize_rows(silu(gate) * up) and quantize_rows(gelu(x)) (the reference fuses
// the same stage for its INT8 path, int8_swiglu_lookup_fusion_20261028_r1.py:9-21).
// ----------------------------------------------------------------------------
namespace sacq {

namespace {

__device__ __forceinline__ float round_bf16(float v) { return bf16_bits_to_float(float_to_bf16_bits(v)); }

// KIND 0: bf16(bf16(silu(a)) * b); KIND 1: bf16(gelu(a)), erf form;
// KIND 2: bf16(bf16(a * bf16(1 + b)) + c), the AdaLN modulation a * (1 + scale) + shift.
template <int KIND>
__device__ __forceinline__ float act_value(float a, float b, float c) {
  if constexpr (KIND == 0) {
    const float s = round_bf16(a / (1.0f + expf(-a)));
    return round_bf16(s * b);
  } else if constexpr (KIND == 1) {
    return round_bf16(a * 0.5f * (1.0f + erff(a * 0.70710678118654752440f)));
  } else {
    return round_bf16(round_bf16(a * round_bf16(1.0f + b)) + c);
  }
}

// VEC: every row of a, b, c and q is 16-byte (q: 8-byte) aligned and K % 8 == 0: 8 elements per
// load and store instead of one.
template <int KIND, bool VEC>
__global__ void __launch_bounds__(kThreads)
act_quant_fp8_kernel(const uint16_t* __restrict__ a, int64_t a_pitch, const uint16_t* __restrict__ b, int64_t b_pitch,
                     const uint16_t* __restrict__ c, int64_t K, uint8_t* __restrict__ q,
                     float* __restrict__ scale_out) {
  extern __shared__ __align__(16) uint16_t yrow[];    // the row's bf16 values, kept on chip between the passes
  __shared__ uint32_t red[kThreads / 32];
  __shared__ float s_scale;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // launched behind the producer of a / b with programmatic serialization
  const int64_t m = blockIdx.x;
  const uint16_t* arow = a + m * a_pitch;
  const uint16_t* brow = KIND == 1 ? nullptr : b + m * b_pitch;      // pitch 0: one vector for every row
  uint32_t mx = 0u;                                  // bit pattern of the running maximum (absmax_bits)
  if constexpr (VEC) {
    for (int64_t ch = threadIdx.x; ch < (K >> 3); ch += kThreads) {
      const uint4 a4 = __ldg(reinterpret_cast<const uint4*>(arow) + ch);
      uint4 b4 = make_uint4(0, 0, 0, 0), c4 = make_uint4(0, 0, 0, 0);
      if constexpr (KIND != 1) b4 = __ldg(reinterpret_cast<const uint4*>(brow) + ch);
      if constexpr (KIND == 2) c4 = __ldg(reinterpret_cast<const uint4*>(c) + ch);
      const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w}, bw[4] = {b4.x, b4.y, b4.z, b4.w},
                     cw[4] = {c4.x, c4.y, c4.z, c4.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float y0 = act_value<KIND>(bf16_bits_to_float(aw[j] & 0xffff), bf16_bits_to_float(bw[j] & 0xffff),
                                         bf16_bits_to_float(cw[j] & 0xffff));
        const float y1 = act_value<KIND>(bf16_bits_to_float(aw[j] >> 16), bf16_bits_to_float(bw[j] >> 16),
                                         bf16_bits_to_float(cw[j] >> 16));
        mx = absmax_bits(absmax_bits(mx, y0), y1);
        o[j] = (uint32_t)float_to_bf16_bits(y0) | ((uint32_t)float_to_bf16_bits(y1) << 16);
      }
      reinterpret_cast<uint4*>(yrow)[ch] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    for (int64_t k = threadIdx.x; k < K; k += kThreads) {
      const float av = bf16_bits_to_float(__ldg(arow + k));
      const float bv = KIND == 1 ? 0.f : bf16_bits_to_float(__ldg(brow + k));
      const float cv = KIND == 2 ? bf16_bits_to_float(__ldg(c + k)) : 0.f;
      const float y = act_value<KIND>(av, bv, cv);
      yrow[k] = float_to_bf16_bits(y);
      mx = absmax_bits(mx, y);
    }
  }
  mx = warp_max_bits(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x < 32) {
    const float v = __uint_as_float(warp_max_bits(threadIdx.x < kThreads / 32 ? red[threadIdx.x] : 0u));
    if (threadIdx.x == 0) {
      const float s = v > 0.f ? __fdiv_rn(v, kE4M3Max) : 1.0f;
      s_scale = s;
      scale_out[m] = s;
    }
  }
  __syncthreads();
  const float s = s_scale;
  uint8_t* qrow = q + m * K;
  if constexpr (VEC) {
    for (int64_t ch = threadIdx.x; ch < (K >> 3); ch += kThreads) {
      const uint4 y4 = reinterpret_cast<const uint4*>(yrow)[ch];
      const uint32_t w[4] = {y4.x, y4.y, y4.z, y4.w};
      uint32_t o[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t lo = float2_to_e4m3x2(sat448(__fdiv_rn(bf16_bits_to_float(w[2 * j] & 0xffff), s)),
                                             sat448(__fdiv_rn(bf16_bits_to_float(w[2 * j] >> 16), s)));
        const uint32_t hi = float2_to_e4m3x2(sat448(__fdiv_rn(bf16_bits_to_float(w[2 * j + 1] & 0xffff), s)),
                                             sat448(__fdiv_rn(bf16_bits_to_float(w[2 * j + 1] >> 16), s)));
        o[j] = lo | (hi << 16);
      }
      *(reinterpret_cast<uint2*>(qrow) + ch) = make_uint2(o[0], o[1]);
    }
  } else {
    for (int64_t k2 = 2 * (int64_t)threadIdx.x; k2 < K; k2 += 2 * kThreads) {
      const float y0 = bf16_bits_to_float(yrow[k2]);
      const float y1 = k2 + 1 < K ? bf16_bits_to_float(yrow[k2 + 1]) : 0.f;
      const uint32_t pair = float2_to_e4m3x2(sat448(__fdiv_rn(y0, s)), sat448(__fdiv_rn(y1, s)));
      if (k2 + 1 < K && (reinterpret_cast<uintptr_t>(qrow + k2) & 1) == 0)
        *reinterpret_cast<uint16_t*>(qrow + k2) = (uint16_t)pair;
      else {
        qrow[k2] = (uint8_t)(pair & 0xff);
        if (k2 + 1 < K) qrow[k2 + 1] = (uint8_t)(pair >> 8);
      }
    }
  }
}

}  // namespace

int launch_act_quant_fp8(int kind, const void* a, int64_t a_pitch, const void* b, int64_t b_pitch, const void* c,
                         int64_t M, int64_t K, void* q, float* scale, cudaStream_t s) {
  if (M == 0 || K == 0) return SACQ_OK;
  if (M > 2147483647LL) return set_error(SACQ_ERR_UNSUPPORTED, "M=%lld exceeds the grid limit", (long long)M);
  const size_t smem = (size_t)K * sizeof(uint16_t);
  if (smem > 200 * 1024) return set_error(SACQ_ERR_UNSUPPORTED, "K=%lld: a row does not fit shared memory", (long long)K);
  const bool vec = (K % 8 == 0) && (a_pitch % 8 == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(q) % 8 == 0) &&
                   (kind == 1 || ((kind == 2 || b_pitch % 8 == 0) && reinterpret_cast<uintptr_t>(b) % 16 == 0)) &&
                   (kind != 2 || reinterpret_cast<uintptr_t>(c) % 16 == 0);
  const void* fns[3][2] = {{(const void*)act_quant_fp8_kernel<0, false>, (const void*)act_quant_fp8_kernel<0, true>},
                           {(const void*)act_quant_fp8_kernel<1, false>, (const void*)act_quant_fp8_kernel<1, true>},
                           {(const void*)act_quant_fp8_kernel<2, false>, (const void*)act_quant_fp8_kernel<2, true>}};
  const void* fn = fns[kind][vec ? 1 : 0];
  static bool configured[3][2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[kind][vec ? 1 : 0][dev])) {
    const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
    if (dev >= 0 && dev < 64) configured[kind][vec ? 1 : 0][dev] = true;
  }
  const uint16_t* ap = static_cast<const uint16_t*>(a);
  const uint16_t* bp = kind == 1 ? nullptr : static_cast<const uint16_t*>(b);
  const uint16_t* cp = kind == 2 ? static_cast<const uint16_t*>(c) : nullptr;
  int64_t bpitch = kind == 0 ? b_pitch : 0;
  uint8_t* qp = static_cast<uint8_t*>(q);
  void* args[] = {&ap, &a_pitch, &bp, &bpitch, &cp, &K, &qp, &scale};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)M);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SACQ_CUDA_TRY(cudaLaunchKernelExC(&cfg, fn, args));
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  return SACQ_OK;
}

}  // namespace sacq

// ----------------------------------------------------------------------------
// LayerNorm (+ AdaLN modulation) fused into the quantizer.
//
// A pre-norm transformer block normalises its input only to feed quantized projections, so
// the normalised tensor need not exist in memory: one launch reads x once, keeps the row in
// shared memory, and emits the e4m3 row and its scale (the reference fuses this stage in
// codex_norm3_regpack_20261029_r1/kernel.cu and codex_adaln_sharedmax_20261029_r2/kernel.cu
// for its INT8 path).  Arithmetic: fp32 mean, fp32 centred variance (two passes over the
// on-chip row), rstd = 1 / sqrt(var + eps), y = bf16((x - mean) * rstd * gamma + beta),
// optionally the AdaLN modulation bf16(bf16(y * bf16(1 + s)) + t), then the quantizer.  The
// reduction order differs from a framework LayerNorm's, so y agrees with it to one bf16 ulp,
// not to the bit; the quantizer's bytes are exactly those of quantizing this kernel's own y.
// ----------------------------------------------------------------------------
namespace sacq {

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();                                   // red may still be read from the previous call
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) t += red[i];   // same order in every thread
  return t;
}

template <bool MOD>
__global__ void __launch_bounds__(kThreads)
layernorm_quant_fp8_kernel(const uint16_t* __restrict__ x, int64_t pitch, const uint16_t* __restrict__ gamma,
                           const uint16_t* __restrict__ beta, float eps, const uint16_t* __restrict__ mod_scale,
                           const uint16_t* __restrict__ mod_shift, int64_t K, uint16_t* __restrict__ y_out,
                           int64_t y_pitch, uint8_t* __restrict__ q, float* __restrict__ scale_out) {
  extern __shared__ __align__(16) float xrow[];       // the row in fp32, later its bf16 result in place
  __shared__ float red[kThreads / 32];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // launched behind the producer of x with programmatic serialization
  const int64_t m = blockIdx.x;
  const uint16_t* row = x + m * pitch;
  float sum = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += kThreads) {
    const float v = bf16_bits_to_float(__ldg(row + k));
    xrow[k] = v;
    sum += v;
  }
  const float mean = block_sum(sum, red) / (float)K;
  float sq = 0.f;
  for (int64_t k = threadIdx.x; k < K; k += kThreads) {
    const float dlt = xrow[k] - mean;
    sq += dlt * dlt;
  }
  const float var = block_sum(sq, red) / (float)K;
  const float rstd = 1.0f / sqrtf(var + eps);
  uint32_t mx = 0u;                                  // bit pattern of the running maximum (absmax_bits)
  for (int64_t k = threadIdx.x; k < K; k += kThreads) {
    float y = (xrow[k] - mean) * rstd;
    if (gamma != nullptr) y = y * bf16_bits_to_float(__ldg(gamma + k));
    if (beta != nullptr) y = y + bf16_bits_to_float(__ldg(beta + k));
    y = round_bf16(y);
    if constexpr (MOD)
      y = round_bf16(round_bf16(y * round_bf16(1.0f + bf16_bits_to_float(__ldg(mod_scale + k)))) +
                     bf16_bits_to_float(__ldg(mod_shift + k)));
    xrow[k] = y;
    if (y_out != nullptr) y_out[m * y_pitch + k] = float_to_bf16_bits(y);
    mx = absmax_bits(mx, y);
  }
  // absmax over the CTA (max is order-independent)
  mx = warp_max_bits(mx);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = __uint_as_float(mx);
  __syncthreads();
  uint32_t vb = 0u;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) vb = max(vb, __float_as_uint(red[i]));
  const float v = __uint_as_float(vb);
  const float s = v > 0.f ? __fdiv_rn(v, kE4M3Max) : 1.0f;
  if (threadIdx.x == 0) scale_out[m] = s;
  uint8_t* qrow = q + m * K;
  for (int64_t k = threadIdx.x; k < K; k += kThreads)
    qrow[k] = (uint8_t)(float2_to_e4m3x2(sat448(__fdiv_rn(xrow[k], s)), 0.f) & 0xff);
}

}  // namespace

int launch_layernorm_quant_fp8(const void* x, int64_t pitch, const void* gamma, const void* beta, float eps,
                               const void* mod_scale, const void* mod_shift, int64_t M, int64_t K, void* y_out,
                               int64_t y_pitch, void* q, float* scale, cudaStream_t s) {
  if (M == 0 || K == 0) return SACQ_OK;
  if (M > 2147483647LL) return set_error(SACQ_ERR_UNSUPPORTED, "M=%lld exceeds the grid limit", (long long)M);
  const size_t smem = (size_t)K * sizeof(float);
  if (smem > 200 * 1024) return set_error(SACQ_ERR_UNSUPPORTED, "K=%lld: a row does not fit shared memory", (long long)K);
  const bool mod = mod_scale != nullptr;
  const void* fn = mod ? (const void*)layernorm_quant_fp8_kernel<true> : (const void*)layernorm_quant_fp8_kernel<false>;
  static bool configured[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[mod][dev])) {
    const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
    if (dev >= 0 && dev < 64) configured[mod][dev] = true;
  }
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const uint16_t* gp = static_cast<const uint16_t*>(gamma);
  const uint16_t* bp = static_cast<const uint16_t*>(beta);
  const uint16_t* sp = static_cast<const uint16_t*>(mod_scale);
  const uint16_t* tp = static_cast<const uint16_t*>(mod_shift);
  uint16_t* yp = static_cast<uint16_t*>(y_out);
  uint8_t* qp = static_cast<uint8_t*>(q);
  void* args[] = {&xp, &pitch, &gp, &bp, &eps, &sp, &tp, &K, &yp, &y_pitch, &qp, &scale};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)M);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SACQ_CUDA_TRY(cudaLaunchKernelExC(&cfg, fn, args));
  count_launch();
  return SACQ_OK;
}

}  // namespace sacq
