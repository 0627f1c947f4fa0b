// Weight reconstruction kernels: packed indices -> bf16 weight (bit-exact with the
// reference), per-output-row FP8 weight producer, and the derived codebook tables.
//
// Reference behaviour restated here:
//   * cosmos_quant_shim.py:409-454 / sacq/index_correction.py:98-108 -- gather, bf16
//     multiply by the group scale, bf16 add of the shift;
//   * a8_accuracy_recovery_2026_10_20_r1/perrow_a8_candidate_r3.py:17-25,52-63 --
//     row scale = absmax/448 (1 for a zero row), bytes = e4m3(clamp(W / scale)).
//
// All three are HBM-bound streaming kernels: the packed stream is read once with
// coalesced word loads, codewords come from L1/L2 (the codebook is at most 1 MB),
// and the output is written with one 16-byte (d=8) or 8-byte (d=4) store per thread.
#include "common.cuh"

#include <math.h>
#include <string.h>

namespace sacq {

namespace {

template <int D>
struct VecStore;  // D bf16 values as one vector store
template <>
struct VecStore<8> { using T = uint4; };
template <>
struct VecStore<4> { using T = uint2; };
template <>
struct VecStore<2> { using T = uint32_t; };

template <int D>
__device__ __forceinline__ void load_codeword(const uint16_t* __restrict__ cb, uint32_t idx, uint32_t (&c)[D]) {
  if constexpr (D == 8) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(cb) + idx);
    c[0] = v.x & 0xffff; c[1] = v.x >> 16; c[2] = v.y & 0xffff; c[3] = v.y >> 16;
    c[4] = v.z & 0xffff; c[5] = v.z >> 16; c[6] = v.w & 0xffff; c[7] = v.w >> 16;
  } else if constexpr (D == 4) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(cb) + idx);
    c[0] = v.x & 0xffff; c[1] = v.x >> 16; c[2] = v.y & 0xffff; c[3] = v.y >> 16;
  } else if constexpr (D == 2) {
    const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(cb) + idx);
    c[0] = v & 0xffff; c[1] = v >> 16;
  }
}

// One thread reconstructs one d-vector.  D = 0 is the scalar path for any d.
template <int D>
__global__ void __launch_bounds__(256)
dequant_bf16_kernel(const uint32_t* __restrict__ words, const uint16_t* __restrict__ cb,
                    const uint16_t* __restrict__ scales, uint16_t* __restrict__ w_out, int64_t total_vectors,
                    int vpr, int d, int bits, int group_size, int num_groups, float shift) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vectors; i += stride) {
    const uint32_t idx = extract_index(words, i, bits);
    // 32-bit arithmetic where it fits: a 64-bit division costs several times the rest of the index math
    const int64_t n = total_vectors <= 0x7fffffffLL ? (int64_t)((uint32_t)i / (uint32_t)vpr) : i / vpr;
    const int v = (int)(i - n * vpr);
    const int g = num_groups == 1 ? 0 : (v * d) / group_size;     // one scale per row: no division
    const float s = bf16_bits_to_float(__ldg(scales + n * num_groups + g));
    if constexpr (D != 0) {
      uint32_t c[D];
      load_codeword<D>(cb, idx, c);
      uint32_t o[D / 2];
#pragma unroll
      for (int j = 0; j < D / 2; ++j) {
        o[j] = reconstruct_bf16x2(c[2 * j], c[2 * j + 1], s, shift);
      }
      typename VecStore<D>::T* dst = reinterpret_cast<typename VecStore<D>::T*>(w_out) + i;
      if constexpr (D == 8) *dst = make_uint4(o[0], o[1], o[2], o[3]);
      if constexpr (D == 4) *dst = make_uint2(o[0], o[1]);
      if constexpr (D == 2) *dst = o[0];
    } else {
      for (int j = 0; j < d; ++j)
        w_out[i * d + j] = reconstruct_bf16(__ldg(cb + (int64_t)idx * d + j), s, shift);
    }
  }
}

// One warp per output row: max |W[n,:]| / limit (448 for e4m3, 127 for int8).
__global__ void __launch_bounds__(256)
weight_row_scale_kernel(const uint32_t* __restrict__ words, const uint16_t* __restrict__ cb,
                        const uint16_t* __restrict__ scales, float* __restrict__ sw, int64_t N, int vpr, int d,
                        int bits, int group_size, int num_groups, float shift, float limit) {
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const int lane = threadIdx.x & 31;
  float m = 0.f;
  for (int v = lane; v < vpr; v += 32) {
    const uint32_t idx = extract_index(words, n * vpr + v, bits);
    const float s = bf16_bits_to_float(__ldg(scales + n * num_groups + (num_groups == 1 ? 0 : (v * d) / group_size)));
    for (int j = 0; j < d; ++j) {
      const uint16_t w = reconstruct_bf16(__ldg(cb + (int64_t)idx * d + j), s, shift);
      m = fmaxf(m, fabsf(bf16_bits_to_float(w)));
    }
  }
  m = warp_max(m);
  if (lane == 0) sw[n] = m > 0.f ? __fdiv_rn(m, limit) : 1.0f;
}

// One thread per d-vector: e4m3(clamp(W / sw[n])).
__global__ void __launch_bounds__(256)
decode_weight_fp8_kernel(const uint32_t* __restrict__ words, const uint16_t* __restrict__ cb,
                         const uint16_t* __restrict__ scales, const float* __restrict__ sw,
                         uint8_t* __restrict__ wq, int64_t total_vectors, int vpr, int d, int bits, int group_size,
                         int num_groups, float shift) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vectors; i += stride) {
    const uint32_t idx = extract_index(words, i, bits);
    // 32-bit arithmetic where it fits: a 64-bit division costs several times the rest of the index math
    const int64_t n = total_vectors <= 0x7fffffffLL ? (int64_t)((uint32_t)i / (uint32_t)vpr) : i / vpr;
    const int v = (int)(i - n * vpr);
    const float s = bf16_bits_to_float(__ldg(scales + n * num_groups + (num_groups == 1 ? 0 : (v * d) / group_size)));
    const float row = __ldg(sw + n);
    auto enc2 = [&](uint32_t pair_bits) -> uint32_t {           // two codeword elements (one bf16 pair) -> two bytes
      const uint32_t w = reconstruct_bf16x2(pair_bits & 0xffffu, pair_bits >> 16, s, shift);
      return float2_to_e4m3x2(sat448(__fdiv_rn(__uint_as_float(w << 16), row)),
                              sat448(__fdiv_rn(__uint_as_float(w & 0xffff0000u), row)));
    };
    if (d == 8 && ((reinterpret_cast<uintptr_t>(cb) & 15) == 0) && ((reinterpret_cast<uintptr_t>(wq) & 7) == 0)) {
      // one 16-byte codeword load, one 8-byte store
      const uint4 c = __ldg(reinterpret_cast<const uint4*>(cb) + idx);
      *reinterpret_cast<uint2*>(wq + i * 8) = make_uint2(enc2(c.x) | (enc2(c.y) << 16), enc2(c.z) | (enc2(c.w) << 16));
    } else if (d == 4 && ((reinterpret_cast<uintptr_t>(cb) & 7) == 0) && ((reinterpret_cast<uintptr_t>(wq) & 3) == 0)) {
      const uint2 c = __ldg(reinterpret_cast<const uint2*>(cb) + idx);
      *reinterpret_cast<uint32_t*>(wq + i * 4) = enc2(c.x) | (enc2(c.y) << 16);
    } else if ((d & 1) == 0) {
      for (int j = 0; j < d; j += 2) {
        const float a = bf16_bits_to_float(reconstruct_bf16(__ldg(cb + (int64_t)idx * d + j), s, shift));
        const float b = bf16_bits_to_float(reconstruct_bf16(__ldg(cb + (int64_t)idx * d + j + 1), s, shift));
        const uint32_t pr = float2_to_e4m3x2(sat448(__fdiv_rn(a, row)), sat448(__fdiv_rn(b, row)));
        wq[i * d + j] = (uint8_t)(pr & 0xff);
        wq[i * d + j + 1] = (uint8_t)(pr >> 8);
      }
    } else {
      for (int j = 0; j < d; ++j) {
        const float a = bf16_bits_to_float(reconstruct_bf16(__ldg(cb + (int64_t)idx * d + j), s, shift));
        wq[i * d + j] = (uint8_t)(float2_to_e4m3x2(sat448(__fdiv_rn(a, row)), 0.f) & 0xff);
      }
    }
  }
}

// One thread per d-vector: int8(round_half_even(clamp(W / sw[n], -127, 127))), the weight bytes
// of the reference's INT8 recipe (perrow_a8_candidate_r3.py:57-60; the conversion is the
// cvt.rni.sat.s8.f32 of int8_direct_integer_round_20261028_r1.py:6-9).
__global__ void __launch_bounds__(256)
decode_weight_int8_kernel(const uint32_t* __restrict__ words, const uint16_t* __restrict__ cb,
                          const uint16_t* __restrict__ scales, const float* __restrict__ sw,
                          int8_t* __restrict__ wq, int64_t total_vectors, int vpr, int d, int bits, int group_size,
                          int num_groups, float shift) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vectors; i += stride) {
    const uint32_t idx = extract_index(words, i, bits);
    // 32-bit arithmetic where it fits: a 64-bit division costs several times the rest of the index math
    const int64_t n = total_vectors <= 0x7fffffffLL ? (int64_t)((uint32_t)i / (uint32_t)vpr) : i / vpr;
    const int v = (int)(i - n * vpr);
    const float s = bf16_bits_to_float(__ldg(scales + n * num_groups + (num_groups == 1 ? 0 : (v * d) / group_size)));
    const float row = __ldg(sw + n);
    // round_half_even(clamp(a / row, +-127)) as a byte.  The rounding is the add of 1.5 * 2^23 (exact RNE for
    // |q| < 2^22; q is clamped to 127), which keeps the float -> int conversion off the conversion pipe that
    // bounds this kernel (ncu: 72 % busy with the reciprocal, two bf16 roundings and one F2I per weight).
    auto q_byte = [&](float a) -> uint32_t {
      const float q = fminf(fmaxf(__fdiv_rn(a, row), -127.f), 127.f);
      return (uint32_t)(__float_as_int(__fadd_rn(q, 12582912.0f)) - 0x4B400000) & 0xffu;
    };
    auto enc_bits = [&](uint32_t c_bits) -> uint32_t { return q_byte(bf16_bits_to_float(reconstruct_bf16(c_bits, s, shift))); };
    auto enc = [&](int j) -> uint32_t { return enc_bits(__ldg(cb + (int64_t)idx * d + j)); };
    auto enc2 = [&](uint32_t pair) -> uint32_t {                // one bf16 pair of the codeword -> two bytes
      const uint32_t w = reconstruct_bf16x2(pair & 0xffffu, pair >> 16, s, shift);
      return q_byte(__uint_as_float(w << 16)) | (q_byte(__uint_as_float(w & 0xffff0000u)) << 8);
    };
    auto enc4 = [&](uint32_t w0, uint32_t w1) -> uint32_t { return enc2(w0) | (enc2(w1) << 16); };
    if (d == 8 && ((reinterpret_cast<uintptr_t>(cb) & 15) == 0) && ((reinterpret_cast<uintptr_t>(wq) & 7) == 0)) {
      // one 16-byte codeword load, one 8-byte store
      const uint4 c = __ldg(reinterpret_cast<const uint4*>(cb) + idx);
      *reinterpret_cast<uint2*>(wq + i * 8) = make_uint2(enc4(c.x, c.y), enc4(c.z, c.w));
    } else if (d == 4 && ((reinterpret_cast<uintptr_t>(cb) & 7) == 0) && ((reinterpret_cast<uintptr_t>(wq) & 3) == 0)) {
      const uint2 c = __ldg(reinterpret_cast<const uint2*>(cb) + idx);
      *reinterpret_cast<uint32_t*>(wq + i * 4) = enc4(c.x, c.y);
    } else if ((d & 3) == 0 && ((reinterpret_cast<uintptr_t>(wq) & 3) == 0)) {
      for (int j = 0; j < d; j += 4)
        *reinterpret_cast<uint32_t*>(wq + i * d + j) = enc(j) | (enc(j + 1) << 8) | (enc(j + 2) << 16) | (enc(j + 3) << 24);
    } else {
      for (int j = 0; j < d; ++j) wq[i * d + j] = (int8_t)enc(j);
    }
  }
}

// ---- derived tables -------------------------------------------------------

__global__ void codebook_absmax_kernel(const uint16_t* __restrict__ cb, int64_t count, float* __restrict__ out) {
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = fabsf(bf16_bits_to_float(__ldg(cb + i)));
    if (v == v && v < 3.0e38f) m = fmaxf(m, v);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));  // m >= 0
}

// Largest index of the packed stream (a payload whose indices reach past the codebook would make
// every kernel read out of bounds; the reference's CPU gather raises IndexError for it).
__global__ void index_max_kernel(const uint32_t* __restrict__ words, int64_t count, int bits, unsigned* __restrict__ out) {
  unsigned m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    m = max(m, extract_index(words, i, bits));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out, m);
}

// cb_f16[i] = fp16(c * 2^e16); cb_hilo[c][0][j] = e4m3(c * 2^e8), cb_hilo[c][1][j] = e4m3(c*2^e8 - hi)
__global__ void build_tables_kernel(const uint16_t* __restrict__ cb, int64_t C, int d, float mul16, float mul8,
                                    __half* __restrict__ cb_f16, uint8_t* __restrict__ cb_hilo) {
  const int64_t count = C * d;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const float c = bf16_bits_to_float(__ldg(cb + i));
    cb_f16[i] = __float2half_rn(c * mul16);
    const float c8 = c * mul8;
    const uint32_t hi_b = float2_to_e4m3x2(sat448(c8), 0.f) & 0xff;
    const float hi = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)hi_b, __NV_E4M3)));
    const uint32_t lo_b = float2_to_e4m3x2(sat448(c8 - hi), 0.f) & 0xff;
    const int64_t cw = i / d;
    const int j = (int)(i - cw * d);
    cb_hilo[(cw * 2 + 0) * d + j] = (uint8_t)hi_b;
    cb_hilo[(cw * 2 + 1) * d + j] = (uint8_t)lo_b;
  }
}

inline int grid_for(int64_t items, int threads, int num_sms) {
  int64_t blocks = (items + threads - 1) / threads;
  const int64_t cap = (int64_t)num_sms * 8;  // grid-stride beyond 8 resident blocks per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace

static float host_bf16_to_float(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, sizeof(f));
  return f;
}

int launch_dequant_bf16(const sacq_layer* L, void* w_out, cudaStream_t s) {
  const sacq_layer_desc& d = L->d;
  const int64_t total = d.out_features * L->vectors_per_row;
  if (total == 0) return SACQ_OK;
  const float shift = host_bf16_to_float(d.shift_bf16);
  const uint32_t* words = static_cast<const uint32_t*>(d.packed);
  const uint16_t* cb = static_cast<const uint16_t*>(d.codebook);
  const uint16_t* sc = static_cast<const uint16_t*>(d.scales);
  uint16_t* out = static_cast<uint16_t*>(w_out);
  const int grid = grid_for(total, 256, L->num_sms);
  const int vd = d.vector_dim;
  const bool vec_ok = aligned(w_out, 2 * (size_t)vd) && aligned(d.codebook, 2 * (size_t)vd);
#define SACQ_DQ(DV)                                                                                              \
  dequant_bf16_kernel<DV><<<grid, 256, 0, s>>>(words, cb, sc, out, total, (int)L->vectors_per_row, vd,           \
                                               d.index_bits, d.group_size, (int)L->num_groups, shift)
  if (vd == 8 && vec_ok) SACQ_DQ(8);
  else if (vd == 4 && vec_ok) SACQ_DQ(4);
  else if (vd == 2 && vec_ok) SACQ_DQ(2);
  else SACQ_DQ(0);
#undef SACQ_DQ
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  return SACQ_OK;
}

int launch_weight_row_scale(const sacq_layer* L, float* sw, cudaStream_t s, float limit) {
  const sacq_layer_desc& d = L->d;
  if (d.out_features == 0) return SACQ_OK;
  const int warps = 8;
  const int grid = (int)((d.out_features + warps - 1) / warps);
  weight_row_scale_kernel<<<grid, warps * 32, 0, s>>>(
      static_cast<const uint32_t*>(d.packed), static_cast<const uint16_t*>(d.codebook),
      static_cast<const uint16_t*>(d.scales), sw, d.out_features, (int)L->vectors_per_row, d.vector_dim,
      d.index_bits, d.group_size, (int)L->num_groups, host_bf16_to_float(d.shift_bf16), limit);
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  return SACQ_OK;
}

int launch_decode_weight_int8(const sacq_layer* L, const float* sw, void* wq, cudaStream_t s) {
  const sacq_layer_desc& d = L->d;
  const int64_t total = d.out_features * L->vectors_per_row;
  if (total == 0) return SACQ_OK;
  decode_weight_int8_kernel<<<grid_for(total, 256, L->num_sms), 256, 0, s>>>(
      static_cast<const uint32_t*>(d.packed), static_cast<const uint16_t*>(d.codebook),
      static_cast<const uint16_t*>(d.scales), sw, static_cast<int8_t*>(wq), total, (int)L->vectors_per_row,
      d.vector_dim, d.index_bits, d.group_size, (int)L->num_groups, host_bf16_to_float(d.shift_bf16));
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  return SACQ_OK;
}

int launch_decode_weight_fp8(const sacq_layer* L, const float* sw, void* wq, cudaStream_t s) {
  const sacq_layer_desc& d = L->d;
  const int64_t total = d.out_features * L->vectors_per_row;
  if (total == 0) return SACQ_OK;
  decode_weight_fp8_kernel<<<grid_for(total, 256, L->num_sms), 256, 0, s>>>(
      static_cast<const uint32_t*>(d.packed), static_cast<const uint16_t*>(d.codebook),
      static_cast<const uint16_t*>(d.scales), sw, static_cast<uint8_t*>(wq), total, (int)L->vectors_per_row,
      d.vector_dim, d.index_bits, d.group_size, (int)L->num_groups, host_bf16_to_float(d.shift_bf16));
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  return SACQ_OK;
}

// Builds the fp16 and FP8 high/low copies of the codebook.  Both are scaled by a
// power of two so the largest |codeword| lands in (0.5, 1] (fp16) or (128, 256]
// (e4m3); the epilogues multiply the exponent back.  Synchronises: load-time only.
int launch_build_tables(sacq_layer* L, cudaStream_t s) {
  const sacq_layer_desc& d = L->d;
  const int64_t count = (int64_t)d.codebook_size * d.vector_dim;
  float* d_max = nullptr;
  SACQ_CUDA_TRY(cudaMalloc(&d_max, sizeof(float)));
  cudaError_t e = cudaMemsetAsync(d_max, 0, sizeof(float), s);
  // the tables hold an even number of entries (whole 16-byte units); the padding entry is zero
  const size_t padded = (size_t)L->cb_entries * d.vector_dim;
  if (e == cudaSuccess) e = cudaMemsetAsync(L->cb_f16, 0, padded * sizeof(__half), s);
  if (e == cudaSuccess) e = cudaMemsetAsync(L->cb_hilo, 0, padded * 2, s);
  if (e == cudaSuccess) {
    codebook_absmax_kernel<<<grid_for(count, 256, L->num_sms), 256, 0, s>>>(
        static_cast<const uint16_t*>(d.codebook), count, d_max);
    count_launch();
    e = cudaGetLastError();
  }
  float h_max = 0.f;
  if (e == cudaSuccess) e = cudaMemcpyAsync(&h_max, d_max, sizeof(float), cudaMemcpyDeviceToHost, s);
  // largest |scale|, for the power-of-two normalisation of the grouped tensor-core kernel
  float h_smax = 0.f;
  const int64_t n_scales = d.out_features * L->num_groups;
  if (e == cudaSuccess && n_scales > 0) {
    e = cudaMemsetAsync(d_max, 0, sizeof(float), s);
    if (e == cudaSuccess) {
      codebook_absmax_kernel<<<grid_for(n_scales, 256, L->num_sms), 256, 0, s>>>(
          static_cast<const uint16_t*>(d.scales), n_scales, d_max);
      count_launch();
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(&h_smax, d_max, sizeof(float), cudaMemcpyDeviceToHost, s);
  }
  // every index must address a codeword (only a codebook smaller than 2^bits leaves room for one that does not)
  unsigned h_imax = 0;
  const int64_t n_idx = d.out_features * L->vectors_per_row;
  const bool check_idx = n_idx > 0 && (int64_t)d.codebook_size < (1LL << d.index_bits);
  if (e == cudaSuccess && check_idx) {
    e = cudaMemsetAsync(d_max, 0, sizeof(float), s);
    if (e == cudaSuccess) {
      index_max_kernel<<<grid_for(n_idx, 256, L->num_sms), 256, 0, s>>>(static_cast<const uint32_t*>(d.packed), n_idx,
                                                                       d.index_bits, reinterpret_cast<unsigned*>(d_max));
      count_launch();
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(&h_imax, d_max, sizeof(unsigned), cudaMemcpyDeviceToHost, s);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaFree(d_max);
  if (e != cudaSuccess) return cuda_fail(e, "codebook absmax");
  if (check_idx && h_imax >= (unsigned)d.codebook_size)
    return set_error(SACQ_ERR_INVALID_ARGUMENT, "packed stream holds index %u but the codebook has %d entries", h_imax,
                     d.codebook_size);
  {
    int sx = 0;
    if (h_smax > 0.f) (void)frexpf(h_smax, &sx);
    L->sc_exp_shift = -sx;
  }
  int ex = 0;
  if (h_max > 0.f) {
    (void)frexpf(h_max, &ex);  // h_max = f * 2^ex, f in [0.5, 1)
  }
  L->cb_exp_shift = -ex;        // c * 2^-ex in [0.5, 1)
  L->cb8_exp_shift = 8 - ex;    // c * 2^(8-ex) in [128, 256)
  build_tables_kernel<<<grid_for(count, 256, L->num_sms), 256, 0, s>>>(
      static_cast<const uint16_t*>(d.codebook), d.codebook_size, d.vector_dim, ldexpf(1.f, L->cb_exp_shift),
      ldexpf(1.f, L->cb8_exp_shift), L->cb_f16, L->cb_hilo);
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  SACQ_CUDA_TRY(cudaStreamSynchronize(s));
  return SACQ_OK;
}

}  // namespace sacq
