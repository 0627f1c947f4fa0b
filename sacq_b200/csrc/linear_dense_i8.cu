// The reference's 8-bit weight recipes as dense 8-bit work on the 5th-generation tensor cores.
// INT8 (the deployed one; FP8 below):
// The reference's deployed INT8 recipe as integer work on the 5th-generation tensor cores
// (sm_100a): per-token int8 activations x per-output-row int8 weights -> int32, then
//   y[m,n] = bf16( fma(sa[m], float(acc[m,n]) * sw[n], bias[n]) )        (bias given)
//   y[m,n] = bf16( sa[m] * (float(acc[m,n]) * sw[n]) )                   (no bias)
// -- weight scale first, then token scale, the bias inside one fused multiply-add
// (int8_small_m_gemm_20261028_r1.py:7-32, int8_ordered_epilogue_20261028_r1.py:11-22).
// Integer accumulation is exact, so the output bytes are a function of the operands alone:
// this path can be, and is tested to be, bit-identical to a CPU restatement of the recipe.
//
// Like the reference (perrow_a8_candidate_r3.py:52-63: "no persistent decoded weight cache")
// the int8 weight matrix is produced per call from the packed stream into the caller's
// workspace (decode_weight_int8_kernel, dequant.cu) and consumed by a plain dense GEMM.  A CTA
// computes 256 tokens x 256 weight rows:
//   warp 0 (one lane) : TMA producer: per 128-byte K block two 128-token activation tiles and one
//                       256-row weight tile, SWIZZLE_128B, no multicast; 3 stages of 64 KB;
//   warp 1 (one lane) : tcgen05.mma kind::i8, M128 x N256 x K32, into TWO int32 accumulators (one
//                       per token sub-tile, 2 x 256 = all 512 TMEM columns) that alternate
//                       instruction by instruction: consecutive MMAs into one accumulator wait
//                       for each other (about 100 ns per instruction against 65 ns of tensor work);
//   warps 2..17       : epilogue: TMEM lane quarter x token sub-tile x column half each.
// A last token tile of at most 128 tokens loads and multiplies one sub-tile only.
// Every mbarrier wait is bounded (status word + CTA-wide abort flag), as in the other
// tensor-core kernels.
//
// The FP8 recipe (`projection_format: fp8_e4m3fn`; a8_joint_pair_r1.py:374,
// perrow_a8_candidate_r3.py:56-69: per-token e4m3 activations x per-output-row e4m3 weights,
// torch._scaled_mm / cutlass_scaled_mm with fp32 accumulation and the same epilogue order) is the
// same kernel with kind::f8f6f4 instructions and fp32 accumulators (FP8 = true).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "umma.cuh"

namespace sacq {

namespace {

using namespace umma;

constexpr int kDBN = 256;                 // weight rows per tile = columns of one accumulator
constexpr int kDBK = 128;                 // bytes per K block
constexpr int kDSub = 2;                  // 128-token sub-tiles per CTA, one accumulator each
constexpr int kDStages = 3;
constexpr int kDTileA = kBM * kDBK;       // 16 KB: one sub-tile of activations
constexpr int kDTileB = kDBN * kDBK;      // 32 KB: the weight tile
constexpr int kDEpiWarps = 16;
constexpr int kDThreads = 64 + kDEpiWarps * 32;

struct DenseParams {
  const float* act_scale;       // [M]
  const float* w_scale;         // [N]
  const uint16_t* bias;         // bf16 [N] or null
  uint16_t* y;                  // bf16 [M, ldy]
  int64_t ldy;
  int* status;
  int M, N, K;
};

// kind::i8 instruction descriptor: int32 accumulate, A = B = signed 8-bit, both K-major.
__host__ __device__ constexpr uint32_t make_idesc_i8(int bn) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// FP8: e4m3 operands, fp32 accumulators (kind::f8f6f4); else int8 operands, int32 accumulators.
template <bool FP8>
__global__ void __launch_bounds__(kDThreads, 1)
dense_i8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ DenseParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  constexpr uint32_t kStageBytes = kDSub * kDTileA + kDTileB;       // 64 KB
  constexpr uint32_t kSwOff = kDStages * kStageBytes, kBiasOff = kSwOff + kDBN * 4, kBarOff = kBiasOff + kDBN * 4,
                     kMiscOff = kBarOff + 16 * 8;
  constexpr int FULL = 0, EMPTY = kDStages, ACC_FULL = 2 * kDStages;
  constexpr uint32_t kTmemCols = kDSub * kDBN;                      // 512
  const uint32_t bars = base + kBarOff;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kMiscOff + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kDBN, m0 = blockIdx.y * (kDSub * kBM);
  const int num_kb = (p.K + kDBK - 1) / kDBK;
  const int subs = (p.M - m0 > kBM) ? 2 : 1;        // token sub-tiles of this CTA that hold tokens

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDStages; ++i) {
      mbar_init(bar(FULL + i), 1);
      mbar_init(bar(EMPTY + i), 1);
    }
    mbar_init(bar(ACC_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int st = kb % kDStages;
        if (!mbar_wait(bar(EMPTY + st), ((kb / kDStages) & 1) ^ 1, abort_flag, p.status)) break;
        mbar_arrive_expect_tx(bar(FULL + st), (uint32_t)(subs * kDTileA + kDTileB));
        const uint32_t dst = base + st * kStageBytes;
        for (int t = 0; t < subs; ++t) tma_load_2d(dst + t * kDTileA, &tmap_a, kb * kDBK, m0 + t * kBM, bar(FULL + st));
        tma_load_2d(dst + kDSub * kDTileA, &tmap_b, kb * kDBK, n0, bar(FULL + st));
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t kIdesc = FP8 ? make_idesc(kDBN) : make_idesc_i8(kDBN);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int st = kb % kDStages;
        ok = mbar_wait(bar(FULL + st), (kb / kDStages) & 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint64_t a0_desc = make_smem_desc(base + st * kStageBytes);
        const uint64_t a1_desc = make_smem_desc(base + st * kStageBytes + kDTileA);
        const uint64_t b_desc = make_smem_desc(base + st * kStageBytes + kDSub * kDTileA);
#pragma unroll
        for (int ks = 0; ks < kDBK / 32; ++ks) {
          const uint64_t adv = (uint64_t)((ks * 32) >> 4);
          if constexpr (FP8) {
            umma_f8(tmem_base, a0_desc + adv, b_desc + adv, kIdesc, (kb | ks) != 0);
            if (subs == 2) umma_f8(tmem_base + kDBN, a1_desc + adv, b_desc + adv, kIdesc, (kb | ks) != 0);
          } else {
            umma_i8(tmem_base, a0_desc + adv, b_desc + adv, kIdesc, (kb | ks) != 0);
            if (subs == 2) umma_i8(tmem_base + kDBN, a1_desc + adv, b_desc + adv, kIdesc, (kb | ks) != 0);
          }
        }
        umma_commit(bar(EMPTY + st));
      }
      if (ok) umma_commit(bar(ACC_FULL));
    }
    __syncwarp();
  } else {
    const int et = threadIdx.x - 64;                  // 0..511
    {
      if (et < kDBN) {
        const int n = min(n0 + et, p.N - 1);
        reinterpret_cast<float*>(sm + kSwOff)[et] = __ldg(p.w_scale + n);
        reinterpret_cast<float*>(sm + kBiasOff)[et] = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kDEpiWarps * 32) : "memory");
    }
    const int ew = warp - 2;                          // 0..15
    const int quarter = warp & 3;                     // the TMEM lane quarter a warp may read is warp % 4
    const int sub = (ew >> 2) & 1, chalf = ew >> 3;   // every four consecutive warps cover the four quarters
    const int m = m0 + sub * kBM + quarter * 32 + lane;
    const float sa = m < p.M ? __ldg(p.act_scale + m) : 0.f;
    const bool ok = mbar_wait(bar(ACC_FULL), 0, abort_flag, p.status);   // tcgen05.ld below is per warp: no CTA-wide collective
    if (__all_sync(0xffffffffu, ok) && sub < subs) {
      tc_fence_after();
      const float* swp = reinterpret_cast<const float*>(sm + kSwOff);
      const float* bp = reinterpret_cast<const float*>(sm + kBiasOff);
      const bool has_bias = p.bias != nullptr;
#pragma unroll 1
      for (int cc = 0; cc < kDBN / 64; ++cc) {
        const int c0 = chalf * (kDBN / 2) + cc * 32;
        if (n0 + c0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(sub * kDBN + c0), r);
        if (m < p.M) {
          uint16_t* yrow = p.y + (int64_t)m * p.ldy + n0 + c0;
          // weight scale first, then the token scale; the bias rides in the same fused multiply-add
          auto fin = [&](int c) -> uint32_t {
            const float scaled = __fmul_rn(FP8 ? __uint_as_float(r[c]) : __int2float_rn((int)r[c]), swp[c0 + c]);
            const float v = has_bias ? fmaf(sa, scaled, bp[c0 + c]) : __fmul_rn(sa, scaled);
            return (uint32_t)float_to_bf16_bits(v);
          };
          const bool vec = (n0 + c0 + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(yrow) & 15) == 0);
          if (vec) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) o[j] = fin(v * 8 + 2 * j) | (fin(v * 8 + 2 * j + 1) << 16);
              *reinterpret_cast<uint4*>(yrow + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (n0 + c0 + c < p.N) yrow[c] = (uint16_t)fin(c);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

constexpr size_t kDenseSmem = kDStages * (kDSub * kDTileA + kDTileB) + 2 * kDBN * 4 + 16 * 8 + 64 + 1024;

}  // namespace

bool dense_i8_supported(const sacq_layer* L) { return L->d.in_features % 16 == 0 && L->d.in_features >= 16; }

// y = epilogue(q [M,K] int8 x wq [N,K] int8): the dense part of the INT8 recipe.
int launch_dense_i8(const sacq_layer* L, const void* q, const float* act_scale, const void* wq, const float* w_scale,
                    int64_t M, void* y, int64_t ldy, cudaStream_t s, bool fp8) {
  const sacq_layer_desc& d = L->d;
  if (M <= 0 || d.out_features == 0) return SACQ_OK;
  if (!dense_i8_supported(L))
    return set_error(SACQ_ERR_UNSUPPORTED, "the 8-bit GEMM needs in_features to be a multiple of 16, got %lld",
                     (long long)d.in_features);
  if (reinterpret_cast<uintptr_t>(q) % 16 != 0 || reinterpret_cast<uintptr_t>(wq) % 16 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "8-bit GEMM operands must be 16-byte aligned");
  if (!fp8 && (int64_t)d.in_features * 127 * 127 > 2147483647LL)
    return set_error(SACQ_ERR_UNSUPPORTED, "in_features=%lld could overflow the int32 accumulator", (long long)d.in_features);
  CUtensorMap ta, tb;
  int rc = encode_bytes_2d(&ta, q, (uint64_t)d.in_features, (uint64_t)M, (uint64_t)d.in_features, kDBK, kBM,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != SACQ_OK) return rc;
  rc = encode_bytes_2d(&tb, wq, (uint64_t)d.in_features, (uint64_t)d.out_features, (uint64_t)d.in_features, kDBK, kDBN,
                       CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != SACQ_OK) return rc;
  DenseParams p{};
  p.act_scale = act_scale;
  p.w_scale = w_scale;
  p.bias = static_cast<const uint16_t*>(d.bias);
  p.y = static_cast<uint16_t*>(y);
  p.ldy = ldy;
  p.status = L->d_status;
  p.M = (int)M; p.N = (int)d.out_features; p.K = (int)d.in_features;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    SACQ_CUDA_TRY(cudaFuncSetAttribute(dense_i8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDenseSmem));
    SACQ_CUDA_TRY(cudaFuncSetAttribute(dense_i8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDenseSmem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid((unsigned)((d.out_features + kDBN - 1) / kDBN), (unsigned)((M + kDSub * kBM - 1) / (kDSub * kBM)), 1);
  if (grid.y > 65535) return set_error(SACQ_ERR_UNSUPPORTED, "M=%lld exceeds the grid limit", (long long)M);
  if (fp8) dense_i8_kernel<true><<<grid, kDThreads, kDenseSmem, s>>>(ta, tb, p);
  else dense_i8_kernel<false><<<grid, kDThreads, kDenseSmem, s>>>(ta, tb, p);
  count_launch();
  SACQ_CUDA_TRY(cudaGetLastError());
  return SACQ_OK;
}

}  // namespace sacq
