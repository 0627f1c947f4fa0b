// Large-M quantized linear for GROUPED scales on the 5th-generation tensor cores (sm_100a):
//   y[m,n] = bf16( s[m] * (sum_k q[m,k] * cb[idx[n,k/d], k%d] * scale[n, k/G]) + bias[n] )
//
// The layouts the reference deployed (dim-4 vectors, one scale per 64 weights, 5- to 11-bit
// indices; gr00t_libero/acceleration/presets/FROZEN_DECODE_SELECTION.json) cannot use the
// FP8 high/low kernel of linear_large_m.cu: the scale changes inside the K loop, so it has
// to be folded into the B operand, and codeword x scale has 16 significant bits.  Here the
// expander warps write fp16(codeword x scale) -- 11 significant bits, finer than the bf16
// rounding of the reference's own reconstruction -- into the K-major, 128B-swizzled B tile
// and the tensor cores run kind::f16 (one MMA per K step instead of the FP8 pair: the same
// tensor time).  The A operand is the e4m3 activation matrix widened to fp16 (exact) by a
// small pre-pass into the caller's workspace, which also produces the per-token sums that a
// non-zero `shift` needs.
//
// Roles, pipeline, bounded waits and exit path are those of linear_large_m.cu:
//   warp 0: TMA producer (fp16 activation tiles, SWIZZLE_128B; packed index super-blocks of
//           128 indices per row = 16*bits bytes, always 16-byte aligned; no multicast)
//   warp 1: tcgen05.mma.kind::f16 issuer, accumulator in TMEM
//   warps 2..9: expanders (runtime index width), then the epilogue.
//
// Replaces, for M above a few dozen rows, the reference's per-forward decode kernel plus 8-bit
// GEMM on these layouts (perrow_int8_fused_decode_r1.py:12-88, perrow_a8_candidate_r3.py:56-69).
#include <math.h>

#include "common.cuh"
#include "umma.cuh"

namespace sacq {

namespace {

using namespace umma;

constexpr int kBKh = 64;                      // fp16 elements per K block: one 128-byte swizzle row
constexpr int kMaxStages = 8;                 // pipeline depth is chosen per launch from what fits
constexpr int kATile = kBM * 128;             // 16 KB
constexpr int kSbIdx = 128;                   // indices per row per index super-block
constexpr float kPreScale = 4096.f;           // keeps fp16(codeword x scale) far from the subnormals

struct GroupedParams {
  const __half* cb_f16;         // [C][D] codebook * 2^cb_exp_shift
  const uint16_t* scales;       // bf16 [N, num_groups]
  const uint16_t* bias;         // bf16 [N] or null
  const float* act_scale;       // [M]
  const float* xsum;            // [M] sum_k q[m,k] (read only when shift != 0)
  uint16_t* y;                  // bf16 [M, ldy]
  const uint16_t* residual;     // bf16 [M, ldr] added to the rounded output, or null
  int64_t ldr;
  int n_bc;                     // further copies of the output (peer GPUs' buffers), same pitch as y
  uint16_t* ybc[kMaxBcast];
  int* status;
  int64_t ldy;
  int M, N, K, C;
  int bits, num_groups, group_size;
  float scale_mul;              // 2^sc_exp_shift * kPreScale, applied to every scale
  float out_mul;                // 2^-(cb_exp_shift + sc_exp_shift) / kPreScale
  float shift;
  int stages;                   // pipeline depth, 2..kMaxStages
  int kbs;                      // K blocks (64 k each) per pipeline stage: 1, 2 or 4
};

struct GroupedLayout {
  uint32_t stage_off, stage_bytes, idx_off, idx_slot, cb_off, sc_off, bias_off, bar_off, misc_off, total;
};

__host__ __device__ inline GroupedLayout grouped_layout(int bn, int mt, int bits, int cb_bytes, int num_groups,
                                                        int stages, int kbs) {
  GroupedLayout L;
  L.stage_off = 0;
  L.stage_bytes = (uint32_t)(kbs * (mt * kATile + bn * 128));
  L.idx_off = stages * L.stage_bytes;
  L.idx_slot = (uint32_t)(bn * 16 * bits);
  L.cb_off = (L.idx_off + 2 * L.idx_slot + 16 + 127) & ~127u;          // + 16: the extractor reads one word ahead
  L.sc_off = L.cb_off + (uint32_t)((cb_bytes + 127) & ~127);
  L.bias_off = L.sc_off + (uint32_t)((bn * num_groups * 2 + 127) & ~127);   // bf16
  L.bar_off = L.bias_off + 128 * 4;
  L.misc_off = L.bar_off + 32 * 8;
  L.total = L.misc_off + 64;
  return L;
}

// e4m3 (or int8, I8) [M, K] -> fp16 [M, K] (exact) and xsum[m] = sum_k q[m, k]; one CTA per token row.
template <bool I8>
__global__ void __launch_bounds__(256) widen_act_kernel(const uint8_t* __restrict__ q, int64_t K,
                                                        __half* __restrict__ a16, float* __restrict__ xsum) {
  __shared__ float red[8];
  const int64_t m = blockIdx.x;
  const uint2* src = reinterpret_cast<const uint2*>(q + m * K);
  uint4* dst = reinterpret_cast<uint4*>(a16 + m * K);
  float sum = 0.f;
  for (int64_t i = threadIdx.x; i < (K >> 3); i += blockDim.x) {
    const uint2 v = __ldg(src + i);
    uint32_t w[4];
    const uint32_t in[2] = {v.x, v.y};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      __half h[4];
      if constexpr (I8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __int2half_rn((int)(int8_t)((in[j] >> (8 * e)) & 0xff));
      } else {
        const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(in[j] & 0xffff), __NV_E4M3);
        const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(in[j] >> 16), __NV_E4M3);
        h[0] = __ushort_as_half(a.x); h[1] = __ushort_as_half(a.y);
        h[2] = __ushort_as_half(b.x); h[3] = __ushort_as_half(b.y);
      }
      w[2 * j] = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
      w[2 * j + 1] = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
      sum += __half2float(h[0]) + __half2float(h[1]) + __half2float(h[2]) + __half2float(h[3]);
    }
    dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    xsum[m] = t;
  }
}

// D in {4, 8}; BN in {32, 64, 128} weight rows per CTA; MT in {1, 2} 128-token sub-tiles that
// share every expanded B tile.  grid = (ceil(N/BN), ceil(M/(128*MT))).  A pipeline stage holds
// p.kbs K blocks (of 64 k each): the per-stage barrier round trips cost several hundred cycles
// for every role, so few large stages beat many small ones.
template <int D, int BN, int MT>
__global__ void __launch_bounds__(kThreads, 1)
large_m_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_idx,
                       const GroupedParams p) {
  // the next kernel of the stream, if launched with programmatic serialization, may be scheduled
  // from here on (its launch latency overlaps this grid); it waits for this grid before it touches memory
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int IDX_PER_KB = kBKh / D;                // indices per row per K block
  constexpr int KB_PER_SB = kSbIdx / IDX_PER_KB;      // K blocks per index super-block
  constexpr int IPC = 8 / D;                          // indices per 16-byte chunk (8 weights)
  constexpr int PASSES = BN / 32;                     // the 8 expander warps cover 32 rows x 8 chunks at a time
  constexpr uint32_t kIdesc = make_idesc(BN);
  constexpr int B_TILE = BN * 128;
  using CwVec = typename std::conditional<D == 8, uint4, uint2>::type;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const int NST = p.stages, KBS = p.kbs;
  const GroupedLayout L = grouped_layout(BN, MT, p.bits, p.C * D * 2, p.num_groups, NST, KBS);
  const uint32_t a_bytes = (uint32_t)(KBS * MT * kATile);   // A part of a stage; the B tiles follow

  constexpr int A_FULL = 0, B_FULL = kMaxStages, EMPTY = 2 * kMaxStages, IDX_FULL = 3 * kMaxStages,
                IDX_EMPTY = 3 * kMaxStages + 2, ACC_FULL = 3 * kMaxStages + 4;
  const uint32_t bars = base + L.bar_off;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + L.misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + L.misc_off + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * (kBM * MT);
  const int num_it = p.K / (kBKh * KBS);              // pipeline iterations
  const int sb_bytes = 16 * p.bits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(bar(A_FULL + i), 1);
      mbar_init(bar(B_FULL + i), kExpanderThreads / 32);
      mbar_init(bar(EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(IDX_FULL + i), 1);
      mbar_init(bar(IDX_EMPTY + i), kExpanderThreads / 32);
    }
    mbar_init(bar(ACC_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_idx);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), (uint32_t)(BN * MT));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int st = 0;
      uint32_t ph = 0;                                 // stage index and phase, kept as counters
      for (int it = 0; it < num_it; ++it) {
        const int kb0 = it * KBS;
        if (kb0 % KB_PER_SB == 0) {
          const int sb = kb0 / KB_PER_SB, slot = sb & 1;
          if (!mbar_wait(bar(IDX_EMPTY + slot), ((sb >> 1) & 1) ^ 1, abort_flag, p.status)) break;
          mbar_arrive_expect_tx(bar(IDX_FULL + slot), (uint32_t)(BN * sb_bytes));
          tma_load_2d(base + L.idx_off + slot * L.idx_slot, &tmap_idx, sb * sb_bytes, n0, bar(IDX_FULL + slot));
        }
        if (!mbar_wait(bar(EMPTY + st), ph ^ 1, abort_flag, p.status)) break;
        mbar_arrive_expect_tx(bar(A_FULL + st), a_bytes);
        const uint32_t dst = base + L.stage_off + st * L.stage_bytes;
        for (int kk = 0; kk < KBS; ++kk)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            tma_load_2d(dst + (uint32_t)((kk * MT + mt) * kATile), &tmap_a, (kb0 + kk) * 128, m0 + mt * kBM,
                        bar(A_FULL + st));
        if (++st == NST) { st = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      for (int it = 0; it < num_it && ok; ++it) {
        ok = mbar_wait(bar(A_FULL + st), ph, abort_flag, p.status) &&
             mbar_wait(bar(B_FULL + st), ph, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = base + L.stage_off + st * L.stage_bytes;
        for (int kk = 0; kk < KBS; ++kk) {
          const uint64_t b_desc = make_smem_desc(a_addr + a_bytes + (uint32_t)(kk * B_TILE));
#pragma unroll
          for (int ks = 0; ks < kBKh / 16; ++ks) {
            const uint64_t adv = (uint64_t)((ks * 32) >> 4);     // 16 fp16 = 32 bytes per K step
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint64_t a_desc = make_smem_desc(a_addr + (uint32_t)((kk * MT + mt) * kATile));
              umma_f16(tmem_base + (uint32_t)(mt * BN), a_desc + adv, b_desc + adv, kIdesc, (it | kk | ks) != 0);
            }
          }
        }
        umma_commit(bar(EMPTY + st));
        if (++st == NST) { st = 0; ph ^= 1; }
      }
      if (ok) umma_commit(bar(ACC_FULL));
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ expanders, then epilogue
    const int et = threadIdx.x - 64;                 // 0..255
    {
      // fp16 codebook, the tile's scales (bf16, all groups) and biases
      const uint4* src = reinterpret_cast<const uint4*>(p.cb_f16);
      uint4* dst = reinterpret_cast<uint4*>(sm + L.cb_off);
      const int n16 = (p.C * D * 2) >> 4;
      for (int i = et; i < n16; i += kExpanderThreads) cp_async_16(dst + i, src + i);
      uint16_t* sc = reinterpret_cast<uint16_t*>(sm + L.sc_off);
      for (int i = et; i < BN * p.num_groups; i += kExpanderThreads) {
        const int r = i / p.num_groups, g = i - r * p.num_groups;
        const int n = min(n0 + r, p.N - 1);
        sc[i] = __ldg(p.scales + (int64_t)n * p.num_groups + g);
      }
      if (et < BN) {
        const int n = min(n0 + et, p.N - 1);
        reinterpret_cast<float*>(sm + L.bias_off)[et] = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
      }
      cp_async_wait_all();
      expander_barrier();
    }
    // Work item = one 16-byte chunk (8 weights) of one row: lanes 8r..8r+7 of a warp write the
    // 8 chunks of a row (conflict-free swizzled stores, neighbouring index fields), the 8 warps
    // cover 32 rows per pass.
    const CwVec* cbs = reinterpret_cast<const CwVec*>(sm + L.cb_off);
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(sm + L.sc_off);
    const uint32_t mask = (1u << p.bits) - 1u;
    const int kb_per_group = p.group_size / kBKh;
    const int chunk = lane & 7;
    const int row_in_pass = (warp - 2) * 4 + (lane >> 3);
    bool ok = true;
    int st = 0, grp = 0, left_in_group = kb_per_group;
    uint32_t ph = 0;
    for (int it = 0; it < num_it && ok; ++it) {
      const int kb0 = it * KBS;
      const int sb = kb0 / KB_PER_SB, slot = sb & 1;
      ok = mbar_wait(bar(IDX_FULL + slot), (sb >> 1) & 1, abort_flag, p.status) &&
           mbar_wait(bar(EMPTY + st), ph ^ 1, abort_flag, p.status);
      if (!ok) break;
      const uint8_t* idx_slot = sm + L.idx_off + slot * L.idx_slot;
      uint8_t* b_stage = sm + L.stage_off + st * L.stage_bytes + a_bytes;
      for (int kk = 0; kk < KBS; ++kk) {
        const int first = ((kb0 + kk) % KB_PER_SB) * IDX_PER_KB + chunk * IPC;   // this lane's first index
#pragma unroll
        for (int ps = 0; ps < PASSES; ++ps) {
          const int row = ps * 32 + row_in_pass;
          // scale * 2^sc_exp_shift * 4096 is a bf16 significand with a small exponent: exact in fp16
          const __half sh = __float2half_rn(bf16_bits_to_float(sc[row * p.num_groups + grp]) * p.scale_mul);
          const __half2 s2 = __half2half2(sh);
          const uint32_t* w32 = reinterpret_cast<const uint32_t*>(idx_slot + row * sb_bytes);
          uint32_t o[4];
          // the chunk's one or two index fields sit in one 64-bit window of the row's bit stream
          const int bit0 = first * p.bits;
          const uint64_t win = (((uint64_t)w32[(bit0 >> 5) + 1] << 32) | w32[bit0 >> 5]) >> (bit0 & 31);
#pragma unroll
          for (int j = 0; j < IPC; ++j) {
            const uint32_t idx = (uint32_t)(win >> (j * p.bits)) & mask;
            const CwVec cw = cbs[idx];
            if constexpr (D == 8) {
              const uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&w4[e]), s2);
                o[e] = *reinterpret_cast<const uint32_t*>(&h);
              }
            } else {
              const uint32_t w2[2] = {cw.x, cw.y};
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&w2[e]), s2);
                o[2 * j + e] = *reinterpret_cast<const uint32_t*>(&h);
              }
            }
          }
          *reinterpret_cast<uint4*>(b_stage + kk * B_TILE + row * 128 + ((chunk ^ (row & 7)) * 16)) =
              make_uint4(o[0], o[1], o[2], o[3]);
        }
        if (--left_in_group == 0) { ++grp; left_in_group = kb_per_group; }
      }
      fence_proxy_async();                            // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(B_FULL + st));
        if ((kb0 + KBS) % KB_PER_SB == 0 || it == num_it - 1) mbar_arrive(bar(IDX_EMPTY + slot));
      }
      if (++st == NST) { st = 0; ph ^= 1; }
    }

    // ---- epilogue: this warp's TMEM lane quarter, half of the 32-column groups
    // the token scales of this warp's rows are fetched before the wait for the accumulator, so
    // their global-memory latency is off the critical path
    float sa_pre[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m = m0 + mt * kBM + (warp & 3) * 32 + lane;
      sa_pre[mt] = m < p.M ? __ldg(p.act_scale + m) : 0.f;
    }
    if (ok) ok = mbar_wait(bar(ACC_FULL), 0, abort_flag, p.status);
    ok = expander_all(ok);                            // uniform over the expanders: tcgen05.ld and the staging barriers are collective
    if (ok) {
      tc_fence_after();
      const int quarter = warp & 3;
      const int col_half = (warp - 2) >> 2;
      const float* bp = reinterpret_cast<const float*>(sm + L.bias_off);
      // staged through shared memory (the pipeline stages are idle now): whole row segments per store
      constexpr int SP = BN * 2 + 16;
      uint8_t* stg = sm + L.stage_off;
      if (p.n_bc == 0) {
        // one GPU: every thread stores its own 64-byte row pieces (measured 2-10 % faster than staging)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int m = m0 + mt * kBM + quarter * 32 + lane;
          const float sa = sa_pre[mt];
          const float add = (m < p.M && p.shift != 0.f) ? p.shift * __ldg(p.xsum + m) : 0.f;
#pragma unroll
          for (int cc = col_half; cc < BN / 32; cc += 2) {
            const int c0 = cc * 32;
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BN + c0), r);
            if (m < p.M) {
              uint16_t* yrow = p.y + (int64_t)m * p.ldy + n0 + c0;
              const uint16_t* rrow = p.residual ? p.residual + (int64_t)m * p.ldr + n0 + c0 : nullptr;
              // bf16(v), or bf16(bf16(v) + residual): the two roundings of `linear(x) + residual`
              auto fin = [&](float v, int c) -> uint32_t {
                uint16_t o = float_to_bf16_bits(v);
                if (rrow != nullptr)
                  o = float_to_bf16_bits(__fadd_rn(bf16_bits_to_float(o), bf16_bits_to_float(__ldg(rrow + c))));
                return (uint32_t)o;
              };
              const bool vec = (n0 + c0 + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(yrow) & 15) == 0);
              if (vec) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  uint32_t o[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const int c = v * 8 + 2 * j;
                    const float y0 = fmaf(sa, fmaf(__uint_as_float(r[c]), p.out_mul, add), bp[c0 + c]);
                    const float y1 = fmaf(sa, fmaf(__uint_as_float(r[c + 1]), p.out_mul, add), bp[c0 + c + 1]);
                    o[j] = fin(y0, c) | (fin(y1, c + 1) << 16);
                  }
                  *reinterpret_cast<uint4*>(yrow + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                }
              } else {
#pragma unroll
                for (int c = 0; c < 32; ++c)
                  if (n0 + c0 + c < p.N)
                    yrow[c] = (uint16_t)fin(fmaf(sa, fmaf(__uint_as_float(r[c]), p.out_mul, add), bp[c0 + c]), c);
              }
            }
          }
        }
      } else {
        // further copies on peer GPUs: stage the tile, then store whole row segments everywhere
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int m = m0 + mt * kBM + quarter * 32 + lane;
          const float sa = sa_pre[mt];
          const float add = (m < p.M && p.shift != 0.f) ? p.shift * __ldg(p.xsum + m) : 0.f;
          uint8_t* srow = stg + (quarter * 32 + lane) * SP;
#pragma unroll
          for (int cc = col_half; cc < BN / 32; cc += 2) {
            const int c0 = cc * 32;
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BN + c0), r);
            const uint16_t* rrow = (p.residual && m < p.M) ? p.residual + (int64_t)m * p.ldr + n0 + c0 : nullptr;
            // bf16(v), or bf16(bf16(v) + residual): the two roundings of `linear(x) + residual`
            auto fin = [&](float v, int c) -> uint32_t {
              uint16_t o = float_to_bf16_bits(v);
              if (rrow != nullptr && n0 + c0 + c < p.N)
                o = float_to_bf16_bits(__fadd_rn(bf16_bits_to_float(o), bf16_bits_to_float(__ldg(rrow + c))));
              return (uint32_t)o;
            };
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int c = v * 8 + 2 * j;
                const float y0 = fmaf(sa, fmaf(__uint_as_float(r[c]), p.out_mul, add), bp[c0 + c]);
                const float y1 = fmaf(sa, fmaf(__uint_as_float(r[c + 1]), p.out_mul, add), bp[c0 + c + 1]);
                o[j] = fin(y0, c) | (fin(y1, c + 1) << 16);
              }
              *reinterpret_cast<uint4*>(srow + (c0 + v * 8) * 2) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
          expander_barrier();                             // the tile is staged
          store_staged_tile<BN>(stg, SP, et, m0 + mt * kBM, p.M, n0, p.N, p.y, p.ldy, p.ybc, p.n_bc);
          expander_barrier();                             // before the next sub-tile reuses the staging rows
        }
      }
    }
  }

  // ---- common exit: every thread arrives here, also after an aborted wait
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)(BN * MT));
}

template <int D, int BN, int MT>
cudaError_t launch_inst(const CUtensorMap& ta, const CUtensorMap& ti, const GroupedParams& p, dim3 grid, size_t smem,
                        cudaStream_t s) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(large_m_grouped_kernel<D, BN, MT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  large_m_grouped_kernel<D, BN, MT><<<grid, kThreads, smem, s>>>(ta, ti, p);
  return cudaGetLastError();
}

template <int D>
cudaError_t launch_d(const CUtensorMap& ta, const CUtensorMap& ti, const GroupedParams& p, int bn, int mt, dim3 grid,
                     size_t smem, cudaStream_t s) {
  if (mt == 2) {
    if (bn == 32) return launch_inst<D, 32, 2>(ta, ti, p, grid, smem, s);
    if (bn == 64) return launch_inst<D, 64, 2>(ta, ti, p, grid, smem, s);
    return launch_inst<D, 128, 2>(ta, ti, p, grid, smem, s);
  }
  if (bn == 32) return launch_inst<D, 32, 1>(ta, ti, p, grid, smem, s);
  if (bn == 64) return launch_inst<D, 64, 1>(ta, ti, p, grid, smem, s);
  return launch_inst<D, 128, 1>(ta, ti, p, grid, smem, s);
}

size_t grouped_smem(const sacq_layer* L, int bn, int mt, int stages, int kbs) {
  return grouped_layout(bn, mt, L->d.index_bits, L->cb_entries * L->d.vector_dim * 2, (int)L->num_groups,
                        stages, kbs).total + 1024;
}

// Deepest pipeline (2..kMaxStages) that fits shared memory, 0 if not even two stages do.  A
// K block is only 128 bytes of K per row, so at small M the loop is bound by the latency of
// the TMA -> expand -> MMA -> release round trip divided by the depth.
int grouped_stages_for(const sacq_layer* L, int bn, int mt, int kbs) {
  for (int st = kMaxStages; st >= 2; --st)
    if (grouped_smem(L, bn, mt, st, kbs) <= 227 * 1024) return st;
  return 0;
}

// K blocks per stage: as many (4, 2, 1) as divide K/64 and still leave three stages.
int grouped_kbs_for(const sacq_layer* L, int bn, int mt) {
  const int64_t num_kb = L->d.in_features / kBKh;
  for (int kbs = 4; kbs > 1; kbs >>= 1)
    if (num_kb % kbs == 0 && grouped_stages_for(L, bn, mt, kbs) >= 3) return kbs;
  return 1;
}

constexpr int64_t kSlabTokens = 1024;   // tokens widened per launch: bounds the fp16 scratch

}  // namespace

bool large_m_grouped_supported(const sacq_layer* L) {
  const sacq_layer_desc& d = L->d;
  if (d.vector_dim != 8 && d.vector_dim != 4) return false;
  if (d.index_bits < 1 || d.index_bits > 16) return false;
  if (!L->rows_16b_aligned) return false;
  if (d.in_features % kBKh != 0 || d.group_size % kBKh != 0) return false;
  if (((size_t)L->cb_entries * d.vector_dim * 2) % 16 != 0) return false;
  if (has_shift(L)) return false;
  return grouped_stages_for(L, 32, 1, 1) >= 2;
}

// Workspace behind the counter region: fp16 activations of one token slab and their row sums.
int64_t large_m_grouped_workspace_bytes(const sacq_layer* L, int64_t M) {
  const int64_t rows = M < kSlabTokens ? M : kSlabTokens;
  return ((rows * L->d.in_features * 2 + 255) & ~(int64_t)255) + ((rows * 4 + 255) & ~(int64_t)255);
}

int launch_large_m_grouped(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                           void* ws, int64_t ws_bytes, cudaStream_t s, const void* residual, int64_t ldr,
                           int act_int8, const BcastDst* bc) {
  const sacq_layer_desc& d = L->d;
  if (!large_m_grouped_supported(L))
    return set_error(SACQ_ERR_UNSUPPORTED, "grouped tensor-core kernel cannot run this layer geometry");
  if (M <= 0 || d.out_features == 0) return SACQ_OK;
  if (reinterpret_cast<uintptr_t>(q) % 8 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "quantized activations must be 8-byte aligned");
  const int64_t need = large_m_grouped_workspace_bytes(L, M);
  if (ws == nullptr || ws_bytes < need)
    return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed behind the counter region, %lld given",
                     (long long)need, (long long)ws_bytes);
  if (reinterpret_cast<uintptr_t>(ws) % 256 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  const int64_t K = d.in_features, N = d.out_features;
  const int64_t slab = M < kSlabTokens ? M : kSlabTokens;
  __half* a16 = static_cast<__half*>(ws);
  float* xsum = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + ((slab * K * 2 + 255) & ~(int64_t)255));

  GroupedParams p{};
  p.cb_f16 = L->cb_f16;
  p.scales = static_cast<const uint16_t*>(d.scales);
  p.bias = static_cast<const uint16_t*>(d.bias);
  p.status = L->d_status;
  p.ldy = ldy;
  p.N = (int)N; p.K = (int)K; p.C = L->cb_entries;
  p.bits = d.index_bits; p.num_groups = (int)L->num_groups; p.group_size = d.group_size;
  p.scale_mul = ldexpf(kPreScale, L->sc_exp_shift);
  p.out_mul = ldexpf(1.f / kPreScale, -(L->cb_exp_shift + L->sc_exp_shift));
  const uint32_t sb = (uint32_t)d.shift_bf16 << 16;
  memcpy(&p.shift, &sb, sizeof(float));
  p.xsum = xsum;

  for (int64_t m0 = 0; m0 < M; m0 += slab) {
    const int64_t rows = (M - m0) < slab ? (M - m0) : slab;
    if (act_int8)
      widen_act_kernel<true><<<(unsigned)rows, 256, 0, s>>>(static_cast<const uint8_t*>(q) + m0 * K, K, a16, xsum);
    else
      widen_act_kernel<false><<<(unsigned)rows, 256, 0, s>>>(static_cast<const uint8_t*>(q) + m0 * K, K, a16, xsum);
    count_launch();
    SACQ_CUDA_TRY(cudaGetLastError());
    // Tile shape: (token sub-tiles per CTA, weight rows per CTA) with the smallest
    // waves x time-per-CTA, where the time per CTA was fitted to measurements at K = 2048:
    // about 1.2 us fixed + 7.8 us per token sub-tile (MMA issue, bound by the operand reads of
    // the A tile) + 0.17 us per weight row (expansion); all three scale with K alike.
    int mt = 1, bn = 0;
    double best = 1e30;
    for (int cand_mt = 1; cand_mt <= (rows > kBM ? 2 : 1); ++cand_mt) {
      const int64_t m_tiles_c = (rows + kBM * cand_mt - 1) / (kBM * cand_mt);
      for (int cand = 128; cand >= 32; cand >>= 1) {
        if (grouped_stages_for(L, cand, cand_mt, 1) < 2) continue;
        const int64_t tiles = ((N + cand - 1) / cand) * m_tiles_c;
        const int64_t waves = (tiles + L->num_sms - 1) / L->num_sms;
        const double cost = (double)waves * (1.2 + 7.8 * cand_mt + 0.169 * cand);
        if (cost < best - 1e-9) { best = cost; bn = cand; mt = cand_mt; }
      }
    }
    const int64_t m_tiles = (rows + kBM * mt - 1) / (kBM * mt);
    if (bn == 0) return set_error(SACQ_ERR_UNSUPPORTED, "grouped tensor-core kernel: no tile fits shared memory");
    CUtensorMap ta, ti;
    int rc = encode_bytes_2d(&ta, a16, (uint64_t)(K * 2), (uint64_t)rows, (uint64_t)(K * 2), 128, kBM,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SACQ_OK) return rc;
    const uint64_t row_bytes = (uint64_t)(L->row_bits / 8);
    rc = encode_bytes_2d(&ti, d.packed, row_bytes, (uint64_t)N, row_bytes, (uint32_t)(16 * d.index_bits),
                         (uint32_t)bn, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != SACQ_OK) return rc;
    p.act_scale = scale + m0;
    p.y = static_cast<uint16_t*>(y) + m0 * ldy;
    p.residual = residual ? static_cast<const uint16_t*>(residual) + m0 * ldr : nullptr;
    p.ldr = ldr;
    p.n_bc = bc ? bc->n : 0;
    for (int i = 0; i < p.n_bc; ++i) p.ybc[i] = static_cast<uint16_t*>(bc->ptr[i]) + m0 * ldy;
    p.M = (int)rows;
    const dim3 grid((unsigned)((N + bn - 1) / bn), (unsigned)m_tiles);
    p.kbs = grouped_kbs_for(L, bn, mt);
    p.stages = grouped_stages_for(L, bn, mt, p.kbs);
    const size_t smem = grouped_smem(L, bn, mt, p.stages, p.kbs);
    const cudaError_t e = d.vector_dim == 8 ? launch_d<8>(ta, ti, p, bn, mt, grid, smem, s)
                                            : launch_d<4>(ta, ti, p, bn, mt, grid, smem, s);
    count_launch();
    if (e != cudaSuccess) return cuda_fail(e, "grouped tensor-core launch");
  }
  return SACQ_OK;
}

}  // namespace sacq
