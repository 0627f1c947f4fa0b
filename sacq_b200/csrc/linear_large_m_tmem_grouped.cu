// Large-M quantized linear for GROUPED scales with the expanded weights in tensor memory:
//   y[m,n] = bf16( s[m] * (sum_k q[m,k] * cb[idx[n,k/d], k%d] * scale[n, k/G]) + bias[n] )
//
// The layouts the reference deployed (dim-4 vectors, one scale per 64 weights, 5- to 11-bit
// indices; gr00t_libero/acceleration/presets/FROZEN_DECODE_SELECTION.json) change their scale
// inside the K loop, so the scale is folded into the weight operand: fp16(codeword x scale),
// tcgen05 kind::f16 (linear_large_m_grouped.cu explains the encoding).  This kernel is the
// tensor-memory form of that one, structured like linear_large_m_tmem.cu:
//   * a CTA owns 128 weight rows (the 128 TMEM lanes) x 128*NT tokens;
//   * the packed index tile of a super-block (128 indices = 16*bits bytes per row) is staged as
//     16-byte column slices, [slice][row][16 B] (one TMA box of 16 bytes x 128 rows per slice): a
//     thread reads its row's slice with one 16-byte load and the 32 lanes of a warp read 512
//     contiguous bytes, free of bank conflicts (row-major rows of 16*bits bytes would put the
//     lanes of a warp 4 to 32 deep on the same banks);
//   * 16 expander warps: a thread owns one weight row and a quarter of each 64-k block (16
//     weights): it extracts its index fields (runtime width) from two slices held in registers,
//     gathers the fp16 codewords from the shared-memory codebook, multiplies by the row's group
//     scale (HMUL2) and writes 8 registers to the weight stage with tcgen05.st -- no
//     shared-memory store;
//   * the fp16 activation tiles (e4m3 or int8 widened exactly by a pre-pass into the caller's
//     workspace) are the MMA's B operand, TMA-loaded K-major / SWIZZLE_128B;
//   * warp 1 issues tcgen05.mma.kind::f16 with A from TMEM: four K = 16 steps per 64-k block
//     (384 tokens as two N = 192 instructions into two accumulators);
//   * epilogue: the shared transposing epilogue (tiled bulk stores of [token][row] bf16 tiles).
// TMEM: 128*NT accumulator columns + weight stages of 64 columns (two K blocks each): two
// stages with three sub-tiles, four otherwise.
//
// Replaces, for batched sizes, the reference's per-forward decode kernel plus 8-bit GEMM on
// these layouts (perrow_int8_fused_decode_r1.py:12-88, perrow_a8_candidate_r3.py:56-69).
#include <cuda.h>
#include <math.h>
#include <string.h>

#include <type_traits>

#include "common.cuh"
#include "tmem_weights.cuh"
#include "umma.cuh"

namespace sacq {

namespace {

using namespace umma;
using namespace tmemw;

constexpr int kBKh = 64;                      // fp16 elements per K block: one 128-byte swizzle row
constexpr int kSbIdx = 128;                   // indices per row per index super-block (16 * bits bytes)
constexpr int kGMaxActStages = 4;
constexpr int kGMaxWStages = 4;               // TMEM weight stages of 64 columns (two K blocks): 4, or 2 beside a 384-column accumulator
constexpr float kPreScale = 4096.f;           // keeps fp16(codeword x scale) far from the subnormals

struct GTmemParams {
  const __half* cb_f16;         // [C][D] codebook * 2^cb_exp_shift
  const uint16_t* scales;       // bf16 [N, num_groups]
  const uint16_t* bias;         // bf16 [N] or null
  const float* act_scale;       // [M]
  TmemOut out;
  int* status;
  int K, C;
  int bits, num_groups, group_size;
  int act_stages;
  float scale_mul;              // 2^sc_exp_shift * kPreScale, applied to every scale
  float out_mul;                // 2^-(cb_exp_shift + sc_exp_shift) / kPreScale
};

struct GTmemLayout {
  uint32_t act_off, act_stage, idx_off, idx_slot, cb_off, sc_off, bias_off, sa_off, bar_off, misc_off, total;
};

__host__ __device__ inline GTmemLayout gtmem_layout(int nt, int act_stages, int bits, int cb_bytes, int num_groups) {
  GTmemLayout L;
  L.act_off = 0;
  L.act_stage = (uint32_t)(nt * kTokTile);
  L.idx_off = act_stages * L.act_stage;
  L.idx_slot = (uint32_t)(kRows * 16 * bits);
  L.cb_off = (L.idx_off + 2 * L.idx_slot + 127) & ~127u;
  L.sc_off = L.cb_off + (uint32_t)((cb_bytes + 127) & ~127);
  // bf16 scales of the tile's rows, row pitch num_groups + 1 (odd or even, never a multiple of the 32 banks'
  // period for the 32 consecutive rows of a warp: an unpadded pitch of 64 bytes made every read a 16-way conflict)
  L.bias_off = L.sc_off + (uint32_t)((kRows * (num_groups | 1) * 2 + 127) & ~127);
  L.sa_off = L.bias_off + kRows * 4;
  L.bar_off = L.sa_off + (uint32_t)(nt * kBM * 4);
  L.misc_off = L.bar_off + 32 * 8;
  L.total = L.misc_off + 64;
  return L;
}

#ifdef SACQ_TRACE
// Profiling builds only (-DSACQ_TRACE): CTA (0, 0) records %globaltimer at a few points per role.
__device__ long long g_gtmem_trace[8][72];
#define SACQ_GTR(role, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (slot) < 72) { long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); g_gtmem_trace[role][slot] = _t; } } while (0)
#else
#define SACQ_GTR(role, slot) do { } while (0)
#endif

// D in {4, 8}; NT = 128-token sub-tiles per CTA (1, 2 or 3).  grid = (ceil(N / 128), ceil(M / (128 * NT))).
template <int D, int NT>
__global__ void __launch_bounds__(kCtaThreads, 1)
large_m_tmem_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_idx,
                            const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ BcastMaps tmap_bc,
                            const __grid_constant__ GTmemParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) SACQ_GTR(0, 0);
  constexpr int BT = kBM * NT;
  constexpr int IDX_PER_KB = kBKh / D;                // indices per row per K block
  constexpr int KB_PER_SB = kSbIdx / IDX_PER_KB;      // K blocks per index super-block
  constexpr int IPT = IDX_PER_KB / 4;                 // indices per expander thread per K block (16 weights)
  // A weight stage holds TWO K blocks (128 k, 64 columns): the per-stage cost of the expanders and of the
  // issuer (barrier waits, tcgen05.wait::st, fences, commits) is paid half as often as with one block per
  // stage.  Two stages fit beside three sub-tiles of accumulators, four otherwise.
  constexpr int kGWStages = NT == 3 ? 2 : kGMaxWStages;
  constexpr uint32_t kWCol0 = BT;
  constexpr uint32_t kTmemCols = 512;
  static_assert(BT + kGWStages * 64 <= 512, "TMEM budget");
  constexpr uint32_t kIdesc256 = make_idesc(256), kIdesc128 = make_idesc(128), kIdesc192 = make_idesc(192);
  using CwVec = typename std::conditional<D == 8, uint4, uint2>::type;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const GTmemLayout L = gtmem_layout(NT, p.act_stages, p.bits, p.C * D * 2, p.num_groups);

  constexpr int ACT_FULL = 0, ACT_EMPTY = kGMaxActStages, W_FULL = 2 * kGMaxActStages,
                W_EMPTY = 2 * kGMaxActStages + kGMaxWStages, IDX_FULL = 2 * kGMaxActStages + 2 * kGMaxWStages,
                IDX_EMPTY = IDX_FULL + 2, ACC_FULL = IDX_FULL + 4;
  const uint32_t bars = base + L.bar_off;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + L.misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + L.misc_off + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kRows;
  const int m0 = blockIdx.y * BT;
  const int num_kb = p.K / kBKh;
  const int act_stages = p.act_stages;
  const int sb_bytes = 16 * p.bits;
  const int nt_valid = min(NT, (p.out.M - m0 + kBM - 1) / kBM);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGMaxActStages; ++i) {
      mbar_init(bar(ACT_FULL + i), 1);
      mbar_init(bar(ACT_EMPTY + i), 1);
    }
    for (int i = 0; i < kGMaxWStages; ++i) {
      mbar_init(bar(W_FULL + i), kXWarps);
      mbar_init(bar(W_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(IDX_FULL + i), 1);
      mbar_init(bar(IDX_EMPTY + i), kXWarps);
    }
    mbar_init(bar(ACC_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_idx);
    if (p.out.y_tma) prefetch_tensormap(&tmap_y);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) SACQ_GTR(0, 1);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        if (kb % KB_PER_SB == 0) {
          const int sb = kb / KB_PER_SB, slot = sb & 1;
          if (!mbar_wait(bar(IDX_EMPTY + slot), ((sb >> 1) & 1) ^ 1, abort_flag, p.status)) break;
          mbar_arrive_expect_tx(bar(IDX_FULL + slot), (uint32_t)(kRows * sb_bytes));
          for (int sl = 0; sl < p.bits; ++sl)          // one 16-byte column slice of the 128 rows per copy
            tma_load_2d(base + L.idx_off + slot * L.idx_slot + sl * (kRows * 16), &tmap_idx, sb * sb_bytes + sl * 16, n0,
                        bar(IDX_FULL + slot));
        }
        const int st = kb % act_stages;
        if (!mbar_wait(bar(ACT_EMPTY + st), ((kb / act_stages) & 1) ^ 1, abort_flag, p.status)) break;
        mbar_arrive_expect_tx(bar(ACT_FULL + st), nt_valid * kTokTile);
#pragma unroll
        for (int t = 0; t < NT; ++t)
          if (t < nt_valid)
            tma_load_2d(base + L.act_off + st * L.act_stage + t * kTokTile, &tmap_a, kb * 128, m0 + t * kBM,
                        bar(ACT_FULL + st));
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int wi = 0; wi < num_kb / 2 && ok; ++wi) {         // weight stage by weight stage: two K blocks each
        const int ws = wi % kGWStages;
        ok = mbar_wait(bar(W_FULL + ws), (wi / kGWStages) & 1, abort_flag, p.status);
#pragma unroll
        for (int sub = 0; sub < 2 && ok; ++sub) {
          const int kb = 2 * wi + sub, st = kb % act_stages;
          ok = mbar_wait(bar(ACT_FULL + st), (kb / act_stages) & 1, abort_flag, p.status);
          if (!ok) break;
          if (sub == 0) tc_fence_after();
          SACQ_GTR(1, kb + 8);
          const uint32_t act_addr = base + L.act_off + st * L.act_stage;
          const uint32_t w_col = kWCol0 + (uint32_t)(ws * 64 + sub * 32);
#pragma unroll
          for (int ks = 0; ks < kBKh / 16; ++ks) {
            const uint64_t adv = (uint64_t)((ks * 32) >> 4);              // 16 fp16 = 32 bytes per K step
            const uint32_t a_tmem = tmem_base + w_col + (uint32_t)(ks * 8);
            const uint32_t acc = (kb | ks) != 0;
            if (NT == 3 && nt_valid == 3) {
              // two N = 192 instructions into two accumulators (an instruction costs about 60 ns whatever its N)
              umma_f16_ts(tmem_base, a_tmem, make_smem_desc(act_addr) + adv, kIdesc192, acc);
              umma_f16_ts(tmem_base + 192u, a_tmem, make_smem_desc(act_addr + kTokTile * 3 / 2) + adv, kIdesc192, acc);
            } else if (NT >= 2 && nt_valid >= 2) {
              umma_f16_ts(tmem_base, a_tmem, make_smem_desc(act_addr) + adv, kIdesc256, acc);
            } else {
              umma_f16_ts(tmem_base, a_tmem, make_smem_desc(act_addr) + adv, kIdesc128, acc);
            }
          }
          umma_commit(bar(ACT_EMPTY + st));
        }
        if (ok) umma_commit(bar(W_EMPTY + ws));
      }
      if (ok) umma_commit(bar(ACC_FULL));
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ expanders, then epilogue
    const int et = threadIdx.x - 64;                 // 0..511
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;             // weight row of the tile = TMEM lane
    const int kpart = (warp - 2) >> 2;               // which 16 weights of the 64-k block (0..3)
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    {
      // fp16 codebook, the tile's scales (bf16, all groups), biases and token scales
      const uint4* src = reinterpret_cast<const uint4*>(p.cb_f16);
      uint4* dst = reinterpret_cast<uint4*>(sm + L.cb_off);
      const int n16 = (p.C * D * 2) >> 4;
      for (int i = et; i < n16; i += kXThreads) cp_async_16(dst + i, src + i);
      uint16_t* sc = reinterpret_cast<uint16_t*>(sm + L.sc_off);
      const int sc_pitch = p.num_groups | 1;
      for (int i = et; i < kRows * p.num_groups; i += kXThreads) {
        const int r = i / p.num_groups, g = i - r * p.num_groups;
        const int n = min(n0 + r, p.out.N - 1);
        sc[r * sc_pitch + g] = __ldg(p.scales + (int64_t)n * p.num_groups + g);
      }
      if (et < kRows) {
        const int n = min(n0 + et, p.out.N - 1);
        reinterpret_cast<float*>(sm + L.bias_off)[et] = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
      }
      for (int i = et; i < BT; i += kXThreads) {
        const int m = m0 + i;
        reinterpret_cast<float*>(sm + L.sa_off)[i] = m < p.out.M ? __ldg(p.act_scale + m) : 0.f;
      }
      cp_async_wait_all();
      xbarrier();
      if (et == 0) SACQ_GTR(0, 2);
    }
    const CwVec* cbs = reinterpret_cast<const CwVec*>(sm + L.cb_off);
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(sm + L.sc_off) + row * (p.num_groups | 1);
    const uint32_t mask = (1u << p.bits) - 1u;
    const int kb_per_group = p.group_size / kBKh;
    bool ok = true;
    int grp = 0, left_in_group = kb_per_group;
    for (int wi = 0; wi < num_kb / 2 && ok; ++wi) {
      const int ws = wi % kGWStages;
      ok = mbar_wait(bar(W_EMPTY + ws), ((wi / kGWStages) & 1) ^ 1, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after();                              // the MMAs that read this stage are complete
      if (warp == 2 && lane == 0) SACQ_GTR(2, wi + 8);
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        const int kb = 2 * wi + sub;
        const int sb = kb / KB_PER_SB, slot = sb & 1;
        if (kb % KB_PER_SB == 0) ok = mbar_wait(bar(IDX_FULL + slot), (sb >> 1) & 1, abort_flag, p.status);
        if (!ok) break;
        // scale * 2^sc_exp_shift * 4096 is a bf16 significand with a small exponent: exact in fp16
        const __half sh = __float2half_rn(bf16_bits_to_float(sc[grp]) * p.scale_mul);
        const __half2 s2 = __half2half2(sh);
        // this thread's IPT index fields: a window of at most 64 bits that starts at bit `bit0` of the row's
        // super-block, i.e. in slice bit0 / 128 and possibly the next one; bit0 is the same for the whole warp
        const int bit0 = ((kb % KB_PER_SB) * IDX_PER_KB + kpart * IPT) * p.bits;
        const int sl0 = bit0 >> 7;
        const uint8_t* slice = sm + L.idx_off + slot * L.idx_slot + row * 16;
        const uint4 a = *reinterpret_cast<const uint4*>(slice + sl0 * (kRows * 16));
        uint4 b = a;                                     // the next slice only when the window crosses into it
        if ((bit0 & 127) + IPT * p.bits > 128) b = *reinterpret_cast<const uint4*>(slice + (sl0 + 1) * (kRows * 16));
        uint32_t lo, mid, hi;
        switch ((bit0 >> 5) & 3) {                       // first word of the window inside slice sl0 (warp-uniform)
          case 0: lo = a.x; mid = a.y; hi = a.z; break;
          case 1: lo = a.y; mid = a.z; hi = a.w; break;
          case 2: lo = a.z; mid = a.w; hi = b.x; break;
          default: lo = a.w; mid = b.x; hi = b.y; break;
        }
        const uint32_t wsh = (uint32_t)(bit0 & 31);
        const uint64_t win = ((uint64_t)__funnelshift_r(mid, hi, wsh) << 32) | __funnelshift_r(lo, mid, wsh);
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
          const CwVec cw = cbs[(uint32_t)(win >> (j * p.bits)) & mask];
          if constexpr (D == 8) {
            const uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&w4[e]), s2);
              o[4 * j + e] = *reinterpret_cast<const uint32_t*>(&h);
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
        tmem_st_32x8(lane_addr + kWCol0 + (uint32_t)(ws * 64 + sub * 32 + kpart * 8), o);
        if (--left_in_group == 0) { ++grp; left_in_group = kb_per_group; }
      }
      if (!ok) break;
      if (warp == 2 && lane == 0) SACQ_GTR(4, wi + 8);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (warp == 2 && lane == 0) SACQ_GTR(5, wi + 8);
      if (lane == 0) {
        mbar_arrive(bar(W_FULL + ws));
        // the index slot is free once its last K block has been read (KB_PER_SB is even: that is an odd block)
        const int kb_last = 2 * wi + 1;
        if ((kb_last + 1) % KB_PER_SB == 0 || kb_last == num_kb - 1) mbar_arrive(bar(IDX_EMPTY + (kb_last / KB_PER_SB & 1)));
      }
    }

    // ---- epilogue
    if (ok) ok = mbar_wait(bar(ACC_FULL), 0, abort_flag, p.status);
    if (warp == 2 && lane == 0) SACQ_GTR(0, 3);
    ok = xall(ok);                                    // tcgen05.ld and the staging barriers are collective
    if (ok) {
      tc_fence_after();
      const float bs = reinterpret_cast<const float*>(sm + L.bias_off)[row];
      tmem_epilogue<NT>(p.out, &tmap_y, tmap_bc.m, lane_addr, row, kpart, et, reinterpret_cast<const float*>(sm + L.sa_off),
                        p.out_mul, bs, sm + L.act_off, (act_stages * NT * kTokTile >= 2 * kStageTile) ? 2 : 1, m0, n0);
    }
  }

  // ---- common exit: every thread arrives here, also after an aborted wait
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) SACQ_GTR(0, 4);
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// e4m3 (or int8, I8) [M, K] -> fp16 [M, K] (exact); one CTA per token row.
template <bool I8>
__global__ void __launch_bounds__(256) widen_act_f16_kernel(const uint8_t* __restrict__ q, int64_t K,
                                                            __half* __restrict__ a16) {
  const int64_t m = blockIdx.x;
  const uint2* src = reinterpret_cast<const uint2*>(q + m * K);
  uint4* dst = reinterpret_cast<uint4*>(a16 + m * K);
  for (int64_t i = threadIdx.x; i < (K >> 3); i += blockDim.x) {
    const uint2 v = __ldg(src + i);
    uint32_t w[4];
    const uint32_t in[2] = {v.x, v.y};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if constexpr (I8) {
        const __half2 a = __halves2half2(__int2half_rn((int)(int8_t)(in[j] & 0xff)), __int2half_rn((int)(int8_t)((in[j] >> 8) & 0xff)));
        const __half2 b = __halves2half2(__int2half_rn((int)(int8_t)((in[j] >> 16) & 0xff)), __int2half_rn((int)(int8_t)(in[j] >> 24)));
        w[2 * j] = *reinterpret_cast<const uint32_t*>(&a);
        w[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b);
      } else {
        const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(in[j] & 0xffff), __NV_E4M3);
        const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(in[j] >> 16), __NV_E4M3);
        w[2 * j] = (uint32_t)a.x | ((uint32_t)a.y << 16);
        w[2 * j + 1] = (uint32_t)b.x | ((uint32_t)b.y << 16);
      }
    }
    dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

constexpr int64_t kGSlabTokens = 3072;   // tokens widened per launch (8 tiles of 384): bounds the fp16 scratch

int g_act_stages(const sacq_layer* L, int nt) {
  const int cb_bytes = L->cb_entries * L->d.vector_dim * 2;
  for (int st = kGMaxActStages; st >= 2; --st)
    if (gtmem_layout(nt, st, L->d.index_bits, cb_bytes, (int)L->num_groups).total + 1024 <= 227 * 1024) return st;
  return 0;
}

template <int D, int NT>
cudaError_t glaunch_nt(const CUtensorMap& ta, const CUtensorMap& ti, const CUtensorMap& ty, const BcastMaps& tb,
                       const GTmemParams& p, dim3 grid, size_t smem, cudaStream_t s) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(large_m_tmem_grouped_kernel<D, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  large_m_tmem_grouped_kernel<D, NT><<<grid, kCtaThreads, smem, s>>>(ta, ti, ty, tb, p);
  return cudaGetLastError();
}

template <int D>
cudaError_t glaunch_d(const CUtensorMap& ta, const CUtensorMap& ti, const CUtensorMap& ty, const BcastMaps& tb,
                      const GTmemParams& p, int nt, dim3 grid, size_t smem, cudaStream_t s) {
  if (nt == 3) return glaunch_nt<D, 3>(ta, ti, ty, tb, p, grid, smem, s);
  if (nt == 2) return glaunch_nt<D, 2>(ta, ti, ty, tb, p, grid, smem, s);
  return glaunch_nt<D, 1>(ta, ti, ty, tb, p, grid, smem, s);
}

}  // namespace

bool large_m_tmem_grouped_supported(const sacq_layer* L) {
  const sacq_layer_desc& d = L->d;
  if (d.vector_dim != 8 && d.vector_dim != 4) return false;
  if (d.index_bits < 1 || d.index_bits > 16) return false;
  if (!L->rows_16b_aligned) return false;
  if (d.in_features % (2 * kBKh) != 0 || d.group_size % kBKh != 0) return false;   // whole weight stages of two K blocks
  if (((size_t)L->cb_entries * d.vector_dim * 2) % 16 != 0) return false;
  if (has_shift(L)) return false;
  return g_act_stages(L, 1) >= 2;
}

// From how many tokens this kernel beats the shared-memory-tile kernel of linear_large_m_grouped.cu
// (measured at d = 4, 10-bit, group 64: 2048x6144 27.6 against 33.1 us at M = 300 and 37 against 66 us
// at M = 1024; 2048x2048 and 6144x2048 break even at M = 1024 and win 1.5-1.9x from M = 4096).
int64_t large_m_tmem_grouped_min_m(const sacq_layer* L) {
  return L->d.out_features >= 5120 ? 288 : 1024;
}

// Workspace behind the counter region: the fp16 activations of one token slab.
int64_t large_m_tmem_grouped_workspace_bytes(const sacq_layer* L, int64_t M) {
  const int64_t rows = M < kGSlabTokens ? M : kGSlabTokens;
  return (rows * L->d.in_features * 2 + 255) & ~(int64_t)255;
}

int launch_large_m_tmem_grouped(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                                void* ws, int64_t ws_bytes, cudaStream_t s, const void* residual, int64_t ldr,
                                int act_int8, const BcastDst* bc, int nt_force) {
  const sacq_layer_desc& d = L->d;
  if (!large_m_tmem_grouped_supported(L))
    return set_error(SACQ_ERR_UNSUPPORTED, "grouped TMEM-weight kernel cannot run this layer geometry");
  if (M <= 0 || d.out_features == 0) return SACQ_OK;
  if (reinterpret_cast<uintptr_t>(q) % 8 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "quantized activations must be 8-byte aligned");
  const int64_t need = large_m_tmem_grouped_workspace_bytes(L, M);
  if (ws == nullptr || ws_bytes < need)
    return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed behind the counter region, %lld given",
                     (long long)need, (long long)ws_bytes);
  if (reinterpret_cast<uintptr_t>(ws) % 256 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  const int64_t K = d.in_features, N = d.out_features;
  const int64_t slab = M < kGSlabTokens ? M : kGSlabTokens;
  __half* a16 = static_cast<__half*>(ws);

  GTmemParams p{};
  p.cb_f16 = L->cb_f16;
  p.scales = static_cast<const uint16_t*>(d.scales);
  p.bias = static_cast<const uint16_t*>(d.bias);
  p.status = L->d_status;
  p.K = (int)K; p.C = L->cb_entries;
  p.bits = d.index_bits; p.num_groups = (int)L->num_groups; p.group_size = d.group_size;
  p.scale_mul = ldexpf(kPreScale, L->sc_exp_shift);
  p.out_mul = ldexpf(1.f / kPreScale, -(L->cb_exp_shift + L->sc_exp_shift));
  p.out.N = (int)N;
  p.out.ldy = ldy;
  p.out.ldr = ldr;
  p.out.n_bc = bc ? bc->n : 0;

  const int64_t row_tiles = (N + kRows - 1) / kRows;
  for (int64_t m0 = 0; m0 < M; m0 += slab) {
    const int64_t rows = (M - m0) < slab ? (M - m0) : slab;
    if (act_int8)
      widen_act_f16_kernel<true><<<(unsigned)rows, 256, 0, s>>>(static_cast<const uint8_t*>(q) + m0 * K, K, a16);
    else
      widen_act_f16_kernel<false><<<(unsigned)rows, 256, 0, s>>>(static_cast<const uint8_t*>(q) + m0 * K, K, a16);
    count_launch();
    SACQ_CUDA_TRY(cudaGetLastError());
    // token sub-tiles per CTA: the largest tile that does not add a wave
    int nt = nt_force;
    if (nt < 1 || nt > 3) {
      double best = 1e30;
      nt = 0;
      for (int cand = 3; cand >= 1; --cand) {
        if (g_act_stages(L, cand) < 2) continue;
        const int64_t tiles = row_tiles * ((rows + kBM * cand - 1) / (kBM * cand));
        const int64_t waves = (tiles + L->num_sms - 1) / L->num_sms;
        // measured per wave at K = 2048 (d = 4, 10-bit, group 64), widening pre-pass and launch included:
        // 27.6 / 33 / 37 us for 1 / 2 / 3 sub-tiles; two sub-tiles lose more than the others once waves queue
        // (42 us per wave), so they are only chosen where they save a wave outright
        const double per_wave = cand == 3 ? 32.0 : cand == 2 ? (waves == 1 ? 28.0 : 37.0) : 22.6;
        const double cost = (double)waves * (5.0 + (double)K / 2048.0 * per_wave);
        if (cost < best - 1e-9) { best = cost; nt = cand; }
      }
    }
    if (nt == 0 || g_act_stages(L, nt) < 2)
      return set_error(SACQ_ERR_UNSUPPORTED, "grouped TMEM-weight kernel: no tile fits shared memory");
    p.act_stages = g_act_stages(L, nt);
    CUtensorMap ta, ti, ty;
    int rc = encode_bytes_2d(&ta, a16, (uint64_t)(K * 2), (uint64_t)rows, (uint64_t)(K * 2), 128, kBM,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SACQ_OK) return rc;
    const uint64_t row_bytes = (uint64_t)(L->row_bits / 8);
    rc = encode_bytes_2d(&ti, d.packed, row_bytes, (uint64_t)N, row_bytes, 16u, (uint32_t)kRows, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != SACQ_OK) return rc;
    uint16_t* y_slab = static_cast<uint16_t*>(y) + m0 * ldy;
    bool y_tma = residual == nullptr && reinterpret_cast<uintptr_t>(y_slab) % 16 == 0 && (ldy * 2) % 16 == 0 && N >= kRows;
    for (int i = 0; i < p.out.n_bc; ++i)
      y_tma = y_tma && reinterpret_cast<uintptr_t>(static_cast<uint16_t*>(bc->ptr[i]) + m0 * ldy) % 16 == 0;
    ty = ta;
    BcastMaps tb = {};
    if (y_tma) {
      rc = encode_bytes_2d(&ty, y_slab, (uint64_t)N * 2, (uint64_t)rows, (uint64_t)ldy * 2, kRows * 2, kBM,
                           CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc != SACQ_OK) return rc;
      for (int i = 0; i < p.out.n_bc; ++i) {         // the peers' copies of a column split take the same tiled stores
        rc = encode_bytes_2d(&tb.m[i], static_cast<uint16_t*>(bc->ptr[i]) + m0 * ldy, (uint64_t)N * 2, (uint64_t)rows,
                             (uint64_t)ldy * 2, kRows * 2, kBM, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != SACQ_OK) return rc;
      }
    }
    p.act_scale = scale + m0;
    p.out.y = y_slab;
    p.out.y_tma = y_tma ? 1 : 0;
    p.out.residual = residual ? static_cast<const uint16_t*>(residual) + m0 * ldr : nullptr;
    for (int i = 0; i < p.out.n_bc; ++i) p.out.ybc[i] = static_cast<uint16_t*>(bc->ptr[i]) + m0 * ldy;
    p.out.M = (int)rows;
    const dim3 grid((unsigned)row_tiles, (unsigned)((rows + kBM * nt - 1) / (kBM * nt)));
    const GTmemLayout lay = gtmem_layout(nt, p.act_stages, d.index_bits, L->cb_entries * d.vector_dim * 2, (int)L->num_groups);
    size_t smem = lay.total + 1024;
    if (smem < 120 * 1024) smem = 120 * 1024;      // two CTAs (each takes all 512 TMEM columns) never share an SM
    const cudaError_t e = d.vector_dim == 8 ? glaunch_d<8>(ta, ti, ty, tb, p, nt, grid, smem, s)
                                            : glaunch_d<4>(ta, ti, ty, tb, p, nt, grid, smem, s);
    count_launch();
    if (e != cudaSuccess) return cuda_fail(e, "grouped TMEM-weight launch");
  }
  return SACQ_OK;
}

}  // namespace sacq

#ifdef SACQ_TRACE
extern "C" SACQ_API int sacq_debug_gtmem_trace(long long* out) {
  return cudaMemcpyFromSymbol(out, sacq::g_gtmem_trace, sizeof(long long) * 8 * 72) == cudaSuccess ? 0 : -1;
}
#endif
