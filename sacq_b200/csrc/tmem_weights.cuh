// Shared pieces of the tensor-core kernels that keep the expanded weights in tensor memory
// (linear_large_m_tmem.cu, linear_large_m_tmem_grouped.cu): thread layout, PTX wrappers for
// tcgen05.mma with the A operand in TMEM, tcgen05.st, tiled bulk stores, and the epilogue that
// transposes the accumulator (lane = weight row, column = token) into y.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace sacq {
namespace tmemw {

using namespace umma;

constexpr int kRows = 128;           // weight rows per CTA = TMEM lanes
constexpr int kTokTile = kBM * 128;  // 16 KB: 128 tokens x one 128-byte K block
constexpr int kXWarps = 16;                  // expander warps: four per TMEM lane quarter
constexpr int kXThreads = kXWarps * 32;
constexpr int kCtaThreads = 64 + kXThreads;  // + TMA producer warp + MMA issuer warp
constexpr int kStageTile = kBM * kRows * 2;  // 32 KB: one staged [128 tokens][128 rows] bf16 output sub-tile

__device__ __forceinline__ void xbarrier() { asm volatile("bar.sync 1, %0;" ::"n"(kXThreads) : "memory"); }
// AND of a predicate over the expander threads (named barrier 1).
__device__ __forceinline__ bool xall(bool v) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)v), "n"(kXThreads)
      : "memory");
  return r != 0;
}
// Tiled bulk store shared -> global (the tile is clipped at the tensor's edges).
__device__ __forceinline__ void tma_store_2d_issue(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}


// D[tmem] (+)= A[tmem] * B[smem desc], e4m3 x e4m3 -> fp32; A = 128 lanes x 8 columns (32 bytes per lane).
__device__ __forceinline__ void umma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 8 consecutive 32-bit columns of the warp's TMEM lane quarter, one lane per thread.
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
// 4 consecutive columns.
__device__ __forceinline__ void tmem_st_32x4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tmem_st_32xn(uint32_t taddr, const uint32_t (&r)[8]) { tmem_st_32x8(taddr, r); }
__device__ __forceinline__ void tmem_st_32xn(uint32_t taddr, const uint32_t (&r)[4]) { tmem_st_32x4(taddr, r); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }


// kind::f16 twin: fp16 x fp16 -> fp32; A = 128 lanes x 8 columns (16 halves per lane).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Where a kernel's result goes.
struct TmemOut {
  uint16_t* y;                  // bf16 [M, ldy]
  int64_t ldy;
  const uint16_t* residual;     // bf16 [M, ldr] added to the rounded output, or null
  int64_t ldr;
  int n_bc;                     // further copies of the output (peer GPUs' buffers), same pitch as y
  uint16_t* ybc[kMaxBcast];
  int M, N;
  int y_tma;                    // y (and every peer copy) takes tiled bulk stores (aligned, no residual)
};

// Tensor maps over the peer GPUs' copies of the output (the column split's exchange): the same
// [M][N] view as y's map, one per peer.  Plain tiled stores into peer memory, no multicast.
struct BcastMaps {
  CUtensorMap m[kMaxBcast];
};

// Epilogue of one CTA, run by all expander threads after the accumulator is complete:
//   y[m0 + token, n0 + row] = bf16(fma(sa[token], acc[row][token] * sw, bs))
// `lane_addr` = TMEM address of the warp's lane quarter (accumulator column 0), `row` = the
// thread's weight row (TMEM lane), `kpart` = which 32 tokens of every 128-token sub-tile the
// warp converts, `sap` = the NT*128 token scales in shared memory, `stage_base` = n_stage idle
// buffers of kStageTile bytes.
template <int NT>
__device__ __forceinline__ void tmem_epilogue(const TmemOut& o, const CUtensorMap* tmap_y, const CUtensorMap* tmap_bc,
                                              uint32_t lane_addr, int row,
                                              int kpart, int et, const float* sap, float sw, float bs,
                                              uint8_t* stage_base, int n_stage, int m0, int n0) {
  // The accumulator holds y transposed (lane = weight row, column = token).  Each 128-token
  // sub-tile goes through shared memory (the activation stages are idle now): a thread
  // writes its row's values of 32 tokens as 2-byte elements of a dense [token][row] bf16
  // tile; the tile then leaves by ONE tiled bulk store (clipped at the edges of y), which
  // overlaps the staging of the next sub-tile in the other buffer.  With a residual, peer
  // copies or an unaligned y the expander threads store the token rows themselves.
  const int c0 = kpart * 32;                      // this warp's 32 tokens of every sub-tile
#pragma unroll 1
  for (int t = 0; t < NT; ++t) {
    if (m0 + t * kBM >= o.M) break;               // uniform over the CTA
    uint8_t* stg = stage_base + (t % n_stage) * kStageTile;
    {
      uint32_t r[32];
      tmem_ld_32x32(lane_addr + (uint32_t)(t * kBM + c0), r);
      uint8_t* dst = stg + c0 * (kRows * 2) + row * 2;
      const float4* sa4 = reinterpret_cast<const float4*>(sap + t * kBM + c0);
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 sa = sa4[c4];                // four token scales per (broadcast) load
        const int c = c4 * 4;
        // two conversions per instruction; the halves go to two token rows of the staging tile
        const __nv_bfloat162 p01 = __floats2bfloat162_rn(fmaf(sa.x, __uint_as_float(r[c]) * sw, bs),
                                                         fmaf(sa.y, __uint_as_float(r[c + 1]) * sw, bs));
        const __nv_bfloat162 p23 = __floats2bfloat162_rn(fmaf(sa.z, __uint_as_float(r[c + 2]) * sw, bs),
                                                         fmaf(sa.w, __uint_as_float(r[c + 3]) * sw, bs));
        const uint32_t w01 = *reinterpret_cast<const uint32_t*>(&p01), w23 = *reinterpret_cast<const uint32_t*>(&p23);
        *reinterpret_cast<uint16_t*>(dst + (c + 0) * (kRows * 2)) = (uint16_t)w01;
        *reinterpret_cast<uint16_t*>(dst + (c + 1) * (kRows * 2)) = (uint16_t)(w01 >> 16);
        *reinterpret_cast<uint16_t*>(dst + (c + 2) * (kRows * 2)) = (uint16_t)w23;
        *reinterpret_cast<uint16_t*>(dst + (c + 3) * (kRows * 2)) = (uint16_t)(w23 >> 16);
      }
    }
    const int m_first = m0 + t * kBM;
    if (o.y_tma) {
      fence_proxy_async();                        // generic-proxy writes -> visible to the bulk store
      xbarrier();                                 // the sub-tile is staged
      if (et == 0) {
        // one bulk-store group per sub-tile: the local copy and, in a column split, every peer's copy
        tma_store_2d_issue(tmap_y, n0 * 2, m_first, smem_u32(stg));
        for (int c = 0; c < o.n_bc; ++c) tma_store_2d_issue(tmap_bc + c, n0 * 2, m_first, smem_u32(stg));
        tma_store_commit();
        // the other buffer's store (the previous sub-tile) must have read its tile before that
        // buffer is written again; with a single buffer, this store itself
        if (n_stage == 2) tma_store_wait_read<1>(); else tma_store_wait_read<0>();
      }
      xbarrier();
    } else {
      xbarrier();                                 // the sub-tile is staged
#pragma unroll 2
      for (int i = et; i < kBM * (kRows / 8); i += kXThreads) {
        const int tok = i >> 4, ch = i & 15;
        const int m = m_first + tok, n = n0 + ch * 8;
        if (m >= o.M || n >= o.N) continue;
        uint4 v = *reinterpret_cast<const uint4*>(stg + tok * (kRows * 2) + ch * 16);
        const int64_t off = (int64_t)m * o.ldy + n;
        const bool full = n + 8 <= o.N;
        if (o.residual != nullptr) {
          // bf16(bf16(v) + residual): the two roundings of `linear(x) + residual`
          const uint16_t* rp = o.residual + (int64_t)m * o.ldr + n;
          uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if (n + e < o.N) {
              const uint32_t a = (w[e >> 1] >> (16 * (e & 1))) & 0xffffu;
              const uint32_t o = float_to_bf16_bits(__fadd_rn(bf16_bits_to_float(a), bf16_bits_to_float(__ldg(rp + e))));
              w[e >> 1] = (w[e >> 1] & ~(0xffffu << (16 * (e & 1)))) | (o << (16 * (e & 1)));
            }
          }
          v = make_uint4(w[0], w[1], w[2], w[3]);
        }
        for (int c = -1; c < o.n_bc; ++c) {
          uint16_t* out = (c < 0 ? o.y : o.ybc[c]) + off;
          if (full && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
            *reinterpret_cast<uint4*>(out) = v;
          } else {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (n + e < o.N) out[e] = (uint16_t)(w[e >> 1] >> (16 * (e & 1)));
          }
        }
      }
      if (n_stage == 1) xbarrier();               // before the next sub-tile reuses the staging rows
    }
  }
  // shared memory stays valid until every store has read it; the writes themselves (local and peer)
  // are in the memory system then, like plain stores, and the grid's end orders them
  if (o.y_tma && et == 0) tma_store_wait_read<0>();
}

}  // namespace tmemw
}  // namespace sacq
