// tcgen05 / TMA / mbarrier PTX wrappers shared by the tensor-core kernels (sm_100a).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace sacq {
namespace umma {

constexpr int kBM = 128;                 // tokens per M tile (TMEM lanes)
constexpr int kExpanderThreads = 256;    // warps 2..9 of a CTA
constexpr int kThreads = 64 + kExpanderThreads;
constexpr int kErrTimeout = 1;           // status word value after an expired wait

// ---- PTX wrappers ----------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: gives up after ~2 s or as soon as another thread of the CTA has aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63) == 63) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > 2000000000ull) {
        *abort_flag = 1;
        atomicExch(status, kErrTimeout);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], e4m3 x e4m3 -> fp32, issued by one thread.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns of the warp's TMEM lane quarter.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile, 128-byte rows, SWIZZLE_128B: start address, leading offset 1
// (unused for swizzled K-major), 1024 bytes between 8-row groups, descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// kind::f8f6f4 instruction descriptor: fp32 accumulate, A = B = e4m3, both K-major, N, M.
__host__ __device__ constexpr uint32_t make_idesc(int bn) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void expander_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kExpanderThreads) : "memory");
}


// kind::f16 with fp16 operands: D[tmem] (+)= A[smem desc] * B[smem desc], fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// AND of a predicate over the 256 expander threads (named barrier 1): makes a per-thread
// "every wait succeeded" flag uniform before code that uses expander_barrier().
__device__ __forceinline__ bool expander_all(bool v) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)v), "n"(kExpanderThreads)
      : "memory");
  return r != 0;
}

// Epilogue, second half: the expander warps have staged a [128 rows][BN] bf16 tile in shared
// memory (row pitch `pitch` bytes); all 256 of their threads store it with 16-byte chunks that
// are consecutive within a row, so a warp writes whole 256-byte row segments -- to y and to
// every further copy of the output (peer GPUs' buffers: large contiguous stores are what
// NVLink moves efficiently).  `et` = thread index among the expanders.
template <int BN>
__device__ __forceinline__ void store_staged_tile(const uint8_t* stg, int pitch, int et, int m_first, int M, int n0, int N,
                                                  uint16_t* y, int64_t ldy, uint16_t* const* ybc, int n_bc) {
  constexpr int CH = BN / 8;                          // 16-byte chunks per row
  for (int idx = et; idx < kBM * CH; idx += kExpanderThreads) {
    const int row = idx / CH, ch = idx - row * CH;
    const int m = m_first + row, n = n0 + ch * 8;
    if (m >= M || n >= N) continue;
    const uint4 v = *reinterpret_cast<const uint4*>(stg + row * pitch + ch * 16);
    const int64_t off = (int64_t)m * ldy + n;
    for (int i = -1; i < n_bc; ++i) {
      uint16_t* dst = (i < 0 ? y : ybc[i]) + off;
      if (n + 8 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        *reinterpret_cast<uint4*>(dst) = v;
      } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (n + e < N) dst[e] = (uint16_t)(w[e >> 1] >> (16 * (e & 1)));
      }
    }
  }
}

}  // namespace umma

// 2-D byte tensor [rows][row_bytes] with a [box_rows][box_bytes] box (linear_large_m.cu).
int encode_bytes_2d(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t pitch_bytes,
                    uint32_t box_bytes, uint32_t box_rows, CUtensorMapSwizzle swizzle);

// Tile map over a layer's packed index rows: box = one index super-block (two 128-k blocks) x
// `rows` weight rows (32, 64 or 128).  Built on first use and kept by the layer.
int large_m_index_map(const sacq_layer* L, int rows, const CUtensorMap** out);

}  // namespace sacq
