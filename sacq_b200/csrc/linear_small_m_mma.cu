// Small-M quantized linear, warp-MMA variant: the same packed-index walk as the CUDA-core
// kernel (linear_small_m.cu), but the 16-token x 8-row x 32-k products of one step are
// two m16n8k16 fp16 MMAs whose B fragments ARE the gathered codewords -- a lane fetches one
// 16-byte codeword from shared memory and feeds its four registers to the tensor pipe
// without ever writing an expanded weight tile.  Per index this costs one shared-memory
// gather and two MMAs instead of 16 activation reads and 64 half2 FMAs, which is what the
// instruction-issue-bound CUDA-core loop could not afford beyond a few tokens.
//
// Fragment bookkeeping (lane = 4*g + t): the lane owns the 8 consecutive indices
// 8t..8t+7 of row (block + g) in the current 32-index span.  In step s the warp multiplies
// vectors {8t+s}: MMA k-slots (2t, 2t+1) carry halfs (0,1) of vector 8t+s and k-slots
// (2t+8, 2t+9) carry halfs (2,3); the second MMA of the step carries halfs (4..7).  The A
// fragments use the same slot order, so the activations a lane needs are the 64
// contiguous e4m3 bytes q[token, (span*32 + 8t)*8 ...) of tokens g and g+8, read straight
// from global memory and widened to fp16 in registers (exactly).
//
// Stands in for the reference's small-M packed GEMMs: codebook_cutlass_kernel.cu:234-583
// (mma.sync m16n8k16 with a reconstructed B tile in shared memory) and
// codebook_linear_triton_2026_08_23.py:499-705.
#include "small_m.cuh"

namespace sacq {
namespace smallm {

namespace {

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D in {4, 8}; BITS in {8, 12, 16}; R8 = 8-row sub-blocks per tile (1, 2, 4; the staged variant also 6).
//
// Work decomposition: a CTA owns a tile of 16 tokens x (8*R8) output rows and loops over
// tiles; its warps split the row's 32-index spans among themselves (warp w takes spans w,
// w + nwarps, ...), so the K reduction ends in shared memory behind one __syncthreads and
// needs neither global scratch nor arrival counters.
template <int D, int BITS, bool CB_SMEM, int R8>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) small_m_mma_kernel(const SmallMParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  using CwVec = typename std::conditional<D == 8, uint4, uint2>::type;   // D halfs
  constexpr int WPG = BITS / 4;            // 32-bit words holding a lane's 8 indices
  constexpr int AREG = D / 2;              // half2 registers per activation vector
  constexpr int QV = D / 4;                // uint4 pairs covering a lane's 8 vectors (8*D bytes)
  constexpr int kFrag = R8 * 4;            // accumulator registers per lane
  const CwVec* cbs = reinterpret_cast<const CwVec*>(smem);
  const int cb_bytes = CB_SMEM ? p.C * D * 2 : 0;
  float* red = reinterpret_cast<float*>(smem + cb_bytes);               // [nwarps][kFrag][32]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  if (CB_SMEM) {
    const uint4* src = reinterpret_cast<const uint4*>(p.cb_f16);
    uint4* dst = reinterpret_cast<uint4*>(smem);
    const int n16 = cb_bytes >> 4;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) cp_async_16(dst + i, src + i);
  }

  int64_t row_off[R8];                       // byte offset of rows (8r + g) of the tile in the packed stream
  uint4 qa[2 * QV], qb[2 * QV];              // raw e4m3 bytes of tokens g / g+8 for the lane's 8 vectors
  uint32_t wd[R8][WPG];                      // the lane's 8 indices for each row sub-block
  bool ok_a = false, ok_b = false;
  const uint8_t* qrow_a = nullptr;
  const uint8_t* qrow_b = nullptr;

  // Issues the global loads of one span: 8*D activation bytes per token and BITS bytes of
  // indices per row sub-block.
  auto load_span = [&](int sp) {
    const int64_t kb = ((int64_t)sp * kSpanIdx + 8 * t) * D;
#pragma unroll
    for (int j = 0; j < 2 * QV; ++j) {
      qa[j] = ok_a ? __ldg(reinterpret_cast<const uint4*>(qrow_a + kb) + j) : make_uint4(0, 0, 0, 0);
      qb[j] = ok_b ? __ldg(reinterpret_cast<const uint4*>(qrow_b + kb) + j) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int r = 0; r < R8; ++r) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(p.packed + row_off[r] + (int64_t)sp * (4 * BITS) + t * BITS);
#pragma unroll
      for (int j = 0; j < WPG; ++j) wd[r][j] = __ldg(src + j);
    }
  };

  int chunk = 0, n_base = 0;
  // Sets the per-tile state the loads depend on.
  auto setup_tile = [&](int64_t tile) {
    const int rt = (int)(tile % p.row_blocks);
    chunk = (int)(tile / p.row_blocks);
    n_base = rt * 8 * R8;
    const int ma = chunk * 16 + g, mb = ma + 8;
    ok_a = ma < p.M;
    ok_b = mb < p.M;
    qrow_a = p.q + (int64_t)(ok_a ? ma : 0) * p.K;
    qrow_b = p.q + (int64_t)(ok_b ? mb : 0) * p.K;
#pragma unroll
    for (int r = 0; r < R8; ++r) {
      int n = n_base + r * 8 + g;
      if (n >= p.N) n = p.N - 1;
      row_off[r] = (int64_t)n * p.row_bytes;
    }
  };

  int64_t tile = blockIdx.x;
  if (tile < p.num_items) {
    setup_tile(tile);
    if (warp < p.spans_per_row) load_span(warp);   // overlaps the codebook copy
  }
  if (CB_SMEM) {
    cp_async_wait_all();
    __syncthreads();                               // every warp of the CTA, with or without a span
  }

  for (; tile < p.num_items; tile += gridDim.x) {
    const int cur_chunk = chunk, cur_n_base = n_base;
    float acc[R8][4];
#pragma unroll
    for (int r = 0; r < R8; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[r][j] = 0.f;
    float xs_a = 0.f, xs_b = 0.f;

    int sp = warp;
    for (; sp < p.spans_per_row; sp += nwarps) {
      // ---- A fragments: widen the e4m3 (or int8) bytes to fp16 (exact)
      uint32_t fa[8][AREG], fb[8][AREG];
      {
        const uint32_t* wa = reinterpret_cast<const uint32_t*>(qa);
        const uint32_t* wb = reinterpret_cast<const uint32_t*>(qb);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if constexpr (D == 8) {
            act4_to_h2(p.act_int8, wa[2 * s], fa[s][0], fa[s][1]);
            act4_to_h2(p.act_int8, wa[2 * s + 1], fa[s][2], fa[s][3]);
            act4_to_h2(p.act_int8, wb[2 * s], fb[s][0], fb[s][1]);
            act4_to_h2(p.act_int8, wb[2 * s + 1], fb[s][2], fb[s][3]);
          } else {
            act4_to_h2(p.act_int8, wa[s], fa[s][0], fa[s][1]);
            act4_to_h2(p.act_int8, wb[s], fb[s][0], fb[s][1]);
          }
        }
      }
      if (p.shift != 0.f) {
        float ta = 0.f, tb = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s)
#pragma unroll
          for (int j = 0; j < AREG; ++j) {
            ta += __low2float(as_h2(fa[s][j])) + __high2float(as_h2(fa[s][j]));
            tb += __low2float(as_h2(fb[s][j])) + __high2float(as_h2(fb[s][j]));
          }
        ta += __shfl_xor_sync(0xffffffffu, ta, 1);
        ta += __shfl_xor_sync(0xffffffffu, ta, 2);
        tb += __shfl_xor_sync(0xffffffffu, tb, 1);
        tb += __shfl_xor_sync(0xffffffffu, tb, 2);
        xs_a += ta;
        xs_b += tb;
      }
      uint32_t wcur[R8][WPG];
#pragma unroll
      for (int r = 0; r < R8; ++r)
#pragma unroll
        for (int j = 0; j < WPG; ++j) wcur[r][j] = wd[r][j];
      if (sp + nwarps < p.spans_per_row) load_span(sp + nwarps);   // next span's loads fly during the MMAs

      float cs[R8][4];
#pragma unroll
      for (int r = 0; r < R8; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) cs[r][j] = 0.f;
      // step-major so the R8 accumulator chains interleave
#pragma unroll
      for (int s = 0; s < 8; ++s) {
#pragma unroll
        for (int r = 0; r < R8; ++r) {
          const uint32_t idx = field8<BITS>(wcur[r], s);
          CwVec c;
          if constexpr (CB_SMEM) c = cbs[idx];
          else c = __ldg(reinterpret_cast<const CwVec*>(p.cb_f16) + idx);
          mma_m16n8k16(cs[r], fa[s][0], fb[s][0], fa[s][1], fb[s][1], c.x, c.y);
          if constexpr (D == 8) mma_m16n8k16(cs[r], fa[s][2], fb[s][2], fa[s][3], fb[s][3], c.z, c.w);
        }
      }
      // ---- fold in the group scale of the two output rows this lane holds per sub-block
      const int grp = (sp * kSpanIdx * D) / p.group_size;
#pragma unroll
      for (int r = 0; r < R8; ++r) {
        const int n0 = min(cur_n_base + r * 8 + 2 * t, p.N - 1);
        const int n1 = min(cur_n_base + r * 8 + 2 * t + 1, p.N - 1);
        const float s0 = bf16_bits_to_float(__ldg(p.scales + (int64_t)n0 * p.num_groups + grp));
        const float s1 = bf16_bits_to_float(__ldg(p.scales + (int64_t)n1 * p.num_groups + grp));
        acc[r][0] = fmaf(s0, cs[r][0], acc[r][0]);
        acc[r][1] = fmaf(s1, cs[r][1], acc[r][1]);
        acc[r][2] = fmaf(s0, cs[r][2], acc[r][2]);
        acc[r][3] = fmaf(s1, cs[r][3], acc[r][3]);
      }
    }

    // ---- the next tile's first loads fly during this tile's reduction and epilogue
    if (tile + gridDim.x < p.num_items) {
      setup_tile(tile + gridDim.x);
      if (warp < p.spans_per_row) load_span(warp);
    }
    // ---- K reduction across the CTA's warps, then the epilogue
#pragma unroll
    for (int r = 0; r < R8; ++r) {
      red[(warp * kFrag + r * 4 + 0) * 32 + lane] = fmaf(acc[r][0], p.out_mul, p.shift * xs_a);
      red[(warp * kFrag + r * 4 + 1) * 32 + lane] = fmaf(acc[r][1], p.out_mul, p.shift * xs_a);
      red[(warp * kFrag + r * 4 + 2) * 32 + lane] = fmaf(acc[r][2], p.out_mul, p.shift * xs_b);
      red[(warp * kFrag + r * 4 + 3) * 32 + lane] = fmaf(acc[r][3], p.out_mul, p.shift * xs_b);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kFrag * 32; e += blockDim.x) {
      float v = 0.f;
      for (int w = 0; w < nwarps; ++w) v += red[w * kFrag * 32 + e];     // fixed order: deterministic
      const int ln = e & 31, j = (e >> 5) & 3, r = e >> 7;
      const int m = cur_chunk * 16 + (ln >> 2) + ((j & 2) ? 8 : 0);
      const int n = cur_n_base + r * 8 + 2 * (ln & 3) + (j & 1);
      if (m < p.M && n < p.N) {
        const float b = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
        store_out(p, m, n, fmaf(__ldg(p.act_scale + m), v, b));
      }
    }
    __syncthreads();                           // red is reused by the next tile
  }
}

// ---- staged variant -------------------------------------------------------------------
//
// Same fragment arithmetic, different data movement: everything a tile touches is brought
// into shared memory by a handful of bulk asynchronous copies (cp.async.bulk, one elected
// thread, completion on an mbarrier) before the warps start: the codebook once per CTA,
// then per tile the 8*R8 packed index rows (one contiguous block of the stream) and the 16
// activation rows.  The inner loop then has no global loads at all, and the memory latency
// is paid once per tile instead of once per span.

constexpr int kActPad = 16;                       // bytes of padding per staged activation row
// ... and per staged index row, where it pays: when a row is a multiple of 128 bytes the eight rows a
// warp reads in one instruction start in the same bank (8-way conflict); padded rows start four banks
// apart but need one bulk copy per row instead of one per tile.  Measured at M = 16: long rows gain
// (6144 x 2048: 7.70 -> 7.21 us; dim-4 vectors on 2048 x 6144: 8.73 -> 7.91 us), rows of 256-384 bytes
// lose 1-3 % to the extra copies, so those keep the single copy.
__host__ __device__ inline uint32_t staged_idx_pad(int64_t row_bytes) {
  return (row_bytes % 128 == 0 && row_bytes >= 768) ? 16u : 0u;
}

__device__ __forceinline__ uint32_t sm_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(sm_addr(dst)), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
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
// Bounded: gives up after about two seconds and reports through the layer's status word.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255) == 255) {
      uint64_t t1;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t1 - t0 > 2000000000ull) {
        atomicExch(status, 2);
        return false;
      }
    }
  }
}

struct StagedLayout {
  uint32_t cb_off, idx_off, act_off, red_off, sa_off, bar_off, total;   // idx region holds two buffers
};
__host__ __device__ inline StagedLayout staged_layout(int C, int D, int K, int64_t row_bytes, int r8, int warps,
                                                      int act_bufs = 1) {
  StagedLayout L;
  L.cb_off = 0;
  L.idx_off = (uint32_t)((C * D * 2 + 127) & ~127);
  L.act_off = L.idx_off + 2 * (uint32_t)((8 * r8 * (row_bytes + staged_idx_pad(row_bytes)) + 127) & ~127);
  L.red_off = L.act_off + (uint32_t)act_bufs * (uint32_t)((16 * (K + kActPad) + 127) & ~127);
  L.sa_off = L.red_off + (uint32_t)(warps * r8 * 4 * 32 * 4);
  L.bar_off = L.sa_off + 512;             // 16 token scales + 48 row scales + 48 row biases
  L.total = L.bar_off + 64;
  return L;
}

__device__ __forceinline__ void mma_m16n8k32_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#ifdef SACQ_TRACE
// Profiling builds only (-DSACQ_TRACE): CTA 0 records %globaltimer at the phase boundaries of
// the staged kernel (thread 0; slots 0..7 prologue, then 6 per tile).
__device__ long long g_small_trace[96];
#define SACQ_ST(slot) do { if (cta == 0 && threadIdx.x == 0 && (slot) < 96) { long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); g_small_trace[slot] = _t; } } while (0)
#else
#define SACQ_ST(slot) do { } while (0)
#endif

// HALVES = warps sharing one 32-index span (each takes 8/HALVES of its MMA steps): with
// two, a CTA runs up to 16 lighter warps, which hides more of the gather -> MMA latency.
// `cta` of `ncta` CTAs work on the layer described by p (a launch may cover several layers).
template <int D, int BITS, int R8, int HALVES>
__device__ __forceinline__ void staged_body(const SmallMParams& p, const int cta, const int ncta) {
  constexpr int NS = 8 / HALVES;           // MMA steps (vectors per lane) of one work item
  constexpr int NQ = NS * D / 16;          // uint4 loads covering them per token row
  extern __shared__ __align__(128) uint8_t smem[];
  using CwVec = typename std::conditional<D == 8, uint4, uint2>::type;
  constexpr int WPG = BITS / 4;
  constexpr int kFrag = R8 * 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const StagedLayout L = staged_layout(p.C, D, p.K, p.row_bytes, R8, nwarps);
  const CwVec* cbs = reinterpret_cast<const CwVec*>(smem + L.cb_off);
  uint8_t* act_base = smem + L.act_off;
  float* red = reinterpret_cast<float*>(smem + L.red_off);
  float* sa_s = reinterpret_cast<float*>(smem + L.sa_off);          // [16] token scales of the current chunk
  float* rowsc_s = sa_s + 16;                                         // [8*R8] scale of the tile's rows (group 0)
  float* rowb_s = rowsc_s + 48;                                       // [8*R8] bias of the tile's rows
  const uint32_t bar_cb = sm_addr(smem + L.bar_off), bar_act0 = bar_cb + 8, bar_idx0 = bar_cb + 24;
  const int act_pitch = p.K + kActPad;
  const uint32_t idx_buf_bytes = (L.act_off - L.idx_off) / 2;
  const uint32_t act_buf_bytes = 0;                  // a single activation tile
  SACQ_ST(0);
#ifdef SACQ_TRACE
  int _tl = -1;
  if (cta == 0 && threadIdx.x == 0) { _tl = (int)(atomicAdd(&g_timeline_count, 1u) & 511u); g_timeline[_tl].kind = 2; g_timeline[_tl].t_entry = tl_now(); }
#endif

  if (threadIdx.x == 0) {
    mbar_init(bar_cb, 1);
    mbar_init(bar_act0, 1);
    mbar_init(bar_act0 + 8, 1);
    mbar_init(bar_idx0, 1);
    mbar_init(bar_idx0 + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Work of this CTA: row tiles rt = blockIdx.x, + gridDim.x, ...; every row tile is
  // multiplied with all token chunks before the next one, so its packed indices are read
  // from HBM once.  Index tiles are double buffered (the next tile's copy flies during this
  // tile's compute); the 16-token activation tile is copied once when there is a single
  // chunk and once per (row tile, chunk) otherwise.
  // Called by threads 0 .. 8*R8-1.  Unpadded rows: thread 0 copies the tile's rows (one contiguous block
  // of the stream) at once.  Padded rows: every thread copies one row into its slot.  Either way thread 0
  // posts the expected byte count (its arrival is the one the barrier waits for).
  const uint32_t idx_pad = staged_idx_pad(p.row_bytes);
  const uint32_t idx_pitch = (uint32_t)p.row_bytes + idx_pad;
  auto issue_idx = [&](int rt, int buf) {
    const int n_base = rt * 8 * R8;
    const int rows = min(8 * R8, p.N - n_base);
    const int r = threadIdx.x;
    uint8_t* dst = smem + L.idx_off + buf * idx_buf_bytes;
    if (r == 0) mbar_expect_tx(bar_idx0 + 8 * buf, (uint32_t)(rows * p.row_bytes));
    if (idx_pad == 0) {
      if (r == 0)
        bulk_copy_g2s(dst, p.packed + (int64_t)n_base * p.row_bytes, (uint32_t)(rows * p.row_bytes), bar_idx0 + 8 * buf);
    } else if (r < rows) {
      bulk_copy_g2s(dst + r * idx_pitch, p.packed + (int64_t)(n_base + r) * p.row_bytes, (uint32_t)p.row_bytes,
                    bar_idx0 + 8 * buf);
    }
  };
  // Called by threads 0..15: thread 0 posts the expected byte count (its arrival is the one
  // the barrier waits for), every thread copies one token row.
  auto issue_act = [&](int chunk, int buf) {
    const int m_base = chunk * 16;
    const int toks = min(16, p.M - m_base);
    uint8_t* dst = act_base + buf * act_buf_bytes;
    const int m = threadIdx.x;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // earlier generic reads of the buffer
    if (m < toks)
      bulk_copy_g2s(dst + m * act_pitch, p.q + (int64_t)(m_base + m) * p.K, (uint32_t)p.K, bar_act0 + 8 * buf);
    if (m == 0) mbar_expect_tx(bar_act0 + 8 * buf, (uint32_t)(toks * p.K));
  };

  // This CTA's share: one token chunk (fixed for the CTA's lifetime, so its activation
  // tile is copied once) and the row tiles rt_first, rt_first + rt_stride, ...  The host
  // makes gridDim.x a multiple of the chunk count.
  const int chunk = cta % p.chunks;
  const int first_rt = cta / p.chunks;
  const int rt_stride = ncta / p.chunks;
  const int m_base = chunk * 16;
  const int toks_here = min(16, p.M - m_base);
  uint8_t* act_s = act_base;
  if (threadIdx.x == 0) {
    const uint32_t cb_bytes = (uint32_t)(p.C * D * 2);
    mbar_expect_tx(bar_cb, cb_bytes);
    bulk_copy_g2s(smem + L.cb_off, p.cb_hilo, cb_bytes, bar_cb);    // layer constants: may overlap
  }                                                                  // the previous kernel of the stream
  if (threadIdx.x < 8 * R8 && first_rt < p.row_blocks) issue_idx(first_rt, 0);
  // the next kernel of the stream (a quantizer or another GEMM launched with programmatic
  // serialization) may be scheduled from here on; it waits for this grid before it touches memory
  SACQ_ST(1);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");                // activations come from that kernel
  SACQ_ST(2);
  SACQ_TL(t_dep);
  if (threadIdx.x < 16 && first_rt < p.row_blocks) {
    issue_act(chunk, 0);
    sa_s[threadIdx.x] = threadIdx.x < toks_here ? __ldg(p.act_scale + m_base + threadIdx.x) : 0.f;
  }
  if (threadIdx.x < 8 * R8 && first_rt < p.row_blocks) {
    const int n = min(first_rt * 8 * R8 + (int)threadIdx.x, p.N - 1);
    rowsc_s[threadIdx.x] = bf16_bits_to_float(__ldg(p.scales + (int64_t)n * p.num_groups));
    rowb_s[threadIdx.x] = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
  }

  bool ok = true;
  uint32_t idx_parity[2] = {0, 0};
  bool first = true;
  int it = 0;
  for (int rt = first_rt; rt < p.row_blocks; rt += rt_stride, ++it) {
    const int buf = it & 1;
    const int n_base = rt * 8 * R8;
    const int rows_here = min(8 * R8, p.N - n_base);
    const uint8_t* idx_s = smem + L.idx_off + buf * idx_buf_bytes;
    // row constants (group-0 scale, bias): the NEXT tile's are fetched now into registers
    // and stored after this tile is done, so their global-memory latency hides behind a
    // whole tile; the first tile's were fetched before the loop
    float next_sc = 0.f, next_b = 0.f;
    if (threadIdx.x < 8 * R8 && rt + rt_stride < p.row_blocks) {
      const int n = min((rt + rt_stride) * 8 * R8 + (int)threadIdx.x, p.N - 1);
      next_sc = bf16_bits_to_float(__ldg(p.scales + (int64_t)n * p.num_groups));
      next_b = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
    }
    if (threadIdx.x < 8 * R8 && rt + rt_stride < p.row_blocks) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the other buffer's readers are done
      issue_idx(rt + rt_stride, buf ^ 1);
    }
    if (first) {
      ok = mbar_wait_bounded(bar_cb, 0, p.status) && ok;
      SACQ_ST(3);
      ok = mbar_wait_bounded(bar_act0, 0, p.status) && ok;
      SACQ_ST(4);
      SACQ_TL(t_ready);
      first = false;
    }
    ok = mbar_wait_bounded(bar_idx0 + 8 * buf, idx_parity[buf], p.status) && ok;
    idx_parity[buf] ^= 1;
    SACQ_ST(8 + 6 * it);
    ok = __syncthreads_and(ok);
    if (!ok) break;                                    // a bounded wait expired: status word is set
    SACQ_ST(8 + 6 * it + 1);

    // per-row scales of the two output rows this lane holds in each sub-block
    float s0[R8], s1[R8];
    int sn0[R8], sn1[R8];
#pragma unroll
    for (int r = 0; r < R8; ++r) {
      sn0[r] = min(n_base + r * 8 + 2 * t, p.N - 1);
      sn1[r] = min(n_base + r * 8 + 2 * t + 1, p.N - 1);
      s0[r] = rowsc_s[r * 8 + 2 * t];
      s1[r] = rowsc_s[r * 8 + 2 * t + 1];
    }
    float acc[R8][4];
#pragma unroll
    for (int r = 0; r < R8; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[r][j] = 0.f;
    float xs_a = 0.f, xs_b = 0.f;

    for (int item = warp; item < p.spans_per_row * HALVES; item += nwarps) {
      const int sp = item / HALVES, hf = item % HALVES;
      // A fragments are the raw e4m3 bytes: vector (8t + first + s) of token rows g and g+8.
      // FP8 MMAs need no widening; slots {4t..4t+3} carry bytes 0-3 and slots {16+4t..}
      // bytes 4-7 of the lane's vector (for d = 4: of its two vectors).
      constexpr int AW = NS * D / 4;             // 32-bit words per token row
      uint32_t fa[AW], fb[AW];
      {
        const int voff = (sp * kSpanIdx + 8 * t + hf * NS) * D;
        const uint4* pa = reinterpret_cast<const uint4*>(act_s + g * act_pitch + voff);
        const uint4* pb = reinterpret_cast<const uint4*>(act_s + (g + 8) * act_pitch + voff);
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
          const uint4 va = pa[j], vb = pb[j];
          fa[4 * j] = va.x; fa[4 * j + 1] = va.y; fa[4 * j + 2] = va.z; fa[4 * j + 3] = va.w;
          fb[4 * j] = vb.x; fb[4 * j + 1] = vb.y; fb[4 * j + 2] = vb.z; fb[4 * j + 3] = vb.w;
        }
      }
      if (g >= toks_here) {
#pragma unroll
        for (int j = 0; j < AW; ++j) fa[j] = 0u;
      }
      if (g + 8 >= toks_here) {
#pragma unroll
        for (int j = 0; j < AW; ++j) fb[j] = 0u;
      }
      if (p.shift != 0.f) {
        float ta = 0.f, tb = 0.f;
#pragma unroll
        for (int j = 0; j < AW; ++j) {
          uint32_t lo, hi;
          e4m3x4_to_h2(fa[j], lo, hi);
          ta += __low2float(as_h2(lo)) + __high2float(as_h2(lo)) + __low2float(as_h2(hi)) + __high2float(as_h2(hi));
          e4m3x4_to_h2(fb[j], lo, hi);
          tb += __low2float(as_h2(lo)) + __high2float(as_h2(lo)) + __low2float(as_h2(hi)) + __high2float(as_h2(hi));
        }
        ta += __shfl_xor_sync(0xffffffffu, ta, 1);
        ta += __shfl_xor_sync(0xffffffffu, ta, 2);
        tb += __shfl_xor_sync(0xffffffffu, tb, 1);
        tb += __shfl_xor_sync(0xffffffffu, tb, 2);
        xs_a += ta;
        xs_b += tb;
      }
      // Sub-blocks are processed RG at a time: their step accumulators interleave (independent MMA
      // chains), while the 48-row tile keeps only half of them live at once (register budget).
      constexpr int RG = R8 == 6 ? 3 : R8;
#pragma unroll
      for (int r0 = 0; r0 < R8; r0 += RG) {
        uint32_t wcur[RG][WPG];
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          const int rr = min((r0 + r) * 8 + g, rows_here - 1);
          const uint32_t* src = reinterpret_cast<const uint32_t*>(idx_s + rr * idx_pitch + sp * (4 * BITS) + t * BITS);
#pragma unroll
          for (int j = 0; j < WPG; ++j) wcur[r][j] = src[j];
        }
        // two accumulators per sub-block (even / odd steps) halve the dependent MMA chain
        float cs[RG][4], ct[RG][4];
#pragma unroll
        for (int r = 0; r < RG; ++r)
#pragma unroll
          for (int j = 0; j < 4; ++j) { cs[r][j] = 0.f; ct[r][j] = 0.f; }
        // the half index selects compile-time field positions, so dispatch on it once
        auto mma_steps = [&](auto HF) {
          constexpr int kFirst = decltype(HF)::value * NS;
          if constexpr (D == 8) {
            // one codeword per step: 16 bytes = e4m3 high half | low half
#pragma unroll
            for (int s8 = 0; s8 < NS; ++s8) {
#pragma unroll
              for (int r = 0; r < RG; ++r) {
                const uint4 c = cbs[field8<BITS>(wcur[r], kFirst + s8)];
                float (&acc2)[4] = (s8 & 1) ? ct[r] : cs[r];
                mma_m16n8k32_e4m3(acc2, fa[2 * s8], fb[2 * s8], fa[2 * s8 + 1], fb[2 * s8 + 1], c.x, c.y);
                mma_m16n8k32_e4m3(acc2, fa[2 * s8], fb[2 * s8], fa[2 * s8 + 1], fb[2 * s8 + 1], c.z, c.w);
              }
            }
          } else {
            // two 4-byte codewords per step (8 bytes each = high | low)
#pragma unroll
            for (int s2 = 0; s2 < NS / 2; ++s2) {
#pragma unroll
              for (int r = 0; r < RG; ++r) {
                const uint2 ca = cbs[field8<BITS>(wcur[r], kFirst + 2 * s2)];
                const uint2 cb2 = cbs[field8<BITS>(wcur[r], kFirst + 2 * s2 + 1)];
                float (&acc2)[4] = (s2 & 1) ? ct[r] : cs[r];
                mma_m16n8k32_e4m3(acc2, fa[2 * s2], fb[2 * s2], fa[2 * s2 + 1], fb[2 * s2 + 1], ca.x, cb2.x);
                mma_m16n8k32_e4m3(acc2, fa[2 * s2], fb[2 * s2], fa[2 * s2 + 1], fb[2 * s2 + 1], ca.y, cb2.y);
              }
            }
          }
        };
        if constexpr (HALVES == 1) {
          mma_steps(std::integral_constant<int, 0>{});
        } else {
          if (hf == 0) mma_steps(std::integral_constant<int, 0>{});
          else mma_steps(std::integral_constant<int, 1>{});
        }
#pragma unroll
        for (int r = 0; r < RG; ++r)
#pragma unroll
          for (int j = 0; j < 4; ++j) cs[r][j] += ct[r][j];
        if (p.num_groups > 1) {
          const int grp = (sp * kSpanIdx * D) / p.group_size;
#pragma unroll
          for (int r = 0; r < RG; ++r) {
            s0[r0 + r] = bf16_bits_to_float(__ldg(p.scales + (int64_t)sn0[r0 + r] * p.num_groups + grp));
            s1[r0 + r] = bf16_bits_to_float(__ldg(p.scales + (int64_t)sn1[r0 + r] * p.num_groups + grp));
          }
        }
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          acc[r0 + r][0] = fmaf(s0[r0 + r], cs[r][0], acc[r0 + r][0]);
          acc[r0 + r][1] = fmaf(s1[r0 + r], cs[r][1], acc[r0 + r][1]);
          acc[r0 + r][2] = fmaf(s0[r0 + r], cs[r][2], acc[r0 + r][2]);
          acc[r0 + r][3] = fmaf(s1[r0 + r], cs[r][3], acc[r0 + r][3]);
        }
      }
    }
    SACQ_ST(8 + 6 * it + 2);
#pragma unroll
    for (int r = 0; r < R8; ++r) {
      red[(warp * kFrag + r * 4 + 0) * 32 + lane] = fmaf(acc[r][0], p.out_mul, p.shift * xs_a);
      red[(warp * kFrag + r * 4 + 1) * 32 + lane] = fmaf(acc[r][1], p.out_mul, p.shift * xs_a);
      red[(warp * kFrag + r * 4 + 2) * 32 + lane] = fmaf(acc[r][2], p.out_mul, p.shift * xs_b);
      red[(warp * kFrag + r * 4 + 3) * 32 + lane] = fmaf(acc[r][3], p.out_mul, p.shift * xs_b);
    }
    __syncthreads();
    SACQ_ST(8 + 6 * it + 3);
    for (int e = threadIdx.x; e < kFrag * 32; e += blockDim.x) {
      float v = 0.f;
      for (int w = 0; w < nwarps; ++w) v += red[w * kFrag * 32 + e];
      const int ln = e & 31, j = (e >> 5) & 3, r = e >> 7;
      const int ml = (ln >> 2) + ((j & 2) ? 8 : 0);
      const int n = n_base + r * 8 + 2 * (ln & 3) + (j & 1);
      if (ml < toks_here && n < p.N) {
        store_out(p, m_base + ml, n, fmaf(sa_s[ml], v, rowb_s[n - n_base]));
      }
    }
    SACQ_ST(8 + 6 * it + 4);
    __syncthreads();                                   // red and the row constants are reused next
    SACQ_ST(8 + 6 * it + 5);
    if (threadIdx.x < 8 * R8) {
      rowsc_s[threadIdx.x] = next_sc;
      rowb_s[threadIdx.x] = next_b;
    }
  }
  if (first) {                                         // a CTA without a row tile still owns its copies
    mbar_wait_bounded(bar_cb, 0, p.status);
  }
  SACQ_ST(5);
  SACQ_TL(t_exit);
}

template <int D, int BITS, int R8, int HALVES>
__global__ void __launch_bounds__(kMaxWarps * 32 * HALVES, 1) small_m_mma_staged_kernel(const SmallMParams p) {
  staged_body<D, BITS, R8, HALVES>(p, (int)blockIdx.x, (int)gridDim.x);
}

// Several layers that read the same quantized activations (q/k/v, gate/up) in one launch:
// CTAs [cta_begin[l], cta_begin[l+1]) work on layer l.  Same geometry (K, d, index width,
// codebook size, grouping) for all layers; only the per-layer buffers and N differ.
template <int D, int BITS, int R8, int HALVES>
__global__ void __launch_bounds__(kMaxWarps * 32 * HALVES, 1) small_m_mma_staged_multi_kernel(const MultiParams g) {
  int l = 0;
  while (l + 1 < g.n_layers && (int)blockIdx.x >= g.cta_begin[l + 1]) ++l;
  SmallMParams p = g.base;
  p.packed = g.packed[l];
  p.cb_hilo = g.cb_hilo[l];
  p.scales = g.scales[l];
  p.bias = g.bias[l];
  p.status = g.status[l];
  p.y = g.y[l];
  p.ldy = g.ldy[l];
  p.N = g.N[l];
  p.row_blocks = g.row_blocks[l];
  p.out_mul = g.out_mul[l];
  p.shift = g.shift[l];
  staged_body<D, BITS, R8, HALVES>(p, (int)blockIdx.x - g.cta_begin[l], g.cta_begin[l + 1] - g.cta_begin[l]);
}

template <int D, int BITS>
cudaError_t launch_staged(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  switch (pl.r8) {
    case 1: return launch_kernel_pdl<small_m_mma_staged_kernel<D, BITS, 1, 2>>(pl, p, s);
    case 2: return launch_kernel_pdl<small_m_mma_staged_kernel<D, BITS, 2, 2>>(pl, p, s);
    case 6: return launch_kernel_pdl<small_m_mma_staged_kernel<D, BITS, 6, 2>>(pl, p, s);
    default: return launch_kernel_pdl<small_m_mma_staged_kernel<D, BITS, 4, 1>>(pl, p, s);
  }
}

template <auto Kern>
cudaError_t launch_multi_kernel(const Plan& pl, const MultiParams& g, cudaStream_t s) {
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
  return cudaLaunchKernelEx(&cfg, Kern, g);
}

template <int D, int BITS>
cudaError_t launch_staged_multi(const Plan& pl, const MultiParams& g, cudaStream_t s) {
  switch (pl.r8) {
    case 1: return launch_multi_kernel<small_m_mma_staged_multi_kernel<D, BITS, 1, 2>>(pl, g, s);
    case 2: return launch_multi_kernel<small_m_mma_staged_multi_kernel<D, BITS, 2, 2>>(pl, g, s);
    case 6: return launch_multi_kernel<small_m_mma_staged_multi_kernel<D, BITS, 6, 2>>(pl, g, s);
    default: return launch_multi_kernel<small_m_mma_staged_multi_kernel<D, BITS, 4, 1>>(pl, g, s);
  }
}

template <int D, int BITS, bool CB>
cudaError_t launch_r8(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  switch (pl.r8) {
    case 1: return launch_kernel<small_m_mma_kernel<D, BITS, CB, 1>>(pl, p, s);
    case 2: return launch_kernel<small_m_mma_kernel<D, BITS, CB, 2>>(pl, p, s);
    default: return launch_kernel<small_m_mma_kernel<D, BITS, CB, 4>>(pl, p, s);
  }
}

template <int D, int BITS>
cudaError_t launch_cb(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  return pl.cb_smem ? launch_r8<D, BITS, true>(pl, p, s) : launch_r8<D, BITS, false>(pl, p, s);
}

}  // namespace

#ifdef SACQ_TRACE
SACQ_TL_DEFINE_DUMP(sacq_debug_timeline_gemm)
extern "C" SACQ_API int sacq_debug_small_trace(long long* out) {
  return cudaMemcpyFromSymbol(out, g_small_trace, sizeof(g_small_trace)) == cudaSuccess ? 0 : -1;
}
#endif

size_t small_m_mma_staged_smem(int C, int D, int K, int64_t row_bytes, int r8, int warps, int act_bufs) {
  return staged_layout(C, D, K, row_bytes, r8, warps, act_bufs).total;
}

cudaError_t launch_small_m_mma_multi(const Plan& pl, const MultiParams& g, cudaStream_t s) {
  if (!pl.staged) return cudaErrorInvalidValue;
  if (pl.D == 8 && pl.BITS == 12) return launch_staged_multi<8, 12>(pl, g, s);
  if (pl.D == 8 && pl.BITS == 8) return launch_staged_multi<8, 8>(pl, g, s);
  if (pl.D == 8 && pl.BITS == 16) return launch_staged_multi<8, 16>(pl, g, s);
  if (pl.D == 4 && pl.BITS == 12) return launch_staged_multi<4, 12>(pl, g, s);
  if (pl.D == 4 && pl.BITS == 8) return launch_staged_multi<4, 8>(pl, g, s);
  if (pl.D == 4 && pl.BITS == 16) return launch_staged_multi<4, 16>(pl, g, s);
  return cudaErrorInvalidValue;
}

cudaError_t launch_small_m_mma(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  if (pl.staged) {
    if (pl.D == 8 && pl.BITS == 12) return launch_staged<8, 12>(pl, p, s);
    if (pl.D == 8 && pl.BITS == 8) return launch_staged<8, 8>(pl, p, s);
    if (pl.D == 8 && pl.BITS == 16) return launch_staged<8, 16>(pl, p, s);
    if (pl.D == 4 && pl.BITS == 12) return launch_staged<4, 12>(pl, p, s);
    if (pl.D == 4 && pl.BITS == 8) return launch_staged<4, 8>(pl, p, s);
    if (pl.D == 4 && pl.BITS == 16) return launch_staged<4, 16>(pl, p, s);
    return cudaErrorInvalidValue;
  }
  if (pl.D == 8 && pl.BITS == 12) return launch_cb<8, 12>(pl, p, s);
  if (pl.D == 8 && pl.BITS == 8) return launch_cb<8, 8>(pl, p, s);
  if (pl.D == 8 && pl.BITS == 16) return launch_cb<8, 16>(pl, p, s);
  if (pl.D == 4 && pl.BITS == 12) return launch_cb<4, 12>(pl, p, s);
  if (pl.D == 4 && pl.BITS == 8) return launch_cb<4, 8>(pl, p, s);
  if (pl.D == 4 && pl.BITS == 16) return launch_cb<4, 16>(pl, p, s);
  return cudaErrorInvalidValue;
}

}  // namespace smallm
}  // namespace sacq
