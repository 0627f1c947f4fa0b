// Small-M quantized linear, warp-MMA variant for ANY index width and group size.
//
// Same tile decomposition and data movement as the staged kernel in
// linear_small_m_mma.cu (bulk async copies of codebook, packed index rows and the 16
// activation rows; K split across the CTA's warps; reduction in shared memory), with two
// differences that make it independent of the bit format and of the scale grouping:
//
//   * after a tile's packed rows arrive, the CTA unpacks them once into 16-bit indices in
//     shared memory (runtime field width, aligned-word reads + funnel shift), so the MMA
//     loop never touches the bit stream;
//   * one MMA step covers 32 CONTIGUOUS k (4 vectors of 8, or 8 vectors of 4): lane t feeds
//     k-bytes [32*step + 8t, +8) of tokens g / g+8 as the A fragment and the matching
//     codeword halves as the B fragment.  A step therefore lies inside one scale group, and
//     the partial sums are folded with scale[n, group] whenever a group ends.
//
// This covers the layouts the reference actually deployed (d = 4, 64-wide groups, 5..11-bit
// indices; gr00t_libero/acceleration/presets/FROZEN_DECODE_SELECTION.json) as well as the
// benchmark's d = 8 / 12-bit / per-channel layers.
#include "small_m.cuh"

namespace sacq {
namespace smallm {

namespace {

constexpr int kActPadU = 32;                      // bytes of padding per staged activation row
constexpr int kMaxWarpsU = 16;

__device__ __forceinline__ uint32_t sm_addr_u(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(sm_addr_u(dst)), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_init_u(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_u(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_u(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ bool mbar_wait_u(uint32_t bar, uint32_t parity, int* status) {
  if (mbar_try_u(bar, parity)) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_u(bar, parity)) return true;
    if ((it & 255) == 255) {
      uint64_t t1;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t1 - t0 > 2000000000ull) {
        atomicExch(status, 3);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct UnpLayout {
  uint32_t cb_off, pk_off, pk_buf, idx_off, idx_pitch, act_off, act_pitch, sc_off, red_off, sa_off, bar_off, total;
};
__host__ __device__ inline UnpLayout unp_layout(int C, int D, int K, int64_t row_bytes, int num_groups, int r8,
                                                int warps) {
  UnpLayout L;
  const int rows = 8 * r8;
  L.cb_off = 0;
  L.pk_off = (uint32_t)((C * D * 2 + 127) & ~127);
  L.pk_buf = (uint32_t)((rows * row_bytes + 16 + 127) & ~127);        // + 16: the unpacker reads one word past a field
  L.idx_off = L.pk_off + 2 * L.pk_buf;
  L.idx_pitch = (uint32_t)((K / D) * 2 + 4);
  L.act_off = L.idx_off + (uint32_t)((rows * L.idx_pitch + 127) & ~127);
  L.act_pitch = (uint32_t)(K + kActPadU);
  L.sc_off = L.act_off + (uint32_t)((16 * L.act_pitch + 127) & ~127);
  L.red_off = L.sc_off + (uint32_t)((rows * num_groups * 4 + 127) & ~127);
  L.sa_off = L.red_off + (uint32_t)(warps * r8 * 4 * 32 * 4);
  L.bar_off = L.sa_off + 256;                                          // 16 token scales + up to 48 row biases
  L.total = L.bar_off + 64;
  return L;
}

template <int D, int R8>
__global__ void __launch_bounds__(kMaxWarpsU * 32, 1) small_m_mma_unpacked_kernel(const SmallMParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  using CwVec = typename std::conditional<D == 8, uint4, uint2>::type;   // e4m3 high half | low half
  constexpr int kFrag = R8 * 4;
  constexpr int kRows = 8 * R8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const UnpLayout L = unp_layout(p.C, D, p.K, p.row_bytes, p.num_groups, R8, nwarps);
  const CwVec* cbs = reinterpret_cast<const CwVec*>(smem + L.cb_off);
  uint16_t* idx16 = reinterpret_cast<uint16_t*>(smem + L.idx_off);
  uint8_t* act_s = smem + L.act_off;
  float* sc_s = reinterpret_cast<float*>(smem + L.sc_off);            // [kRows][num_groups]
  float* red = reinterpret_cast<float*>(smem + L.red_off);
  float* sa_s = reinterpret_cast<float*>(smem + L.sa_off);            // [16] token scales
  float* rowb_s = sa_s + 16;                                          // [kRows] biases
  const uint32_t bar_cb = sm_addr_u(smem + L.bar_off), bar_act = bar_cb + 8, bar_pk0 = bar_cb + 16;
  const int vpr = p.K / D;                                            // indices per row
  const int steps_total = p.K / 32;
  const int spg = p.group_size / 32;                                  // MMA steps per scale group
  const int spw = (steps_total + nwarps - 1) / nwarps;                // steps per warp

  if (threadIdx.x == 0) {
    mbar_init_u(bar_cb, 1);
    mbar_init_u(bar_act, 1);
    mbar_init_u(bar_pk0, 1);
    mbar_init_u(bar_pk0 + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // One token chunk per CTA (fixed), row tiles first_rt, first_rt + rt_stride, ...
  const int chunk = blockIdx.x % p.chunks;
  const int first_rt = blockIdx.x / p.chunks;
  const int rt_stride = gridDim.x / p.chunks;
  const int m_base = chunk * 16;
  const int toks_here = min(16, p.M - m_base);

  auto issue_packed = [&](int rt, int buf) {                          // thread 0 only
    const int n_base = rt * kRows;
    const uint32_t bytes = (uint32_t)(min(kRows, p.N - n_base) * p.row_bytes);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_expect_u(bar_pk0 + 8 * buf, bytes);
    bulk_g2s(smem + L.pk_off + buf * L.pk_buf, p.packed + (int64_t)n_base * p.row_bytes, bytes, bar_pk0 + 8 * buf);
  };

  if (threadIdx.x == 0) {
    const uint32_t cb_bytes = (uint32_t)(p.C * D * 2);
    mbar_expect_u(bar_cb, cb_bytes);
    bulk_g2s(smem + L.cb_off, p.cb_hilo, cb_bytes, bar_cb);           // layer constants: may overlap the
    if (first_rt < p.row_blocks) issue_packed(first_rt, 0);           // previous kernel of the stream
  }
  // the next kernel of the stream, if launched with programmatic serialization, may be scheduled
  // from here on (its launch latency overlaps this grid); it waits for this grid before it touches memory
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");                  // activations come from that kernel
  if (threadIdx.x < 16 && first_rt < p.row_blocks) {
    const int m = threadIdx.x;
    if (m < toks_here) bulk_g2s(act_s + m * L.act_pitch, p.q + (int64_t)(m_base + m) * p.K, (uint32_t)p.K, bar_act);
    if (m == 0) mbar_expect_u(bar_act, (uint32_t)(toks_here * p.K));
    sa_s[m] = m < toks_here ? __ldg(p.act_scale + m_base + m) : 0.f;
  }

  bool ok = true;
  uint32_t pk_parity[2] = {0, 0};
  bool first = true;
  int it = 0;
  for (int rt = first_rt; rt < p.row_blocks; rt += rt_stride, ++it) {
    const int buf = it & 1;
    const int n_base = rt * kRows;
    const int rows_here = min(kRows, p.N - n_base);
    if (threadIdx.x == 0 && rt + rt_stride < p.row_blocks) issue_packed(rt + rt_stride, buf ^ 1);
    // row constants of this tile: group scales and bias
    for (int e = threadIdx.x; e < kRows * p.num_groups; e += blockDim.x) {
      const int r = e / p.num_groups, gi = e - r * p.num_groups;
      const int n = min(n_base + r, p.N - 1);
      sc_s[e] = bf16_bits_to_float(__ldg(p.scales + (int64_t)n * p.num_groups + gi));
    }
    if (threadIdx.x < kRows) {
      const int n = min(n_base + (int)threadIdx.x, p.N - 1);
      rowb_s[threadIdx.x] = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
    }
    if (first) {
      ok = mbar_wait_u(bar_cb, 0, p.status) && ok;
      ok = mbar_wait_u(bar_act, 0, p.status) && ok;
      first = false;
    }
    ok = mbar_wait_u(bar_pk0 + 8 * buf, pk_parity[buf], p.status) && ok;
    pk_parity[buf] ^= 1;

    // ---- unpack the tile's bit stream into 16-bit indices, 8 fields per thread and turn
    {
      const uint32_t* pk = reinterpret_cast<const uint32_t*>(smem + L.pk_off + buf * L.pk_buf);
      const int groups_per_row = vpr >> 3;                            // K % 32 == 0 makes vpr a multiple of 4; see host
      const uint32_t mask = (1u << p.bits) - 1u;
      const int row_words = (int)(p.row_bytes >> 2);
      for (int e = threadIdx.x; e < rows_here * groups_per_row; e += blockDim.x) {
        const int r = e / groups_per_row, gq = e - r * groups_per_row;
        const uint32_t* w32 = pk + r * row_words;
        uint32_t out[4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int bit = (gq * 8 + i) * p.bits;
          const uint32_t v = __funnelshift_r(w32[bit >> 5], w32[(bit >> 5) + 1], bit & 31) & mask;
          if (i & 1) out[i >> 1] |= v << 16; else out[i >> 1] = v;
        }
        uint32_t* dst = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(idx16) + r * L.idx_pitch) + gq * 4;
        dst[0] = out[0]; dst[1] = out[1]; dst[2] = out[2]; dst[3] = out[3];
      }
    }
    ok = __syncthreads_and(ok);
    if (!ok) break;                                                   // a bounded wait expired: status word is set

    // ---- MMA steps of this warp: 32 contiguous k each
    float acc[R8][4], cs[R8][4];
#pragma unroll
    for (int r = 0; r < R8; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[r][j] = 0.f; cs[r][j] = 0.f; }
    float xs_a = 0.f, xs_b = 0.f;
    const int st_begin = warp * spw, st_end = min(st_begin + spw, steps_total);
    const uint8_t* arow_a = act_s + g * L.act_pitch + 8 * t;
    const uint8_t* arow_b = act_s + (g + 8) * L.act_pitch + 8 * t;
    const bool live_a = g < toks_here, live_b = g + 8 < toks_here;
    int ridx[R8];                                                     // byte offset of this lane's index row
#pragma unroll
    for (int r = 0; r < R8; ++r) ridx[r] = min(r * 8 + g, rows_here - 1) * (int)L.idx_pitch;

    int grp = st_begin / spg;                                         // scale group of the current step
    int to_fold = spg - (st_begin - grp * spg);                       // steps left in it
#pragma unroll 2
    for (int st = st_begin; st < st_end; ++st) {
      uint2 xa = *reinterpret_cast<const uint2*>(arow_a + st * 32);
      uint2 xb = *reinterpret_cast<const uint2*>(arow_b + st * 32);
      if (!live_a) xa = make_uint2(0u, 0u);
      if (!live_b) xb = make_uint2(0u, 0u);
      if (p.shift != 0.f) {
        uint32_t lo, hi;
        float ta = 0.f, tb = 0.f;
        e4m3x4_to_h2(xa.x, lo, hi);
        ta += __low2float(as_h2(lo)) + __high2float(as_h2(lo)) + __low2float(as_h2(hi)) + __high2float(as_h2(hi));
        e4m3x4_to_h2(xa.y, lo, hi);
        ta += __low2float(as_h2(lo)) + __high2float(as_h2(lo)) + __low2float(as_h2(hi)) + __high2float(as_h2(hi));
        e4m3x4_to_h2(xb.x, lo, hi);
        tb += __low2float(as_h2(lo)) + __high2float(as_h2(lo)) + __low2float(as_h2(hi)) + __high2float(as_h2(hi));
        e4m3x4_to_h2(xb.y, lo, hi);
        tb += __low2float(as_h2(lo)) + __high2float(as_h2(lo)) + __low2float(as_h2(hi)) + __high2float(as_h2(hi));
        ta += __shfl_xor_sync(0xffffffffu, ta, 1);
        ta += __shfl_xor_sync(0xffffffffu, ta, 2);
        tb += __shfl_xor_sync(0xffffffffu, tb, 1);
        tb += __shfl_xor_sync(0xffffffffu, tb, 2);
        xs_a += ta;
        xs_b += tb;
      }
#pragma unroll
      for (int r = 0; r < R8; ++r) {
        const uint8_t* irow = reinterpret_cast<const uint8_t*>(idx16) + ridx[r];
        if constexpr (D == 8) {
          const uint32_t idx = *reinterpret_cast<const uint16_t*>(irow + (st * 4 + t) * 2);
          const uint4 c = cbs[idx];
          mma_e4m3(cs[r], xa.x, xb.x, xa.y, xb.y, c.x, c.y);
          mma_e4m3(cs[r], xa.x, xb.x, xa.y, xb.y, c.z, c.w);
        } else {
          const uint32_t pair = *reinterpret_cast<const uint32_t*>(irow + (st * 8 + 2 * t) * 2);
          const uint2 c0 = cbs[pair & 0xffffu];
          const uint2 c1 = cbs[pair >> 16];
          mma_e4m3(cs[r], xa.x, xb.x, xa.y, xb.y, c0.x, c1.x);
          mma_e4m3(cs[r], xa.x, xb.x, xa.y, xb.y, c0.y, c1.y);
        }
      }
      --to_fold;
      if (to_fold == 0 || st + 1 == st_end) {                         // group (or this warp's share of it) ends
#pragma unroll
        for (int r = 0; r < R8; ++r) {
          const float s0 = sc_s[(r * 8 + 2 * t) * p.num_groups + grp];
          const float s1 = sc_s[(r * 8 + 2 * t + 1) * p.num_groups + grp];
          acc[r][0] = fmaf(s0, cs[r][0], acc[r][0]);
          acc[r][1] = fmaf(s1, cs[r][1], acc[r][1]);
          acc[r][2] = fmaf(s0, cs[r][2], acc[r][2]);
          acc[r][3] = fmaf(s1, cs[r][3], acc[r][3]);
          cs[r][0] = cs[r][1] = cs[r][2] = cs[r][3] = 0.f;
        }
        if (to_fold == 0) { ++grp; to_fold = spg; }
      }
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
      for (int w = 0; w < nwarps; ++w) v += red[w * kFrag * 32 + e];   // fixed order: deterministic
      const int ln = e & 31, j = (e >> 5) & 3, r = e >> 7;
      const int ml = (ln >> 2) + ((j & 2) ? 8 : 0);
      const int nl = r * 8 + 2 * (ln & 3) + (j & 1);
      if (ml < toks_here && n_base + nl < p.N)
        store_out(p, m_base + ml, n_base + nl, fmaf(sa_s[ml], v, rowb_s[nl]));
    }
    __syncthreads();                                                  // red, indices and row constants are reused
  }
  if (first) mbar_wait_u(bar_cb, 0, p.status);                        // never exit with the codebook copy in flight
}

template <int D>
cudaError_t launch_d(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  switch (pl.r8) {
    case 1: return launch_kernel_pdl<small_m_mma_unpacked_kernel<D, 1>>(pl, p, s);
    case 2: return launch_kernel_pdl<small_m_mma_unpacked_kernel<D, 2>>(pl, p, s);
    case 6: return launch_kernel_pdl<small_m_mma_unpacked_kernel<D, 6>>(pl, p, s);
    default: return launch_kernel_pdl<small_m_mma_unpacked_kernel<D, 4>>(pl, p, s);
  }
}

}  // namespace

size_t small_m_mma_unpacked_smem(int C, int D, int K, int64_t row_bytes, int num_groups, int r8, int warps) {
  return unp_layout(C, D, K, row_bytes, num_groups, r8, warps).total;
}

cudaError_t launch_small_m_mma_unpacked(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  if (pl.D == 8) return launch_d<8>(pl, p, s);
  if (pl.D == 4) return launch_d<4>(pl, p, s);
  return cudaErrorInvalidValue;
}

}  // namespace smallm
}  // namespace sacq
