// Small-M ("decode") quantized linear: y = s[m] * sum_k q[m,k] * W[n,k] + bias[n] for a
// handful of activation rows, reading the packed index stream exactly once.
//
// Stands in for the reference's small-M packed GEMMs (Triton
// codebook_linear_triton_2026_08_23.py:499-705 incl. its split-K variant, and the A8
// decode + small-M GEMM pair a8_accuracy_recovery_2026_10_20_r1/
// int8_aligned_index_decoder_20261028_r1.py:26-112 + int8_small_m_gemm_20261028_r1.py:7-32)
// without ever writing an expanded weight.
//
// Design (CUDA cores; tensor cores are left to the large-M kernel):
//   * persistent grid, one CTA per SM; each CTA stages the fp16 codebook in shared
//     memory once (64 KB for 4096 x 8);
//   * work item = (token chunk, block of 32 output rows, span group); a WARP owns an item,
//     lane = output row, and walks its row's slice of the index stream with 128-bit loads
//     (32 indices = 48 bytes at 12 bits);
//   * per index: one 128-bit shared-memory gather of the codeword, and per token one
//     broadcast 128-bit read of the activations and four HFMA2; fp16 partial sums are
//     flushed to fp32 every 32 products;
//   * K is split across warps/CTAs; partial sums meet in a global scratch buffer and the
//     last warp to arrive for a row block (arrival counter, no spinning) adds them in a
//     fixed order and applies the epilogue, so results do not depend on scheduling.
//
// Roofline: bound by HBM on the packed indices in principle (1.5 bits per weight); in
// practice the shared-memory gather rate (one 16-byte lookup per 8 weights) caps it.
#include "small_m.cuh"

namespace sacq {

using namespace smallm;

namespace {

// Adds the partial sums of one row block in span-group order and writes y.  Called by
// the last warp to arrive (or directly when K is not split).  `val` holds this warp's
// own MT partial sums for row n (already in true units).
template <int MT>
__device__ __forceinline__ void finish_rows(const SmallMParams& p, int chunk, int rb, int sg, float (&val)[MT],
                                            int n, bool row_ok) {
  const int m0 = chunk * MT;
  if (p.num_sg > 1) {
    // publish, then count arrivals
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (row_ok && m0 + m < p.M) p.partial[((int64_t)sg * p.M + (m0 + m)) * p.N + n] = val[m];
    __threadfence();
    __syncwarp();
    int old = 0;
    int* ctr = p.counters + (int64_t)chunk * p.row_blocks + rb;
    if ((threadIdx.x & 31) == 0) old = atomicAdd(ctr, 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != p.num_sg - 1) return;
    __threadfence();
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float t = 0.f;
      if (row_ok && m0 + m < p.M)
        for (int g = 0; g < p.num_sg; ++g) t += __ldcg(p.partial + ((int64_t)g * p.M + (m0 + m)) * p.N + n);
      val[m] = t;
    }
    __syncwarp();
    if ((threadIdx.x & 31) == 0) *ctr = 0;  // leave the counter region zero for the next call
  }
  if (!row_ok) return;
  const float b = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    if (m0 + m < p.M) {
      const float sa = __ldg(p.act_scale + m0 + m);
      store_out(p, m0 + m, n, fmaf(sa, val[m], b));
    }
  }
}

// Fast path: D in {4, 8}, BITS in {8, 12, 16}, rows of the packed stream 16-byte aligned,
// group_size a multiple of kSpanIdx * D.
//
// The inner loop is deliberately NOT unrolled over the whole span: a warp runs an item
// once, so straight-line code would be fetched from the instruction cache exactly once
// per warp; the body handles 8 indices (BITS/4 words) and is reused 4 times per span.
template <int D, int BITS, int MT, bool CB_SMEM>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) small_m_kernel(const SmallMParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  using CwVec = typename std::conditional<D == 8, uint4, uint2>::type;   // D halfs
  constexpr int WPG = BITS / 4;                                          // words per group of 8 indices
  constexpr int kFlush = 32 / D;        // indices between fp16 -> fp32 flushes (32 products)
  CwVec* cbs = reinterpret_cast<CwVec*>(smem);
  const int cb_bytes = CB_SMEM ? p.C * D * 2 : 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  // per-warp activation staging: [MT][kSpanIdx] vectors of D halfs
  CwVec* xs = reinterpret_cast<CwVec*>(smem + cb_bytes) + (size_t)warp * MT * kSpanIdx;

  if (CB_SMEM) {
    // asynchronous copies: every thread issues all of its 16-byte chunks before anyone waits
    const uint4* src = reinterpret_cast<const uint4*>(p.cb_f16);
    uint4* dst = reinterpret_cast<uint4*>(smem);
    const int n16 = cb_bytes >> 4;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) cp_async_16(dst + i, src + i);
  }

  // state of the current item
  int sg = 0, rb = 0, chunk = 0, m0 = 0, n = 0, nr = 0, sp_begin = 0, sp_end = 0;
  bool row_ok = false;
  const uint32_t* wsrc = nullptr;
  uint32_t wg[WPG];
  float xsum[MT];

  auto decode_item = [&](int64_t item) {
    sg = (int)(item % p.num_sg);
    const int64_t t1 = item / p.num_sg;
    rb = (int)(t1 % p.row_blocks);
    chunk = (int)(t1 / p.row_blocks);
    m0 = chunk * MT;
    n = rb * 32 + lane;
    row_ok = n < p.N;
    nr = row_ok ? n : p.N - 1;
    sp_begin = sg * p.spans_per_item;
    sp_end = min(sp_begin + p.spans_per_item, p.spans_per_row);
  };

  // Loads the lane's first 8 indices of span `sp` and stages the span's activations as
  // fp16 in the warp's shared-memory slice: xs[m][i] = q[m0+m, (sp*32+i)*D .. +D).
  auto load_span = [&](int sp) {
    wsrc = reinterpret_cast<const uint32_t*>(p.packed + (int64_t)nr * p.row_bytes + (int64_t)sp * (4 * BITS));
#pragma unroll
    for (int j = 0; j < WPG; ++j) wg[j] = __ldg(wsrc + j);
    __syncwarp();                       // previous span's readers are done with xs
    uint2 o[MT];
    const int64_t kbyte = ((int64_t)sp * kSpanIdx + lane) * D;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      o[m] = make_uint2(0, 0);
      if (m0 + m < p.M) {
        const uint8_t* src = p.q + (int64_t)(m0 + m) * p.K + kbyte;
        if constexpr (D == 8) o[m] = __ldg(reinterpret_cast<const uint2*>(src));
        else o[m].x = __ldg(reinterpret_cast<const uint32_t*>(src));
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      CwVec h;
      act4_to_h2(p.act_int8, o[m].x, h.x, h.y);
      if constexpr (D == 8) act4_to_h2(p.act_int8, o[m].y, h.z, h.w);
      xs[m * kSpanIdx + lane] = h;
      if (p.shift != 0.f) {
        float t = __low2float(as_h2(h.x)) + __high2float(as_h2(h.x)) + __low2float(as_h2(h.y)) +
                  __high2float(as_h2(h.y));
        if constexpr (D == 8)
          t += __low2float(as_h2(h.z)) + __high2float(as_h2(h.z)) + __low2float(as_h2(h.w)) +
               __high2float(as_h2(h.w));
        xsum[m] += warp_sum(t);
      }
    }
    __syncwarp();
  };

  const int64_t total_warps = (int64_t)gridDim.x * nwarps;
  int64_t item = (int64_t)warp * gridDim.x + blockIdx.x;
  bool have = item < p.num_items;
#pragma unroll
  for (int m = 0; m < MT; ++m) xsum[m] = 0.f;
  if (have) {
    decode_item(item);
    load_span(sp_begin);                // overlaps the codebook copy
  }
  if (CB_SMEM) {
    cp_async_wait_all();
    __syncthreads();                    // reached by every warp, with or without an item
  }

  while (have) {
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;

    for (int sp = sp_begin; sp < sp_end; ++sp) {
      float sacc[MT];
      __half2 hacc[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) { sacc[m] = 0.f; hacc[m] = __float2half2_rn(0.f); }

#pragma unroll 1
      for (int g = 0; g < kSpanIdx / 8; ++g) {
        uint32_t wn[WPG];
#pragma unroll
        for (int j = 0; j < WPG; ++j) wn[j] = (g + 1 < kSpanIdx / 8) ? __ldg(wsrc + (g + 1) * WPG + j) : 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t idx = field8<BITS>(wg, j);
          CwVec c;
          if constexpr (CB_SMEM) c = cbs[idx];
          else c = __ldg(reinterpret_cast<const CwVec*>(p.cb_f16) + idx);
          const CwVec* xrow = xs + g * 8 + j;
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const CwVec xv = xrow[m * kSpanIdx];
            hacc[m] = __hfma2(as_h2(c.x), as_h2(xv.x), hacc[m]);
            hacc[m] = __hfma2(as_h2(c.y), as_h2(xv.y), hacc[m]);
            if constexpr (D == 8) {
              hacc[m] = __hfma2(as_h2(c.z), as_h2(xv.z), hacc[m]);
              hacc[m] = __hfma2(as_h2(c.w), as_h2(xv.w), hacc[m]);
            }
          }
          if ((j % kFlush) == kFlush - 1) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              sacc[m] += __low2float(hacc[m]) + __high2float(hacc[m]);
              hacc[m] = __float2half2_rn(0.f);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < WPG; ++j) wg[j] = wn[j];
      }
      const int g = (sp * kSpanIdx * D) / p.group_size;
      const float s = bf16_bits_to_float(__ldg(p.scales + (int64_t)nr * p.num_groups + g));
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[m] = fmaf(s, sacc[m], acc[m]);
      if (sp + 1 < sp_end) load_span(sp + 1);
    }

    float val[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      val[m] = fmaf(acc[m], p.out_mul, p.shift * xsum[m]);
      xsum[m] = 0.f;
    }
    finish_rows<MT>(p, chunk, rb, sg, val, n, row_ok);

    item += total_warps;
    have = item < p.num_items;
    if (have) {
      decode_item(item);
      load_span(sp_begin);
    }
  }
}

// Generic path: any vector_dim, index width <= 24 bits, any group size, rows at any bit
// offset.  Same item structure, scalar fp32 math, codewords fetched from global memory.
template <int MT>
__global__ void __launch_bounds__(kMaxWarps * 32) small_m_generic_kernel(const SmallMParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int span_k = p.span_idx * p.d;
  float* xs = reinterpret_cast<float*>(smem) + (size_t)warp * MT * span_k;  // [MT][span_k]
  const uint32_t* words = reinterpret_cast<const uint32_t*>(p.packed);

  const int64_t total_warps = (int64_t)gridDim.x * nwarps;
  for (int64_t item = (int64_t)warp * gridDim.x + blockIdx.x; item < p.num_items; item += total_warps) {
    const int sg = (int)(item % p.num_sg);
    const int64_t t1 = item / p.num_sg;
    const int rb = (int)(t1 % p.row_blocks);
    const int chunk = (int)(t1 / p.row_blocks);
    const int m0 = chunk * MT;
    const int n = rb * 32 + lane;
    const bool row_ok = n < p.N;
    const int nr = row_ok ? n : p.N - 1;
    const int sp_begin = sg * p.spans_per_item;
    const int sp_end = min(sp_begin + p.spans_per_item, p.spans_per_row);

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;

    for (int sp = sp_begin; sp < sp_end; ++sp) {
      __syncwarp();
      const int kbase = sp * span_k;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        for (int k = lane; k < span_k; k += 32) {
          float v = 0.f;
          if (m0 + m < p.M) {
            const uint8_t b = __ldg(p.q + (int64_t)(m0 + m) * p.K + kbase + k);
            v = p.act_int8 ? (float)(int8_t)b
                           : __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3)));
          }
          xs[m * span_k + k] = v;
        }
      }
      __syncwarp();
      float sacc[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) sacc[m] = 0.f;
      const int64_t i0 = (int64_t)nr * p.vpr + (int64_t)sp * p.span_idx;
      const int g = kbase / p.group_size;
      const float s = bf16_bits_to_float(__ldg(p.scales + (int64_t)nr * p.num_groups + g));
      if (p.shift != 0.f) {
        // A shifted layer is contracted against the reference's reconstruction itself,
        // bf16(bf16(c * s) + shift) (cosmos_quant_shim.py:451-453): a large shift leaves the
        // weight only a few significant bits, so both roundings have to be reproduced.
        for (int i = 0; i < p.span_idx; ++i) {
          const uint32_t idx = extract_index(words, i0 + i, p.bits);
          for (int j = 0; j < p.d; ++j) {
            const float w = bf16_bits_to_float(reconstruct_bf16(__ldg(p.cb_bf16 + (int64_t)idx * p.d + j), s, p.shift));
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[m] = fmaf(w, xs[m * span_k + i * p.d + j], acc[m]);
          }
        }
        continue;
      }
      for (int i = 0; i < p.span_idx; ++i) {
        const uint32_t idx = extract_index(words, i0 + i, p.bits);
        for (int j = 0; j < p.d; ++j) {
          const float c = bf16_bits_to_float(__ldg(p.cb_bf16 + (int64_t)idx * p.d + j));
#pragma unroll
          for (int m = 0; m < MT; ++m) sacc[m] = fmaf(c, xs[m * span_k + i * p.d + j], sacc[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[m] = fmaf(s, sacc[m], acc[m]);
    }
    float val[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) val[m] = acc[m] * p.out_mul;
    finish_rows<MT>(p, chunk, rb, sg, val, n, row_ok);
  }
}

// ---- host side ---------------------------------------------------------------

inline int pick_mt(int64_t M) {
  if (M <= 1) return 1;
  if (M <= 2) return 2;
  if (M <= 4) return 4;
  if (M <= 8) return 8;
  return 16;
}

bool fast_eligible(const sacq_layer* L) {
  const sacq_layer_desc& d = L->d;
  if (d.vector_dim != 8 && d.vector_dim != 4) return false;
  if (d.index_bits != 8 && d.index_bits != 12 && d.index_bits != 16) return false;
  if (!L->rows_16b_aligned) return false;
  const int span_k = kSpanIdx * d.vector_dim;
  if (d.in_features % span_k != 0) return false;
  if (d.group_size % span_k != 0) return false;
  if (has_shift(L)) return false;            // shifted layers need the exact reconstruction (generic kernel)
  return true;
}

// The index-unpacking warp-MMA variant: any index width up to 16 bits, scale groups of any
// multiple of 32 weights.
bool unpacked_eligible(const sacq_layer* L) {
  const sacq_layer_desc& d = L->d;
  if (d.vector_dim != 8 && d.vector_dim != 4) return false;
  if (d.index_bits < 1 || d.index_bits > 16) return false;
  if (!L->rows_16b_aligned) return false;
  if (d.in_features % (8 * d.vector_dim) != 0 || d.in_features % 32 != 0) return false;
  if (d.group_size % 32 != 0) return false;
  const size_t cb_bytes = (size_t)L->cb_entries * d.vector_dim * 2;
  if (cb_bytes > 64 * 1024 || cb_bytes % 16 != 0) return false;
  if (has_shift(L)) return false;
  return true;
}

// Tallest tile (in 8-row sub-blocks) the planners may pick; compile-time switches for A/B measurements.
#ifndef SACQ_STAGED_MAX_R8
#define SACQ_STAGED_MAX_R8 6
#endif
#ifndef SACQ_UNPACKED_MAX_R8
#define SACQ_UNPACKED_MAX_R8 6
#endif

// Fills the plan for that variant; false if no tile height fits shared memory.
bool plan_unpacked(const sacq_layer* L, Plan& pl) {
  const sacq_layer_desc& d = L->d;
  const int64_t sub = (d.out_features + 7) / 8;
  const int steps = (int)(d.in_features / 32);
  const int warps = steps < 16 ? steps : 16;
  int64_t stride = L->num_sms / pl.chunks;
  if (stride < 1) stride = 1;
  double best_cost = -1.0;
  int best = 0;
  const int r8_choices[4] = {1, 2, 4, 6};                 // 48-row tiles: one tile per SM on 6144-row layers
  for (int ci = 0; ci < 4; ++ci) {
    const int r8 = r8_choices[ci];
    if (r8 > SACQ_UNPACKED_MAX_R8) continue;
    const size_t need = small_m_mma_unpacked_smem(L->cb_entries, d.vector_dim, (int)d.in_features, L->row_bits / 8,
                                                  (int)L->num_groups, r8, warps);
    if (need > kSmemBudget) continue;
    const int64_t row_tiles = (sub + r8 - 1) / r8;
    const int64_t waves = (row_tiles + stride - 1) / stride;
    // measured (us, dim-4 vectors with 64-wide groups on 2048 x 6144: 13.9 with three 16-row rounds, 11.95
    // with one 48-row tile): 2.5 of launch and codebook copy, then per pass over the tiles 1.0 of fixed cost plus
    // 1.4 per 8-row sub-block and 2048 of K (dim-8 vectors gather half as often)
    const double cost = 2.5 + (double)waves * (1.0 + (d.vector_dim == 4 ? 1.4 : 0.8) * r8 * (double)d.in_features / 2048.0);
    if (best_cost < 0 || cost < best_cost - 1e-9) { best_cost = cost; best = r8; }
  }
  if (best == 0) return false;
  pl.unpacked = true;
  pl.mma = true;
  pl.staged = true;
  pl.r8 = best;
  pl.warps = warps;
  pl.row_blocks = (int)((sub + best - 1) / best);
  pl.num_sg = 1;
  pl.spans_per_item = pl.spans_per_row;
  pl.num_items = (int64_t)pl.row_blocks * pl.chunks;
  if (stride > pl.row_blocks) stride = pl.row_blocks;
  pl.grid = (int)(stride * pl.chunks);
  if (pl.grid < 1) pl.grid = 1;
  pl.act_bufs = 1;
  pl.smem = small_m_mma_unpacked_smem(L->cb_entries, d.vector_dim, (int)d.in_features, L->row_bits / 8,
                                      (int)L->num_groups, best, warps);
  return true;
}

// M from which the warp-MMA variant is preferred over the CUDA-core one.
constexpr int64_t kMmaMinM = 1;

// halves_req: 0 = free choice of the tile height; 2 / 1 = only tile heights whose staged kernel
// runs two / one warp per span (the summation order of an output depends on that, not on N).
Plan make_plan(const sacq_layer* L, int64_t M, int halves_req = 0) {
  const sacq_layer_desc& d = L->d;
  Plan pl{};
  pl.fast = fast_eligible(L);
  pl.mma = pl.fast && (L->force_kernel == 4 || L->force_kernel == 5 || (L->force_kernel != 3 && M >= kMmaMinM));
  pl.MT = pl.mma ? 16 : pick_mt(M);
  pl.chunks = (int)((M + pl.MT - 1) / pl.MT);
  pl.row_blocks = (int)((d.out_features + 31) / 32);
  pl.D = d.vector_dim;
  pl.BITS = d.index_bits;
  if (pl.fast) {
    pl.span_idx = kSpanIdx;
    const size_t cb_bytes = (size_t)L->cb_entries * d.vector_dim * 2;
    pl.cb_smem = cb_bytes <= 64 * 1024;
  } else {
    // largest span (<= 32 vectors) that stays inside one scale group and divides the row
    int s = 32;
    const int vpg = d.group_size / d.vector_dim;
    while (s > 1 && (vpg % s != 0 || L->vectors_per_row % s != 0 || (size_t)s * d.vector_dim > 512)) s >>= 1;
    if (vpg % s != 0 || L->vectors_per_row % s != 0) s = 1;
    pl.span_idx = s;
    pl.cb_smem = false;
  }
  pl.spans_per_row = (int)(L->vectors_per_row / pl.span_idx);
  // Layers the span-based fast kernels cannot take (odd index widths, narrow scale groups)
  // go to the index-unpacking warp-MMA variant; selector 6 forces it for any eligible layer.
  if (unpacked_eligible(L) && (L->force_kernel == 6 || (!pl.fast && L->force_kernel != 3))) {
    const int mt = pl.MT, chunks = pl.chunks;
    pl.MT = 16;
    pl.chunks = (int)((M + 15) / 16);
    if (plan_unpacked(L, pl)) return pl;
    pl.MT = mt;
    pl.chunks = chunks;
  }
  if (pl.mma) {
    // tile = 16 tokens x 8*r8 rows; the CTA's warps split the K spans.
    const int64_t sub = (d.out_features + 7) / 8;
    pl.warps = pl.spans_per_row < kMaxWarps ? pl.spans_per_row : kMaxWarps;
    const size_t cb_bytes = pl.cb_smem ? (size_t)L->cb_entries * d.vector_dim * 2 : 0;
    const bool staged_ok = pl.cb_smem && L->force_kernel != 5 && d.in_features % 16 == 0 && cb_bytes % 16 == 0;
    int best = 1;
    bool best_staged = false;
    double best_cost = -1.0;
    // 48-row tiles (r8 = 6, staged kernel only): a 6144-row layer is then ONE tile on each of 128 SMs
    // instead of three 16-row tiles on each of 148, which saves two of the three per-tile round trips
    // (index wait, CTA barrier, cross-warp reduction, epilogue: about 1 us each)
    const int r8_choices[4] = {1, 2, 4, 6};
    for (int ci = 0; ci < 4; ++ci) {
      const int r8 = r8_choices[ci];
      if (halves_req != 0 && staged_halves(r8) != halves_req) continue;
      if (r8 > SACQ_STAGED_MAX_R8) continue;
      const int64_t row_tiles = (sub + r8 - 1) / r8;
      // staged kernel: a CTA walks row tiles and, inside each, all token chunks; the fixed
      // start-up (launch, codebook copy) is paid once.  Unit = one sub-block of one span set.
      // tiles of at most 16 rows run two warps per span (up to 16 warps per CTA)
      const int halves = staged_halves(r8);
      const int st_warps = pl.spans_per_row * halves < kMaxWarps * halves ? pl.spans_per_row * halves
                                                                          : kMaxWarps * halves;
      const size_t need = small_m_mma_staged_smem(L->cb_entries, d.vector_dim, (int)d.in_features,
                                                  L->row_bits / 8, r8, st_warps, 1);
      if (staged_ok && need <= kSmemBudget) {
        // CTAs are grouped per token chunk: a group walks the row tiles with this stride
        int64_t stride = L->num_sms / pl.chunks;
        if (stride < 1) stride = 1;
        const int64_t waves = (row_tiles + stride - 1) / stride;
        // measured (us): 2.5 of launch and codebook copy, then per pass over the tiles about 1.0 of fixed cost (index
        // wait, barriers, cross-warp reduction, epilogue) plus 0.7 per 8-row sub-block and 2048 of K
        const double cost = 2.5 + (double)waves * (1.0 + 0.7 * r8 * (double)d.in_features / 2048.0);
        if (best_cost < 0 || cost < best_cost - 1e-9 || !best_staged) { best_cost = cost; best = r8; best_staged = true; }
      } else if (!best_staged && r8 <= 4) {
        const int64_t tiles = row_tiles * pl.chunks;
        const int64_t waves = (tiles + L->num_sms - 1) / L->num_sms;
        const double cost = (double)waves * (3 + r8);
        if (best_cost < 0 || cost <= best_cost) { best_cost = cost; best = r8; }
      }
    }
    pl.r8 = best;
    pl.staged = best_staged;
    pl.row_blocks = (int)((sub + best - 1) / best);
    pl.spans_per_item = pl.spans_per_row;
    pl.num_sg = 1;
    pl.num_items = (int64_t)pl.row_blocks * pl.chunks;
    if (pl.staged) {
      // grid = chunks x (row-tile lanes per chunk), a multiple of the chunk count
      int64_t stride = L->num_sms / pl.chunks;
      if (stride < 1) stride = 1;
      if (stride > pl.row_blocks) stride = pl.row_blocks;
      pl.grid = (int)(stride * pl.chunks);
    } else {
      pl.grid = (int)(pl.num_items < L->num_sms ? pl.num_items : L->num_sms);
    }
    if (pl.grid < 1) pl.grid = 1;
    pl.act_bufs = 1;
    if (pl.staged) {
      const int halves = staged_halves(pl.r8);
      pl.warps = pl.spans_per_row * halves < kMaxWarps * halves ? pl.spans_per_row * halves : kMaxWarps * halves;
    }
    pl.smem = pl.staged ? small_m_mma_staged_smem(L->cb_entries, d.vector_dim, (int)d.in_features, L->row_bits / 8,
                                                  pl.r8, pl.warps, pl.act_bufs)
                        : cb_bytes + (size_t)pl.warps * pl.r8 * 4 * 32 * sizeof(float);
    return pl;
  }
  // Spread the row's spans over enough items to occupy every warp of the device once,
  // but no finer than one span per item.
  const int64_t base = (int64_t)pl.row_blocks * pl.chunks;
  const int64_t want = (int64_t)L->num_sms * 4;
  int per_item = pl.spans_per_row;
  while (per_item > 1 && base * ((pl.spans_per_row + per_item - 1) / per_item) < want) per_item = (per_item + 1) / 2;
  pl.spans_per_item = per_item;
  pl.num_sg = (pl.spans_per_row + per_item - 1) / per_item;
  pl.num_items = base * pl.num_sg;
  // one CTA per SM; warps per CTA: enough for the items, at most 8
  pl.grid = (int)(pl.num_items < L->num_sms ? pl.num_items : L->num_sms);
  if (pl.grid < 1) pl.grid = 1;
  int64_t warps_needed = (pl.num_items + pl.grid - 1) / pl.grid;
  pl.warps = (int)(warps_needed < 1 ? 1 : (warps_needed > kMaxWarps ? kMaxWarps : warps_needed));
  if (pl.fast) {
    const size_t cb_bytes = pl.cb_smem ? (size_t)L->cb_entries * d.vector_dim * 2 : 0;
    pl.smem = cb_bytes + (pl.mma ? 0 : (size_t)pl.warps * pl.MT * kSpanIdx * d.vector_dim * 2);
  } else {
    const size_t per_warp = (size_t)pl.MT * pl.span_idx * d.vector_dim * 4;
    while (pl.warps > 1 && per_warp * pl.warps > kSmemBudget) --pl.warps;
    pl.smem = per_warp * pl.warps;
  }
  return pl;
}

template <int D, int BITS, bool CB_SMEM>
cudaError_t launch_fast_mt(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  switch (pl.MT) {
    case 1: return launch_kernel<small_m_kernel<D, BITS, 1, CB_SMEM>>(pl, p, s);
    case 2: return launch_kernel<small_m_kernel<D, BITS, 2, CB_SMEM>>(pl, p, s);
    case 4: return launch_kernel<small_m_kernel<D, BITS, 4, CB_SMEM>>(pl, p, s);
    case 8: return launch_kernel<small_m_kernel<D, BITS, 8, CB_SMEM>>(pl, p, s);
    default: return launch_kernel<small_m_kernel<D, BITS, 16, CB_SMEM>>(pl, p, s);
  }
}

template <int D, int BITS>
cudaError_t launch_fast_cb(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  return pl.cb_smem ? launch_fast_mt<D, BITS, true>(pl, p, s) : launch_fast_mt<D, BITS, false>(pl, p, s);
}

cudaError_t launch_generic(const Plan& pl, const SmallMParams& p, cudaStream_t s) {
  switch (pl.MT) {
    case 1: return launch_kernel<small_m_generic_kernel<1>>(pl, p, s);
    case 2: return launch_kernel<small_m_generic_kernel<2>>(pl, p, s);
    case 4: return launch_kernel<small_m_generic_kernel<4>>(pl, p, s);
    case 8: return launch_kernel<small_m_generic_kernel<8>>(pl, p, s);
    default: return launch_kernel<small_m_generic_kernel<16>>(pl, p, s);
  }
}

}  // namespace

int small_m_int8_selector(const sacq_layer* L) { return fast_eligible(L) ? 5 : 3; }

bool small_m_supported(const sacq_layer* L) {
  return L->d.index_bits <= 24 && L->d.vector_dim <= 64;
}

int64_t small_m_workspace_bytes(const sacq_layer* L, int64_t M) {
  if (M <= 0) return sacq_workspace_counter_bytes();
  const Plan pl = make_plan(L, M);
  int64_t bytes = sacq_workspace_counter_bytes();
  if (pl.num_sg > 1) bytes += (int64_t)pl.num_sg * M * L->d.out_features * (int64_t)sizeof(float);
  return bytes;
}

// Scratch bytes (counter region included) and arrival counters the launch plan for (layer, M)
// uses; both come from the same plan launch_small_m() will make.
void small_m_scratch_need(const sacq_layer* L, int64_t M, int64_t* bytes, int64_t* counters) {
  const Plan pl = make_plan(L, M);
  *bytes = small_m_workspace_bytes(L, M);
  *counters = pl.num_sg > 1 ? (int64_t)pl.chunks * pl.row_blocks : 0;
}

namespace {
SmallMParams fill_params(const sacq_layer* L, const Plan& pl, const void* q, const float* scale, int64_t M, void* y,
                         int64_t ldy, void* ws) {
  const sacq_layer_desc& d = L->d;
  SmallMParams p{};
  p.packed = static_cast<const uint8_t*>(d.packed);
  p.cb_f16 = L->cb_f16;
  p.cb_hilo = L->cb_hilo;
  p.cb_bf16 = static_cast<const uint16_t*>(d.codebook);
  p.scales = static_cast<const uint16_t*>(d.scales);
  p.bias = static_cast<const uint16_t*>(d.bias);
  p.q = static_cast<const uint8_t*>(q);
  p.act_scale = scale;
  p.status = L->d_status;
  p.y = static_cast<uint16_t*>(y);
  p.counters = static_cast<int*>(ws);
  p.partial = ws ? reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + sacq_workspace_counter_bytes()) : nullptr;
  p.ldy = ldy;
  p.row_bytes = L->row_bits / 8;
  p.N = (int)d.out_features; p.K = (int)d.in_features; p.M = (int)M;
  p.vpr = (int)L->vectors_per_row;
  p.d = d.vector_dim; p.bits = d.index_bits;
  p.num_groups = (int)L->num_groups; p.group_size = d.group_size;
  p.C = L->cb_entries;
  p.span_idx = pl.span_idx; p.spans_per_row = pl.spans_per_row; p.spans_per_item = pl.spans_per_item;
  p.num_sg = pl.num_sg; p.row_blocks = pl.row_blocks; p.chunks = pl.chunks; p.num_items = pl.num_items;
  p.act_bufs = pl.act_bufs > 0 ? pl.act_bufs : 1;
  const uint32_t sb = (uint32_t)d.shift_bf16 << 16;
  memcpy(&p.shift, &sb, sizeof(float));
  p.out_mul = ldexpf(1.f, -L->cb8_exp_shift);
  return p;
}
}  // namespace

int launch_small_m(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                   void* ws, int64_t ws_bytes, cudaStream_t s, const void* residual, int64_t ldr, int act_int8,
                   const BcastDst* bc) {
  const sacq_layer_desc& d = L->d;
  if (M == 0 || d.out_features == 0) return SACQ_OK;
  if (M > (1 << 20)) return set_error(SACQ_ERR_UNSUPPORTED, "small-M kernel: M=%lld too large", (long long)M);
  const Plan pl = make_plan(L, M);
  if (L->force_kernel == 6 && !pl.unpacked)
    return set_error(SACQ_ERR_UNSUPPORTED, "index-unpacking warp-MMA variant cannot run this layer");
  if (has_shift(L) && L->force_kernel >= 4 && L->force_kernel <= 6)
    return set_error(SACQ_ERR_UNSUPPORTED, "a layer with a non-zero shift needs the exact reconstruction; the "
                                           "warp-MMA variants contract bare codewords");
  if (pl.smem > kSmemBudget)
    return set_error(SACQ_ERR_UNSUPPORTED, "small-M kernel needs %zu bytes of shared memory", pl.smem);
  const int64_t need = small_m_workspace_bytes(L, M);
  if (pl.num_sg > 1 && (int64_t)pl.chunks * pl.row_blocks * (int64_t)sizeof(int) > sacq_workspace_counter_bytes())
    return set_error(SACQ_ERR_UNSUPPORTED, "small-M kernel: %d x %d row-block counters exceed the counter region",
                     pl.chunks, pl.row_blocks);
  if (pl.num_sg > 1 && (ws == nullptr || ws_bytes < need))
    return set_error(SACQ_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given", (long long)need,
                     (long long)ws_bytes);
  if (pl.num_sg > 1 && reinterpret_cast<uintptr_t>(ws) % 16 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "workspace must be 16-byte aligned");

  SmallMParams p = fill_params(L, pl, q, scale, M, y, ldy, ws);
  p.residual = static_cast<const uint16_t*>(residual);
  p.ldr = ldr;
  p.act_int8 = act_int8;
  if (bc != nullptr) {
    p.n_bc = bc->n;
    for (int i = 0; i < bc->n; ++i) p.ybc[i] = static_cast<uint16_t*>(bc->ptr[i]);
  }
  if (act_int8 && pl.mma && (pl.staged || pl.unpacked))
    return set_error(SACQ_ERR_UNSUPPORTED, "the FP8 warp-MMA variants cannot take int8 activations");
  cudaError_t e;
  if (pl.unpacked) {
    if (reinterpret_cast<uintptr_t>(q) % 16 != 0)
      return set_error(SACQ_ERR_ALIGNMENT, "small-M MMA kernel: q must be 16-byte aligned");
    p.out_mul = ldexpf(1.f, -L->cb8_exp_shift);
    e = launch_small_m_mma_unpacked(pl, p, s);
  } else if (pl.fast) {
    if (reinterpret_cast<uintptr_t>(q) % 8 != 0 || d.in_features % 8 != 0)
      return set_error(SACQ_ERR_ALIGNMENT, "quantized activations must be 8-byte aligned with K %% 8 == 0");
    p.out_mul = ldexpf(1.f, (pl.mma && pl.staged) ? -L->cb8_exp_shift : -L->cb_exp_shift);
    if (pl.mma) {
      if (reinterpret_cast<uintptr_t>(q) % 16 != 0)
        return set_error(SACQ_ERR_ALIGNMENT, "small-M MMA kernel: q must be 16-byte aligned");
      e = launch_small_m_mma(pl, p, s);
    } else if (pl.D == 8 && pl.BITS == 12) e = launch_fast_cb<8, 12>(pl, p, s);
    else if (pl.D == 8 && pl.BITS == 8) e = launch_fast_cb<8, 8>(pl, p, s);
    else if (pl.D == 8 && pl.BITS == 16) e = launch_fast_cb<8, 16>(pl, p, s);
    else if (pl.D == 4 && pl.BITS == 12) e = launch_fast_cb<4, 12>(pl, p, s);
    else if (pl.D == 4 && pl.BITS == 8) e = launch_fast_cb<4, 8>(pl, p, s);
    else e = launch_fast_cb<4, 16>(pl, p, s);
  } else {
    p.out_mul = 1.f;
    e = launch_generic(pl, p, s);
  }
  count_launch();
  if (e != cudaSuccess) return cuda_fail(e, "small-M launch");
  return SACQ_OK;
}


// Several layers on the same quantized activations in one launch of the staged warp-MMA
// kernel.  Returns SACQ_ERR_UNSUPPORTED (and launches nothing) when the layers do not share a
// geometry that kernel can run; the caller then falls back to one launch per layer.
int launch_small_m_multi(const sacq_layer* const* layers, int n, const void* q, const float* scale, int64_t M,
                         void* const* ys, const int64_t* ldys, cudaStream_t s) {
  if (n < 2 || n > kMaxMulti || M <= 0 || M > (1 << 20)) return SACQ_ERR_UNSUPPORTED;
  const sacq_layer* L0 = layers[0];
  int64_t n_total = 0;
  for (int l = 0; l < n; ++l) {
    const sacq_layer_desc& a = layers[l]->d;
    const sacq_layer_desc& b = L0->d;
    if (a.in_features != b.in_features || a.vector_dim != b.vector_dim || a.index_bits != b.index_bits ||
        a.codebook_size != b.codebook_size || a.group_size != b.group_size || a.device != b.device ||
        layers[l]->force_kernel != 0 || a.out_features <= 0 || a.out_features % 8 != 0)
      return SACQ_ERR_UNSUPPORTED;
    n_total += a.out_features;
  }
  if (reinterpret_cast<uintptr_t>(q) % 16 != 0) return SACQ_ERR_UNSUPPORTED;
  // Every layer alone must be on the staged kernel with the same warps-per-span class: the
  // order in which an output's partial sums are added depends on it, and the results of
  // the shared launch are to be byte-identical to separate launches.
  int halves = 0;
  for (int l = 0; l < n; ++l) {
    const Plan one = make_plan(layers[l], M);
    if (!one.mma || !one.staged || one.unpacked) return SACQ_ERR_UNSUPPORTED;
    const int h = staged_halves(one.r8);
    if (halves != 0 && h != halves) return SACQ_ERR_UNSUPPORTED;
    halves = h;
  }
  // plan for the concatenation of the layers' rows: tile height and CTA count
  sacq_layer virt = *L0;
  virt.d.out_features = n_total;
  Plan pl = make_plan(&virt, M, halves);
  if (!pl.mma || !pl.staged || pl.unpacked || pl.smem > kSmemBudget || staged_halves(pl.r8) != halves)
    return SACQ_ERR_UNSUPPORTED;
  const int rows_per_tile = 8 * pl.r8;
  int rb[kMaxMulti], stride[kMaxMulti];
  int64_t rb_total = 0;
  for (int l = 0; l < n; ++l) {
    rb[l] = (int)((layers[l]->d.out_features + rows_per_tile - 1) / rows_per_tile);
    rb_total += rb[l];
  }
  int64_t stride_total = L0->num_sms / pl.chunks;
  if (stride_total < n) return SACQ_ERR_UNSUPPORTED;            // fewer CTA groups than layers
  if (stride_total > rb_total) stride_total = rb_total;
  int64_t used = 0;
  for (int l = 0; l < n; ++l) {
    int64_t v = stride_total * rb[l] / rb_total;
    if (v < 1) v = 1;
    if (v > rb[l]) v = rb[l];
    stride[l] = (int)v;
    used += v;
  }
  while (used > stride_total) {                                  // rounding up of small layers: take from the best served
    int best = -1;
    for (int l = 0; l < n; ++l)
      if (stride[l] > 1 && (best < 0 || (double)rb[l] / stride[l] < (double)rb[best] / stride[best])) best = l;
    if (best < 0) return SACQ_ERR_UNSUPPORTED;
    --stride[best];
    --used;
  }
  while (used < stride_total) {                                  // spare CTA groups go to the layer with the longest walk
    int best = -1;
    for (int l = 0; l < n; ++l)
      if (stride[l] < rb[l] && (best < 0 || (double)rb[l] / stride[l] > (double)rb[best] / stride[best])) best = l;
    if (best < 0) break;
    ++stride[best];
    ++used;
  }
  MultiParams g{};
  g.base = fill_params(L0, pl, q, scale, M, ys[0], ldys[0], nullptr);
  g.n_layers = n;
  int cta = 0;
  for (int l = 0; l < n; ++l) {
    const sacq_layer* L = layers[l];
    g.cta_begin[l] = cta;
    cta += stride[l] * pl.chunks;
    g.packed[l] = static_cast<const uint8_t*>(L->d.packed);
    g.cb_hilo[l] = L->cb_hilo;
    g.scales[l] = static_cast<const uint16_t*>(L->d.scales);
    g.bias[l] = static_cast<const uint16_t*>(L->d.bias);
    g.status[l] = L->d_status;
    g.y[l] = static_cast<uint16_t*>(ys[l]);
    g.ldy[l] = ldys[l];
    g.N[l] = (int)L->d.out_features;
    g.row_blocks[l] = rb[l];
    g.out_mul[l] = ldexpf(1.f, -L->cb8_exp_shift);
    const uint32_t sb = (uint32_t)L->d.shift_bf16 << 16;
    memcpy(&g.shift[l], &sb, sizeof(float));
  }
  g.cta_begin[n] = cta;
  pl.grid = cta;
  const cudaError_t e = launch_small_m_mma_multi(pl, g, s);
  count_launch();
  if (e != cudaSuccess) return cuda_fail(e, "small-M multi-layer launch");
  return SACQ_OK;
}
}  // namespace sacq
