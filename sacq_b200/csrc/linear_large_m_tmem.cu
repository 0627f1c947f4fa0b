// Large-M quantized linear with the expanded weights held in TENSOR MEMORY (sm_100a):
//   y[m,n] = bf16( s[m] * (sum_k q[m,k] * cb[idx[n,k/d], k%d]) * scale[n] + bias[n] )
//
// The kernel of linear_large_m.cu writes every expanded weight tile to shared memory, from
// where the tensor core reads it back together with the activation tile; its profile shows
// shared memory, not the tensor pipe, as the limit (codeword gathers + two tile stores per
// gather + the MMA's own operand reads all go through the same 128 bytes per clock).  Here
// the roles of the operands are swapped:
//   * the WEIGHTS are the MMA's A operand (128 weight rows = the 128 TMEM lanes) and live in
//     tensor memory: an expander thread owns one weight row, gathers its codewords' FP8 high
//     and low halves from the shared-memory codebook into registers and writes them with
//     tcgen05.st -- no shared-memory store, no swizzle arithmetic;
//   * the ACTIVATIONS are the B operand (N = tokens), TMA-loaded K-major / SWIZZLE_128B
//     tiles, read by the tensor core straight from shared memory;
//   * D[weight row, token] accumulates in TMEM: 128 lanes x (128 * NT) fp32 columns.
// Per 32-wide K step the issuer thread runs one MMA with the high and one with the low
// codeword halves into the same accumulator, so the summation order of an output element is
// the same for every tile shape (row shards of a layer reproduce it bit for bit).
//
// Shared-memory traffic per 128-k block drops to: activation operand reads + one 16-byte
// gather per codeword.  With NT = 3 (384 tokens per CTA: one N = 256 and one N = 128 MMA
// per half and K step) that is below what the tensor pipe needs for the same block.
//
// TMEM columns: [0, 128*NT) accumulator, then the weight stages: 64 columns each (32 = 128
// e4m3 bytes per lane of high halves, 32 of low halves); 2 stages with NT = 3, else 4.
//
// Roles: warp 0 = TMA producer (activation tiles, packed index tiles; no multicast),
// warp 1 = MMA issuer and TMEM owner, warps 2..9 = expanders and afterwards the epilogue
// (tcgen05.ld of the thread's weight row, fma(s[m], acc * scale[n], bias[n]), bf16 stores:
// the 32 lanes of a warp hold 32 consecutive n of one token, i.e. one 64-byte segment).
// Every mbarrier wait is bounded as in linear_large_m.cu.
//
// Stands in for the reference's decode-to-8-bit + 8-bit GEMM pair at batched sizes
// (a8_joint_pair_r1.py:38-127,374; perrow_a8_candidate_r3.py:56-69) and for its
// decode-in-mainloop GEMM (codebook_cutlass_kernel.cu:234-583).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "umma.cuh"
#include "tmem_weights.cuh"

namespace sacq {

namespace {

using namespace umma;
using namespace tmemw;

constexpr int kBK = 128;             // e4m3 bytes per K block (one 128-byte swizzle row)
constexpr int kMaxActStages = 4;
constexpr int kMaxWStages = 4;
struct TmemParams {
  const uint8_t* cb_hilo;       // [C][2][D] e4m3
  const uint16_t* scales;       // bf16 [N]
  const uint16_t* bias;         // bf16 [N] or null
  const float* act_scale;       // [M]
  uint16_t* y;                  // bf16 [M, ldy]
  const uint16_t* residual;     // bf16 [M, ldr] or null
  int64_t ldr;
  int64_t ldy;
  int n_bc;                     // further copies of the output (peer GPUs' buffers), same pitch as y
  uint16_t* ybc[kMaxBcast];
  int* status;
  int M, N, K, C;
  int act_stages;               // shared-memory activation stages, 2..kMaxActStages
  int y_tma;                    // the output goes out by tiled bulk stores (aligned y, no residual, no peer copies)
  float out_mul;                // 2^-cb8_exp_shift
};

struct TmemLayout {
  uint32_t act_off, act_stage, idx_off, idx_slot, cb_off, sw_off, bias_off, sa_off, bar_off, misc_off, total;
};

__host__ __device__ inline TmemLayout tmem_layout(int nt, int act_stages, int sb_bytes, int cb_bytes) {
  TmemLayout L;
  L.act_off = 0;
  L.act_stage = (uint32_t)(nt * kTokTile);
  L.idx_off = act_stages * L.act_stage;
  L.idx_slot = (uint32_t)(kRows * sb_bytes);
  L.cb_off = (L.idx_off + 2 * L.idx_slot + 127) & ~127u;
  L.sw_off = L.cb_off + (uint32_t)((cb_bytes + 127) & ~127);
  L.bias_off = L.sw_off + kRows * 4;
  L.sa_off = L.bias_off + kRows * 4;
  L.bar_off = L.sa_off + (uint32_t)(nt * kBM * 4);
  L.misc_off = L.bar_off + 32 * 8;
  L.total = L.misc_off + 64;
  return L;
}

// NIDX consecutive BITS-wide fields starting at field `first` (a multiple of NIDX) of a
// little-endian stream that begins at the 4-byte aligned address `base`.
template <int BITS, int NIDX>
__device__ __forceinline__ void load_fields_w(const uint8_t* base, int first, uint32_t (&out)[NIDX]) {
  constexpr int kBits = BITS * NIDX;
  constexpr uint32_t kMask = (1u << BITS) - 1u;
  if constexpr (kBits % 32 == 0) {
    constexpr int NW = kBits / 32;
    const uint32_t* w32 = reinterpret_cast<const uint32_t*>(base) + first * BITS / 32;
    uint32_t w[NW];
#pragma unroll
    for (int j = 0; j < NW; ++j) w[j] = w32[j];
#pragma unroll
    for (int j = 0; j < NIDX; ++j) {
      const int bit = j * BITS, word = bit >> 5, off = bit & 31;
      out[j] = (off + BITS <= 32) ? ((w[word] >> off) & kMask)
                                  : (__funnelshift_r(w[word], w[word + 1 < NW ? word + 1 : word], off) & kMask);
    }
  } else {
    // a window of at most 48 bits at a 16-bit aligned offset: two words (the second may belong to
    // the next row of the index tile; it is read, not used)
    static_assert(kBits <= 48, "unaligned windows must fit 64 bits after a 16-bit offset");
    const uint32_t* w32 = reinterpret_cast<const uint32_t*>(base);
    const int start = first * BITS;
    const uint64_t v = (((uint64_t)w32[(start >> 5) + 1] << 32) | w32[start >> 5]) >> (start & 31);
#pragma unroll
    for (int j = 0; j < NIDX; ++j) out[j] = (uint32_t)(v >> (j * BITS)) & kMask;
  }
}

#ifdef SACQ_TRACE
// Profiling builds only (-DSACQ_TRACE): CTA (0, 0) records %globaltimer at a few points per role.
__device__ long long g_tmem_trace[8][72];
#define SACQ_TR(role, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (slot) < 72) { long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); g_tmem_trace[role][slot] = _t; } } while (0)
// Ablation switches of profiling builds (results are wrong with any of them set): 1 = no codeword gathers,
// 2 = no tcgen05.st of the weights, 4 = activation tiles loaded for the first round of stages only, 8 = no MMAs.
__device__ int g_tmem_ablate = 0;
#define SACQ_ABLATE(bit) (g_tmem_ablate & (bit))
#else
#define SACQ_TR(role, slot) do { } while (0)
#define SACQ_ABLATE(bit) false
#endif

// D in {4, 8}; BITS in {8, 12, 16}; NT = 128-token sub-tiles per CTA (1, 2 or 3); CB_SMEM: the
// high/low codebook is staged in shared memory, else (a table too large for it: 65,536 entries)
// gathered from global memory, where it stays L2-resident.
// grid = (ceil(N / 128), ceil(M / (128 * NT))).  The last token tile may hold fewer valid
// sub-tiles: only those are loaded and multiplied.
template <int D, int BITS, int NT, bool CB_SMEM>
__global__ void __launch_bounds__(kCtaThreads, 1)
large_m_tmem_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_idx,
                    const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ BcastMaps tmap_bc,
                    const __grid_constant__ TmemParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int BT = kBM * NT;                        // tokens per CTA = accumulator columns
  constexpr int IDX_PER_KB = kBK / D;                 // indices per row per K block
  constexpr int KB_BYTES = IDX_PER_KB * BITS / 8;     // index bytes per row per K block
  constexpr int SB_BYTES = 2 * KB_BYTES;              // ... per super block (two K blocks): multiple of 16
  constexpr int CW_BYTES = 2 * D;                     // hi + lo bytes per codeword
  // A TMEM weight stage holds W_K k of the 128 rows.  Half-block stages (W_K = 64, four of them beside
  // a 384-column accumulator instead of two whole blocks) were measured SLOWER (2048x6144 at M = 8192:
  // 217 against 183 us): the per-stage cost of the expanders (barrier waits, tcgen05.wait::st, fences)
  // does not shrink with the stage.
  constexpr int W_K = 128;
  constexpr int WPB = kBK / W_K;                      // weight stages per K block
  constexpr int W_COLS = W_K / 2;                     // TMEM columns of a stage: W_K / 4 high + W_K / 4 low
  constexpr int WQ = W_K / 16;                        // 32-bit words a thread writes per half (4 or 8)
  constexpr int IPT = (W_K / D) / 4;                  // indices per expander thread per weight stage (a quarter row)
  constexpr int kWStages = NT == 3 ? 2 : kMaxWStages; // TMEM weight stages
  constexpr uint32_t kWCol0 = BT;                     // first weight-stage column
  constexpr uint32_t kTmemCols = 512;
  static_assert(BT + kWStages * W_COLS <= 512, "TMEM budget");
  constexpr uint32_t kIdesc256 = make_idesc(256), kIdesc128 = make_idesc(128), kIdesc192 = make_idesc(192);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const TmemLayout L = tmem_layout(NT, p.act_stages, SB_BYTES, CB_SMEM ? p.C * CW_BYTES : 0);

  // barrier indices
  constexpr int ACT_FULL = 0, ACT_EMPTY = kMaxActStages, W_FULL = 2 * kMaxActStages,
                W_EMPTY = 2 * kMaxActStages + kMaxWStages, IDX_FULL = 2 * kMaxActStages + 2 * kMaxWStages,
                IDX_EMPTY = IDX_FULL + 2, ACC_FULL = IDX_FULL + 4, CB_FULL = IDX_FULL + 5;
  const uint32_t bars = base + L.bar_off;
  auto bar = [&](int i) { return bars + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + L.misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + L.misc_off + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kRows;
  const int m0 = blockIdx.y * BT;
  const int num_kb = p.K / kBK;
  const int act_stages = p.act_stages;
  const uint32_t cb_bytes = (uint32_t)(p.C * CW_BYTES);
  const int nt_valid = min(NT, (p.M - m0 + kBM - 1) / kBM);       // sub-tiles of this CTA that hold tokens

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxActStages; ++i) {
      mbar_init(bar(ACT_FULL + i), 1);
      mbar_init(bar(ACT_EMPTY + i), 1);
    }
    for (int i = 0; i < kMaxWStages; ++i) {
      mbar_init(bar(W_FULL + i), kXWarps);
      mbar_init(bar(W_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(IDX_FULL + i), 1);
      mbar_init(bar(IDX_EMPTY + i), kXWarps);
    }
    mbar_init(bar(ACC_FULL), 1);
    mbar_init(bar(CB_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_idx);
    if (p.y_tma) prefetch_tensormap(&tmap_y);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) SACQ_TR(0, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      if constexpr (CB_SMEM) {
        mbar_arrive_expect_tx(bar(CB_FULL), cb_bytes);
        bulk_load(base + L.cb_off, p.cb_hilo, cb_bytes, bar(CB_FULL));
      }
      for (int kb = 0; kb < num_kb; ++kb) {
        if ((kb & 1) == 0) {
          const int sb = kb >> 1, slot = sb & 1;
          if (!mbar_wait(bar(IDX_EMPTY + slot), ((sb >> 1) & 1) ^ 1, abort_flag, p.status)) break;
          mbar_arrive_expect_tx(bar(IDX_FULL + slot), kRows * SB_BYTES);
          tma_load_2d(base + L.idx_off + slot * L.idx_slot, &tmap_idx, sb * SB_BYTES, n0, bar(IDX_FULL + slot));
        }
        const int st = kb % act_stages;
        if (!mbar_wait(bar(ACT_EMPTY + st), ((kb / act_stages) & 1) ^ 1, abort_flag, p.status)) break;
        if (SACQ_ABLATE(4) && kb >= act_stages) {      // no loads: the stage keeps its first tile
          mbar_arrive(bar(ACT_FULL + st));
          continue;
        }
        mbar_arrive_expect_tx(bar(ACT_FULL + st), nt_valid * kTokTile);
#pragma unroll
        for (int t = 0; t < NT; ++t)
          if (t < nt_valid)
            tma_load_2d(base + L.act_off + st * L.act_stage + t * kTokTile, &tmap_a, kb * kBK, m0 + t * kBM,
                        bar(ACT_FULL + st));
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int wb = 0; wb < num_kb * WPB && ok; ++wb) {
        const int kb = wb / WPB, sub = wb % WPB;       // K block and which part of it this weight stage holds
        const int st = kb % act_stages, ws = wb % kWStages;
        ok = (sub != 0 || mbar_wait(bar(ACT_FULL + st), (kb / act_stages) & 1, abort_flag, p.status)) &&
             mbar_wait(bar(W_FULL + ws), (wb / kWStages) & 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        SACQ_TR(1, wb + 8);
        const uint32_t act_addr = base + L.act_off + st * L.act_stage;
        const uint32_t w_col = kWCol0 + (uint32_t)(ws * W_COLS);
#pragma unroll
        for (int ksl = 0; ksl < W_K / 32; ++ksl) {
          const int ks = sub * (W_K / 32) + ksl;       // 32-byte K step inside the 128-byte activation rows
          const uint64_t adv = (uint64_t)((ks * 32) >> 4);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (SACQ_ABLATE(8)) continue;
            const uint32_t a_tmem = tmem_base + w_col + (uint32_t)(half * (W_COLS / 2) + ksl * 8);
            const uint32_t acc = (wb | ksl | half) != 0;
            // 384 tokens go as two N = 192 instructions into two accumulators, not as N = 256 + N = 128: an
            // instruction costs about the same 60 ns for any N from 128 to 256 (microbenchmark: the pair
            // takes 114 against 126 ns), and consecutive instructions into ONE accumulator wait for each
            // other (137 ns each), so the two accumulators alternate
            if (NT == 3 && nt_valid == 3) {
              umma_f8_ts(tmem_base, a_tmem, make_smem_desc(act_addr) + adv, kIdesc192, acc);
              umma_f8_ts(tmem_base + 192u, a_tmem, make_smem_desc(act_addr + kTokTile * 3 / 2) + adv, kIdesc192, acc);
            } else if (NT >= 2 && nt_valid >= 2) {
              umma_f8_ts(tmem_base, a_tmem, make_smem_desc(act_addr) + adv, kIdesc256, acc);
            } else {
              umma_f8_ts(tmem_base, a_tmem, make_smem_desc(act_addr) + adv, kIdesc128, acc);
            }
          }
        }
        if (sub == WPB - 1) umma_commit(bar(ACT_EMPTY + st));
        umma_commit(bar(W_EMPTY + ws));
      }
      if (ok) umma_commit(bar(ACC_FULL));
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ expanders, then epilogue
    const int et = threadIdx.x - 64;                 // 0..511
    const int quarter = warp & 3;                    // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;             // weight row of the tile = TMEM lane
    const int kpart = (warp - 2) >> 2;               // which 32 bytes of the 128-byte K block (0..3)
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    {
      if (et < kRows) {
        const int n = min(n0 + et, p.N - 1);
        reinterpret_cast<float*>(sm + L.sw_off)[et] = bf16_bits_to_float(__ldg(p.scales + n)) * p.out_mul;
        reinterpret_cast<float*>(sm + L.bias_off)[et] = p.bias ? bf16_bits_to_float(__ldg(p.bias + n)) : 0.f;
      }
      for (int i = et; i < BT; i += kXThreads) {
        const int m = m0 + i;
        reinterpret_cast<float*>(sm + L.sa_off)[i] = m < p.M ? __ldg(p.act_scale + m) : 0.f;
      }
      xbarrier();
    }
    const uint8_t* cbs = CB_SMEM ? sm + L.cb_off : p.cb_hilo;
    bool ok = CB_SMEM ? mbar_wait(bar(CB_FULL), 0, abort_flag, p.status) : true;
    for (int wb = 0; wb < num_kb * WPB && ok; ++wb) {
      const int kb = wb / WPB, sub = wb % WPB;
      const int sb = kb >> 1, slot = sb & 1;
      const int ws = wb % kWStages;
      ok = (sub != 0 || mbar_wait(bar(IDX_FULL + slot), (sb >> 1) & 1, abort_flag, p.status)) &&
           mbar_wait(bar(W_EMPTY + ws), ((wb / kWStages) & 1) ^ 1, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after();                              // the MMAs that read this stage are complete
      if (warp == 2 && lane == 0) SACQ_TR(2, wb + 8);
      uint32_t idx[IPT];
      load_fields_w<BITS, IPT>(sm + L.idx_off + slot * L.idx_slot + row * SB_BYTES + (kb & 1) * KB_BYTES +
                                   sub * (KB_BYTES / WPB),
                               kpart * IPT, idx);
      uint32_t hi[WQ], lo[WQ];
      if (SACQ_ABLATE(1)) {
#pragma unroll
        for (int j = 0; j < WQ; ++j) { hi[j] = idx[j % IPT]; lo[j] = idx[j % IPT] >> 3; }
      } else if constexpr (D == 8) {
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
          const uint4 c = CB_SMEM ? *reinterpret_cast<const uint4*>(cbs + (size_t)idx[j] * 16)
                                  : __ldg(reinterpret_cast<const uint4*>(cbs + (size_t)idx[j] * 16));
          hi[2 * j] = c.x; hi[2 * j + 1] = c.y;
          lo[2 * j] = c.z; lo[2 * j + 1] = c.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
          const uint2 c = CB_SMEM ? *reinterpret_cast<const uint2*>(cbs + (size_t)idx[j] * 8)
                                  : __ldg(reinterpret_cast<const uint2*>(cbs + (size_t)idx[j] * 8));
          hi[j] = c.x;
          lo[j] = c.y;
        }
      }
      // the thread's quarter of the stage's k: WQ columns of the high half, WQ of the low half
      const uint32_t w_addr = lane_addr + kWCol0 + (uint32_t)(ws * W_COLS + kpart * WQ);
      if (!SACQ_ABLATE(2)) {
        tmem_st_32xn(w_addr, hi);
        tmem_st_32xn(w_addr + (uint32_t)(W_COLS / 2), lo);
      } else if (hi[0] + lo[WQ - 1] == 0x12345678u) {
        p.status[0] = 99;                              // never true in practice: keeps the gathers alive
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (warp == 2 && lane == 0) SACQ_TR(5, wb + 8);
      if (lane == 0) {
        mbar_arrive(bar(W_FULL + ws));
        if (sub == WPB - 1 && ((kb & 1) == 1 || kb == num_kb - 1)) mbar_arrive(bar(IDX_EMPTY + slot));
      }
    }

    // ---- epilogue
    if (ok) ok = mbar_wait(bar(ACC_FULL), 0, abort_flag, p.status);
    if (warp == 2 && lane == 0) SACQ_TR(0, 3);
    ok = xall(ok);                                    // tcgen05.ld and the staging barriers are collective
    if (ok) {
      tc_fence_after();
      TmemOut o;
      o.y = p.y; o.ldy = p.ldy; o.residual = p.residual; o.ldr = p.ldr; o.n_bc = p.n_bc;
      for (int i = 0; i < p.n_bc; ++i) o.ybc[i] = p.ybc[i];
      o.M = p.M; o.N = p.N; o.y_tma = p.y_tma;
      const float sw = reinterpret_cast<const float*>(sm + L.sw_off)[row];
      const float bs = reinterpret_cast<const float*>(sm + L.bias_off)[row];
      tmem_epilogue<NT>(o, &tmap_y, tmap_bc.m, lane_addr, row, kpart, et, reinterpret_cast<const float*>(sm + L.sa_off), sw, bs,
                        sm + L.act_off, (act_stages * L.act_stage >= 2u * kStageTile) ? 2 : 1, m0, n0);
    }
  }

  // ---- common exit: every thread arrives here, also after an aborted wait
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) SACQ_TR(0, 4);
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

int sb_bytes_of(const sacq_layer* L) { return 2 * (kBK / L->d.vector_dim) * L->d.index_bits / 8; }

// Shared memory of a launch; the request is padded above half an SM's capacity so that two CTAs
// (each of which takes all 512 TMEM columns) never share an SM.
size_t smem_request(const TmemLayout& lay) {
  const size_t need = lay.total + 1024;
  return need < 120 * 1024 ? 120 * 1024 : need;
}

// Codebooks up to 64 KB (high + low halves) are staged in shared memory, larger ones gathered from global memory.
bool cb_in_smem(const sacq_layer* L) { return (size_t)L->cb_entries * L->d.vector_dim * 2 <= 64 * 1024; }

int pick_act_stages(const sacq_layer* L, int nt) {
  const int cb_bytes = cb_in_smem(L) ? L->cb_entries * L->d.vector_dim * 2 : 0;
  for (int st = (nt == 3 ? 3 : kMaxActStages); st >= 2; --st)
    if (tmem_layout(nt, st, sb_bytes_of(L), cb_bytes).total + 1024 <= 227 * 1024) return st;
  return 0;
}

template <int D, int BITS, int NT, bool CB_SMEM>
cudaError_t launch_nt(const CUtensorMap& ta, const CUtensorMap& ti, const CUtensorMap& ty, const BcastMaps& tb,
                      const TmemParams& p, dim3 grid, size_t smem, cudaStream_t s) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(large_m_tmem_kernel<D, BITS, NT, CB_SMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  large_m_tmem_kernel<D, BITS, NT, CB_SMEM><<<grid, kCtaThreads, smem, s>>>(ta, ti, ty, tb, p);
  return cudaGetLastError();
}

template <int D, int BITS>
cudaError_t launch_db(const CUtensorMap& ta, const CUtensorMap& ti, const CUtensorMap& ty, const BcastMaps& tb,
                      const TmemParams& p, int nt, bool cb_smem, dim3 grid, size_t smem, cudaStream_t s) {
  if (!cb_smem) {
    if (nt == 3) return launch_nt<D, BITS, 3, false>(ta, ti, ty, tb, p, grid, smem, s);
    if (nt == 2) return launch_nt<D, BITS, 2, false>(ta, ti, ty, tb, p, grid, smem, s);
    return launch_nt<D, BITS, 1, false>(ta, ti, ty, tb, p, grid, smem, s);
  }
  if (nt == 3) return launch_nt<D, BITS, 3, true>(ta, ti, ty, tb, p, grid, smem, s);
  if (nt == 2) return launch_nt<D, BITS, 2, true>(ta, ti, ty, tb, p, grid, smem, s);
  return launch_nt<D, BITS, 1, true>(ta, ti, ty, tb, p, grid, smem, s);
}

}  // namespace

#ifdef SACQ_TRACE
extern "C" SACQ_API int sacq_debug_tmem_trace(long long* out) {
  return cudaMemcpyFromSymbol(out, g_tmem_trace, sizeof(long long) * 8 * 72) == cudaSuccess ? 0 : -1;
}
extern "C" SACQ_API int sacq_debug_tmem_ablate(int flags) {
  return cudaMemcpyToSymbol(g_tmem_ablate, &flags, sizeof(int)) == cudaSuccess ? 0 : -1;
}
#endif

bool large_m_tmem_supported(const sacq_layer* L) {
  const sacq_layer_desc& d = L->d;
  if (d.vector_dim != 8 && d.vector_dim != 4) return false;
  if (d.index_bits != 8 && d.index_bits != 12 && d.index_bits != 16) return false;
  if (!L->rows_16b_aligned) return false;
  if (d.in_features % (2 * kBK) != 0) return false;
  if (L->num_groups != 1 || has_shift(L)) return false;
  if (((size_t)L->cb_entries * d.vector_dim * 2) % 16 != 0) return false;
  return pick_act_stages(L, 1) >= 2;
}

// Token sub-tiles per CTA (1..3) for M tokens: the largest tile that does not add a wave, or 0
// when the kernel cannot run the layer.
int large_m_tmem_pick_nt(const sacq_layer* L, int64_t M) {
  if (!large_m_tmem_supported(L)) return 0;
  const int64_t row_tiles = (L->d.out_features + kRows - 1) / kRows;
  int best = 0;
  double best_cost = 1e30;
  for (int nt = 3; nt >= 1; --nt) {
    if (pick_act_stages(L, nt) < 2) continue;
    const int64_t tiles = row_tiles * ((M + kBM * nt - 1) / (kBM * nt));
    const int64_t waves = (tiles + L->num_sms - 1) / L->num_sms;
    // whole waves x time of one CTA, fitted to measurements of 2048x6144, 2048x2048 and 6144x2048 at
    // 1,024 - 8,192 tokens (us; k = K / 2048): 4.5 + 10 k, 5.6 + 13.5 k and 5.4 + 17.2 k for 1, 2, 3 sub-tiles
    const double k = (double)L->d.in_features / 2048.0;
    const double per_cta = nt == 3 ? 5.4 + 17.2 * k : nt == 2 ? 5.6 + 13.5 * k : 4.5 + 10.0 * k;
    const double cost = (double)waves * per_cta;
    if (cost < best_cost - 1e-9) { best_cost = cost; best = nt; }
  }
  return best;
}

int launch_large_m_tmem(const sacq_layer* L, const void* q, const float* scale, int64_t M, void* y, int64_t ldy,
                        cudaStream_t s, const void* residual, int64_t ldr, const BcastDst* bc, int nt_force) {
  const sacq_layer_desc& d = L->d;
  if (!large_m_tmem_supported(L)) return set_error(SACQ_ERR_UNSUPPORTED, "TMEM-weight kernel cannot run this layer geometry");
  if (M <= 0 || d.out_features == 0) return SACQ_OK;
  if (M > (1 << 30)) return set_error(SACQ_ERR_UNSUPPORTED, "M=%lld too large", (long long)M);
  if (reinterpret_cast<uintptr_t>(q) % 16 != 0)
    return set_error(SACQ_ERR_ALIGNMENT, "quantized activations must be 16-byte aligned");
  int nt = nt_force > 0 ? nt_force : large_m_tmem_pick_nt(L, M);
  if (nt < 1 || nt > 3) return set_error(SACQ_ERR_UNSUPPORTED, "TMEM-weight kernel: no tile shape fits");
  const bool cb_smem = cb_in_smem(L);
  const int act_stages = pick_act_stages(L, nt);
  if (act_stages < 2) return set_error(SACQ_ERR_UNSUPPORTED, "TMEM-weight kernel: shared memory too small for %d sub-tiles", nt);
  CUtensorMap ta;
  {
    const int rc = encode_bytes_2d(&ta, q, (uint64_t)d.in_features, (uint64_t)M, (uint64_t)d.in_features, kBK, kBM,
                                   CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SACQ_OK) return rc;
  }
  const CUtensorMap* ti = nullptr;
  {
    const int rc = large_m_index_map(L, kRows, &ti);
    if (rc != SACQ_OK) return rc;
  }
  // the output leaves by tiled bulk stores when y (and every peer copy of a column split) allows it:
  // 16-byte aligned base and row pitch
  bool y_tma = residual == nullptr && reinterpret_cast<uintptr_t>(y) % 16 == 0 && (ldy * 2) % 16 == 0 &&
               d.out_features >= kRows;
  for (int i = 0; bc != nullptr && i < bc->n; ++i) y_tma = y_tma && reinterpret_cast<uintptr_t>(bc->ptr[i]) % 16 == 0;
  CUtensorMap ty = ta;                                // a valid map is passed either way
  static const BcastMaps kNoMaps = {};
  BcastMaps tb_local;
  const BcastMaps* tb = &kNoMaps;
  if (y_tma) {
    int rc = encode_bytes_2d(&ty, y, (uint64_t)d.out_features * 2, (uint64_t)M, (uint64_t)ldy * 2, kRows * 2, kBM,
                             CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != SACQ_OK) return rc;
    if (bc != nullptr && bc->n > 0) {
      tb_local = kNoMaps;
      for (int i = 0; i < bc->n; ++i) {
        rc = encode_bytes_2d(&tb_local.m[i], bc->ptr[i], (uint64_t)d.out_features * 2, (uint64_t)M, (uint64_t)ldy * 2,
                             kRows * 2, kBM, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != SACQ_OK) return rc;
      }
      tb = &tb_local;
    }
  }
  TmemParams p{};
  p.y_tma = y_tma ? 1 : 0;
  p.cb_hilo = L->cb_hilo;
  p.scales = static_cast<const uint16_t*>(d.scales);
  p.bias = static_cast<const uint16_t*>(d.bias);
  p.act_scale = scale;
  p.y = static_cast<uint16_t*>(y);
  p.residual = static_cast<const uint16_t*>(residual);
  p.ldr = ldr;
  p.ldy = ldy;
  if (bc != nullptr) {
    p.n_bc = bc->n;
    for (int i = 0; i < bc->n; ++i) p.ybc[i] = static_cast<uint16_t*>(bc->ptr[i]);
  }
  p.status = L->d_status;
  p.M = (int)M; p.N = (int)d.out_features; p.K = (int)d.in_features; p.C = L->cb_entries;
  p.act_stages = act_stages;
  p.out_mul = ldexpf(1.f, -L->cb8_exp_shift);
  const TmemLayout lay = tmem_layout(nt, act_stages, sb_bytes_of(L), cb_smem ? L->cb_entries * d.vector_dim * 2 : 0);
  const size_t smem = smem_request(lay);
  const dim3 grid((unsigned)((d.out_features + kRows - 1) / kRows), (unsigned)((M + kBM * nt - 1) / (kBM * nt)), 1);
  if (grid.y > 65535) return set_error(SACQ_ERR_UNSUPPORTED, "M=%lld exceeds the grid limit", (long long)M);
  cudaError_t e;
  const int D = d.vector_dim, B = d.index_bits;
  if (D == 8 && B == 12) e = launch_db<8, 12>(ta, *ti, ty, *tb, p, nt, cb_smem, grid, smem, s);
  else if (D == 8 && B == 8) e = launch_db<8, 8>(ta, *ti, ty, *tb, p, nt, cb_smem, grid, smem, s);
  else if (D == 8 && B == 16) e = launch_db<8, 16>(ta, *ti, ty, *tb, p, nt, cb_smem, grid, smem, s);
  else if (D == 4 && B == 12) e = launch_db<4, 12>(ta, *ti, ty, *tb, p, nt, cb_smem, grid, smem, s);
  else if (D == 4 && B == 8) e = launch_db<4, 8>(ta, *ti, ty, *tb, p, nt, cb_smem, grid, smem, s);
  else e = launch_db<4, 16>(ta, *ti, ty, *tb, p, nt, cb_smem, grid, smem, s);
  count_launch();
  if (e != cudaSuccess) return cuda_fail(e, "TMEM-weight large-M launch");
  return SACQ_OK;
}

}  // namespace sacq
