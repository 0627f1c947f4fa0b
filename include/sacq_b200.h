/*
 * sacq_b200 -- C ABI of the B200 (sm_100a) implementation of SACQ's packed
 * vector-codebook quantized-linear forward ("W1.5A8" path).
 *
 * Plain C, no torch types: device pointers are `void*`, the CUDA stream is a
 * `void*` holding a cudaStream_t, sizes are int64_t.  Every function returns
 * an int status (0 = ok, negative = error, see SACQ_ERR_*) and never aborts
 * or traps; `sacq_last_error()` returns a thread-local message for the last
 * failure.  All launches go to the stream the caller passes and do not
 * synchronise, allocate or free device memory (layer creation and destruction
 * excepted), so a forward can sit inside a larger stream-ordered program.
 *
 * File/line citations name the interface of the reference (haesunglee116/SACQ)
 * that each entry point stands in for.  `SHIM` abbreviates
 * gr00t_libero/sources/libero_pro_eval/Isaac-GR00T-N1.7/gr00t/eval/cosmos_quant_shim.py,
 * `REC` abbreviates gr00t_libero/acceleration/sources/libero_pro_eval/
 * inference_acceleration_2026_10_11/a8_accuracy_recovery_2026_10_20_r1.
 */
#ifndef SACQ_B200_H_
#define SACQ_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SACQ_ABI_VERSION 1

#if defined(__GNUC__)
#define SACQ_API __attribute__((visibility("default")))
#else
#define SACQ_API
#endif

#define SACQ_OK 0
#define SACQ_ERR_INVALID_ARGUMENT (-1) /* null pointer, negative size, inconsistent geometry      */
#define SACQ_ERR_UNSUPPORTED (-2)      /* geometry outside what the kernels implement              */
#define SACQ_ERR_ALIGNMENT (-3)        /* a pointer or pitch misses its stated alignment           */
#define SACQ_ERR_WORKSPACE (-4)        /* workspace missing or smaller than sacq_workspace_bytes() */
#define SACQ_ERR_CUDA (-5)             /* a CUDA runtime/driver call failed (message has detail)   */
#define SACQ_ERR_DEVICE_TIMEOUT (-6)   /* a bounded device-side wait expired (see sacq_layer_status) */

/* Guard bytes that must be readable after the packed stream.  The reference
 * keeps `index_window_bytes - 1` zero bytes (SHIM:348-360); the kernels here read
 * aligned 32-bit and 128-bit words, so they ask for a little more. */
#define SACQ_PACKED_GUARD_BYTES 16

typedef struct sacq_layer sacq_layer_t; /* opaque; owns only small derived tables */

/* One `packed_vector_codebook_v1` layer as produced by
 * sacq/vector_quantization.py:369-382 and bit-packed by
 * sacq/calibration_layers.py:44-74.  Every pointer is DEVICE memory that the
 * caller keeps alive until sacq_layer_destroy(); the library borrows it. */
typedef struct sacq_layer_desc {
  uint32_t struct_size;     /* sizeof(sacq_layer_desc), for ABI checking                         */
  int32_t device;           /* CUDA device ordinal that owns every pointer below                 */
  int64_t out_features;     /* N                                                                 */
  int64_t in_features;      /* K                                                                 */
  int32_t group_size;       /* G, scales are [N, K/G]                                            */
  int32_t vector_dim;       /* d, codebook is [C, d]                                             */
  int32_t codebook_size;    /* C                                                                 */
  int32_t index_bits;       /* b, index i occupies bits [i*b, i*b+b) of the little-endian stream */
  const void* packed;       /* uint8, ceil(N*(K/d)*b/8) bytes + SACQ_PACKED_GUARD_BYTES readable,
                               16-byte aligned                                                    */
  int64_t packed_bytes;     /* bytes of the stream proper (without the guard)                    */
  const void* codebook;     /* bf16 [C, d]                                                       */
  const void* scales;       /* bf16 [N, K/G]                                                     */
  const void* bias;         /* bf16 [N] or NULL                                                  */
  uint16_t shift_bf16;      /* scalar shift as a bf16 bit pattern (0 in every fitted payload)    */
  uint16_t reserved0;
  uint32_t reserved1;
} sacq_layer_desc;

/* Replaces PrecomputedPackedVectorCodebookLinear.__init__ (SHIM:316-407): validates
 * the geometry, and builds the layer's derived device tables (an fp16 copy of the
 * codebook and an FP8 high/low split of it, a few times C*d bytes).  Allocates; call
 * at load time, not inside a captured region. */
SACQ_API int sacq_layer_create(const sacq_layer_desc* desc, sacq_layer_t** out_layer);
SACQ_API int sacq_layer_destroy(sacq_layer_t* layer);

/* Bytes of device memory the layer's derived tables hold (for residency accounting). */
SACQ_API int64_t sacq_layer_resident_bytes(const sacq_layer_t* layer);

/* Replaces .dequantize_weight() (SHIM:409-454) == decode_fixed
 * (sacq/index_correction.py:98-108) == QuantLinear.weight_
 * (sacq/calibration_layers.py:100-113):
 *   W[n, g*G + v*d + j] = bf16( bf16(codebook[idx[n,g,v], j] * scales[n,g]) + shift )
 * w_out: bf16 [N, K] row-major.  Bit-exact with the reference. */
SACQ_API int sacq_dequant_bf16(const sacq_layer_t* layer, void* w_out, void* stream);

/* Replaces quantize_rows(x, 'fp8_e4m3fn') (REC/perrow_a8_candidate_r3.py:17-25):
 *   s[m] = max_k |x[m,k]| / 448 (1 when the row is all zero)
 *   q[m,k] = e4m3_rne( clamp(x[m,k] / s[m], -448, 448) )
 * x: bf16 [M, K] row-major with row pitch `x_pitch` elements; q: uint8 [M, K];
 * scale: float [M].  Bit-exact with the reference, non-finite input included: a NaN in a row
 * fails the reference's `maximum > 0` test, so the row keeps scale 1 and the NaN stays a NaN
 * byte (0x7f / 0xff); an infinity gives an infinite scale, zeros for the row's finite elements
 * and NaN for the infinite ones (the sign of that NaN is the platform's). */
SACQ_API int sacq_quant_act_fp8(const void* x_bf16, int64_t x_pitch, int64_t M, int64_t K, void* q_out, float* scale_out,
                       void* stream);

/* Replaces the per-output-row 8-bit weight producer of the reference's A8 recipe
 * (REC/perrow_a8_candidate_r3.py:52-53 for the scale, :61-63 for the bytes):
 * sacq_weight_row_scale writes sw[n] = max_k |W[n,k]| / 448 (1 for a zero row);
 * sacq_decode_weight_fp8 writes wq[n,k] = e4m3_rne(clamp(W[n,k] / sw[n], +-448))
 * from the packed stream without materialising the bf16 weight. */
SACQ_API int sacq_weight_row_scale(const sacq_layer_t* layer, float* sw_out, void* stream);
SACQ_API int sacq_decode_weight_fp8(const sacq_layer_t* layer, const float* sw, void* wq_out, void* stream);

/* Scratch a forward with M activation rows needs (split-K partial sums and the
 * arrival counters of the small-M kernel).  The counter region -- the FIRST
 * sacq_workspace_counter_bytes() bytes -- must be zero before the first call
 * that uses the buffer; every call leaves it zero again.  One workspace may be
 * shared by calls that are ordered on one stream, never by concurrent ones. */
SACQ_API int64_t sacq_workspace_bytes(const sacq_layer_t* layer, int64_t M);
SACQ_API int64_t sacq_workspace_counter_bytes(void);

/* Replaces the A8 forward of the reference overlay, i.e. decode + 8-bit GEMM +
 * ordered epilogue (REC/perrow_a8_candidate_r3.py:56-69,
 * REC/int8_ordered_epilogue_20261028_r1.py:11-22), with the weight side kept at the
 * reconstruction's precision:
 *   y[m,n] = bf16( s[m] * sum_k q[m,k] * W[n,k]  + bias[n] )
 * q: e4m3 bytes [M, K]; scale: float [M]; y_out: bf16 [M, ldy] (ldy >= N elements).
 * Chooses the kernel from M and the layer geometry alone: warp-MMA kernels that gather
 * codewords straight into mma.sync fragments up to a few dozen rows, TMA + tcgen05 kernels
 * above that (expanded weight tiles in shared memory, or in tensor memory from 1024 rows);
 * a layer with a non-zero shift runs on the kernel that rebuilds the reference's two-rounding
 * reconstruction per weight. */
SACQ_API int sacq_linear_a8(const sacq_layer_t* layer, const void* q, const float* scale, int64_t M, void* y_out,
                   int64_t ldy, void* workspace, int64_t workspace_bytes, void* stream);

/* Output-split (column-parallel) layers across the GPUs of one node: the GEMM whose epilogue
 * writes every output element to this GPU's buffer AND to the buffers of `num_peers` other
 * GPUs (plain peer stores over NVLink, no multicast), so the exchange of the column blocks
 * overlaps the computation instead of following it as an all-gather.  y_out and peer_outs[i]
 * point at the first column this rank owns inside each [M, ldy] result buffer (the caller adds
 * its column offset); all buffers share the row pitch ldy.  The caller orders the launch
 * against the peers' use of their buffers (a barrier between producing and consuming, two
 * buffers alternating).  The reference has no counterpart (single GPU).
 *
 * sacq_peer_buffer_*: device buffers that other processes of the node can map through CUDA IPC
 * (`handle` is SACQ_PEER_HANDLE_BYTES bytes to be sent to the peers by any host channel). */
#define SACQ_PEER_HANDLE_BYTES 64
SACQ_API int sacq_linear_a8_bcast(const sacq_layer_t* layer, const void* q, const float* scale, int64_t M, void* y_out,
                                  void* const* peer_outs, int num_peers, int64_t ldy, void* workspace,
                                  int64_t workspace_bytes, void* stream);
SACQ_API int sacq_peer_buffer_create(int device, int64_t bytes, void** dev_ptr, void* handle_out);
SACQ_API int sacq_peer_buffer_open(int device, const void* handle, void** dev_ptr);
SACQ_API int sacq_peer_buffer_close(int device, void* dev_ptr);
SACQ_API int sacq_peer_buffer_destroy(int device, void* dev_ptr);

/* INT8 per-token activations, the format of the reference's deployed recipe
 * (quantize_rows(x, 'int8_symmetric'), perrow_a8_candidate_r3.py:17-25):
 *   s = max|x| / 127 per row (1 for an all-zero row), q = int8(round_half_even(clamp(x / s, -127, 127))).
 * sacq_linear_a8i is sacq_linear_a8 for such activations: the same exact weights (no 8-bit
 * rounding of the weights, unlike the reference's INT8 GEMM), int8 widened to fp16 in front of
 * fp16 tensor-core MMAs (tcgen05 kind::f16 from 48 rows, warp MMAs below).  Its workspace is
 * sacq_workspace_bytes_int8(layer, M) bytes, 256-byte aligned, zero-filled once. */
SACQ_API int sacq_quant_act_int8(const void* x_bf16, int64_t x_pitch, int64_t M, int64_t K, void* q_out,
                                 float* scale_out, void* stream);
SACQ_API int64_t sacq_workspace_bytes_int8(const sacq_layer_t* layer, int64_t M);
SACQ_API int sacq_linear_a8i(const sacq_layer_t* layer, const void* q_int8, const float* scale, int64_t M, void* y_out,
                             int64_t ldy, void* workspace, int64_t workspace_bytes, void* stream);

/* The reference's deployed INT8 recipe as integer work (`projection_format: int8_symmetric`,
 * dynamic per-token activation x per-output-row weight, perrow_a8_candidate_r3.py:52-69):
 *   sw[n]   = max_k |W[n,k]| / 127 (1 for a zero row)                 sacq_weight_row_scale_int8
 *   wq[n,k] = int8(round_half_even(clamp(W[n,k] / sw[n], -127, 127)))  sacq_decode_weight_int8
 *   acc     = q_int8 (per-token, sacq_quant_act_int8) x wq^T, int32, exact
 *   y[m,n]  = bf16(fma(sa[m], float(acc) * sw[n], bias[n]))  or  bf16(sa[m] * (float(acc) * sw[n])) without bias
 * -- the rounding of int8_direct_integer_round_20261028_r1.py:6-9 and the epilogue order of
 * int8_small_m_gemm_20261028_r1.py:7-32 / int8_ordered_epilogue_20261028_r1.py:11-22.  Integer
 * accumulation is exact, so y is bit-identical to any correct evaluation of these formulas.
 * sacq_linear_w8a8_int8 decodes the int8 weight rows per call into `workspace`
 * (sacq_workspace_bytes_w8a8 bytes, 256-byte aligned; its leading sacq_workspace_counter_bytes() are
 * left untouched, so one buffer can serve every entry point; nothing expanded is kept between calls,
 * as in the reference) and runs a tcgen05 kind::i8 GEMM on them.  `w_scale` is the vector written by
 * sacq_weight_row_scale_int8 (the reference keeps it as a small per-layer buffer).  in_features must
 * be a multiple of 16. */
SACQ_API int sacq_weight_row_scale_int8(const sacq_layer_t* layer, float* sw_out, void* stream);
SACQ_API int sacq_decode_weight_int8(const sacq_layer_t* layer, const float* sw, void* wq_out, void* stream);
SACQ_API int64_t sacq_workspace_bytes_w8a8(const sacq_layer_t* layer, int64_t M);
SACQ_API int sacq_linear_w8a8_int8(const sacq_layer_t* layer, const void* q_int8, const float* act_scale,
                                   const float* w_scale, int64_t M, void* y_out, int64_t ldy, void* workspace,
                                   int64_t workspace_bytes, void* stream);

/* The reference's FP8 recipe (`projection_format: fp8_e4m3fn`): per-token e4m3 activations
 * (sacq_quant_act_fp8) x per-output-row e4m3 weights (sacq_weight_row_scale + sacq_decode_weight_fp8,
 * decoded per call into `workspace` exactly as above), fp32 accumulation on the tensor cores and
 *   y[m,n] = bf16(fma(sa[m], acc * sw[n], bias[n]))  or  bf16(sa[m] * (acc * sw[n])) without bias
 * -- what torch._scaled_mm(aq, wq.t(), sa, sw, bias) and cutlass_scaled_mm compute in
 * a8_joint_pair_r1.py:374 / perrow_a8_candidate_r3.py:56-69.  The weights are RE-QUANTIZED to 8 bits
 * here, as in the reference; sacq_linear_a8 is the path that multiplies the exact codebook weights.
 * The operands are bit-exact with the reference; the sum is fp32 in the tensor core's order. */
SACQ_API int sacq_linear_w8a8_fp8(const sacq_layer_t* layer, const void* q_e4m3, const float* act_scale,
                                  const float* w_scale, int64_t M, void* y_out, int64_t ldy, void* workspace,
                                  int64_t workspace_bytes, void* stream);

/* Activation function fused into the per-token quantizer (the producer of the MLP's down
 * projection; the reference fuses this stage for its INT8 path,
 * int8_swiglu_lookup_fusion_20261028_r1.py:9-21).  One launch, the [M, K] intermediate is
 * never written:
 *   SACQ_ACT_SILU_MUL: y = bf16( bf16(silu(a)) * b )      a = gate, b = up projection output
 *   SACQ_ACT_GELU:     y = bf16( gelu(a) )  (erf form)     b is ignored
 * followed by sacq_quant_act_fp8's arithmetic on y; the bytes equal quantizing the result of
 * the separate bf16 tensor operations.  a, b: bf16 [M, pitch] with pitch >= K elements. */
#define SACQ_ACT_SILU_MUL 0
#define SACQ_ACT_GELU 1
SACQ_API int sacq_act_quant_fp8(int kind, const void* a_bf16, int64_t a_pitch, const void* b_bf16, int64_t b_pitch,
                                int64_t M, int64_t K, void* q_out, float* scale_out, void* stream);

/* LayerNorm, optionally followed by the AdaLN modulation, fused into the quantizer (the
 * reference fuses these stages in codex_norm3_regpack_20261029_r1/kernel.cu:150 and
 * codex_adaln_sharedmax_20261029_r2/kernel.cu:140):
 *   y = bf16( (x - mean) / sqrt(var + eps) * gamma + beta )          gamma, beta: bf16 [K] or null
 *   y = bf16( bf16( y * bf16(1 + s) ) + t )                           when mod_scale / mod_shift are given
 * followed by sacq_quant_act_fp8's arithmetic on y.  mean and the centred variance are fp32
 * sums over the row; their order differs from a framework LayerNorm's, so y matches it to one
 * bf16 ulp, not to the bit.  y_out (bf16 [M, y_pitch]) receives y when it is not null. */
SACQ_API int sacq_layernorm_quant_fp8(const void* x_bf16, int64_t x_pitch, const void* gamma_bf16, const void* beta_bf16,
                                      float eps, const void* mod_scale_bf16, const void* mod_shift_bf16, int64_t M,
                                      int64_t K, void* y_out_bf16, int64_t y_pitch, void* q_out, float* scale_out,
                                      void* stream);

/* AdaLN modulation fused into the quantizer (the reference fuses the same stage,
 * codex_adaln_sharedmax_fusion_20261029_r2.py): for a normalised input x [M, K] and per-channel
 * vectors scale, shift [K] (bf16),
 *   y = bf16( bf16( x * bf16(1 + scale) ) + shift )
 * -- the three bf16 roundings of `x * (1 + scale) + shift` as tensor operations -- followed by
 * sacq_quant_act_fp8's arithmetic on y, in one launch. */
SACQ_API int sacq_modulate_quant_fp8(const void* x_bf16, int64_t x_pitch, const void* scale_vec_bf16,
                                     const void* shift_vec_bf16, int64_t M, int64_t K, void* q_out, float* scale_out,
                                     void* stream);

/* sacq_linear_a8 with a residual added in the GEMM epilogue, as the reference's down-projection
 * epilogue does (int8_ffdown_residual_epilogue_20261028_r2.py:8-24):
 *   y[m,n] = bf16( bf16( s[m] * sum_k q[m,k] * W[n,k] + bias[n] ) + residual[m,n] )
 * -- the two bf16 roundings of `linear(x) + residual` evaluated as two tensor operations.
 * residual: bf16 [M, ldr] (ldr >= N); it must not overlap y_out. */
SACQ_API int sacq_linear_a8_residual(const sacq_layer_t* layer, const void* q, const float* scale, int64_t M,
                                     const void* residual, int64_t ldr, void* y_out, int64_t ldy, void* workspace,
                                     int64_t workspace_bytes, void* stream);

/* Sibling projections that read the same activations (q/k/v, gate/up): the result of
 * sacq_linear_a8 for every layer, on one set of quantized activations
 * (int8_shared_padded_activation_20261028_r1.py:44-63 shares the quantized input,
 * int8_grouped_qkv_aligned_frozen_20261028_r1.py:9-40 and int8_grouped_gateup_20261028_r1.py:7-54
 * group the GEMMs).  Up to four layers of one geometry (same K, vector_dim, index width,
 * codebook size and group size) run as ONE launch when they would all use the small-M warp-MMA
 * kernel (out_features a multiple of 8; the grid is split between the layers) or all the FP8
 * tensor-core kernel (the layer is a grid dimension); anything else runs one launch per layer.
 * `workspace` must be large enough for the largest sacq_workspace_bytes(layer, M).  Results are
 * byte-identical to separate sacq_linear_a8 calls. */
SACQ_API int sacq_linear_a8_multi(const sacq_layer_t* const* layers, int num_layers, const void* q, const float* scale,
                                  int64_t M, void* const* y_outs, const int64_t* ldys, void* workspace,
                                  int64_t workspace_bytes, void* stream);

/* Convenience: sacq_quant_act_fp8 + sacq_linear_a8 for a bf16 input (the module's
 * forward(x), SHIM:456-541).  `q_scratch` (M*K bytes) and `scale_scratch` (M floats)
 * are caller-provided device buffers. */
SACQ_API int sacq_linear_bf16(const sacq_layer_t* layer, const void* x_bf16, int64_t x_pitch, int64_t M, void* q_scratch,
                     float* scale_scratch, void* y_out, int64_t ldy, void* workspace, int64_t workspace_bytes,
                     void* stream);

/* The module's forward for a caller whose activations and results live in HOST memory
 * (the reference's CPU-side callers hand the module host tensors and read host tensors
 * back, SHIM:456-541): copies x (bf16 [M, K], contiguous; pinned memory makes the copies
 * asynchronous) to the device, runs sacq_linear_bf16 and copies y (bf16 [M, N]) back, all
 * on `stream`, without synchronising.  When a host buffer is pinned (page-locked and mapped,
 * 16-byte aligned) and its transfer is at most 1 MiB, no copy engine is involved: the
 * quantizer kernel reads x from host memory directly and a copy kernel stores y to host
 * memory; the bytes crossing the bus are the same.  `dev_scratch` is caller-owned device memory of
 * sacq_host_forward_scratch_bytes(layer, M) bytes, 256-byte aligned, zero-filled once
 * before its first use; it may be reused by later calls on the same stream. */
SACQ_API int sacq_linear_bf16_host(const sacq_layer_t* layer, const void* x_host, int64_t M, void* y_host,
                                   void* dev_scratch, int64_t dev_scratch_bytes, void* stream);
SACQ_API int64_t sacq_host_forward_scratch_bytes(const sacq_layer_t* layer, int64_t M);

/* The same forward as sacq_linear_a8's split-K small-M kernel, for callers that cannot
 * allocate device memory (a control loop with a frozen memory budget, a server whose
 * arena already owns the GPU, a plugin that is handed nothing but its inputs and
 * outputs).  It has no counterpart in the reference.  The split-K partial sums and
 * arrival counters live in an array built into the library: sacq_static_scratch_bytes()
 * bytes (8 MiB) of device memory on every GPU that loads it, held until the process
 * exits.  The call allocates and frees nothing.  Limits and rules:
 *   - a call whose partial sums (M * N * 4 bytes per K split; at least one split's worth
 *     must fit, whatever the launch plan of the device at hand needs) or arrival counters
 *     (at most 16384) do not fit the array returns SACQ_ERR_WORKSPACE and launches nothing:
 *     M * N may not exceed 2,080,768 outputs; the decode shapes (M <= 64, N <= 6144) need
 *     at most about 2 MiB;
 *   - the first call on a device looks up the array's device address; make that call
 *     before starting any stream capture;
 *   - every call uses the same array: calls that may overlap on the GPU (different
 *     streams) race, calls ordered on one stream do not.  The counters are cleared at
 *     the start of each call, the partial sums are overwritten before they are read. */
SACQ_API int sacq_linear_a8_static_scratch(const sacq_layer_t* layer, const void* q, const float* scale, int64_t M,
                                           void* y_out, int64_t ldy, void* stream);
SACQ_API int64_t sacq_static_scratch_bytes(void);

/* Forces a GEMM kernel (for tests and benchmarks): 0 = automatic, 1 = small-M kernel
 * (its own choice of variant), 2 = tensor-core kernel with expanded weight tiles in shared
 * memory, 3 = small-M CUDA-core variant, 4 = small-M warp-MMA variant, 5 = warp-MMA variant
 * without shared-memory staging, 6 = warp-MMA variant that unpacks the indices in shared memory
 * (any index width, any group size that is a multiple of 32), 7 = tensor-core kernel for grouped
 * scales, 8 = tensor-core kernel with the expanded weights in tensor memory (9, 10, 11: the same
 * with 1, 2, 3 token sub-tiles of 128 per CTA), 12 = that design for grouped scales (13, 14, 15:
 * 1, 2, 3 sub-tiles).
 * Returns SACQ_ERR_UNSUPPORTED from the next forward if the forced kernel cannot run the layer. */
SACQ_API int sacq_layer_set_kernel(sacq_layer_t* layer, int which);
/* Which kernel a forward with M rows would use (1 = small-M, 2 = tensor-core kernel with
 * shared-memory weight tiles, 3 = tensor-core kernel for grouped scales, 4 = tensor-core kernel
 * with tensor-memory weights), or a negative error. */
SACQ_API int sacq_layer_kernel_for(const sacq_layer_t* layer, int64_t M);

/* Reads the layer's device-side status word (synchronises the device): 0, or a
 * nonzero code written by a kernel whose bounded wait gave up. */
SACQ_API int sacq_layer_status(const sacq_layer_t* layer, int* status_out);

/* Kernels launched by this library since it was loaded (all devices, all streams). */
SACQ_API int64_t sacq_launch_count(void);

SACQ_API const char* sacq_last_error(void);
SACQ_API int sacq_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SACQ_B200_H_ */
