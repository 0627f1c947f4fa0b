"""GPU parity tests: every kernel, called through the C ABI (via the ctypes-backed
module), against the CPU oracle and the reference-generated fixtures.

Bars: bit-exact for the weight reconstruction, the activation quantizer and the FP8
weight producer; relative Frobenius error <= 1e-2 for the quantized linear against
reconstruct-then-matmul on identical quantized activations."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import golden_layer_names, load_golden
from oracle import sacq_oracle as O

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-2          # relative Frobenius norm, the tolerance the task states


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def bf16_bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bf16_bits(a, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).to(device)


def payload_from_golden(g, packed=True):
    p = dict(codebook=from_bf16_bits(g["codebook"], "cpu"), scales=from_bf16_bits(g["scales"], "cpu"),
             shift=from_bf16_bits(g["shift"], "cpu").reshape(()), in_features=int(g["K"]),
             out_features=int(g["N"]), group_size=int(g["G"]), vector_dim=int(g["d"]))
    if packed:
        p.update(packed_indices=torch.from_numpy(g["packed"]), index_bits=int(g["index_bits"]),
                 index_shape=tuple(g["indices"].shape))
    else:
        dt = torch.uint8 if str(g["indices_dtype"]) == "torch.uint8" else torch.int32
        p["indices"] = torch.from_numpy(g["indices"]).to(dt)
    return p


def module_from_golden(g, packed=True):
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    bias = from_bf16_bits(g["bias"], "cpu") if "bias" in g else None
    return PrecomputedPackedVectorCodebookLinear(payload_from_golden(g, packed), bias, "cuda")


def oracle_weight(payload):
    """bf16 bits [N, K] from a payload dict via the numpy oracle."""
    cb = bf16_bits(payload["codebook"])
    sc = bf16_bits(payload["scales"])
    sh = int(bf16_bits(payload["shift"].reshape(1))[0])
    return O.dequantize_packed_bf16_bits(payload["packed_indices"].numpy(), payload["index_bits"], cb, sc, sh,
                                         payload["out_features"], payload["in_features"], payload["group_size"])


# --------------------------------------------------------------------------- reconstruction

@pytest.mark.parametrize("name", golden_layer_names())
@pytest.mark.parametrize("packed", [True, False])
def test_dequant_matches_reference_fixture(name, packed):
    _need_gpu()
    g = load_golden("layer_" + name)
    mod = module_from_golden(g, packed)
    w = mod.dequantize_weight()
    assert w.dtype == torch.bfloat16 and tuple(w.shape) == (int(g["N"]), int(g["K"]))
    assert np.array_equal(bf16_bits(w), g["w_ref"])
    assert mod.index_bits == int(g["index_bits"])
    assert mod.packed_indices.numel() == g["packed"].size + mod.index_window_bytes - 1
    assert mod.device_status() == 0


@pytest.mark.parametrize("d,C,N,K", [(8, 4096, 2048, 2048), (8, 256, 512, 2048), (8, 65536, 256, 2048),
                                     (4, 4096, 512, 2048), (2, 16, 64, 96), (16, 64, 32, 128), (3, 8, 10, 12)])
def test_dequant_full_size_against_oracle(d, C, N, K):
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, seed=11, iters=1, device="cuda",
                     sample_size=max(65536, C))
    mod = PrecomputedPackedVectorCodebookLinear(p, None, "cuda")
    w = mod.dequantize_weight()
    assert np.array_equal(bf16_bits(w), oracle_weight(p))
    # idempotent and leaves the payload untouched
    assert torch.equal(mod.dequantize_weight(), w)
    assert np.array_equal(mod.packed_indices[: p["packed_indices"].numel()].cpu().numpy(), p["packed_indices"].numpy())


# --------------------------------------------------------------------------- activation quantizer

@pytest.mark.parametrize("name", golden_layer_names())
def test_act_quant_matches_reference_fixture(name):
    _need_gpu()
    from sacq_b200 import quantize_rows
    g = load_golden("layer_" + name)
    q, s = quantize_rows(from_bf16_bits(g["x"]), "fp8_e4m3fn")
    assert q.dtype == torch.float8_e4m3fn and tuple(s.shape) == (g["x"].shape[0], 1)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), g["q"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), g["act_scale"].view(np.uint32))


@pytest.mark.parametrize("M,K", [(1, 2048), (4, 2048), (16, 2048), (64, 6144), (3, 100), (5, 8200), (2, 7), (300, 1536),
                                 (1000, 2048), (257, 8), (256, 2056), (300, 6144)])
def test_act_quant_against_oracle(M, K):
    _need_gpu()
    from sacq_b200 import quantize_rows
    from sacq_b200.synthetic import make_activations
    x = make_activations(M, K, seed=M * 7 + K)
    if M > 2:
        x[1].zero_()
        x[2] *= 1e-4
    xq, xs = O.quantize_rows_e4m3(bf16_bits(x))
    q, s = quantize_rows(x.cuda())
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), xq)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), xs.view(np.uint32))
    # a row-strided view gives the same bytes
    wide = torch.zeros(M, K + 24, dtype=torch.bfloat16, device="cuda")
    wide[:, :K] = x.cuda()
    q2, s2 = quantize_rows(wide[:, :K])
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)


def test_act_quant_every_bf16_value():
    _need_gpu()
    from sacq_b200 import quantize_rows
    bits = np.arange(65536, dtype=np.uint16)
    vals = O.bf16_bits_to_f32(bits)
    keep = np.isfinite(vals)
    rows = bits[keep].reshape(-1, 1)                      # one value per row: scale = |v|/448, q = +-448
    rows = np.concatenate([rows, np.zeros_like(rows)], axis=1)
    xq, xs = O.quantize_rows_e4m3(rows)
    q, s = quantize_rows(from_bf16_bits(rows))
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), xq)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), xs.view(np.uint32))
    # all values in one row against a fixed scale: every rounding boundary of e4m3
    f = load_golden("formats")
    row = bits[keep & (np.abs(vals) <= 448.0)]
    row = np.concatenate([row, O.f32_to_bf16_bits(np.array([448.0], dtype=np.float32))]).reshape(1, -1)
    q1, s1 = quantize_rows(from_bf16_bits(row))
    assert float(s1[0, 0]) == 1.0
    assert np.array_equal(q1.view(torch.uint8).cpu().numpy()[0, :-1], f["e4m3_of_all_bf16"][row[0, :-1]])


# --------------------------------------------------------------------------- FP8 weight producer

@pytest.mark.parametrize("name", golden_layer_names())
def test_weight_fp8_producer_matches_reference_fixture(name):
    _need_gpu()
    g = load_golden("layer_" + name)
    mod = module_from_golden(g)
    sw = mod.weight_row_scale()
    assert np.array_equal(sw.cpu().numpy().view(np.uint32), g["w_scale"].view(np.uint32))
    wq = mod.decode_weight_fp8(sw)
    assert np.array_equal(wq.view(torch.uint8).cpu().numpy(), g["wq"])


# --------------------------------------------------------------------------- quantized linear

def test_shifted_layer_is_reconstructed_exactly():
    """A shift twelve times the weight magnitude: bf16(bf16(c*s) + shift) keeps 3-4 bits of the
    weight, so only a kernel that rebuilds both roundings stays within tolerance.  The automatic
    choice must do that at every M; the kernels that contract bare codewords must refuse."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200._lib import SacqError
    from sacq_b200.synthetic import make_activations, make_payload
    g = load_golden("layer_d8_c4096_bigshift")
    mod = module_from_golden(g)
    assert np.array_equal(bf16_bits(mod.dequantize_weight()), g["w_ref"])
    q = torch.from_numpy(g["q"]).cuda().view(torch.float8_e4m3fn)
    sc = torch.from_numpy(g["act_scale"]).cuda()
    y = mod.linear_a8(q, sc)
    assert O.rel_frobenius(y.float().cpu().numpy(), g["y_ref"]) <= GEMM_TOL
    for k in FAST_KERNELS:
        mod.set_kernel(k)
        with pytest.raises(SacqError) as e:
            mod.linear_a8(q, sc)
        assert e.value.code == -2, k
    mod.set_kernel("auto")
    # a full-width layer with the same shift, at decode and prefill sizes
    N, K = 512, 2048
    p = make_payload(N, K, seed=21, device="cuda", iters=1)
    p["shift"] = torch.tensor(-0.25, dtype=torch.bfloat16)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.05).to(torch.bfloat16)
    big = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    assert np.array_equal(bf16_bits(big.dequantize_weight()), w_bits)
    for M in (1, 16, 300):
        q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M + 9)))
        outs = _check_linear(big, q_bits, s, w_bits, bf16_bits(bias), kernels=("auto", "small_simt") + FAST_KERNELS)
        assert set(outs) == {"auto", "small_simt"}
        # the INT8-activation entry point takes the same exact path
        x = make_activations(M, K, seed=M + 9)
        from sacq_b200 import quantize_rows
        qi, si = quantize_rows(x.cuda(), "int8_symmetric")
        yi = big.linear_a8i(qi, si)
        ref = O.linear_a8i_reference(qi.cpu().numpy(), si.cpu().numpy().reshape(-1), w_bits, bf16_bits(bias))
        assert O.rel_frobenius(yi.float().cpu().numpy(), ref) <= GEMM_TOL


def test_out_of_range_index_is_refused():
    """An index that does not address a codeword: IndexError for an unpacked payload (as the
    reference's gather raises), an invalid-argument status from the library for a packed one."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200._lib import SacqError
    from sacq_b200.packing import pack_payload
    from sacq_b200.synthetic import make_payload
    N, K, C = 64, 256, 251
    p = make_payload(N, K, vector_dim=8, codebook_size=C, seed=4, device="cuda", iters=1, fit=False)
    PrecomputedPackedVectorCodebookLinear(p, None, "cuda")          # valid as generated
    bad = dict(p)
    packed = p["packed_indices"].clone()
    packed[packed.numel() // 2] = 255                               # 8-bit fields: index 255 >= 251
    bad["packed_indices"] = packed
    with pytest.raises(SacqError) as e:
        PrecomputedPackedVectorCodebookLinear(bad, None, "cuda")
    assert e.value.code == -1 and "index" in str(e.value)
    idx = torch.randint(0, C, (N, 1, K // 8), dtype=torch.int32)
    idx[3, 0, 5] = C
    unpacked = {k: v for k, v in p.items() if k not in ("packed_indices", "index_bits", "index_shape")}
    unpacked["indices"] = idx
    with pytest.raises(IndexError):
        PrecomputedPackedVectorCodebookLinear(unpacked, None, "cuda")

ALL_SMALL = ("auto", "small_simt", "small_mma", "small_mma_direct", "small_mma_unpacked")
ALL_KERNELS = ALL_SMALL + ("large", "large_tmem")
FAST_KERNELS = ("small_mma", "small_mma_direct", "small_mma_unpacked", "large", "large_grouped", "large_tmem")


def _check_linear(mod, q_bits, s, w_bits, bias_bits, kernels=ALL_SMALL):
    ref = O.linear_a8_reference(q_bits, s, w_bits, bias_bits)
    q = torch.from_numpy(q_bits).cuda().view(torch.float8_e4m3fn)
    sc = torch.from_numpy(s).cuda()
    outs = {}
    shifted = float(mod.shift.float().abs().item()) != 0.0
    for k in kernels:
        mod.set_kernel(k)
        if k in ("large", "large_grouped", "large_tmem") and mod._lib.sacq_layer_kernel_for(mod._handle, q.shape[0]) < 0:
            continue                                   # geometry outside the tensor-core kernel
        try:
            y = mod.linear_a8(q, sc)
        except Exception as e:                         # the forced variant may not take this geometry
            refusable = k == "small_mma_unpacked" or (shifted and k in FAST_KERNELS)
            if refusable and getattr(e, "code", 0) == -2:
                continue
            raise
        torch.cuda.synchronize()
        assert y.dtype == torch.bfloat16
        err = O.rel_frobenius(y.float().cpu().numpy(), ref)
        assert err <= GEMM_TOL, (k, err)
        y2 = mod.linear_a8(q, sc)
        assert torch.equal(y, y2), "forward must be deterministic"
        outs[k] = (y, err)
    mod.set_kernel("auto")
    assert mod.device_status() == 0
    return outs


@pytest.mark.parametrize("name", golden_layer_names())
def test_linear_matches_reference_fixture(name):
    _need_gpu()
    g = load_golden("layer_" + name)
    mod = module_from_golden(g)
    outs = _check_linear(mod, g["q"], g["act_scale"], g["w_ref"], g.get("bias"))
    y, _ = outs["auto"]
    assert O.rel_frobenius(y.float().cpu().numpy(), g["y_ref"]) <= GEMM_TOL
    # module forward on the bf16 input = fused quantizer + GEMM, same bytes
    yf = mod(from_bf16_bits(g["x"]))
    assert torch.equal(yf, y)
    # a [B, T, K] input keeps its leading shape
    x3 = from_bf16_bits(g["x"]).reshape(1, g["x"].shape[0], -1)
    assert tuple(mod(x3).shape) == (1, g["x"].shape[0], int(g["N"]))
    assert mod(x3.float()).dtype == torch.float32


CONFIG0 = [(2048, 2048, 8, 4096)]
DECODE = [(2048, 2048), (2048, 1024), (2048, 6144), (6144, 2048)]      # (K, N)


@pytest.mark.parametrize("M", [1, 4, 16])
def test_linear_config0(M):
    """K = N = 2048, d = 8, 4096 codewords, M in {1, 4, 16}."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(2048, 2048, seed=0, device="cuda")
    mod = PrecomputedPackedVectorCodebookLinear(p, None, "cuda")
    w_bits = oracle_weight(p)
    assert np.array_equal(bf16_bits(mod.dequantize_weight()), w_bits)
    q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, 2048)))
    _check_linear(mod, q_bits, s, w_bits, None)


@pytest.mark.parametrize("K,N", DECODE)
def test_linear_decode_shapes(K, N):
    """The decoder-linear sweep: every M of the sweep on one layer per shape."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, seed=K + N, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(5)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    for M in (1, 2, 4, 8, 16, 32, 64):
        x = make_activations(M, K, seed=M)
        q_bits, s = O.quantize_rows_e4m3(bf16_bits(x))
        outs = _check_linear(mod, q_bits, s, w_bits, bf16_bits(bias))
        # the bf16 forward = quantizer + GEMM: same bytes as the two-step path
        assert torch.equal(mod(x.cuda()), outs["auto"][0])
        wide = torch.zeros(M, K + 8, dtype=torch.bfloat16, device="cuda")
        wide[:, :K] = x.cuda()
        assert torch.equal(mod(wide[:, :K]), outs["auto"][0])


@pytest.mark.parametrize("N,K,d,C,G,same_as", [
    (5992, 2048, 8, 4096, None, "small_mma"), (6144, 1536, 8, 4096, None, "small_mma"),
    (5000, 2048, 4, 512, 64, "small_mma_unpacked"), (6144, 2048, 4, 4096, None, "small_mma"),
    # grouped scales on the packed-index kernel (a scale per 256 or 512 weights), one with a last tile of 40 rows
    (6144, 2048, 8, 4096, 256, "small_mma"), (5992, 2048, 8, 256, 512, "small_mma")])
def test_linear_small_m_48_row_tiles(N, K, d, C, G, same_as):
    """Layers wide enough that the warp-MMA kernels walk them in 48-row tiles (one tile per SM), with a
    last tile of 40 or 8 rows: packed-index and index-unpacking variants against the oracle, and the
    automatic choice gives the bytes of the variant it is expected to pick."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=N + C, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(11)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    kernels = ("auto", "small_simt", "small_mma") + (("small_mma_unpacked",) if G is None or G == 64 else ())
    for M in (1, 3, 16):
        q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M + 7)))
        outs = _check_linear(mod, q_bits, s, w_bits, bf16_bits(bias), kernels=kernels)
        assert same_as in outs
        assert mod.kernel_for(M) == "small"
        assert torch.equal(outs["auto"][0], outs[same_as][0])


@pytest.mark.parametrize("d,C", [(8, 256), (8, 4096), (8, 65536), (4, 4096)])
@pytest.mark.parametrize("M", [1, 16, 256])
def test_linear_mixed_bits(d, C, M):
    """1 / 1.5 / 2 / 3 bits per weight on a 2048 x 6144 layer."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    N, K = 6144, 2048
    p = make_payload(N, K, vector_dim=d, codebook_size=C, seed=C + d, device="cuda", iters=1,
                     sample_size=max(65536, 2 * C), fit=(C < 65536))
    mod = PrecomputedPackedVectorCodebookLinear(p, None, "cuda")
    w_bits = oracle_weight(p)
    q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M + 1)))
    _check_linear(mod, q_bits, s, w_bits, None, kernels=ALL_KERNELS)


@pytest.mark.parametrize("K,N", [(2048, 6144), (6144, 2048)])
@pytest.mark.parametrize("M", [256, 1024])
def test_linear_large_m_batched_shapes(K, N, M):
    """The batched-throughput layers on the TMA + tcgen05 kernel."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, seed=K // 7 + N, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(6)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    # from 1024 rows the kernel with the weights in tensor memory takes over, whatever the width
    assert mod.kernel_for(M) == ("large_tmem" if M >= 1024 else "large")
    w_bits = oracle_weight(p)
    q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M + 3)))
    outs = _check_linear(mod, q_bits, s, w_bits, bf16_bits(bias), kernels=("large", "small_mma", "large_tmem", "auto"))
    assert torch.equal(outs["auto"][0], outs[mod.kernel_for(M)][0])
    assert O.rel_frobenius(outs["large_tmem"][0].float().cpu().numpy(), outs["large"][0].float().cpu().numpy()) < 1e-3
    # both kernels see the same operands; they may differ only by summation order and the
    # fp16 vs FP8 hi+lo codeword encodings
    a, b = outs["large"][0].float().cpu().numpy(), outs["small_mma"][0].float().cpu().numpy()
    assert O.rel_frobenius(a, b) < 5e-3


@pytest.mark.parametrize("K,N", [(2048, 6144), (6144, 2048)])
@pytest.mark.parametrize("M", [4096, 8192])
def test_linear_batched_sweep_sizes_against_oracle(K, N, M):
    """The sizes the batched-throughput figures are quoted on (multi-wave grids, partial last
    token tile), with a bias, against the float64 reconstruct-then-matmul oracle."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, seed=K // 5 + N, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(8)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M - 37, K, seed=M + 5)))   # ragged last tile
    outs = _check_linear(mod, q_bits, s, w_bits, bf16_bits(bias), kernels=("auto", "large", "large_tmem"))
    assert set(outs) == {"auto", "large", "large_tmem"}
    assert mod.kernel_for(M - 37) in ("large", "large_tmem")


def test_linear_large_m_two_subtiles():
    """Enough tiles that a CTA takes two 128-token sub-tiles (two TMEM accumulators); the
    last CTA's second sub-tile is partial.  Checked against the float64 oracle."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    N, K, M = 2048, 2048, 4800
    p = make_payload(N, K, seed=9, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(4)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    q, s = quantize_rows(make_activations(M, K, seed=12).cuda())
    mod.set_kernel("large")
    y = mod.linear_a8(q, s)
    dense = O.linear_a8_reference(q.view(torch.uint8).cpu().numpy(), s.cpu().numpy().reshape(-1), oracle_weight(p),
                                  bf16_bits(bias))
    assert O.rel_frobenius(y.float().cpu().numpy(), dense) <= GEMM_TOL
    assert torch.equal(y, mod.linear_a8(q, s))
    # rows of the partial sub-tile against the small-M kernel on the same operands
    mod.set_kernel("small_mma")
    tail = mod.linear_a8(q[4736:], s[4736:])
    mod.set_kernel("auto")
    assert O.rel_frobenius(y[4736:].float().cpu().numpy(), tail.float().cpu().numpy()) < 5e-3
    assert mod.device_status() == 0


@pytest.mark.parametrize("M", [5, 70])
@pytest.mark.parametrize("C,G", [(251, None), (81, 64), (1001, 64)])
def test_linear_odd_codebook_size(M, C, G):
    """d = 4 with an odd number of codewords: the codebook's byte size is not a multiple of 16, and the
    last codeword (about 1/C of all weights use it) must still reach every kernel's shared-memory copy."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    N, K = 264, 1024
    kw = {} if G is None else {"group_size": G}
    p = make_payload(N, K, vector_dim=4, codebook_size=C, seed=C + M, device="cuda", iters=1, **kw)
    mod = PrecomputedPackedVectorCodebookLinear(p, None, "cuda")
    w_bits = oracle_weight(p)
    assert np.array_equal(mod.dequantize_weight().view(torch.int16).cpu().numpy().view(np.uint16), w_bits)
    q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M + 9)))
    outs = _check_linear(mod, q_bits, s, w_bits, None, kernels=ALL_KERNELS + ("large_grouped",))
    assert "auto" in outs and "small_simt" in outs
    assert "large" in outs if G is None else "large_grouped" in outs
    # the INT8 path reads the same derived tables
    from sacq_b200 import quantize_rows
    x = make_activations(M, K, seed=M + 9)
    qo, so = O.quantize_rows_int8(bf16_bits(x))
    q8, s8 = quantize_rows(x.cuda(), "int8_symmetric")
    y8 = mod.linear_a8i(q8, s8)
    assert O.rel_frobenius(y8.float().cpu().numpy(), O.linear_a8i_reference(qo, so, w_bits, None)) <= GEMM_TOL


@pytest.mark.parametrize("M,N,K,d,C", [(77, 200, 512, 8, 4096), (300, 1000, 256, 8, 256), (129, 136, 768, 4, 4096),
                                       (1, 128, 256, 8, 4096), (128, 128, 1024, 4, 256), (65, 136, 512, 4, 251)])
def test_linear_large_m_ragged(M, N, K, d, C):
    """Partial tiles in M and N, both vector widths, 8- and 12-bit indices, a codebook whose byte size
    is not a multiple of 16 (staged by plain copies instead of the bulk copy)."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, seed=M, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(8)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M + 5)))
    outs = _check_linear(mod, q_bits, s, w_bits, bf16_bits(bias), kernels=("large",))
    assert "large" in outs
    # rows of a wider output buffer beyond N stay untouched
    q = torch.from_numpy(q_bits).cuda().view(torch.float8_e4m3fn)
    out = torch.full((M, N + 40), 3.0, dtype=torch.bfloat16, device="cuda")
    mod.set_kernel("large")
    mod.linear_a8(q, torch.from_numpy(s).cuda(), out=out[:, :N])
    mod.set_kernel("auto")
    assert torch.equal(out[:, :N], outs["large"][0]) and float(out[:, N:].float().min()) == 3.0


@pytest.mark.parametrize("shift", [0.0, 0.0078125])
@pytest.mark.parametrize("N,K,d,C,G", [(40, 128, 4, 32, 64), (100, 256, 4, 2048, 64), (33, 512, 8, 4096, 256),
                                       (7, 24, 4, 8, 24), (64, 1536, 4, 128, 64)])
def test_linear_grouped_and_ragged_geometries(N, K, d, C, G, shift):
    """Group-64 scales, odd index widths, rows that are not byte aligned, N % 32 != 0; without a
    shift on every small-M variant, with one on the exact-reconstruction path."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=N, device="cuda", iters=1)
    p["shift"] = torch.tensor(shift, dtype=torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, None, "cuda")
    w_bits = oracle_weight(p)
    assert np.array_equal(bf16_bits(mod.dequantize_weight()), w_bits)
    for M in (1, 3, 17):
        q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M)))
        _check_linear(mod, q_bits, s, w_bits, None)


@pytest.mark.parametrize("N,K,C,G", [(2048, 2048, 128, 64), (6144, 2048, 1024, 64), (1536, 1536, 64, 64),
                                     (2048, 6144, 32, 64), (1000, 2048, 2048, 128), (520, 1024, 512, 32)])
def test_linear_deployed_layouts(N, K, C, G):
    """The layouts of the reference's frozen decode selection: dim-4 vectors, 64-wide scale
    groups, 5- to 11-bit indices, zero shift (the reference refuses to accelerate a deployed
    layer with any other, gr00t_libero/acceleration/install.py:145-155); on the index-unpacking
    warp-MMA variant."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=4, codebook_size=C, group_size=G, seed=N + C, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    assert np.array_equal(bf16_bits(mod.dequantize_weight()), w_bits)
    for M in (1, 16, 41):
        q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M)))
        outs = _check_linear(mod, q_bits, s, w_bits, bf16_bits(bias),
                             kernels=("auto", "small_simt", "small_mma_unpacked"))
        assert "small_mma_unpacked" in outs
        if mod.kernel_for(M) == "small":               # wide layers go to the tensor-core kernel from 33 rows
            assert torch.equal(outs["auto"][0], outs["small_mma_unpacked"][0])
        else:
            assert mod.kernel_for(M) == "large_grouped" and N >= 4736


@pytest.mark.parametrize("N,K,d,C,G,M", [
    (2048, 2048, 4, 128, 64, 149), (6144, 2048, 4, 1024, 64, 300), (1536, 1536, 4, 64, 64, 41),
    (2048, 6144, 4, 32, 64, 256), (1000, 2048, 4, 2048, 128, 129), (136, 1024, 8, 512, 64, 77),
    (520, 1024, 8, 4096, 256, 1), (2048, 2048, 8, 4096, 2048, 1300), (6144, 2048, 4, 1024, 64, 1300),
    (2048, 2048, 4, 128, 64, 4000)])
def test_linear_grouped_tensor_core(N, K, d, C, G, M):
    """Grouped scales on the tcgen05 kind::f16 kernel: the deployed dim-4 / group-64 layouts at
    prefill sizes, partial tiles in M and N, one and two token sub-tiles, a token count above
    one widening slab, a bias."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=N + M, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(7)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    q_bits, s = O.quantize_rows_e4m3(bf16_bits(make_activations(M, K, seed=M + 2)))
    small = ("small",) if M <= 1300 else ()               # the warp-MMA kernel walks the weights once per 16 tokens
    outs = _check_linear(mod, q_bits, s, w_bits, bf16_bits(bias),
                         kernels=("large_grouped", "large_tmem_grouped", "large_tmem_grouped1", "auto") + small)
    assert "large_grouped" in outs and "large_tmem_grouped" in outs
    a = outs["large_grouped"][0].float().cpu().numpy()
    if small:
        assert O.rel_frobenius(a, outs["small"][0].float().cpu().numpy()) < 5e-3
    # the tensor-memory form sums an output in the same order whatever its tile shape
    assert torch.equal(outs["large_tmem_grouped"][0], outs["large_tmem_grouped1"][0])
    assert O.rel_frobenius(a, outs["large_tmem_grouped"][0].float().cpu().numpy()) < 1e-3
    if M >= 96 and G < K:
        assert mod.kernel_for(M) in ("large_grouped", "large_tmem_grouped")
    if (N, M) == (6144, 1300):
        assert mod.kernel_for(M) == "large_tmem_grouped"
    # rows of a wider output buffer beyond N stay untouched
    q = torch.from_numpy(q_bits).cuda().view(torch.float8_e4m3fn)
    out = torch.full((M, N + 24), 3.0, dtype=torch.bfloat16, device="cuda")
    mod.set_kernel("large_grouped")
    mod.linear_a8(q, torch.from_numpy(s).cuda(), out=out[:, :N])
    mod.set_kernel("auto")
    assert torch.equal(out[:, :N], outs["large_grouped"][0]) and float(out[:, N:].float().min()) == 3.0


@pytest.mark.parametrize("K,Ns,d,C", [(2048, (2048, 1024, 1024), 8, 4096), (2048, (6144, 6144), 8, 4096),
                                        (1536, (1536, 1536, 1536, 1536), 8, 4096), (1024, (512, 256), 4, 256),
                                        (2048, (1024, 1000), 8, 4096)])
def test_sibling_layers_in_one_launch(K, Ns, d, C):
    """q/k/v and gate/up style groups on shared quantized activations: one launch at small M
    for layers of one geometry, byte-identical to separate calls; a group the single launch
    cannot take (an out_features that is not a multiple of 8, the tensor-core range of M)
    falls back to one launch per layer with the same bytes."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, forward_shared, linear_a8_multi, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    mods = []
    for i, N in enumerate(Ns):
        p = make_payload(N, K, vector_dim=d, codebook_size=C, seed=10 * i + N % 7, device="cuda", iters=1)
        bias = (torch.randn(N, generator=torch.Generator().manual_seed(i)) * 0.05).to(torch.bfloat16) if i % 2 else None
        mods.append(PrecomputedPackedVectorCodebookLinear(p, bias, "cuda"))
    lib = mods[0]._lib
    for M in (1, 16, 33, 64, 200):
        x = make_activations(M, K, seed=M + 11).cuda()
        q, s = quantize_rows(x)
        want = [m.linear_a8(q, s) for m in mods]
        before = lib.sacq_launch_count()
        got = linear_a8_multi(mods, q, s)
        launches = lib.sacq_launch_count() - before
        torch.cuda.synchronize()
        for a, b in zip(want, got):
            assert torch.equal(a, b)
        assert launches in (1, len(mods)), (M, launches)
        if M <= 16 and all(N % 8 == 0 for N in Ns):
            assert launches == 1, (M, launches)
        kinds = {m.kernel_for(M) for m in mods}
        if kinds == {"small"} and any(N % 8 for N in Ns):
            assert launches == len(mods), (M, launches)     # the small-M shared launch needs whole 8-row blocks
        if kinds == {"large"}:
            assert launches == 1, (M, launches)             # tensor-core kernel: one launch, blockIdx.z = layer
        if len(kinds) > 1:
            assert launches == len(mods), (M, launches)
        for a, b in zip(want, forward_shared(mods, x)):
            assert torch.equal(a, b)
    assert all(m.device_status() == 0 for m in mods)


@pytest.mark.parametrize("N,K,d,C,G,Ms", [(2048, 2048, 8, 4096, None, (1, 16, 40, 300)),
                                            (1000, 1024, 4, 256, None, (3, 130)),
                                            (1536, 1536, 4, 64, 64, (16, 41, 149)),
                                            (264, 512, 8, 65536, None, (5,)), (40, 128, 4, 32, 64, (2,))])
def test_linear_residual_epilogue(N, K, d, C, G, Ms):
    """Residual added in the epilogue of every GEMM kernel (warp-MMA staged / unpacked / direct,
    CUDA-core, both tcgen05 kernels): the bytes of `linear_a8(q, s) + residual`."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=N, device="cuda", iters=1,
                     sample_size=max(65536, 2 * C), fit=(C < 65536))
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    for M in Ms:
        x = make_activations(M, K, seed=M).cuda()
        q, s = quantize_rows(x)
        res = (torch.randn(M, N, generator=torch.Generator().manual_seed(M)) * 0.5).to(torch.bfloat16).cuda()
        wide = torch.zeros(M, N + 8, dtype=torch.bfloat16, device="cuda")
        wide[:, :N] = res
        for k in ("auto", "small", "small_simt", "small_mma_direct", "small_mma_unpacked", "large", "large_grouped"):
            mod.set_kernel(k)
            try:
                plain = mod.linear_a8(q, s)
            except Exception as e:
                if getattr(e, "code", 0) == -2:
                    continue                      # this variant cannot run the geometry
                raise
            want = plain + res
            assert torch.equal(mod.linear_a8(q, s, residual=res), want), (k, M)
            assert torch.equal(mod.linear_a8(q, s, residual=wide[:, :N]), want), (k, M)
        mod.set_kernel("auto")
        assert torch.equal(mod.forward_residual(x, res), mod(x) + res)
    assert mod.device_status() == 0
    with pytest.raises(ValueError):
        mod.linear_a8(q, s, residual=res[:, :-1])


@pytest.mark.parametrize("M,K", [(1, 6144), (16, 6144), (300, 6144), (256, 4096), (5, 100), (3, 7)])
def test_activation_fused_into_quantizer(M, K):
    """silu(gate) * up and gelu(x) fused into the quantizer: the bytes and scales of quantizing
    the result of the separate bf16 tensor operations."""
    _need_gpu()
    import torch.nn.functional as F
    from sacq_b200 import act_quantize_rows, quantize_rows
    g = torch.Generator().manual_seed(M * 7 + K)
    a = (torch.randn(M, K, generator=g) * 2.0).to(torch.bfloat16).cuda()
    b = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    a[0, 0] = 30.0                                       # saturated and tiny arguments
    a[-1, -1] = -30.0
    for kind, ref in (("silu_mul", F.silu(a) * b), ("gelu", F.gelu(a))):
        q, s = act_quantize_rows(kind, a, b if kind == "silu_mul" else None)
        qr, sr = quantize_rows(ref)
        assert torch.equal(s.view(torch.int32), sr.view(torch.int32)), kind
        assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8)), kind
    wide = torch.zeros(M, K + 8, dtype=torch.bfloat16, device="cuda")
    wide[:, :K] = a
    q2, s2 = act_quantize_rows("gelu", wide[:, :K])
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)
    z, zs = act_quantize_rows("gelu", torch.zeros(2, K, dtype=torch.bfloat16, device="cuda"))
    assert int(z.view(torch.uint8).max()) == 0 and float(zs.min()) == 1.0
    with pytest.raises(TypeError):
        act_quantize_rows("silu_mul", a)


def test_nonfinite_activations_are_not_hidden():
    """NaN and infinite activations through the FP8 quantizer: bytes and scale bits of the fixture
    generated by the reference's quantize_rows (a NaN keeps scale 1 and stays NaN, an infinity gives an
    infinite scale).  NaN bytes are compared without their sign: inf / inf is a negative NaN on the CPU
    that wrote the fixture and a positive one on the GPU."""
    _need_gpu()
    from sacq_b200 import quantize_rows
    f = load_golden("act_nonfinite")
    q, s = quantize_rows(from_bf16_bits(f["x"]).cuda())
    got = q.view(torch.uint8).cpu().numpy()
    canon = lambda b: np.where((b & 0x7F) == 0x7F, 0x7F, b)
    assert np.array_equal(canon(got), canon(f["q"]))
    assert np.array_equal(s.cpu().numpy().view(np.uint32).ravel(), f["s"].ravel())
    # the batched (one warp per row) quantizer takes over from 256 rows: same bytes for the same rows
    many = from_bf16_bits(f["x"]).repeat(50, 1).cuda()
    qm, sm = quantize_rows(many)
    assert np.array_equal(canon(qm.view(torch.uint8).cpu().numpy()), canon(np.tile(f["q"], (50, 1))))
    assert np.array_equal(sm.cpu().numpy().view(np.uint32).ravel(), np.tile(f["s"].ravel(), 50))
    # the fused producers use the same reduction: a NaN gate makes the row's scale 1, not a finite maximum
    from sacq_b200 import act_quantize_rows
    a = from_bf16_bits(f["x"]).cuda()
    qa, sa = act_quantize_rows("gelu", a)
    assert float(sa.reshape(-1)[1]) == 1.0 and int(qa.view(torch.uint8)[1, 17]) & 0x7F == 0x7F


def test_int8_activation_quantizer():
    """quantize_rows(x, 'int8_symmetric'): bytes and scale bits of the reference fixture and of
    the oracle on larger and ragged inputs."""
    _need_gpu()
    from sacq_b200 import quantize_rows
    from sacq_b200.synthetic import make_activations
    f = load_golden("act_int8")
    q, s = quantize_rows(from_bf16_bits(f["x"]).cuda(), "int8_symmetric")
    assert q.dtype == torch.int8
    assert np.array_equal(q.cpu().numpy(), f["q"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), f["s"].view(np.uint32))
    for M, K in ((1, 2048), (64, 6144), (3, 100), (5, 8200), (2, 7), (300, 1536), (1000, 2048), (256, 2056)):
        x = make_activations(M, K, seed=M + K)
        if M > 2:
            x[1].zero_()
        qo, so = O.quantize_rows_int8(bf16_bits(x))
        q, s = quantize_rows(x.cuda(), "int8_symmetric")
        assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(s.cpu().numpy().view(np.uint32), so.view(np.uint32))


@pytest.mark.parametrize("N,K,d,C,G,shift", [
    (2048, 2048, 8, 4096, None, 0.0), (1536, 1536, 4, 64, 64, 0.0), (6144, 2048, 4, 1024, 64, 0.0),
    (1000, 1024, 4, 256, None, 0.0), (100, 256, 4, 2048, 64, 0.00390625), (264, 512, 8, 65536, None, 0.0)])
def test_linear_int8_activations(N, K, d, C, G, shift):
    """GEMM on INT8 per-token activations against the oracle (exact weights, reconstruct then
    matmul): fp16 warp-MMA and CUDA-core kernels at small M, tcgen05 kind::f16 from 48 rows."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=N + 3, device="cuda", iters=1,
                     sample_size=max(65536, 2 * C), fit=(C < 65536))
    p["shift"] = torch.tensor(shift, dtype=torch.bfloat16)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    for M in (1, 16, 47, 48, 300):
        x = make_activations(M, K, seed=M)
        qo, so = O.quantize_rows_int8(bf16_bits(x))
        ref = O.linear_a8i_reference(qo, so, w_bits, bf16_bits(bias))
        q, s = quantize_rows(x.cuda(), "int8_symmetric")
        y = mod.linear_a8i(q, s)
        torch.cuda.synchronize()
        assert O.rel_frobenius(y.float().cpu().numpy(), ref) <= GEMM_TOL, M
        assert torch.equal(y, mod.linear_a8i(q, s)) and torch.equal(y, mod.forward_int8(x.cuda()))
    assert mod.device_status() == 0


@pytest.mark.parametrize("name", golden_layer_names())
def test_int8_recipe_matches_reference_fixture(name):
    """The reference's deployed INT8 recipe on its own fixtures: the per-output-row weight scale
    and the int8 weight bytes of quantize_rows(W, 'int8_symmetric'), and the GEMM's bf16 output
    bit for bit (integer accumulation is exact)."""
    _need_gpu()
    from sacq_b200._lib import SacqError
    g = load_golden("layer_" + name)
    mod = module_from_golden(g)
    sw = mod.weight_row_scale("int8_symmetric")
    assert np.array_equal(sw.cpu().numpy().view(np.uint32), g["w_scale_i8"].view(np.uint32))
    wq = mod.decode_weight_int8(sw)
    assert wq.dtype == torch.int8 and np.array_equal(wq.cpu().numpy(), g["wq_i8"])
    q = torch.from_numpy(g["q_i8"]).cuda()
    sa = torch.from_numpy(g["act_scale_i8"]).cuda()
    if int(g["K"]) % 16:
        with pytest.raises(SacqError) as e:
            mod.linear_w8a8_int8(q, sa, sw)
        assert e.value.code == -2
        return
    y = mod.linear_w8a8_int8(q, sa, sw)
    want = O.linear_w8a8_int8_reference(g["q_i8"], g["act_scale_i8"], g["wq_i8"], g["w_scale_i8"], g.get("bias"))
    assert np.array_equal(bf16_bits(y), want)
    assert torch.equal(y, mod.linear_w8a8_int8(q, sa, sw))
    assert mod.device_status() == 0


@pytest.mark.parametrize("N,K,d,C,G,with_bias", [
    (2048, 2048, 4, 128, 64, True), (6144, 2048, 4, 1024, 64, False), (1536, 1536, 4, 64, 64, True),
    (2048, 6144, 4, 32, 64, True), (1000, 2048, 4, 2048, 128, False), (2048, 2048, 8, 4096, None, True),
    (200, 144, 8, 256, None, True)])
def test_int8_recipe_deployed_layouts(N, K, d, C, G, with_bias):
    """The deployed layouts (dim-4 vectors, 64-wide scale groups, 5- to 11-bit indices) and the
    1.5-bit layer at the token counts of the reference's frozen tables: output bytes equal to the
    CPU restatement of decode -> int8 x int8 -> int32 -> ordered epilogue."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=N + C, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.05).to(torch.bfloat16) if with_bias else None
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    wq_ref, sw_ref = O.quantize_weight_rows_int8(w_bits)
    sw = mod.weight_row_scale("int8_symmetric")
    assert np.array_equal(sw.cpu().numpy().view(np.uint32), sw_ref.view(np.uint32))
    assert np.array_equal(mod.decode_weight_int8(sw).cpu().numpy(), wq_ref)
    for M in (1, 41, 149, 512):
        x = make_activations(M, K, seed=M + 4)
        if M > 2:
            x[1].zero_()
        q_ref, sa_ref = O.quantize_rows_int8(bf16_bits(x))
        q, sa = quantize_rows(x.cuda(), "int8_symmetric")
        assert np.array_equal(q.cpu().numpy(), q_ref)
        y = mod.linear_w8a8_int8(q, sa, sw)
        want = O.linear_w8a8_int8_reference(q_ref, sa_ref, wq_ref, sw_ref, None if bias is None else bf16_bits(bias))
        assert np.array_equal(bf16_bits(y), want), M
        # a wider output buffer: columns beyond N stay untouched
        out = torch.full((M, N + 8), 3.0, dtype=torch.bfloat16, device="cuda")
        mod.linear_w8a8_int8(q, sa, sw, out=out[:, :N])
        assert torch.equal(out[:, :N], y) and float(out[:, N:].float().min()) == 3.0
    assert mod.device_status() == 0


@pytest.mark.parametrize("N,K,d,C,G,with_bias", [
    (2048, 2048, 4, 128, 64, True), (6144, 2048, 4, 1024, 64, False), (2048, 6144, 4, 32, 64, True),
    (2048, 2048, 8, 4096, None, True), (200, 144, 8, 256, None, False)])
def test_fp8_recipe_against_oracle(N, K, d, C, G, with_bias):
    """The reference's FP8 recipe (per-row e4m3 weights x per-token e4m3 activations, fp32 accumulation,
    scale order weight then token, bias in the same fma): the operands are the reference's bytes
    (weight bytes and row scales against the CPU restatement), the product is compared with the
    float64 evaluation of the same operands (fp32 summation order is the tensor core's)."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=N + C, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.05).to(torch.bfloat16) if with_bias else None
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    w_bits = oracle_weight(p)
    wq_ref, sw_ref = O.quantize_weight_rows_e4m3(w_bits)
    sw = mod.weight_row_scale("fp8_e4m3fn")
    assert np.array_equal(sw.cpu().numpy().view(np.uint32).ravel(), sw_ref.view(np.uint32).ravel())
    assert np.array_equal(mod.decode_weight_fp8(sw).view(torch.uint8).cpu().numpy(), wq_ref)
    for M in (1, 41, 300, 600):
        x = make_activations(M, K, seed=M + 4)
        q_ref, sa_ref = O.quantize_rows_e4m3(bf16_bits(x))
        q, sa = quantize_rows(x.cuda())
        y = mod.linear_w8a8_fp8(q, sa, sw)
        want = O.linear_w8a8_fp8_reference(q_ref, sa_ref, wq_ref, sw_ref, None if bias is None else bf16_bits(bias))
        assert O.rel_frobenius(y.float().cpu().numpy(), want) <= 3e-3, M      # bf16 rounding of the output: 2.3e-3
        assert torch.equal(y, mod.linear_w8a8_fp8(q, sa, sw))
        # the recipe re-quantizes the weights: it stays near, not at, the exact-weight product
        exact = mod.linear_a8(q, sa)
        assert O.rel_frobenius(y.float().cpu().numpy(), exact.float().cpu().numpy()) <= 6e-2, M
        out = torch.full((M, N + 8), 3.0, dtype=torch.bfloat16, device="cuda")
        mod.linear_w8a8_fp8(q, sa, sw, out=out[:, :N])
        assert torch.equal(out[:, :N], y) and float(out[:, N:].float().min()) == 3.0
    assert mod.device_status() == 0


@pytest.mark.parametrize("M,K", [(16, 1536), (1, 2048), (300, 1024), (5, 100)])
def test_modulation_fused_into_quantizer(M, K):
    """x * (1 + scale) + shift fused into the quantizer: bytes and scales of quantizing the
    result of the three bf16 tensor operations."""
    _need_gpu()
    from sacq_b200 import modulate_quantize_rows, quantize_rows
    g = torch.Generator().manual_seed(M + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    sc = (torch.randn(K, generator=g) * 0.3).to(torch.bfloat16).cuda()
    sh = (torch.randn(K, generator=g) * 0.2).to(torch.bfloat16).cuda()
    q, s = modulate_quantize_rows(x, sc, sh)
    qr, sr = quantize_rows(x * (1 + sc) + sh)
    assert torch.equal(s.view(torch.int32), sr.view(torch.int32))
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    with pytest.raises(TypeError):
        modulate_quantize_rows(x, sc[:-1], sh)


@pytest.mark.parametrize("M,K,affine", [(16, 1536, False), (300, 2048, True), (256, 1024, True), (3, 100, True)])
def test_layernorm_fused_into_quantizer(M, K, affine):
    """LayerNorm (+ AdaLN modulation) + quantizer in one launch.  The normalised tensor must
    agree with the float64 oracle and with PyTorch's LayerNorm to one bf16 ulp (the reduction
    order differs, so not to the bit); the quantized bytes and scales must be exactly those of
    quantizing the kernel's own normalised tensor, with and without the modulation."""
    _need_gpu()
    import torch.nn.functional as F
    from sacq_b200 import layernorm_quantize_rows, quantize_rows
    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, K, generator=g) * 1.7 + 0.3).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16) if affine else None
    b = (0.1 * torch.randn(K, generator=g)).to(torch.bfloat16) if affine else None
    xc, wc, bc = x.cuda(), None if w is None else w.cuda(), None if b is None else b.cuda()
    q, s, y = layernorm_quantize_rows(xc, wc, bc, 1e-5, return_normalized=True)
    qr, sr = quantize_rows(y)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8)) and torch.equal(s.view(torch.int32), sr.view(torch.int32))
    q2, s2 = layernorm_quantize_rows(xc, wc, bc, 1e-5)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)

    def ulp_check(ours, ref):
        ours, ref = ours.float(), ref.float()
        ulp = torch.maximum(ref.abs(), torch.tensor(1e-30)) * 2.0 ** -7      # one bf16 ulp is at most 2^-7 relative
        assert bool(((ours - ref).abs() <= ulp + 1e-6).all())
        assert float((ours != ref).float().mean()) < 0.01                   # and almost all values are identical
    ref64 = O.layernorm_bf16_reference(bf16_bits(x), None if w is None else bf16_bits(w),
                                       None if b is None else bf16_bits(b), 1e-5)
    ulp_check(y.cpu(), torch.from_numpy(ref64))
    ulp_check(y, F.layer_norm(xc, (K,), wc, bc, 1e-5))
    # with the AdaLN modulation: exactly the three bf16 operations applied to the kernel's own y
    sc = (torch.randn(K, generator=g) * 0.3).to(torch.bfloat16).cuda()
    sh = (torch.randn(K, generator=g) * 0.2).to(torch.bfloat16).cuda()
    qm, sm, ym = layernorm_quantize_rows(xc, wc, bc, 1e-5, mod_scale=sc, mod_shift=sh, return_normalized=True)
    assert torch.equal(ym, y * (1 + sc) + sh)
    qmr, smr = quantize_rows(ym)
    assert torch.equal(qm.view(torch.uint8), qmr.view(torch.uint8)) and torch.equal(sm.view(torch.int32), smr.view(torch.int32))
    with pytest.raises(ValueError):
        layernorm_quantize_rows(xc, wc, bc, 1e-5, mod_scale=sc)


def test_linear_properties_and_edges():
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    N, K = 2048, 6144
    p = make_payload(N, K, seed=4, device="cuda", iters=1)
    mod = PrecomputedPackedVectorCodebookLinear(p, None, "cuda")
    x = make_activations(8, K, seed=9).cuda()
    q, s = quantize_rows(x)
    y = mod.linear_a8(q, s)
    # against the dense product of the library's own (bit-exact) reconstruction, at full size
    dense = (q.float() @ mod.dequantize_weight().float().t()) * s
    assert O.rel_frobenius(y.float().cpu().numpy(), dense.cpu().numpy()) <= GEMM_TOL
    # scaling the activation scales scales the output (up to the bf16 output rounding)
    y2 = mod.linear_a8(q, s * 2.0)
    assert O.rel_frobenius(y2.float().cpu().numpy(), 2.0 * y.float().cpu().numpy()) < 1e-6
    # zero activations give the bias (zero here); empty batch gives an empty result
    z = mod.linear_a8(torch.zeros_like(q), s)
    assert float(z.float().abs().max()) == 0.0
    e = mod(torch.zeros(0, K, dtype=torch.bfloat16, device="cuda"))
    assert tuple(e.shape) == (0, N)
    # output into a wider row pitch leaves the padding untouched
    out = torch.full((8, N + 64), 7.0, dtype=torch.bfloat16, device="cuda")
    mod.linear_a8(q, s, out=out[:, :N])
    assert torch.equal(out[:, :N], y) and float(out[:, N:].float().min()) == 7.0
    # the arrival counters are back to zero after every call
    from sacq_b200.linear import _Workspace
    ws = _Workspace.get(q.device).ws
    assert int(ws[: mod._lib.sacq_workspace_counter_bytes()].sum()) == 0
    # host-buffer forward: pinned host activations in, host result out, same bytes
    xh = x.cpu().pin_memory()
    yh = mod.forward_host(xh)
    torch.cuda.synchronize()
    assert not yh.is_cuda and torch.equal(yh, mod(x).cpu())
    with pytest.raises(TypeError):
        mod.forward_host(x)
    with pytest.raises(ValueError):
        mod(torch.zeros(2, K - 8, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        mod(torch.zeros(2, K, dtype=torch.bfloat16))


@pytest.mark.parametrize("M,pinned", [(1, True), (16, True), (3, False), (700, True), (700, False)])
def test_host_forward_routes(M, pinned):
    """Host-buffer forward: pinned buffers up to 1 MiB are read and written by the kernels
    themselves, larger or pageable ones go through copies; the bytes are those of the device
    forward every time.  M = 700 x 2048 x 2 B is above the direct-transfer limit."""
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.synthetic import make_activations, make_payload
    N, K = 1000, 2048                                   # N*2 bytes per row is not a multiple of 16
    p = make_payload(N, K, seed=21, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(3)) * 0.05).to(torch.bfloat16)
    mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
    x = make_activations(M, K, seed=M)
    xh = x.pin_memory() if pinned else x.clone()
    yh = torch.full((M, N), 5.0, dtype=torch.bfloat16)
    yh = yh.pin_memory() if pinned else yh
    before = mod._lib.sacq_launch_count()
    out = mod.forward_host(xh, yh)
    torch.cuda.synchronize()
    launches = mod._lib.sacq_launch_count() - before
    assert out is yh and torch.equal(yh, mod(x.cuda()).cpu())
    direct = pinned and M * N * 2 <= (1 << 20)
    assert launches == (3 if direct else 2)             # quantizer + GEMM (+ the copy-out kernel)
    # a second call on the same buffers gives the same bytes
    again = mod.forward_host(xh, yh.clone() if not pinned else yh)
    torch.cuda.synchronize()
    assert torch.equal(again, yh)


def test_c_abi_error_codes_on_device():
    _need_gpu()
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, _lib
    from sacq_b200.synthetic import make_payload
    p = make_payload(64, 256, seed=1, device="cuda", iters=1)
    mod = PrecomputedPackedVectorCodebookLinear(p, None, "cuda")
    lib = mod._lib
    y = torch.empty(4, 64, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(4, 256, dtype=torch.uint8, device="cuda")
    s = torch.ones(4, device="cuda")
    assert lib.sacq_linear_a8(mod._handle, q.data_ptr(), s.data_ptr(), 4, y.data_ptr(), 32, None, 0, None) == -1
    assert "ldy" in _lib.last_error()
    assert lib.sacq_linear_a8(mod._handle, q.data_ptr(), s.data_ptr(), -1, y.data_ptr(), 64, None, 0, None) == -1
    assert lib.sacq_linear_a8(mod._handle, None, s.data_ptr(), 4, y.data_ptr(), 64, None, 0, None) == -1
    need = lib.sacq_workspace_bytes(mod._handle, 4)
    if need > lib.sacq_workspace_counter_bytes():
        assert lib.sacq_linear_a8(mod._handle, q.data_ptr(), s.data_ptr(), 4, y.data_ptr(), 64, None, 0, None) == -4
    assert lib.sacq_layer_set_kernel(mod._handle, 16) == -1
    assert lib.sacq_layer_set_kernel(mod._handle, 0) == 0
    assert lib.sacq_launch_count() > 0
    # misaligned packed pointer is refused at creation
    d = _lib.LayerDesc()
    d.struct_size = ctypes.sizeof(d)
    d.device = 0
    d.out_features, d.in_features, d.group_size, d.vector_dim, d.codebook_size, d.index_bits = 64, 256, 256, 8, 4096, 12
    d.packed = mod._packed_storage.data_ptr() + 4
    d.packed_bytes = 64 * 32 * 12 // 8
    d.codebook = mod.codebook.data_ptr()
    d.scales = mod.scales.data_ptr()
    h = ctypes.c_void_p()
    assert lib.sacq_layer_create(ctypes.byref(d), ctypes.byref(h)) == -3
