"""The numpy oracle against fixtures produced by the reference's own code
(tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest

from conftest import load_golden
from oracle import sacq_oracle as O


def test_bit_packing_known_answers():
    kat = load_golden("pack_kat")
    for bits in (1, 2, 3, 5, 7, 8, 9, 11, 12, 16):
        idx = kat[f"idx_{bits}"]
        want = kat[f"packed_{bits}"]
        got = O.pack_indices(idx, bits)
        assert got.dtype == np.uint8 and np.array_equal(got, want)
        assert np.array_equal(O.unpack_indices(want, bits, idx.size), idx)


def test_bit_packing_against_big_integer():
    # the reference's own check (tests/test_core.py:142-151): an independent
    # arbitrary-precision unpacker, including widths whose fields cross bytes
    rng = np.random.default_rng(5)
    for bits in (1, 2, 3, 7, 8, 9, 11, 16):
        idx = rng.integers(0, 1 << bits, size=79)
        payload = bytes(O.pack_indices(idx, bits).tolist())
        integer = int.from_bytes(payload, "little")
        recovered = [(integer >> (j * bits)) & ((1 << bits) - 1) for j in range(idx.size)]
        assert recovered == idx.tolist()
        assert len(payload) == (idx.size * bits + 7) // 8


def test_pack_rejects_bad_arguments():
    with pytest.raises(ValueError):
        O.pack_indices(np.array([0, 1]), 0)
    with pytest.raises(ValueError):
        O.pack_indices(np.array([0, 1]), 57)
    with pytest.raises(ValueError):
        O.pack_indices(np.array([0, 8]), 3)


def test_window_bytes():
    assert [O.index_window_bytes(b) for b in (1, 8, 11, 12, 16)] == [1, 1, 3, 2, 2]
    assert [O.index_bits_for(c) for c in (1, 2, 32, 256, 257, 4096, 65536)] == [1, 1, 5, 8, 9, 12, 16]


def test_reconstruction_bit_exact(golden_layer):
    g = golden_layer
    shift = int(g["shift"][0])
    w = O.dequantize_bf16_bits(g["codebook"], g["indices"], g["scales"], shift,
                               int(g["N"]), int(g["K"]), int(g["G"]))
    assert np.array_equal(w, g["w_ref"])
    w2 = O.dequantize_packed_bf16_bits(g["packed"], int(g["index_bits"]), g["codebook"], g["scales"], shift,
                                       int(g["N"]), int(g["K"]), int(g["G"]))
    assert np.array_equal(w2, g["w_ref"])
    assert np.array_equal(O.pack_indices(g["indices"], int(g["index_bits"])), g["packed"])


def test_tiny_hand_written_payload():
    # tests/test_cache.py:10-14 of the reference
    want = load_golden("tiny_cache_payload")["w_ref"]
    cb = O.f32_to_bf16_bits(np.array([[1., 2.], [3., 4.]], dtype=np.float32))
    sc = O.f32_to_bf16_bits(np.ones((2, 1), dtype=np.float32))
    got = O.dequantize_bf16_bits(cb, np.array([[[0, 1]], [[1, 0]]]), sc, 0, 2, 4, 4)
    assert np.array_equal(got, want)
    assert O.bf16_bits_to_f32(got).tolist() == [[1, 2, 3, 4], [3, 4, 1, 2]]


def test_activation_quantizer_bit_exact(golden_layer):
    g = golden_layer
    q, s = O.quantize_rows_e4m3(g["x"])
    assert np.array_equal(q, g["q"])
    assert np.array_equal(s.view(np.uint32), g["act_scale"].view(np.uint32))


def test_weight_row_quantizer_bit_exact(golden_layer):
    g = golden_layer
    wq, sw = O.quantize_weight_rows_e4m3(g["w_ref"])
    assert np.array_equal(wq, g["wq"])
    assert np.array_equal(sw.view(np.uint32), g["w_scale"].view(np.uint32))


def test_linear_reference(golden_layer):
    g = golden_layer
    y = O.linear_a8_reference(g["q"], g["act_scale"], g["w_ref"], g.get("bias"))
    # same composition evaluated by torch in fp32 when the fixture was made
    assert O.rel_frobenius(y, g["y_ref"]) < 1e-5
    # and the stock dense bf16 forward of the reference module stays close to it
    # (activation quantization is the only difference)
    dense = O.bf16_bits_to_f32(g["y_dense"])
    assert O.rel_frobenius(y, dense) < 0.08


def test_scalar_formats():
    f = load_golden("formats")
    allbf = O.bf16_bits_to_f32(np.arange(65536, dtype=np.uint16))
    finite = ~np.isnan(allbf)
    got = O.f32_to_e4m3_bits(np.clip(allbf, -448.0, 448.0))
    assert np.array_equal(got[finite], f["e4m3_of_all_bf16"][finite])
    # decode table round trip
    vals = O.e4m3_bits_to_f32(np.arange(256, dtype=np.uint8))
    ok = ~np.isnan(vals)
    assert np.array_equal(O.f32_to_e4m3_bits(vals[ok]), np.arange(256, dtype=np.uint8)[ok])
    q6, s6 = O.quantize_rows_e4m3(f["x6"])
    assert np.array_equal(q6, f["q6"]) and np.array_equal(s6.view(np.uint32), f["s6"].view(np.uint32))
    assert float(s6[1, 0]) == 1.0                     # all-zero row keeps scale 1
    # bf16 multiply and add roundings
    prod = O.f32_to_bf16_bits(O.bf16_bits_to_f32(f["mul_a"]) * O.bf16_bits_to_f32(f["mul_b"]))
    assert np.array_equal(prod, f["mul_out"])
    summed = O.f32_to_bf16_bits(O.bf16_bits_to_f32(prod) + O.bf16_bits_to_f32(f["add_c"])[0])
    assert np.array_equal(summed, f["add_out"])


def test_int8_activation_quantizer_matches_reference_fixture():
    """quantize_rows(x, 'int8_symmetric') of the reference: bytes and scale bits, including
    the round-half-to-even ties and the all-zero row."""
    f = load_golden("act_int8")
    q, s = O.quantize_rows_int8(f["x"])
    assert np.array_equal(q, f["q"])
    assert np.array_equal(s.view(np.uint32), f["s"].view(np.uint32))
    assert list(q[5, 1:5]) == [0, 2, 2, 4] and float(s[1, 0]) == 1.0


def test_fp8_recipe_reference_on_fixture_operands():
    """The FP8 recipe's CPU evaluation on the reference-generated operands of a fixture (e4m3
    activation bytes, per-row e4m3 weight bytes, both scale vectors): equal to a plain float64
    evaluation written out element by element, and within the weight re-quantization error of the
    exact-weight product the same fixture holds."""
    f = load_golden("layer_d8_c4096_b12")
    bias = f["bias"] if "bias" in f else None
    y = O.linear_w8a8_fp8_reference(f["q"], f["act_scale"], f["wq"], f["w_scale"], bias)
    a = O.e4m3_bits_to_f32(f["q"]).astype(np.float64)
    w = O.e4m3_bits_to_f32(f["wq"]).astype(np.float64)
    m, n = 1, 3
    acc = sum(a[m, k] * w[n, k] for k in range(a.shape[1]))
    val = float(f["act_scale"].reshape(-1)[m]) * (acc * float(f["w_scale"].reshape(-1)[n]))
    if bias is not None:
        val += float(O.bf16_bits_to_f32(bias)[n])
    assert abs(float(y[m, n]) - val) <= 2.0 ** -8 * abs(val) + 1e-30
    exact = O.bf16_bits_to_f32(f["y_ref"]) if f["y_ref"].dtype == np.uint16 else f["y_ref"]
    assert O.rel_frobenius(y, exact) < 6e-2


def test_nonfinite_activations_match_reference_fixture():
    """A NaN in a row: scale 1 (the reference's `maximum > 0` is false for NaN) and the NaN stays a
    NaN; an infinity: infinite scale, zeros for the finite elements, NaN for the infinite ones."""
    f = load_golden("act_nonfinite")
    with np.errstate(invalid="ignore"):
        q, s = O.quantize_rows_e4m3(f["x"])
    assert np.array_equal(s.view(np.uint32).ravel(), f["s"].ravel())
    assert np.array_equal(q, f["q"])
    assert f["q"][1, 17] & 0x7F == 0x7F and f["q"][2, 0] == 0 and f["q"][4, 100] == 0x7E
    assert float(s[1, 0]) == 1.0 and np.isinf(s[2, 0]) and np.isinf(s[3, 0])


def test_layernorm_reference_against_torch_cpu():
    """The float64 LayerNorm reference agrees with PyTorch's CPU LayerNorm to one bf16 ulp."""
    import torch
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(7, 384, generator=g) * 2 + 0.5).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(384, generator=g)).to(torch.bfloat16)
    b = (0.1 * torch.randn(384, generator=g)).to(torch.bfloat16)
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    ours = O.layernorm_bf16_reference(bits(x), bits(w), bits(b), 1e-5)
    ref = torch.nn.functional.layer_norm(x.float(), (384,), w.float(), b.float(), 1e-5).to(torch.bfloat16).float().numpy()
    assert np.all(np.abs(ours - ref) <= np.maximum(np.abs(ref), 1e-30) * 2.0 ** -7 + 1e-6)
    assert np.mean(ours != ref) < 0.01


def test_int8_recipe_operands_match_reference_fixture(golden_layer):
    """The deployed INT8 recipe's operands: per-token int8 activations, per-output-row int8
    weights and the integer product, as the reference's quantize_rows produced them."""
    g = golden_layer
    q8, s8 = O.quantize_rows_int8(g["x"])
    assert np.array_equal(q8, g["q_i8"])
    assert np.array_equal(s8.view(np.uint32), g["act_scale_i8"].view(np.uint32))
    wq8, sw8 = O.quantize_weight_rows_int8(g["w_ref"])
    assert np.array_equal(wq8, g["wq_i8"])
    assert np.array_equal(sw8.view(np.uint32), g["w_scale_i8"].view(np.uint32))
    acc = q8.astype(np.int64) @ wq8.astype(np.int64).T
    assert np.array_equal(acc.astype(np.int32), g["acc_i32"])


def test_int8_recipe_epilogue_and_fused_multiply_add():
    """fma_f32 is correctly rounded (checked with exact rational arithmetic, including sums that
    land on a float64 half-way point), and the GEMM reference applies weight scale, token scale and
    bias in the reference's order."""
    from fractions import Fraction
    rng = np.random.default_rng(3)
    a = rng.standard_normal(4000).astype(np.float32)
    b = rng.standard_normal(4000).astype(np.float32)
    for c in ((-(a.astype(np.float64) * b.astype(np.float64))).astype(np.float32),      # heavy cancellation
              (rng.standard_normal(4000) * 2.0 ** -20).astype(np.float32), rng.standard_normal(4000).astype(np.float32)):
        r = O.fma_f32(a, b, c)
        for i in range(0, 4000, 13):
            exact = Fraction(float(a[i])) * Fraction(float(b[i])) + Fraction(float(c[i]))
            x = np.float32(float(exact))
            cands = [np.nextafter(x, np.float32(-np.inf)), x, np.nextafter(x, np.float32(np.inf))]
            best = min(cands, key=lambda v: (abs(Fraction(float(v)) - exact), int(np.float32(v).view(np.uint32)) & 1))
            assert np.float32(best) == r[i]
    # a case where rounding the product first would change the result
    q = np.array([[3, -7, 127, 0]], dtype=np.int8)
    wq = np.array([[127, 5, -128 + 1, 9], [1, 1, 1, 1]], dtype=np.int8)
    sa = np.array([0.0123], dtype=np.float32)
    sw = np.array([0.00071, 0.25], dtype=np.float32)
    bias = O.f32_to_bf16_bits(np.array([0.5, -1.0], dtype=np.float32))
    y = O.linear_w8a8_int8_reference(q, sa, wq, sw, bias)
    acc = q.astype(np.int64) @ wq.astype(np.int64).T
    want = [O.fma_f32(sa, (np.float32(acc[0, n]) * sw[n]).astype(np.float32), O.bf16_bits_to_f32(bias[n:n + 1]))
            for n in range(2)]
    assert np.array_equal(y[0], O.f32_to_bf16_bits(np.concatenate(want)))
    # without a bias the product sa * scaled keeps the sign of a negative zero
    y0 = O.linear_w8a8_int8_reference(np.array([[0, 0, 0, 0]], dtype=np.int8), np.array([-1.0], dtype=np.float32), wq, sw)
    assert y0[0, 0] == 0x8000
