"""CPU tests of the host-side code: bit packing, payload handling, the shared library's
exported symbols.  No compute call is made (there is no GPU here)."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import load_golden
import sacq_b200
from sacq_b200 import _lib, packing, synthetic
from oracle import sacq_oracle as O


def test_pack_matches_reference_fixtures():
    kat = load_golden("pack_kat")
    for bits in (1, 2, 3, 5, 7, 8, 9, 11, 12, 16):
        idx = torch.from_numpy(kat[f"idx_{bits}"])
        got = packing.pack_indices(idx, bits)
        assert got.dtype == torch.uint8
        assert np.array_equal(got.numpy(), kat[f"packed_{bits}"])
        assert torch.equal(packing.unpack_indices(got, bits, idx.numel()), idx)


def test_pack_layer_fixtures(golden_layer):
    g = golden_layer
    got = packing.pack_indices(torch.from_numpy(g["indices"]), int(g["index_bits"]))
    assert np.array_equal(got.numpy(), g["packed"])


def test_pack_errors():
    with pytest.raises(ValueError):
        packing.pack_indices(torch.tensor([0, 1]), 0)
    with pytest.raises(ValueError):
        packing.pack_indices(torch.tensor([0, 1]), 57)
    with pytest.raises(ValueError):
        packing.pack_indices(torch.tensor([0, 4]), 2)
    with pytest.raises(ValueError):
        packing.pack_indices(torch.tensor([-1]), 4)
    assert packing.pack_indices(torch.zeros(0, dtype=torch.int64), 12).numel() == 0


def test_pack_payload_roundtrip():
    p = synthetic.make_payload(16, 64, vector_dim=8, codebook_size=4096, seed=3, packed=False)
    assert p["indices"].dtype == torch.int32 and tuple(p["indices"].shape) == (16, 1, 8)
    q = packing.pack_payload(p)
    assert "indices" not in q and q["index_bits"] == 12 and q["index_shape"] == (16, 1, 8)
    back = packing.unpack_indices(q["packed_indices"], 12, 16 * 8)
    assert torch.equal(back, p["indices"].reshape(-1).long())
    with pytest.raises(ValueError):
        packing.pack_payload(q)


def test_synthetic_payload_format():
    # the keys, dtypes and shapes the reference's fitter returns (sacq/vector_quantization.py:369-382)
    p = synthetic.make_payload(24, 128, vector_dim=4, codebook_size=256, group_size=64, seed=1, packed=False)
    assert p["format"] == "packed_vector_codebook_v1"
    assert p["codebook"].dtype == torch.bfloat16 and tuple(p["codebook"].shape) == (256, 4)
    assert p["indices"].dtype == torch.uint8 and tuple(p["indices"].shape) == (24, 2, 16)
    assert p["scales"].dtype == torch.bfloat16 and tuple(p["scales"].shape) == (24, 2)
    assert p["shift"].dtype == torch.bfloat16 and float(p["shift"]) == 0.0
    assert float(p["codebook"].float().abs().max()) <= 1.0
    # deterministic in the seed
    p2 = synthetic.make_payload(24, 128, vector_dim=4, codebook_size=256, group_size=64, seed=1, packed=False)
    assert torch.equal(p["indices"], p2["indices"]) and torch.equal(p["codebook"], p2["codebook"])
    # the fitted layer approximates its weights: reconstruct with the oracle and compare
    w = O.bf16_bits_to_f32(O.dequantize_bf16_bits(
        p["codebook"].view(torch.int16).numpy().view(np.uint16), p["indices"].numpy(),
        p["scales"].view(torch.int16).numpy().view(np.uint16), 0, 24, 128, 64))
    gen = torch.Generator().manual_seed(1)
    W = (torch.randn(24, 128, generator=gen) * 0.02).numpy()
    assert O.rel_frobenius(w, W) < 0.35


def test_algorithmic_bytes_formula():
    # 2048 x 2048, 12-bit indices, one token: indices + codebook + scales + activations + output
    assert synthetic.algorithmic_bytes(2048, 2048, 1) == 786432 + 65536 + 4096 + 2052 + 4096
    assert synthetic.algorithmic_bytes(6144, 2048, 1, codebook_size=256) - synthetic.algorithmic_bytes(
        6144, 2048, 0, codebook_size=256) == 2048 + 4 + 2 * 6144


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert len(declared) >= 15
    assert sorted(_lib.SIGNATURES) == declared
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.sacq_abi_version() == 1
    assert lib.sacq_workspace_counter_bytes() > 0
    assert ctypes.sizeof(_lib.LayerDesc) == 88


def test_layer_create_argument_errors_without_gpu():
    lib = _lib.load()
    h = ctypes.c_void_p()
    assert lib.sacq_layer_create(None, ctypes.byref(h)) == -1
    d = _lib.LayerDesc()
    d.struct_size = 4
    assert lib.sacq_layer_create(ctypes.byref(d), ctypes.byref(h)) == -1
    assert "struct_size" in _lib.last_error()
    d.struct_size = ctypes.sizeof(d)
    d.out_features, d.in_features, d.group_size, d.vector_dim, d.codebook_size, d.index_bits = 4, 8, 6, 4, 4, 2
    assert lib.sacq_layer_create(ctypes.byref(d), ctypes.byref(h)) == -1          # K % G != 0
    d.group_size = 8
    d.packed_bytes = 1
    assert lib.sacq_layer_create(ctypes.byref(d), ctypes.byref(h)) == -1          # wrong byte count
    assert "expected 2" in _lib.last_error()
    d.packed_bytes = 2
    d.index_bits = 30
    assert lib.sacq_layer_create(ctypes.byref(d), ctypes.byref(h)) == -2          # unsupported width
    assert lib.sacq_layer_destroy(None) == 0
    assert lib.sacq_linear_a8(None, None, None, 1, None, 1, None, 0, None) == -1
    assert lib.sacq_quant_act_fp8(None, 8, -1, 8, None, None, None) == -1


def test_module_refuses_cpu():
    p = synthetic.make_payload(8, 32, vector_dim=4, codebook_size=16, seed=0)
    with pytest.raises(ValueError):
        sacq_b200.PrecomputedPackedVectorCodebookLinear(p, None, "cpu")
    with pytest.raises(ValueError):
        sacq_b200.PrecomputedPackedVectorCodebookLinear({"codebook": p["codebook"]}, None, "cuda")
    with pytest.raises(ValueError):
        sacq_b200.quantize_rows(torch.zeros(2, 8, dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        sacq_b200.quantize_rows(torch.zeros(2, 8))


def test_fused_quantizers_refuse_cpu_and_bad_arguments():
    """The fused producers validate their arguments before touching the device and have no CPU path."""
    import torch
    from sacq_b200 import (act_quantize_rows, layernorm_quantize_rows, linear_a8_multi, modulate_quantize_rows,
                           quantize_rows)
    x = torch.zeros(2, 16, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        quantize_rows(x)                                   # CPU tensor
    with pytest.raises(ValueError):
        quantize_rows(x, "int4")
    with pytest.raises(ValueError):
        act_quantize_rows("relu", x)
    with pytest.raises(TypeError):
        act_quantize_rows("gelu", x)                        # CPU tensor
    with pytest.raises(TypeError):
        modulate_quantize_rows(x, x[0], x[0])
    with pytest.raises(TypeError):
        layernorm_quantize_rows(x.float())
    with pytest.raises(TypeError):
        layernorm_quantize_rows(x)
    with pytest.raises(Exception):
        linear_a8_multi([], x.view(torch.uint8), torch.ones(2))


def test_c_abi_argument_errors_of_the_new_entry_points_without_gpu():
    """Argument checks that run before any CUDA call."""
    import ctypes
    from sacq_b200 import _lib
    lib = _lib.load()
    assert lib.sacq_act_quant_fp8(7, None, 0, None, 0, 1, 8, None, None, None) == -1
    assert "activation kind" in _lib.last_error()
    assert lib.sacq_act_quant_fp8(1, None, 0, None, 0, 1, 8, None, None, None) == -1
    assert lib.sacq_modulate_quant_fp8(None, 0, None, None, 1, 8, None, None, None) == -1
    assert lib.sacq_layernorm_quant_fp8(None, 0, None, None, ctypes.c_float(1e-5), None, None, 1, 8, None, 0, None,
                                        None, None) == -1
    assert lib.sacq_quant_act_int8(None, 0, -1, 8, None, None, None) == -1
    assert lib.sacq_linear_a8_multi(None, 0, None, None, 1, None, None, None, 0, None) == -1
    assert lib.sacq_linear_a8_bcast(None, None, None, 1, None, None, 9, 0, None, 0, None) == -1
    assert lib.sacq_linear_a8_residual(None, None, None, 1, None, 0, None, 0, None, 0, None) == -1
    assert lib.sacq_peer_buffer_create(0, 0, None, None) == -1
    assert lib.sacq_workspace_bytes_int8(None, 4) == 0
    assert lib.sacq_linear_a8_static_scratch(None, None, None, 0, None, 0, None) == -1      # null layer, whatever M is
    assert "layer handle" in _lib.last_error()
    assert lib.sacq_act_quant_fp8(0, None, 0, None, 0, 0, 8, None, None, None) == 0      # M = 0 is a no-op


def test_index_range_check():
    """An index that does not address a codeword is refused before anything is uploaded (the
    reference's CPU gather raises IndexError for it; a GPU gather would read out of bounds)."""
    import pytest
    import torch
    from sacq_b200.packing import check_index_range
    check_index_range(torch.tensor([[0, 250], [3, 7]], dtype=torch.int32), 251)
    check_index_range(torch.zeros(0, dtype=torch.uint8), 4)
    with pytest.raises(IndexError):
        check_index_range(torch.tensor([0, 251], dtype=torch.int32), 251)
    with pytest.raises(IndexError):
        check_index_range(torch.tensor([-1, 2], dtype=torch.int32), 251)
