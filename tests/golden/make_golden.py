"""Generate the golden fixtures in this folder by running the reference's own
Python code on CPU.

Run once, in a checkout that has the reference tree available:

    python tests/golden/make_golden.py --reference /path/to/SACQ

The fixtures (``*.npz``) are committed; the tests never need the reference
tree.  Every array is stored as raw integer bit patterns (bf16 -> uint16,
e4m3 -> uint8) so numpy can hold it without a bf16/fp8 dtype.

Reference entry points exercised:
  * sacq.vector_quantization.quantize_vector_codebook(..., return_packed=True)
  * sacq.calibration_layers.pack_indices and QuantLinear.weight_
  * gr00t_final_seed17_20260922/pack_sacq_reference.py: pack_payload
  * sacq.index_correction.decode_fixed
  * cosmos_quant_shim.PrecomputedPackedVectorCodebookLinear (cpu):
    dequantize_weight(), forward()
  * a8_accuracy_recovery_2026_10_20_r1/perrow_a8_candidate_r3.py: quantize_rows
    (both 'fp8_e4m3fn' and 'int8_symmetric', on activations and on reconstructed weights)
  * a8_rtn_r2.py: Quantizer.quantize (per-tensor twin, zero-scale rule)
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

SHIM = "gr00t_libero/sources/libero_pro_eval/Isaac-GR00T-N1.7/gr00t/eval/cosmos_quant_shim.py"
SRC = "gr00t_libero/acceleration/sources/libero_pro_eval/inference_acceleration_2026_10_11"
PACKER = "gr00t_libero/acceleration/bootstrap_sources/gr00t_final_seed17_20260922/pack_sacq_reference.py"


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def e4m3_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.uint8).numpy().copy()


def make_activations(m, k, seed, zero_row=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    n_out = max(1, k // 100)
    cols = torch.randperm(k, generator=torch.Generator().manual_seed(seed + 1))[:n_out]
    x[:, cols] *= 20.0
    if zero_row and m > 1:
        x[1].zero_()
    if m > 2:
        x[2] *= 1e-3        # a row of tiny values: exercises e4m3 subnormals after scaling
    return x.to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the SACQ reference tree")
    ap.add_argument("--only-int8", action="store_true", help="regenerate act_int8.npz only")
    ap.add_argument("--only-nonfinite", action="store_true", help="regenerate act_nonfinite.npz only")
    args = ap.parse_args()
    ref = args.reference
    sys.path.insert(0, ref)
    from sacq.vector_quantization import quantize_vector_codebook
    from sacq.calibration_layers import pack_indices, QuantLinear
    from sacq.index_correction import decode_fixed

    shim = load_by_path("ref_shim", os.path.join(ref, SHIM))
    packer = load_by_path("ref_packer", os.path.join(ref, PACKER))
    # the per-row quantizer's module imports a hashing helper that is not part
    # of the arithmetic; give it a stand-in so the file can be loaded
    stub = types.ModuleType("fused_ffup_cutlass_probe_r1b")
    stub.bitsha = lambda x: None
    sys.modules["fused_ffup_cutlass_probe_r1b"] = stub
    perrow = load_by_path("ref_perrow", os.path.join(ref, SRC, "a8_accuracy_recovery_2026_10_20_r1",
                                                     "perrow_a8_candidate_r3.py"))
    rtn = load_by_path("ref_rtn", os.path.join(ref, SRC, "a8_rtn_r2.py"))

    # ---- 0a. non-finite activations through the FP8 per-token quantizer: a row with a NaN keeps
    # scale 1 (NaN > 0 is false in the reference's torch.where) and its NaN stays NaN; a row with an
    # infinity gets an infinite scale, zeros for its finite elements and NaN for the infinite ones
    xn = make_activations(6, 256, seed=902)
    xn[1, 17] = float("nan")
    xn[2, 40] = float("inf")
    xn[3, 41] = float("-inf")
    xn[4, 5] = float("nan")
    xn[4, 77] = float("inf")
    xn[4, 100] = 1000.0                                  # above the e4m3 range on a scale-1 row: clamps to 448
    qn, sn = perrow.quantize_rows(xn, "fp8_e4m3fn")
    np.savez_compressed(os.path.join(HERE, "act_nonfinite.npz"), x=bf16_bits(xn), q=e4m3_bits(qn),
                        s=sn.numpy().astype(np.float32).view(np.uint32))
    if args.only_nonfinite:
        print("act_nonfinite.npz written")
        return

    # ---- 0. INT8 per-token quantizer (the deployed recipe's activation format) ----
    # rows spanning magnitudes, an all-zero row, and rows built so that x/scale lands on
    # exact .5 ties (round-half-to-even) and on the clamp boundary
    xi = make_activations(7, 512, seed=901, zero_row=True)
    ties = torch.zeros(512)
    ties[0] = 127.0                                      # row maximum -> scale 1.0
    ties[1:128] = torch.arange(1, 128).float() - 0.5     # 0.5, 1.5, ... 126.5
    ties[128:255] = -(torch.arange(1, 128).float() - 0.5)
    xi[5] = ties.to(torch.bfloat16)
    qi, si = perrow.quantize_rows(xi, "int8_symmetric")
    np.savez_compressed(os.path.join(HERE, "act_int8.npz"), x=bf16_bits(xi), q=qi.numpy().astype(np.int8),
                        s=si.numpy())
    if args.only_int8:
        print("act_int8.npz written")
        return

    # ---- 1. bit-packing known answers -------------------------------------
    pack = {}
    g = torch.Generator().manual_seed(1234)
    for bits in (1, 2, 3, 5, 7, 8, 9, 11, 12, 16):
        idx = torch.randint(0, 1 << bits, (79,), generator=g)
        pack[f"idx_{bits}"] = idx.numpy().astype(np.int64)
        pack[f"packed_{bits}"] = pack_indices(idx, bits).numpy()
    np.savez_compressed(os.path.join(HERE, "pack_kat.npz"), **pack)

    # ---- 2. layers: fit -> pack -> reconstruct -> quantized linear ---------
    # (name, N, K, group_size, d, C, shift, bias, M)
    cases = [
        ("d8_c256_u8", 48, 128, 128, 8, 256, 0.0, False, 4),
        ("d8_c4096_b12", 32, 256, 256, 8, 4096, 0.0, True, 5),
        ("d4_c32_g64", 40, 128, 64, 4, 32, 0.0, False, 3),
        ("d4_c2048_b11_g64", 24, 128, 64, 4, 2048, 0.0, True, 2),
        ("d4_c8_b3_ragged", 5, 24, 24, 4, 8, 0.0, False, 3),
        ("d8_c65536_b16", 16, 64, 64, 8, 65536, 0.0, False, 1),
        ("d8_c4096_shift", 16, 128, 128, 8, 4096, 0.0123, True, 4),
        ("d4_c4096_b12", 32, 128, 128, 4, 4096, 0.0, False, 16),
        # a shift twelve times the weight magnitude: bf16(w + shift) keeps only 3-4 bits of w, so a
        # GEMM has to reproduce both roundings of the reconstruction to stay within tolerance
        ("d8_c4096_bigshift", 32, 256, 256, 8, 4096, -0.25, True, 16),
    ]
    for ci, (name, N, K, G, d, C, shift, with_bias, M) in enumerate(cases):
        torch.manual_seed(100 + ci)
        W = torch.randn(N, K) * 0.02
        _, payload = quantize_vector_codebook(
            W, group_size=G, vector_dim=d, codebook_size=C, sample_size=max(65536, 2 * C), iters=4,
            seed=ci, metric="euclidean", scalar_importance=None, return_packed=True)
        if shift:
            payload["shift"] = torch.tensor(shift, dtype=torch.bfloat16)
        bits = max(1, (C - 1).bit_length())
        packed = pack_indices(payload["indices"], bits)
        packed2 = packer.pack_payload(payload)
        assert torch.equal(packed2["packed_indices"], packed) and packed2["index_bits"] == bits
        w_ref = decode_fixed(payload, "cpu")                                  # fp32 holding bf16 values
        bias = (torch.randn(N, generator=torch.Generator().manual_seed(7 + ci)) * 0.1).to(torch.bfloat16) \
            if with_bias else None
        mod = shim.PrecomputedPackedVectorCodebookLinear(packed2, bias, "cpu")
        w_mod = mod.dequantize_weight()
        assert torch.equal(w_mod.float(), w_ref)
        mod_unpacked = shim.PrecomputedPackedVectorCodebookLinear(payload, bias, "cpu")
        assert torch.equal(mod_unpacked.dequantize_weight().float(), w_ref)
        ql = QuantLinear(payload, None, "cpu")
        assert torch.equal(ql.weight_().float(), w_ref)

        x = make_activations(M, K, seed=500 + ci, zero_row=True)
        q, s = perrow.quantize_rows(x, "fp8_e4m3fn")
        y_ref = (q.float() @ w_ref.t()) * s
        if bias is not None:
            y_ref = y_ref + bias.float()
        y_dense = mod(x)                                                       # stock bf16 forward
        wq, sw = perrow.quantize_rows(w_mod, "fp8_e4m3fn")                     # per-output-row weight producer
        # the deployed INT8 recipe: per-token int8 activations, per-output-row int8 weights and
        # the exact integer product the GEMM accumulates (its scaling epilogue is CUDA-only code)
        q8, s8 = perrow.quantize_rows(x, "int8_symmetric")
        wq8, sw8 = perrow.quantize_rows(w_mod, "int8_symmetric")
        acc8 = q8.to(torch.int32) @ wq8.to(torch.int32).t()

        out = dict(
            N=N, K=K, G=G, d=d, C=C, index_bits=bits,
            codebook=bf16_bits(payload["codebook"]),
            indices=payload["indices"].numpy().astype(np.int32),
            indices_dtype=str(payload["indices"].dtype),
            scales=bf16_bits(payload["scales"]),
            shift=bf16_bits(payload["shift"].reshape(1)),
            packed=packed.numpy(),
            w_ref=bf16_bits(w_ref),
            x=bf16_bits(x), q=e4m3_bits(q), act_scale=s.numpy().astype(np.float32),
            y_ref=y_ref.numpy().astype(np.float32),
            y_dense=bf16_bits(y_dense),
            wq=e4m3_bits(wq), w_scale=sw.numpy().astype(np.float32),
            q_i8=q8.numpy().astype(np.int8), act_scale_i8=s8.numpy().astype(np.float32),
            wq_i8=wq8.numpy().astype(np.int8), w_scale_i8=sw8.numpy().astype(np.float32),
            acc_i32=acc8.numpy().astype(np.int32),
        )
        if bias is not None:
            out["bias"] = bf16_bits(bias)
        np.savez_compressed(os.path.join(HERE, f"layer_{name}.npz"), **out)
        print(name, "ok", "packed bytes", packed.numel())

    # ---- 3. the hand-written payload of the reference's cache test ---------
    tiny = dict(out_features=2, in_features=4, group_size=4, vector_dim=2,
                codebook=torch.tensor([[1., 2.], [3., 4.]]), scales=torch.ones(2, 1),
                indices=torch.tensor([[[0, 1]], [[1, 0]]]))
    w_tiny = decode_fixed(dict(tiny, shift=0.0), "cpu")
    np.savez_compressed(os.path.join(HERE, "tiny_cache_payload.npz"), w_ref=bf16_bits(w_tiny))

    # ---- 4. scalar format sweeps -------------------------------------------
    allbf = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    z = allbf.float()
    clamped = z.clamp(-448.0, 448.0)
    e4 = clamped.to(torch.float8_e4m3fn)
    # per-row quantizer on rows that span magnitudes, and the per-tensor twin
    xs = make_activations(6, 512, seed=900, zero_row=True)
    q6, s6 = perrow.quantize_rows(xs, "fp8_e4m3fn")
    qt, st = rtn.Quantizer("fp8_e4m3fn").quantize(xs)
    # products and sums that exercise both bf16 roundings of the reconstruction
    gen = torch.Generator().manual_seed(77)
    a = torch.randn(4096, generator=gen).to(torch.bfloat16)
    b = (torch.randn(4096, generator=gen) * 0.02).to(torch.bfloat16)
    c = torch.tensor(0.0123, dtype=torch.bfloat16)
    prod = a.clone().mul_(b)
    summed = prod.clone().add_(c)
    np.savez_compressed(
        os.path.join(HERE, "formats.npz"),
        e4m3_of_all_bf16=e4m3_bits(e4), x6=bf16_bits(xs), q6=e4m3_bits(q6), s6=s6.numpy(),
        q_tensor=e4m3_bits(qt), s_tensor=st.numpy().reshape(1),
        mul_a=bf16_bits(a), mul_b=bf16_bits(b), mul_out=bf16_bits(prod), add_c=bf16_bits(c.reshape(1)),
        add_out=bf16_bits(summed))
    print("done")


if __name__ == "__main__":
    main()
