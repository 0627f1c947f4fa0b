"""The C oracle (oracle/sacq_oracle.c) against the reference-generated fixtures and the
numpy oracle.  CPU only."""
import numpy as np

from oracle import build_oracle as C
from oracle import sacq_oracle as O


def test_c_unpack_and_reconstruction(golden_layer):
    g = golden_layer
    N, K, G, bits = int(g["N"]), int(g["K"]), int(g["G"]), int(g["index_bits"])
    idx = C.unpack(g["packed"], bits, g["indices"].size)
    assert np.array_equal(idx, g["indices"].reshape(-1))
    w = C.dequant(g["packed"], bits, g["codebook"], g["scales"], int(g["shift"][0]), N, K, G)
    assert np.array_equal(w, g["w_ref"])


def test_c_activation_quantizer(golden_layer):
    g = golden_layer
    q, s = C.quant_rows(g["x"])
    assert np.array_equal(q, g["q"])
    assert np.array_equal(s.view(np.uint32), g["act_scale"].view(np.uint32))


def test_c_int8_activation_quantizer():
    from conftest import load_golden
    f = load_golden("act_int8")
    q, s = C.quant_rows_int8(f["x"])
    assert np.array_equal(q, f["q"]) and np.array_equal(s.view(np.uint32), f["s"].view(np.uint32))


def test_c_linear(golden_layer):
    g = golden_layer
    N, K, G, bits = int(g["N"]), int(g["K"]), int(g["G"]), int(g["index_bits"])
    y = C.linear(g["packed"], bits, g["codebook"], g["scales"], int(g["shift"][0]), g.get("bias"), N, K, G,
                 g["q"], g["act_scale"])
    assert O.rel_frobenius(y, g["y_ref"]) < 1e-5


def test_c_threads_setting():
    n = C.threads()
    assert n >= 1
    C.set_threads(1)
    assert C.threads() == 1
    C.set_threads(n)
