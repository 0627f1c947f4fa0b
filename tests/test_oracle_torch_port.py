"""The torch restatement of the reference's CPU path (the timed baseline) against the
reference-generated fixtures.  CPU only."""
import numpy as np
import torch

from oracle import sacq_oracle as O
from oracle import torch_port as T


def _bf(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def test_torch_port_bit_exact(golden_layer):
    g = golden_layer
    payload = dict(codebook=_bf(g["codebook"]), scales=_bf(g["scales"]), shift=_bf(g["shift"]).reshape(()),
                   packed_indices=torch.from_numpy(g["packed"]), index_bits=int(g["index_bits"]),
                   index_shape=tuple(g["indices"].shape), in_features=int(g["K"]), out_features=int(g["N"]),
                   group_size=int(g["G"]))
    w = T.reconstruct(payload)
    assert np.array_equal(w.view(torch.int16).numpy().view(np.uint16), g["w_ref"])
    q, s = T.quantize_rows(_bf(g["x"]))
    assert np.array_equal(q.view(torch.uint8).numpy(), g["q"])
    assert np.array_equal(s.numpy().view(np.uint32), g["act_scale"].view(np.uint32))
    bias = _bf(g["bias"]) if "bias" in g else None
    y = T.forward(payload, _bf(g["x"]), bias)
    assert O.rel_frobenius(y.numpy(), g["y_ref"]) < 1e-5
