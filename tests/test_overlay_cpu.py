"""Overlay loader: entry resolution, dense and packed entries, strict counts (CPU; the packed
module is replaced by a recording stand-in because the real one needs a GPU)."""
import pytest
import torch

from sacq_b200 import overlay
from sacq_b200.synthetic import make_payload


class Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj = torch.nn.Linear(16, 8, bias=True)
        self.k_proj = torch.nn.Linear(16, 8, bias=False)
        self.norm = torch.nn.LayerNorm(16)


class Toy(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = torch.nn.ModuleList([Block(), Block()])


class FakePacked(torch.nn.Module):
    def __init__(self, payload, bias, device):
        super().__init__()
        self.payload, self.bias_seen, self.device_seen = payload, bias, device


def make_overlay():
    p = make_payload(8, 16, vector_dim=4, codebook_size=16, seed=0)
    return {"weights": {"layers.0.q_proj": p, "layers.1.k_proj": p, "layers.1.q_proj": torch.zeros(8, 16)},
            "expected_applied": 3, "expected_packed_applied": 2, "meta": {"note": "test"}}


def test_apply_overlay_mixed_entries(tmp_path):
    model = Toy()
    bias0 = model.layers[0].q_proj.bias
    path = tmp_path / "overlay.pt"
    torch.save(make_overlay(), path)
    n = overlay.apply_overlay(model, str(path), "cpu", scope="vlm", packed_factory=FakePacked)
    assert n == 3
    q0 = model.layers[0].q_proj
    assert isinstance(q0, FakePacked) and q0.bias_seen is bias0 and q0.runtime_scope == "vlm"
    assert q0.runtime_name == "layers.0.q_proj"
    assert isinstance(model.layers[1].k_proj, FakePacked) and model.layers[1].k_proj.bias_seen is None
    dense = model.layers[1].q_proj
    assert isinstance(dense, torch.nn.Linear) and dense.weight.dtype == torch.bfloat16 and dense.bias is not None


def test_overlay_strictness():
    ov = make_overlay()
    with pytest.raises(RuntimeError):
        overlay.apply_overlay(Toy(), dict(ov, expected_applied=4), "cpu", packed_factory=FakePacked)
    assert overlay.apply_overlay(Toy(), ov, "cpu", packed_only=True, packed_factory=FakePacked) == 2
    with pytest.raises(RuntimeError):
        overlay.apply_overlay(Toy(), dict(ov, expected_packed_applied=3), "cpu", packed_only=True,
                              packed_factory=FakePacked)
    assert overlay.apply_overlay(Toy(), ov, "cpu", skip_packed=True, packed_factory=FakePacked) == 1
    bad = {"weights": {"layers.5.q_proj": ov["weights"]["layers.0.q_proj"]}}
    with pytest.raises(KeyError):
        overlay.apply_overlay(Toy(), bad, "cpu", packed_factory=FakePacked)
    with pytest.raises(KeyError):
        overlay.apply_overlay(Toy(), ov, "cpu", required_substring="action_head.", packed_factory=FakePacked)
    unchecked = {"weights": ov["weights"]}
    assert overlay.apply_overlay(Toy(), unchecked, "cpu", allowed_suffixes=(".k_proj",), packed_factory=FakePacked) == 1
    with pytest.raises(ValueError):
        overlay.load_overlay({"weights": {}})
    with pytest.raises(FileNotFoundError):
        overlay.load_overlay("/nonexistent/overlay.pt")


def test_overlay_from_env(monkeypatch, tmp_path):
    monkeypatch.delenv("VLM_CODEBOOK_OVERLAY_PATH", raising=False)
    assert overlay.apply_overlay_from_env(Toy(), "VLM_CODEBOOK_OVERLAY_PATH", "cpu") == 0
    path = tmp_path / "o.pt"
    ov = make_overlay()
    all_packed = {"weights": {k: v for k, v in ov["weights"].items() if overlay.is_packed(v)}, "expected_applied": 2}
    torch.save(all_packed, path)
    monkeypatch.setenv("VLM_CODEBOOK_OVERLAY_PATH", str(path))
    assert overlay.apply_overlay_from_env(Toy(), "VLM_CODEBOOK_OVERLAY_PATH", "cpu", packed_only=True,
                                          packed_factory=FakePacked) == 2


def test_separate_qkv_entry_installs_three_role_layers():
    """A fused q/k/v projection whose row blocks keep their own codebooks: three packed layers in
    the order q, k, v, the bias split by their row counts, counted as one applied entry."""
    class Fused(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = torch.nn.Linear(16, 8 + 4 + 4, bias=True)

    roles = {"q": make_payload(8, 16, vector_dim=4, codebook_size=16, seed=1),
             "k": make_payload(4, 16, vector_dim=4, codebook_size=8, seed=2),
             "v": make_payload(4, 16, vector_dim=4, codebook_size=32, seed=3)}
    entry = {"format": "packed_separate_qkv_codebooks_v1", "roles": roles}
    model = Fused()
    bias = model.qkv.bias.detach().clone()
    ov = {"weights": {"qkv": entry}, "expected_applied": 1, "expected_packed_applied": 1}
    assert overlay.is_packed(entry)
    assert overlay.apply_overlay(model, ov, "cpu", scope="vlm", packed_only=True, packed_factory=FakePacked) == 1
    fused = model.qkv
    assert isinstance(fused, overlay.SeparateQKVCodebookLinear) and fused.runtime_scope == "vlm"
    assert (fused.in_features, fused.out_features) == (16, 16)
    assert [m.payload is roles[r] for m, r in zip(fused.roles, "qkv")] == [True] * 3
    assert torch.equal(torch.cat([m.bias_seen for m in fused.roles]), bias)
    # the reference's checks: exactly the roles q, k, v, one input width, matching bias length
    with pytest.raises(ValueError):
        overlay.split_qkv_roles({"format": "packed_separate_qkv_codebooks_v1", "roles": {"q": roles["q"]}})
    wide = dict(roles, v=make_payload(4, 32, vector_dim=4, codebook_size=8, seed=4))
    with pytest.raises(ValueError):
        overlay.split_qkv_roles({"format": "packed_separate_qkv_codebooks_v1", "roles": wide})
    with pytest.raises(ValueError):
        overlay.SeparateQKVCodebookLinear(entry, torch.zeros(15), "cpu", FakePacked)


def test_overlay_files_load_without_pickle_execution(tmp_path):
    """Overlay files are read with weights_only=True; a file that needs the full unpickler is
    refused unless the caller opts in."""
    class Evil:
        def __reduce__(self):
            return (print, ("executed",))

    path = tmp_path / "evil.pt"
    torch.save({"weights": {"layers.0.q_proj": torch.zeros(8, 16)}, "meta": Evil()}, path)
    with pytest.raises(Exception):
        overlay.load_overlay(str(path))
    good = tmp_path / "good.pt"
    torch.save(make_overlay(), good)
    assert set(overlay.load_overlay(str(good))["weights"]) == set(make_overlay()["weights"])
