"""GHOSTFLW / GFCP / safetensors files are written byte for byte as the format descriptions say
(ghostflow-core/src/serialize.rs, ghostflow-nn/src/serialization.rs) and read back to the same values."""
import json
import struct

import torch

from ghost_flow_b200 import io as gio


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<I", len(b)) + b


def test_ghostflw_golden_bytes_and_roundtrip(tmp_path):
    w = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    b = torch.tensor([0.5, -0.5], dtype=torch.bfloat16)
    p = tmp_path / "m.gf"
    gio.save_state_dict({"fc.weight": w, "fc.bias": b}, p)
    golden = b"GHOSTFLW" + struct.pack("<II", 1, 2)
    golden += _s("fc.weight") + bytes([2]) + struct.pack("<I", 2) + struct.pack("<QQ", 2, 3) + struct.pack("<6f", 1, 2, 3, 4, 5, 6)
    golden += _s("fc.bias") + bytes([1]) + struct.pack("<I", 1) + struct.pack("<Q", 2) + struct.pack("<2f", 0.5, -0.5)
    assert p.read_bytes() == golden
    sd = gio.load_state_dict(p, restore_dtype=True)
    assert torch.equal(sd["fc.weight"], w) and sd["fc.bias"].dtype == torch.bfloat16
    assert torch.equal(sd["fc.bias"], b)


def test_ghostflw_reader_rejects_newer_version(tmp_path):
    p = tmp_path / "bad.gf"
    p.write_bytes(b"GHOSTFLW" + struct.pack("<II", 2, 0))
    try:
        gio.load_state_dict(p)
        assert False, "version 2 must be rejected"
    except IOError as e:
        assert "version" in str(e)


def test_gfcp_golden_bytes_and_roundtrip(tmp_path):
    ck = gio.Checkpoint({"w": torch.tensor([[1.0, -2.0]])}, {"exp_avg.w": torch.tensor([0.25, 0.75])}, epoch=7,
                        loss=1.5, model_name="tiny", version="1.0.0", framework_version="0.4.0",
                        extra={"lr": "0.001"})
    p = tmp_path / "c.gfcp"
    gio.save_checkpoint(ck, p)
    golden = b"GFCP" + bytes([0, 4, 0]) + _s("tiny") + _s("1.0.0") + _s("0.4.0")
    golden += struct.pack("<Q", 7) + struct.pack("<f", 1.5) + struct.pack("<I", 1) + _s("lr") + _s("0.001")
    golden += struct.pack("<I", 1) + _s("w") + struct.pack("<I", 2) + struct.pack("<QQ", 1, 2) + struct.pack("<Q", 2)
    golden += struct.pack("<2f", 1.0, -2.0)
    golden += bytes([1]) + struct.pack("<I", 1) + _s("exp_avg.w") + struct.pack("<Q", 2) + struct.pack("<2f", 0.25, 0.75)
    assert p.read_bytes() == golden
    back = gio.load_checkpoint(p)
    assert back.epoch == 7 and back.loss == 1.5 and back.extra == {"lr": "0.001"} and back.model_name == "tiny"
    assert torch.equal(back.parameters["w"], ck.parameters["w"])
    assert torch.equal(back.optimizer_state["exp_avg.w"], ck.optimizer_state["exp_avg.w"])
    # without optimizer state the flag byte is 0 and nothing follows
    gio.save_checkpoint(gio.Checkpoint({"w": torch.zeros(1)}), p)
    assert p.read_bytes().endswith(struct.pack("<f", 0.0) + bytes([0]))
    assert gio.load_checkpoint(p).optimizer_state is None


def test_safetensors_layout_and_roundtrip(tmp_path):
    p = tmp_path / "m.safetensors"
    a, b = torch.arange(6, dtype=torch.float32).reshape(2, 3), torch.tensor([9.0])
    gio.save_state_dict({"a": a, "b": b}, p, fmt="safetensors")
    raw = p.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + hlen])
    assert hdr["a"] == {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]}
    assert hdr["b"]["data_offsets"] == [24, 28] and "__metadata__" not in hdr
    assert raw[8 + hlen:] == struct.pack("<7f", 0, 1, 2, 3, 4, 5, 9)
    sd = gio.load_state_dict(p)
    assert torch.equal(sd["a"], a) and torch.equal(sd["b"], b)
    # a file produced by another writer: metadata entry and a BF16 tensor
    h2 = json.dumps({"__metadata__": {"format": "pt"}, "x": {"dtype": "BF16", "shape": [2], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h2)) + h2 + torch.tensor([1.5, -2.0], dtype=torch.bfloat16).view(torch.int16).numpy().tobytes())
    assert gio.load_state_dict(p)["x"].tolist() == [1.5, -2.0]
