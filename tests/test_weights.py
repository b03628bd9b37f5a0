"""Safetensors reader/writer, loading by name with one error report, random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import helpers
from boring_llm_b200 import Qwen2Config, WeightsError, build_model, write_random_model
from boring_llm_b200.weights import (SafetensorsError, SafetensorsFile, TensorSpec, load_checkpoint,
                                     write_safetensors, INT_TABLE)


def test_write_read_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "e": torch.empty(0, 4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, {"format": "pt"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(t)
    for k in t:
        assert f.info(k) == (t[k].dtype, tuple(t[k].shape))
        assert torch.equal(f.tensor(k), t[k])
    assert f.metadata == {"format": "pt"}
    with pytest.raises(SafetensorsError, match="not found"):
        f.tensor("zzz")


def test_reader_matches_the_installed_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(4, 6).to(torch.bfloat16), "v": torch.randn(5)}
    st.save_file(t, str(tmp_path / "pkg.safetensors"))
    f = SafetensorsFile(str(tmp_path / "pkg.safetensors"))
    for k in t:
        assert torch.equal(f.tensor(k), t[k])
    write_safetensors(str(tmp_path / "own.safetensors"), t)
    back = st.load_file(str(tmp_path / "own.safetensors"))
    for k in t:
        assert torch.equal(back[k], t[k])


def _raw(tmp_path, header: bytes, data: bytes = b"", n=None):
    path = str(tmp_path / "bad.safetensors")
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header) if n is None else n) + header + data)
    return path


def test_hostile_files_give_errors_not_crashes(tmp_path):
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(_write_short(tmp_path))
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(_raw(tmp_path, b"{}", n=1 << 40))
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(_raw(tmp_path, b"{nope"))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(_raw(tmp_path, hdr, b"\0" * 8))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    with pytest.raises(SafetensorsError, match="needs 16"):
        SafetensorsFile(_raw(tmp_path, hdr, b"\0" * 8))
    hdr = json.dumps({"t": {"dtype": "Q4_K", "shape": [4], "data_offsets": [0, 8]}}).encode()
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(_raw(tmp_path, hdr, b"\0" * 8))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 8]}}).encode()
    with pytest.raises(SafetensorsError, match="invalid shape"):
        SafetensorsFile(_raw(tmp_path, hdr, b"\0" * 8))


def _write_short(tmp_path):
    path = str(tmp_path / "short.safetensors")
    with open(path, "wb") as f:
        f.write(b"\1\2\3")
    return path


def test_random_mode_is_seeded_and_follows_the_distributions(tmp_path):
    cfg = Qwen2Config.from_dict(helpers.TINY["B"])
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    write_random_model(a, cfg, 5, "float32", 0.02)
    write_random_model(b, cfg, 5, "float32", 0.02)
    write_random_model(c, cfg, 6, "float32", 0.02)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert sorted(fa.names()) == sorted(build_model(cfg).tensor_specs())
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    assert not torch.equal(fa.tensor("lm_head.weight"), fc.tensor("lm_head.weight"))
    w = fa.tensor("model.layers.1.mlp.up_proj.weight")
    assert abs(w.mean().item()) < 2e-3 and abs(w.std().item() - 0.02) < 2e-3
    nw = fa.tensor("model.norm.weight")
    assert abs(nw.mean().item() - 1.0) < 0.02
    bias = fa.tensor("model.layers.0.self_attn.q_proj.bias")
    assert abs(bias.std().item() - 0.02) < 0.01
    with open(os.path.join(a, "config.json")) as f:
        assert Qwen2Config.from_dict(json.load(f)) == cfg
    write_random_model(str(tmp_path / "h"), cfg, 5, "bfloat16", 0.02)
    fh = SafetensorsFile(os.path.join(str(tmp_path / "h"), "model.safetensors"))
    assert fh.info("lm_head.weight")[0] == torch.bfloat16
    assert torch.equal(fh.tensor("lm_head.weight"), fa.tensor("lm_head.weight").to(torch.bfloat16))


def test_random_tensors_depend_on_seed_name_and_index_only(tmp_path):
    """The folder that the random mode writes holds, bit for bit, the tensors that the in-memory mode makes; a
    tensor does not depend on which other tensors exist or in which order they are made; a prefix of a longer
    tensor of the same name is the shorter tensor (values are keyed by the flat index)."""
    from boring_llm_b200.weights import TensorSpec, random_tensor, random_tensors
    cfg = Qwen2Config.from_dict(helpers.TINY["C"])
    d = str(tmp_path / "m")
    write_random_model(d, cfg, 9, "bfloat16", 0.02)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    specs = build_model(cfg).tensor_specs()
    mem = random_tensors(specs, 9, torch.bfloat16, 0.02)
    assert sorted(mem) == sorted(f.names()) and len(mem) == len(specs)
    for n in reversed(sorted(specs)):                       # another order than the writer's
        assert torch.equal(mem[n], f.tensor(n)), n
    alone = random_tensor("model.norm.weight", specs["model.norm.weight"], 9, torch.bfloat16, 0.02)
    assert torch.equal(alone, f.tensor("model.norm.weight"))
    long = random_tensor("x", TensorSpec((7, 1000)), 1, torch.float32, 1.0).flatten()
    short = random_tensor("x", TensorSpec((3, 100)), 1, torch.float32, 1.0).flatten()
    assert torch.equal(long[:300], short)
    assert not torch.equal(random_tensor("y", TensorSpec((300,)), 1, torch.float32, 1.0), short)
    # a standard normal: moments, tails and no correlation between neighbours
    z = random_tensor("z", TensorSpec((1000, 1000)), 2, torch.float32, 1.0).double()
    assert abs(z.mean().item()) < 5e-3 and abs(z.std().item() - 1) < 5e-3
    assert abs((z ** 4).mean().item() - 3.0) < 0.05 and 4.0 < z.abs().max().item() < 6.5
    assert abs((z[:, 1:] * z[:, :-1]).mean().item()) < 5e-3 and abs((z[1:] * z[:-1]).mean().item()) < 5e-3
    q = torch.quantile(z.flatten()[:1 << 20].float(), torch.tensor([0.01, 0.25, 0.75, 0.99]))
    assert torch.allclose(q, torch.tensor([-2.3263, -0.6745, 0.6745, 2.3263]), atol=0.02)
    ids = random_tensor("t", TensorSpec((5000,), "int_table"), 2, vocab_size=37)
    assert ids.dtype == torch.int32 and ids.min().item() == 0 and ids.max().item() == 36


def test_tied_model_has_no_output_matrix(tmp_path):
    cfg = Qwen2Config.from_dict(helpers.TINY["A"])
    specs = build_model(cfg).tensor_specs()
    assert "lm_head.weight" not in specs and "model.embed_tokens.weight" in specs
    d = str(tmp_path / "m")
    write_random_model(d, cfg, 0, "float32")
    # a stored copy of the shared matrix is tolerated
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    m = build_model(cfg)
    load_checkpoint(d, m.tensor_specs(), m.ignorable_tensors)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen2Config.from_dict(helpers.TINY["B"])
    d = str(tmp_path / "m")
    write_random_model(d, cfg, 1, "float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.2.mlp.down_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(3)
    t["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(33)
    t["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(96, 96, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightsError) as e:
        load_checkpoint(d, build_model(cfg).tensor_specs())
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.2.mlp.down_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.9.extra.weight" in msg
    assert "wrong shapes (1)" in msg and "k_proj.bias: file has [33], configuration needs [32]" in msg
    assert "wrong dtypes (1)" in msg and "q_proj.weight" in msg


def test_dtypes_are_kept(tmp_path):
    specs = {"m": TensorSpec((2, 3)), "v": TensorSpec((3,)), "h": TensorSpec((3,)), "i": TensorSpec((4,), INT_TABLE)}
    t = {"m": torch.randn(2, 3).to(torch.bfloat16), "v": torch.randn(3), "h": torch.randn(3).to(torch.float16),
         "i": torch.arange(4, dtype=torch.int64)}
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    out = load_checkpoint(str(tmp_path / "m"), specs)
    assert out["m"].dtype == torch.bfloat16 and out["v"].dtype == torch.float32
    assert out["h"].dtype == torch.float32 and torch.equal(out["h"], t["h"].float())
    assert out["i"].dtype == torch.int32
    with pytest.raises(WeightsError, match="no model.safetensors"):
        load_checkpoint(str(tmp_path), specs)


def test_sharded_folder(tmp_path):
    cfg = Qwen2Config.from_dict(helpers.TINY["A"])
    d = str(tmp_path / "m")
    write_random_model(d, cfg, 0, "float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = sorted(f.names())
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    wm = {}
    for fname, ns in parts.items():
        write_safetensors(os.path.join(d, fname), {n: f.tensor(n).clone() for n in ns})
        wm.update({n: fname for n in ns})
    whole = {n: f.tensor(n).clone() for n in names}
    f.close()
    os.remove(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    out = load_checkpoint(d, build_model(cfg).tensor_specs())
    for n in names:
        assert torch.equal(out[n], whole[n])
