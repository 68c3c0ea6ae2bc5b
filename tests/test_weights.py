"""Safetensors reading/writing, the manifest check and its one error, random weights (CPU)."""

import json
import os
import struct

import pytest
import torch

import tiny
from mini_infer_b200.config import build_model_spec
from mini_infer_b200.engine.model import Model, declared_tensors
from mini_infer_b200.weights import (CheckpointFolder, FolderSource, RandomSource, SafetensorsError, WeightError,
                                     check_manifest, write_model_folder, write_safetensors)


def test_written_folder_is_read_back_by_the_safetensors_package(tmp_path):
    import safetensors.torch as st
    folder = write_model_folder(str(tmp_path), tiny.CONFIG_A, seed=5, dtype=torch.bfloat16)
    theirs = st.load_file(os.path.join(folder, "model.safetensors"))
    ours = CheckpointFolder(folder)
    assert set(theirs) == set(ours.names())
    for k, v in theirs.items():
        assert v.dtype == torch.bfloat16
        assert torch.equal(v, ours.read(k)), k
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["Qwen2MoeForCausalLM"]


def test_files_written_by_the_safetensors_package_are_read(tmp_path):
    import safetensors.torch as st
    t = {"a": torch.randn(3, 5), "b": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "c": torch.randn(4).to(torch.bfloat16), "d": torch.randn(2, 2).half()}
    st.save_file(t, str(tmp_path / "model.safetensors"))
    ck = CheckpointFolder(str(tmp_path))
    for k, v in t.items():
        got = ck.read(k)
        assert got.dtype == v.dtype and torch.equal(got, v)


def test_sharded_checkpoint(tmp_path):
    import safetensors.torch as st
    st.save_file({"x": torch.ones(2)}, str(tmp_path / "s1.safetensors"))
    st.save_file({"y": torch.zeros(3)}, str(tmp_path / "s2.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    ck = CheckpointFolder(str(tmp_path))
    assert sorted(ck.names()) == ["x", "y"] and ck.read("y").shape == (3,)


def test_same_seed_same_bytes_other_seed_other_bytes(tmp_path):
    a = write_model_folder(str(tmp_path / "a"), tiny.CONFIG_B, seed=7, dtype=torch.float32)
    b = write_model_folder(str(tmp_path / "b"), tiny.CONFIG_B, seed=7, dtype=torch.float32)
    c = write_model_folder(str(tmp_path / "c"), tiny.CONFIG_B, seed=8, dtype=torch.float32)
    ra = open(os.path.join(a, "model.safetensors"), "rb").read()
    assert ra == open(os.path.join(b, "model.safetensors"), "rb").read()
    assert ra != open(os.path.join(c, "model.safetensors"), "rb").read()
    w = tiny.read_weights(a)
    assert abs(float(w["model.layers.1.mlp.experts.2.up_proj.weight"].std()) - 0.02) < 0.004
    assert abs(float(w["model.norm.weight"].mean()) - 1.0) < 0.02
    assert "lm_head.weight" not in w                    # tied embeddings: no separate head is written


def test_manifest_names_follow_the_checkpoint_layout():
    names = {d.name: d.shape for d in declared_tensors(build_model_spec(tiny.CONFIG_B))}
    assert names["model.layers.0.mlp.gate_proj.weight"] == (160, 96)           # dense layer 0
    assert names["model.layers.1.mlp.gate.weight"] == (6, 96)                  # router
    assert names["model.layers.1.mlp.experts.5.down_proj.weight"] == (96, 48)
    assert names["model.layers.1.mlp.shared_expert_gate.weight"] == (1, 96)
    assert names["model.layers.2.self_attn.k_proj.bias"] == (24,)
    assert names["model.layers.2.self_attn.q_proj.weight"] == (96, 96)
    assert "model.layers.1.mlp.gate_proj.weight" not in names
    c = {d.name for d in declared_tensors(build_model_spec(tiny.CONFIG_C))}
    assert "model.layers.0.self_attn.q_proj.bias" not in c
    assert "model.layers.0.mlp.shared_expert.up_proj.weight" not in c and "lm_head.weight" in c


def _rewrite(folder, mutate):
    import safetensors.torch as st
    path = os.path.join(folder, "model.safetensors")
    t = st.load_file(path)
    mutate(t)
    st.save_file(t, path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_model_folder(str(tmp_path), tiny.CONFIG_A, seed=1, dtype=torch.float32)

    def mutate(t):
        del t["model.layers.0.self_attn.q_proj.bias"]
        del t["model.layers.1.mlp.experts.3.up_proj.weight"]
        t["model.layers.0.extra.weight"] = torch.zeros(2)
        t["model.norm.weight"] = torch.zeros(65)
        t["model.layers.1.mlp.gate.weight"] = torch.zeros(64, 8)
    _rewrite(folder, mutate)
    m = Model(build_model_spec(tiny.CONFIG_A))
    with pytest.raises(WeightError) as ei:
        check_manifest(m.tensor_decls(), FolderSource(folder))
    e = ei.value
    assert e.missing == ["model.layers.0.self_attn.q_proj.bias", "model.layers.1.mlp.experts.3.up_proj.weight"]
    assert e.unexpected == ["model.layers.0.extra.weight"]
    assert {w[0] for w in e.wrong_shape} == {"model.norm.weight", "model.layers.1.mlp.gate.weight"}
    msg = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)",
                   "model.layers.1.mlp.gate.weight: found [64, 8], expected [8, 64]"):
        assert needle in msg


def test_integer_tensor_where_a_float_is_expected(tmp_path):
    folder = write_model_folder(str(tmp_path), tiny.CONFIG_A, seed=1, dtype=torch.float32)
    _rewrite(folder, lambda t: t.__setitem__("model.norm.weight", torch.ones(64, dtype=torch.int32)))
    with pytest.raises(WeightError, match="wrong dtypes"):
        check_manifest(Model(build_model_spec(tiny.CONFIG_A)).tensor_decls(), FolderSource(folder))


def test_tied_model_may_carry_a_head(tmp_path):
    folder = write_model_folder(str(tmp_path), tiny.CONFIG_B, seed=1, dtype=torch.float32)
    _rewrite(folder, lambda t: t.__setitem__("lm_head.weight", torch.zeros(384, 96)))
    m = Model(build_model_spec(tiny.CONFIG_B))
    check_manifest(m.tensor_decls(), FolderSource(folder), allow_unexpected=["lm_head.weight"])
    with pytest.raises(WeightError, match="unexpected"):
        check_manifest(m.tensor_decls(), FolderSource(folder))


def test_broken_files(tmp_path):
    with pytest.raises(SafetensorsError, match="neither model.safetensors"):
        CheckpointFolder(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        CheckpointFolder(str(tmp_path))
    header = json.dumps({"a": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        CheckpointFolder(str(tmp_path))
    header = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not match"):
        CheckpointFolder(str(tmp_path))


def test_random_source_is_order_independent():
    decls = declared_tensors(build_model_spec(tiny.CONFIG_A))
    s1 = RandomSource(decls, 3, torch.float32)
    s2 = RandomSource(decls, 3, torch.float32)
    names = s1.names()
    a = {n: s1.read(n) for n in names}
    b = {n: s2.read(n) for n in reversed(names)}
    assert all(torch.equal(a[n], b[n]) for n in names)


def test_the_reference_loader_finds_what_our_writer_wrote(tmp_path):
    """tests/golden/reference_safetensors_A.json is what the reference's own loader
    (src/model/safetensors_loader.cpp:44-116, compiled on the host by
    tests/golden/make_safetensors_golden.py) found in the file this repository's writer produces for
    configuration A with seed 11: names, dtype codes (src/core/tensor.h:11-17: 2 = BF16), shapes, byte
    sizes and a hash of every tensor's bytes.  The same folder written again and read by our own
    reader must give the same."""
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "golden", "reference_safetensors_A.json")) as f:
        golden = json.load(f)
    folder = str(tmp_path / "model")
    tiny.make_folder(folder, tiny.CONFIGS["A"], seed=11, dtype=torch.bfloat16)
    ck = CheckpointFolder(folder)
    assert sorted(ck.names()) == sorted(golden)
    for name, ref in golden.items():
        t = ck.read(name)
        assert t.dtype == torch.bfloat16 and ref["dtype"] == 2
        assert list(t.shape) == ref["shape"]
        raw = t.contiguous().view(torch.uint8).numpy().tobytes()
        assert len(raw) == ref["nbytes"]
        h = 1469598103934665603
        for b in raw:
            h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        assert f"{h:016x}" == ref["fnv64"], name
    ck.close()
