"""Safetensors reading and writing, the loader's storage rule and its one error (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from gophonic_b200.weights import (Checkpoint, CheckpointError, InitScales, WeightsError, declare_model,
                                   load_tensors, write_random_model, write_safetensors)
from gophonic_b200.weights.safetensors_io import bf16_bits_to_float32, float32_to_bf16_bits
from tests.conftest import tiny_configs


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.1415927], dtype=np.float32)
    # 1 + 2^-8 lies halfway between 1 and 1 + 2^-7: ties to even (1.0); 1 + 3*2^-8 ties up to 1 + 2^-6
    back = bf16_bits_to_float32(float32_to_bf16_bits(x))
    assert back[0] == 1.0 and back[1] == 1.0 and back[2] == np.float32(1.015625) and back[3] == -2.5
    assert abs(back[4] - 3.140625) < 1e-6
    t = torch.tensor(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(back, t)


def test_round_trip_is_bit_exact(model_dirs):
    cfg = tiny_configs()["B"]
    decls = declare_model(cfg.model_spec())
    with Checkpoint(model_dirs["B"]) as ck:
        assert sorted(ck.names()) == sorted(d.name for d in decls)
        raw = {n: ck.read(n).copy() for n in ck.names()}
    tensors = load_tensors(model_dirs["B"], decls, "bfloat16", "cpu")
    for d in decls:
        t = tensors[d.name]
        if d.role == "norm":
            assert t.dtype == torch.float32
            assert np.array_equal(t.numpy(), bf16_bits_to_float32(raw[d.name]))
        else:
            assert t.dtype == torch.bfloat16
            assert np.array_equal(t.view(torch.int16).numpy().view(np.uint16), raw[d.name])
    wide = load_tensors(model_dirs["B"], decls, "float32", "cpu")
    for d in decls:
        assert wide[d.name].dtype == torch.float32
        assert np.array_equal(wide[d.name].numpy(), bf16_bits_to_float32(raw[d.name]))


def test_a_tensor_stored_in_32_bit_stays_so(model_dirs):
    cfg = tiny_configs()["A"]
    decls = declare_model(cfg.model_spec())
    t = load_tensors(model_dirs["A32"], decls, "bfloat16", "cpu")
    assert t["model.layers.0.self_attn.q_proj.weight"].dtype == torch.float32
    assert t["model.embed_tokens.weight"].dtype == torch.float32
    assert "lm_head.weight" not in t  # tied: the head is absent and that is no error


def test_random_weights_are_a_function_of_seed_and_name(tmp_path):
    cfg = tiny_configs()["A"]
    a, b, c = (str(tmp_path / n) for n in "abc")
    write_random_model(cfg, 5, a)
    write_random_model(cfg, 5, b)
    write_random_model(cfg, 6, c)
    with Checkpoint(a) as ca, Checkpoint(b) as cb, Checkpoint(c) as cc:
        for n in ca.names():
            assert np.array_equal(ca.read(n), cb.read(n))
        assert not np.array_equal(ca.read("model.embed_tokens.weight"), cc.read("model.embed_tokens.weight"))
        norm = bf16_bits_to_float32(ca.read("model.norm.weight"))
        assert abs(norm.mean() - 1.0) < 0.05
    assert json.load(open(os.path.join(a, "config.json")))["tie_word_embeddings"] is True


def _rewrite(src_dir, dst_dir, edit):
    with Checkpoint(src_dir) as ck:
        tensors = {n: (ck.tensors[n].dtype, ck.tensors[n].shape, ck.read(n).reshape(-1).copy()) for n in ck.names()}
    edit(tensors)
    os.makedirs(dst_dir, exist_ok=True)
    write_safetensors(os.path.join(dst_dir, "model.safetensors"), tensors)
    with open(os.path.join(src_dir, "config.json")) as f, open(os.path.join(dst_dir, "config.json"), "w") as g:
        g.write(f.read())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_dirs, tmp_path):
    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.9.extra.weight"] = ("BF16", (2, 2), np.zeros(4, dtype=np.uint16))
        dt, shape, arr = t["model.layers.0.self_attn.q_proj.weight"]
        t["model.layers.0.self_attn.q_proj.weight"] = (dt, (shape[1], shape[0]), arr)
        t["model.layers.2.self_attn.q_norm.weight"] = ("I32", (32,), np.zeros(32, dtype=np.int32))
    bad = str(tmp_path / "bad")
    _rewrite(model_dirs["B"], bad, edit)
    decls = declare_model(tiny_configs()["B"].model_spec())
    with pytest.raises(WeightsError) as ei:
        load_tensors(bad, decls, "bfloat16", "cpu")
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert len(e.wrong_shape) == 1 and "q_proj" in e.wrong_shape[0] and "[96, 192]" in e.wrong_shape[0]
    assert len(e.wrong_dtype) == 1 and "q_norm" in e.wrong_dtype[0]
    msg = str(e)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "unusable dtypes (1)"):
        assert word in msg


def test_tensors_nobody_declared_are_left_alone_unless_strict(model_dirs, tmp_path):
    """A snapshot that carries a tensor beyond the model's own loads (the reference resolves by name
    and ignores the rest: internal/qwen3lm/weights.go:291-351); the name is reported in a warning,
    and ``strict`` turns it into the error."""
    def edit(t):
        t["model.rotary_emb.inv_freq"] = ("F32", (8,), np.zeros(8, dtype=np.float32))
    d = str(tmp_path / "extra")
    _rewrite(model_dirs["A"], d, edit)
    decls = declare_model(tiny_configs()["A"].model_spec())
    with pytest.warns(UserWarning, match="model.rotary_emb.inv_freq"):
        t = load_tensors(d, decls, "bfloat16", "cpu")
    assert "model.rotary_emb.inv_freq" not in t and "model.norm.weight" in t
    with pytest.raises(WeightsError) as ei:
        load_tensors(d, decls, "bfloat16", "cpu", strict=True)
    assert ei.value.unexpected == ["model.rotary_emb.inv_freq"] and not ei.value.missing


def test_half_precision_matrices_are_widened_not_rounded(model_dirs, tmp_path):
    """An F16 matrix has three more mantissa bits than bfloat16: it becomes float32, exactly, in both
    modes (the reference refuses matrices that are not BF16: internal/qwen3lm/weights.go:754-756)."""
    vals = (np.arange(64 * 64, dtype=np.float32).reshape(64, 64) / 4096 + 1 / 1024).astype(np.float16)

    def edit(t):
        t["model.layers.0.self_attn.o_proj.weight"] = ("F16", (64, 64), vals.reshape(-1).copy())
    d = str(tmp_path / "half")
    _rewrite(model_dirs["A"], d, edit)
    decls = declare_model(tiny_configs()["A"].model_spec())
    for mode in ("bfloat16", "float32"):
        t = load_tensors(d, decls, mode, "cpu")["model.layers.0.self_attn.o_proj.weight"]
        assert t.dtype == torch.float32 and np.array_equal(t.numpy(), vals.astype(np.float32))


def test_the_same_seed_gives_the_same_bits_on_every_path(tmp_path):
    """One fill for the folder writer and for whoever restates it: element i of a tensor depends on
    (seed, tensor name, i) alone.  The plain implementation's own restatement of the formula gives
    the writer's bits; the values have the wanted mean and deviation."""
    from gophonic_b200.weights import InitScales, write_random_model
    from gophonic_b200.weights.random_init import counter_fill, fill_constant
    from tests.plain import qwen3_plain as P
    cfg = tiny_configs()["B"]
    d = str(tmp_path / "m")
    scales = InitScales(matrix=0.02, embedding=0.5, head=0.1, norm=0.05)
    write_random_model(cfg, seed=11, out_dir=d, weight_dtype="bfloat16", scales=scales)
    _, stored = P.read_model(d)
    made = P.random_weights(json.load(open(os.path.join(d, "config.json"))), 11, matrix=0.02, embedding=0.5, head=0.1, norm=0.05)
    assert sorted(stored) == sorted(made)
    for name in stored:
        assert np.array_equal(stored[name], made[name]), name
    # a tensor cut anywhere is the same tensor; the moments are the normal law's
    whole = counter_fill(12345, (1 << 22) + 77, 0.02, 0.0)
    assert np.array_equal(whole[:1000], counter_fill(12345, 1000, 0.02, 0.0))
    assert abs(float(whole.mean())) < 1e-4 and abs(float(whole.std()) / 0.02 - 1) < 2e-3
    assert float(np.abs(whole).max()) <= 262140 * float(fill_constant(0.02)) * 1.0001
    assert abs(float(counter_fill(9, 1 << 16, 0.05, 1.0).mean()) - 1.0) < 1e-3


def test_untied_model_without_head_reports_it_only_if_it_cannot_tie(model_dirs, tmp_path):
    # Qwen3's head may always be tied to the embedding: a checkpoint without lm_head loads
    def edit(t):
        del t["lm_head.weight"]
    d = str(tmp_path / "nohead")
    _rewrite(model_dirs["B"], d, edit)
    t = load_tensors(d, declare_model(tiny_configs()["B"].model_spec()), "bfloat16", "cpu")
    assert "lm_head.weight" not in t


def test_truncated_and_corrupt_files(model_dirs, tmp_path):
    src = os.path.join(model_dirs["A"], "model.safetensors")
    data = open(src, "rb").read()
    d = tmp_path / "trunc"
    d.mkdir()
    (d / "model.safetensors").write_bytes(data[:len(data) - 100])
    with pytest.raises(CheckpointError, match="invalid data offsets"):
        Checkpoint(str(d))
    (d / "model.safetensors").write_bytes(data[:4])
    with pytest.raises(CheckpointError, match="too short"):
        Checkpoint(str(d))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + data[8:])
    with pytest.raises(CheckpointError, match="invalid header length"):
        Checkpoint(str(d))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 16) + b"not json at all!" + b"\0" * 32)
    with pytest.raises(CheckpointError, match="cannot parse header"):
        Checkpoint(str(d))
    with pytest.raises(CheckpointError, match="cannot open"):
        Checkpoint(str(tmp_path / "nothing-here"))


def test_sharded_index_and_plain_shard_names(model_dirs, tmp_path):
    with Checkpoint(model_dirs["A"]) as ck:
        tensors = {n: (ck.tensors[n].dtype, ck.tensors[n].shape, ck.read(n).reshape(-1).copy()) for n in ck.names()}
    names = sorted(tensors)
    d = tmp_path / "sharded"
    d.mkdir()
    half = len(names) // 2
    write_safetensors(str(d / "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(str(d / "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[half:]})
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with Checkpoint(str(d)) as ck:
        assert ck.names() == names
        assert np.array_equal(ck.read(names[-1]).reshape(-1), tensors[names[-1]][2])
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../evil.safetensors"}}))
    with pytest.raises(CheckpointError, match="plain file name"):
        Checkpoint(str(d))


def test_non_finite_norm_vector_is_rejected(model_dirs, tmp_path):
    def edit(t):
        dt, shape, arr = t["model.norm.weight"]
        arr = arr.copy()
        arr[3] = 0x7FC0  # bfloat16 NaN
        t["model.norm.weight"] = (dt, shape, arr)
    d = str(tmp_path / "nan")
    _rewrite(model_dirs["A"], d, edit)
    with pytest.raises(CheckpointError, match="non-finite"):
        load_tensors(d, declare_model(tiny_configs()["A"].model_spec()), "bfloat16", "cpu")
