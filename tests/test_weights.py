import json
import os

import pytest
import torch

import citlali_b200 as cb
from helpers import SEEDS, make_model_dir, tiny_config


def test_safetensors_round_trip_agrees_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int64).view(2, 3), "e": torch.empty(0, 4)}
    ours = str(tmp_path / "ours.safetensors")
    cb.write_safetensors(ours, list(tensors.items()), metadata={"k": "v"})
    theirs = load_file(ours)
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and torch.equal(theirs[k], v)
    lib = str(tmp_path / "lib.safetensors")
    save_file(tensors, lib)
    f = cb.SafetensorsFile(lib)
    assert sorted(f.names()) == sorted(tensors)
    for k, v in tensors.items():
        got = f.read(k)
        assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape) and torch.equal(got, v)
    f.close()


def test_corrupt_files_are_refused(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"\x00\x01")
    with pytest.raises(cb.CitlaliError, match="too short"):
        cb.SafetensorsFile(str(p))
    p.write_bytes((10 ** 6).to_bytes(8, "little") + b"{}")
    with pytest.raises(cb.CitlaliError, match="exceeds the file size"):
        cb.SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\x00" * 8)
    with pytest.raises(cb.CitlaliError, match="do not fit shape"):
        cb.SafetensorsFile(str(p))


def test_random_model_folder_is_reproducible_and_complete(tmp_path):
    a = make_model_dir(str(tmp_path / "a"), "B", "float32")
    b = make_model_dir(str(tmp_path / "b"), "B", "float32")
    c = make_model_dir(str(tmp_path / "c"), "B", "float32", seed=SEEDS["B"] + 1)
    fa, fb, fc = (cb.SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    cfg = tiny_config("B")
    names = [s.name for s in cb.expected_tensors(cfg.to_model_spec())]
    assert sorted(fa.names()) == sorted(names)
    assert len(names) == 3 + 11 * cfg.num_hidden_layers      # embedding, final norm, head, 11 per layer
    for n in names:
        assert torch.equal(fa.read(n), fb.read(n))
        assert not torch.equal(fa.read(n), fc.read(n))
    emb = fa.read("model.embed_tokens.weight")
    assert emb.dtype == torch.float32 and abs(emb.std().item() - 0.02) < 2e-3
    gain = fa.read("model.layers.0.self_attn.q_norm.weight")
    assert abs(gain.mean().item() - 1.0) < 0.1 and gain.std().item() > 0.02
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 96
    # a tied model stores no head
    t = make_model_dir(str(tmp_path / "t"), "A", "bfloat16")
    ft = cb.SafetensorsFile(os.path.join(t, "model.safetensors"))
    assert "lm_head.weight" not in ft and ft.dtype("model.embed_tokens.weight") == torch.bfloat16


def _rewrite(folder, change):
    path = os.path.join(folder, "model.safetensors")
    f = cb.SafetensorsFile(path)
    tensors = {n: f.read(n) for n in f.names()}
    f.close()
    change(tensors)
    cb.write_safetensors(path, list(tensors.items()))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "B", "float32")

    def change(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.extra.weight"] = torch.zeros(2)
        t["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 95)
        t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(32, dtype=torch.int32)
    _rewrite(d, change)
    loader = cb.WeightLoader(d)
    with pytest.raises(cb.CitlaliError) as e:
        loader.check(cb.expected_tensors(tiny_config("B").to_model_spec()))
    text = str(e.value)
    assert "missing tensors (2)" in text and "model.layers.1.mlp.up_proj.weight" in text and "model.norm.weight" in text
    assert "unexpected tensors (1)" in text and "model.layers.0.extra.weight" in text
    assert "wrong shapes (1)" in text and "got [64, 95], expected [64, 96]" in text
    assert "wrong dtypes (1)" in text and "q_norm" in text
    with pytest.raises(cb.CitlaliError, match="missing required tensor: nope"):
        loader.load_required("nope")
    assert loader.load_optional("nope") is None


def test_stored_dtypes_are_kept(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "A", "bfloat16")
    _rewrite(d, lambda t: t.update({"model.norm.weight": t["model.norm.weight"].to(torch.float32)}))
    loader = cb.WeightLoader(d)
    w = loader.load_all(cb.expected_tensors(tiny_config("A").to_model_spec()))
    assert w["model.norm.weight"].dtype == torch.float32          # stored in 32-bit, stays so
    assert w["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert w["model.layers.0.self_attn.q_proj.weight"].out_features == 64
    assert w["model.layers.0.mlp.down_proj.weight"].in_features == 192


def test_tied_and_untied_heads(tmp_path):
    spec_b = tiny_config("B").to_model_spec()
    d = make_model_dir(str(tmp_path / "b"), "B", "float32")
    _rewrite(d, lambda t: t.pop("lm_head.weight"))
    with pytest.raises(cb.CitlaliError, match="lm_head.weight"):
        cb.WeightLoader(d).check(cb.expected_tensors(spec_b))        # untied and absent: an error
    spec_a = tiny_config("A").to_model_spec()
    da = make_model_dir(str(tmp_path / "a"), "A", "float32")
    cb.WeightLoader(da).check(cb.expected_tensors(spec_a))           # tied and absent: fine
    _rewrite(da, lambda t: t.update({"lm_head.weight": t["model.embed_tokens.weight"].clone()}))
    cb.WeightLoader(da).check(cb.expected_tensors(spec_a))           # tied and present: ignored


def test_missing_files(tmp_path):
    with pytest.raises(cb.CitlaliError, match="no config.json"):
        cb.config_from_model_dir(str(tmp_path))
    with pytest.raises(cb.CitlaliError, match="no model.safetensors"):
        cb.WeightLoader(str(tmp_path))


def test_handles_read_on_demand_and_fill_buffers_in_place(tmp_path):
    """A handle holds no values; ``tensor`` reads a copy, ``copy_into`` fills a buffer of another dtype or a
    strided view of a larger one (how stacked and interleaved matrices are bound)."""
    d = make_model_dir(str(tmp_path / "m"), "B", "bfloat16")
    loader = cb.WeightLoader(d)
    w = loader.load_all(cb.expected_tensors(tiny_config("B").to_model_spec()))
    h = w["model.layers.0.mlp.gate_proj.weight"]
    assert h.dtype == torch.bfloat16 and h.shape == (160, 96) and h.nbytes == 160 * 96 * 2
    a, b = h.tensor, h.tensor
    assert a.data_ptr() != b.data_ptr() and torch.equal(a, b)           # nothing is kept behind the handle
    wide = torch.zeros(160, 96, dtype=torch.float32)
    h.copy_into(wide)
    assert torch.equal(wide, a.float())
    stacked = torch.zeros(10, 2, 16, 96, dtype=torch.bfloat16)           # runs of 16 rows, gate and up alternating
    h.copy_into(stacked[:, 0])
    w["model.layers.0.mlp.up_proj.weight"].copy_into(stacked[:, 1])
    flat = stacked.view(320, 96)
    assert torch.equal(flat[0:16], a[0:16]) and torch.equal(flat[32:48], a[16:32])
    assert torch.equal(flat[16:32], w["model.layers.0.mlp.up_proj.weight"].tensor[0:16])
    with pytest.raises(cb.CitlaliError, match="elements"):
        h.copy_into(torch.zeros(10, 10))
    loader.close()


def test_float16_checkpoints_reach_the_32_bit_path_exactly(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "A", "float32")
    halves = {}

    def change(t):
        for k in list(t):
            t[k] = t[k].to(torch.float16)
            halves[k] = t[k].clone()
    _rewrite(d, change)
    loader = cb.WeightLoader(d)
    w = loader.load_all(cb.expected_tensors(tiny_config("A").to_model_spec()))
    h = w["model.layers.1.self_attn.o_proj.weight"]
    assert h.dtype == torch.float16
    wide = torch.zeros(h.shape, dtype=torch.float32)
    h.copy_into(wide)
    assert torch.equal(wide, halves[h.name].float())                     # no bits lost on the way to 32-bit
    narrow = torch.zeros(h.shape, dtype=torch.bfloat16)
    h.copy_into(narrow)
    assert torch.equal(narrow, halves[h.name].to(torch.bfloat16))        # one rounding on the way to bfloat16
    loader.close()
