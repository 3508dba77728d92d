import json

import pytest
import torch

import helpers as H
import plain_llama as P
from batchspec_b200.config import config_from_json_dict
from batchspec_b200.models import get_model
from batchspec_b200.parts import Runtime
from batchspec_b200.weights import (WeightsError, load_weights, open_model_files, random_weights, write_random_model,
                                    write_safetensors)

CPU = Runtime(torch.float32, torch.device("cpu"))


def _specs(cfg_json):
    model = get_model(config_from_json_dict(cfg_json), CPU)
    return model, model.param_specs()


def test_folder_has_the_architecture_s_names_and_shapes(tmp_path):
    folder = H.make_folder(tmp_path, H.TINY_A, seed=0)
    f = open_model_files(folder)[0]
    assert f.entries["model.embed_tokens.weight"] == (torch.float32, (512, 64))
    assert f.entries["model.layers.1.self_attn.k_proj.weight"][1] == (2 * 16, 64)
    assert f.entries["model.layers.0.mlp.gate_proj.weight"][1] == (176, 64)
    assert f.entries["lm_head.weight"][1] == (512, 64)
    tied = open_model_files(H.make_folder(tmp_path / "b", H.TINY_B, seed=1))[0]
    assert "lm_head.weight" not in tied.entries
    # the plain reader (which shares no code) reads the same numbers
    _, w = P.read_model_folder(folder)
    assert torch.equal(w["model.norm.weight"].float(), f.tensor("model.norm.weight"))


def test_random_mode_is_a_function_of_seed_and_name(tmp_path):
    model, specs = _specs(H.TINY_A)
    a = random_weights(specs, 3, torch.float32, "cpu")
    b = random_weights(dict(reversed(list(specs.items()))), 3, torch.float32, "cpu")
    assert all(torch.equal(a[k], b[k]) for k in a)
    c = random_weights(specs, 4, torch.float32, "cpu")
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    folder = write_random_model(config_from_json_dict(H.TINY_A), tmp_path, 3, dtype=torch.float32)
    loaded = load_weights(folder, specs, torch.float32, "cpu")
    assert all(torch.equal(a[k], loaded[k]) for k in a)
    w = a["model.layers.0.mlp.up_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 2e-3 and abs(float(a["model.norm.weight"].mean()) - 1) < 0.01


def test_dtype_rule(tmp_path):
    model, specs = _specs(H.TINY_A)
    f32 = H.make_folder(tmp_path / "f32", H.TINY_A, 0, dtype=torch.float32)
    bf = H.make_folder(tmp_path / "bf", H.TINY_A, 0, dtype=torch.bfloat16)
    held = load_weights(f32, specs, torch.bfloat16, "cpu")
    assert held["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16      # matrices: run dtype
    assert held["model.norm.weight"].dtype == torch.float32                            # stored in 32-bit: stays
    held = load_weights(bf, specs, torch.bfloat16, "cpu")
    assert held["model.norm.weight"].dtype == torch.bfloat16
    held = load_weights(bf, specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in held.values())


def test_one_error_lists_everything(tmp_path):
    model, specs = _specs(H.TINY_A)
    good = random_weights(specs, 0, torch.float32, "cpu")
    bad = dict(good)
    del bad["model.layers.1.mlp.down_proj.weight"], bad["model.norm.weight"]
    bad["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    bad["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)        # ignored by rule
    bad["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    bad["extra.bias"] = torch.zeros(3)
    (tmp_path / "config.json").write_text(json.dumps(H.TINY_A))
    write_safetensors(tmp_path / "model.safetensors", bad.items())
    with pytest.raises(WeightsError) as ei:
        load_weights(tmp_path, specs, torch.float32, "cpu", ignore_suffixes=model.spec.ignore_suffixes)
    e = ei.value
    assert sorted(e.missing) == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert sorted(e.unexpected) == ["extra.bias", "model.layers.7.mlp.up_proj.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 63), (64, 64))]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shapes", "extra.bias", "[64, 63]", "model.norm.weight"):
        assert word in msg


def test_tied_head_and_missing_files(tmp_path):
    model, specs = _specs(H.TINY_B)
    assert "lm_head.weight" not in specs
    tensors = random_weights(specs, 1, torch.float32, "cpu")
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()     # some checkpoints store it anyway
    write_safetensors(tmp_path / "model.safetensors", tensors.items())
    load_weights(tmp_path, specs, torch.float32, "cpu", must_equal=model.spec.must_equal)
    # ... but a stored head that is not the embedding contradicts tie_word_embeddings: an error, not a choice
    other = tmp_path / "unequal"
    other.mkdir()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"] + 1e-3
    write_safetensors(other / "model.safetensors", tensors.items())
    with pytest.raises(WeightsError, match="lm_head.weight differs from model.embed_tokens.weight") as err:
        load_weights(other, specs, torch.float32, "cpu", must_equal=model.spec.must_equal)
    assert err.value.unequal == [("lm_head.weight", "model.embed_tokens.weight")]
    with pytest.raises(FileNotFoundError):
        load_weights(tmp_path / "nowhere", specs, torch.float32, "cpu")
    untied, uspecs = _specs(H.TINY_A)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_weights(tmp_path, uspecs, torch.float32, "cpu")


def test_sharded_index(tmp_path):
    model, specs = _specs(H.TINY_A)
    t = random_weights(specs, 0, torch.float32, "cpu")
    names = list(t)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", [(n, t[n]) for n in names[:5]])
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", [(n, t[n]) for n in names[5:]])
    wm = {n: ("model-00001-of-00002.safetensors" if i < 5 else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    loaded = load_weights(tmp_path, specs, torch.float32, "cpu")
    assert all(torch.equal(t[k], loaded[k]) for k in t)
