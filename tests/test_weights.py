"""Weights by tensor name: what is kept in which dtype, the one error for everything that is wrong,
and the random-weights folder."""
import json

import pytest
import torch

from helpers import make_model_folder
from tiny_configs import TINY_A, TINY_B

from llm_infrence_engine_b200.models import build_model_spec
from llm_infrence_engine_b200.weights import (SafetensorsFile, WeightsError, load_weights, random_tensors, write_random_model,
                                              write_safetensors)


def test_random_folder_is_reproducible_and_loads_elsewhere(tmp_path):
    a = write_random_model(TINY_A, tmp_path / "a", 0)
    b = write_random_model(TINY_A, tmp_path / "b", 0)
    c = write_random_model(TINY_A, tmp_path / "c", 1)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    from safetensors.torch import load_file  # the library reads what the package wrote

    t = load_file(str(a / "model.safetensors"))
    assert "lm_head.weight" not in t and t["model.embed_tokens.weight"].shape == (256, 64)
    assert abs(t["model.layers.0.mlp.up_proj.weight"].std().item() - 0.02) < 2e-3
    n = t["model.layers.1.input_layernorm.weight"]
    assert 0.9 <= n.min() and n.max() <= 1.1 and n.std() > 0.01
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    assert "lm_head.weight" in random_tensors(TINY_B, 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dtypes_and_fusing(tmp_path, dtype):
    folder = make_model_folder(tmp_path, "B")
    spec = build_model_spec(TINY_B)
    load_weights(spec, folder, dtype, "cpu")
    f = SafetensorsFile(folder / "model.safetensors")
    m = spec.layers[2].mixer
    assert m.w_qkv.dtype == dtype and m.w_qkv.shape == (5 * 32, 96)
    want = torch.cat([f.tensor(f"model.layers.2.self_attn.{n}_proj.weight") for n in "qkv"]).to(dtype)
    assert torch.equal(m.w_qkv, want)
    assert m.b_qkv.dtype == torch.float32  # vectors stay 32-bit
    assert spec.layers[0].norm1.weight.dtype == torch.float32
    assert spec.final_norm.weight.dtype == torch.float32
    assert torch.equal(spec.layers[1].ff.w_gate_up[200:], f.tensor("model.layers.1.mlp.up_proj.weight").to(dtype))
    assert spec.head.matrix().shape == (320, 96)


def test_tied_head_shares_the_table(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    spec = build_model_spec(TINY_A)
    load_weights(spec, folder, torch.float32, "cpu")
    assert spec.head.matrix() is spec.embedding.table


def test_one_error_lists_everything(tmp_path):
    folder = make_model_folder(tmp_path, "B")
    f = SafetensorsFile(folder / "model.safetensors")
    t = {n: f.tensor(n) for n in f.names()}
    f.close()
    del t["model.layers.1.mlp.down_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 90)
    t["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    t["model.layers.0.input_layernorm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(folder / "model.safetensors", t)
    with pytest.raises(WeightsError) as e:
        load_weights(build_model_spec(TINY_B), folder, torch.float32, "cpu")
    msg = str(e.value)
    assert "model.layers.1.mlp.down_proj.weight" in msg and "model.norm.weight" in msg and "missing (2)" in msg
    assert "unexpected (1): model.layers.7.mlp.up_proj.weight" in msg
    assert "model.layers.0.self_attn.q_proj.weight is [96, 90], the model needs [96, 96]" in msg
    assert "wrong dtype: model.layers.0.input_layernorm.weight" in msg
    assert e.value.missing == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]


def test_tied_checkpoint_may_carry_the_head_name(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    f = SafetensorsFile(folder / "model.safetensors")
    t = {n: f.tensor(n) for n in f.names()}
    f.close()
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(folder / "model.safetensors", t)
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("error")   # equal to the table: no error, no warning; the name is known and not needed
        load_weights(build_model_spec(TINY_A), folder, torch.float32, "cpu")
    t["lm_head.weight"][3, 5] += 1.0
    write_safetensors(folder / "model.safetensors", t)
    spec = build_model_spec(TINY_A)
    with pytest.warns(UserWarning, match="lm_head.weight.*differs.*model.embed_tokens.weight"):
        load_weights(spec, folder, torch.float32, "cpu")
    assert spec.head.matrix() is spec.embedding.table   # the table is what is used, as the configuration says


def test_no_file(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_weights(build_model_spec(TINY_A), tmp_path, torch.float32, "cpu")
