"""Weights by tensor name: loading, the one error that lists every fault, random weights (no GPU)."""
import json

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from helpers import make_folder
from tiny_configs import TINY_A, TINY_B
import tessweave_engine_b200 as tw
from tessweave_engine_b200.weights import WeightError


def read_all(folder):
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        return {k: f.get_tensor(k) for k in f.keys()}


def test_random_folder_has_checkpoint_names_and_is_reproducible(tmp_path):
    a = make_folder(tmp_path / "1", "A")
    b = make_folder(tmp_path / "2", "A")
    ta, tb = read_all(a), read_all(b)
    assert set(ta) == set(tb) and all(torch.equal(ta[k], tb[k]) for k in ta)
    assert "lm_head.weight" not in ta                       # tied: one matrix only
    assert "model.layers.1.self_attn.q_proj.bias" in ta and "model.layers.0.self_attn.o_proj.bias" not in ta
    assert ta["model.layers.0.mlp.gate_proj.weight"].shape == (128, 64)
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    tbb = read_all(make_folder(tmp_path / "3", "B"))
    assert tbb["lm_head.weight"].shape == (384, 96)
    # the rule per tensor: norm weights around one, the rest around zero with the config's scale
    assert abs(float(ta["model.norm.weight"].float().mean()) - 1) < 0.1
    assert abs(float(tbb["model.layers.2.mlp.down_proj.weight"].float().std()) - 0.05) < 0.01


def test_load_keeps_matrices_in_run_type_and_vectors_in_fp32(tmp_path):
    folder = make_folder(tmp_path, "B", store_dtype="float32")
    stored = read_all(folder)
    for dtype in (torch.float32, torch.bfloat16):
        model = tw.load_model(folder, dtype, "cpu")
        decls = model.weight_decls()
        assert decls["model.layers.0.self_attn.q_proj.weight"].dest.dtype == dtype
        assert decls["model.layers.0.input_layernorm.weight"].dest.dtype == torch.float32   # stored in 32 bits, stays so
        assert decls["model.layers.0.self_attn.k_proj.bias"].dest.dtype == torch.float32
        attn = model.blocks[0].mixer
        q = stored["model.layers.0.self_attn.q_proj.weight"].to(dtype)
        assert torch.equal(attn.w_qkv[: q.shape[0]], q)                    # packed rows [q; k; v]
        v = stored["model.layers.0.self_attn.v_proj.weight"].to(dtype)
        assert torch.equal(attn.w_qkv[-v.shape[0]:], v)
        up = stored["model.layers.0.mlp.up_proj.weight"].to(dtype)
        gate = stored["model.layers.0.mlp.gate_proj.weight"].to(dtype)
        packed = model.blocks[0].feed_forward.w_gate_up          # groups of eight gate rows and their eight up rows
        assert torch.equal(packed[:8], gate[:8]) and torch.equal(packed[8:16], up[:8])
        assert torch.equal(packed[-8:], up[-8:]) and torch.equal(packed[-16:-8], gate[-8:])
    tied = tw.load_model(make_folder(tmp_path, "A"), "float32", "cpu")
    assert tied.head.weight.data_ptr() == tied.embedding.weight.data_ptr()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(tmp_path, "B", store_dtype="float32")
    tensors = read_all(folder)
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.extra.weight"] = torch.zeros(2, 2)
    tensors["model.layers.2.self_attn.k_proj.bias"] = torch.zeros(7)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)      # derived: skipped
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as info:
        tw.load_model(folder, "float32", "cpu")
    text = str(info.value)
    assert "model.layers.1.mlp.down_proj.weight" in text and "model.norm.weight" in text
    assert "model.layers.0.self_attn.extra.weight" in text
    assert "model.layers.2.self_attn.k_proj.bias" in text and "[7]" in text and "[32]" in text
    assert "inv_freq" not in text


def test_tied_checkpoint_may_carry_the_output_matrix(tmp_path):
    folder = make_folder(tmp_path, "A", store_dtype="float32")
    tensors = read_all(folder)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()      # flow_engine/model.py:139-140
    save_file(tensors, str(folder / "model.safetensors"))
    tw.load_model(folder, "float32", "cpu")


def test_sharded_checkpoint_and_unsafe_shard_names(tmp_path):
    folder = make_folder(tmp_path, "A", store_dtype="float32")
    tensors = read_all(folder)
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(folder / "part-1.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(folder / "part-2.safetensors"))
    (folder / "model.safetensors").unlink()
    index = {"weight_map": {k: ("part-1.safetensors" if i < half else "part-2.safetensors") for i, k in enumerate(names)}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    model = tw.load_model(folder, "float32", "cpu")
    assert torch.equal(model.embedding.weight, tensors["model.embed_tokens.weight"])
    index["weight_map"][names[0]] = "../evil.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightError, match="unsafe"):
        tw.load_model(folder, "float32", "cpu")


def test_missing_folder_and_forward_without_weights(tmp_path):
    with pytest.raises(FileNotFoundError):
        tw.load_model(tmp_path / "nowhere", "float32", "cpu")
    with pytest.raises(ValueError):
        tw.load_model(make_folder(tmp_path, "A"), "float16", "cpu")
