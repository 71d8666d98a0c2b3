"""Converter preflight on tiny synthetic HF-style checkpoints: the rejections the reference's converter tests
pin (tests/test_bonsai_converter.py:59-167: every incomplete or malformed source raises ValueError with that
text and leaves no output behind; an existing output is never touched), the 4B shape table, and a valid
conversion.  CPU only; stand-in shapes, never real weights."""
import copy
import json

import pytest
import torch
from safetensors.torch import save_file

from bitmtp_b200 import checkpoint_validation as CVAL, convert_bonsai_mtp_to_gpu as CV

BASE = {"hidden_size": 128, "num_hidden_layers": 1, "num_attention_heads": 1, "num_key_value_heads": 1,
        "head_dim": 128, "intermediate_size": 128, "vocab_size": 16, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
        "rope_scaling": {"original_max_position_embeddings": 32, "factor": 4.0}, "tie_word_embeddings": True,
        "block_size": 4, "causal_attn": True, "text_mask_token_id": 15}


def _weights():
    w = {"model.embed_tokens.weight": torch.ones(16, 128), "model.norm.weight": torch.ones(128)}
    p = "model.layers.0."
    for n in ("input_layernorm", "post_attention_layernorm", "self_attn.q_norm", "self_attn.k_norm"):
        w[p + n + ".weight"] = torch.ones(128)
    for n in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
              "mlp.up_proj", "mlp.down_proj"):
        w[p + n + ".weight"] = torch.ones(128, 128)
    return w


@pytest.fixture
def dirs(tmp_path):
    src, out = tmp_path / "hf", tmp_path / "converted"
    src.mkdir()
    (src / "config.json").write_text(json.dumps(BASE))
    return src, out


def _rejected(src, out, pattern, **options):
    with pytest.raises(ValueError, match=pattern):
        CV.convert(str(src), str(out), **options)
    assert not out.exists(), "an invalid source left conversion artifacts behind"


def test_sources_that_are_not_a_complete_checkpoint(dirs):
    src, out = dirs
    _rejected(src, out, "safe_serialization=True")                                    # no shards at all
    (src / "pytorch_model.bin").write_bytes(b"not model weights")
    _rejected(src, out, "safe_serialization=True")                                    # .bin only
    (src / "model.safetensors").write_bytes(b"not safetensors")
    _rejected(src, out, "invalid HF safetensors shard")
    save_file({}, str(src / "model.safetensors"))
    _rejected(src, out, "empty safetensors shard")
    (src / "config.json").unlink()
    _rejected(src, out, "missing HF config.json")


@pytest.mark.parametrize("mutate,pattern", [
    (lambda w: w.pop("model.layers.0.self_attn.k_proj.weight"), "incomplete HF checkpoint.*missing 1 core"),
    (lambda w: w.__setitem__("model.layers.0.self_attn.q_proj.weight", torch.ones(127, 128)), "tensor shape mismatch"),
    (lambda w: w.__setitem__("model.embed_tokens.weight", torch.ones(16, 128, dtype=torch.int8)), "floating-point HF weights"),
    (lambda w: w.__setitem__("unrecognized.weight", torch.ones(1)), "unsupported tensor key"),
])
def test_malformed_tensors(dirs, mutate, pattern):
    src, out = dirs
    w = _weights()
    mutate(w)
    save_file(w, str(src / "model.safetensors"))
    _rejected(src, out, pattern)


def test_layer_count_duplicates_and_untied_head(dirs):
    src, out = dirs
    save_file(_weights(), str(src / "model-1.safetensors"))
    save_file({"model.norm.weight": torch.ones(128)}, str(src / "model-2.safetensors"))
    _rejected(src, out, "duplicate tensor key across shards")
    (src / "model-2.safetensors").unlink()
    (src / "config.json").write_text(json.dumps(dict(BASE, num_hidden_layers=2)))
    _rejected(src, out, "incomplete HF checkpoint.*missing 11 core")
    (src / "config.json").write_text(json.dumps(dict(BASE, tie_word_embeddings=False)))
    _rejected(src, out, "incomplete HF checkpoint.*lm_head")


@pytest.mark.parametrize("key,bad", [("rope_scaling", None), ("hidden_size", 127), ("tie_word_embeddings", "true"),
                                     ("text_mask_token_id", 100), ("head_dim", 127), ("num_key_value_heads", 3),
                                     ("rms_norm_eps", 0), ("causal_attn", "yes"), ("block_size", 0)])
def test_bad_config_is_rejected_before_any_output(dirs, key, bad):
    src, out = dirs
    save_file(_weights(), str(src / "model.safetensors"))
    cfg = copy.deepcopy(BASE)
    cfg[key] = bad
    (src / "config.json").write_text(json.dumps(cfg))
    _rejected(src, out, "config.json")


def test_existing_output_is_never_touched(dirs):
    src, out = dirs
    out.mkdir()
    (out / "sentinel.txt").write_text("keep")
    with pytest.raises(ValueError):                                   # invalid source, existing output
        CV.convert(str(src), str(out))
    save_file(_weights(), str(src / "model.safetensors"))
    with pytest.raises(ValueError, match="output already exists"):   # valid source, existing output
        CV.convert(str(src), str(out))
    assert [p.name for p in out.iterdir()] == ["sentinel.txt"] and (out / "sentinel.txt").read_text() == "keep"
    (out / "sentinel.txt").unlink()
    with pytest.raises(ValueError, match="output already exists"):   # empty directory
        CV.convert(str(src), str(out))
    out.rmdir()
    out.write_bytes(b"keep")
    with pytest.raises(ValueError, match="output already exists"):   # a file
        CV.convert(str(src), str(out))
    out.unlink()
    out.symlink_to(out.parent / "missing")
    with pytest.raises(ValueError, match="output already exists"):   # a dangling link
        CV.convert(str(src), str(out))
    assert out.is_symlink()


def test_option_combinations_that_write_nothing(dirs):
    src, out = dirs
    save_file(_weights(), str(src / "model.safetensors"))
    _rejected(src, out, "at least one output", pack_kernel=False, pack_fp16=False)
    _rejected(src, out, "Q1-only", quantize_embedding=False)
    _rejected(src, out, "quant must be", quant="not-a-grid")


def test_sdlm_metadata_must_agree_with_the_config(dirs):
    src, out = dirs
    save_file(_weights(), str(src / "model.safetensors"))
    (src / "sdlm_config.json").write_text(json.dumps({"block_size": 8, "causal_attn": True, "text_mask_token_id": 15}))
    _rejected(src, out, "sdlm_config.json conflicts with config.json: block_size")
    (src / "sdlm_config.json").write_text(json.dumps({"block_size": 4, "causal_attn": True}))
    _rejected(src, out, "invalid or missing text_mask_token_id")
    (src / "sdlm_config.json").write_text(json.dumps({"block_size": 4, "causal_attn": True, "text_mask_token_id": 15}))
    CV.convert(str(src), str(out))
    assert (out / "model_state_t2g128.pt").is_file()


def test_valid_conversion_and_the_4b_shape_table(dirs):
    src, out = dirs
    save_file(_weights(), str(src / "model.safetensors"))
    CV.convert(str(src), str(out))
    packed = torch.load(out / "model_state_t2g128.pt", weights_only=True)
    key = "layers.0.attention.q_proj"
    assert packed[key + ".weight"].dtype == torch.int8 and tuple(packed[key + ".weight"].shape) == (128, 32)
    assert packed[key + ".weight_scale"].dtype == torch.bfloat16
    assert packed["norm.weight"].dtype == torch.bfloat16 and packed["embed_tokens.weight"].dtype == torch.bfloat16
    cfg = json.loads((out / "bonsai_gpu_config.json").read_text())
    assert cfg["kernel_kind"] == "t2g128" and cfg["block_size"] == 4
    shapes = CVAL.expected_tensor_shapes(dict(BASE, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8,
                                              intermediate_size=9728))
    assert shapes["model.layers.0.self_attn.q_proj.weight"] == (4096, 2560)
    assert shapes["model.layers.0.self_attn.k_proj.weight"] == (1024, 2560)
    assert shapes["model.layers.0.self_attn.o_proj.weight"] == (2560, 4096)
    assert shapes["model.layers.0.mlp.down_proj.weight"] == (2560, 9728)
