"""CPU-side contracts of the drop-in boundary: the C-ABI library loads and exports every
declared symbol, metadata validation fires before any native load, the CLI's --check-only
never imports torch, and the converter writes the reference's checkpoint layout."""
import json
import os
import subprocess
import sys

import pytest
import torch

from bitmtp_b200 import contracts, native, synthetic

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = native.lib()
    names = native.exported_symbols()
    assert "t2g128_int8xint2_linear" in names and "bm_t2_gemv" in names and len(names) >= 18
    for n in names:
        assert hasattr(lib, n), n
    assert b"sm_100a" in lib.bm_version()
    # host-only arithmetic entry points are callable without a GPU
    assert lib.bm_t2_gemv_bytes(1, 6144, 2048, 0) == 3356676           # the baseline's byte count
    assert lib.bm_t2_gemv_bytes(8, 2048, 6144, 0) == 3424288
    assert lib.bm_verify_attention_scratch_bytes(16, 16, 1024) > 0


def test_validation_precedes_native_load():
    """Meta tensors allocate nothing; a bad shape must be rejected before the library is
    touched (the reference's own guard test: tests/test_bonsai_cpu.py:44-54)."""
    from bitmtp_b200 import model
    a = torch.empty((4, 2560), dtype=torch.int8, device="meta")
    b = torch.empty((151936, 640), dtype=torch.int8, device="meta")
    s = torch.empty((4, 1), dtype=torch.float32, device="meta")
    ws = torch.empty((151936, 20), dtype=torch.bfloat16, device="meta")
    saved, model._t2_lib = model._t2_lib, None
    try:
        with pytest.raises(RuntimeError, match="unsupported t2g128 kernel shape"):
            model.t2g128_int8xint2_linear(a, b, s, ws, validate_registry=True)   # M=4 is not a 4B width
        with pytest.raises(RuntimeError, match="contiguous CUDA tensors"):
            model.t2g128_int8xint2_linear(a, b, s, ws)
        with pytest.raises(RuntimeError, match="invalid weight scale shape"):
            model.t2g128_int8xint2_linear(a, b, s, ws[:, :10])
        assert model._t2_lib is None
    finally:
        model._t2_lib = saved


def test_registry_and_scope():
    assert contracts.supports_kernel_shape("t2g128", 9, 4096, 2048)
    assert contracts.supports_kernel_shape("t2g128", 16, 19456, 2560)
    assert not contracts.supports_kernel_shape("t2g128", 2, 4096, 2048)
    assert contracts.supports_native_shape(2, 4096, 2048) and contracts.supports_native_shape(8, 28672, 8192)
    assert not contracts.supports_native_shape(33, 4096, 2048)
    assert not contracts.supports_native_shape(1, 4100, 2048)
    contracts.validate_public_device_scope({"dim": 2560}, (10, 0))
    with pytest.raises(ValueError):
        contracts.validate_public_device_scope({"dim": 2560}, (9, 0))
    with pytest.raises(ValueError, match="rabv_margin=0"):
        contracts.validate_verification_options(0.5)
    with pytest.raises(ValueError):
        contracts.validate_graph_roles(("ar", "verify_fp8"))


def _write_tiny_ckpt(tmp_path, public_geometry=False):
    geometry = synthetic.BONSAI_1P7B if public_geometry else synthetic.TINY
    cfg = synthetic.make_config(dict(geometry, n_layers=1 if public_geometry else 2))
    ck = tmp_path / "ckpt"
    ck.mkdir()
    (ck / "bonsai_gpu_config.json").write_text(json.dumps(cfg))
    (ck / "model_state_t2g128.pt").write_bytes(b"")
    tok = tmp_path / "tok"
    tok.mkdir()
    (tok / "tokenizer_config.json").write_text("{}")
    (tok / "tokenizer.json").write_text("{}")
    return ck, tok, cfg


def test_check_only_never_imports_torch(tmp_path):
    ck, tok, cfg = _write_tiny_ckpt(tmp_path, public_geometry=True)
    cfg["n_layers"] = 28
    (ck / "bonsai_gpu_config.json").write_text(json.dumps(cfg))
    code = f'''
import builtins, sys
sys.path.insert(0, {ROOT!r})
real = builtins.__import__
def guard(name, *a, **k):
    if name == "torch" or name.startswith("torch.") or name == "transformers":
        raise AssertionError("forbidden import: " + name)
    return real(name, *a, **k)
builtins.__import__ = guard
from bitmtp_b200 import run_generation
run_generation.main(["--ckpt", {str(ck)!r}, "--hf-ckpt", {str(tok)!r}, "--block-size", "8",
                     "--mode", "hybrid", "--prompt", "hi", "--check-only"])
assert "torch" not in sys.modules
'''
    r = subprocess.run([sys.executable, "-B", "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    out = json.loads(r.stdout)
    assert out["gpu_executed"] is False and out["widths"] == [1, 8, 9, 10, 12, 16, 17]
    assert out["roles"] == ["ar", "draft", "verify"] and out["min_chain"] == 6


def test_cli_rejects_bad_options(tmp_path):
    from bitmtp_b200 import run_generation as RG
    ck, tok, _ = _write_tiny_ckpt(tmp_path, public_geometry=True)
    base = ["--ckpt", str(ck), "--hf-ckpt", str(tok), "--block-size", "8", "--prompt", "x", "--check-only"]
    for extra in (["--mode", "ar", "--min-chain", "3"], ["--mode", "hybrid", "--margin", "0.5"],
                  ["--mode", "conf", "--exact-m1-verify"], ["--mode", "ar", "--draft-precision", "fp8"],
                  ["--mode", "hybrid", "--threshold", "1.5"]):
        with pytest.raises(SystemExit):
            RG.main(base + extra)


def tiny_hf_checkpoint(tmp_path):
    """A tiny HF-style (Qwen3 naming) bf16 safetensors checkpoint of the TINY geometry; returns its directory."""
    from safetensors.torch import save_file
    g = synthetic.TINY
    hf = {"hidden_size": g["dim"], "num_hidden_layers": g["n_layers"], "num_attention_heads": g["n_heads"],
          "num_key_value_heads": g["n_kv_heads"], "head_dim": 128, "intermediate_size": g["ffn_dim"],
          "vocab_size": g["vocab_size"], "rms_norm_eps": 1e-6, "rope_theta": 1e6,
          "rope_scaling": {"original_max_position_embeddings": 8192, "factor": 4.0},
          "tie_word_embeddings": True, "block_size": 8, "causal_attn": True,
          "text_mask_token_id": g["vocab_size"] - 1}
    src = tmp_path / "hf"
    src.mkdir()
    (src / "config.json").write_text(json.dumps(hf))
    gen = torch.Generator().manual_seed(0)
    dim, ffn, qd, kd = g["dim"], g["ffn_dim"], g["n_heads"] * 128, g["n_kv_heads"] * 128
    t = {"model.embed_tokens.weight": torch.randn(g["vocab_size"], dim, generator=gen),
         "model.norm.weight": torch.ones(dim), "lm_head.weight": torch.zeros(g["vocab_size"], dim)}
    for i in range(g["n_layers"]):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = torch.ones(dim)
        t[p + "post_attention_layernorm.weight"] = torch.ones(dim)
        t[p + "self_attn.q_norm.weight"] = torch.ones(128)
        t[p + "self_attn.k_norm.weight"] = torch.ones(128)
        for n, (o, k) in {"self_attn.q_proj": (qd, dim), "self_attn.k_proj": (kd, dim),
                          "self_attn.v_proj": (kd, dim), "self_attn.o_proj": (dim, qd),
                          "mlp.gate_proj": (ffn, dim), "mlp.up_proj": (ffn, dim),
                          "mlp.down_proj": (dim, ffn)}.items():
            t[p + n + ".weight"] = torch.randn(o, k, generator=gen) * 0.02
    save_file({k: v.to(torch.bfloat16) for k, v in t.items()}, str(src / "model.safetensors"))
    return src


def test_converter_layout(tmp_path):
    """A tiny HF-style checkpoint through convert(): key names, dtypes and shapes of the
    reference's packed layout (tests/test_bonsai_converter.py:184-196), and a state dict the
    loader accepts."""
    from bitmtp_b200 import convert_bonsai_mtp_to_gpu as CV, generate
    g = synthetic.TINY
    dim, ffn, qd = g["dim"], g["ffn_dim"], g["n_heads"] * 128
    src = tiny_hf_checkpoint(tmp_path)
    out = tmp_path / "out"
    CV.convert(str(src), str(out))
    with pytest.raises(ValueError, match="already exists"):
        CV.convert(str(src), str(out))
    cfg = json.loads((out / "bonsai_gpu_config.json").read_text())
    assert cfg["kernel_kind"] == "t2g128" and cfg["dim"] == dim and cfg["mask_token_id"] == g["vocab_size"] - 1
    sd = torch.load(out / "model_state_t2g128.pt")
    w = sd["layers.0.attention.q_proj.weight"]
    ws = sd["layers.0.attention.q_proj.weight_scale"]
    assert w.dtype == torch.int8 and tuple(w.shape) == (qd, dim // 4)
    assert ws.dtype == torch.bfloat16 and tuple(ws.shape) == (qd, dim // 128)
    assert sd["embed_tokens.weight"].dtype == torch.bfloat16 and "lm_head.weight" not in sd
    # every code is 1, 2 or 3 and the unpacked grid equals the frozen bf16 dump
    codes = torch.stack([(w.view(torch.uint8) >> (2 * i)) & 3 for i in range(4)], -1).view(qd, dim)
    assert int(codes.min()) >= 1
    dense = torch.load(out / "model_state_fp16.pt")["layers.0.attention.q_proj.weight"]
    rebuilt = ((codes.float() - 2).view(qd, dim // 128, 128) * ws.float().unsqueeze(-1)).view(qd, dim)
    assert torch.equal(rebuilt.to(torch.bfloat16), dense)
    cfg["mask_token_id"] = 5
    m = generate.model_from_state(generate.args_from_config(cfg), sd, "cpu")
    assert m.layers[1].feed_forward.down_proj.weight.shape == (dim, ffn // 4)


def test_safetensors_copy_loads_to_the_same_state(tmp_path):
    """--safetensors writes the packed state a second time under the same names; build_model prefers it and
    gets the tensors torch.load gives."""
    from bitmtp_b200 import convert_bonsai_mtp_to_gpu as CV, generate
    src = tiny_hf_checkpoint(tmp_path)
    out = tmp_path / "out"
    CV.convert(str(src), str(out), pack_fp16=False, safetensors_copy=True)   # what `--no-fp16 --safetensors` passes
    ns = CV.make_parser().parse_args(["--src", "a", "--out", "b", "--safetensors", "--device", "cuda:0"])
    assert ns.safetensors and ns.device == "cuda:0"
    assert CV.make_parser().parse_args(["--src", "a", "--out", "b"]).device == "cpu"
    assert (out / "model_state_t2g128.safetensors").is_file() and not (out / "model_state_fp16.pt").exists()
    pt = torch.load(out / "model_state_t2g128.pt")
    st = generate.load_packed_state(str(out), "cpu")
    assert sorted(pt) == sorted(st)
    for k in pt:
        assert st[k].dtype == pt[k].dtype and torch.equal(st[k], pt[k]), k
    m = generate.build_model(str(out), use_kernel=True, device="cpu")
    assert torch.equal(m.layers[0].attention.q_proj.weight.data, pt["layers.0.attention.q_proj.weight"])
    (out / "model_state_t2g128.safetensors").unlink()
    again = generate.load_packed_state(str(out), "cpu")
    assert torch.equal(again["norm.weight"], pt["norm.weight"])
