"""Helpers for driving the reference's own C++ host (its pybind `redline` module, built by
`make -C oracle gpuref` over this library's kernels or over the reference's own) from the tests.

* `write_model_dir` saves a random-init model as the checkpoint directory the reference's loader
  accepts: `config.json` / `generation_config.json` with the constants src/core/config.cpp:255-355
  validates and one `model.safetensors` with the 338 tensors of docs/MODEL_SPEC.md:182-199 (F16, which
  src/loader/weights.cpp:80 accepts beside BF16), un-fusing this library's qkv and gate|up matrices.
* `run_host` runs one of the two builds in a child process (both modules are called `redline` and
  register the same C++ types, so they cannot share an interpreter) and returns what it printed.
"""
from __future__ import annotations

import json
import os
import struct
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

CONFIG_JSON = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 1536, "num_hidden_layers": 28,
    "num_attention_heads": 12, "num_key_value_heads": 2, "intermediate_size": 8960, "vocab_size": 151936,
    "max_position_embeddings": 32768, "rope_theta": 1000000.0, "rms_norm_eps": 1e-06,
    "tie_word_embeddings": True, "torch_dtype": "bfloat16", "hidden_act": "silu", "use_sliding_window": False,
    "bos_token_id": 151643, "eos_token_id": 151645,
}
GENERATION_CONFIG_JSON = {"eos_token_id": [151645, 151643]}


def _tensors(cfg, w):
    """(name, 2-byte-element torch tensor) in the order the file stores them."""
    qw, kw = cfg.q_width, cfg.kv_width
    yield "model.embed_tokens.weight", w.embed
    for i, L in enumerate(w.layers):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", L["in_norm"]
        yield p + "self_attn.q_proj.weight", L["qkv"][:qw]
        yield p + "self_attn.q_proj.bias", L["qkv_bias"][:qw]
        yield p + "self_attn.k_proj.weight", L["qkv"][qw:qw + kw]
        yield p + "self_attn.k_proj.bias", L["qkv_bias"][qw:qw + kw]
        yield p + "self_attn.v_proj.weight", L["qkv"][qw + kw:]
        yield p + "self_attn.v_proj.bias", L["qkv_bias"][qw + kw:]
        yield p + "self_attn.o_proj.weight", L["o"]
        yield p + "post_attention_layernorm.weight", L["post_norm"]
        yield p + "mlp.gate_proj.weight", L["gate_up"][:cfg.inter]
        yield p + "mlp.up_proj.weight", L["gate_up"][cfg.inter:]
        yield p + "mlp.down_proj.weight", L["down"]
    yield "model.norm.weight", w.final_norm


def write_model_dir(path: str, cfg, weights) -> str:
    """Writes the checkpoint directory; returns `path`."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(CONFIG_JSON, f)
    with open(os.path.join(path, "generation_config.json"), "w") as f:
        json.dump(GENERATION_CONFIG_JSON, f)
    header, off = {"__metadata__": {"format": "pt"}}, 0
    items = list(_tensors(cfg, weights))
    for name, t in items:
        n = t.numel() * 2
        header[name] = {"dtype": "F16", "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for _, t in items:
            f.write(t.contiguous().cpu().numpy().view(np.uint16).tobytes())
    return path


def run_host(module_dir: str, model_dir: str, requests, engine_kwargs: dict, timeout: int = 900) -> dict:
    """Runs tests/ref_host_driver.py in a child process against the `redline` module in `module_dir`.
    `requests` = [{"prompt": [...], "max_new_tokens": n, "forced_tokens": [...] | None}, ...]."""
    job = {"module_dir": module_dir, "model_dir": model_dir, "requests": requests, "engine": engine_kwargs}
    r = subprocess.run([sys.executable, os.path.join(HERE, "ref_host_driver.py")], input=json.dumps(job),
                       capture_output=True, text=True, timeout=timeout)
    if r.returncode != 0:
        raise RuntimeError(f"reference host ({module_dir}) exited {r.returncode}:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}")
    return json.loads(r.stdout.strip().splitlines()[-1])
