"""Makes tests/golden/tiny_attention.npz from the reference's own fixtures.

    python tests/golden/make_tiny_attention.py /path/to/qubivex

Reads (never copies code from) the reference's tiny SafeTensors models
(fixtures/models/{dense-tiny,olmoe-tiny}) and its transformers-generated golden file
(fixtures/oracle/forward.json: per-layer attention outputs after o_proj for a 14-token prompt,
f32 bit patterns; checked by crates/qubivex-runtime/tests/oracle.rs at 1e-5 relative), and keeps
only what the attention stage needs: the embedding rows of the prompt, each layer's input norm,
Q/K/V/O projections (and OLMoE's full-width q_norm / k_norm), the previous layer's output as the
next layer's input, and the expected attention outputs.  Weights are stored as f32 (the models
are bf16; widening is exact).
"""
import json
import sys
from pathlib import Path

import numpy as np
from safetensors.torch import load_file

if len(sys.argv) != 2:
    sys.exit("usage: python tests/golden/make_tiny_attention.py /path/to/qubivex")
ref = Path(sys.argv[1])
golden = json.loads((ref / "fixtures/oracle/forward.json").read_text())
prompt = np.array(golden["prompt"], dtype=np.int64)
out = {"prompt": prompt}


def f32(bits):
    return np.array(bits, dtype=np.uint32).view(np.float32)


for name in ("dense-tiny", "olmoe-tiny"):
    cfg = json.loads((ref / f"fixtures/models/{name}/config.json").read_text())
    w = {k: v.float().numpy() for k, v in load_file(str(ref / f"fixtures/models/{name}/model.safetensors")).items()}
    hidden = cfg["hidden_size"]
    heads, kvh = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or hidden // heads
    out[f"{name}/meta"] = np.array([hidden, heads, kvh, d, cfg["num_hidden_layers"]], dtype=np.int64)
    out[f"{name}/eps_theta"] = np.array([cfg["rms_norm_eps"], cfg["rope_theta"]], dtype=np.float64)
    out[f"{name}/embed"] = w["model.embed_tokens.weight"][prompt]           # the prompt's rows only
    layers = golden["models"][name]["layers"]
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        out[f"{name}/{l}/input_layernorm"] = w[p + "input_layernorm.weight"]
        for m in ("q", "k", "v", "o"):
            out[f"{name}/{l}/{m}_proj"] = w[p + f"self_attn.{m}_proj.weight"]
        if p + "self_attn.q_norm.weight" in w:
            out[f"{name}/{l}/q_norm"] = w[p + "self_attn.q_norm.weight"]
            out[f"{name}/{l}/k_norm"] = w[p + "self_attn.k_norm.weight"]
        out[f"{name}/{l}/attention"] = f32(layers[l]["attention"]).reshape(len(prompt), hidden)
        out[f"{name}/{l}/hidden"] = f32(layers[l]["hidden"]).reshape(len(prompt), hidden)   # the layer's output

dst = Path(__file__).resolve().parent / "tiny_attention.npz"
np.savez_compressed(dst, **out)
print(dst, dst.stat().st_size, "bytes")
