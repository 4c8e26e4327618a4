"""Small Solulix configurations and weights for the tests: sizes that differ from one another
wherever the design allows it (query against key/value heads, key against value size, taps,
windows that are no multiple of a page, experts with and without identity or shared ones), and
weights drawn here."""

import json
import os

import numpy as np
import torch


def attention(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, scale=0.3, size=11, keep_first=3, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale,
                      "mask": {"size": size, "keep_first": keep_first}}}


def delta(heads=4, kv_heads=2, dim=12, vdim=20, conv=4, mlp=None):
    return {"type": "delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=1, top=2, scale=1.5, ff=12, shared=20):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(layers, width=48, vocab=101, loop=None, eps=1e-5):
    cfg = {"architecture": "Solulix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = loop
    return cfg


# every kind of layer and feed-forward, a layer without feed-forward, a repeated run of three layers that starts
# behind the first layer; windows of 11 and 20 tokens on pages of 8
MIXED = config([delta(mlp=dense(56)), attention(mlp=moe()), delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=2),
                attention(heads=3, kv_heads=3, dim=8, vdim=8, conv=1, scale=0.5, size=20, keep_first=0, mlp=dense(24)),
                attention(heads=6, kv_heads=1, dim=24, vdim=8, conv=4, scale=0.2, size=5, keep_first=9,
                          mlp=moe(experts=3, identity=2, top=3, scale=0.7, ff=16, shared=0))],
               loop={"start": 1, "stop": 4, "times": 2})


def expected(cfg):
    from kv_cache_optimization_for_llm_b200.models.spec import expected_weights
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    return expected_weights(arch.build_spec(arch.parse_config(cfg)))


def draw_weights(cfg, seed, gain=1.0):
    """Every tensor the model expects, drawn here and rounded to bfloat16 so that both precisions load
    the same numbers: matrices N(0, gain / sqrt(fan-in)), norm weights about 1, taps and small vectors about 0,
    routers wide enough that the chosen experts change from token to token."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, ws in sorted(expected(cfg).items()):
        if ws.kind == "vector":
            t = 1.0 + 0.2 * rng.normal(size=ws.shape)
        elif name.endswith(".conv"):
            t = rng.normal(size=ws.shape) * 0.7
        elif name.endswith(".router"):
            t = rng.normal(size=ws.shape) * (3.0 / np.sqrt(ws.shape[-1]))
        elif name.endswith(".correction"):
            t = rng.normal(size=ws.shape) * 0.1
        elif name == "loop.step":
            t = rng.normal(size=ws.shape) * 0.5
        elif ws.kind == "bias":
            t = 0.5 * rng.normal(size=ws.shape)
        else:
            t = rng.normal(size=ws.shape) * (gain / np.sqrt(ws.shape[-1]))
        out[name] = torch.as_tensor(t, dtype=torch.float32).to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, gain=1.0, weights=None):
    from kv_cache_optimization_for_llm_b200.weights.safetensors_io import write_tensors
    os.makedirs(folder, exist_ok=True)
    tensors = weights if weights is not None else draw_weights(cfg, seed, gain)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_tensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return {k: v.float().numpy().astype(np.float64) for k, v in tensors.items()}
