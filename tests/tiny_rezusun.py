"""Small Rezusun configurations and weights for the tests: sizes that differ from one
another wherever the design allows it (heads against query/key heads, key against value
size, rotary dimensions against the rotated part, ranks), odd sizes, and weights drawn here."""

import json
import os

import numpy as np
import torch


def latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=20, kv_rank=16, rot_dims=None, base=10000.0, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": float((dim + rot_dim) ** -0.5), "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def general(heads=2, dim=16, rank=6, ff=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def channel(heads=4, kv_heads=2, dim=12, vdim=20, conv=4, rank=5, gate_rank=7, ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                               "conv": conv, "decay_rank": rank, "gate_rank": gate_rank},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, width=48, vocab=101, loop=None, eps=1e-5):
    return {"architecture": "Rezusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
            "loop": loop}


# mixes every kind, a repeated run of two layers, a feed-forward on a delta layer, a layer with one tap; the
# first attention layer's sizes keep it on the plain kernel in bfloat16, the last one's put it on tensor cores
MIXED = config([general(), channel(ff=40), latent(ff=56), channel(heads=2, kv_heads=2, dim=8, vdim=8, conv=1),
                general(heads=3, dim=20, rank=9), latent(heads=2, dim=8, rot_dim=16, vdim=8, q_rank=12, kv_rank=32)],
               loop={"start": 1, "stop": 3, "times": 2})


def expected(cfg):
    from kv_cache_optimization_for_llm_b200.models.spec import expected_weights
    from kv_cache_optimization_for_llm_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    return expected_weights(arch.build_spec(arch.parse_config(cfg)))


def draw_weights(cfg, seed, std=0.25):
    """Every tensor the model expects, drawn here and rounded to bfloat16 so that both precisions
    load the same numbers: matrices N(0, std / sqrt(fan-in) * 4), norm weights and scales about 1,
    the branches' scales about 0.5, small vectors about 0."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, ws in sorted(expected(cfg).items()):
        if ws.kind == "vector":
            t = 1.0 + 0.2 * rng.normal(size=ws.shape)
            if name.endswith((".ls1", ".ls2")):
                t = 0.5 + 0.1 * rng.normal(size=ws.shape)
        elif ws.kind == "bias":
            t = 0.5 * rng.normal(size=ws.shape)
            if name.endswith(".conv"):
                t = rng.normal(size=ws.shape)
        else:
            t = rng.normal(size=ws.shape) * (4.0 * std / np.sqrt(ws.shape[-1]))
        out[name] = torch.as_tensor(t, dtype=torch.float32).to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, std=0.25, weights=None):
    from kv_cache_optimization_for_llm_b200.weights.safetensors_io import write_tensors
    os.makedirs(folder, exist_ok=True)
    tensors = weights if weights is not None else draw_weights(cfg, seed, std)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_tensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return {k: v.float().numpy().astype(np.float64) for k, v in tensors.items()}
