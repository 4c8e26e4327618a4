"""The Rezusun decoder as a model description.

Layers of three kinds of mixer (attention over a cached latent, and two members of the
delta-rule family that carry a matrix state per head), each sublayer between a layer norm in
front and a layer norm with a per-channel scale behind, some layers with a gated dense
feed-forward; a run of layers may be repeated with the same weights, each pass keeping a
cache or state of its own.  config.json names the layers one by one; the ranks of the
low-rank branches are the shapes of their tensors.
"""

from __future__ import annotations

import dataclasses
from typing import Mapping, Sequence

from ..config.model_config import ConfigError, RezusunConfig, RezusunLayerConfig
from ..registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# sizes that config.json may leave to the checkpoint: mixer type -> (key, tensor under '<layer>.mix.', axis)
_FROM_SHAPES = {
    "general_delta": (("decay_rank", "w1", 0),),
    "channel_delta": (("decay_rank", "a1", 0), ("gate_rank", "g1", 0)),
    "latent_attention": (),
}


def complete_from_shapes(cfg: RezusunConfig, shapes: Mapping[str, Sequence[int]]) -> RezusunConfig:
    """Fills the sizes that the configuration leaves open from the shapes of the checkpoint's tensors."""
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer = dict(layer.mixer)
        for key, tensor, axis in _FROM_SHAPES[layer.type]:
            name = f"l{i}.mix.{tensor}"
            if mixer.get(key) is None and name in shapes:
                mixer[key] = int(shapes[name][axis])
        layers.append(RezusunLayerConfig(layer.type, mixer, layer.mlp))
    return dataclasses.replace(cfg, layers=tuple(layers))


def _size(mixer: Mapping, key: str, i: int) -> int:
    if mixer.get(key) is None:
        raise ConfigError(f"layer {i}: the mixer's {key!r} is given neither by config.json nor by a tensor's shape")
    return int(mixer[key])


def _mixer(cfg: RezusunConfig, i: int, layer: RezusunLayerConfig) -> PartSpec:
    m, p, W = layer.mixer, f"l{i}.mix.", cfg.width
    if layer.type == "latent_attention":
        rope = PartSpec("rope_interleaved", {"dims": int(m["rot"]["dims"]), "base": float(m["rot"]["base"])})
        return PartSpec("latent_attention", {
            "hidden_size": W, "heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
            "vdim": int(m["vdim"]), "q_rank": int(m["q_rank"]), "kv_rank": int(m["kv_rank"]),
            # the scores' factor; a file that leaves it out gets one over the root of a head's key size
            "scale": float(m["scale"]) if m.get("scale") is not None else (int(m["dim"]) + int(m["rot_dim"])) ** -0.5,
            "eps": cfg.norm_eps, "position": rope,
        }, {"dq": p + "dq", "dq_norm": p + "dq.norm", "uq": p + "uq", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm",
            "uk": p + "uk", "uv": p + "uv", "sink": p + "sink", "o": p + "o"})
    if layer.type == "general_delta":
        return PartSpec("general_delta", {
            "hidden_size": W, "heads": int(m["heads"]), "dim": int(m["dim"]),
            "decay_rank": _size(m, "decay_rank", i), "eps": cfg.norm_eps,
        }, {"r": p + "r", "k": p + "k", "v": p + "v", "g": p + "g", "a": p + "a", "a_bias": p + "a.b",
            "w1": p + "w1", "w2": p + "w2", "w0": p + "w0", "norm": p + "norm", "o": p + "o"})
    return PartSpec("channel_delta", {
        "hidden_size": W, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
        "vdim": int(m["vdim"]), "conv": int(m["conv"]), "decay_rank": _size(m, "decay_rank", i),
        "gate_rank": _size(m, "gate_rank", i), "eps": cfg.norm_eps,
    }, {"q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
        "v_conv": p + "v.conv", "b": p + "b", "A_log": p + "A_log", "norm": p + "norm", "a1": p + "a1",
        "a2": p + "a2", "dt_bias": p + "dt_bias", "g1": p + "g1", "g2": p + "g2", "o": p + "o"})


def build_rezusun_spec(cfg: RezusunConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps

    def norm(name, scale=None):
        if scale is None:
            return PartSpec("layernorm", {"size": W, "eps": eps}, {"weight": name})
        return PartSpec("layernorm", {"size": W, "eps": eps, "scaled": True}, {"weight": name, "scale": scale})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = dict(mixer=_mixer(cfg, i, layer), mixer_norm=norm(p + "norm1"),
                     mixer_post_norm=norm(p + "norm1b", p + "ls1"))
        if layer.mlp is None:
            layers.append(LayerSpec("sandwich_mixer_only", parts))
            continue
        parts.update(
            feed_forward=PartSpec("gated_dense", {"hidden_size": W, "intermediate_size": int(layer.mlp["ff"]),
                                                  "activation": "gelu_tanh", "bias": True},
                                  {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down",
                                   "gate_bias": p + "mlp.gate.b", "up_bias": p + "mlp.up.b",
                                   "down_bias": p + "mlp.down.b"}),
            ff_norm=norm(p + "norm2"), ff_post_norm=norm(p + "norm2b", p + "ls2"))
        layers.append(LayerSpec("sandwich", parts))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W}, {"table": "embed"}),
        layers=layers,
        # every pass of a repeated layer keeps a cache or state of its own
        schedule=[ScheduleEntry(i) for i in cfg.layer_order()],
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W}, {"weight": "head"}),
        eos_token_ids=cfg.eos_token_ids,
    )
    spec.validate()
    return spec


register_architecture("Rezusun", RezusunConfig.from_dict, build_rezusun_spec, complete=complete_from_shapes)
