"""The Solulix decoder as a model description.

A token's embedding passes an RMS norm before it starts the residual stream.  Every layer has
one RMS norm whose output both its mixer and its feed-forward read; their outputs join the stream
together.  Mixers are of two kinds: attention without positions over queries, keys and values
that pass a short convolution, with a sliding window that keeps the first tokens and a softmax
whose denominator counts one more; and a gated delta rule with a matrix state per head.  The
feed-forward is a gated dense one or a set of small experts chosen per token.  A run of layers
may be repeated with the same weights, each pass keeping a cache or state of its own; every pass
starts by adding a learned vector to the stream, and every pass but the first the embedding's
output as well.  config.json names the layers one by one.
"""

from __future__ import annotations

from ..config.model_config import SolulixConfig, SolulixLayerConfig
from ..registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(cfg: SolulixConfig, i: int, layer: SolulixLayerConfig) -> PartSpec:
    m, p, W = layer.mixer, f"l{i}.mix.", cfg.width
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
             "v_conv": p + "v.conv", "o": p + "o"}
    if layer.type == "attention":
        return PartSpec("conv_window_attention", {
            "hidden_size": W, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
            "vdim": int(m["vdim"]), "conv": int(m["conv"]), "scale": float(m["scale"]),
            "window": int(m["mask"]["size"]), "keep_first": int(m["mask"]["keep_first"]), "one_more": True,
        }, names)
    names.update(b=p + "b", a=p + "a", A_log=p + "A_log", dt_bias=p + "dt_bias", norm=p + "norm", g=p + "g")
    return PartSpec("gated_delta", {
        "hidden_size": W, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
        "vdim": int(m["vdim"]), "conv": int(m["conv"]), "eps": cfg.norm_eps,
    }, names)


def _feed_forward(cfg: SolulixConfig, i: int, mlp) -> PartSpec:
    p, W = f"l{i}.mlp.", cfg.width
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", {"hidden_size": W, "intermediate_size": int(mlp["ff"])},
                        {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    router = mlp["router"]
    E = int(router["experts"])
    shared = int(mlp["shared"]["ff"]) if mlp.get("shared") else 0
    names = {"router": p + "router", "correction": p + "correction"}
    for e in range(E):
        names[f"up{e}"] = f"{p}e{e}.up"
        names[f"down{e}"] = f"{p}e{e}.down"
    if shared:
        names.update(shared_up=p + "shared.up", shared_down=p + "shared.down")
    return PartSpec("routed_experts", {
        "hidden_size": W, "experts": E, "identity": int(router["identity"]), "top": int(router["top"]),
        "scale": float(router["scale"]), "expert_ff": int(mlp["expert"]["ff"]), "shared_ff": shared,
    }, names)


def build_solulix_spec(cfg: SolulixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps

    def norm(name):
        return PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = dict(mixer=_mixer(cfg, i, layer), norm=norm(f"l{i}.norm1"))
        if layer.mlp is None:
            layers.append(LayerSpec("parallel_mixer_only", parts))
        else:
            parts["feed_forward"] = _feed_forward(cfg, i, layer.mlp)
            layers.append(LayerSpec("parallel", parts))
    times = cfg.loop[2] if cfg.loop is not None else 0
    schedule = []
    for i, pass_no in cfg.passes():
        before = None
        if pass_no is not None:
            before = PartSpec("pass_start", {"size": W, "passes": times, "index": pass_no, "add_embedding": pass_no > 0},
                              {"steps": "loop.step"})
        # every pass of a repeated layer keeps a cache or state of its own
        schedule.append(ScheduleEntry(i, before=before))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("normed_token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "eps": eps},
                           {"table": "embed", "norm": "embed.norm"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W}, {"weight": "head"}),
        eos_token_ids=cfg.eos_token_ids,
    )
    spec.validate()
    return spec


register_architecture("Solulix", SolulixConfig.from_dict, build_solulix_spec)
