"""Topidra as a list of layers: every layer is a block with a norm before and after each sub-layer
around one of two mixers (softmax attention over a sliding window, with a whole-row RMSNorm of q
and k, a sink per head, a sigmoid gate per head and no rotation; or linear attention with a
constant decay per head and a gated RMSNorm), and a relu-gated feed-forward or none. A span of
layers may run several times in a row with the same weights; each pass has a cache or state of its
own, and the embedding output is added to the stream before every pass but the first. The residual
stream is 32-bit in either precision. Tensor names are the checkpoint's own: `embed`,
`l<i>.norm1 / norm1b / norm2 / norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`."""

from __future__ import annotations

from ..config.base import register_architecture
from ..config.topidra import TopidraConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

# no position ever enters a score or a state, so a request may be as long as the cache allows
UNBOUNDED_POSITIONS = 1 << 30


def topidra_spec(cfg: TopidraConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": cfg.width, "eps": cfg.norm_eps, "weight": weight})

    layers = []
    for index, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixer = PartSpec("attention", {
                "hidden": cfg.width, "q_heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "scale": float(m["scale"]), "window": int(m["mask"]["size"]),
                "qk_norm": "whole", "qk_norm_eps": cfg.norm_eps, "position": None,
                "q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm",
                "sink": "mix.sink", "gate": "mix.g"})
        else:
            mixer = PartSpec("decay_linear_attention", {
                "hidden": cfg.width, "heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
                "decay": m["decay"], "norm_eps": cfg.norm_eps, "activation": "silu",
                "q": "mix.q", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "o": "mix.o", "norm": "mix.norm"})
        mlp = layer.get("mlp")
        block = PartSpec("sandwich_norm", {
            "input_norm": norm("norm1"), "mixer": mixer, "mixer_out_norm": norm("norm1b"),
            "post_norm": norm("norm2") if mlp else None,
            "feed_forward": PartSpec("gated_mlp", {"hidden": cfg.width, "inter": mlp["ff"], "activation": "relu",
                                                   "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}) if mlp else None,
            "ff_out_norm": norm("norm2b") if mlp else None,
        })
        layers.append(LayerSpec(block, f"l{index}."))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_position=UNBOUNDED_POSITIONS,
        embedding="embed",
        final_norm=norm("final.norm"),
        head="head",
        layers=layers,
        schedule=[ScheduleEntry(layer, adds_embedding=adds) for layer, adds in cfg.layer_runs()],
        residual_dtype="float32",
    )


register_architecture(TopidraConfig.architecture, TopidraConfig.model_type, TopidraConfig, topidra_spec)
