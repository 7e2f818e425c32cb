"""Limazen as a list of layers: every layer is a parallel block (one LayerNorm with weight and bias;
the mixer and the feed-forward both read its output and their outputs join the stream together) of
grouped-query attention (biases on q, k, v; a rotation of the first channels of a head with linearly
scaled frequencies; a chunked mask; values blended with the first blending layer's; a sigmoid gate per
channel) and a feed-forward that is dense (down(relu(up x)^2)), a mixture of gated experts with a
sigmoid router and a gated shared expert, or absent. The model's final norm is a LayerNorm too, and the
logits pass a soft cap. The residual stream is 32-bit in either precision. Tensor names are the
checkpoint's own: `embed`, `l<i>.norm1(.b)`, `l<i>.mix.{q,k,v}(.b)`, `l<i>.mix.{vmix,g,o}`,
`l<i>.mlp.{up,down}`, `l<i>.mlp.router`, `l<i>.mlp.e<j>.{gate,up,down}`,
`l<i>.mlp.shared.{gate,up,down,sg}`, `final.norm(.b)`, `head`."""

from __future__ import annotations

from ..config.base import register_architecture
from ..config.limazen import LimazenConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec

# the rotation's angles are 32-bit products of position and frequency; the cache bounds a request's length
UNBOUNDED_POSITIONS = 1 << 30


def limazen_spec(cfg: LimazenConfig) -> ModelSpec:
    def norm(weight: str) -> PartSpec:
        return PartSpec("layernorm", {"dim": cfg.width, "eps": cfg.norm_eps, "weight": weight, "bias": weight + ".b"})

    layers, ignorable, keeps = [], set(), None
    for index, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        rot = m["rot"]
        blend = None
        if m.get("v_mix"):
            blend = "keep" if keeps is None else "blend"
            keeps = index if keeps is None else keeps
        if blend != "blend":
            ignorable.add(f"l{index}.mix.vmix")      # stored for every blending layer, unused where nothing is blended
        mixer = PartSpec("attention", {
            "hidden": cfg.width, "q_heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "scale": float(m["scale"]), "chunk": int(m["mask"]["size"]),
            "position": PartSpec("rotary_half", {"dim": m["dim"], "theta": float(rot["base"]), "rotated": int(rot["dims"]),
                                                 "linear_factor": float((rot.get("scaling") or {}).get("factor", 1.0))}),
            "q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o",
            "q_bias": "mix.q.b", "k_bias": "mix.k.b", "v_bias": "mix.v.b",
            "gate": "mix.g", "gate_kind": "channel",
            "value_blend": blend, "value_blend_weight": "mix.vmix"})
        mlp = layer.get("mlp")
        if mlp is None:
            feed_forward = None
        elif mlp["kind"] == "dense":
            feed_forward = PartSpec("mlp", {"hidden": cfg.width, "inter": mlp["ff"], "activation": "relu2",
                                            "up": "mlp.up", "down": "mlp.down"})
        else:
            shared = mlp.get("shared")
            feed_forward = PartSpec("routed_experts", {
                "hidden": cfg.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "inter": mlp["expert"]["ff"], "activation": "silu", "score": "sigmoid", "weight_on": "input",
                "router": "mlp.router", "expert_gate": "mlp.e{}.gate", "expert_up": "mlp.e{}.up", "expert_down": "mlp.e{}.down",
                "shared": PartSpec("gated_mlp", {"hidden": cfg.width, "inter": shared["ff"], "activation": "silu",
                                                 "gate": "mlp.shared.gate", "up": "mlp.shared.up",
                                                 "down": "mlp.shared.down"}) if shared else None,
                "shared_gate": "mlp.shared.sg" if shared else None})
        block = PartSpec("parallel", {"input_norm": norm("norm1"), "mixer": mixer, "feed_forward": feed_forward})
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
        residual_dtype="float32",
        logit_softcap=cfg.logit_softcap,
        ignorable_tensors=frozenset(ignorable),
    )


register_architecture(LimazenConfig.architecture, LimazenConfig.model_type, LimazenConfig, limazen_spec)
