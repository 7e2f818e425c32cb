"""Typed configuration of Limazen, read from its own config.json keys.

Limazen is a decoder whose layers are listed one by one. Every layer is a parallel block: one
LayerNorm (weight and bias) whose output both the mixer and the feed-forward read, and both outputs
are added to the stream together. The one mixer (`type`: "attention") is grouped-query softmax
attention with biases on q, k and v, a rotation of the first `rot.dims` channels of a head (rotate-half
pairing, base `rot.base`, every frequency divided by `rot.scaling.factor`), a scale of its own, a
chunked mask (`mask.size`: a query sees earlier keys of its own chunk of positions only), values
blended with the first blending layer's values (`v_mix`), and a sigmoid gate per channel before the
output product. The feed-forward (`mlp`) is `{"kind": "dense", "ff": N}` (down(relu(up x)^2)),
`{"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared": {"ff"} or absent}` (sigmoid
router, the chosen scores scale the experts' inputs, a gated shared expert), or null. Other keys:
`vocab`, `width`, `norm.eps`, `logit_softcap`. Nothing else is read, and nothing that these keys give
stands anywhere in code.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

MIXER_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot")


def _positive_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool) and value > 0


@dataclass(frozen=True)
class LimazenConfig:
    vocab: int
    width: int
    layers: tuple            # of dicts {"type", "mixer", "mlp"}, as config.json lists them
    norm_eps: float = 1e-5
    logit_softcap: float | None = None
    eos_token_id: int | None = field(default=None, compare=False)

    architecture = "Limazen"
    model_type = "limazen"

    def __post_init__(self):
        for name in ("vocab", "width"):
            if not _positive_int(getattr(self, name)):
                raise ValueError(f"{name} must be a positive integer, got {getattr(self, name)!r}")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ValueError("logit_softcap must be positive (or absent)")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        blended = None
        for index, layer in enumerate(self.layers):
            if layer.get("type") != "attention":
                raise ValueError(f"layer {index}: unknown type {layer.get('type')!r}; known: ['attention']")
            mixer = layer.get("mixer") or {}
            missing = [k for k in MIXER_KEYS if k not in mixer]
            if missing:
                raise ValueError(f"layer {index}: mixer lacks {missing}")
            for k in ("heads", "kv_heads", "dim", "vdim"):
                if not _positive_int(mixer[k]):
                    raise ValueError(f"layer {index}: mixer.{k} must be a positive integer, got {mixer[k]!r}")
            if mixer["heads"] % mixer["kv_heads"]:
                raise ValueError(f"layer {index}: heads ({mixer['heads']}) must be a multiple of kv_heads ({mixer['kv_heads']})")
            if not _positive_int((mixer["mask"] or {}).get("size")):
                raise ValueError(f"layer {index}: mask.size must be a positive integer")
            rot = mixer["rot"] or {}
            if not _positive_int(rot.get("dims")) or rot["dims"] % 2 or rot["dims"] > mixer["dim"] or not float(rot.get("base", 0)) > 0:
                raise ValueError(f"layer {index}: rot needs an even dims <= dim and a positive base, got {rot!r}")
            if not float((rot.get("scaling") or {}).get("factor", 1.0)) > 0:
                raise ValueError(f"layer {index}: rot.scaling.factor must be positive")
            if mixer.get("v_mix"):
                shape = (mixer["kv_heads"], mixer["vdim"])
                if blended is not None and shape != blended:
                    raise ValueError(f"layer {index}: layers that blend values must have the same kv_heads and vdim")
                blended = shape
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                if not _positive_int(mlp.get("ff")):
                    raise ValueError(f"layer {index}: mlp.ff must be a positive integer")
            elif mlp.get("kind") == "moe":
                router, expert, shared = mlp.get("router") or {}, mlp.get("expert") or {}, mlp.get("shared")
                if not _positive_int(router.get("experts")) or not _positive_int(router.get("top")) or router["top"] > router["experts"]:
                    raise ValueError(f"layer {index}: mlp.router needs experts and 1 <= top <= experts, got {router!r}")
                if not _positive_int(expert.get("ff")) or (shared is not None and not _positive_int(shared.get("ff"))):
                    raise ValueError(f"layer {index}: mlp.expert.ff (and mlp.shared.ff) must be positive integers")
            else:
                raise ValueError(f"layer {index}: unknown mlp kind {mlp.get('kind')!r}; known: ['dense', 'moe']")

    @classmethod
    def from_hf_dict(cls, raw: dict) -> "LimazenConfig":
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks {missing}")
        eos = raw.get("eos_token_id")
        cap = raw.get("logit_softcap")
        return cls(
            vocab=raw["vocab"], width=raw["width"],
            layers=tuple(copy.deepcopy(layer) for layer in raw["layers"]),
            norm_eps=float((raw.get("norm") or {}).get("eps", 1e-5)),
            logit_softcap=None if cap is None else float(cap),
            eos_token_id=eos[0] if isinstance(eos, list) else eos,
        )

    def to_hf_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        out = {
            "architecture": self.architecture,
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out


def limazen_layer(heads, kv_heads, dim, vdim, chunk, rot_dims=None, base=10000.0, factor=1.0, scale=None, v_mix=True,
                  ff=None, experts=None, top=1, expert_ff=None, shared_ff=None) -> dict:
    """One entry of `layers`: `ff` gives a dense feed-forward, `experts` a routed one, neither none."""
    if experts:
        mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}}
        if shared_ff:
            mlp["shared"] = {"ff": shared_ff}
    else:
        mlp = {"kind": "dense", "ff": ff} if ff else None
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                      "rot": {"base": base, "dims": rot_dims or dim, "scaling": {"factor": factor}},
                      "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix}}


# Named shapes for the command line and the benchmark (inputs, like a parsed config.json).
LIMAZEN_PRESETS: dict[str, dict] = {
    "limazen-tiny": dict(
        vocab=384, width=128, norm_eps=1e-5, logit_softcap=20.0,
        layers=(limazen_layer(4, 2, 32, 16, 40, rot_dims=16, factor=2.0, ff=192),
                limazen_layer(4, 2, 32, 16, 40, rot_dims=16, factor=2.0, experts=6, top=2, expert_ff=48, shared_ff=80),
                limazen_layer(2, 1, 16, 32, 24, v_mix=False, experts=4, top=1, expert_ff=64))),
}
