"""Typed configuration of Topidra, read from its own config.json keys.

Topidra is a decoder whose layers are listed one by one: each entry of `layers` names its mixer
(`type`: "attention", softmax attention over a sliding window with a sink per head, or
"lightning", linear attention with a constant decay per head), the mixer's sizes and constants
(`mixer`) and its feed-forward (`mlp`: `{"kind": "dense", "ff": N}`, or null for a layer without
one). `loop` = `{start, stop, times}` runs layers start .. stop-1 `times` times in a row with the
same weights. Other keys: `vocab`, `width`, `norm.eps`. Nothing else is read, and nothing that
these keys give stands anywhere in code.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "mask"),
    "lightning": ("heads", "dim", "vdim", "decay"),
}


@dataclass(frozen=True)
class TopidraConfig:
    vocab: int
    width: int
    layers: tuple            # of dicts {"type", "mixer", "mlp"}, as config.json lists them
    norm_eps: float = 1e-6
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_id: int | None = field(default=None, compare=False)

    architecture = "Topidra"
    model_type = "topidra"

    def __post_init__(self):
        for name in ("vocab", "width"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ValueError(f"{name} must be a positive integer, got {value!r}")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        for index, layer in enumerate(self.layers):
            kind = layer.get("type")
            if kind not in MIXER_KEYS:
                raise ValueError(f"layer {index}: unknown type {kind!r}; known: {sorted(MIXER_KEYS)}")
            mixer = layer.get("mixer") or {}
            missing = [k for k in MIXER_KEYS[kind] if k not in mixer]
            if missing:
                raise ValueError(f"layer {index} ({kind}): mixer lacks {missing}")
            for k in ("heads", "dim", "vdim"):
                if not isinstance(mixer[k], int) or mixer[k] <= 0:
                    raise ValueError(f"layer {index}: mixer.{k} must be a positive integer, got {mixer[k]!r}")
            if kind == "attention":
                if not isinstance(mixer["kv_heads"], int) or mixer["kv_heads"] <= 0 or mixer["heads"] % mixer["kv_heads"]:
                    raise ValueError(f"layer {index}: heads ({mixer['heads']}) must be a multiple of kv_heads "
                                     f"({mixer['kv_heads']})")
                size = (mixer["mask"] or {}).get("size")
                if not isinstance(size, int) or size <= 0:
                    raise ValueError(f"layer {index}: mask.size must be a positive integer, got {size!r}")
            else:
                decay = mixer["decay"]
                values = decay if isinstance(decay, (list, tuple)) else [decay] * mixer["heads"]
                if len(values) != mixer["heads"] or not all(0.0 <= float(d) <= 1.0 for d in values):
                    raise ValueError(f"layer {index}: decay must be one number in [0, 1], or one per head")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ValueError(f"layer {index}: unknown mlp kind {mlp.get('kind')!r}; known: ['dense']")
                if not isinstance(mlp.get("ff"), int) or mlp["ff"] <= 0:
                    raise ValueError(f"layer {index}: mlp.ff must be a positive integer")
        if not (0 <= self.loop_start <= self.loop_stop <= len(self.layers)) or self.loop_times < 1:
            raise ValueError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit "
                             f"{len(self.layers)} layers")

    @classmethod
    def from_hf_dict(cls, raw: dict) -> "TopidraConfig":
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks {missing}")
        loop = raw.get("loop") or {}
        eos = raw.get("eos_token_id")
        return cls(
            vocab=raw["vocab"], width=raw["width"],
            layers=tuple(copy.deepcopy(layer) for layer in raw["layers"]),
            norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
            loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)),
            eos_token_id=eos[0] if isinstance(eos, list) else eos,
        )

    def to_hf_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        return {
            "architecture": self.architecture,
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }

    def layer_runs(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding output is added to the stream right before it) in running
        order: the looped layers `loop_times` times in a row, the embedding output before every pass
        but the first."""
        runs = [(i, False) for i in range(self.loop_start)]
        for lap in range(self.loop_times):
            runs += [(i, lap > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, False) for i in range(self.loop_stop, len(self.layers))]


def _attention(heads, kv_heads, dim, vdim, window, scale=None, ff=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": window}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _spread(heads: int, low: float, high: float) -> list[float]:
    return [low + (high - low) * h / max(1, heads - 1) for h in range(heads)]


# Named shapes for the command line and the benchmark (inputs, like a parsed config.json).
# "topidra-4b-like" has the widths of the benchmark's Qwen3-4B shape, layer for layer.
TOPIDRA_PRESETS: dict[str, dict] = {
    "topidra-tiny": dict(
        vocab=320, width=96, norm_eps=1e-5, loop_start=0, loop_stop=2, loop_times=2,
        layers=(_lightning(3, 16, 32, [0.7, 0.9, 0.99]), _attention(4, 2, 32, 16, 24, 0.2, ff=160),
                _attention(2, 1, 16, 48, 9, ff=None))),
    "topidra-4b-like": dict(
        vocab=151936, width=2560, norm_eps=1e-6, loop_start=0, loop_stop=0, loop_times=1,
        layers=tuple(_lightning(32, 128, 128, _spread(32, 0.9, 0.999), ff=9728) if i % 4 != 3
                     else _attention(32, 8, 128, 128, 4096, ff=9728) for i in range(36))),
}
