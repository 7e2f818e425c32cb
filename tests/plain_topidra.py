"""A plain, slow Topidra in float64 torch on the CPU: the oracle of the Topidra tests.

One function per mechanism, written from the design's equations and sharing nothing with the
package: every sequence is taken alone and whole, token by token where the design is a recurrence,
with no cache, no pages and no batching. `forward` returns the logits of every position and the
residual stream after every layer run.

Notation: n tokens, W the model width, H query heads, G key/value heads, d the query/key size of a
head, e its value size.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def exact(t: torch.Tensor) -> torch.Tensor:
    return t


def through_bfloat16(t: torch.Tensor) -> torch.Tensor:
    """What a tensor becomes when it is stored in bfloat16. `forward(..., stored=through_bfloat16)` rounds
    what a bfloat16 run keeps in bfloat16 (inputs and outputs of matrix products); the difference to the
    exact run says how much such rounding can move a row of logits at all."""
    return t.to(torch.bfloat16).to(F)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def sink_softmax_attention(q, k, v, sink, scale: float, window: int) -> torch.Tensor:
    """q [n, H, d], k [n, G, d], v [n, G, e], sink [H] -> [n, H, e].

    Query i sees key j when 0 <= i - j < window. The weights are exp(s_ij) / (exp(sink_h) + sum_j
    exp(s_ij)) with s_ij = scale * q_i . k_j: the sink adds to the denominator only."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.zeros(n, heads, v.shape[2], dtype=F)
    for h in range(heads):
        g = h // group
        for i in range(n):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            top = max(s.max().item(), sink[h].item())
            w = torch.exp(s - top)
            out[i, h] = (w[:, None] * v[lo:i + 1, g]).sum(0) / (w.sum() + math.exp(sink[h].item() - top))
    return out


def attention_mixer(h, t: dict, mixer: dict, eps: float, stored=exact) -> torch.Tensor:
    """The softmax mixer: projections, one RMS norm over the whole q row and one over the whole k
    row, windowed attention with a sink, a sigmoid gate per head, the output projection."""
    heads, kv, d, e = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    q = stored(rms_norm(stored(h @ t["q"].T), t["q.norm"], eps)).view(n, heads, d)
    k = stored(rms_norm(stored(h @ t["k"].T), t["k.norm"], eps)).view(n, kv, d)
    v = stored(h @ t["v"].T).view(n, kv, e)
    o = sink_softmax_attention(q, k, v, t["sink"], float(mixer["scale"]), int(mixer["mask"]["size"]))
    gate = torch.sigmoid(stored(h @ t["g"].T))             # [n, H]
    return stored(stored(o * gate[:, :, None]).reshape(n, heads * e) @ t["o"].T)


def decayed_outer_product_scan(q, k, v, decay) -> torch.Tensor:
    """q, k [n, H, d], v [n, H, e], decay [H] -> [n, H, e], token by token:
    S_t = decay_h S_(t-1) + k_t v_t^T (S is d x e and starts at zero), o_t = S_t^T q_t."""
    n, heads, d = q.shape
    out = torch.zeros(n, heads, v.shape[2], dtype=F)
    for h in range(heads):
        state = torch.zeros(d, v.shape[2], dtype=F)
        for i in range(n):
            state = decay[h] * state + torch.outer(k[i, h], v[i, h])
            out[i, h] = state.T @ q[i, h]
    return out


def lightning_mixer(h, t: dict, mixer: dict, eps: float, stored=exact) -> torch.Tensor:
    """The linear mixer: silu on q, k, v, the decayed scan per head, an RMS norm over all heads
    together, a sigmoid gate per channel, the output projection."""
    heads, d, e = mixer["heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    silu = torch.nn.functional.silu
    q, k = silu(stored(h @ t["q"].T)).view(n, heads, d), silu(stored(h @ t["k"].T)).view(n, heads, d)
    v = silu(stored(h @ t["v"].T)).view(n, heads, e)
    decay = mixer["decay"]
    decay = torch.tensor(decay if isinstance(decay, (list, tuple)) else [decay] * heads, dtype=F)
    o = decayed_outer_product_scan(q, k, v, decay).reshape(n, heads * e)
    return stored(stored(rms_norm(o, t["norm"], eps) * torch.sigmoid(stored(h @ t["g"].T))) @ t["o"].T)


def dense_feed_forward(h, t: dict, stored=exact) -> torch.Tensor:
    """down(relu(gate h) * (up h))."""
    return stored(stored(torch.relu(stored(h @ t["gate"].T)) * stored(h @ t["up"].T)) @ t["down"].T)


def sub(tensors: dict, prefix: str) -> dict:
    return {name[len(prefix):]: value for name, value in tensors.items() if name.startswith(prefix)}


def layer(x, index: int, entry: dict, tensors: dict, eps: float, stored=exact) -> torch.Tensor:
    """x + norm1b(mixer(norm1 x)), then, with a feed-forward, x + norm2b(ff(norm2 x))."""
    t = sub(tensors, f"l{index}.")
    mix = {"attention": attention_mixer, "lightning": lightning_mixer}[entry["type"]]
    x = x + rms_norm(mix(stored(rms_norm(x, t["norm1"], eps)), sub(t, "mix."), entry["mixer"], eps, stored), t["norm1b"], eps)
    if entry.get("mlp") is not None:
        x = x + rms_norm(dense_feed_forward(stored(rms_norm(x, t["norm2"], eps)), sub(t, "mlp."), stored), t["norm2b"], eps)
    return x


def layer_runs(config: dict) -> list[tuple[int, bool]]:
    """(layer, whether the embedding output is added before it) in the order the layers run."""
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    count = len(config["layers"])
    runs = [(i, False) for i in range(loop["start"])]
    for lap in range(loop["times"]):
        runs += [(i, lap > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], count)]


def forward(config: dict, tensors: dict, tokens: list[int], stored=exact):
    """(logits [n, vocab], residual stream after every layer run [runs, n, W]) of one whole sequence.
    `stored`: what happens to a tensor that a reduced-precision run keeps in its own type (see
    `through_bfloat16`); the stream, norms, scores, weights and the recurrence are never touched."""
    tensors = {name: (value.to(F) if value.is_floating_point() else value) for name, value in tensors.items()}
    eps = float(config["norm"]["eps"])
    embedded = tensors["embed"][torch.tensor(tokens, dtype=torch.long)]
    x, after = embedded, []
    for index, adds in layer_runs(config):
        if adds:
            x = x + embedded
        x = layer(x, index, config["layers"][index], tensors, eps, stored)
        after.append(x)
    logits = stored(rms_norm(x, tensors["final.norm"], eps)) @ tensors["head"].T
    return logits, torch.stack(after)
