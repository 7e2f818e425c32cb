"""A plain, slow Limazen in float64 torch on the CPU: the oracle of the Limazen tests.

One function per mechanism, written from the design's equations and sharing nothing with the
package: every sequence is taken alone and whole, with no cache, no pages and no batching.
`forward` returns the logits of every position and the residual stream after every layer.

Notation: n tokens, W the model width, H query heads, G key/value heads, d the query/key size of a
head, e its value size, r the number of rotated channels of a head, C the chunk size of the mask.
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


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias over the last axis."""
    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(dim=-1, keepdim=True) + eps) * weight + bias


def rotate_partial(x: torch.Tensor, positions: torch.Tensor, r: int, base: float, factor: float) -> torch.Tensor:
    """x [n, heads, d]: channels i and i + r/2 (i < r/2) of every head turn by the angle
    position * base^(-2i/r) / factor; channels r.. stay as they are."""
    half = r // 2
    freq = torch.tensor([base ** (-2.0 * i / r) / factor for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:r]
    out[..., :half] = u * cos - v * sin
    out[..., half:r] = v * cos + u * sin
    return out


def chunked_softmax_attention(q, k, v, scale: float, chunk: int) -> torch.Tensor:
    """q [n, H, d], k [n, G, d], v [n, G, e] -> [n, H, e]. Query i sees key j when j <= i and both lie
    in the same chunk of `chunk` positions counted from 0; weights are a softmax of scale * q_i . k_j."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.zeros(n, heads, v.shape[2], dtype=F)
    for h in range(heads):
        g = h // group
        for i in range(n):
            lo = (i // chunk) * chunk
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            w = torch.softmax(s, dim=0)
            out[i, h] = (w[:, None] * v[lo:i + 1, g]).sum(0)
    return out


def attention_mixer(h, t: dict, mixer: dict, first_values, stored=exact):
    """The mixer: projections with biases, partial rotation of q and k, values blended with the
    first blending layer's values of the same token, chunked attention, a sigmoid gate per channel of
    the concatenated heads, the output projection. Returns (output, this layer's values before any
    blending if it is the first blending layer, else `first_values` unchanged)."""
    heads, kv, d, e = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    h = stored(h)
    q = (h @ t["q"].T + t["q.b"]).view(n, heads, d)
    k = (h @ t["k"].T + t["k.b"]).view(n, kv, d)
    v = (h @ t["v"].T + t["v.b"]).view(n, kv, e)
    rot = mixer["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    positions = torch.arange(n)
    q = stored(rotate_partial(q, positions, rot["dims"], float(rot["base"]), factor))
    k = stored(rotate_partial(k, positions, rot["dims"], float(rot["base"]), factor))
    if mixer.get("v_mix"):
        if first_values is None:
            first_values = v
        else:
            lam = t["vmix"]
            v = (1.0 - lam) * v + lam * first_values
    v = stored(v)
    mixed = chunked_softmax_attention(q, k, v, float(mixer["scale"]), int(mixer["mask"]["size"]))
    gate = torch.sigmoid(h @ t["g"].T)
    return stored(stored(mixed.reshape(n, heads * e) * gate) @ t["o"].T), first_values


def dense_feed_forward(h, t: dict, stored=exact) -> torch.Tensor:
    """down(relu(up h)^2)."""
    h = stored(h)
    return stored(stored(torch.relu(h @ t["up"].T) ** 2) @ t["down"].T)


def gated_expert(h, t: dict, stored=exact) -> torch.Tensor:
    """down(silu(gate h) * (up h))."""
    h = stored(h)
    g = h @ t["gate"].T
    return stored(stored(g * torch.sigmoid(g) * (h @ t["up"].T)) @ t["down"].T)


def routed_feed_forward(h, t: dict, mlp: dict, stored=exact) -> torch.Tensor:
    """Every token goes to the `top` experts with the largest sigmoid(router h); an expert is fed
    score * h (its score is not renormalised and scales its INPUT); a shared expert, where there is
    one, is added with the per-token factor sigmoid(sg . h)."""
    n = h.shape[0]
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.sigmoid(stored(h) @ t["router"].T)
    out = torch.zeros_like(h)
    for i in range(n):
        chosen = torch.topk(scores[i], top).indices.tolist()
        for e in chosen:
            sub = {k.split(".", 1)[1]: v for k, v in t.items() if k.startswith(f"e{e}.")}
            out[i] += gated_expert((scores[i, e] * h[i])[None], sub, stored)[0]
    if mlp.get("shared"):
        sub = {k.split(".", 1)[1]: v for k, v in t.items() if k.startswith("shared.")}
        out = out + torch.sigmoid(stored(h) @ sub["sg"].T) * gated_expert(h, sub, stored)
    return out


def forward(config: dict, tensors: dict, tokens: list[int], stored=exact):
    """(logits [n, vocab], the residual stream after every layer [layers, n, W]) of one sequence."""
    tensors = {name: value.to(F) for name, value in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = tensors["embed"][torch.tensor(tokens, dtype=torch.long)]
    streams, first_values = [], None
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        mix = {k[len(prefix) + 4:]: v for k, v in tensors.items() if k.startswith(prefix + "mix.")}
        mlp_t = {k[len(prefix) + 4:]: v for k, v in tensors.items() if k.startswith(prefix + "mlp.")}
        h = layer_norm(x, tensors[prefix + "norm1"], tensors[prefix + "norm1.b"], eps)
        mixed, first_values = attention_mixer(h, mix, layer["mixer"], first_values, stored)
        mlp = layer.get("mlp")
        if mlp is None:
            fed = 0.0
        elif mlp["kind"] == "dense":
            fed = dense_feed_forward(h, mlp_t, stored)
        else:
            fed = routed_feed_forward(h, mlp_t, mlp, stored)
        x = x + (mixed + fed)
        streams.append(x.clone())
    h = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    logits = stored(h) @ tensors["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits, torch.stack(streams)
