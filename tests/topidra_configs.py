"""Small Topidra configurations for the tests: every size differs from layer to layer, values
that could hide a fault by being equal (key and value sizes, query and key/value head counts) or
by being 1 are mixed on purpose, and layers run several times in different places."""

from __future__ import annotations


def attention(heads, kv_heads, dim, vdim, window, scale, ff=None):
    return {"type": "attention", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}}


def lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def config(vocab, width, layers, loop=(0, 0, 1), eps=1e-6):
    return {"architecture": "Topidra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
            "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}}


CONFIGS = {
    # both mixers, a span in the middle that runs four times and begins with a linear layer
    "mid_loop": config(211, 64, [
        lightning(2, 16, 8, [0.8, 0.995], ff=96),
        lightning(1, 24, 40, 0.9),
        attention(4, 2, 16, 8, 12, 0.3, ff=80),
        attention(2, 1, 8, 16, 7, 0.5),
    ], loop=(1, 3, 4)),
    # the span starts at layer 0 with an attention layer and ends the model; a window of 1; one head
    "front_loop": config(150, 48, [
        attention(3, 3, 12, 12, 21, 0.25, ff=72),
        lightning(3, 8, 12, [0.5, 0.9, 1.0], ff=64),
        attention(1, 1, 16, 4, 1, 1.0),
    ], loop=(0, 3, 2), eps=1e-5),
    # no span at all, a window longer than any request, wider than one page of keys
    "no_loop": config(97, 40, [
        attention(2, 2, 20, 36, 500, 0.2),
        lightning(2, 40, 20, [0.99, 0.6], ff=56),
    ]),
    # head sizes that are multiples of 16: in bfloat16 the attention runs on the tensor-core kernels, with keys
    # and values of different sizes on pages of the larger one; four query heads per key/value head
    "wide_heads": config(120, 64, [
        attention(4, 1, 32, 16, 24, 0.2, ff=64),
        lightning(2, 32, 16, [0.9, 0.97]),
        attention(2, 2, 16, 64, 10, 0.3),
        attention(4, 2, 48, 48, 70, 0.15, ff=48),
    ], loop=(0, 2, 2)),
    # only linear layers: no pages anywhere; only attention layers: no state anywhere
    "linear_only": config(64, 32, [lightning(2, 8, 16, 0.97, ff=48), lightning(1, 36, 8, [0.75])], loop=(0, 1, 2)),
    "softmax_only": config(80, 32, [attention(2, 1, 16, 16, 9, 0.3, ff=40), attention(4, 4, 8, 12, 33, 0.4)], loop=(1, 2, 2)),
}
PAGES = {"mid_loop": 4, "front_loop": 16, "no_loop": 8, "wide_heads": 16, "linear_only": 16, "softmax_only": 2}
INIT = dict(std=0.25, norm_std=0.3)
