"""Small Limazen configurations for the tests: sizes differ from layer to layer, values that could
hide a fault by being equal (key and value sizes, query and key/value head counts, rotated channels
and head size) or by being 1 (a scaling factor, the number of chosen experts) are mixed on purpose."""

from __future__ import annotations


def layer(heads, kv_heads, dim, vdim, chunk, rot_dims, base, factor, scale, v_mix, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "rot": rot,
                      "scale": scale, "v_mix": v_mix}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def config(vocab, width, layers, eps=1e-5, cap=None):
    out = {"architecture": "Limazen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if cap is not None:
        out["logit_softcap"] = cap
    return out


CONFIGS = {
    # every feed-forward kind, two chosen experts, a layer that does not blend between layers that do, head sizes that
    # are no multiple of 16 (the 32-bit attention kernel in both precisions), chunks of 24 and 10
    "mixed_kinds": config(211, 64, [
        layer(4, 2, 12, 20, 24, 8, 10000.0, 2.0, 0.3, True, dense(96)),
        layer(2, 1, 24, 8, 10, 24, 500.0, None, 0.2, False, moe(5, 2, 24, shared=40)),
        layer(4, 2, 12, 20, 24, 4, 10000.0, 1.0, 0.25, True, None),
        layer(2, 2, 8, 20, 24, 8, 777.0, 3.0, 0.4, True, moe(3, 1, 32)),
    ], cap=12.0),
    # head sizes that are multiples of 16: the tensor-core attention in bfloat16, keys and values of different sizes on
    # pages of the larger size; the first layer does not blend, so the second is the one whose values are kept
    "wide_heads": config(150, 96, [
        layer(4, 1, 32, 16, 40, 16, 20000.0, 5.0, 0.2, False, moe(6, 3, 16, shared=48)),
        layer(2, 2, 16, 48, 33, 16, 10000.0, 2.0, 0.3, True, dense(64)),
        layer(6, 2, 64, 48, 7, 32, 10000.0, None, 0.15, True, moe(4, 4, 24, shared=16)),
        layer(4, 2, 48, 48, 64, 48, 1000.0, 8.0, 0.18, True, dense(80)),
    ], eps=1e-6),
    # one layer, one head, a chunk of 1 (a token sees only itself), no soft cap, every expert chosen
    "smallest": config(64, 32, [layer(1, 1, 16, 4, 1, 2, 100.0, None, 1.0, True, moe(2, 2, 8))]),
    # a chunk longer than any request, no layer blends, no feed-forward in the last layer
    "one_chunk": config(97, 48, [
        layer(3, 3, 16, 16, 1000, 16, 10000.0, 1.5, 0.25, False, dense(72)),
        layer(2, 1, 20, 36, 1000, 10, 10000.0, 1.0, 0.22, False, None),
    ], cap=50.0),
}
PAGES = {"mixed_kinds": 4, "wide_heads": 16, "smallest": 2, "one_chunk": 8}
INIT = dict(std=0.25, norm_std=0.3)
