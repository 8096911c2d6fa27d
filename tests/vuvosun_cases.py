"""Small Vuvosun configurations for the tests.  They differ from one another in every
size and option: streams (1, 2, 4), layer order, layers without a feed-forward, key
and value sizes that differ, rotation over a part of a head or all of it, grouped
heads or not, taps of the convolution, windows and kept first tokens, page sizes."""
from __future__ import annotations

import os

STD = 0.08       # as the other models' tests: wider than an initialiser's 0.02, so a wrong key, state or gate moves the logits


def _left(heads, kv, dim, vdim, dims, size, keep, scale, base=10000.0):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"base": base, "dims": dims}, "mask": {"size": size, "keep_first": keep}}


def _right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _parallel(left, right, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _mlstm(heads, dim, vdim, cap, ff):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


CASES = {
    "vu-a": dict(seed=3, page_tokens=16, config={
        "architecture": "Vuvosun", "vocab": 300, "width": 64, "streams": 2, "norm": {"eps": 1e-6},
        "layers": [_parallel(_left(4, 2, 32, 16, 16, 24, 3, 0.2), _right(4, 4, 16, 24, 3), 0.7, 1.3, 96),
                   _mlstm(2, 16, 32, 10.0, 0),
                   _parallel(_left(4, 2, 32, 16, 16, 24, 3, 0.2), _right(4, 4, 16, 24, 3), 0.7, 1.3, 96),
                   # a layer whose attention differs (window, heads, sizes, all features turned): its
                   # keys live in pages of their own; no feed-forward
                   _parallel(_left(2, 1, 16, 16, 16, 9, 0, 0.3, 300.0), _right(2, 1, 8, 8, 4), -0.5, 1.0, 0)]}),
    # no layer keeps keys: the engine has no page pool at all; one stream
    "vu-b": dict(seed=4, page_tokens=32, config={
        "architecture": "Vuvosun", "vocab": 211, "width": 96, "streams": 1, "norm": {"eps": 1e-5},
        "layers": [_mlstm(3, 32, 32, 15.0, 160), _mlstm(3, 32, 32, 15.0, 0)]}),
    # four streams, every layer parallel, one key/value head, nothing kept, two taps,
    # sizes that let the bfloat16 products run on the tensor cores
    "vu-c": dict(seed=5, page_tokens=8, config={
        "architecture": "Vuvosun", "vocab": 400, "width": 128, "streams": 4, "norm": {"eps": 1e-5},
        "layers": [_parallel(_left(2, 1, 64, 64, 64, 17, 0, 0.125, 500.0), _right(2, 1, 64, 64, 2), 1.0, 0.5, 0),
                   _parallel(_left(2, 1, 64, 64, 64, 17, 0, 0.125, 500.0), _right(2, 1, 64, 64, 2), 1.0, 0.5, 256)]}),
}


def make_folder(tmp_path, name, config=None, seed=None) -> str:
    from crucible_b200.weights import write_random_model
    out = os.path.join(str(tmp_path), name)
    case = CASES.get(name, {})
    write_random_model(config or case["config"], out, case.get("seed", 0) if seed is None else seed, std=STD)
    return out
