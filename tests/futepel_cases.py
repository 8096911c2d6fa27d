"""Small Futepel configurations for the tests.  They differ from one another in every size
and option: layer order, heads, key, value and state sizes, groups, taps, norm groups, the
latent's rank and rotated part with and without stretched frequencies, dense and routed
feed-forwards with and without a shared expert, layers without a feed-forward, the bigram
hash's constants, page sizes."""
from __future__ import annotations

import os

STD = 0.08       # wider than an initialiser's 0.02, so a wrong key, state or gate moves the logits


def wkv(heads, dim, mlp, rank=None):
    mixer = {"heads": heads, "dim": dim}
    if rank is not None:
        mixer["decay_rank"] = rank
    return {"type": "wkv", "mixer": mixer, "mlp": mlp}


def mamba(heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                      "norm_groups": norm_groups}}


def latent(heads, dim, rot, vdim, rank, scale, base, scaling, mlp):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot, "scaling": scaling}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}

CASES = {
    # every mixer once, then the attention a second time with other sizes (pages of its own)
    "fu-a": dict(seed=3, page_tokens=16, config={
        "architecture": "Futepel", "vocab": 300, "width": 64, "max_positions": 512, "norm": {"eps": 1e-6},
        "embedding": {"scale": 4.0, "bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 5}},
        "layers": [latent(2, 24, 8, 16, 40, 0.2, 10000.0, YARN, moe(6, 2, 40, 24)),
                   wkv(2, 16, dense(96), rank=8),
                   mamba(4, 16, 24, 2, 3, 2, None),
                   latent(3, 16, 16, 24, 48, 0.25, 500.0, None, dense(72))]}),
    # no attention at all (the engine has no page pool); one group, one norm group, two taps;
    # top == 1 (a softmax over one logit) and no shared expert; a hash whose product needs 64 bits
    "fu-b": dict(seed=4, page_tokens=32, config={
        "architecture": "Futepel", "vocab": 211, "width": 96, "max_positions": 400, "norm": {"eps": 1e-5},
        "embedding": {"scale": 1.0, "bigram": {"buckets": 1009, "mul_prev": 2147483647, "mul_cur": 65537}},
        "layers": [mamba(3, 32, 16, 1, 2, 1, moe(4, 1, 48, 0)),
                   wkv(3, 32, None),
                   mamba(2, 48, 32, 2, 4, 4, dense(160))]}),
    # sizes that let the bfloat16 products and the attention run on the tensor cores
    "fu-c": dict(seed=5, page_tokens=8, config={
        "architecture": "Futepel", "vocab": 400, "width": 128, "max_positions": 640, "norm": {"eps": 1e-5},
        "embedding": {"scale": 8.0, "bigram": {"buckets": 255, "mul_prev": 7, "mul_cur": 3}},
        "layers": [wkv(2, 64, moe(8, 8, 64, 64), rank=16),
                   latent(4, 32, 32, 32, 96, 0.15, 20000.0, {"factor": 2.0, "original": 128, "fast": 8.0, "slow": 1.0},
                          moe(8, 3, 64, 128)),
                   latent(4, 32, 32, 32, 96, 0.15, 20000.0, {"factor": 2.0, "original": 128, "fast": 8.0, "slow": 1.0},
                          dense(256))]}),
}


def make_folder(tmp_path, name, config=None, seed=None) -> str:
    from crucible_b200.weights import write_random_model
    out = os.path.join(str(tmp_path), name)
    case = CASES.get(name, {})
    write_random_model(config or case["config"], out, case.get("seed", 0) if seed is None else seed, std=STD)
    return out
