"""A plain, slow restatement of the Futepel design in PyTorch on the CPU, one function
per mechanism, written from the design's equations and sharing no code with the
engine.  Whole sequences only: no cache, no state handed between calls; recurrences
are token-by-token loops.  `dtype` is the arithmetic type (float64 for an oracle).

Notation: T tokens, W model width, H heads; weights are [out, in] and applied as
x @ w.T; positions count from 0.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return rms_unit(x, eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ---- embedding --------------------------------------------------------------------------

def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous, current); the first
    token of a sequence takes the row after the buckets."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * mul_prev + cur * mul_cur) % buckets)
    return torch.tensor(rows[:len(tokens)], dtype=torch.long)


def embed(tokens, w, emb_cfg):
    t = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][t] * emb_cfg.get("scale", 1.0)
    if emb_cfg.get("bigram") is not None:
        b = emb_cfg["bigram"]
        x = x + w["bigram"][bigram_rows(list(tokens), b["buckets"], b["mul_prev"], b["mul_cur"])]
    if "pos" in w:
        x = x + w["pos"][:len(tokens)]
    return x


# ---- the wkv mixer ------------------------------------------------------------------------

def shifted(h):
    """The previous token's row for every token, zeros for the first."""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)


def wkv_recurrence(r, k, v, w, u):
    """r, k, w: [T, H, D]; v: [T, H, E]; u: [H, D].  Per head, from S = 0 [D, E]:
    o_t = (S + diag(u) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T."""
    T, H, D = k.shape
    E = v.shape[2]
    S = torch.zeros(H, D, E, dtype=r.dtype)
    out = torch.zeros(T, H, E, dtype=r.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S + u[:, :, None] * kv, r[t])
        S = w[t][:, :, None] * S + kv
    return out


def wkv_mixer(h, w, cfg, eps):
    T = h.shape[0]
    H, D = cfg["heads"], cfg["dim"]
    prev = shifted(h)
    mix = {s: h + (prev - h) * w[f"mu.{s}"] for s in "rkvgw"}
    r = (mix["r"] @ w["r"].T).view(T, H, D)
    k = (mix["k"] @ w["k"].T).view(T, H, D)
    v = (mix["v"] @ w["v"].T).view(T, H, D)
    gate = silu(mix["g"] @ w["g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w["w1"].T) @ w["w2"].T + w["w0"])).view(T, H, D)
    o = wkv_recurrence(r, k, v, decay, w["u"])
    o = rms_unit(o, eps).reshape(T, H * D) * w["norm"] * gate
    return o @ w["o"].T


# ---- latent attention -----------------------------------------------------------------------

def yarn_frequencies(dims, base, scaling, dtype):
    """The rotation's frequencies and the factor on cos and sin."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(scaling["fast"])), 0)
    hi = min(math.ceil(dim_of(scaling["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, freq, mscale):
    """x: [T, heads, n]: the first dims = 2 len(freq) features turn, feature i with i + dims/2;
    the rest pass unchanged."""
    half = freq.shape[0]
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = (torch.cos(ang) * mscale)[:, None, :], (torch.sin(ang) * mscale)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], -1)


def latent_attention(h, w, cfg, eps, positions):
    T = h.shape[0]
    H, D, R, E, C = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    rot = cfg["rot"]
    freq, mscale = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
    q = (h @ w["q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_half(q[..., D:], positions, freq, mscale)
    dkv = h @ w["dkv"].T
    c = rms_norm(dkv[:, :C], w["dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, None, C:], positions, freq, mscale)          # [T, 1, R]
    k_plain = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, E)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain)
         + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * cfg["scale"]
    mask = positions[None, :] <= positions[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hij,jhe->ihe", p, v)
    o = o * torch.sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * E) @ w["o"].T


# ---- mamba2 -----------------------------------------------------------------------------------

def causal_conv(x, taps_w, bias):
    """x: [T, C]; taps_w: [C, taps], the last column meets the current token; zeros before
    the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = bias.expand(T, C).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * taps_w[:, j]
    return out


def ssd_recurrence(x, B, Cm, dt, a_log, skip, groups):
    """x: [T, H, P]; B, Cm: [T, G, N]; dt: [T, H].  Per head (group = head // (H / G)), from
    S = 0 [N, P]:  S <- exp(-exp(a_log) dt) S + dt B x^T;  y = S^T C + skip x."""
    T, H, P = x.shape
    N = B.shape[2]
    per = H // groups
    S = torch.zeros(H, N, P, dtype=x.dtype)
    y = torch.zeros(T, H, P, dtype=x.dtype)
    for t in range(T):
        for hd in range(H):
            g = hd // per
            S[hd] = torch.exp(-torch.exp(a_log[hd]) * dt[t, hd]) * S[hd] \
                + dt[t, hd] * B[t, g][:, None] * x[t, hd][None, :]
            y[t, hd] = S[hd].T @ Cm[t, g] + skip[hd] * x[t, hd]
    return y


def mamba2_mixer(h, w, cfg, eps):
    T = h.shape[0]
    H, P, N, G = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"]
    inner = H * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = ssd_recurrence(x, B, Cm, dt, w["A_log"], w["D"], G).reshape(T, inner)
    y = y * silu(z)
    parts = cfg.get("norm_groups", 1)
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


# ---- feed-forwards ------------------------------------------------------------------------------

def relu2_ff(h, w):
    return torch.relu(h @ w["up"].T) ** 2 @ w["down"].T


def gated_ff(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(logits, top):
    """The `top` largest logits of every row and the softmax over them alone."""
    vals, idx = torch.topk(logits, top, dim=-1)
    return idx, torch.softmax(vals, -1)


def moe_ff(h, w, cfg):
    n, top = cfg["router"]["experts"], cfg["router"]["top"]
    idx, weight = route(h @ w["router"].T, top)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += weight[t, j] * gated_ff(h[t:t + 1], sub(w, f"e{e}."))[0]
    if cfg.get("shared") is not None:
        out = out + gated_ff(h, sub(w, "shared."))
    return out


# ---- the model ----------------------------------------------------------------------------------

def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=torch.float64, layer_outputs=None):
    """Logits [T, vocab] of one sequence; `layer_outputs`, a list, receives the residual
    after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = embed(tokens, w, config.get("embedding", {}))
    for li, layer in enumerate(config["layers"]):
        lw = sub(w, f"l{li}.")
        mw = sub(lw, "mix.")
        hn = rms_norm(x, lw["norm1"], eps)
        kind = layer["type"]
        if kind == "wkv":
            x = x + wkv_mixer(hn, mw, layer["mixer"], eps)
        elif kind == "latent_attention":
            x = x + latent_attention(hn, mw, layer["mixer"], eps, positions)
        elif kind == "mamba2":
            x = x + mamba2_mixer(hn, mw, layer["mixer"], eps)
        else:
            raise ValueError(kind)
        mlp = layer.get("mlp")
        if mlp is not None:
            hn = rms_norm(x, lw["norm2"], eps)
            fw = sub(lw, "mlp.")
            x = x + (relu2_ff(hn, fw) if mlp["kind"] == "dense" else moe_ff(hn, fw, mlp))
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def read_folder(model_dir, dtype=torch.float64):
    """(config.json as a dict, tensors by name) of a model folder."""
    import json
    import os
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    tensors = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return config, tensors


def greedy(config, tensors, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]
