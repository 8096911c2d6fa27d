"""A plain, slow restatement of the Vuvosun design in PyTorch on the CPU, one
function per mechanism, written from the design's equations and sharing no code
with the engine.  Whole sequences only: no cache, no state handed between
calls; recurrences are token-by-token loops.  `dtype` is the arithmetic type
(float64 for an oracle, float32 to see what rounding does).

Notation: T tokens, W model width, H heads, G key/value heads, D key size,
E value size; weights are [out, in] and applied as x @ w.T.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return rms_unit(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_interleaved(x, positions, base, dims):
    """x: [T, heads, D].  Features (2i, 2i+1), i < dims/2, turn by the angle
    position * base^(-2i/dims); features from `dims` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]             # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible(i, j, size, keep_first):
    """Whether position i sees position j under a window that keeps the first tokens."""
    return j <= i and (i - j < size or j < keep_first)


def attend(q, k, v, positions, sink, scale, size, keep_first):
    """q: [T, H, D], k: [T, G, D], v: [T, G, E] of one sequence at `positions` (already
    turned and normalised); sink: [H] or None; size None: every earlier key.
    Returns [T, H, E]."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    allowed = torch.tensor([[visible(int(i), int(j), size if size is not None else 1 << 60, keep_first)
                             for j in positions] for i in positions])
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        m = s.max(-1).values
        if sink is not None:
            m = torch.maximum(m, sink[head])
        e = torch.exp(s - m[:, None])
        denom = e.sum(-1)
        if sink is not None:
            denom = denom + torch.exp(sink[head] - m)
        out[:, head] = (e / denom[:, None]) @ v[:, g]
    return out


def sink_window_attention(h, w, cfg, eps, prefix=""):
    """Softmax attention with grouped heads, a window that keeps the first tokens, a
    per-head sink in the denominator, unit-rms values and a sigmoid output gate.
    Returns the projected result [T, W]."""
    T = h.shape[0]
    H, G, D, E = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = (h @ w[prefix + "q"].T).view(T, H, D)
    k = (h @ w[prefix + "k"].T).view(T, G, D)
    v = (h @ w[prefix + "v"].T).view(T, G, E)
    pos = torch.arange(T)
    if cfg.get("rot") is not None:
        q = rotate_interleaved(q, pos, cfg["rot"]["base"], cfg["rot"]["dims"])
        k = rotate_interleaved(k, pos, cfg["rot"]["base"], cfg["rot"]["dims"])
    v = rms_unit(v, eps)
    mask = cfg.get("mask")
    out = attend(q, k, v, pos, w[prefix + "sink"], cfg["scale"],
                 mask["size"] if mask else None, mask.get("keep_first", 0) if mask else 0)
    gate = torch.sigmoid(h @ w[prefix + "g"].T)
    return (out.reshape(T, H * E) * gate) @ w[prefix + "o"].T


def causal_conv(x, taps_w):
    """x: [T, C]; taps_w: [C, taps], last column meets the current token; zeros before
    the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j:j + T] * taps_w[:, j][None, :]
    return out


def delta_rule(q, k, v, beta, decay, S=None):
    """One head.  q, k: [T, D] (unit vectors, q scaled), v: [T, E], beta, decay: [T].
    S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Returns (o [T, E], S)."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype) if S is None else S.clone()
    out = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out, S


def gated_delta(h, w, cfg, eps, prefix=""):
    """The gated delta rule with short convolutions; returns the projected result."""
    T = h.shape[0]
    H, G, D, E = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = silu(causal_conv(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).view(T, H, E)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)                       # [T, H]
    rate = torch.nn.functional.softplus(h @ w[prefix + "a"].T + w[prefix + "dt_bias"])
    decay = torch.exp(-torch.exp(w[prefix + "A_log"]) * rate)        # [T, H]
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        out[:, head], _ = delta_rule(q[:, g], k[:, g], v[:, head], beta[:, head], decay[:, head])
    out = rms_unit(out, eps) * w[prefix + "norm"]
    gate = silu(h @ w[prefix + "g"].T).view(T, H, E)
    return (out * gate).reshape(T, H * E) @ w[prefix + "o"].T


def parallel_mixer(h, w, cfg, eps):
    left = sink_window_attention(h, w, cfg["left"], eps, "left.")
    right = gated_delta(h, w, cfg["right"], eps, "right.")
    return cfg["left_scale"] * left + cfg["right_scale"] * right


def matrix_memory(q, k, v, log_in, log_keep):
    """One head of the mLSTM.  q (scaled), k: [T, D], v: [T, E], log gates [T].  The
    running maximum starts at zero.  Returns o [T, E]."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype)
    n = torch.zeros(D, dtype=q.dtype)
    m = torch.zeros((), dtype=q.dtype)
    out = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(log_keep[t] + m, log_in[t])
        a = torch.exp(log_keep[t] + m - m_new)
        b = torch.exp(log_in[t] - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        out[t] = (S.T @ q[t]) / (torch.maximum((n @ q[t]).abs(), torch.exp(-m)) + 1e-6)
    return out


def capped_log_gates(pre_i, pre_f, cap):
    log_in = cap * torch.tanh(pre_i / cap)
    log_keep = torch.nn.functional.logsigmoid(cap * torch.tanh(pre_f / cap))
    return log_in, log_keep


def mlstm(h, w, cfg, eps):
    """Matrix memory with exponential gates kept stable by a running maximum that
    starts at zero."""
    T = h.shape[0]
    H, D, E, cap = cfg["heads"], cfg["dim"], cfg["vdim"], cfg["gate_cap"]
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, E)
    log_in, log_keep = capped_log_gates(h @ w["i"].T + w["i.b"], h @ w["f"].T + w["f.b"], cap)
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for head in range(H):
        out[:, head] = matrix_memory(q[:, head], k[:, head], v[:, head], log_in[:, head],
                                     log_keep[:, head])
    out = rms_unit(out, eps).reshape(T, H * E) * w["norm"]
    return (out * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def polynorm(z, coef, eps):
    a, b, c, e = coef
    return a * rms_unit(z, eps) + b * rms_unit(z ** 2, eps) + c * rms_unit(z ** 3, eps) + e


def polynorm_ff(h, w, eps):
    return polynorm(h @ w["up"].T, w["act"], eps) @ w["down"].T


def hyper_sublayer(streams, y_of, gain, eps, w_in, w_mix, w_out):
    """streams: list of [T, W].  u = sum_s in[s] x_s; y = y_of(norm(u));
    x_t <- sum_s mix[s, t] x_s + out[t] y, all t from the old streams."""
    n = len(streams)
    u = sum(w_in[s] * streams[s] for s in range(n))
    y = y_of(rms_norm(u, gain, eps))
    return [sum(w_mix[s, t] * streams[s] for s in range(n)) + w_out[t] * y for t in range(n)]


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=torch.float64, layer_outputs=None):
    """Logits [T, vocab] for one sequence of token ids.  `layer_outputs`, a list,
    receives the sum of the streams after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x0 = rms_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
    n_streams = config.get("streams")
    streams = [x0.clone() for _ in range(n_streams or 1)]

    def sublayer(fn, norm_gain, hc):
        nonlocal streams
        if n_streams is None:
            streams = [streams[0] + fn(rms_norm(streams[0], norm_gain, eps))]
            return
        streams = hyper_sublayer(streams, fn, norm_gain, eps, hc["in"], hc["mix"], hc["out"])

    for li, layer in enumerate(config["layers"]):
        lw = sub(w, f"l{li}.")
        mw = sub(lw, "mix.")
        if layer["type"] == "parallel":
            mixer = lambda h: parallel_mixer(h, mw, layer["mixer"], eps)
        elif layer["type"] == "mlstm":
            mixer = lambda h: mlstm(h, mw, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        sublayer(mixer, lw["norm1"], sub(lw, "hc1."))
        if layer.get("mlp") is not None:
            fw = sub(lw, "mlp.")
            sublayer(lambda h: polynorm_ff(h, fw, eps), lw["norm2"], sub(lw, "hc2."))
        if layer_outputs is not None:
            layer_outputs.append(sum(streams))
    x = rms_norm(sum(streams), w["final.norm"], eps)
    return x @ w["embed"].T


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
