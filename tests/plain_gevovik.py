"""Gevovik, written out plainly: whole sequences, float64, no cache, no state carried, nothing imported from
the package.  One function per mechanism; ``forward`` puts them together from the configuration's JSON form
and a dict of tensors by name.  It is the oracle of ``tests/test_gevovik.py``.

Notation: h [T, D] the residual stream of one sequence, positions 0 .. T-1, ``w`` a dict name -> float64 tensor.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def causal_conv(u, taps_w, bias=None):
    """u [T, C], taps_w [C, taps] with the last column the current token's, zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros((taps - 1, C), dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * taps_w[:, j]
    return y if bias is None else y + bias


# ---- embedding ---------------------------------------------------------------------------------------------
def embedding(cfg, w, tokens):
    e = cfg["embedding"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] * float(e["scale"])
    b = e.get("bigram")
    if b is not None:
        n = int(b["buckets"])
        rows = [n]
        for prev, cur in zip(tokens[:-1], tokens[1:]):
            rows.append((int(prev) * int(b["mul_prev"]) + int(cur) * int(b["mul_cur"])) % n)
        x = x + w["bigram"][torch.tensor(rows)]
    return x


# ---- rotations ---------------------------------------------------------------------------------------------
def rotary_frequencies(rot):
    """Inverse frequencies of the dims / 2 pairs and the factor on cos and sin (1 without scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, rot, interleaved):
    """x [T, heads, d]: the first rot.dims coordinates of each head turned by position * frequency."""
    T = x.shape[0]
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    ang = torch.arange(T, dtype=F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]
    cos, sin = (torch.cos(ang) * m)[:, None, :], (torch.sin(ang) * m)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * cos - v * sin
        out[..., dims // 2:dims] = v * cos + u * sin
    return out


# ---- mixers ------------------------------------------------------------------------------------------------
def mamba2(m, w, p, h, eps):
    T = h.shape[0]
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                       # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)          # [T, H]
    y = torch.zeros((T, H, P), dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros((N, P), dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def talking_window_attention(m, w, p, h, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = rms_unit(q, eps) * w[p + "q.norm"]
    k = rms_unit(k, eps) * w[p + "k.norm"]
    if m.get("rot") is not None:
        q, k = rotate(q, m["rot"], False), rotate(k, m["rot"], False)
    kk = k[:, [hd // (H // G) for hd in range(H)]]               # [T, H, d]
    vv = v[:, [hd // (H // G) for hd in range(H)]]
    s = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"])
    s = s * w[p + "temp"][:, None, None]
    s = torch.einsum("hg,gij->hij", w[p + "talk"], s)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i)
    if m.get("mask") is not None:
        seen = seen & (i - j < int(m["mask"]["size"]))
    s = s.masked_fill(~seen[None], float("-inf"))
    a = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", a, vv)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def gated_delta(m, w, p, h, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                       # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, d))
    o = torch.zeros((T, H, dv), dtype=F64)
    for hd in range(H):
        qk = hd // (H // G)
        S = torch.zeros((d, dv), dtype=F64)
        for t in range(T):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, qk])
            S = S + torch.outer(k[t, qk], u)
            o[t, hd] = S.T @ q[t, qk]
    o = rms_unit(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * dv) * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T)
    return o @ w[p + "o"].T


def parallel(m, w, p, h, eps):
    return (float(m["left_scale"]) * talking_window_attention(m["left"], w, p + "left.", h, eps)
            + float(m["right_scale"]) * gated_delta(m["right"], w, p + "right.", h, eps))


def latent_rows(m, w, p, h, eps):
    """What a latent attention layer leaves per token: c [T, rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    R, r = int(m["kv_rank"]), int(m["rot_dim"])
    ckr = h @ w[p + "dkv"].T
    c = rms_unit(ckr[:, :R], eps) * w[p + "dkv.norm"]
    kr = rotate(ckr[:, None, R:], m["rot"], True)[:, 0]
    return c, kr


def latent_attention(m, w, p, h, eps, rows):
    T = h.shape[0]
    H, d, r, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    c, kr = rows
    q = (h @ w[p + "q"].T).reshape(T, H, d + r)
    qn, qr = q[..., :d], rotate(q[..., d:], m["rot"], True)
    kn = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * float(m["scale"])
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    s = s.masked_fill(~(j <= i)[None], float("-inf"))
    sink = w[p + "sink"][:, None, None].expand(H, T, 1)
    a = torch.softmax(torch.cat([s, sink], -1), -1)[..., :T]      # the sink has no value
    o = torch.einsum("hij,jhd->ihd", a, v)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def relu2_ffn(w, p, h):
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


# ---- the model ---------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that gets the stream after every layer."""
    w = {k: v.to(F64) if v.is_floating_point() else v for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    h = embedding(cfg, w, list(tokens))
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m, t = f"l{i}.", layer["mixer"], layer["type"]
        if t == "mamba2":
            a = mamba2(m, w, p + "mix.", h, eps)
        elif t == "parallel":
            a = parallel(m, w, p + "mix.", h, eps)
        elif t == "latent_attention":
            if m.get("kv_from") is not None:
                rows = kept[int(m["kv_from"])]
            else:
                rows = kept[i] = latent_rows(m, w, p + "mix.", h, eps)
            a = latent_attention(m, w, p + "mix.", h, eps, rows)
        else:
            raise ValueError(f"layer type {t!r}")
        h = h + rms_unit(a, eps) * w[p + "norm1"]
        if layer.get("mlp") is not None:
            h = h + rms_unit(relu2_ffn(w, p + "mlp.", h), eps) * w[p + "norm2"]
        if layers_out is not None:
            layers_out.append(h.clone())
    return (rms_unit(h, eps) * w["final.norm"]) @ w["head"].T


def generate(cfg, w, prompt, n):
    """Greedy continuation (ties -> lowest id)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, w, toks)[-1]).item()))
    return toks[len(prompt):]
