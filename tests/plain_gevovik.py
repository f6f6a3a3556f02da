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
    """x over the root of (its mean square along the last axis, plus eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def causal_conv(u, taps_w, bias=None):
    """u [T, C], taps_w [C, taps]: y[t] = sum_j taps_w[:, j] * u[t - (taps - 1) + j], with u = 0 at negative times."""
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


greedy = generate


# ---- configurations of the tests and random weights ----------------------------------------------------------
def ssm(heads, vdim, state, groups, conv, norm_groups):
    return ("mamba2", {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                       "norm_groups": norm_groups})


def talking(heads, kv_heads, dim, vdim, scale, window=None, rot=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window is not None:
        m["mask"] = {"size": window}
    return m


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def pair(left, right, left_scale, right_scale):
    return ("parallel", {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale})


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return ("latent_attention", m)


def model(vocab, width, eps, layers, scale=1.0, bigram=None):
    """``layers``: [((type, mixer), ff or None)]; ``bigram``: (buckets, mul_prev, mul_cur)."""
    e = {"scale": scale}
    if bigram is not None:
        e["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return {"architecture": "Gevovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": e,
            "layers": [{"type": t, "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
                       for (t, m), ff in layers]}


# name -> (configuration, {layer: (a_rank, g_rank)} of the delta rule's narrow projections, page size)
CONFIGS = {
    # a pair first, a window of 24 over pages of 8, half of each head rotated with stretched slow pairs, a layer
    # without feed-forward, a latent layer that reads another one's rows
    "A": (model(96, 64, 1e-5, [
        (pair(talking(4, 2, 16, 8, 0.25, window=24, rot=(8, 10000.0), scaling=(4.0, 16, 4.0, 1.0)),
              delta(2, 1, 8, 16, 4), 0.7, 1.2), 48),
        (ssm(4, 8, 16, 2, 3, 2), 40),
        (latent(2, 8, 4, 8, 16, 0.3), None),
        (latent(3, 8, 4, 16, 16, 0.25, kv_from=2), 48),
        (ssm(2, 16, 8, 1, 4, 1), None)], scale=3.0, bigram=(53, 5, 3)), {0: (6, 4)}, 8),
    # sizes that are multiples of nothing; one head; no pair table; no mask (every earlier key); no scaling; one tap
    "B": (model(70, 44, 1e-6, [
        (latent(1, 6, 2, 10, 12, 0.4), 36),
        (ssm(3, 5, 7, 1, 2, 3), 28),
        (pair(talking(1, 1, 10, 6, 0.3, rot=(10, 500.0)), delta(1, 1, 6, 10, 1), 1.0, 0.5), None),
        (ssm(3, 4, 6, 3, 1, 1), 20)], scale=1.0), {2: (3, 5)}, 4),
    # six heads over two that talk, a window shorter than a page and one of a single token, no rotation in one
    # pair, latent rows that the tensor-core form takes, two layers reading them
    "C": (model(128, 96, 1e-5, [
        (ssm(6, 16, 32, 2, 4, 3), 64),
        (latent(4, 16, 16, 16, 32, 0.2, base=1000.0), 64),
        (pair(talking(6, 2, 16, 16, 0.25, window=5, rot=(16, 10000.0), scaling=(2.0, 8, 8.0, 2.0)),
              delta(4, 2, 16, 8, 2), 0.9, 0.8), 64),
        (latent(2, 32, 16, 8, 32, 0.15, base=1000.0, kv_from=1), None),
        (pair(talking(2, 1, 32, 16, 0.2, window=1), delta(2, 2, 8, 8, 3), 1.1, 1.0), 32),
        (latent(4, 8, 16, 24, 32, 0.2, base=1000.0, kv_from=1), 64)], scale=2.0, bigram=(31, 1, 7)),
          {2: (8, 8), 4: (2, 16)}, 16),
}


def config(name):
    cfg, ranks, page = CONFIGS[name]
    return cfg, dict(ranks), page


def tensor_shapes(cfg, ranks):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "final.norm": (), "head": (V, D)}
    b = cfg["embedding"].get("bigram")
    if b is not None:
        s["bigram"] = (b["buckets"] + 1, D)
    for i, layer in enumerate(cfg["layers"]):
        p, m, t = f"l{i}.", layer["mixer"], layer["type"]
        s[p + "norm1"] = ()
        q = p + "mix."
        if t == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            s.update({q + "in": (2 * inner + 2 * gn + m["heads"], D), q + "conv": (inner + 2 * gn, m["conv"]),
                      q + "conv.b": (inner + 2 * gn,), q + "dt_bias": (m["heads"],), q + "A_log": (m["heads"],),
                      q + "D": (m["heads"],), q + "norm": (inner,), q + "o": (D, inner)})
        elif t == "parallel":
            a, d = m["left"], m["right"]
            l, r = q + "left.", q + "right."
            s.update({l + "q": (a["heads"] * a["dim"], D), l + "k": (a["kv_heads"] * a["dim"], D),
                      l + "v": (a["kv_heads"] * a["vdim"], D), l + "q.norm": (a["dim"],), l + "k.norm": (a["dim"],),
                      l + "talk": (a["heads"], a["heads"]), l + "temp": (a["heads"],), l + "g": (a["heads"], D),
                      l + "o": (D, a["heads"] * a["vdim"])})
            ra, rg = ranks[i]
            qk, vw = d["kv_heads"] * d["dim"], d["heads"] * d["vdim"]
            s.update({r + "q": (qk, D), r + "q.conv": (qk, d["conv"]), r + "k": (qk, D), r + "k.conv": (qk, d["conv"]),
                      r + "v": (vw, D), r + "v.conv": (vw, d["conv"]), r + "b": (d["heads"], D),
                      r + "A_log": (d["heads"],), r + "norm": (d["vdim"],), r + "a1": (ra, D),
                      r + "a2": (d["heads"] * d["dim"], ra), r + "dt_bias": (d["heads"] * d["dim"],),
                      r + "g1": (rg, D), r + "g2": (vw, rg), r + "o": (D, vw)})
        else:
            H = m["heads"]
            s.update({q + "q": (H * (m["dim"] + m["rot_dim"]), D), q + "uk": (H * m["dim"], m["kv_rank"]),
                      q + "uv": (H * m["vdim"], m["kv_rank"]), q + "sink": (H,), q + "o": (D, H * m["vdim"])})
            if m.get("kv_from") is None:
                s.update({q + "dkv": (m["kv_rank"] + m["rot_dim"], D), q + "dkv.norm": (m["kv_rank"],)})
        if layer["mlp"] is not None:
            s.update({p + "norm2": (), p + "mlp.up": (layer["mlp"]["ff"], D), p + "mlp.down": (D, layer["mlp"]["ff"])})
    return s


def random_weights(cfg, ranks, seed, sharp=1.0):
    """Random tensors (values that bfloat16 holds exactly).  Matrices N(0, 1 / fan-in); norm weights around one;
    ``sharp`` multiplies the attention layers' queries, so that the softmax sits on few keys."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        leaf = name.split(".")[-1]
        if name.endswith(("norm1", "norm2", "final.norm", ".norm", ".D", ".temp")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf in ("A_log", "dt_bias", "sink", "b") and len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif leaf == "talk":
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = 0.5 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            if name.endswith((".left.q", "mix.q")) and "right" not in name:
                t = t * sharp
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


def random_config(seed):
    """A configuration drawn at random: (config, ranks, page size).  Every size, count, constant and option that a
    configuration may state is drawn, the order of the layers too."""
    import random
    r = random.Random(seed)
    width = r.choice([32, 40, 48, 64, 96])
    layers, ranks, own_latents = [], {}, []
    n_layers = r.randint(2, 6)
    for i in range(n_layers):
        kind = r.choice(["mamba2", "parallel", "latent_attention"])
        if kind == "mamba2":
            heads = r.choice([1, 2, 3, 4, 6, 8])
            vdim = r.choice([4, 8, 16, 32])
            groups = r.choice([g for g in (1, 2, 3, 4) if heads % g == 0])
            norm_groups = r.choice([g for g in (1, 2, 3, heads) if (heads * vdim) % g == 0])
            mix = ssm(heads, vdim, r.choice([4, 8, 16, 48, 64]), groups, r.randint(1, 4), norm_groups)
        elif kind == "parallel":
            kv = r.choice([1, 2, 4])
            dim = r.choice([8, 16, 24, 32, 48, 64])
            rot = scaling = None
            if r.random() < 0.8:
                rot = (r.choice([d for d in (2, 4, 8, 16, 32, 64, dim) if d <= dim]), r.choice([100.0, 10000.0, 500000.0]))
                if r.random() < 0.6:
                    scaling = (r.choice([1.5, 2.0, 8.0]), r.choice([8, 64, 512]), r.choice([4.0, 32.0]), r.choice([0.5, 1.0]))
            window = r.choice([None, 1, 3, 7, 16, 33, 72])
            left = talking(kv * r.choice([1, 2, 3]), kv, dim, r.choice([8, 16, 24, 32, 48, 64]),
                           dim ** -0.5 * r.choice([0.7, 1.0, 1.6]), window=window, rot=rot, scaling=scaling)
            kv2 = r.choice([1, 2])
            right = delta(kv2 * r.choice([1, 2]), kv2, r.choice([4, 8, 16, 32]), r.choice([4, 8, 16, 32]), r.randint(1, 4))
            mix = pair(left, right, r.choice([0.5, 0.8, 1.0]), r.choice([0.6, 0.9, 1.3]))
            ranks[i] = (r.randint(2, 8), r.randint(2, 8))
        else:
            heads, dim, vdim = r.randint(1, 6), r.choice([4, 8, 16, 32, 64]), r.choice([4, 8, 16, 64])
            if own_latents and r.random() < 0.5:
                j = r.choice(own_latents)
                src = layers[j][0][1]
                mix = latent(heads, dim, src["rot_dim"], vdim, src["kv_rank"], r.choice([0.1, 0.2, 0.35]),
                             base=src["rot"]["base"], kv_from=j)
            else:
                mix = latent(heads, dim, r.choice([2, 4, 8, 16]), vdim, r.choice([8, 16, 24, 32, 64]),
                             r.choice([0.1, 0.2, 0.35]), base=r.choice([100.0, 10000.0, 1000000.0]))
                own_latents.append(i)
        layers.append((mix, r.choice([None, 16, 24, 40, 64, 100])))
    bigram = (r.choice([7, 31, 53, 97]), r.randint(1, 40), r.randint(1, 40)) if r.random() < 0.7 else None
    cfg = model(r.randint(50, 200), width, r.choice([1e-5, 1e-6]), layers,
                scale=r.choice([1.0, 0.5, float(width) ** 0.5]), bigram=bigram)
    return cfg, ranks, r.choice([4, 8, 16])
