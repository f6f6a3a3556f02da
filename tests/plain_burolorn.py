"""Plain implementation of Burolorn: whole sequences in float64, no cache, no state between calls, one function
per mechanism, nothing imported from the package.  The oracle of ``test_burolorn.py``.

Notation: x [T, D] the residual stream, h a sublayer's input, W[name] the tensors (linear weights [out, in]).
"""
import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the first row."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def rotate(x, pos, base, dims):
    """x [T, H, n]: pairs (i, i + dims / 2) of the first ``dims`` coordinates turn by pos * base^(-2i / dims)."""
    half = dims // 2
    if half == 0:
        return x
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = pos.to(F64)[:, None] * freq
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def chunk_mask(T, size):
    """[T, T] bool: key j is seen from i when j <= i and both lie in the same run of ``size`` positions counted
    from 0 (size None: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size is not None:
        m = m & ((i // size) == (j // size))
    return m


def sink_softmax(s, sink):
    """s [H, T, T] with -inf where a key is not seen; one more term exp(sink_h) in every denominator (sink None:
    a plain softmax)."""
    if sink is None:
        return torch.softmax(s, dim=-1)
    sink = sink.view(-1, 1, 1)
    mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - mx)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))


def attention_mixer(h, W, p, m, eps, v_first):
    """Returns (output [T, D], the values [T, G, dv] as they are attended to).  ``v_first``: the values of the
    first value-mixing layer, or None where this layer is it (or mixes nothing)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    if m.get("conv"):
        q, k, v = short_conv(q, W[p + "q.conv"]), short_conv(k, W[p + "k.conv"]), short_conv(v, W[p + "v.conv"])
    q = rms_norm(q.view(T, H, d), W[p + "q.norm"], eps)
    k = rms_norm(k.view(T, G, d), W[p + "k.norm"], eps)
    v = v.view(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot is not None:
        q, k = rotate(q, pos, rot["base"], rot["dims"]), rotate(k, pos, rot["base"], rot["dims"])
    if m.get("v_mix") and v_first is not None:
        lam = W[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rep = H // G
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    size = m["mask"]["size"] if m.get("mask") is not None else None
    s = s.masked_fill(~chunk_mask(T, size)[None], float("-inf"))
    pr = sink_softmax(s, W.get(p + "sink"))
    o = torch.einsum("hij,jhd->ihd", pr, vv)
    gate = torch.sigmoid(h @ W[p + "g"].T)            # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T, v


def glu(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(z, r):
    """z [T, E] router logits -> (chosen experts [T, top], their weights [T, top])."""
    T, E = z.shape
    s = torch.sigmoid(z)
    allowed = torch.ones(T, E, dtype=torch.bool)
    gr = r.get("groups")
    if gr is not None and gr["count"] > 1:
        n, per = gr["count"], E // gr["count"]
        sg = s.view(T, n, per)
        score = sg.topk(min(2, per), dim=-1).values.sum(-1)          # [T, n]
        best = score.topk(gr["keep"], dim=-1).indices
        ok = torch.zeros(T, n, dtype=torch.bool)
        ok.scatter_(1, best, True)
        allowed = ok[:, :, None].expand(T, n, per).reshape(T, E)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    idx = masked.topk(r["top"], dim=-1).indices
    w = s.gather(1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return idx, w


def moe(h, W, p, q):
    r = q["router"]
    idx, w = route(h @ W[p + "router"].T, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(r["top"]):
            e = int(idx[t, c])
            out[t] += w[t, c] * glu(h[t:t + 1], W, p + f"e{e}.")[0]
    if q.get("shared") is not None:
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * glu(h, W, p + "shared.")
    return out


def side_input(x, tokens, W, p, layer, dim, eps):
    e = W["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ W[p + "gate"].T) * e
    y = g @ W[p + "proj"].T
    return rms_norm(y, W[p + "norm"], eps)


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, layers_out=None):
    """logits [T, V] (float64) of one whole sequence."""
    W = {k: v.to(F64) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    side = cfg["token_side"]["dim"] if cfg.get("token_side") is not None else None
    x = W["embed"][tokens]
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        a, v = attention_mixer(rms_norm(x, W[p + "norm1"], eps), W, p + "mix.", m, eps, v_first)
        if m.get("v_mix") and v_first is None:
            v_first = v
        x = x + a
        if L["mlp"] is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            x = x + (glu(h, W, p + "mlp.") if L["mlp"]["kind"] == "dense" else moe(h, W, p + "mlp.", L["mlp"]))
        if side is not None:
            x = x + side_input(x, tokens, W, p + "side.", i, side, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, W["final.norm"], eps)
    return (x @ W["head"].T) * cfg.get("logit_scale", 1.0)


def decode_by_recurrence(cfg, weights, tokens):
    """The same logits, token by token, from what a serving engine keeps: per layer the last taps - 1 projected
    rows of q, k, v and the normed, rotated keys and mixed values seen so far.  A second restatement that the
    whole-sequence form above is checked against (and the engine against both)."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    side = cfg["token_side"]["dim"] if cfg.get("token_side") is not None else None
    keep = [dict(u=[], k=[], v=[]) for _ in cfg["layers"]]
    out = []
    for pos, tok in enumerate(tokens):
        x = W["embed"][tok][None]
        v_first = None
        for i, L in enumerate(cfg["layers"]):
            p, m, st = f"l{i}.mix.", L["mixer"], keep[i]
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            h = rms_norm(x, W[f"l{i}.norm1"], eps)
            u = torch.cat([h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T], dim=-1)[0]
            if m.get("conv"):
                taps = m["conv"]
                wc = torch.cat([W[p + "q.conv"], W[p + "k.conv"], W[p + "v.conv"]], dim=0)
                rows = st["u"][-(taps - 1):] if taps > 1 else []
                rows = [torch.zeros_like(u)] * (taps - 1 - len(rows)) + rows + [u]
                st["u"].append(u)
                u = sum(wc[:, j] * rows[j] for j in range(taps))
            q, k, v = u[:H * d].view(1, H, d), u[H * d:H * d + G * d].view(1, G, d), u[H * d + G * d:].view(1, G, dv)
            q, k = rms_norm(q, W[p + "q.norm"], eps), rms_norm(k, W[p + "k.norm"], eps)
            if m.get("rot") is not None:
                at = torch.tensor([pos])
                q, k = rotate(q, at, m["rot"]["base"], m["rot"]["dims"]), rotate(k, at, m["rot"]["base"], m["rot"]["dims"])
            if m.get("v_mix"):
                if v_first is None:
                    v_first = v
                else:
                    v = (1.0 - W[p + "vmix"]) * v + W[p + "vmix"] * v_first
            st["k"].append(k[0])
            st["v"].append(v[0])
            size = m["mask"]["size"] if m.get("mask") is not None else None
            j0 = (pos // size) * size if size is not None else 0
            K, Vv = torch.stack(st["k"][j0:]), torch.stack(st["v"][j0:])          # [n, G, .]
            o = torch.zeros(H, dv, dtype=F64)
            for hh in range(H):
                g = hh // (H // G)
                s = (K[:, g] @ q[0, hh]) * m["scale"]
                terms = torch.cat([s, W[p + "sink"][hh:hh + 1]]) if (p + "sink") in W else s
                pr = torch.softmax(terms, dim=0)[:s.shape[0]]
                o[hh] = pr @ Vv[:, g]
            o = o * torch.sigmoid(h[0] @ W[p + "g"].T)[:, None]
            x = x + (o.reshape(1, H * dv) @ W[p + "o"].T)
            if L["mlp"] is not None:
                h2 = rms_norm(x, W[f"l{i}.norm2"], eps)
                x = x + (glu(h2, W, f"l{i}.mlp.") if L["mlp"]["kind"] == "dense" else moe(h2, W, f"l{i}.mlp.", L["mlp"]))
            if side is not None:
                x = x + side_input(x, torch.tensor([tok]), W, f"l{i}.side.", i, side, eps)
        x = rms_norm(x, W["final.norm"], eps)
        out.append(((x @ W["head"].T) * cfg.get("logit_scale", 1.0))[0])
    return torch.stack(out)


# ---------------------------------------------------------------------------------------------
# small configurations and random weights for the tests
# ---------------------------------------------------------------------------------------------
def attn(heads, kv_heads, dim, vdim, scale, conv=None, rot=None, chunk=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def experts(n, top, ff, groups=None, scale=None, shared=None):
    r = {"experts": n, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        r["scale"] = scale
    q = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        q["shared"] = {"ff": shared}
    return q


def model(vocab, width, eps, layers, side=None, logit_scale=None):
    cfg = {"architecture": "Burolorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [{"type": "attention", "mixer": m, "mlp": f} for m, f in layers]}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


# name -> (configuration, page size of the test)
CONFIGS = {
    # the first layer mixes no values (the second is the first that does); chunks that are no multiple of a page;
    # dense, mixture, none, mixture; groups of which some are kept; a side input; logits scaled down
    "A": (model(96, 64, 1e-5,
                [(attn(4, 2, 16, 24, 0.3, conv=3, rot=(8, 100.0), chunk=24), dense(96)),
                 (attn(4, 2, 16, 24, 0.3, conv=3, rot=(8, 100.0), chunk=24, v_mix=True),
                  experts(8, 2, 32, groups=(4, 2), scale=1.5, shared=48)),
                 (attn(4, 2, 16, 24, 0.3, conv=3, rot=(8, 100.0), chunk=24, v_mix=True), None),
                 (attn(4, 2, 16, 24, 0.3, conv=3, rot=(8, 100.0), chunk=24, v_mix=True),
                  experts(8, 3, 32, groups=(2, 1), scale=1.0, shared=48))],
                side=8, logit_scale=0.5), 8),
    # sizes that are multiples of nothing: one head, the whole head rotated, no mask in one layer, two and four
    # taps, no side input, no shared expert, no groups, no scale of the router or of the logits
    "B": (model(100, 77, 1e-6,
                [(attn(1, 1, 10, 14, 0.4, conv=2, rot=(10, 50.0), chunk=9, v_mix=True), experts(6, 3, 20, groups=(3, 2))),
                 (attn(3, 1, 12, 14, 0.25, conv=4, v_mix=False), None),
                 (attn(5, 1, 6, 14, 0.5, conv=2, rot=(2, 500.0), chunk=30, v_mix=True), experts(5, 2, 12))]), 4),
    # as many key heads as query heads, equal key and value sizes of 64, a chunk of 33, four taps, every group kept
    "C": (model(200, 128, 1e-6,
                [(attn(4, 4, 64, 64, 0.125, conv=4, rot=(32, 10000.0), chunk=33, v_mix=True),
                  experts(16, 4, 64, groups=(4, 4), scale=2.5, shared=64)),
                 (attn(8, 2, 32, 32, 0.2, conv=4, rot=(32, 10000.0), chunk=70), dense(192)),
                 (attn(4, 4, 64, 64, 0.125, conv=4, rot=(16, 3000.0), chunk=33, v_mix=True),
                  experts(4, 4, 128, groups=(2, 2), shared=32))],
                side=16, logit_scale=3.0), 16),
    # twelve heads over three, values larger than keys, a chunk shorter than a page and a chunk of one position,
    # a convolution of one tap (no state), a layer without convolution
    "D": (model(300, 192, 1e-5,
                [(attn(12, 3, 40, 56, 0.16, conv=3, rot=(20, 3000.0), chunk=5, v_mix=True), dense(128)),
                 (attn(12, 3, 40, 56, 0.16, conv=1, rot=(40, 3000.0), chunk=100, v_mix=True),
                  experts(12, 3, 48, groups=(3, 2), scale=0.7, shared=80)),
                 (attn(2, 2, 128, 16, 0.1, chunk=1), dense(64)),
                 (attn(6, 3, 24, 56, 0.2, conv=5, rot=(8, 20.0), chunk=100, v_mix=True), experts(3, 1, 64))],
                side=12), 16),
}


def config(name):
    cfg, page = CONFIGS[name]
    return cfg, page


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    side = cfg["token_side"]["dim"] if cfg.get("token_side") is not None else None
    if side is not None:
        s["side.embed"] = (V, len(cfg["layers"]) * side)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        s[p + "norm1"] = (D,)
        s.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.v": (G * dv, D), p + "mix.q.norm": (d,),
                  p + "mix.k.norm": (d,), p + "mix.sink": (H,), p + "mix.g": (H, D), p + "mix.o": (D, H * dv)})
        if m.get("conv"):
            s.update({p + "mix.q.conv": (H * d, m["conv"]), p + "mix.k.conv": (G * d, m["conv"]),
                      p + "mix.v.conv": (G * dv, m["conv"])})
        if m.get("v_mix"):
            s[p + "mix.vmix"] = ()
        q = L["mlp"]
        if q is not None:
            s[p + "norm2"] = (D,)
            if q["kind"] == "dense":
                s.update({p + "mlp.gate": (q["ff"], D), p + "mlp.up": (q["ff"], D), p + "mlp.down": (D, q["ff"])})
            else:
                F = q["expert"]["ff"]
                s[p + "mlp.router"] = (q["router"]["experts"], D)
                for e in range(q["router"]["experts"]):
                    s.update({p + f"mlp.e{e}.gate": (F, D), p + f"mlp.e{e}.up": (F, D), p + f"mlp.e{e}.down": (D, F)})
                if q.get("shared") is not None:
                    S = q["shared"]["ff"]
                    s.update({p + "mlp.shared.gate": (S, D), p + "mlp.shared.up": (S, D), p + "mlp.shared.down": (D, S),
                              p + "mlp.shared.sg": (1, D)})
        if side is not None:
            s.update({p + "side.gate": (side, D), p + "side.proj": (D, side), p + "side.norm": (D,)})
    return s


def random_weights(cfg, seed, sharp=1.0):
    """float32 tensors whose values are bfloat16 numbers.  Matrices ~ N(0, 1 / in), the query projections times
    ``sharp``, up projections larger (expert outputs of visible size), router and gates wide enough that scores
    spread; convolution taps of both signs with the newest around one; mixing factors between 0.2 and 0.8; sinks
    of the size of a score; norm weights around one."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "conv":
            t = 0.4 * torch.randn(shape, generator=g)
            t[:, -1] += 1.0
        elif last == "vmix":
            t = 0.2 + 0.6 * torch.rand((), generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif name in ("embed", "side.embed"):
            t = torch.randn(shape, generator=g)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if last in ("router", "g", "sg"):
                t = t * 2.0
            if last == "up":
                t = t * 1.5
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        w[name] = t
    for i in range(len(cfg["layers"])):
        w[f"l{i}.mix.q"] = w[f"l{i}.mix.q"] * sharp
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


def greedy(cfg, weights, prompt, n):
    """n tokens, each the largest logit after everything before it (ties: the lowest id)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, weights, toks)[-1])))
    return toks[len(prompt):]
