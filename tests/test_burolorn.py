"""Burolorn in the engine against the plain implementation of ``plain_burolorn``.

Configuration, plan and the chunked cache group on the CPU; on the GPU each mechanism alone (the short convolution
with its state, the router's rule, the gated experts in both forms, the attention mixer with mask, sink, mixed
values and gate), then whole models under every way of cutting the work: whole prompts, token-by-token decoding
from the first token, portions down to two tokens, mixed batches with pages and state slots that are used again;
keys just inside and just outside a chunk, in prompts and in decoding; a far key among hundreds; a sink that
decides; the first tokens of a sequence; long decoding; greedy generation through the Python entry point and its
scheduler; the programs.
"""
import json
import math
import os

import numpy as np
import pytest
import torch

import helpers
import plain_burolorn as plain

gpu = pytest.mark.gpu

TOL32 = 3e-5          # relative to the largest logit of the request
TOL16 = 6e-2
SHARP = {"float32": 3.0, "bfloat16": 1.5}   # the queries times this: the softmax sits on few keys


def write_model(path, name=None, cfg=None, seed=0, sharp=1.0, edit=None):
    from safetensors.torch import save_file
    if cfg is None:
        cfg, _ = plain.config(name)
    w = plain.random_weights(cfg, seed, sharp)
    if edit is not None:
        edit(w)
        w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
    os.makedirs(path, exist_ok=True)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return cfg, w


def engine_of(path, dtype, page, pool, max_requests=4, use_graphs=False, step_tokens=None):
    from ccinfer_b200.engine.engine import Engine, EngineOptions
    return Engine.from_model_dir(path, EngineOptions(
        dtype=dtype, page_size=page, kv_tokens=pool, max_requests=max_requests,
        max_tokens_per_step=step_tokens or pool, max_context=pool, use_graphs=use_graphs))


def compare(rows, ref, dtype, what):
    """32-bit: every row within TOL32.  bfloat16: a router picks its experts by a hard comparison, and rounding
    turns a close call the other way now and then, which moves that row by the size of an expert's output: up
    to one row in 25 may lie beyond TOL16 while nine in ten lie within a third of it."""
    if dtype == "float32":
        return helpers.compare(rows, ref, TOL32, what)
    errs = []
    for (rid, pos), row in rows.items():
        assert np.isfinite(row).all(), what
        errs.append(float(np.abs(row - ref[rid][pos]).max()) / max(1e-6, float(np.abs(ref[rid]).max())))
    errs = np.sort(np.array(errs))
    beyond = int((errs > TOL16).sum())
    assert beyond <= max(1, len(errs) // 25), f"{what}: {beyond} of {len(errs)} rows beyond {TOL16}"
    p90 = errs[int(0.9 * (len(errs) - 1))]
    assert p90 <= TOL16 / 3, f"{what}: nine rows in ten should lie within {TOL16 / 3:.1e}, not {p90:.2e}"
    return float(p90)


def requests_of(cfg, lengths, seed):
    rng = np.random.RandomState(seed)
    return {f"r{i}": rng.randint(0, cfg["vocab"], size=n).tolist() for i, n in enumerate(lengths)}


# ---------------------------------------------------------------------------------------------
# CPU: configuration, plan, the plain implementation's two forms, the chunked cache group
# ---------------------------------------------------------------------------------------------
def test_config_is_read_written_and_refused():
    from ccinfer_b200.config.burolorn import BurolornConfig, DenseConfig, MoeConfig
    from ccinfer_b200.config.registry import architecture_of
    from ccinfer_b200.errors import ModelConfigInvalid
    for name in plain.CONFIGS:
        cfg, _ = plain.config(name)
        c = BurolornConfig.from_json(cfg)
        assert BurolornConfig.from_json(c.to_json()) == c
        assert architecture_of(cfg).name == "Burolorn"
    cfg, _ = plain.config("A")
    c = BurolornConfig.from_json(cfg)
    assert c.vocab == 96 and c.width == 64 and c.side_dim == 8 and c.logit_scale == 0.5 and c.norm_eps == 1e-5
    m = c.layers[1].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.conv, m.rot_dims, m.rot_base, m.chunk, m.v_mix) == \
        (4, 2, 16, 24, 3, 8, 100.0, 24, True)
    assert c.first_value_mix_layer() == 1 and not c.layers[0].mixer.v_mix
    assert isinstance(c.layers[0].mlp, DenseConfig) and c.layers[2].mlp is None
    q = c.layers[1].mlp
    assert isinstance(q, MoeConfig) and (q.experts, q.top, q.expert_ff, q.groups, q.keep, q.scale, q.shared_ff) == \
        (8, 2, 32, 4, 2, 1.5, 48)
    b = BurolornConfig.from_json(plain.config("B")[0])
    assert b.side_dim is None and b.logit_scale == 1.0 and b.layers[1].mixer.chunk is None
    assert b.layers[1].mixer.rot_dims == 0 and b.layers[2].mlp.groups == 1 and b.layers[2].mlp.shared_ff == 0

    def broken(edit):
        j = json.loads(json.dumps(cfg))
        edit(j)
        with pytest.raises(ModelConfigInvalid):
            BurolornConfig.from_json(j)

    broken(lambda j: j.pop("width"))
    broken(lambda j: j["norm"].pop("eps"))
    broken(lambda j: j["layers"][0].update(type="convolution"))
    broken(lambda j: j["layers"][0]["mixer"].pop("scale"))
    broken(lambda j: j["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda j: j["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda j: j["layers"][2]["mixer"].update(vdim=8))            # its values cannot be mixed with the first's
    broken(lambda j: j["layers"][1]["mlp"]["router"].update(top=5))     # more than the kept groups hold
    broken(lambda j: j["layers"][1]["mlp"].update(kind="sparse"))
    broken(lambda j: j["layers"][0].pop("mlp"))


def test_plan_names_every_tensor():
    from ccinfer_b200.config.registry import architecture_of
    for name in plain.CONFIGS:
        cfg, _ = plain.config(name)
        arch = architecture_of(cfg)
        plan = arch.build_plan(arch.parse_config(cfg))
        specs = {s.name: tuple(s.shape) for s in plan.tensor_specs()}
        shapes = dict(plain.tensor_shapes(cfg))
        # the first value-mixing layer's factor is in the file and unused: the plan may or may not ask for it
        for k in [k for k in shapes if k.endswith(".vmix") and k not in specs]:
            shapes.pop(k)
        assert specs == shapes, (name, set(specs) ^ set(shapes))
        assert len(plan.order) == len(cfg["layers"])


def test_the_plain_implementation_agrees_with_itself():
    """Whole sequences against token-by-token decoding from what an engine would keep, in float64."""
    for name in plain.CONFIGS:
        cfg, _ = plain.config(name)
        w = plain.random_weights(cfg, 3, 2.0)
        toks = np.random.RandomState(1).randint(0, cfg["vocab"], size=45).tolist()
        a, b = plain.forward(cfg, w, toks), plain.decode_by_recurrence(cfg, w, toks)
        assert float((a - b).abs().max()) < 1e-9 * float(a.abs().max())


def test_a_chunked_group_gives_back_the_pages_behind_the_run():
    """The host core by itself: a group whose queries see only their own run of 10 positions, pages of 4."""
    from ccinfer_b200.cache.manager import CacheManager, GroupSpec
    cm = CacheManager([GroupSpec(("chunk", 10), None, 4, 12, 10)], 2, 64, 400)
    cm.open("a")
    held = []
    for n in (9, 1, 1, 7, 2, 1, 30, 3):
        cm.reserve("a", n)
        cm.commit("a")
        ctx = cm.get("a").ctx_len
        first = (ctx // 10 * 10) // 4          # the page that holds the first position of the next token's run
        assert cm.first_needed_page(0, ctx) == first
        held.append(cm.pools[0].used_pages)
        assert cm.pools[0].used_pages == -(-ctx // 4) - first, (ctx, held)
    assert max(held) <= 4
    cm.close("a")
    assert cm.pools[0].used_pages == 0
    cm.check_consistency()


# ---------------------------------------------------------------------------------------------
# GPU: each mechanism alone
# ---------------------------------------------------------------------------------------------
@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,C", [(3, 40), (2, 7), (4, 300), (1, 24), (7, 64)])
def test_short_convolution_kernel(dtype, taps, C):
    """Three requests in steps of unequal portions (single tokens, two tokens, more than the taps) over four state
    slots, one of them given to a second request afterwards: every row against the convolution of the request's
    whole sequence.  Then the same with the trailing channels as value heads that are kept, or mixed."""
    from ccinfer_b200 import kernels
    dev = "cuda"
    g = torch.Generator().manual_seed(taps * 100 + C)
    w = torch.randn(C, taps, generator=g)
    seqs = {0: torch.randn(23, C, generator=g), 2: torch.randn(9, C, generator=g), 3: torch.randn(40, C, generator=g)}
    seqs = {s: u.to(dtype) for s, u in seqs.items()}
    want = {s: plain.short_conv(u.double(), w.double()) for s, u in seqs.items()}
    state = torch.full((4, max(taps - 1, 1), C), 7.0, dtype=dtype, device=dev)[:, :taps - 1]
    state[[0, 2, 3]] = 0          # (a slot is zeroed when it is given out)
    plans = [{0: 1, 2: 2, 3: 11}, {0: 1, 3: 1}, {0: 5, 2: 1, 3: 2}, {0: 2, 2: 6, 3: 26}, {0: 14}]
    at = {s: 0 for s in seqs}
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for plan in plans:
        # single-token entries first, as the engine lays a step out
        order = sorted(plan, key=lambda s: (plan[s] != 1, s))
        rows = torch.cat([seqs[s][at[s]:at[s] + plan[s]] for s in order]).to(dev)
        cu = np.cumsum([0] + [plan[s] for s in order]).astype(np.int32)
        eot = np.repeat(np.arange(len(order)), [plan[s] for s in order]).astype(np.int32)
        n_single = sum(1 for s in order if plan[s] == 1)
        out = torch.empty_like(rows)
        cu_d, eot_d = torch.from_numpy(cu).to(dev), torch.from_numpy(eot).to(dev)
        slot_d = torch.tensor(order, dtype=torch.int32, device=dev)
        kernels.conv_rows(out, rows, w.t().contiguous().to(dev), taps, C, state if taps > 1 else None, eot_d, cu_d,
                          slot_d, len(order))
        if taps > 1:
            kernels.conv_state_rows(rows, taps, C, state, cu_d, slot_d, n_single, len(order) - n_single)
        for i, s in enumerate(order):
            got = out[cu[i]:cu[i + 1]].double().cpu()
            ref = want[s][at[s]:at[s] + plan[s]]
            assert (got - ref).abs().max() <= tol * max(1.0, float(ref.abs().max())), (taps, C, plan, s)
            at[s] += plan[s]
    if taps > 1:
        assert (state[1] == 7.0).all()       # nobody's slot
        for s, u in seqs.items():
            if at[s] >= taps - 1:
                assert torch.equal(state[s].cpu(), u[at[s] - taps + 1:at[s]])


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,hd,vd,v_off", [(3, 8, 5, 16), (2, 32, 24, 64), (1, 16, 16, 8)])
def test_short_convolution_keeps_and_mixes_values(dtype, heads, hd, vd, v_off):
    """Value heads of 5 real coordinates laid out in 8 (and sizes that the kernel of eight channels a thread
    takes): the first layer's results are kept as rows of real coordinates, a later layer's are mixed with them;
    the other channels and the padding are left alone."""
    from ccinfer_b200 import kernels
    dev = "cuda"
    g = torch.Generator().manual_seed(5)
    T, taps = 6, 2
    C = v_off + heads * hd
    w = torch.randn(C, taps, generator=g)
    u1, u2 = torch.randn(T, C, generator=g).to(dtype), torch.randn(T, C, generator=g).to(dtype)
    lam = torch.tensor([0.3])
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    eot = torch.zeros(T, dtype=torch.int32, device=dev)
    slot = torch.zeros(1, dtype=torch.int32, device=dev)
    first = torch.zeros(T, heads * vd, dtype=dtype, device=dev)
    y1, y2 = torch.empty(T, C, dtype=dtype, device=dev), torch.empty(T, C, dtype=dtype, device=dev)
    for u, y, l in ((u1, y1, None), (u2, y2, lam.to(dev))):
        state = torch.zeros(1, taps - 1, C, dtype=dtype, device=dev)
        kernels.conv_rows(y, u.to(dev), w.t().contiguous().to(dev), taps, C, state, eot, cu, slot, 1,
                          values=(v_off, heads, hd, vd, first, l))
    c1, c2 = plain.short_conv(u1.double(), w.double()), plain.short_conv(u2.double(), w.double())
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (y1.double().cpu() - c1).abs().max() < tol * 4
    real = torch.tensor([v_off + h * hd + e for h in range(heads) for e in range(vd)])
    assert (first.double().cpu() - c1[:, real]).abs().max() < tol * 4
    want = c2.clone()
    want[:, real] = 0.7 * c2[:, real] + 0.3 * first.double().cpu()
    assert (y2.double().cpu() - want).abs().max() < tol * 4


@gpu
@pytest.mark.parametrize("E,groups,keep,top,scale", [(16, 4, 3, 4, 2.0), (8, 2, 1, 2, 1.0), (6, 3, 2, 3, 0.5),
                                                     (5, 1, 1, 2, 1.0), (64, 8, 4, 8, 2.5), (12, 4, 4, 1, 1.0),
                                                     (3, 1, 1, 3, 1.0), (6, 6, 3, 2, 1.5), (12, 3, 1, 4, 1.0)])
def test_router_rule(E, groups, keep, top, scale):
    """Sigmoid scores, a group's score the sum of its two best (its one score where a group is one expert), the
    chosen scores divided by their sum and multiplied by the router's scale."""
    from ccinfer_b200 import kernels
    g = torch.Generator().manual_seed(E * 100 + top)
    T = 60
    z = 2 * torch.randn(T, E, generator=g)
    r = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}
    idx, w = plain.route(z.double(), r)
    if groups > 1 and keep < groups and E // groups > 1:
        # the rule differs from "a group's best score" for some token of the draw
        one = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}
        s = torch.sigmoid(z.double()).view(T, groups, -1)
        by_max = s.max(-1).values.topk(keep, dim=-1).indices.sort(-1).values
        by_two = s.topk(2, dim=-1).values.sum(-1).topk(keep, dim=-1).indices.sort(-1).values
        assert not torch.equal(by_max, by_two)
    rule = kernels.RouteRule("sigmoid", 2, renorm=True, scale=scale)
    di = torch.empty(T, top, dtype=torch.int32, device="cuda")
    dw = torch.empty(T, top, device="cuda")
    dense = torch.empty(T, E, device="cuda")
    kernels.moe_route(z.cuda(), None, di, dw, dense, groups, keep, rule=rule)
    assert torch.equal(di.cpu().long(), idx)
    assert (dw.cpu().double() - w).abs().max() < 1e-6 * max(1.0, scale)
    want = torch.zeros(T, E, dtype=torch.float64).scatter_(1, idx, w)
    assert (dense.cpu().double() - want).abs().max() < 1e-6 * max(1.0, scale)
    assert (dw.sum(-1).cpu() - scale).abs().max() < 1e-5 * scale


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sparse", [False, True])
@pytest.mark.parametrize("E,top,F,D,groups,SF,scale", [(8, 2, 64, 64, (4, 2), 32, 2.0), (16, 4, 32, 128, None, 0, 1.0),
                                                       (5, 5, 8, 40, None, 8, 0.5), (4, 2, 6, 22, (2, 1), 10, 1.0),
                                                       (12, 3, 48, 96, (3, 2), 80, 1.5)])
def test_gated_experts_alone(dtype, sparse, E, top, F, D, groups, SF, scale):
    """The mixture by itself, in both of its forms, from one token to so many that an expert's rows fill several
    tiles of every size; the shared expert behind its gate."""
    from ccinfer_b200 import kernels
    from ccinfer_b200.engine.runtime import Runtime
    from ccinfer_b200.parts import MixtureOfExperts
    rt = Runtime("cuda:0", dtype, 640, 4)
    m = plain.experts(E, top, F, groups=groups, scale=scale, shared=SF or None)
    g = torch.Generator().manual_seed(E + F)
    W = {"router": 3 * torch.randn(E, D, generator=g) / math.sqrt(D)}
    for e in range(E):
        W[f"e{e}.gate"] = 2 * torch.randn(F, D, generator=g) / math.sqrt(D)
        W[f"e{e}.up"] = torch.randn(F, D, generator=g) / math.sqrt(D)
        W[f"e{e}.down"] = torch.randn(D, F, generator=g) / math.sqrt(F)
    if SF:
        W["shared.gate"], W["shared.up"] = 2 * torch.randn(SF, D, generator=g) / math.sqrt(D), torch.randn(SF, D, generator=g) / math.sqrt(D)
        W["shared.down"], W["shared.sg"] = torch.randn(D, SF, generator=g) / math.sqrt(SF), 3 * torch.randn(1, D, generator=g) / math.sqrt(D)
    W = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    names = {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down",
             "shared_gate_proj": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down",
             "shared_gate": "shared.sg"}
    part = MixtureOfExperts(D, E, top, F, names, *(groups or (1, 1)), SF, activation="swiglu", sparse=sparse,
                            rule=kernels.RouteRule("sigmoid", 2, renorm=True, scale=scale))
    part.bind(rt, lambda n: W[n].cuda().to(dtype) if W[n].dim() == 2 else W[n].cuda())
    # (the grouped products of the bfloat16 path want 16-byte rows; other sizes run the dense form)
    assert part.use_sparse == (sparse and (dtype == torch.float32 or (D % 8 == 0 and F % 8 == 0)))
    for T in (1, 5, 70, 300, 640):
        x = torch.randn(T, D, generator=g).to(torch.bfloat16)
        want = plain.moe(x.double(), {k: v.double() for k, v in W.items()}, "", m)
        got = part.forward(x.cuda().to(dtype), None).double().cpu()
        err = (got - want).abs().amax(-1) / want.abs().max()
        tol = 2e-6 if dtype == torch.float32 else 1.5e-2
        # (in bfloat16 a router's close call may go the other way for a token or two)
        assert (err > tol).sum() <= (0 if dtype == torch.float32 else max(1, T // 50)), (T, err.max())
    rt.check_status()


# ---------------------------------------------------------------------------------------------
# GPU: one attention layer with each option, then whole models under every cutting
# ---------------------------------------------------------------------------------------------
SINGLE = {
    "bare": plain.attn(2, 2, 16, 16, 0.25),
    "convolution": plain.attn(2, 1, 16, 16, 0.25, conv=3),
    "rotation of a part": plain.attn(4, 2, 16, 16, 0.25, rot=(6, 30.0)),
    "chunks": plain.attn(2, 1, 16, 16, 0.25, chunk=7),
    "values larger than keys": plain.attn(3, 1, 8, 40, 0.35),
    "keys larger than values": plain.attn(2, 2, 72, 8, 0.12, rot=(72, 1000.0), chunk=11),
    "everything": plain.attn(6, 2, 24, 20, 0.2, conv=2, rot=(12, 100.0), chunk=13),
    # head sizes of the tensor-core kernels (bfloat16): pairs of heads of a group, one head a group, heads of 64
    "heads of 128 in groups of four": plain.attn(4, 1, 128, 128, 0.09, rot=(64, 1000.0), chunk=130),
    "heads of 128 alone": plain.attn(3, 3, 112, 128, 0.1, conv=2, rot=(112, 1000.0), chunk=37),
    "heads of 64": plain.attn(4, 2, 64, 48, 0.125, conv=3, rot=(32, 100.0), chunk=64),
}
LONG_KINDS = [k for k in SINGLE if k.startswith("heads of")]


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", list(SINGLE))
def test_one_attention_layer_with_each_option(tmp_path, kind, dtype):
    """Sink and head gate are in every layer; here they are made large enough to matter (sinks around the scores'
    size, gates far from one half)."""
    cfg = plain.model(50, 40, 1e-5, [(SINGLE[kind], None)])
    d = str(tmp_path / "m")

    def edit(w):
        w["l0.mix.sink"] = w["l0.mix.sink"] * 2.0 + 1.0
        w["l0.mix.g"] = w["l0.mix.g"] * 3.0

    cfg, w = write_model(d, cfg=cfg, seed=3, sharp=SHARP[dtype], edit=edit)
    # (the long prompts fill several tiles of 128 queries and end just past a chunk's edge)
    reqs = requests_of(cfg, [1, 2, 31, 50] + ([131, 300] if kind in LONG_KINDS else []), 1)
    ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    eng = engine_of(d, dtype, 8, 640)
    for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=64),
                  helpers.trace_portions(reqs, sizes=(2, 5, 3, 2, 11, 70, 140)),
                  helpers.trace_mixed(reqs, max_live=4, seed=3)):
        rows = helpers.replay(eng, steps)
        worst = compare(rows, ref, dtype, f"{kind} {dtype}")
        print(f"[worst] one layer, {kind}, {dtype}: {worst:.3e}")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_values_mixed_with_the_first_layers(tmp_path, dtype):
    """Three layers that mix values; the factors are made unequal and far from zero, and the plain result must
    differ visibly from the one without mixing, so that the comparison says something."""
    m = plain.attn(4, 2, 16, 24, 0.25, conv=2, chunk=40, v_mix=True)
    cfg = plain.model(60, 48, 1e-5, [(plain.attn(4, 2, 16, 24, 0.25), None), (m, None), (m, None), (m, None)])
    d = str(tmp_path / "m")

    def edit(w):
        w["l1.mix.vmix"] = torch.tensor(0.9)        # the first such layer: unused
        w["l2.mix.vmix"] = torch.tensor(0.75)
        w["l3.mix.vmix"] = torch.tensor(0.4)

    cfg, w = write_model(d, cfg=cfg, seed=5, sharp=SHARP[dtype], edit=edit)
    reqs = requests_of(cfg, [1, 2, 19, 64], 2)
    ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    unmixed = dict(w)
    unmixed["l2.mix.vmix"] = unmixed["l3.mix.vmix"] = torch.tensor(0.0)
    far = plain.forward(cfg, unmixed, reqs["r3"]).numpy()
    assert np.abs(far - ref["r3"]).max() > 0.1 * np.abs(ref["r3"]).max()
    eng = engine_of(d, dtype, 16, 256)
    for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=10 ** 6),
                  helpers.trace_mixed(reqs, max_live=3, seed=2)):
        compare(helpers.replay(eng, steps), ref, dtype, f"value mixing {dtype}")


# lengths just below, at and just above every chunk's and page's border of the configuration
LENGTHS = {"A": [1, 2, 23, 24, 25, 26, 48, 49, 97], "B": [1, 3, 8, 9, 10, 11, 30, 31, 59],
           "C": [2, 32, 33, 34, 35, 66, 67, 70, 71, 141], "D": [1, 4, 5, 6, 16, 17, 99, 100, 101, 201]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in plain.CONFIGS:
        for dtype, sharp in SHARP.items():
            d = str(tmp_path_factory.mktemp("bur" + name))
            cfg, w = write_model(d, name, seed=ord(name), sharp=sharp)
            reqs = requests_of(cfg, LENGTHS[name], 2)
            ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
            out[name, dtype] = (d, cfg, w, reqs, ref, plain.CONFIGS[name][1])
    return out


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(plain.CONFIGS))
@pytest.mark.parametrize("mode", ["whole", "decode from the first token", "decode40", "portions", "mixed"])
def test_replay_matches_plain(models, name, dtype, mode):
    """Prompt lengths sit just below, at and just above every chunk and page border, and the attention is sharp
    (queries times three in the 32-bit runs), so a key one place off shows."""
    d, cfg, w, reqs, ref, page = models[name, dtype]
    if mode == "whole":
        steps = helpers.trace_whole(reqs)
    elif mode == "decode from the first token":
        steps = helpers.trace_prefill_then_decode(reqs, tail=10 ** 6)
    elif mode == "decode40":
        steps = helpers.trace_prefill_then_decode(reqs, tail=40)
    elif mode == "portions":
        steps = helpers.trace_portions(reqs)
    else:
        steps = helpers.trace_mixed(reqs, max_live=4, seed=5)
    pool = helpers.max_live_tokens(steps, round_to=max(64, page))
    eng = engine_of(d, dtype, page, pool, max_requests=4)
    rows = helpers.replay(eng, steps)
    assert len(rows) == sum(len(t) for t in reqs.values())
    worst = compare(rows, ref, dtype, f"{name} {dtype} {mode}")
    print(f"[worst] {name}, {dtype}, {mode}: {worst:.3e}")
    eng.cache.check_consistency()
    assert all(p.used_pages == 0 for p in eng.cache.pools)
    assert eng.cache.slots.free_slots == 4


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_and_graphs(models, dtype):
    """Portions of more than 64 and more than 128 tokens after a cached prefix (they start and end inside chunks)
    beside decode steps replayed from CUDA graphs."""
    d, cfg, w, reqs, ref, page = models["C", dtype]
    rng = np.random.RandomState(3)
    reqs = {f"L{i}": rng.randint(0, cfg["vocab"], size=n).tolist() for i, n in enumerate((300, 181, 260, 75))}
    ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    steps = helpers.trace_mixed(reqs, max_live=3, seed=13, prefill_frac=0.8, portion_choices=(70, 130, 65, 2, 100))
    pool = helpers.max_live_tokens(steps, round_to=64)
    eng = engine_of(d, dtype, page, pool, max_requests=4, use_graphs=True)
    rows = helpers.replay(eng, steps)
    worst = compare(rows, ref, dtype, f"C {dtype} long portions, graphs")
    print(f"[worst] C, {dtype}, long portions, graphs: {worst:.3e}")
    assert eng.graph_replays > 0


@gpu
def test_a_slot_that_is_used_again_starts_from_zero(models):
    """Two state slots, five requests one after another and in pairs: every later request gets a slot whose
    convolution rows an earlier one left behind, and pages that held another request's keys."""
    d, cfg, w, reqs, ref, page = models["A", "float32"]
    eng = engine_of(d, "float32", page, 256, max_requests=2)
    ids = list(reqs)[3:8]
    for group in ([ids[0]], [ids[1], ids[2]], [ids[3], ids[4]]):
        steps = helpers.trace_mixed({r: reqs[r] for r in group}, max_live=2, seed=1)
        compare(helpers.replay(eng, steps), ref, "float32", "slots used again")
    assert eng.cache.slots.free_slots == 2


# ---------------------------------------------------------------------------------------------
# GPU: inputs made so that one key, or the sink, decides
# ---------------------------------------------------------------------------------------------
def marker_model(path, chunk):
    """One layer.  Queries and keys read the first half of the stream (both query heads have the key projection's
    rows, the convolutions pass the newest row through), values the second half, and tokens 0 and 1
    have the same first half: the query of token 1 matches the key of token 0 as well as its own (a score of 32
    against a spread of 6 for any other) and hardly any other key.  The rotated coordinates of the heads are left
    out of the match (their rows of the projections are zero: a rotation by a far distance would take several
    units off the marker's score), and token 0's value is three times the others' size."""
    cfg = plain.model(64, 64, 1e-5, [(plain.attn(2, 1, 32, 32, 1.0, conv=3, rot=(4, 10000.0), chunk=chunk), None)])

    def edit(w):
        w["l0.norm1"] = torch.ones_like(w["l0.norm1"])
        w["l0.mix.k"][:, 32:] = 0
        w["l0.mix.k"][:4] = 0
        w["l0.mix.v"][:, :32] = 0
        w["l0.mix.q"] = torch.cat([w["l0.mix.k"], w["l0.mix.k"]])
        w["l0.mix.q.norm"] = torch.ones_like(w["l0.mix.q.norm"])
        w["l0.mix.k.norm"] = torch.ones_like(w["l0.mix.k.norm"])
        for t in ("q", "k", "v"):
            w[f"l0.mix.{t}.conv"] = torch.zeros_like(w[f"l0.mix.{t}.conv"])
            w[f"l0.mix.{t}.conv"][:, -1] = 1.0
        w["l0.mix.g"] = torch.zeros_like(w["l0.mix.g"])
        w["embed"][1, :32] = w["embed"][0, :32]
        w["embed"][0, 32:] *= 3.0

    return write_model(path, cfg=cfg, seed=8, edit=edit)


def marker_case(d, cfg, w, length, marker_at, decides, cuts):
    """Token 0 at ``marker_at``, token 1 last.  ``decides``: whether the last query sees the marker."""
    rng = np.random.RandomState(length + marker_at)
    toks = rng.randint(2, 64, size=length).tolist()
    toks[marker_at], toks[-1] = 0, 1
    ref = plain.forward(cfg, w, toks).numpy()
    without = plain.forward(cfg, w, toks[:marker_at] + [2] + toks[marker_at + 1:]).numpy()
    moved = np.abs(ref[-1] - without[-1]).max() / np.abs(ref[-1]).max()
    assert (moved > 0.15) if decides else (moved < 1e-9), (length, marker_at, moved)
    reqs = {"a": toks}
    for dtype in ("float32", "bfloat16"):
        eng = engine_of(d, dtype, 8, -(-length // 64) * 64 + 64)
        for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=3),
                      helpers.trace_prefill_then_decode(reqs, tail=length - marker_at + 2),
                      helpers.trace_portions(reqs, sizes=cuts)):
            rows = helpers.replay(eng, steps)
            helpers.compare(rows, {"a": ref}, TOL32 if dtype == "float32" else TOL16,
                            f"marker at {marker_at} of {length}, {dtype}")


@gpu
def test_a_far_key_decides(tmp_path):
    """The marker stands at ONE far place among 300 (the first token, the last of a page, the first of the next,
    the middle) in a chunk that holds them all: dropping or misplacing its key would change the last logits by
    their own size.  The marker is in the prompt, or (last cutting but one) decoded itself."""
    d = str(tmp_path / "far")
    cfg, w = marker_model(d, 512)
    for far_at in (0, 7, 8, 150):
        marker_case(d, cfg, w, 300, far_at, True, (150, 2, 100, 47, 1))


@gpu
def test_keys_just_inside_and_just_outside_a_chunk(tmp_path):
    """Chunks of 50 positions over pages of 8.  The marker at the first position of the last query's chunk
    decides; one place earlier it is not seen, and a mask one position off would let it in.  The last query is
    the last of its chunk, the first of the next (which sees itself alone), or in the middle; it is part of a
    prompt, of a portion that starts inside the chunk, or decoded alone."""
    d = str(tmp_path / "edge")
    cfg, w = marker_model(d, 50)
    cuts = (97, 2, 2, 30, 2, 17, 1, 1)
    for length, marker_at, decides in ((120, 100, True), (120, 99, False), (150, 100, True), (150, 99, False),
                                       (151, 149, False), (151, 100, False), (102, 100, True), (101, 99, False),
                                       (50, 0, True), (51, 0, False), (300, 250, True), (300, 249, False)):
        marker_case(d, cfg, w, length, marker_at, decides, cuts)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sink_that_decides(tmp_path, dtype):
    """Sinks well above the scores: most of every softmax's weight goes to the sink and the mixer's output
    shrinks accordingly; without the sink the logits would differ by their own size."""
    cfg = plain.model(40, 32, 1e-5, [(plain.attn(4, 2, 16, 16, 0.1, conv=2, chunk=20), None),
                                     (plain.attn(4, 1, 16, 16, 0.1), plain.dense(48))])
    d = str(tmp_path / "sink")

    def edit(w):
        w["l0.mix.sink"] = torch.tensor([3.0, -2.0, 5.0, 1.0])
        w["l1.mix.sink"] = torch.tensor([4.0, 4.5, -1.0, 6.0])

    cfg, w = write_model(d, cfg=cfg, seed=11, edit=edit)
    reqs = requests_of(cfg, [1, 2, 20, 21, 45], 4)
    ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    no_sink = {k: (torch.full_like(v, -60.0) if k.endswith(".sink") else v) for k, v in w.items()}
    other = plain.forward(cfg, no_sink, reqs["r4"]).numpy()
    assert np.abs(other - ref["r4"]).max() > 0.2 * np.abs(ref["r4"]).max()
    eng = engine_of(d, dtype, 8, 192)
    for steps in (helpers.trace_whole(reqs), helpers.trace_prefill_then_decode(reqs, tail=10 ** 6),
                  helpers.trace_mixed(reqs, max_live=4, seed=7)):
        compare(helpers.replay(eng, steps), ref, dtype, f"sink {dtype}")


@gpu
def test_long_decoding(models):
    """260 tokens one by one: the runs of 24 (and of 5, 100 and 1) positions pass many times, their pages are
    given back behind them."""
    rng = np.random.RandomState(9)
    for name in ("A", "D"):
        for dtype in ("float32", "bfloat16"):
            d, cfg, w, reqs, ref, page = models[name, dtype]
            toks = rng.randint(0, cfg["vocab"], size=260).tolist()
            want = plain.forward(cfg, w, toks).numpy()
            eng = engine_of(d, dtype, page, 320, use_graphs=(dtype == "bfloat16"))
            rows = helpers.replay(eng, helpers.trace_prefill_then_decode({"a": toks}, tail=10 ** 6))
            worst = compare(rows, {"a": want}, dtype, f"long decoding {name} {dtype}")
            print(f"[worst] long decoding, {name}, {dtype}: {worst:.3e}")


# ---------------------------------------------------------------------------------------------
# GPU: the entry point, its scheduler, the programs
# ---------------------------------------------------------------------------------------------
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    """Prompts of unequal length in portions of 7 through ``LLM.generate`` and its scheduler."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, reqs, ref, page = models["A", dtype]
    rng = np.random.RandomState(4)
    prompts = [rng.randint(0, cfg["vocab"], size=n).tolist() for n in (1, 9, 20, 33)]
    llm = LLM(d, dtype=dtype, page_size=page, kv_tokens=512, prefill_chunk_size=7, max_requests=4,
              max_tokens_per_step=64)
    got = llm.generate(prompts, SamplingParams(max_tokens=30))
    if dtype == "float32":
        assert got == [plain.greedy(cfg, w, p, 30) for p in prompts]
    else:
        # rounding may flip an argmax between two close logits, and a router's close call moves a row by the size
        # of an expert's output (see ``compare``): nearly every token must be (nearly) the best one after the
        # tokens before it
        off = 0
        for p, new in zip(prompts, got):
            toks = list(p)
            for t in new:
                row = plain.forward(cfg, w, toks)[-1]
                off += bool(row[t] < row.max() - 0.05 * row.abs().max())
                toks.append(t)
        assert off <= sum(len(new) for new in got) // 25, off
    assert all(pool.used_pages == 0 for pool in llm.engine.cache.pools)


@gpu
def test_a_preempted_request_starts_its_state_again(models):
    """So few pages that a request is preempted and computed again (its slot is closed and opened: the
    convolution's rows start from zero): the greedy tokens are those of a calm run."""
    from ccinfer_b200 import LLM, SamplingParams
    d, cfg, w, reqs, ref, page = models["B", "float32"]
    rng = np.random.RandomState(6)
    prompts = [rng.randint(0, cfg["vocab"], size=n).tolist() for n in (20, 26, 17)]
    llm = LLM(d, dtype="float32", page_size=page, kv_tokens=14 * page, prefill_chunk_size=16, max_requests=4,
              max_tokens_per_step=64)
    got = llm.generate(prompts, [SamplingParams(max_tokens=n) for n in (24, 20, 28)])
    assert llm.scheduler.preemptions > 0
    assert got == [plain.greedy(cfg, w, p, n) for p, n in zip(prompts, (24, 20, 28))]
    llm.engine.cache.check_consistency()


@gpu
def test_the_programs_as_a_user_calls_them(models, tmp_path):
    """bin/ccinfer: greedy tokens of a model folder, and a random model written from a configuration that
    generates the same tokens as the same configuration drawn on the device; bin/trace_run: a mixed trace over
    four request slots, in both types, its files against the plain logits."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, cfg, w, reqs, ref, page = models["A", "float32"]
    exe = [sys.executable, os.path.join(root, "bin", "ccinfer")]
    prompt = list(reqs.values())[4]
    r = subprocess.run(exe + ["--model-path", d, "--dtype", "float32", "--page-size", str(page), "--kv-tokens", "256",
                              "--max-tokens", "6", "--prompt-ids", ",".join(map(str, prompt))],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[0])["token_ids"] == plain.greedy(cfg, w, prompt, 6)

    cj = str(tmp_path / "config.json")
    with open(cj, "w") as f:
        json.dump(cfg, f)
    common = ["--dtype", "float32", "--kv-tokens", "256", "--max-tokens", "5", "--random-prompts", "9,4",
              "--weights-seed", "5", "--weights-std", "0.3"]
    a = subprocess.run(exe + ["--random-config", cj] + common, capture_output=True, text=True, timeout=600)
    assert a.returncode == 0, a.stderr[-2000:]
    made = str(tmp_path / "made")
    wr = subprocess.run(exe + ["--model-path", made, "--write-random-model", cj, "--weights-seed", "5",
                               "--weights-std", "0.3", "--store-dtype", "float32"], capture_output=True, text=True,
                        timeout=600)
    assert wr.returncode == 0, wr.stderr[-2000:]
    b = subprocess.run(exe + ["--model-path", made] + common, capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-2000:]
    assert a.stdout == b.stdout and len(a.stdout.strip().splitlines()) == 2

    steps = helpers.trace_mixed(reqs, max_live=4, seed=3)
    pool = helpers.max_live_tokens(steps)
    lines = "".join(json.dumps({"step": i, **st}) + "\n" for i, st in enumerate(steps))
    for dtype in ("float32", "bfloat16"):
        out_dir = tmp_path / ("out_" + dtype)
        dd, _, _, _, dref, _ = models["A", dtype]
        dreqs = models["A", dtype][3]
        assert dreqs == reqs
        t = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", dd, "--dtype", dtype, "--out",
                            str(out_dir), "--max-tokens", str(pool)], input=lines, capture_output=True, text=True,
                           timeout=600)
        assert t.returncode == 0, t.stderr[-2000:]
        assert t.stdout.split() == [x for i in range(len(steps)) for x in ("done", str(i))]
        rows, seen = {}, {rid: 0 for rid in reqs}
        for i, st in enumerate(steps):
            n_want = sum(len(e["want"]) for e in st["entries"])
            arr = np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(n_want, cfg["vocab"])
            at = 0
            for e in st["entries"]:
                for wnt in e["want"]:
                    rows[(e["id"], seen[e["id"]] + wnt)] = arr[at]
                    at += 1
                seen[e["id"]] += len(e["tokens"])
        assert len(rows) == sum(len(x) for x in reqs.values())
        compare(rows, dref, dtype, "trace_run " + dtype)


# ---------------------------------------------------------------------------------------------
# GPU: configurations drawn at random
# ---------------------------------------------------------------------------------------------
def draw_config(seed):
    """Every size, option and constant that a configuration may state, drawn at random: widths and vocabularies
    that are multiples of nothing, any number of heads and groups, key and value sizes from 4 to 130 (often the
    sizes of the tensor-core kernels), any order of dense, mixture and absent feed-forwards, taps from none to
    five, rotations of none, a part or all of a head, runs from one position to beyond the prompts, layers that
    mix values or not, routers with and without groups, scales and shared experts, with and without a side
    input and a scale of the logits.  Key-value heads and the value size are one per model (mixed values must
    have one shape)."""
    rng = np.random.RandomState(7000 + seed)
    width = int(rng.choice([int(rng.randint(20, 150)), 64, 96, 128]))
    vocab = int(rng.randint(40, 260))
    G = int(rng.choice([1, 2, 3, 4]))
    fast = rng.rand() < 0.5
    vdim = int(rng.choice([64, 128])) if fast else int(rng.randint(2, 66)) * 2
    layers = []
    for _ in range(int(rng.randint(1, 6))):
        H = G * int(rng.choice([1, 2, 3, 4, 6]))
        if fast:
            dim = int(rng.choice([d for d in (32, 48, 64, 112, 128) if -(-max(d, vdim) // 16) * 16 in (64, 128)]))
        else:
            dim = int(rng.randint(2, 66)) * 2
        rot = None
        if rng.rand() < 0.8:
            rot = (int(rng.choice([2, dim // 2 // 2 * 2 or 2, dim])), float(rng.choice([20.0, 1000.0, 50000.0])))
            rot = (min(rot[0], dim), rot[1])
        mixer = plain.attn(H, G, dim, vdim, float(dim ** -0.5 * rng.uniform(0.7, 1.5)),
                           conv=[None, 1, 2, 3, 4, 5][int(rng.randint(6))], rot=rot,
                           chunk=[None, 1, int(rng.randint(2, 20)), int(rng.randint(20, 90)), 500][int(rng.randint(5))],
                           v_mix=bool(rng.rand() < 0.6))
        kind = int(rng.randint(4))
        if kind == 0:
            mlp = None
        elif kind == 1:
            mlp = plain.dense(int(rng.randint(8, 120)))
        else:
            count = int(rng.choice([1, 2, 3, 4]))
            per = int(rng.randint(1, 5))
            keep = int(rng.randint(1, count + 1))
            top = int(rng.randint(1, per * keep + 1))
            mlp = plain.experts(count * per, top, int(rng.randint(1, 9)) * 8,
                                groups=(count, keep) if rng.rand() < 0.7 or keep < count else None,
                                scale=float(rng.uniform(0.5, 3.0)) if rng.rand() < 0.6 else None,
                                shared=int(rng.randint(1, 9)) * 8 if rng.rand() < 0.6 else None)
        layers.append((mixer, mlp))
    cfg = plain.model(vocab, width, float(rng.choice([1e-5, 1e-6])), layers,
                      side=int(rng.randint(1, 20)) if rng.rand() < 0.6 else None,
                      logit_scale=float(rng.choice([0.5, 2.0, 1.7])) if rng.rand() < 0.6 else None)
    page = int(rng.choice([8, 16, 32] if fast else [4, 8, 16]))
    lengths = [1, 2] + [int(rng.randint(3, 140)) for _ in range(5)] + ([int(rng.randint(140, 300))] if fast else [])
    return cfg, page, lengths


FUZZ_SEEDS = int(os.environ.get("CCB_FUZZ_SEEDS", "10"))


@gpu
@pytest.mark.parametrize("seed", range(FUZZ_SEEDS))
def test_random_configurations(tmp_path, seed):
    """A mixed trace over four request slots with a pool that is just large enough, then every request whole, in
    32-bit and in bfloat16, against the plain implementation.  Drawn models have rows that magnify any rounding
    a thousandfold (a side input of one or two columns is normalised whatever its size; a sharp softmax between
    two equal keys), so the 32-bit bound of a row grows with how far that row moves in the plain implementation
    when every weight is changed by a millionth."""
    cfg, page, lengths = draw_config(seed)
    for dtype in ("float32", "bfloat16"):
        d = str(tmp_path / dtype)
        cfg, w = write_model(d, cfg=cfg, seed=seed, sharp=SHARP[dtype])
        reqs = requests_of(cfg, lengths, seed)
        ref = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
        steps = helpers.trace_mixed(reqs, max_live=4, seed=seed)
        whole = helpers.trace_whole(reqs)
        pool = max(helpers.max_live_tokens(steps, round_to=max(64, page)),
                   helpers.max_live_tokens(whole, round_to=max(64, page)))
        eng = engine_of(d, dtype, page, pool, max_requests=4)
        if dtype == "float32":
            gen = torch.Generator().manual_seed(seed)
            moved = {k: v.double() * (1 + 1e-6 * torch.randn(v.shape, dtype=torch.float64, generator=gen))
                     for k, v in w.items()}
            bound = {}
            for rid, t in reqs.items():
                scale = max(1e-6, float(np.abs(ref[rid]).max()))
                bound[rid] = TOL32 + 10 * np.abs(plain.forward(cfg, moved, t).numpy() - ref[rid]).max(1) / scale
        for trace in (steps, whole):
            rows = helpers.replay(eng, trace)
            assert len(rows) == sum(len(t) for t in reqs.values())
            what = f"random configuration {seed} {dtype}: {json.dumps(cfg)}"
            if dtype == "float32":
                for (rid, pos), row in rows.items():
                    err = float(np.abs(row - ref[rid][pos]).max()) / max(1e-6, float(np.abs(ref[rid]).max()))
                    assert np.isfinite(row).all() and err <= bound[rid][pos], \
                        f"{what}: relative error {err:.3e} at {rid}, {pos} beyond {bound[rid][pos]:.3e}"
            else:
                compare(rows, ref, dtype, what)
        assert all(p.used_pages == 0 for p in eng.cache.pools)
