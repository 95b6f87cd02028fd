"""Nulezen on the GPU against the plain restatement in ``nulezen_oracle.py``: every mechanism alone, then whole models of several
shapes through prefill, decoding, portions, ragged batches, reused slots and the generation entry points."""
from __future__ import annotations

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import nulezen_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def K():
    from lit_gpt_b200 import kernels

    return kernels


# ---------------------------------------------------------------------------------------------------------
# configurations and random checkpoints
# ---------------------------------------------------------------------------------------------------------
def attn(heads, kv_heads, dim, vdim, size, scale=None):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=size), scale=scale if scale is not None else dim ** -0.5)


def attn2(heads, kv_heads, dim, vdim, size, rot_dims, base=100.0, scale=None):
    m = attn(heads, kv_heads, dim, vdim, size, scale)
    m["rot"] = dict(base=base, dims=rot_dims)
    return m


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))
    if shared is not None:
        m["shared"] = dict(ff=shared[0], limit=shared[1])
    return m


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def config(width, vocab, layers, loop=None, emb=2.0, logit=0.7):
    cfg = dict(architecture="Nulezen", embedding=dict(scale=emb), layers=layers, logit_scale=logit, norm=dict(eps=1e-5), vocab=vocab, width=width)
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


# odd sizes on purpose: a width no vector access fits, grouped heads, key size != value size, a layer without feed-forward, experts
# with and without a shared expert (whose size differs from theirs), a rotation of part of the head, the middle two layers run three times
CFG_ODD = config(width=42, vocab=83, loop=(1, 3, 3), layers=[
    layer("attention", attn(4, 2, 12, 10, size=7, scale=0.9), dense(50)),
    layer("attention_2", attn2(6, 3, 10, 6, size=5, rot_dims=6), moe(6, 2, 14, 1.2, shared=(22, 0.8))),
    layer("attention", attn(2, 1, 16, 12, size=3), None),
    layer("attention_2", attn2(1, 1, 20, 9, size=33, rot_dims=20, base=50.0), moe(5, 3, 11, 0.9)),
])
# heads wider than one value chunk of the attention tile (> 128), a window of one position, a window longer than any prompt here, one
# expert per token, every expert for every token, no loop at all, a model without embedding or logit scale
CFG_WIDE = config(width=64, vocab=120, emb=1.0, logit=1.0, layers=[
    layer("attention", attn(2, 2, 72, 136, size=1), dense(96)),
    layer("attention_2", attn2(3, 1, 24, 24, size=300, rot_dims=8, base=1e4, scale=0.35), moe(4, 1, 40, 2.0, shared=(24, 1.5))),
    layer("attention", attn(4, 4, 16, 16, size=33), moe(8, 8, 24, 1.1)),
])
# head sizes the tensor-core prompt kernel takes in bf16 (64 and 128, grouped and not), a window that ends inside a key tile, a
# loop that starts at the first layer and leaves the last one out
CFG_TILES = config(width=96, vocab=140, loop=(0, 2, 2), layers=[
    layer("attention", attn(4, 2, 64, 64, size=44), moe(8, 3, 48, 1.4, shared=(64, 1.0))),
    layer("attention_2", attn2(2, 1, 128, 128, size=100, rot_dims=64, base=1e4, scale=0.2), dense(200)),
    layer("attention_2", attn2(4, 4, 64, 64, size=70, rot_dims=64, base=2e5), None),
])


def checkpoint(cfg, seed):
    """Random bf16 weights of a size that keeps every mechanism alive (clamps that fire, gates away from 0 and 1, a distance bias that
    matters, a loop entry that mixes stream and embedding)."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    d = cfg["width"]
    w = {"embed": rnd(cfg["vocab"], d, std=0.6)}

    def put_norm(name):
        w[name], w[name + ".b"], w[name + ".alpha"] = rnd(d, std=0.2, mean=1.0), rnd(d, std=0.1), rnd(1, std=0.1, mean=0.6).reshape(())

    put_norm("final.norm")
    loop = cfg.get("loop")
    if loop:
        eye = torch.eye(d)
        w["loop.in"] = (torch.cat([0.8 * eye, 0.4 * eye], dim=1) + torch.randn(d, 2 * d, generator=g) * 0.3 * d ** -0.5).to(torch.bfloat16)
        w["loop.step"] = rnd(loop["times"], d, std=0.3)
    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        put_norm(p + "norm1")
        w[p + "ls1"] = rnd(d, std=0.3, mean=1.0)
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        second = ly["type"] == "attention_2"
        for name, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
            w[p + "mix." + name] = rnd(rows, d, std=1.5 * d ** -0.5)
            if second:
                w[p + "mix." + name + ".b"] = rnd(rows, std=0.3)
        w[p + "mix.g"] = rnd(H if second else H * dv, d, std=2.0 * d ** -0.5)
        if not second:
            w[p + "mix.r1"] = (0.4 + 0.4 * torch.rand(H, generator=g)).to(torch.bfloat16)
            w[p + "mix.r2"] = (0.2 + torch.rand(H, generator=g)).to(torch.bfloat16)
        w[p + "mix.o"] = rnd(d, H * dv, std=(H * dv) ** -0.5)
        f = ly["mlp"]
        if f is None:
            continue
        w[p + "ls2"] = rnd(d, std=0.3, mean=1.0)
        if f["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.down"] = rnd(f["ff"], d, std=d ** -0.5), rnd(d, f["ff"], std=f["ff"] ** -0.5)
            w[p + "mlp.act"] = rnd(2, std=0.8)
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"], w[p + "mlp.router.b"] = rnd(E, d, std=2.0 * d ** -0.5), rnd(E, std=0.5)
            names = [(f"e{e}.", ff) for e in range(E)] + ([("shared.", f["shared"]["ff"])] if f.get("shared") else [])
            for nm, n in names:
                w[f"{p}mlp.{nm}gate"], w[f"{p}mlp.{nm}up"] = rnd(n, d, std=1.5 * d ** -0.5), rnd(n, d, std=1.5 * d ** -0.5)
                w[f"{p}mlp.{nm}down"] = rnd(d, n, std=n ** -0.5)
    return w


def build(cfg, weights, dtype, slots=2):
    from lit_gpt_b200.config import NulezenConfig
    from lit_gpt_b200.nulezen import Nulezen

    model = Nulezen(NulezenConfig.from_dict(cfg)).to("cuda").to(dtype)
    model.load_tensors(weights)
    model.set_kv_cache(batch_size=slots)
    return model.eval()


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def rel_err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def assert_close(got, want, dtype, what=""):
    """fp32: the whole block within rounding.  bf16: a rounding difference ahead of a router can move a token to another expert (in
    exact arithmetic on bf16-rounded inputs just as well), so the typical row and four rows in five must be within bf16 rounding; the
    fp32 runs of the same tests are the sharp ones."""
    if dtype == torch.float32:
        assert rel_err(got, want) < 3e-5, (what, rel_err(got, want))
        return
    got, want = got.double().cpu(), want.double().cpu()
    rows = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-30)
    assert float(rows.median()) < 6e-2 and float((rows < 0.12).double().mean()) >= 0.8, (what, rows)


# ---------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [42, 64, 1024])
def test_scaled_residual_and_dynamic_tanh(dtype, d):
    """x += y0 s0 + (y1 + y2) s1 + extra + row_add, the copy in the product dtype and the norm, with every subset of the terms."""
    k = K()
    g = torch.Generator().manual_seed(d)
    n = 9
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype)   # noqa: E731
    x0 = torch.randn(n, d, generator=g)
    y0, y1, y2, s0, s1, ra = mk(n, d), mk(n, d), mk(n, d), mk(d), mk(d), mk(d)
    extra = torch.randn(n, d, generator=g)
    alpha, nw, nb = torch.tensor([0.7]).to(dtype), mk(d), mk(d)
    cases = [dict(y0=y0, s0=s0, y1=y1, y2=y2, s1=s1), dict(y0=y0, s0=s0), dict(y0=y0, s0=s0, y1=y1, s1=s1), dict(extra=extra, row_add=ra), dict(),
             dict(y0=y0, y2=y2)]
    for case in cases:
        want = x0.double()
        if "y0" in case:
            want = want + y0.double() * (s0.double() if "s0" in case else 1.0)
        ff = sum(case[nm].double() for nm in ("y1", "y2") if nm in case)
        if "y1" in case or "y2" in case:
            want = want + ff * (s1.double() if "s1" in case else 1.0)
        if "extra" in case:
            want = want + extra.double() + ra.double()
        x = x0.clone().cuda()
        cast, act = torch.empty(n, d, dtype=dtype, device="cuda"), torch.empty(n, d, dtype=dtype, device="cuda")
        k.scaled_residual(x, cast=cast, norm=(alpha.cuda(), nw.cuda(), nb.cuda()), act=act, **{nm: t.cuda() for nm, t in case.items()})
        assert rel_err(x, want) < 1e-6, sorted(case)
        tol = 1e-6 if dtype == torch.float32 else 6e-3
        assert rel_err(cast, want) < tol
        assert rel_err(act, torch.tanh(alpha.double() * want) * nw.double() + nb.double()) < tol
    x = x0.clone().cuda()
    k.scaled_residual(x, y0=y0.cuda())        # no norm, no copy
    assert rel_err(x, x0.double() + y0.double()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,ff", [(7, 22), (5, 64), (300, 200)])
def test_xielu_and_clamped_gate(dtype, rows, ff):
    k = K()
    g = torch.Generator().manual_seed(rows)
    z = (torch.randn(rows, ff, generator=g) * 2).to(dtype)
    pq = torch.tensor([0.3, -0.8]).to(dtype)
    got = k.xielu_(z.clone().cuda(), pq.cuda())
    tol = 2e-6 if dtype == torch.float32 else 6e-3
    assert rel_err(got, O.xielu(z.double(), pq[0].double(), pq[1].double())) < tol
    both = (torch.randn(rows, 2 * ff, generator=g) * 2).to(dtype)
    for limit, alpha in ((1.2, 1.702), (0.4, 1.0), (50.0, 1.702)):
        gt, up = both[:, :ff].double().clamp(max=limit), both[:, ff:].double().clamp(-limit, limit)
        want = gt * torch.sigmoid(alpha * gt) * (up + 1.0)
        assert rel_err(k.glu_clamped(both.cuda(), limit, alpha), want) < tol, (limit, alpha)


@pytest.mark.parametrize("experts,top", [(18, 5), (6, 1), (8, 8), (5, 3)])
def test_router_takes_the_largest_biased_logits_and_weights_them_among_themselves(experts, top):
    k = K()
    g = torch.Generator().manual_seed(experts)
    d, n = 40, 64
    x = torch.randn(n, d, generator=g).to(torch.bfloat16)
    W = {"router": (torch.randn(experts, d, generator=g) * 0.4).to(torch.bfloat16).double(), "router.b": torch.randn(experts, generator=g).to(torch.bfloat16).double()}
    ids, wts = k.moe_route(x.cuda(), W["router"].to(torch.bfloat16).cuda(), W["router.b"].to(torch.bfloat16).cuda(), top, 1, 1, topk_softmax=True, bias=True)
    want_ids, want_w = O.route(x.double(), W, "", top)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert rel_err(wts, want_w) < 1e-5
    assert float((wts.sum(-1) - 1.0).abs().max()) < 1e-5
    # the bias decides: a large bias on one expert puts it first for every token
    W["router.b"][experts - 1] = 50.0
    ids, _ = k.moe_route(x.cuda(), W["router"].to(torch.bfloat16).cuda(), W["router.b"].to(torch.bfloat16).cuda(), top, 1, 1, topk_softmax=True, bias=True)
    assert bool((ids[:, 0] == experts - 1).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 5, 150])   # the few-pairs path and the grouped path, with experts that get no token
def test_clamped_experts_with_shared_expert(dtype, n):
    from lit_gpt_b200 import moe as M

    ml = moe(6, 2, 24, 0.7, shared=(40, 0.5))
    cfg = config(width=48, vocab=11, layers=[layer("attention", attn(1, 1, 8, 8, size=4), ml)])
    w = checkpoint(cfg, 21)
    model = build(cfg, w, dtype)
    g = torch.Generator().manual_seed(n)
    h = torch.randn(n, 48, generator=g).to(torch.bfloat16)
    W = {kk: v.double() for kk, v in w.items()}
    want = O.sparse_ff(h.double(), W, "l0.mlp.", ml)
    mlp = model.blocks[0].mlp
    got = mlp(h.to(dtype).cuda()).float() + mlp.shared(h.to(dtype).cuda()).float()
    # the module and the oracle get the same (bf16-rounded) rows, so both route alike and EVERY row must be within rounding
    rows = (got.double().cpu() - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-30)
    assert float(rows.max()) < (3e-5 if dtype == torch.float32 else 2e-2), rows
    if dtype == torch.bfloat16 and n > 64:   # the vendor's grouped product against this library's own grouped kernel
        M.VENDOR_GROUPED_GEMM = False
        try:
            own = mlp(h.to(dtype).cuda()).float()
        finally:
            M.VENDOR_GROUPED_GEMM = True
        assert rel_err(own, mlp(h.to(dtype).cuda()).float()) < 2e-2


def _drive(mixer, state, h, cuts, slot, dtype):
    """Feed the rows of h to `mixer` in steps of the given sizes for one sequence in `slot`; returns all output rows."""
    from lit_gpt_b200.ragged import state_batch

    out, at = [], 0
    for n in cuts:
        batch, _ = state_batch([(slot, at, n)], torch.device("cuda"), positions=True)
        out.append(mixer(h[at : at + n].to(dtype).cuda().contiguous(), batch, state).float().cpu())
        at += n
    assert at == h.shape[0]
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cuts", [[37], [1] * 37, [2, 2, 3, 1, 17, 2, 8, 2], [36, 1]])
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_each_mixer_alone(kind, dtype, cuts):
    """Distance bias or rotation and biases, the window's edge, grouped heads, both gates and the ring, in prompts, portions down to two
    tokens and single tokens, in a slot whose rings hold another sequence's leftovers.  The score scale is large, so the softmax is
    nearly one-hot and a key that is one position off moves the output far beyond rounding."""
    m = attn(4, 2, 10, 6, size=7, scale=2.5) if kind == "attention" else attn2(4, 2, 10, 6, size=7, rot_dims=6, scale=2.5)
    cfg = config(width=24, vocab=11, layers=[layer(kind, m, None)])
    w = checkpoint(cfg, 3)
    model = build(cfg, w, dtype, slots=3)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(37, 24, generator=g).to(torch.bfloat16).double()
    want = O.attention(h, {kk: v.double() for kk, v in w.items()}, "l0.mix.", m, kind)
    state = model.states[0]
    for t in state.tensors():
        t.fill_(7.0)
    got = _drive(model.blocks[0].mixer, state, h, cuts, slot=1, dtype=dtype)
    assert rel_err(got, want) < (2e-5 if dtype == torch.float32 else 4e-2), rel_err(got, want)


def _reference_attention(q, kk, v, H, G, dk, dv, size, scale, r1=None, r2=None, gate=None, per_head=False):
    """float64 attention of one sequence from position 0 on given projected rows"""
    n = q.shape[0]
    pen = None if r1 is None else (lambda h, dist: r1[h].double() * torch.log(1.0 + r2[h].double() * dist))
    o = O.windowed_softmax_attention(q.double().view(n, H, dk), kk.double().view(n, G, dk), v.double().view(n, G, dv), scale, size, pen)
    if gate is not None:
        s = torch.sigmoid(gate.double())
        o = o * (s[:, :, None] if per_head else s.view(n, H, dv))
    return o.reshape(n, H * dv)


def test_window_edge_and_a_far_key_in_prompt_and_decoding():
    """One key is made loud (aligned with later queries): the query `size - 1` positions later must still find it, hundreds of quiet keys
    in between, and the next query must not -- in a prompt, in a later portion and in single-token steps, through the tiled and the
    single-row kernel.  The distance bias is on and must not hide it: its size at that distance is known."""
    k = K()
    from lit_gpt_b200.ragged import state_batch

    H, G, dk, dv, size = 2, 1, 8, 5, 230
    g = torch.Generator().manual_seed(9)
    n = 300
    q = torch.randn(n, H * dk, generator=g) * 0.3
    kk = torch.randn(n, G * dk, generator=g) * 0.1
    v = torch.randn(n, G * dv, generator=g)
    loud = 31
    q[loud + size - 1, :dk] = torch.randn(dk, generator=g) * 1.5
    kk[loud] = q[loud + size - 1, :dk] * 4.0         # aligned with the query of the last position that may see it
    q[loud + size] = q[loud + size - 1]              # the next query looks for the same key, which has left its window
    r1, r2 = torch.tensor([0.5, 0.25]), torch.tensor([1.0, 3.0])
    want = _reference_attention(q, kk, v, H, G, dk, dv, size, 1.0, r1, r2)
    assert (want[loud + size - 1, :dv] - v[loud].double()).abs().max() < 1e-3      # the loud key owns that row ...
    assert (want[loud + size, :dv] - v[loud].double()).abs().max() > 1e-2          # ... and is gone one position later
    for cuts in ([n], [loud + 2, n - loud - 2], [loud + size - 1, 1, 1, n - loud - size - 1], [1] * n):
        for tiled in (False, True):
            if tiled and len(cuts) == n:
                continue
            old = k.window_attn_tune(force_tiled_kernel=tiled)
            try:
                k_ring, v_ring = torch.full((2, size, G * dk), 9.0, device="cuda"), torch.full((2, size, G * dv), 9.0, device="cuda")
                got, at = [], 0
                for c in cuts:
                    batch, _ = state_batch([(1, at, c)], torch.device("cuda"))
                    got.append(k.window_attn(q[at : at + c].cuda(), kk[at : at + c].cuda(), v[at : at + c].cuda(), k_ring, v_ring, None,
                                             batch.seq_state, batch.row_seq, c, H, G, dk, dv, size, 1.0, dist=(r1.cuda(), r2.cuda())).cpu())
                    at += c
            finally:
                k.window_attn_tune(force_tiled_kernel=old)
            assert rel_err(torch.cat(got), want) < 1e-5, (cuts[:4], tiled)


def test_distance_bias_has_its_exact_size():
    """Two keys with equal scores at distances 0 and t: their weights differ by exactly (1 + r2 t)^r1."""
    k = K()
    from lit_gpt_b200.ragged import state_batch

    t, r1, r2 = 5, 0.75, 2.0
    q = torch.zeros(t + 1, 4)
    kk = torch.zeros(t + 1, 4)
    v = torch.zeros(t + 1, 2)
    v[0, 0] = 1.0          # the far key's value
    v[t, 1] = 1.0          # the row's own
    batch, _ = state_batch([(0, 0, t + 1)], torch.device("cuda"))
    ring = torch.zeros(1, t + 1, 4, device="cuda"), torch.zeros(1, t + 1, 2, device="cuda")
    out = k.window_attn(q.cuda(), kk.cuda(), v.cuda(), ring[0], ring[1], None, batch.seq_state, batch.row_seq, t + 1, 1, 1, 4, 2, t + 1, 1.0,
                        dist=(torch.tensor([r1]).cuda(), torch.tensor([r2]).cuda())).cpu()
    assert abs(float(out[t, 1] / out[t, 0]) - (1.0 + r2 * t) ** r1) < 1e-4


@pytest.mark.parametrize("hs,size,per_head", [(64, 100, False), (64, 64, True), (128, 1, False), (128, 150, True), (64, 1000, False)])
def test_gated_window_prefill_on_the_tensor_cores(hs, size, per_head):
    """bf16 prompts with 64- / 128-wide heads take the tensor-core tiles: windows that end inside a key tile, at its edge, of one
    position and longer than the prompt; grouped heads; distance bias; both gates; three sequences of unequal length in one launch.
    Compared with exact attention on the same bf16 operands and with the any-size kernel."""
    k = K()
    from lit_gpt_b200.ragged import state_batch

    H, G = 4, 2
    g = torch.Generator().manual_seed(hs + size)
    lens = [200, 37, 300]
    n = sum(lens)
    q = torch.randn(n, H * hs, generator=g).to(torch.bfloat16)
    kk = torch.randn(n, G * hs, generator=g).to(torch.bfloat16)
    v = torch.randn(n, G * hs, generator=g).to(torch.bfloat16)
    gate = (torch.randn(n, H if per_head else H * hs, generator=g) * 2).to(torch.bfloat16)
    biased = not per_head
    r1, r2 = torch.tensor([0.5, 1.0, 0.25, 2.0]).to(torch.bfloat16), torch.tensor([1.0, 0.5, 3.0, 0.125]).to(torch.bfloat16)
    scale = 2.0 * hs ** -0.5           # sharp: the few largest scores carry the row
    want, at = [], 0
    for ln in lens:
        s = slice(at, at + ln)
        want.append(_reference_attention(q[s], kk[s], v[s], H, G, hs, hs, size, scale, r1 if biased else None, r2 if biased else None, gate[s], per_head))
        at += ln
    want = torch.cat(want)
    batch, _ = state_batch([(0, 0, lens[0]), (2, 0, lens[1]), (1, 0, lens[2])], torch.device("cuda"))
    ring = min(size, 400)
    outs = {}
    for mma in (True, False):
        k.WINDOW_PREFILL_MMA = mma
        try:
            k_ring, v_ring = torch.zeros(3, ring, G * hs, dtype=torch.bfloat16, device="cuda"), torch.zeros(3, ring, G * hs, dtype=torch.bfloat16, device="cuda")
            outs[mma] = k.window_attn(q.cuda(), kk.cuda(), v.cuda(), k_ring, v_ring, None, batch.seq_state, batch.row_seq, max(lens), H, G, hs, hs,
                                      min(size, ring), scale, from_start=True, dist=(r1.cuda(), r2.cuda()) if biased else None, gate=gate.cuda(),
                                      gate_per_head=per_head).float().cpu()
        finally:
            k.WINDOW_PREFILL_MMA = True
        # the rings hold every sequence's last positions whichever kernel ran
        for slot, first, ln in ((0, 0, lens[0]), (2, lens[0], lens[1]), (1, lens[0] + lens[1], lens[2])):
            for p in range(max(0, ln - ring), ln):
                assert torch.equal(k_ring[slot, p % ring].cpu(), kk[first + p]) and torch.equal(v_ring[slot, p % ring].cpu(), v[first + p])
    assert rel_err(outs[False], want) < 6e-3
    assert rel_err(outs[True], want) < 1.2e-2


def test_distance_bias_beyond_the_tabulated_reach():
    """A prompt and a window longer than the distances a CTA tabulates: the tensor-core tiles compute the bias in place and agree
    with the any-size kernel."""
    k = K()
    from lit_gpt_b200.ragged import state_batch

    H, G, hs, n, size = 2, 1, 64, 8300, 9000
    g = torch.Generator().manual_seed(77)
    q = torch.randn(n, H * hs, generator=g).to(torch.bfloat16).cuda()
    kk = torch.randn(n, G * hs, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(n, G * hs, generator=g).to(torch.bfloat16).cuda()
    r1, r2 = torch.tensor([1.5, 0.75]).to(torch.bfloat16).cuda(), torch.tensor([0.5, 4.0]).to(torch.bfloat16).cuda()
    batch, _ = state_batch([(0, 0, n)], torch.device("cuda"))
    outs = {}
    for mma in (True, False):
        k.WINDOW_PREFILL_MMA = mma
        try:
            k_ring, v_ring = torch.zeros(1, size, G * hs, dtype=torch.bfloat16, device="cuda"), torch.zeros(1, size, G * hs, dtype=torch.bfloat16, device="cuda")
            outs[mma] = k.window_attn(q, kk, v, k_ring, v_ring, None, batch.seq_state, batch.row_seq, n, H, G, hs, hs, size, 3.0 * hs ** -0.5,
                                      from_start=True, dist=(r1, r2)).float().cpu()
        finally:
            k.WINDOW_PREFILL_MMA = True
    assert rel_err(outs[True], outs[False]) < 1.2e-2
    assert rel_err(outs[True][-200:], outs[False][-200:]) < 1.2e-2     # the rows that look farthest back


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg,seed", [(CFG_ODD, 11), (CFG_WIDE, 12), (CFG_TILES, 13)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_matches_oracle(cfg, seed, dtype):
    w = checkpoint(cfg, seed)
    toks = tokens_for(cfg, 150, seed)
    model = build(cfg, w, dtype)
    got = model.step(toks, [(1, 0, len(toks))])
    assert_close(got, O.forward(cfg, w, toks), dtype)


def test_layers_follow_the_oracle_one_by_one():
    """The stream after every layer run in fp32, looped passes included (each with its own state and its own entry)."""
    for cfg, seed in ((CFG_ODD, 31), (CFG_TILES, 32), (CFG_WIDE, 33)):
        w = checkpoint(cfg, seed)
        toks = tokens_for(cfg, 60, seed)
        model = build(cfg, w, torch.float32)
        model.trace = []
        model.step(toks, [(0, 0, len(toks))])
        want = []
        O.forward(cfg, w, toks, trace=want)
        assert len(model.trace) == len(want) == len(model.runs)
        for r, (a, b) in enumerate(zip(model.trace, want)):
            assert rel_err(a, b) < 1e-5, (r, rel_err(a, b))


@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_WIDE, CFG_TILES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decoding_token_by_token_equals_prefill(dtype, cfg):
    w = checkpoint(cfg, 41)
    toks = tokens_for(cfg, 90, 41)
    model = build(cfg, w, dtype)
    whole = model.step(toks, [(0, 0, len(toks))])
    single = torch.cat([model.step([t], [(1, p, 1)]) for p, t in enumerate(toks)])
    if dtype == torch.float32:
        assert rel_err(single, whole) < 2e-5
        assert rel_err(single, O.forward(cfg, w, toks)) < 3e-5
    else:
        assert_close(single, whole.float(), dtype)


@pytest.mark.parametrize("portions", [[2, 2, 2, 30, 3, 34, 1, 35, 2], [109, 2], [1, 110], [5] * 22 + [1]])
@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_WIDE])
def test_prompt_in_portions(portions, cfg):
    """A prompt cut into portions of several sizes, down to two tokens and one, gives the logits of the whole prompt."""
    w = checkpoint(cfg, 51)
    toks = tokens_for(cfg, sum(portions), 51)
    model = build(cfg, w, torch.float32)
    want = O.forward(cfg, w, toks)
    got, at = [], 0
    for n in portions:
        got.append(model.step(toks[at : at + n], [(1, at, n)]))
        at += n
    assert rel_err(torch.cat(got), want) < 3e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_batch_equals_each_alone(dtype):
    """Requests of unequal length in one batch (prefill together, then decoding together with the shorter ones leaving) against each alone."""
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_ODD
    w = checkpoint(cfg, 61)
    model = build(cfg, w, dtype)
    reqs = {"a": tokens_for(cfg, 50, 62), "b": tokens_for(cfg, 9, 63), "c": tokens_for(cfg, 23, 64), "d": tokens_for(cfg, 1, 65)}
    pre = {"a": 40, "b": 3, "c": 20, "d": 1}
    session = Session(model, slots=2)       # grows while the batch is live
    rows = {rid: [] for rid in reqs}
    out = session.step([(rid, reqs[rid][: pre[rid]], None) for rid in reqs], end=["d"])
    at = 0
    for rid in reqs:
        rows[rid].append(out[at : at + pre[rid]])
        at += pre[rid]
    pos = dict(pre)
    while True:
        live = [rid for rid in reqs if pos[rid] < len(reqs[rid])]
        if not live:
            break
        out = session.step([(rid, [reqs[rid][pos[rid]]], None) for rid in live], end=[rid for rid in live if pos[rid] + 1 == len(reqs[rid])])
        for i, rid in enumerate(live):
            rows[rid].append(out[i : i + 1])
            pos[rid] += 1
    assert model.slots.in_use == 0
    for rid, toks in reqs.items():
        got = torch.cat(rows[rid])
        assert_close(got, O.forward(cfg, w, toks), dtype, rid)


def test_freed_slots_are_reused_without_leftovers():
    """A request ends, another takes its slot (whose rings still hold the first one's keys), starting with a two-token portion."""
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_WIDE
    w = checkpoint(cfg, 71)
    model = build(cfg, w, torch.float32, slots=1)
    session = Session(model, slots=1)
    a, b = tokens_for(cfg, 80, 72), tokens_for(cfg, 45, 73)
    session.step([("a", a, [])], end=["a"])
    got = [session.step([("b", b[:2], None)])]
    got.append(session.step([("b", b[2:40], None)]))
    got += [session.step([("b", [t], None)]) for t in b[40:]]
    assert model.slots.capacity == 1
    assert rel_err(torch.cat(got), O.forward(cfg, w, b)) < 3e-5


def test_long_decoding_wraps_the_rings_many_times():
    """250 single-token steps behind a prompt: windows of 3 to 33 positions wrap their rings dozens of times."""
    cfg = CFG_ODD
    w = checkpoint(cfg, 81)
    toks = tokens_for(cfg, 290, 81)
    model = build(cfg, w, torch.float32)
    got = [model.step(toks[:40], [(0, 0, 40)])]
    got += [model.step([t], [(0, p, 1)]) for p, t in enumerate(toks[40:], start=40)]
    assert rel_err(torch.cat(got), O.forward(cfg, w, toks)) < 3e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompts_on_the_tensor_cores_then_decoding_over_their_rings(dtype):
    """Head sizes that take the tensor-core prompt tiles in bf16: two prompts together, decoding over the rings they left, and a third
    request that arrives in portions; windows pass over decoded tokens."""
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_TILES
    w = checkpoint(cfg, 85)
    model = build(cfg, w, dtype)
    a, b, c = tokens_for(cfg, 230, 86), tokens_for(cfg, 140, 87), tokens_for(cfg, 75, 88)
    session = Session(model, slots=3)
    out = session.step([("a", a[:150], None), ("b", b[:60], None)])
    rows = {"a": [out[:150]], "b": [out[150:]], "c": []}
    rows["c"].append(session.step([("c", c[:33], None)]))
    rows["c"].append(session.step([("c", c[33:35], None)]))
    rows["c"].append(session.step([("c", c[35:], None)]))
    for p in range(80):
        out = session.step([("a", [a[150 + p]], None), ("b", [b[60 + p]], None)])
        rows["a"].append(out[:1])
        rows["b"].append(out[1:])
    for rid, toks in (("a", a), ("b", b), ("c", c)):
        assert_close(torch.cat(rows[rid]), O.forward(cfg, w, toks), dtype, rid)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_generate_entry_points(dtype):
    """Greedy generation through generate() (captured decode graph) and through the batch scheduler give the oracle's tokens."""
    from lit_gpt_b200.generate.base import generate
    from lit_gpt_b200.generate.serve import generate_batch

    cfg = CFG_ODD
    w = checkpoint(cfg, 91)
    prompt = tokens_for(cfg, 9, 91)
    seq = O.greedy(cfg, w, prompt, 14)
    model = build(cfg, w, dtype, slots=1)
    model.max_seq_length = 64
    y = generate(model, torch.tensor(prompt, device="cuda"), len(seq), temperature=0.0)
    if dtype == torch.float32:
        assert y.tolist() == seq
    other = tokens_for(cfg, 4, 92)
    model.set_kv_cache(batch_size=2)
    ys = generate_batch(model, [prompt, other], 14)
    assert ys[0] == y.tolist() and len(ys[1]) == 4 + 14 and model.slots.in_use == 0
    if dtype == torch.float32:
        assert ys[1] == O.greedy(cfg, w, other, 14)


def test_forward_signature_of_the_other_models():
    """forward(idx, input_pos) with batch rows = slots and shared positions, as GPT.forward: a prompt, then single tokens."""
    cfg = CFG_WIDE
    w = checkpoint(cfg, 95)
    model = build(cfg, w, torch.float32, slots=2)
    a, b = tokens_for(cfg, 12, 96), tokens_for(cfg, 12, 97)
    idx = torch.tensor([a, b], device="cuda")
    out = model(idx[:, :10], torch.arange(10, device="cuda"))
    for p in (10, 11):
        out = torch.cat([out, model(idx[:, p : p + 1], torch.tensor([p], device="cuda"))], dim=1)
    assert out.shape == (2, 12, cfg["vocab"])
    assert rel_err(out[0], O.forward(cfg, w, a)) < 3e-5 and rel_err(out[1], O.forward(cfg, w, b)) < 3e-5


def _write_checkpoint(folder, cfg, weights):
    import json
    import struct

    header, blob = {}, b""
    for name, t in weights.items():
        raw = t.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    hj = json.dumps(header).encode()
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    (folder / "config.json").write_text(json.dumps(cfg))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_end_to_end(tmp_path, dtype):
    """The command-line replayer on a checkpoint directory written here: a ragged first step, decoding together, a request that
    ends, a new one in its slot, steps without anything wanted -- the files it writes against the oracle."""
    import json
    import subprocess

    import numpy as np

    cfg = CFG_ODD
    w = checkpoint(cfg, 101)
    _write_checkpoint(tmp_path, cfg, w)
    a, b, c = tokens_for(cfg, 40, 102), tokens_for(cfg, 9, 103), tokens_for(cfg, 70, 104)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:37], "want": [0, 36]}, {"id": "b", "tokens": b[:6], "want": [5]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [a[37]], "want": []}, {"id": "b", "tokens": [b[6]], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": [a[38]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": [a[39]], "want": [0]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": c, "want": [0, 1, 63, 64, 69]}], "end": ["c"]},
    ]
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", dtype, "--out", str(out), "--max-tokens", "120"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done ")] == [f"done {i}" for i in range(5)]
    assert sorted(os.listdir(out)) == ["0.f32", "2.f32", "3.f32", "4.f32"]        # step 1 wanted nothing
    full = {kk: O.forward(cfg, w, t) for kk, t in (("a", a), ("b", b), ("c", c))}
    want = {0: torch.stack([full["a"][0], full["a"][36], full["b"][5]]), 2: torch.stack([full["a"][38], full["b"][7]]),
            3: full["a"][39:40], 4: full["c"][[0, 1, 63, 64, 69]]}
    for step, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert got.shape == ref.shape
        if dtype == "float32":
            assert rel_err(got, ref) < 3e-5, f"step {step}"
    if dtype == "bfloat16":
        got = torch.cat([torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, cfg["vocab"])) for step in want])
        assert_close(got, torch.cat(list(want.values())), torch.bfloat16)


def test_generate_command_line(tmp_path):
    """`python -m lit_gpt_b200.generate.base` on a checkpoint directory without a tokenizer: a prompt of token ids in, the oracle's greedy
    continuation out."""
    import subprocess

    cfg = CFG_WIDE
    w = checkpoint(cfg, 111)
    _write_checkpoint(tmp_path, cfg, w)
    prompt = tokens_for(cfg, 6, 112)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-m", "lit_gpt_b200.generate.base", " ".join(str(t) for t in prompt), "--checkpoint_dir", str(tmp_path),
                          "--precision", "32-true", "--temperature", "0", "--max_new_tokens", "9"], cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    printed = [int(t) for t in res.stdout.strip().splitlines()[-1].split()]
    assert printed == O.greedy(cfg, w, prompt, 9)
