"""Fizadra on the GPU against the plain restatement in ``fizadra_oracle.py``: every mechanism alone, then whole models of several
shapes through prefill, decoding, portions, ragged batches, reused slots and the generation entry points."""
from __future__ import annotations

import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import fizadra_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def K():
    from lit_gpt_b200 import kernels

    return kernels


# ---------------------------------------------------------------------------------------------------------
# configurations and random checkpoints
# ---------------------------------------------------------------------------------------------------------
def rot(dims, base=100.0, scaling=None):
    r = dict(base=base, dims=dims)
    if scaling is not None:
        r["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    return r


def latent(kind, heads, dim, rot_dim, vdim, kv_rank, q_rank, scale=None, base=100.0, scaling=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, rot=rot(rot_dim, base, scaling),
             scale=scale if scale is not None else (dim + rot_dim) ** -0.5)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return kind, m


def talking(heads, kv_heads, dim, vdim, rot_dims, scale=None, base=100.0):
    return "attention", dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=rot(rot_dims, base), scale=scale if scale is not None else dim ** -0.5)


def layer(mixer, ff):
    return dict(type=mixer[0], mixer=mixer[1], mlp=None if ff is None else dict(kind="dense", ff=ff))


def config(width, vocab, groups, layers, eps=1e-5):
    return dict(architecture="Fizadra", layers=layers, norm=dict(eps=eps, groups=groups), vocab=vocab, width=width)


FIRST, SECOND = "latent_attention", "latent_attention_2"

# odd sizes on purpose: norm groups of 14 numbers (no 16-byte access fits), grouped heads with a partly rotated head, key size !=
# value size, a layer without feed-forward, both latent kinds lending their cache to a later layer with other head counts, one head
CFG_ODD = config(width=42, vocab=83, groups=3, layers=[
    layer(talking(6, 2, 10, 6, rot_dims=6, scale=0.9), 50),
    layer(latent(FIRST, 3, 10, 6, 7, kv_rank=12, q_rank=9, scaling=(3.0, 16, 4.0, 1.0), scale=0.7), None),
    layer(latent(SECOND, 2, 6, 4, 5, kv_rank=10, q_rank=7, base=50.0), 30),
    layer(latent(FIRST, 5, 4, 6, 3, kv_rank=12, q_rank=5, scaling=(3.0, 16, 4.0, 1.0), kv_from=1), 26),
    layer(latent(SECOND, 1, 9, 4, 11, kv_rank=10, q_rank=6, base=50.0, kv_from=2), None),
    layer(talking(1, 1, 8, 8, rot_dims=8, base=1e4), 20),
])
# sizes that take the vectorised and tensor-core paths: one norm group, latents of 64 + 32 numbers (bf16 single rows on the tensor
# cores), value heads wider than one column chunk of the prompt tiles, an attention head wider than 64, sixteen query heads
CFG_WIDE = config(width=64, vocab=120, groups=1, eps=1e-3, layers=[
    layer(latent(SECOND, 4, 24, 32, 136, kv_rank=64, q_rank=40, base=1e4), 96),
    layer(talking(4, 4, 72, 136, rot_dims=20, base=1e5, scale=0.2), None),
    layer(latent(FIRST, 16, 16, 32, 8, kv_rank=64, q_rank=24, base=1e4, scaling=(8.0, 32, 16.0, 2.0), kv_from=0), 80),
    layer(talking(8, 2, 16, 24, rot_dims=16, base=50.0), 64),
])


# head sizes the tensor-core prompt tiles take in bf16: unrotated = value size 64 and 128, rotated part 64 (and 128), a borrowed cache,
# and an attention layer between them
CFG_TILES = config(width=96, vocab=140, groups=2, layers=[
    layer(latent(FIRST, 2, 64, 64, 64, kv_rank=32, q_rank=24, base=1e4, scaling=(4.0, 64, 8.0, 1.0)), 100),
    layer(latent(SECOND, 3, 128, 64, 128, kv_rank=64, q_rank=48, base=1e5), 120),
    layer(talking(4, 2, 64, 64, rot_dims=32, base=1e4), None),
    layer(latent(SECOND, 2, 64, 128, 64, kv_rank=32, q_rank=40, base=1e3), 80),
    layer(latent(FIRST, 2, 128, 64, 128, kv_rank=64, q_rank=16, base=1e5, scaling=(2.0, 32, 4.0, 1.0), kv_from=1), 64),
])


def checkpoint(cfg, seed, sink_mean=0.5):
    """Random bf16 weights of a size that keeps every mechanism alive."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    d = cfg["width"]
    w = {"embed": rnd(cfg["vocab"], d), "final.norm": rnd(d, std=0.2, mean=1.0), "head": rnd(cfg["vocab"], d, std=d ** -0.5)}
    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        for nm in ("norm1", "norm1b", "norm2", "norm2b"):
            w[p + nm] = rnd(d, std=0.2, mean=1.0)
        w[p + "dwa"] = rnd(i + 2, std=0.3, mean=0.4)
        q = p + "mix."
        if ly["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for name, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                w[q + name] = rnd(rows, d, std=d ** -0.5)
                w[q + name + ".b"] = rnd(rows, std=0.3)
            w[q + "q.norm"], w[q + "k.norm"] = rnd(dk, std=0.3, mean=1.5), rnd(dk, std=0.3, mean=1.5)
            w[q + "talk"] = (torch.eye(H) + torch.randn(H, H, generator=g) * 0.3).to(torch.bfloat16)
            w[q + "o"] = rnd(d, H * dv, std=(H * dv) ** -0.5)
        else:
            H, dn, dr, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[q + "dq"], w[q + "dq.norm"] = rnd(qr, d, std=d ** -0.5), rnd(qr, std=0.2, mean=1.0)
            w[q + "uq"] = rnd(H * (dn + dr), qr, std=2.0 * qr ** -0.5)
            if m.get("kv_from") is None:
                w[q + "dkv"], w[q + "dkv.norm"] = rnd(r + dr, d, std=d ** -0.5), rnd(r, std=0.2, mean=1.0)
            w[q + "uk"], w[q + "uv"] = rnd(H * dn, r, std=2.0 * r ** -0.5), rnd(H * dv, r, std=r ** -0.5)
            if ly["type"] == FIRST:
                w[q + "sink"] = rnd(H, std=1.0, mean=sink_mean)
                w[q + "g"] = rnd(H * dv, d, std=2.0 * d ** -0.5)
            else:
                w[q + "g"] = rnd(H, d, std=2.0 * d ** -0.5)
            w[q + "o"] = rnd(d, H * dv, std=(H * dv) ** -0.5)
        if ly["mlp"] is None:
            del w[p + "norm2"], w[p + "norm2b"]
        else:
            ff = ly["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"] = rnd(ff, d, std=d ** -0.5), rnd(d, ff, std=ff ** -0.5)
    return w


def build(cfg, weights, dtype, slots=2, max_seq=256):
    from lit_gpt_b200.config import FizadraConfig
    from lit_gpt_b200.fizadra import Fizadra

    model = Fizadra(FizadraConfig.from_dict(cfg)).to("cuda").to(dtype)
    model.load_tensors(weights)
    model.max_seq_length = max_seq
    model.set_kv_cache(batch_size=slots)
    return model.eval()


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def rel_err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def assert_close(got, want, dtype, what=""):
    """fp32: the whole block within rounding.  bf16: the typical row and nine rows in ten within bf16 rounding of a model a few
    dozen channels wide; the fp32 runs of the same tests are the sharp ones."""
    if dtype == torch.float32:
        assert rel_err(got, want) < 3e-5, (what, rel_err(got, want))
        return
    got, want = got.double().cpu(), want.double().cpu()
    rows = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-30)
    assert float(rows.median()) < 5e-2 and float((rows < 0.1).double().mean()) >= 0.9, (what, rows)


def poison(model):
    for t in model.state_tensors():
        t.fill_(40.0)


# ---------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,groups", [(42, 3), (64, 1), (96, 4), (1024, 8), (30, 30)])
def test_group_norms_residual_and_depth_sum(dtype, d, groups):
    """Post-norm in groups, residual sum, weighted sum over the earlier results and the next pre-norm, each part optional."""
    k = K()
    g = torch.Generator().manual_seed(d + groups)
    n, m, eps = 7, 4, 1e-3
    y = torch.randn(n, d, generator=g).to(dtype)
    pw, nw = (1 + 0.3 * torch.randn(d, generator=g)).to(dtype), (1 + 0.3 * torch.randn(d, generator=g)).to(dtype)
    dw = torch.randn(m, generator=g).to(dtype)
    stack = torch.randn(m, n, d, generator=g)
    x_in = torch.randn(n, d, generator=g)
    X = x_in.double() + O.group_norm(y.double(), pw.double(), eps, groups)
    avg = sum(dw[j].double() * stack[j].double() for j in range(m - 1)) + dw[m - 1].double() * X
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    # everything at once, the result written into the stack
    sc = stack.clone().cuda()
    a, act = torch.empty(n, d, device="cuda"), torch.empty(n, d, device="cuda", dtype=dtype)
    k.depth_residual(x_in.cuda(), sc[m - 1], eps, groups, y=y.cuda(), post_w=pw.cuda(), stack=sc, m=m, depth_w=dw.cuda(), avg=a, pre_w=nw.cuda(), act=act)
    assert rel_err(sc[m - 1], X) < 1e-6 and rel_err(a, avg) < 1e-6
    assert rel_err(act, O.group_norm(avg, nw.double(), eps, groups)) < tol
    assert torch.equal(sc[: m - 1].cpu(), stack[: m - 1])
    # no sum over depth, in place
    x = x_in.clone().cuda()
    k.depth_residual(x, x, eps, groups, y=y.cuda(), post_w=pw.cuda(), pre_w=nw.cuda(), act=act)
    assert rel_err(x, X) < 1e-6 and rel_err(act, O.group_norm(X, nw.double(), eps, groups)) < tol
    # only a norm (what feeds the first layer)
    k.depth_residual(x_in.cuda(), x_in.cuda(), eps, groups, pre_w=nw.cuda(), act=act)
    assert rel_err(act, O.group_norm(x_in.double(), nw.double(), eps, groups)) < tol
    # a sum of one result only
    k.depth_residual(x_in.cuda(), x, eps, groups, y=y.cuda(), post_w=pw.cuda(), m=1, depth_w=dw.cuda(), avg=a)
    assert rel_err(a, dw[0].double() * X) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("shape", [(14, 6, 4), (16, 8, 4), (16, 16, 0), (72, 20, 0)])    # head size, rotated dimensions, first rotated dimension
def test_head_norm_rotation_and_scatter(dtype, interleaved, shape):
    """Three groups of heads in one launch: a normed and partly rotated one in place, a normed one scattered into cache rows, a plain
    copy into cache rows; rows with nowhere to go are skipped; positions up to a few thousand."""
    k = K()
    g = torch.Generator().manual_seed(3)
    n, H, G, dv = 9, 3, 2, 5 if shape[0] == 14 else 6
    dk, rd, off = shape
    src = torch.randn(n, H * dk + G * dk + G * dv, generator=g).to(dtype)
    wq, wk = (1 + 0.3 * torch.randn(dk, generator=g)).to(dtype), (1 + 0.3 * torch.randn(dk, generator=g)).to(dtype)
    pos = torch.tensor([0, 1, 2, 5, 70, 300, 1000, 4000, 3], dtype=torch.int32)
    spec = dict(dims=rd, base=70.0, scaling=dict(factor=2.5, original=64, fast=8.0, slow=1.0))
    f, mag = O.rotary_frequencies(spec)
    rows = torch.tensor([4, 0, 7, -1, 2, 9, 1, 5, 3], dtype=torch.int64)
    pad = 3 if dk == 14 else 4      # odd sizes keep every access to one element, even ones allow two at a time
    kc, vc = torch.full((10, G * dk + pad), 9.0, dtype=dtype, device="cuda"), torch.full((10, G * dv), 9.0, dtype=dtype, device="cuda")
    buf = src.clone().cuda()
    q, kk, v = buf[:, : H * dk], buf[:, H * dk : (H + G) * dk], buf[:, (H + G) * dk :]
    fr, wq_d, wk_d, rows_d = f.float().cuda(), wq.cuda(), wk.cuda(), rows.cuda()    # a group only records addresses: the tensors must live on
    k.head_rope(n, pos.cuda(), 1e-3,
                k.rope_seg(q, q, H, dk, norm_w=wq_d, freq=fr, rot_off=off, rot_dims=rd, interleaved=interleaved, mag=mag),
                k.rope_seg(kk, kc[:, pad:], G, dk, norm_w=wk_d, freq=fr, rot_off=0, rot_dims=rd, interleaved=interleaved, mag=mag, out_rows=rows_d),
                k.rope_seg(v, vc, G, dv, out_rows=rows_d), dtype=dtype, device=torch.device("cuda"))

    def turned(x, w, off_):
        x = O.unit_rms(x.double(), 1e-3) * w.double()
        out = x.clone()
        for i in range(n):      # the oracle rotates row t by position t: one row at a time, shifted to its position
            pad = torch.zeros(int(pos[i]) + 1, x.shape[1], x.shape[2] - off_, dtype=torch.float64)
            pad[-1] = x[i, :, off_:]
            out[i, :, off_:] = O.rotate(pad, spec, interleaved)[-1]
        return out

    tol = 5e-5 if dtype == torch.float32 else 1e-2      # the angle is an fp32 product: at position 4000 half a unit in its last place is 1.2e-4 rad
    assert rel_err(q.reshape(n, H, dk), turned(src[:, : H * dk].reshape(n, H, dk), wq, off)) < tol
    want_k = turned(src[:, H * dk : (H + G) * dk].reshape(n, G, dk), wk, 0).reshape(n, G * dk)
    keep = rows >= 0
    assert rel_err(kc[rows[keep].cuda(), pad:], want_k[keep]) < tol
    assert torch.equal(vc[rows[keep].cuda()].cpu(), src[keep][:, (H + G) * dk :])
    assert float(kc[6].float().min()) == 9.0 and float(kc[8].float().min()) == 9.0 and float(kc[:, :pad].float().min()) == 9.0   # untouched rows and columns


def _softmax_rows(scores, sink):
    """scores (n_keys,) float64 -> probabilities with exp(sink) in the denominator (sink None: none)."""
    m = scores.max() if sink is None else torch.maximum(scores.max(), sink)
    e = torch.exp(scores - m)
    return e / (e.sum() + (torch.exp(sink - m) if sink is not None else 0.0))


def _latent_reference(q, c, kr, w_uk, w_uv, sink, gate, H, dn, dr, dv, scale, start):
    """float64: queries q (n, H (dn + dr)) at positions start .., latents c and shared key parts kr of positions 0 .. start + n - 1."""
    n = q.shape[0]
    q, c, kr = q.double().view(n, H, dn + dr), c.double(), kr.double()
    k, v = (c @ w_uk.double().T).view(-1, H, dn), (c @ w_uv.double().T).view(-1, H, dv)
    out = torch.zeros(n, H, dv, dtype=torch.float64)
    for i in range(n):
        m = start + i + 1
        for h in range(H):
            s = (k[:m, h] @ q[i, h, :dn] + kr[:m] @ q[i, h, dn:]) * scale
            o = _softmax_rows(s, None if sink is None else sink[h].double()) @ v[:m, h]
            if gate is not None:
                gd = gate.double()[i]
                o = o * (torch.sigmoid(gd[h]) if gate.shape[1] == H else torch.sigmoid(gd[h * dv : (h + 1) * dv]))
            out[i, h] = o
    return out.reshape(n, H * dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 10, 6, 7, 12), (4, 24, 32, 136, 64), (16, 16, 32, 8, 64), (2, 64, 64, 128, 96), (2, 64, 64, 64, 96),
                                   (3, 128, 64, 128, 64), (2, 64, 128, 64, 32), (2, 128, 128, 128, 32)])
@pytest.mark.parametrize("options", ["sink+element", "head", "none"])
def test_latent_attention_kernels_with_a_shared_key_part(dtype, sizes, options):
    """Prompt tiles (a sequence from position 0 and one continuing at position 70, together) and single rows (any-size and, for
    bf16 latents of 64 + 32 numbers, tensor-core splits) against exact attention on the same operands; one loud key far back."""
    k = K()
    H, dn, dr, dv, r = sizes
    g = torch.Generator().manual_seed(H * dn + dv)
    L, S = 200, 3
    scale = 2.0 * (dn + dr) ** -0.5
    cache = (torch.randn(S, L, r + dr, generator=g) * 0.7).to(dtype)
    w_uk, w_uv = (torch.randn(H * dn, r, generator=g) * r ** -0.5).to(dtype), (torch.randn(H * dv, r, generator=g) * r ** -0.5).to(dtype)
    sink = torch.randn(H, generator=g).to(dtype) if "sink" in options else None
    gcols = H * dv if "element" in options else H if "head" in options else 0
    lens = [(1, 0, 150), (2, 70, 41)]      # (slot, first position, rows)
    n = sum(x[2] for x in lens)
    q = torch.randn(n, H * (dn + dr), generator=g).to(dtype)
    # the query at position 149 of slot 1 looks for position 3, far back, and finds it among 150
    loud = torch.randn(dr, generator=g)
    cache[1, 3, r:] = (loud * 4).to(dtype)
    q.view(n, H, dn + dr)[149, :, dn:] = (loud * 4).to(dtype)
    gate_all = torch.randn(n, 5 + gcols, generator=g).to(dtype) if gcols else None
    gate = gate_all[:, 5:] if gcols else None
    want, at = [], 0
    for slot, start, rows in lens:
        want.append(_latent_reference(q[at : at + rows], cache[slot, : start + rows, :r], cache[slot, : start + rows, r:], w_uk, w_uv, sink,
                                      None if gate is None else gate[at : at + rows], H, dn, dr, dv, scale, start))
        at += rows
    want = torch.cat(want)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    # prompts: gathered context rows, keys and values expanded by a matrix product
    ctx_rows, seqs, first = [], [], 0
    for slot, start, rows in lens:
        seqs.append((first, rows, start, len(ctx_rows)))
        ctx_rows += list(range(slot * L, slot * L + start + rows))
        first += rows
    cg = cache.cuda()
    ctx = k.gather_rows(cg.view(-1, r + dr), torch.tensor(ctx_rows, dtype=torch.int64, device="cuda"))
    kv = torch.nn.functional.linear(ctx[:, :r].float(), torch.cat([w_uk, w_uv]).cuda().float()).to(dtype)
    tiles = dtype == torch.bfloat16 and dn == dv and dv in (64, 128) and dr in (64, 128)     # sizes the tensor-core tiles take
    for mma in ((True, False) if tiles else (True,)):
        k.LATENT_PREFILL_MMA = mma
        try:
            launches = k.launch_count()
            got = k.latent_prefill(q.cuda(), kv[:, : H * dn], kv[:, H * dn :], torch.tensor(seqs, dtype=torch.int32, device="cuda"), 150, H, dn + dr, dv,
                                   scale, k_shared=ctx[:, r:], sink=None if sink is None else sink.cuda(),
                                   gate=None if gate is None else gate_all.cuda()[:, 5:])
            assert k.launch_count() - launches == 1
        finally:
            k.LATENT_PREFILL_MMA = True
        assert rel_err(got, want) < (tol if dtype == torch.float32 else 4e-2), (mma, rel_err(got, want))   # bf16: K and V rounded after the expansion
    # single rows: the last row of each sequence, over splits of several sizes; what lies past the context is loud and must stay unseen
    cg[1, 150:, :] = 30.0
    cg[2, 111:, :] = 30.0
    last = [149, 190]
    qd = q[last].cuda()
    gd = None if gate is None else gate_all[last].cuda()[:, 5:]
    slot_t, pos_t = torch.tensor([1, 2], dtype=torch.int32, device="cuda"), torch.tensor([149, 110], dtype=torch.int32, device="cuda")
    for any_size in (False, True):
        old = k.latent_decode_tune(force_any_size_kernel=any_size)
        try:
            for splits in (1, 2, 3, 7):
                got = k.latent_decode(qd, w_uk.cuda(), w_uv.cuda(), cg, slot_t, pos_t, H, dn, dv, scale, splits, shared_dims=dr,
                                      sink=None if sink is None else sink.cuda(), gate=gd)
                assert rel_err(got, want[last]) < tol, (any_size, splits, rel_err(got, want[last]))
        finally:
            k.latent_decode_tune(force_any_size_kernel=old)


def _talking_reference(q, kk, v, talk, sink, H, G, dk, dv, scale, start):
    n, per = q.shape[0], H // G
    q, kk, v = q.double().view(n, H, dk), kk.double().view(-1, G, dk), v.double().view(-1, G, dv)
    out = torch.zeros(n, H, dv, dtype=torch.float64)
    for i in range(n):
        m = start + i + 1
        raw = torch.stack([kk[:m, h // per] @ q[i, h] for h in range(H)]) * scale      # (H, m)
        mixed = talk.double() @ raw
        for h in range(H):
            out[i, h] = _softmax_rows(mixed[h], None if sink is None else sink[h].double()) @ v[:m, h // per]
    return out.reshape(n, H * dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 2, 10, 6), (4, 4, 72, 136), (1, 1, 8, 8), (16, 4, 64, 64), (40, 8, 128, 128)])
def test_mixed_score_attention_kernel(dtype, sizes):
    """Prompt tiles (two sequences in one launch, one continuing at position 37) and single rows over several split counts against
    exact attention; a loud key far back that only the mixing matrix makes visible to its head; loud rows past the context."""
    k = K()
    H, G, dk, dv = sizes
    g = torch.Generator().manual_seed(H + dk)
    L, S = 160, 3
    scale = 1.5 * dk ** -0.5
    kc, vc = (torch.randn(S, L, G * dk, generator=g)).to(dtype), torch.randn(S, L, G * dv, generator=g).to(dtype)
    talk = (torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)).to(dtype)
    sink = torch.zeros(H, dtype=dtype)
    lens = [(2, 0, 101), (0, 37, 50)]
    n = sum(x[2] for x in lens)
    q = torch.randn(n, H * dk, generator=g).to(dtype)
    loud = torch.randn(dk, generator=g)
    kc[2, 2, :dk] = (loud * 3).to(dtype)         # position 2 of slot 2, first key head
    q[100, :dk] = (loud * 3).to(dtype)           # the last row of that sequence, first query head
    want, at = [], 0
    for slot, start, rows in lens:
        want.append(_talking_reference(q[at : at + rows], kc[slot, : start + rows], vc[slot, : start + rows], talk, sink, H, G, dk, dv, scale, start))
        at += rows
    want = torch.cat(want)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    kg, vg = kc.cuda(), vc.cuda()
    kg[2, 101:] = 25.0
    kg[0, 87:] = 25.0
    seqs = torch.tensor([(0, 101, 0, 2), (101, 50, 37, 0)], dtype=torch.int32, device="cuda")
    got = k.talk_attn(q.cuda(), kg.view(-1, G * dk), vg.view(-1, G * dv), seqs, 101, H, G, dk, dv, L, scale, 1, talk=talk.cuda(), sink=sink.cuda())
    assert rel_err(got, want) < tol, rel_err(got, want)
    if dtype == torch.bfloat16 and dk == dv and dk in (64, 128):
        # the same prompts on the tensor-core tiles: raw scores into fp32 planes, mixing in place, softmax and values from the planes
        for tk in (talk.cuda(), None):
            launches = k.launch_count()
            got = k.talk_attn(q.cuda(), kg.view(-1, G * dk), vg.view(-1, G * dv), seqs, 101, H, G, dk, dv, L, scale, 1, talk=tk, sink=sink.cuda(), context=101)
            assert k.launch_count() - launches == (3 if tk is not None else 2)
            if tk is not None:
                assert rel_err(got, want) < 3e-2, rel_err(got, want)
            else:
                k.TALK_PREFILL_MMA = False
                try:
                    other = k.talk_attn(q.cuda(), kg.view(-1, G * dk), vg.view(-1, G * dv), seqs, 101, H, G, dk, dv, L, scale, 1, sink=sink.cuda(), context=101)
                finally:
                    k.TALK_PREFILL_MMA = True
                assert rel_err(got, other) < 3e-2
    last = [100, 150]
    seqs1 = torch.tensor([(0, 1, 100, 2), (1, 1, 86, 0)], dtype=torch.int32, device="cuda")
    for splits in (1, 2, 4, 9):
        got = k.talk_attn(q[last].cuda(), kg.view(-1, G * dk), vg.view(-1, G * dv), seqs1, 1, H, G, dk, dv, L, scale, splits, talk=talk.cuda(), sink=sink.cuda())
        assert rel_err(got, want[last]) < tol, (splits, rel_err(got, want[last]))
    # without mixing and without a sink the same kernel is ordinary grouped attention
    got = k.talk_attn(q.cuda(), kg.view(-1, G * dk), vg.view(-1, G * dv), seqs, 101, H, G, dk, dv, L, scale, 1)
    plain = torch.cat([_talking_reference(q[:101], kc[2, :101], vc[2, :101], torch.eye(H), None, H, G, dk, dv, scale, 0),
                       _talking_reference(q[101:], kc[0, :87], vc[0, :87], torch.eye(H), None, H, G, dk, dv, scale, 37)])
    assert rel_err(got, plain) < tol


def test_the_sink_only_joins_the_denominator():
    """With one visible key the output is the value times 1 / (1 + exp(sink - score)): a sink that were scaled, counted twice or
    given a value would show."""
    k = K()
    H, G, dk, dv = 2, 1, 4, 3
    q = torch.tensor([[1.0, 0, 0, 0, 0, 2.0, 0, 0]], device="cuda")
    kc = torch.tensor([[[1.0, 0.5, 0, 0]]], device="cuda")
    vc = torch.tensor([[[1.0, 2.0, 3.0]]], device="cuda")
    sink = torch.tensor([0.7, -0.2], device="cuda")
    seqs = torch.tensor([(0, 1, 0, 0)], dtype=torch.int32, device="cuda")
    got = k.talk_attn(q, kc.view(-1, 4), vc.view(-1, 3), seqs, 1, H, G, dk, dv, 1, 0.5, 1, sink=sink).cpu().view(H, dv)
    for h, s in enumerate((0.5 * 1.0, 0.5 * 1.0)):
        want = vc.cpu().view(3) / (1 + math.exp(float(sink[h]) - s))
        assert (got[h] - want).abs().max() < 1e-6


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------
def _single(kind):
    """One-layer models: the mechanism with its norms and nothing else (no feed-forward; a sharp score scale)."""
    if kind == "attention":
        return config(width=24, vocab=31, groups=2, layers=[layer(talking(4, 2, 10, 6, rot_dims=6, scale=2.0), None)])
    return config(width=24, vocab=31, groups=2, layers=[layer(latent(kind, 3, 10, 6, 7, kv_rank=12, q_rank=9, scaling=(3.0, 16, 4.0, 1.0), scale=1.5), None)])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", [FIRST, SECOND, "attention"])
@pytest.mark.parametrize("cuts", [[37], [1] * 37, [2, 2, 3, 1, 17, 2, 8, 2], [36, 1]])
def test_each_mixer_alone(dtype, kind, cuts):
    """A prompt, single tokens, portions down to two tokens: every cut of the same tokens gives the oracle's logits, in a slot that
    another sequence has used."""
    cfg = _single(kind)
    w = checkpoint(cfg, 7)
    model = build(cfg, w, dtype, slots=3)
    poison(model)
    toks = tokens_for(cfg, 37, 8)
    want = O.forward(cfg, w, toks)
    got, at = [], 0
    for c in cuts:
        got.append(model.step(toks[at : at + c], [(1, at, c)]))
        at += c
    assert_close(torch.cat(got), want, dtype, (kind, cuts))


@pytest.mark.parametrize("cfg,seed", [(CFG_ODD, 11), (CFG_WIDE, 12), (CFG_TILES, 13)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_matches_oracle(cfg, seed, dtype):
    w = checkpoint(cfg, seed)
    model = build(cfg, w, dtype)
    toks = tokens_for(cfg, 90, seed)
    assert_close(model.step(toks, [(0, 0, len(toks))]), O.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_WIDE])
def test_layers_follow_the_oracle_one_by_one(cfg):
    w = checkpoint(cfg, 21)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, 33, 22)
    streams = []
    O.forward(cfg, w, toks, streams)
    model.trace = []
    model.step(toks, [(1, 0, len(toks))])
    assert len(model.trace) == len(streams)
    for i, (a, b) in enumerate(zip(model.trace, streams)):
        assert rel_err(a, b) < 1e-5, f"layer {i}"


@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_WIDE, CFG_TILES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decoding_token_by_token_equals_prefill(dtype, cfg):
    w = checkpoint(cfg, 31)
    model = build(cfg, w, dtype)
    poison(model)
    toks = tokens_for(cfg, 70, 32)
    want = O.forward(cfg, w, toks)
    got = torch.cat([model.step([t], [(1, p, 1)]) for p, t in enumerate(toks)])
    assert_close(got, want, dtype)


@pytest.mark.parametrize("portions", [[2, 2, 2, 30, 3, 34, 1, 35, 2], [109, 2], [1, 110], [5] * 22 + [1]])
@pytest.mark.parametrize("cfg", [CFG_ODD, CFG_WIDE])
def test_prompt_in_portions(portions, cfg):
    w = checkpoint(cfg, 41)
    model = build(cfg, w, torch.float32)
    toks = tokens_for(cfg, sum(portions), 42)
    want = O.forward(cfg, w, toks)
    got, at = [], 0
    for c in portions:
        got.append(model.step(toks[at : at + c], [(0, at, c)]))
        at += c
    assert rel_err(torch.cat(got), want) < 3e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_batch_equals_each_alone(dtype):
    """Three requests of unequal length as one batch (prompts together, then one token each, the shortest leaving first, the session
    growing from one slot) against the oracle's logits for each request alone."""
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_ODD
    w = checkpoint(cfg, 51)
    model = build(cfg, w, dtype, slots=1)
    session = Session(model, slots=1, max_seq_length=128)
    reqs = {"a": tokens_for(cfg, 50, 52), "b": tokens_for(cfg, 7, 53), "c": tokens_for(cfg, 31, 54)}
    cut = {"a": 40, "b": 2, "c": 30}
    want = {r: O.forward(cfg, w, t) for r, t in reqs.items()}
    out = session.step([(r, reqs[r][: cut[r]], None) for r in reqs])
    assert_close(out, torch.cat([want[r][: cut[r]] for r in reqs]), dtype, "prompts")
    at = dict(cut)
    got = {r: [] for r in reqs}
    while any(at[r] < len(reqs[r]) for r in reqs):
        live = [r for r in reqs if at[r] < len(reqs[r])]
        out = session.step([(r, [reqs[r][at[r]]], [0]) for r in live], end=[r for r in live if at[r] + 1 == len(reqs[r])])
        for i, r in enumerate(live):
            got[r].append(out[i : i + 1])
            at[r] += 1
    for r in reqs:
        assert_close(torch.cat(got[r]), want[r][cut[r] :], dtype, r)
    assert model.slots.in_use == 0 and model.slots.capacity >= 3


def test_freed_slots_are_reused_without_leftovers():
    """A long request fills a slot and ends; a shorter one takes the same slot, starting with a two-token portion; then both slots are
    freed and taken in the other order."""
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_WIDE
    w = checkpoint(cfg, 61)
    model = build(cfg, w, torch.float32, slots=2)
    session = Session(model, slots=2, max_seq_length=128)
    long_, short = tokens_for(cfg, 100, 62), tokens_for(cfg, 20, 63)
    session.step([("x", long_, [])], end=["x"])
    out = session.step([("y", short[:2], None)])
    out = torch.cat([out, session.step([("y", short[2:], None)])])
    assert session.live["y"][0] == 0
    assert rel_err(out, O.forward(cfg, w, short)) < 3e-5
    out = session.step([("z", long_[:60], [59])], end=["y"])
    out2 = session.step([("u", short, [19]), ("z", [long_[60]], [0])], end=["u", "z"])
    full = O.forward(cfg, w, long_)
    assert rel_err(out, full[59:60]) < 3e-5 and rel_err(out2, torch.stack([O.forward(cfg, w, short)[19], full[60]])) < 3e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_finds_a_far_token(dtype):
    """250 single-token steps behind a prompt of 450 through every split count the context passes, in a slot used before."""
    cfg = CFG_ODD
    w = checkpoint(cfg, 71)
    model = build(cfg, w, dtype, slots=2, max_seq=768)
    poison(model)
    toks = tokens_for(cfg, 700, 72)
    want = O.forward(cfg, w, toks)
    got = [model.step(toks[:450], [(1, 0, 450)], [449])]
    for p in range(450, 700):
        got.append(model.step([toks[p]], [(1, p, 1)]))
    assert_close(torch.cat(got), want[449:], dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_generate_entry_points(dtype):
    """Greedy generation through generate() (captured decode graph) and through the batch scheduler give the oracle's tokens."""
    from lit_gpt_b200.generate.base import generate
    from lit_gpt_b200.generate.serve import generate_batch

    cfg = CFG_ODD
    w = checkpoint(cfg, 91)
    prompt = tokens_for(cfg, 9, 91)
    seq = O.greedy(cfg, w, prompt, 14)
    model = build(cfg, w, dtype, slots=1, max_seq=64)
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
    assert [l for l in res.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    assert sorted(os.listdir(out)) == ["0.f32", "2.f32", "3.f32", "4.f32"]        # step 1 wanted nothing
    full = {k_: O.forward(cfg, w, t) for k_, t in (("a", a), ("b", b), ("c", c))}
    want = {0: torch.stack([full["a"][0], full["a"][36], full["b"][5]]), 2: torch.stack([full["a"][38], full["b"][7]]),
            3: full["a"][39:40], 4: full["c"][[0, 1, 63, 64, 69]]}
    got = {step: torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, cfg["vocab"])) for step in want}
    for step, ref in want.items():
        assert got[step].shape == ref.shape
    assert_close(torch.cat([got[s] for s in want]), torch.cat(list(want.values())), torch.float32 if dtype == "float32" else torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompts_on_the_tensor_cores_then_decoding(dtype):
    """Two unequal prompts in one step (bf16: the tensor-core tiles for every latent layer), one longer than a query tile, then single
    tokens for both while a third request arrives in portions."""
    from lit_gpt_b200.generate.serve import Session

    cfg = CFG_TILES
    w = checkpoint(cfg, 61)
    model = build(cfg, w, dtype)
    session = Session(model, slots=2, max_seq_length=256)
    a, b, c = tokens_for(cfg, 190, 62), tokens_for(cfg, 95, 63), tokens_for(cfg, 60, 64)
    want = {r: O.forward(cfg, w, t) for r, t in (("a", a), ("b", b), ("c", c))}
    out = session.step([("a", a[:160], [0, 63, 64, 127, 128, 159]), ("b", b[:65], [64])])
    assert_close(out, torch.cat([want["a"][[0, 63, 64, 127, 128, 159]], want["b"][64:65]]), dtype, "prompts")
    got = {"a": [], "b": [], "c": []}
    for i in range(30):
        entries = [("a", [a[160 + i]], [0]), ("b", [b[65 + i]], [0])]
        if i % 10 == 5:                       # c's portions of 20 tokens ride along with the single-token steps
            j = (i // 10) * 20
            entries.append(("c", c[j : j + 20], None))
        out = session.step(entries)
        got["a"].append(out[0:1]); got["b"].append(out[1:2])
        if len(entries) == 3:
            got["c"].append(out[2:])
    assert_close(torch.cat(got["a"]), want["a"][160:190], dtype, "a")
    assert_close(torch.cat(got["b"]), want["b"][65:95], dtype, "b")
    assert_close(torch.cat(got["c"]), want["c"], dtype, "c")


def test_generate_command_line(tmp_path):
    """`python -m lit_gpt_b200.generate.base` on a checkpoint directory without a tokenizer: a prompt of token ids in, the oracle's greedy
    continuation out."""
    import subprocess

    cfg = CFG_ODD
    w = checkpoint(cfg, 111)
    _write_checkpoint(tmp_path, cfg, w)
    prompt = tokens_for(cfg, 6, 112)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-m", "lit_gpt_b200.generate.base", " ".join(str(t) for t in prompt), "--checkpoint_dir", str(tmp_path),
                          "--precision", "32-true", "--temperature", "0", "--max_new_tokens", "9"], cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    printed = [int(t) for t in res.stdout.strip().splitlines()[-1].split()]
    assert printed == O.greedy(cfg, w, prompt, 9)
