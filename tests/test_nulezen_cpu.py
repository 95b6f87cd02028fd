"""Nulezen without a GPU: the configuration reader and its validation, the schedule of layer runs, the checkpoint loader (names, fused
rows, missing and unexpected tensors), the registry, and closed-form checks of the plain restatement the GPU tests compare with."""
from __future__ import annotations

import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import nulezen_oracle as O  # noqa: E402
from test_gpu_nulezen import CFG_ODD, CFG_TILES, CFG_WIDE, attn, attn2, checkpoint, config, dense, layer, moe  # noqa: E402

from lit_gpt_b200.config import ClampedMoESpec, DenseMLPSpec, NulezenConfig, architectures, load_config, model_class  # noqa: E402


def test_configuration_reads_every_size_and_constant():
    c = NulezenConfig.from_dict(CFG_ODD)
    assert (c.vocab_size, c.n_embd, c.embedding_scale, c.logit_scale, c.norm_eps) == (83, 42, 2.0, 0.7, 1e-5)
    assert (c.loop_start, c.loop_stop, c.loop_times, c.looped) == (1, 3, 3, True)
    m0, m1 = c.layers[0].mixer, c.layers[1].mixer
    assert (m0.heads, m0.kv_heads, m0.dim, m0.vdim, m0.window, m0.scale) == (4, 2, 12, 10, 7, 0.9)
    assert m0.distance and not m0.bias and m0.rot is None and m0.gate == "element"
    assert m1.bias and not m1.distance and m1.gate == "head" and (m1.rot.dims, m1.rot.base, m1.rot.interleaved) == (6, 100.0, False)
    assert isinstance(c.layers[0].mlp, DenseMLPSpec) and c.layers[0].mlp.ff == 50
    e = c.layers[1].mlp
    assert isinstance(e, ClampedMoESpec) and (e.experts, e.top, e.ff, e.limit, e.shared_ff, e.shared_limit) == (6, 2, 14, 1.2, 22, 0.8)
    assert c.layers[2].mlp is None and c.layers[3].mlp.shared_ff == 0
    w = NulezenConfig.from_dict(CFG_WIDE)
    assert not w.looped and w.embedding_scale == 1.0 and w.logit_scale == 1.0


def test_defaults_of_absent_keys():
    js = config(24, 11, [layer("attention", dict(heads=3, dim=8, mask=dict(size=4), scale=0.5), None)])
    del js["embedding"], js["logit_scale"]
    c = NulezenConfig.from_dict(js)
    m = c.layers[0].mixer
    assert (m.kv_heads, m.vdim) == (3, 8) and c.embedding_scale == 1.0 and c.logit_scale == 1.0 and not c.looped
    no_rot = config(24, 11, [layer("attention_2", attn(2, 1, 8, 8, size=4), None)])
    assert NulezenConfig.from_dict(no_rot).layers[0].mixer.rot is None


def test_schedule_of_layer_runs():
    runs = NulezenConfig.from_dict(CFG_ODD).schedule()
    assert [r[0] for r in runs] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [r[1] for r in runs] == list(range(8))                       # every run has a state of its own
    assert [r[2] for r in runs] == [-1, 0, -1, 1, -1, 2, -1, -1]        # the runs that open a pass
    runs = NulezenConfig.from_dict(CFG_TILES).schedule()
    assert [(r[0], r[2]) for r in runs] == [(0, 0), (1, -1), (0, 1), (1, -1), (2, -1)]
    assert [(r[0], r[2]) for r in NulezenConfig.from_dict(CFG_WIDE).schedule()] == [(0, -1), (1, -1), (2, -1)]


@pytest.mark.parametrize("bad", [
    lambda js: js["layers"][0].__setitem__("type", "attention_3"),
    lambda js: js["layers"][0]["mixer"].__setitem__("kv_heads", 3),
    lambda js: js["layers"][1]["mixer"]["rot"].__setitem__("dims", 7),
    lambda js: js["layers"][1]["mixer"]["rot"].__setitem__("dims", 12),
    lambda js: js["layers"][1]["mlp"]["router"].__setitem__("top", 7),
    lambda js: js["layers"][0]["mlp"].__setitem__("kind", "other"),
    lambda js: js["loop"].__setitem__("stop", 9),
])
def test_configuration_is_validated(bad):
    import copy

    js = copy.deepcopy(CFG_ODD)
    bad(js)
    with pytest.raises(ValueError):
        NulezenConfig.from_dict(js)


def test_registry_and_checkpoint_directory(tmp_path):
    import json

    assert "Nulezen" in architectures
    (tmp_path / "config.json").write_text(json.dumps(CFG_ODD))
    c = load_config(tmp_path)
    assert isinstance(c, NulezenConfig) and model_class(c).__name__ == "Nulezen"


def _cpu_model(cfg):
    from lit_gpt_b200.nulezen import Nulezen

    return Nulezen(NulezenConfig.from_dict(cfg))


def test_loader_fuses_projections_and_stacks_experts():
    w = checkpoint(CFG_ODD, 5)
    model = _cpu_model(CFG_ODD).to(torch.bfloat16)
    model.load_tensors(w)
    mx = model.blocks[1].mixer
    assert torch.equal(mx.w_in, torch.cat([w["l1.mix.q"], w["l1.mix.k"], w["l1.mix.v"], w["l1.mix.g"]]))
    assert torch.equal(mx.b_in[: -mx.gate_cols], torch.cat([w["l1.mix.q.b"], w["l1.mix.k.b"], w["l1.mix.v.b"]])) and not mx.b_in[-mx.gate_cols :].any()
    assert mx.gate_cols == 6 and model.blocks[0].mixer.gate_cols == 4 * 10 and model.blocks[0].mixer.b_in is None
    assert torch.equal(model.blocks[0].mixer.r2, w["l0.mix.r2"])
    e = model.blocks[1].mlp
    assert torch.equal(e.w_up[4], torch.cat([w["l1.mlp.e4.gate"], w["l1.mlp.e4.up"]])) and torch.equal(e.w_down[2], w["l1.mlp.e2.down"])
    assert torch.equal(e.router.correction, w["l1.mlp.router.b"]) and torch.equal(e.shared.w_up[22:], w["l1.mlp.shared.up"])
    assert torch.equal(torch.cat([model.loop_in_x, model.loop_in_e], dim=1), w["loop.in"]) and torch.equal(model.loop_step, w["loop.step"])
    assert torch.equal(model.final_norm.alpha.reshape(()), w["final.norm.alpha"]) and model.blocks[2].mlp is None and model.blocks[3].mlp.shared is None
    assert model.head is model.embed


def test_loader_rejects_missing_and_unexpected_tensors():
    w = checkpoint(CFG_WIDE, 6)
    model = _cpu_model(CFG_WIDE).to(torch.bfloat16)
    short = dict(w)
    del short["l1.mix.q.b"]
    with pytest.raises(KeyError):
        model.load_tensors(short)
    with pytest.raises(KeyError):
        model.load_tensors(dict(w, **{"l0.mix.q.b": torch.zeros(144, dtype=torch.bfloat16)}))
    with pytest.raises(ValueError):
        model.load_tensors(dict(w, **{"l0.ls1": torch.zeros(65, dtype=torch.bfloat16)}))
    model.load_tensors(w)


# ---- the restatement itself, on cases with a closed form ---------------------------------------------------------------------
def test_oracle_window_of_one_returns_the_value_and_gate_halves_at_zero():
    T, H, dk, dv = 5, 2, 4, 3
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(T, H, d, generator=g, dtype=torch.float64) for d in (dk, dk, dv))
    assert torch.allclose(O.windowed_softmax_attention(q, k, v, 1.0, 1), v)
    out = O.windowed_softmax_attention(q, k, v, 0.0, 3)          # flat scores: the mean of the visible values
    assert torch.allclose(out[4], v[2:5].mean(0))
    assert torch.allclose(out[1], v[0:2].mean(0))


def test_oracle_distance_penalty_and_rotation():
    v = torch.zeros(4, 1, 2, dtype=torch.float64)
    v[0, 0, 0] = v[3, 0, 1] = 1.0
    z = torch.zeros(4, 1, 3, dtype=torch.float64)
    out = O.windowed_softmax_attention(z, z, v, 1.0, 4, lambda h, dist: 0.5 * torch.log(1.0 + 2.0 * dist))
    assert abs(float(out[3, 0, 1] / out[3, 0, 0]) - (1.0 + 2.0 * 3) ** 0.5) < 1e-12
    x = torch.zeros(2, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0          # pair (0, 2) of dims = 4; dimensions 4, 5 pass
    x[:, 0, 5] = 3.0
    r = O.rotate_half_split(x, torch.tensor([0, 7]), 4, 100.0)
    assert torch.allclose(r[0], x[0]) and abs(float(r[1, 0, 0]) - math.cos(7.0)) < 1e-12 and abs(float(r[1, 0, 2]) - math.sin(7.0)) < 1e-12
    assert float(r[1, 0, 5]) == 3.0 and float(r[1, 0, 1]) == 0.0
    q = torch.randn(3, 1, 4, dtype=torch.float64)
    a, b = O.rotate_half_split(q, torch.tensor([5, 6, 7]), 4, 10.0), O.rotate_half_split(q, torch.tensor([105, 106, 107]), 4, 10.0)
    assert torch.allclose((a[2] * a[0]).sum(), (b[2] * b[0]).sum())      # scores depend on the distance only


def test_oracle_activations_and_router():
    z = torch.tensor([-1e-9, 0.0, 1e-9], dtype=torch.float64)
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.4, dtype=torch.float64)
    assert torch.allclose(O.xielu(z, p, q), 0.5 * z, atol=1e-15)                      # continuous at 0 with slope 1/2
    big = O.xielu(torch.tensor([3.0], dtype=torch.float64), p, q)
    assert abs(float(big) - (math.log1p(math.exp(0.3)) * 9.0 + 1.5)) < 1e-12
    W = {"gate": torch.eye(2, dtype=torch.float64), "up": torch.eye(2, dtype=torch.float64), "down": torch.eye(2, dtype=torch.float64)}
    h = torch.tensor([[5.0, -5.0]], dtype=torch.float64)
    out = O.clamped_expert(h, W, "", 1.0)
    assert abs(float(out[0, 0]) - (1.0 / (1.0 + math.exp(-1.702)) * 2.0)) < 1e-12     # gate capped at the limit, up at the limit, plus one
    assert abs(float(out[0, 1]) - (-5.0 / (1.0 + math.exp(5.0 * 1.702)) * 0.0)) < 1e-12     # up clamped to -limit: (u + 1) = 0
    R = {"router": torch.zeros(3, 2, dtype=torch.float64), "router.b": torch.tensor([0.0, math.log(3.0), -9.0], dtype=torch.float64)}
    ids, wts = O.route(h, R, "", 2)
    assert ids.tolist() == [[1, 0]] and torch.allclose(wts, torch.tensor([[0.75, 0.25]], dtype=torch.float64))


def test_small_configs_are_self_consistent():
    """A model without feed-forward and without loop runs through the restatement; the loop's entry changes the result."""
    cfg = config(16, 13, [layer("attention", attn(2, 1, 4, 4, size=3), None), layer("attention_2", attn2(2, 2, 4, 4, size=2, rot_dims=2), dense(8))])
    w = checkpoint(cfg, 2)
    toks = [1, 5, 2, 7, 7, 3]
    a = O.forward(cfg, w, toks)
    assert a.shape == (6, 13) and torch.isfinite(a).all()
    assert torch.allclose(O.forward(cfg, w, toks[:4]), a[:4])                          # causal
    looped = dict(cfg, loop=dict(start=0, stop=1, times=2))
    w2 = checkpoint(looped, 2)
    assert not torch.allclose(O.forward(looped, w2, toks), O.forward(cfg, w2, toks))
    m = moe(4, 2, 6, 0.9, shared=(5, 0.7))
    assert m["shared"] == dict(ff=5, limit=0.7)
