"""Host-side parts of the Fizadra integration: configuration reader and registry, weight mapping on the CPU, rotary frequencies, and
closed-form checks of the plain restatement itself."""
from __future__ import annotations

import json
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import fizadra_oracle as O  # noqa: E402
from test_gpu_fizadra import CFG_ODD, CFG_WIDE, _write_checkpoint, checkpoint, tokens_for  # noqa: E402

from lit_gpt_b200.config import FizadraConfig, RotarySpec, load_config, model_class  # noqa: E402


def test_config_reader_and_registry(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG_ODD))
    cfg = load_config(tmp_path)
    assert isinstance(cfg, FizadraConfig) and cfg.n_layer == 6 and cfg.n_embd == 42 and cfg.norm_groups == 3
    assert model_class(cfg).__name__ == "Fizadra"
    a, l1, l2, l3 = (cfg.layers[i].mixer for i in range(4))
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.rot.dims, a.rot.interleaved, a.sink_logit) == (6, 2, 10, 6, 0.9, 6, False, 0.0)
    assert l1.sink and l1.gate == "element" and l1.rot.interleaved and l1.rot.factor == 3.0 and l1.kv_from is None and cfg.layers[1].mlp is None
    assert not l2.sink and l2.gate == "head" and not l2.rot.interleaved and l2.rot.factor is None
    assert l3.kv_from == 1 and cfg.layers[3].mlp.ff == 26


@pytest.mark.parametrize("edit,msg", [
    (lambda c: c["layers"][3]["mixer"].update(kv_from=4), "earlier latent-attention layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "earlier latent-attention layer"),     # layer 0 keeps keys and values, not latents
    (lambda c: c["layers"][4]["mixer"].update(kv_from=3), "earlier latent-attention layer"),     # layer 3 borrows its cache itself
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=16), "differ from those of layer 1"),
    (lambda c: (c["layers"][3]["mixer"].update(rot_dim=8), c["layers"][3]["mixer"]["rot"].update(dims=8)), "differ from those of layer 1"),
    (lambda c: c["layers"][3]["mixer"]["rot"].update(dims=4), "rotated whole"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "do not divide"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=12), "at most the head size"),
    (lambda c: c["norm"].update(groups=4), "do not divide the width"),
    (lambda c: c["layers"][2]["mlp"].update(kind="moe"), "unknown feed-forward"),
    (lambda c: c["layers"][0].update(type="convolution"), "unknown mixer"),
])
def test_config_validation(edit, msg):
    cfg = json.loads(json.dumps(CFG_ODD))
    edit(cfg)
    with pytest.raises(ValueError, match=msg):
        FizadraConfig.from_dict(cfg)


def test_rotary_frequencies_follow_the_restatement():
    for spec in (dict(dims=6, base=100.0, scaling=dict(factor=3.0, original=16, fast=4.0, slow=1.0)), dict(dims=32, base=1e4),
                 dict(dims=64, base=5e5, scaling=dict(factor=8.0, original=4096, fast=32.0, slow=1.0))):
        want, mag = O.rotary_frequencies(spec)
        got = RotarySpec.from_dict(spec, interleaved=False)
        assert torch.allclose(torch.tensor(got.frequencies(), dtype=torch.float64), want, rtol=1e-13) and got.magnitude == pytest.approx(mag)
        assert not got.interleaved


def test_loader_maps_names_and_fuses_projections(tmp_path):
    from lit_gpt_b200.checkpoint import load_registered

    w = checkpoint(CFG_ODD, 5)
    _write_checkpoint(tmp_path, CFG_ODD, w)
    model = load_registered(tmp_path, dtype=torch.float32, device="cpu")
    m1, m3, a = model.blocks[1].mixer, model.blocks[3].mixer, model.blocks[0].mixer
    assert m1.owns_latent and not m3.owns_latent and m3.source is m1 and model.blocks[4].mixer.source is model.blocks[2].mixer
    assert torch.equal(m1.w_down, torch.cat([w["l1.mix.dq"], w["l1.mix.dkv"], w["l1.mix.g"]]).float())
    assert torch.equal(m3.w_down, torch.cat([w["l3.mix.dq"], w["l3.mix.g"]]).float()) and m3.kv_norm is None
    assert torch.equal(m1.w_uk, w["l1.mix.uk"].float()) and torch.equal(m1.w_uv, w["l1.mix.uv"].float())
    assert torch.equal(m1.sink, w["l1.mix.sink"].float()) and model.blocks[2].mixer.sink is None
    assert torch.equal(a.w_qkv, torch.cat([w["l0.mix.q"], w["l0.mix.k"], w["l0.mix.v"]]).float()) and torch.equal(a.sink, torch.zeros(6))
    assert torch.equal(model.blocks[5].dwa, w["l5.dwa"].float()) and model.blocks[1].mlp is None and model.blocks[1].norm_2 is None
    missing = dict(w)
    del missing["l3.mix.sink"]
    _write_checkpoint(tmp_path, CFG_ODD, missing)
    with pytest.raises(KeyError, match="l3.mix.sink"):
        load_registered(tmp_path, dtype=torch.float32, device="cpu")
    extra = dict(w)
    extra["l3.mix.dkv"] = w["l1.mix.dkv"]
    _write_checkpoint(tmp_path, CFG_ODD, extra)
    with pytest.raises(KeyError, match="unexpected"):
        load_registered(tmp_path, dtype=torch.float32, device="cpu")


def test_restatement_closed_forms():
    """The plain restatement against hand-computed values: grouped norm, both pairings of the rotation, the sink's share."""
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64)
    got = O.group_norm(x, torch.tensor([1.0, 1.0, 2.0, 2.0], dtype=torch.float64), 0.0, 2)
    r1, r2 = math.sqrt(12.5), math.sqrt(2.0)
    assert torch.allclose(got, torch.tensor([[3 / r1, 4 / r1, 0.0, 4 / r2]], dtype=torch.float64))
    v = torch.zeros(2, 1, 4, dtype=torch.float64)
    v[1, 0] = torch.tensor([1.0, 0.0, 0.0, 0.0])
    spec = dict(dims=4, base=100.0)       # frequencies 1 and 0.1; row 1 is position 1
    il, hf = O.rotate(v, spec, True)[1, 0], O.rotate(v, spec, False)[1, 0]
    assert torch.allclose(il, torch.tensor([math.cos(1.0), math.sin(1.0), 0.0, 0.0], dtype=torch.float64))
    assert torch.allclose(hf, torch.tensor([math.cos(1.0), 0.0, math.sin(1.0), 0.0], dtype=torch.float64))
    p = O.causal_probabilities(torch.zeros(1, 2, 2, dtype=torch.float64), torch.tensor([math.log(2.0)], dtype=torch.float64))
    assert torch.allclose(p[0], torch.tensor([[1 / 3, 0.0], [0.25, 0.25]], dtype=torch.float64))


def test_depth_sum_weights_reach_back_to_the_embedding():
    """With the newest result's weight at zero in the last layer the logits cannot depend on that layer's own weights."""
    cfg = CFG_WIDE
    w = checkpoint(cfg, 9)
    last = len(cfg["layers"]) - 1
    w[f"l{last}.dwa"][-1] = 0.0
    toks = tokens_for(cfg, 6, 10)
    a = O.forward(cfg, w, toks)
    w2 = dict(w)
    w2[f"l{last}.mlp.down"] = w[f"l{last}.mlp.down"] * 3
    assert torch.equal(a, O.forward(cfg, w2, toks))
