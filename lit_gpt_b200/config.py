"""Model hyper-parameters: same public surface as the reference's ``lit_gpt/config.py:16-144`` (field names,
``from_name`` / ``from_json`` / ``from_checkpoint``, derived ``head_size`` / ``rope_n_elem`` /
``padded_vocab_size``) so a ``lit_config.json`` written by the reference loads unchanged.

The registry below holds the model families on the hot path named by BASELINE.json (pythia for the plumbing config,
Llama-2 / CodeLlama / Mistral / TinyLlama for the quantized decode configs); other families can be passed as kwargs
or through ``lit_config.json``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Literal, Optional, Tuple, Type, Union

import torch


def find_multiple(n: int, k: int) -> int:
    """Smallest multiple of k that is >= n (reference lit_gpt/utils.py find_multiple)."""
    return n if n % k == 0 else n + k - (n % k)


@dataclass
class Config:
    name: str = ""
    hf_config: dict = field(default_factory=dict)
    block_size: int = 4096
    vocab_size: int = 50254
    padding_multiple: int = 512
    padded_vocab_size: Optional[int] = None
    n_layer: int = 16
    n_head: int = 32
    n_embd: int = 4096
    rotary_percentage: float = 0.25
    parallel_residual: bool = True
    bias: bool = True
    lm_head_bias: bool = False
    # n_query_groups == n_head: MHA; 1: MQA; in between: GQA (reference config.py:31-51)
    n_query_groups: Optional[int] = None
    shared_attention_norm: bool = False
    _norm_class: Literal["LayerNorm", "RMSNorm"] = "LayerNorm"
    norm_eps: float = 1e-5
    _mlp_class: Literal["GptNeoxMLP", "LLaMAMLP"] = "GptNeoxMLP"
    gelu_approximate: str = "none"
    intermediate_size: Optional[int] = None
    rope_condense_ratio: int = 1
    rope_base: int = 10000
    n_expert: int = 0
    n_expert_per_token: int = 0

    def __post_init__(self) -> None:
        if not self.name:
            self.name = self.hf_config.get("name", self.name)
        assert self.n_embd % self.n_head == 0
        self.head_size = self.n_embd // self.n_head
        if self.padded_vocab_size is None:
            self.padded_vocab_size = find_multiple(self.vocab_size, self.padding_multiple)
        else:
            self.vocab_size = min(self.vocab_size, self.padded_vocab_size)
        if self.n_query_groups is not None:
            assert self.n_head % self.n_query_groups == 0
        else:
            self.n_query_groups = self.n_head
        if self.intermediate_size is None:
            if self._mlp_class == "LLaMAMLP":
                raise ValueError("The config needs to set the `intermediate_size`")
            self.intermediate_size = 4 * self.n_embd
        self.rope_n_elem = int(self.rotary_percentage * self.head_size)

    @classmethod
    def from_name(cls, name: str, **kwargs: Any) -> "Config":
        if name in name_to_config:
            conf = dict(name_to_config[name])
        else:
            matches = [c for c in configs if c["hf_config"]["name"] == name]
            if not matches:
                raise ValueError(f"{name!r} is not a supported config name")
            conf = dict(matches[0])
        if "condense_ratio" in kwargs:  # legacy key
            kwargs["rope_condense_ratio"] = kwargs.pop("condense_ratio")
        conf.update(kwargs)
        return cls(**conf)

    @classmethod
    def from_json(cls, path: Union[str, Path], **kwargs: Any) -> "Config":
        with open(path, encoding="utf-8") as fp:
            js = json.load(fp)
        for d in (js, kwargs):
            if "condense_ratio" in d:
                d["rope_condense_ratio"] = d.pop("condense_ratio")
        if "org" in js:
            js["hf_config"] = {"name": js["name"], "org": js.pop("org")}
        if "org" in kwargs:
            kwargs["hf_config"] = {"name": kwargs.get("name", js["name"]), "org": kwargs.pop("org")}
        js.update(kwargs)
        return cls(**js)

    @classmethod
    def from_checkpoint(cls, path: Path, **kwargs: Any) -> "Config":
        if (config_path := path / "lit_config.json").is_file():
            return cls.from_json(config_path, **kwargs)
        if (model_name := path.name) in name_to_config:
            return cls.from_name(model_name, **kwargs)
        raise FileNotFoundError(f"For {str(path)!r} neither 'lit_config.json' nor matching config exists.")

    @property
    def mlp_class(self) -> Type:
        import lit_gpt_b200.model as model

        return getattr(model, self._mlp_class)

    @property
    def norm_class(self) -> Type:
        if self._norm_class == "RMSNorm":
            from lit_gpt_b200.rmsnorm import RMSNorm

            return RMSNorm
        return getattr(torch.nn, self._norm_class)


# ---------------------------------------------------------------------------------------------------------
# registry
# ---------------------------------------------------------------------------------------------------------
configs: List[Dict[str, Any]] = []


def _add(name: str, org: str, hf_name: Optional[str] = None, **kw: Any) -> None:
    configs.append(dict(name=name, hf_config=dict(org=org, name=hf_name or name), **kw))


# EleutherAI Pythia (GPT-NeoX: LayerNorm, GELU MLP, bias, parallel residual, 25 % rotary)
_PYTHIA = {
    "pythia-14m": dict(block_size=512, n_layer=6, n_embd=128, n_head=4, padding_multiple=128),
    "pythia-31m": dict(block_size=1024, n_layer=6, n_embd=256, n_head=8, padding_multiple=128),
    "pythia-70m": dict(block_size=2048, n_layer=6, n_embd=512, n_head=8, padding_multiple=128),
    "pythia-160m": dict(block_size=2048, n_layer=12, n_embd=768, n_head=12, padding_multiple=128),
    "pythia-410m": dict(block_size=2048, n_layer=24, n_embd=1024, n_head=16, padding_multiple=128),
    "pythia-1b": dict(block_size=2048, n_embd=2048, n_head=8, padding_multiple=128),
    "pythia-1.4b": dict(block_size=2048, n_layer=24, n_embd=2048, n_head=16, padding_multiple=128),
    "pythia-2.8b": dict(block_size=2048, n_layer=32, n_embd=2560, padding_multiple=128),
    "pythia-6.9b": dict(block_size=2048, n_layer=32, padding_multiple=256),
    "pythia-12b": dict(block_size=2048, n_layer=36, n_embd=5120, n_head=40),
}
for _n, _kw in _PYTHIA.items():
    _add(_n, "EleutherAI", **_kw)
    if _n not in ("pythia-14m", "pythia-31m"):
        _add(f"{_n}-deduped", "EleutherAI", **_kw)

# Llama-family decoder: RMSNorm, SwiGLU MLP, no bias, sequential residual, full rotary
_LLAMA = dict(rotary_percentage=1.0, parallel_residual=False, bias=False, _norm_class="RMSNorm", _mlp_class="LLaMAMLP")
_LLAMA2 = {
    "7b": dict(n_layer=32, intermediate_size=11008),
    "13b": dict(n_layer=40, n_head=40, n_embd=5120, intermediate_size=13824),
    "70b": dict(n_layer=80, n_head=64, n_embd=8192, n_query_groups=8, intermediate_size=28672),
}
for _size, _kw in _LLAMA2.items():
    for _kind in ("", "-chat"):
        _add(f"Llama-2-{_size}{_kind}-hf", "meta-llama", vocab_size=32000, padding_multiple=64, **_LLAMA, **_kw)

_CODELLAMA = {
    "7b": dict(n_layer=32, intermediate_size=11008),
    "13b": dict(n_layer=40, n_head=40, n_embd=5120, intermediate_size=13824),
    "34b": dict(n_layer=48, n_head=64, n_embd=8192, n_query_groups=8, intermediate_size=22016),
}
for _size, _kw in _CODELLAMA.items():
    for _kind, _vocab in (("", 32016), ("-Python", 32000), ("-Instruct", 32016)):
        _v = 32000 if _size == "34b" else _vocab
        _add(f"CodeLlama-{_size}{_kind}-hf", "codellama", vocab_size=_v, padding_multiple=16, block_size=16384,
             rope_base=1000000, **_LLAMA, **_kw)

for _kind in ("", "Instruct-"):
    # block_size 4096: sliding-window attention is not implemented (same limit as the reference, config.py:1278)
    _add(f"Mistral-7B-{_kind}v0.1", "mistralai", padded_vocab_size=32000, block_size=4096, n_layer=32, n_query_groups=8,
         norm_eps=1e-05, intermediate_size=14336, **_LLAMA)

for _kind, _hf in (("", "-intermediate-step-1431k-3T"), ("-chat", "-Chat-v1.0")):
    _add(f"tiny-llama-1.1b{_kind}", "TinyLlama", hf_name=f"TinyLlama-1.1B{_hf}", block_size=2048, vocab_size=32000,
         padding_multiple=64, n_layer=22, n_head=32, n_embd=2048, n_query_groups=4, intermediate_size=5632, **_LLAMA)

name_to_config: Dict[str, Dict[str, Any]] = {c["name"]: c for c in configs}


# ---------------------------------------------------------------------------------------------------------
# Architectures described by a nested ``config.json`` (a list of layers, each with a mixer and an optional feed-forward)
# instead of the flat ``lit_config.json`` above.  ``load_config`` picks the configuration class by the file a checkpoint
# directory holds and its "architecture" key; ``model_class`` maps a configuration to the module that runs it.
# ---------------------------------------------------------------------------------------------------------
@dataclass
class LatentMixerSpec:
    """Latent attention: queries through a q_rank bottleneck, keys / values up-projected per head from a cached kv_rank latent."""

    heads: int
    dim: int                       # query-key size per head
    vdim: int                      # value size per head
    kv_rank: int
    q_rank: int
    scale: float                   # multiplies q . k
    kv_from: Optional[int] = None  # attend over that layer's cached latents instead of projecting own ones


@dataclass
class MoESpec:
    """Sparse experts with a sigmoid router: `top` of `experts` per token, chosen among the `keep` best of `groups` groups."""

    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1


@dataclass
class LayerSpec:
    type: str
    mixer: LatentMixerSpec
    mlp: Optional[MoESpec] = None


@dataclass
class PomipelConfig:
    """Pomipel: learned absolute positions, post-normed blocks (x += norm(branch(x)) with zero-centred norm weights) of latent
    attention and sparse experts, fp32 residual stream, scaled embedding and scaled logits."""

    name: str = "Pomipel"
    vocab_size: int = 0
    n_embd: int = 0
    block_size: int = 0            # size of the position table
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    layers: List[LayerSpec] = field(default_factory=list)

    def __post_init__(self) -> None:
        self.padded_vocab_size = self.vocab_size
        self.n_layer = len(self.layers)
        for i, layer in enumerate(self.layers):
            if layer.type != "latent_attention":
                raise ValueError(f"layer {i}: unknown mixer type {layer.type!r}")
            src = layer.mixer.kv_from
            if src is not None:
                if not (0 <= src < i) or self.layers[src].mixer.kv_from is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer that projects its own latents")
                if self.layers[src].mixer.kv_rank != layer.mixer.kv_rank:
                    raise ValueError(f"layer {i}: kv_rank differs from that of layer {src}, whose latents it reads")
            m = layer.mlp
            if m is not None and (m.experts % m.groups or not 0 < m.keep <= m.groups or m.keep * (m.experts // m.groups) < m.top):
                raise ValueError(f"layer {i}: expert groups {m.groups} / keep {m.keep} do not fit {m.experts} experts, top {m.top}")

    @classmethod
    def from_dict(cls, js: Dict[str, Any]) -> "PomipelConfig":
        layers = []
        for i, entry in enumerate(js["layers"]):
            mx = entry["mixer"]
            mixer = LatentMixerSpec(heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]), kv_rank=int(mx["kv_rank"]),
                                    q_rank=int(mx["q_rank"]), scale=float(mx["scale"]),
                                    kv_from=None if mx.get("kv_from") is None else int(mx["kv_from"]))
            mlp = None
            if entry.get("mlp") is not None:
                ml = entry["mlp"]
                if ml.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
                router, groups = ml["router"], ml["router"].get("groups") or {}
                mlp = MoESpec(experts=int(router["experts"]), top=int(router["top"]), ff=int(ml["expert"]["ff"]),
                              groups=int(groups.get("count", 1)), keep=int(groups.get("keep", groups.get("count", 1))))
            layers.append(LayerSpec(type=entry["type"], mixer=mixer, mlp=mlp))
        return cls(name=js.get("architecture", "Pomipel"), vocab_size=int(js["vocab"]), n_embd=int(js["width"]),
                   block_size=int(js["max_positions"]), norm_eps=float(js["norm"]["eps"]),
                   embedding_scale=float(js.get("embedding", {}).get("scale", 1.0)), logit_scale=float(js.get("logit_scale", 1.0)),
                   layers=layers)

    @classmethod
    def from_json(cls, path: Union[str, Path]) -> "PomipelConfig":
        with open(path, encoding="utf-8") as fp:
            return cls.from_dict(json.load(fp))


@dataclass
class RotarySpec:
    """Rotary positions on the first `dims` dimensions of a head, frequency base^(-2i / dims) for pair i; pairs are (2i, 2i + 1)
    when `interleaved`, else (i, i + dims / 2).  With `factor` set the frequencies are blended towards f / factor over a ramp
    between the dimensions whose wavelength fits `fast` and `slow` times into `original` positions (YaRN), and cos / sin are
    scaled by 0.1 ln(factor) + 1."""

    dims: int
    base: float
    factor: Optional[float] = None
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0
    interleaved: bool = True

    @classmethod
    def from_dict(cls, rot: Dict[str, Any], interleaved: bool = True) -> "RotarySpec":
        sc = rot.get("scaling") or {}
        return cls(dims=int(rot["dims"]), base=float(rot["base"]), factor=float(sc["factor"]) if sc else None,
                   original=float(sc.get("original", 0.0)), fast=float(sc.get("fast", 32.0)), slow=float(sc.get("slow", 1.0)),
                   interleaved=interleaved)

    def frequencies(self) -> List[float]:
        """Angular frequency of every pair, as Python floats (double precision)."""
        import math

        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        if self.factor is None:
            return f

        def pair_of(turns: float) -> float:   # the (fractional) pair index whose wavelength makes `turns` turns over `original`
            return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

        lo = max(math.floor(pair_of(self.fast)), 0)
        hi = min(math.ceil(pair_of(self.slow)), self.dims - 1)
        out = []
        for i, fi in enumerate(f):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / self.factor * ramp + fi * (1.0 - ramp))
        return out

    @property
    def magnitude(self) -> float:
        import math

        return 1.0 if self.factor is None else 0.1 * math.log(self.factor) + 1.0


@dataclass
class WindowMixerSpec:
    """Sliding-window attention with a sink: biased projections, a short convolution on q, k and v, rotary positions and a
    weightless per-head RMS norm on q and k."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                      # taps of the short convolution (1: none)
    window: int                    # a position sees itself and the window - 1 before it
    scale: float
    rot: Optional[RotarySpec] = None


@dataclass
class DeltaMixerSpec:
    """Gated delta rule: `heads` value heads of size vdim over `kv_heads` query / key heads of size dim; one decay per head, or
    (`channel`) one per head and key channel through a low-rank projection, with a low-rank sigmoid output gate."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    channel: bool = False
    decay_rank: int = 0            # inner size of the low-rank decay and gate projections (channel); read from the weights' shapes
    gate_rank: int = 0


@dataclass
class ParallelMixerSpec:
    left: WindowMixerSpec
    right: DeltaMixerSpec


@dataclass
class DenseMLPSpec:
    ff: int


@dataclass
class GatedMoESpec:
    """Softmax router over all experts, group-limited choice (a group ranks by its largest score), weights = the chosen scores;
    experts W_down (silu(W_gate h) * (W_up h))."""

    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1


@dataclass
class LefalixLayerSpec:
    type: str                      # "parallel" | "channel_delta"
    mixer: Any                     # ParallelMixerSpec | DeltaMixerSpec
    mlp: Any = None                # DenseMLPSpec | GatedMoESpec | None


@dataclass
class LefalixConfig:
    """Lefalix: blocks with RMS norms before and after each sublayer over an fp32 residual stream; mixers are a gated delta
    rule with per-channel decay, or sliding-window attention and a gated delta rule side by side; feed-forwards dense (gelu)
    or sparse gated experts.  Layers loop_start .. loop_stop - 1 run loop_times times with the same weights (each pass with
    its own state), the embedding re-entering before every pass but the first."""

    name: str = "Lefalix"
    vocab_size: int = 0
    n_embd: int = 0
    norm_eps: float = 1e-5
    layers: List[LefalixLayerSpec] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    block_size: int = 1 << 30      # no position table and constant-size state: positions are bounded by int32 only

    def __post_init__(self) -> None:
        self.padded_vocab_size = self.vocab_size
        self.n_layer = len(self.layers)
        if self.loop_times < 1 or not 0 <= self.loop_start <= self.loop_stop <= self.n_layer:
            raise ValueError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit {self.n_layer} layers")
        for i, layer in enumerate(self.layers):
            if layer.type not in ("parallel", "channel_delta"):
                raise ValueError(f"layer {i}: unknown mixer type {layer.type!r}")
            deltas = [layer.mixer.right] if layer.type == "parallel" else [layer.mixer]
            if layer.type == "parallel":
                w = layer.mixer.left
                if w.heads % w.kv_heads or w.window < 1 or w.conv < 1:
                    raise ValueError(f"layer {i}: bad window-attention shape")
                if w.rot is not None and (w.rot.dims % 2 or w.rot.dims > w.dim):
                    raise ValueError(f"layer {i}: rotary dimensions must be even and at most the head size")
            for m in deltas:
                if m.heads % m.kv_heads or m.conv < 1:
                    raise ValueError(f"layer {i}: bad delta-rule shape")
            m = layer.mlp
            if isinstance(m, GatedMoESpec) and (m.experts % m.groups or not 0 < m.keep <= m.groups or m.keep * (m.experts // m.groups) < m.top):
                raise ValueError(f"layer {i}: expert groups {m.groups} / keep {m.keep} do not fit {m.experts} experts, top {m.top}")

    def schedule(self) -> List[Tuple[int, int, bool]]:
        """The layer runs in order: (layer index, state index, first run of a repeated pass).  Every run has a state of its own."""
        runs: List[Tuple[int, int, bool]] = []
        order = [(i, False) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            order += [(i, t > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        order += [(i, False) for i in range(self.loop_stop, self.n_layer)]
        for n, (i, reenter) in enumerate(order):
            runs.append((i, n, reenter))
        return runs

    @staticmethod
    def _delta(mx: Dict[str, Any], channel: bool) -> DeltaMixerSpec:
        return DeltaMixerSpec(heads=int(mx["heads"]), kv_heads=int(mx["kv_heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
                              conv=int(mx.get("conv", 1)), channel=channel, decay_rank=int(mx.get("decay_rank", 0)),
                              gate_rank=int(mx.get("gate_rank", 0)))

    @classmethod
    def from_dict(cls, js: Dict[str, Any]) -> "LefalixConfig":
        layers = []
        for i, entry in enumerate(js["layers"]):
            mx, kind = entry["mixer"], entry["type"]
            if kind == "parallel":
                lf = mx["left"]
                rot = None
                if lf.get("rot") is not None:
                    r = lf["rot"]
                    sc = r.get("scaling")
                    rot = RotarySpec(dims=int(r["dims"]), base=float(r["base"])) if sc is None else RotarySpec(
                        dims=int(r["dims"]), base=float(r["base"]), factor=float(sc["factor"]), original=float(sc["original"]),
                        fast=float(sc["fast"]), slow=float(sc["slow"]))
                left = WindowMixerSpec(heads=int(lf["heads"]), kv_heads=int(lf["kv_heads"]), dim=int(lf["dim"]), vdim=int(lf["vdim"]),
                                       conv=int(lf.get("conv", 1)), window=int(lf["mask"]["size"]), scale=float(lf["scale"]), rot=rot)
                mixer: Any = ParallelMixerSpec(left=left, right=cls._delta(mx["right"], False))
            elif kind == "channel_delta":
                mixer = cls._delta(mx, True)
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            mlp: Any = None
            if entry.get("mlp") is not None:
                ml = entry["mlp"]
                if ml.get("kind") == "dense":
                    mlp = DenseMLPSpec(ff=int(ml["ff"]))
                elif ml.get("kind") == "moe":
                    router, groups = ml["router"], ml["router"].get("groups") or {}
                    mlp = GatedMoESpec(experts=int(router["experts"]), top=int(router["top"]), ff=int(ml["expert"]["ff"]),
                                       groups=int(groups.get("count", 1)), keep=int(groups.get("keep", groups.get("count", 1))))
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
            layers.append(LefalixLayerSpec(type=kind, mixer=mixer, mlp=mlp))
        loop = js.get("loop") or {}
        return cls(name=js.get("architecture", "Lefalix"), vocab_size=int(js["vocab"]), n_embd=int(js["width"]),
                   norm_eps=float(js["norm"]["eps"]), layers=layers, loop_start=int(loop.get("start", 0)),
                   loop_stop=int(loop.get("stop", loop.get("start", 0))), loop_times=int(loop.get("times", 1)))

    @classmethod
    def from_json(cls, path: Union[str, Path]) -> "LefalixConfig":
        with open(path, encoding="utf-8") as fp:
            return cls.from_dict(json.load(fp))


@dataclass
class RotaryLatentSpec:
    """Latent attention with a rotated key part: queries through a q_rank bottleneck, per head `dim` unrotated and `rot_dim` rotated
    query / key numbers; the unrotated keys and the values are up-projected from a cached kv_rank latent, the rotated key part is
    one vector per position shared by all heads and cached beside the latent.  `sink`: a learned logit per head in the softmax
    denominator; `gate`: sigmoid output gate per output number ("element") or per head ("head") or none."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotarySpec
    sink: bool = False
    gate: Optional[str] = None
    kv_from: Optional[int] = None


@dataclass
class TalkingMixerSpec:
    """Grouped-head attention with biased projections, a weighted RMS norm on every query and key head before the rotation,
    scores mixed over the heads by an (heads, heads) matrix before the softmax, and a softmax sink of logit `sink_logit` (0: an
    extra 1 in the denominator; None: none)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotarySpec] = None
    sink_logit: Optional[float] = 0.0


@dataclass
class FizadraLayerSpec:
    type: str                      # "latent_attention" | "latent_attention_2" | "attention"
    mixer: Any
    mlp: Optional[DenseMLPSpec] = None


@dataclass
class FizadraConfig:
    """Fizadra: blocks with grouped RMS norms before and after each sublayer over an fp32 residual stream; what a layer hands on
    is a learned weighted sum of the embedding and every layer's own result so far.  Mixers: two kinds of latent attention with a
    rotated key part (interleaved pairs, blended frequencies, sink and per-number gate; or half-split pairs and a per-head gate)
    and grouped-head attention with mixed scores; feed-forwards dense with squared relu, or none."""

    name: str = "Fizadra"
    vocab_size: int = 0
    n_embd: int = 0
    norm_eps: float = 1e-5
    norm_groups: int = 1
    layers: List[FizadraLayerSpec] = field(default_factory=list)
    block_size: int = 1 << 20      # no position table: the bound of a sequence is what the cache is sized for

    def __post_init__(self) -> None:
        self.padded_vocab_size = self.vocab_size
        self.n_layer = len(self.layers)
        if self.norm_groups < 1 or self.n_embd % self.norm_groups:
            raise ValueError(f"{self.norm_groups} norm groups do not divide the width {self.n_embd}")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type in ("latent_attention", "latent_attention_2"):
                if m.rot.dims != m.rot_dim or m.rot_dim % 2:
                    raise ValueError(f"layer {i}: the rotated part must be rotated whole and have an even size")
                src = m.kv_from
                if src is not None:
                    other = self.layers[src].mixer if 0 <= src < i else None
                    if not isinstance(other, RotaryLatentSpec) or other.kv_from is not None:
                        raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer that projects its own latents")
                    if (other.kv_rank, other.rot_dim) != (m.kv_rank, m.rot_dim):     # the rotated key part is taken as that cache holds it
                        raise ValueError(f"layer {i}: latent or rotated size differ from those of layer {src}, whose cache it reads")
            elif layer.type == "attention":
                if m.heads % m.kv_heads:
                    raise ValueError(f"layer {i}: {m.kv_heads} key heads do not divide {m.heads} query heads")
                if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                    raise ValueError(f"layer {i}: rotary dimensions must be even and at most the head size")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {layer.type!r}")

    @classmethod
    def from_dict(cls, js: Dict[str, Any]) -> "FizadraConfig":
        layers = []
        for i, entry in enumerate(js["layers"]):
            mx, kind = entry["mixer"], entry["type"]
            if kind in ("latent_attention", "latent_attention_2"):
                second = kind == "latent_attention_2"
                mixer: Any = RotaryLatentSpec(
                    heads=int(mx["heads"]), dim=int(mx["dim"]), rot_dim=int(mx["rot_dim"]), vdim=int(mx["vdim"]), kv_rank=int(mx["kv_rank"]),
                    q_rank=int(mx["q_rank"]), scale=float(mx["scale"]), rot=RotarySpec.from_dict(mx["rot"], interleaved=not second),
                    sink=not second, gate="head" if second else "element", kv_from=None if mx.get("kv_from") is None else int(mx["kv_from"]))
            elif kind == "attention":
                rot = mx.get("rot")
                mixer = TalkingMixerSpec(heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                                         vdim=int(mx.get("vdim", mx["dim"])), scale=float(mx["scale"]),
                                         rot=RotarySpec.from_dict(rot, interleaved=False) if rot and int(rot["dims"]) > 0 else None)
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            mlp = None
            if entry.get("mlp") is not None:
                if entry["mlp"].get("kind", "dense") != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {entry['mlp'].get('kind')!r}")
                mlp = DenseMLPSpec(ff=int(entry["mlp"]["ff"]))
            layers.append(FizadraLayerSpec(type=kind, mixer=mixer, mlp=mlp))
        return cls(name=js.get("architecture", "Fizadra"), vocab_size=int(js["vocab"]), n_embd=int(js["width"]), norm_eps=float(js["norm"]["eps"]),
                   norm_groups=int(js["norm"].get("groups", 1)), layers=layers)

    @classmethod
    def from_json(cls, path: Union[str, Path]) -> "FizadraConfig":
        with open(path, encoding="utf-8") as fp:
            return cls.from_dict(json.load(fp))


@dataclass
class GatedWindowSpec:
    """Sliding-window attention with a sigmoid output gate: optional biases on the q, k, v projections, optional rotary positions
    (half-split pairs) on q and k, an optional distance bias (score -= r1_h ln(1 + r2_h (i - j)), two learned numbers per head), and
    a gate per output number ("element") or per head ("head") projected from the mixer's input."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int                    # a position sees itself and the window - 1 before it
    scale: float
    rot: Optional[RotarySpec] = None
    bias: bool = False
    distance: bool = False
    gate: Optional[str] = "element"


@dataclass
class ClampedMoESpec:
    """Experts chosen by the largest biased router logits, weighted by a softmax among those `top` logits; expert:
    W_down (g sigmoid(alpha g) (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); optionally a shared expert of
    the same form (its own ff and limit) that every token uses."""

    experts: int
    top: int
    ff: int
    limit: float
    alpha: float = 1.702
    shared_ff: int = 0             # 0: no shared expert
    shared_limit: float = 0.0


@dataclass
class NulezenLayerSpec:
    type: str                      # "attention" (distance bias, gate per number) | "attention_2" (biases, rotary, gate per head)
    mixer: GatedWindowSpec
    mlp: Any = None                # DenseMLPSpec | ClampedMoESpec | None


@dataclass
class NulezenConfig:
    """Nulezen: parallel blocks over an fp32 residual stream -- one dynamic-tanh norm feeds the mixer and the feed-forward, whose results
    join the stream scaled per channel.  Mixers: two kinds of gated sliding-window attention; feed-forwards: dense with xIELU, or
    clamped gated experts with a shared expert.  With `loop_times` > 0 the layers loop_start .. loop_stop - 1 run loop_times times with
    the same weights (each pass with its own cache); every pass starts from a projection of [stream | embedding] plus a vector of the
    pass.  The head is the embedding table."""

    name: str = "Nulezen"
    vocab_size: int = 0
    n_embd: int = 0
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    layers: List[NulezenLayerSpec] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0            # 0: no loop (no entry projection either)
    block_size: int = 1 << 30      # constant-size state, no position table: positions are bounded by int32 only

    def __post_init__(self) -> None:
        self.padded_vocab_size = self.vocab_size
        self.n_layer = len(self.layers)
        if self.loop_times < 0 or not 0 <= self.loop_start <= self.loop_stop <= self.n_layer:
            raise ValueError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit {self.n_layer} layers")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type not in ("attention", "attention_2"):
                raise ValueError(f"layer {i}: unknown mixer type {layer.type!r}")
            if m.heads < 1 or m.kv_heads < 1 or m.heads % m.kv_heads or m.window < 1 or m.dim < 1 or m.vdim < 1:
                raise ValueError(f"layer {i}: bad attention shape")
            if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                raise ValueError(f"layer {i}: rotary dimensions must be even and at most the head size")
            if m.gate not in (None, "element", "head"):
                raise ValueError(f"layer {i}: unknown gate kind {m.gate!r}")
            e = layer.mlp
            if isinstance(e, ClampedMoESpec) and (not 0 < e.top <= e.experts or e.limit <= 0 or (e.shared_ff and e.shared_limit <= 0)):
                raise ValueError(f"layer {i}: bad expert shape (top {e.top} of {e.experts}, limits must be positive)")

    @property
    def looped(self) -> bool:
        return self.loop_times > 0 and self.loop_stop > self.loop_start

    def schedule(self) -> List[Tuple[int, int, int]]:
        """The layer runs in order: (layer index, state index, number of the pass this run opens or -1).  Every run has a state of
        its own."""
        if not self.looped:
            return [(i, i, -1) for i in range(self.n_layer)]
        order = [(i, -1) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            order += [(i, t if i == self.loop_start else -1) for i in range(self.loop_start, self.loop_stop)]
        order += [(i, -1) for i in range(self.loop_stop, self.n_layer)]
        return [(i, n, t) for n, (i, t) in enumerate(order)]

    @classmethod
    def from_dict(cls, js: Dict[str, Any]) -> "NulezenConfig":
        layers = []
        for i, entry in enumerate(js["layers"]):
            mx, kind = entry["mixer"], entry["type"]
            if kind not in ("attention", "attention_2"):
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            second = kind == "attention_2"
            rot = mx.get("rot") if second else None
            mixer = GatedWindowSpec(heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                                    vdim=int(mx.get("vdim", mx["dim"])), window=int(mx["mask"]["size"]), scale=float(mx["scale"]),
                                    rot=RotarySpec.from_dict(rot, interleaved=False) if rot and int(rot["dims"]) > 0 else None,
                                    bias=second, distance=not second, gate="head" if second else "element")
            mlp: Any = None
            ml = entry.get("mlp")
            if ml is not None:
                if ml.get("kind") == "dense":
                    mlp = DenseMLPSpec(ff=int(ml["ff"]))
                elif ml.get("kind") == "moe":
                    sh = ml.get("shared") or {}
                    mlp = ClampedMoESpec(experts=int(ml["router"]["experts"]), top=int(ml["router"]["top"]), ff=int(ml["expert"]["ff"]),
                                         limit=float(ml["expert"]["limit"]), shared_ff=int(sh.get("ff", 0)), shared_limit=float(sh.get("limit", 0.0)))
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
            layers.append(NulezenLayerSpec(type=kind, mixer=mixer, mlp=mlp))
        loop = js.get("loop") or {}
        return cls(name=js.get("architecture", "Nulezen"), vocab_size=int(js["vocab"]), n_embd=int(js["width"]), norm_eps=float(js["norm"]["eps"]),
                   embedding_scale=float((js.get("embedding") or {}).get("scale", 1.0)), logit_scale=float(js.get("logit_scale", 1.0)), layers=layers,
                   loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", loop.get("start", 0))), loop_times=int(loop.get("times", 0)))

    @classmethod
    def from_json(cls, path: Union[str, Path]) -> "NulezenConfig":
        with open(path, encoding="utf-8") as fp:
            return cls.from_dict(json.load(fp))


# "architecture" value of config.json -> (configuration class, "module:class" of the model)
architectures: Dict[str, Any] = {"Pomipel": (PomipelConfig, "lit_gpt_b200.pomipel:Pomipel"),
                                 "Lefalix": (LefalixConfig, "lit_gpt_b200.lefalix:Lefalix"),
                                 "Fizadra": (FizadraConfig, "lit_gpt_b200.fizadra:Fizadra"),
                                 "Nulezen": (NulezenConfig, "lit_gpt_b200.nulezen:Nulezen")}


def load_config(checkpoint_dir: Union[str, Path], **kwargs: Any) -> Any:
    """The configuration of a checkpoint directory: ``lit_config.json`` (-> Config, as ``Config.from_checkpoint``) or a
    ``config.json`` whose "architecture" names an entry of ``architectures``."""
    path = Path(checkpoint_dir)
    if (path / "lit_config.json").is_file() or not (path / "config.json").is_file():
        return Config.from_checkpoint(path, **kwargs)
    with open(path / "config.json", encoding="utf-8") as fp:
        js = json.load(fp)
    arch = js.get("architecture")
    if arch not in architectures:
        raise ValueError(f"{str(path / 'config.json')!r}: unknown architecture {arch!r} (known: {sorted(architectures)})")
    return architectures[arch][0].from_dict(js)


def model_class(config: Any) -> Type:
    """The module class that runs `config`: GPT for the flat configurations, else the registered class of its architecture."""
    import importlib

    if isinstance(config, Config):
        from lit_gpt_b200.model import GPT

        return GPT
    for cfg_cls, target in architectures.values():
        if isinstance(config, cfg_cls):
            mod, _, name = target.partition(":")
            return getattr(importlib.import_module(mod), name)
    raise TypeError(f"no model is registered for {type(config).__name__}")
