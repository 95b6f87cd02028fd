"""Nulezen: a decoder-only model of PARALLEL blocks over an fp32 residual stream, normed by dynamic tanh, whose head is its embedding.

    x0 = embed[token] * embedding_scale                                                  (fp32)
    per layer run:  h = dyt(x);  x += ls1 * mixer(h) + ls2 * ff(h)                        dyt(x) = tanh(alpha x) * w + b
    logits = (embed . dyt_final(x)) * logit_scale

Mixers (``window.GatedWindowAttention``): sliding-window attention with a sigmoid output gate -- ``attention`` has a distance bias in
its scores and a gate per output number, ``attention_2`` biased projections, rotary positions on half-split pairs and a gate per head.
Feed-forwards: dense with xIELU (``moe.DenseMLP``), clamped gated experts chosen by the largest router logits plus a shared expert
(``moe.ClampedSparseExperts``), or none.  A run of consecutive layers may repeat with the same weights, every repetition with states
of its own; every pass t starts from  x <- W_in [x ; x0] + step[t].

The residual stream, the norm, scores and softmax, router and positions are fp32 whatever the matrix-product dtype is; the products go
to the vendor GEMM, everything else is this library's kernels: ``K.scaled_residual`` does a block's scaled residual sum and the next
block's norm in one elementwise launch (the norm needs no statistics).

Sequences live in slots: per layer run and slot the key / value rings of one window, so a sequence can be any length.  The model plugs
into the entry points the other slot-served models use: ``forward(idx, input_pos)`` for ``generate.base`` (single-token steps are
CUDA-graph capturable) and ``step`` over ragged batches for ``generate.serve.Session``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from . import kernels as K
from .config import ClampedMoESpec, DenseMLPSpec, NulezenConfig, NulezenLayerSpec
from .moe import ClampedSparseExperts, DenseMLP
from .ragged import RaggedBatch, SlotAllocator, SlotServed, state_batch
from .window import GatedWindowAttention


class DynamicTanh(nn.Module):
    """tanh(alpha x) * weight + bias: a norm without statistics (applied inside ``K.scaled_residual``)."""

    def __init__(self, width: int) -> None:
        super().__init__()
        self.alpha = nn.Parameter(torch.ones(1), requires_grad=False)
        self.weight = nn.Parameter(torch.ones(width), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(width), requires_grad=False)

    def terms(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return self.alpha, self.weight, self.bias


class NulezenBlock(nn.Module):
    def __init__(self, config: NulezenConfig, spec: NulezenLayerSpec) -> None:
        super().__init__()
        d = config.n_embd
        self.norm = DynamicTanh(d)
        self.mixer = GatedWindowAttention(d, spec.mixer, config.norm_eps)
        self.ls1 = nn.Parameter(torch.ones(d), requires_grad=False)
        if isinstance(spec.mlp, DenseMLPSpec):
            self.mlp: Optional[nn.Module] = DenseMLP(d, spec.mlp.ff, xielu=True)
        elif isinstance(spec.mlp, ClampedMoESpec):
            self.mlp = ClampedSparseExperts(d, spec.mlp)
        else:
            self.mlp = None
        self.ls2 = nn.Parameter(torch.ones(d), requires_grad=False) if self.mlp is not None else None

    def forward(self, x: torch.Tensor, act: torch.Tensor, batch: RaggedBatch, state: nn.Module, next_norm: Optional[DynamicTanh],
                cast: Optional[torch.Tensor]) -> None:
        """x fp32 (n, d) residual, updated in place; act (n, d) = this block's norm of x in the matrix-product dtype on entry, on exit
        the stream normed by `next_norm` (None: left as it is); cast: receives the new stream in the matrix-product dtype."""
        y = self.mixer(act, batch, state)
        ff = self.mlp(act) if self.mlp is not None else None
        shared = self.mlp.shared(act) if isinstance(self.mlp, ClampedSparseExperts) and self.mlp.shared is not None else None
        K.scaled_residual(x, y0=y, s0=self.ls1, y1=ff, y2=shared, s1=self.ls2, cast=cast, norm=next_norm.terms() if next_norm is not None else None,
                          act=act)


class Nulezen(SlotServed, nn.Module):

    def __init__(self, config: NulezenConfig) -> None:
        super().__init__()
        self.config = config
        d = config.n_embd
        self.embed = nn.Parameter(torch.empty(config.vocab_size, d), requires_grad=False)
        self.blocks = nn.ModuleList(NulezenBlock(config, spec) for spec in config.layers)
        self.final_norm = DynamicTanh(d)
        if config.looped:
            # the entry projection of a pass, split by what it reads: [stream | embedding]
            self.loop_in_x = nn.Parameter(torch.empty(d, d), requires_grad=False)
            self.loop_in_e = nn.Parameter(torch.empty(d, d), requires_grad=False)
            self.loop_step = nn.Parameter(torch.zeros(config.loop_times, d), requires_grad=False)
        self.runs = config.schedule()                       # (layer, state index, pass this run opens or -1)
        self._max_seq_length = config.block_size
        self.slots: Optional[SlotAllocator] = None
        self.states: Optional[nn.ModuleList] = None         # one state per layer RUN: a repeated layer has one per repetition
        self.trace: Optional[List[torch.Tensor]] = None     # debugging: set to a list to receive the stream after every layer run

    @property
    def head(self) -> torch.Tensor:
        return self.embed

    # ---- the surface generate() uses (with ``SlotServed``) --------------------------------------------------------
    def set_kv_cache(self, batch_size: int, rope_cache_length: Optional[int] = None, device: Optional[torch.device] = None,
                     dtype: Optional[torch.dtype] = None) -> None:
        """`batch_size` state slots for every layer run.  A state is constant in size: nothing depends on `max_seq_length`."""
        device = device if device is not None else self.device
        dtype = dtype if dtype is not None else self.dtype
        self.states = nn.ModuleList(self.blocks[layer].mixer.build_state(batch_size, device, dtype) for layer, _, _ in self.runs)
        self.slots = SlotAllocator(batch_size)
        self._drop_graphs()

    def clear_kv_cache(self) -> None:
        self.states = None
        self.slots = None
        self._drop_graphs()

    def reset_caches(self) -> None:
        for t in self.state_tensors():
            t.zero_()

    def state_tensors(self) -> List[torch.Tensor]:
        return [t for st in (self.states or []) for t in st.tensors()]

    def _apply(self, fn, recurse: bool = True):
        self._drop_graphs()
        return super()._apply(fn, recurse)

    # ---- weights ----------------------------------------------------------------------------------------------------
    def reset_parameters(self, seed: int = 1234, std: float = 0.02) -> None:
        """Random weights for benchmarks and smoke runs: N(0, std) matrices (the entry projection of a pass near [I | 0]), unit norm
        weights and layer scales, zero biases, a mild distance bias."""
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for name, p in self.named_parameters():
            leaf = name.rsplit(".", 1)[-1]
            if leaf in ("weight", "alpha", "ls1", "ls2") and p.dim() <= 1:
                p.data.fill_(1.0)
            elif leaf == "r1":
                p.data.fill_(0.5)
            elif leaf == "r2":
                p.data.fill_(1.0)
            elif p.dim() == 1 or leaf == "loop_step":
                p.data.zero_()
            else:
                p.data.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=gen))
                if leaf == "loop_in_x":
                    p.data.add_(torch.eye(p.shape[0], device=p.device, dtype=p.dtype))

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Fill the parameters from the checkpoint's tensors: ``embed``, ``final.norm`` (with ``.alpha`` and ``.b``), ``loop.in`` and
        ``loop.step`` of a looping model, and per layer i ``l<i>.norm1`` (``.alpha``, ``.b``), ``l<i>.ls1|ls2``, the mixer under
        ``l<i>.mix.`` (``q|k|v|g|o``, with ``.b`` biases or ``r1|r2`` as its kind has them) and the feed-forward under ``l<i>.mlp.``
        (``up|down|act``, or ``router``, ``router.b``, ``e<j>.gate|up|down`` and ``shared.gate|up|down``).  Projections that read the
        same input are stored fused, expert weights stacked."""
        used = set()

        def take(name: str) -> torch.Tensor:
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            return tensors[name]

        def put(param: nn.Parameter, value: torch.Tensor) -> None:
            if tuple(param.shape) != tuple(value.shape):
                raise ValueError(f"shape mismatch: parameter {tuple(param.shape)} vs checkpoint {tuple(value.shape)}")
            param.data.copy_(value)

        def put_norm(norm: DynamicTanh, name: str) -> None:
            put(norm.weight, take(name))
            put(norm.bias, take(name + ".b"))
            put(norm.alpha, take(name + ".alpha").reshape(1))

        d = self.config.n_embd
        put(self.embed, take("embed"))
        put_norm(self.final_norm, "final.norm")
        if self.config.looped:
            w_in = take("loop.in")
            if tuple(w_in.shape) != (d, 2 * d):
                raise ValueError(f"shape mismatch: loop.in {tuple(w_in.shape)} vs {(d, 2 * d)}")
            put(self.loop_in_x, w_in[:, :d])
            put(self.loop_in_e, w_in[:, d:])
            put(self.loop_step, take("loop.step"))
        else:
            used.update(n for n in ("loop.in", "loop.step") if n in tensors)    # a model that never loops has no use for them
        for i, block in enumerate(self.blocks):
            p, mx = f"l{i}.", block.mixer
            put_norm(block.norm, p + "norm1")
            put(block.ls1, take(p + "ls1"))
            q = p + "mix."
            names = [q + "q", q + "k", q + "v"] + ([q + "g"] if mx.gate_cols else [])
            put(mx.w_in, torch.cat([take(n) for n in names], dim=0))
            if mx.b_in is not None:   # the gate's projection has no bias
                bias = [take(n + ".b") for n in names[:3]]
                put(mx.b_in, torch.cat(bias + [torch.zeros(mx.gate_cols, dtype=bias[0].dtype)], dim=0))
            if mx.r1 is not None:
                put(mx.r1, take(q + "r1"))
                put(mx.r2, take(q + "r2"))
            put(mx.w_o, take(q + "o"))
            if block.mlp is None:
                used.update(n for n in (p + "ls2",) if n in tensors)
                continue
            put(block.ls2, take(p + "ls2"))
            m = p + "mlp."
            if isinstance(block.mlp, DenseMLP):
                put(block.mlp.w_up, take(m + "up"))
                put(block.mlp.w_down, take(m + "down"))
                put(block.mlp.act, take(m + "act"))
            else:
                E = block.mlp.spec.experts
                put(block.mlp.router.weight, take(m + "router"))
                put(block.mlp.router.correction, take(m + "router.b"))
                put(block.mlp.w_up, torch.stack([torch.cat([take(f"{m}e{j}.gate"), take(f"{m}e{j}.up")], dim=0) for j in range(E)]))
                put(block.mlp.w_down, torch.stack([take(f"{m}e{j}.down") for j in range(E)]))
                if block.mlp.shared is not None:
                    put(block.mlp.shared.w_up, torch.cat([take(m + "shared.gate"), take(m + "shared.up")], dim=0))
                    put(block.mlp.shared.w_down, take(m + "shared.down"))
        extra = sorted(set(tensors) - used)
        if extra:
            raise KeyError(f"unexpected tensors in the checkpoint: {extra[:6]}")

    # ---- one step ---------------------------------------------------------------------------------------------------
    def _mm(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """a (n, k) @ w (m, k)^T accumulated and returned in fp32"""
        return torch.mm(a, w.t()) if a.dtype == torch.float32 else torch.mm(a, w.t(), out_dtype=torch.float32)

    def _run(self, tokens: torch.Tensor, batch: RaggedBatch, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """tokens int32 (n,) -> fp32 logits (rows wanted or n, vocab)"""
        c = self.config
        n, runs = tokens.numel(), self.runs
        with self._true_fp32():
            x, emb = K.embed_pos(tokens, None, self.embed, None, c.embedding_scale)     # the stream and the embedding in the product dtype
            act = torch.empty_like(emb)
            cast = emb                                            # the stream in the product dtype, where a pass's entry reads it
            from_emb = self._mm(emb, self.loop_in_e) if c.looped else None     # the embedding's share of every pass's entry
            if not runs or runs[0][2] < 0:
                K.scaled_residual(x, norm=(self.blocks[runs[0][0]].norm if runs else self.final_norm).terms(), act=act)
            for r, (layer, state, opens) in enumerate(runs):
                block = self.blocks[layer]
                if opens >= 0:   # x <- W_in [x ; x0] + step[t], then this block's norm
                    x = self._mm(cast, self.loop_in_x)
                    K.scaled_residual(x, extra=from_emb, row_add=self.loop_step[opens], norm=block.norm.terms(), act=act)
                nxt, cast_out = None, None
                if r + 1 < len(runs):
                    if runs[r + 1][2] >= 0:
                        cast_out = cast = torch.empty_like(emb)
                    else:
                        nxt = self.blocks[runs[r + 1][0]].norm
                block(x, act, batch, self.states[state], nxt, cast_out)
                if self.trace is not None:
                    self.trace.append(x.clone())
            xw = x if want_rows is None else K.gather_rows(x, want_rows)
            xn = torch.empty(xw.shape, dtype=self.dtype, device=x.device)
            K.scaled_residual(xw, norm=self.final_norm.terms(), act=xn)
            return K.scale_f32(self._mm(xn, self.embed), c.logit_scale)

    @torch.inference_mode()
    def step(self, tokens: Sequence[int], seqs: Sequence[Tuple[int, int, int]], want: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One step over a ragged batch.  `tokens`: the new tokens of all sequences, sequence after sequence; `seqs`: per
        sequence (state slot, position of its first new token, number of new tokens); `want`: indices into `tokens` of the rows
        whose logits are returned (default: all).  Returns fp32 (rows, vocab).  A sequence's slot must hold the rings its earlier
        tokens left; a reused slot needs no clearing, since only a sequence's own positions are ever read."""
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        dev = self.device
        n = len(tokens)
        if n == 0 or n != sum(s[2] for s in seqs):
            raise ValueError("step: the sequence lengths must add up to the number of tokens (> 0)")
        for slot, start, length in seqs:
            if not 0 <= slot < self.slots.capacity or length <= 0 or start < 0 or start + length > self.max_seq_length:
                raise ValueError(f"step: sequence (slot {slot}, start {start}, length {length}) does not fit {self.slots.capacity} slots")
        batch, toks = state_batch(seqs, dev, tokens, positions=True)
        want_rows = None if want is None else torch.tensor(list(want), dtype=torch.int64).to(dev, non_blocking=True)
        return self._run(toks, batch, want_rows)

    def forward(self, idx: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """idx (B, T) token ids, batch row b = state slot b, all rows at the positions `input_pos` (T,), as ``GPT.forward``.
        Returns fp32 logits (B, T, vocab).  T = 1 runs without any host synchronisation (CUDA-graph capturable)."""
        B, T = idx.shape
        if input_pos is None:
            raise TypeError("Nulezen runs over its states: pass input_pos")
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        if B > self.slots.capacity:
            raise ValueError(f"batch of {B} rows, but only {self.slots.capacity} state slots")
        dev = idx.device
        const = self.__dict__.get("_const")
        if const is None or const[0].numel() < B or const[0].device != dev:
            slots = torch.arange(max(B, self.slots.capacity), dtype=torch.int32, device=dev)
            const = self.__dict__["_const"] = (slots, torch.ones_like(slots))
        ar = const[0][:B]
        pos32 = input_pos.to(torch.int32)
        if T == 1:
            seq_state = torch.stack([ar, const[1][:B], pos32.expand(B), ar], dim=1).contiguous()
            batch = RaggedBatch(row_pos=pos32.expand(B).contiguous(), row_slot=None, cache_rows=None, decode=True, context_hint=self.max_seq_length,
                                seq_state=seq_state, row_seq=ar)
            return self._run(idx.reshape(B).to(torch.int32), batch, None).view(B, 1, -1)
        start = int(input_pos[0])   # host read: the prompt's rows are laid out on the host
        if start + T > self.max_seq_length:
            raise ValueError(f"Cannot forward sequence of length {start + T}, max seq length is only {self.max_seq_length}.")
        seq_state = torch.tensor([(b * T, T, start, b) for b in range(B)], dtype=torch.int32).to(dev)
        batch = RaggedBatch(row_pos=pos32.repeat(B), row_slot=None, cache_rows=None, decode=False, context_hint=start + T, max_q_len=T,
                            seq_state=seq_state, identity_ctx=start == 0, row_seq=ar.repeat_interleave(T))
        return self._run(idx.reshape(B * T).to(torch.int32), batch, None).view(B, T, -1)
