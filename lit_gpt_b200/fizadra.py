"""Fizadra: a decoder-only model of blocks with GROUPED norms before and after each sublayer over an fp32 residual stream, whose
layers hand on a learned weighted sum over depth.

    X_0 = embed[token]                                                                     (fp32)
    layer i reads x (x = X_0 for the first):  x' = x + gnorm_1b(mixer(gnorm_1(x)));  X_{i+1} = x' + gnorm_2b(ff(gnorm_2(x')))
    what the next layer (or the head) reads:  x = sum_{j <= i+1} dwa_i[j] X_j
    logits = head(gnorm_final(x))

gnorm cuts a row into `norm_groups` equal consecutive pieces and divides each by its own root mean square before the weight.
Mixers: latent attention with a rotated key part in two variants (``latent.RotaryLatentAttention``; a layer may read another
layer's cached latents and rotated key part) and grouped-head attention with mixed scores (``talking.TalkingHeadsAttention``).
Feed-forward: dense with squared relu (``moe.DenseMLP``), or none.

The residual stream, every layer's result X_j, the sums over depth, norms and softmax are fp32 whatever the matrix-product dtype
is; the products go to the vendor GEMM, everything else is this library's kernels: ``K.depth_residual`` does a sublayer's
post-norm, the residual sum, the sum over depth and the next sublayer's pre-norm in one launch.

Sequences live in cache slots (per latent owner a ``LatentCache``, per attention layer a ``KeyValueCache``).  The model plugs into
the entry points ``Pomipel`` and ``Lefalix`` use: ``forward(idx, input_pos)`` for ``generate.base`` (single-token steps are
CUDA-graph capturable) and ``step`` over ragged batches for ``generate.serve.Session``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from .config import FizadraConfig, FizadraLayerSpec
from .latent import RotaryLatentAttention
from .moe import DenseMLP
from .ragged import RaggedBatch, SlotAllocator, SlotServed
from .talking import TalkingHeadsAttention


class FizadraBlock(nn.Module):
    def __init__(self, config: FizadraConfig, index: int, spec: FizadraLayerSpec, source: Optional[nn.Module]) -> None:
        super().__init__()
        d = config.n_embd
        if spec.type == "attention":
            self.mixer: nn.Module = TalkingHeadsAttention(d, spec.mixer, config.norm_eps)
        else:
            self.mixer = RotaryLatentAttention(d, spec.mixer, config.norm_eps, source)
        self.norm_1 = nn.Parameter(torch.ones(d), requires_grad=False)
        self.norm_1b = nn.Parameter(torch.ones(d), requires_grad=False)
        self.mlp = DenseMLP(d, spec.mlp.ff, K.ACT_RELU2) if spec.mlp is not None else None
        self.norm_2 = nn.Parameter(torch.ones(d), requires_grad=False) if self.mlp is not None else None
        self.norm_2b = nn.Parameter(torch.ones(d), requires_grad=False) if self.mlp is not None else None
        # weights of X_0 .. X_{index + 1} in what this layer hands on
        self.dwa = nn.Parameter(torch.zeros(index + 2), requires_grad=False)


class Fizadra(SlotServed, nn.Module):

    def __init__(self, config: FizadraConfig) -> None:
        super().__init__()
        self.config = config
        d = config.n_embd
        self.embed = nn.Parameter(torch.empty(config.vocab_size, d), requires_grad=False)
        blocks: List[FizadraBlock] = []
        for i, layer in enumerate(config.layers):
            src = None if getattr(layer.mixer, "kv_from", None) is None else blocks[layer.mixer.kv_from].mixer
            blocks.append(FizadraBlock(config, i, layer, src))
        self.blocks = nn.ModuleList(blocks)
        self.final_norm = nn.Parameter(torch.ones(d), requires_grad=False)
        self.head = nn.Parameter(torch.empty(config.vocab_size, d), requires_grad=False)
        self._max_seq_length = min(config.block_size, 4096)
        self.slots: Optional[SlotAllocator] = None
        self.trace: Optional[List[torch.Tensor]] = None     # debugging: set to a list to receive what every layer hands on

    # ---- the surface generate() uses (with ``SlotServed``) --------------------------------------------------------
    def set_kv_cache(self, batch_size: int, rope_cache_length: Optional[int] = None, device: Optional[torch.device] = None,
                     dtype: Optional[torch.dtype] = None) -> None:
        """`batch_size` cache slots of `max_seq_length` positions for every layer that keeps latents or keys and values of its own."""
        device = device if device is not None else self.device
        dtype = dtype if dtype is not None else self.dtype
        for block in self.blocks:
            block.mixer.cache = block.mixer.build_cache(batch_size, self.max_seq_length, device, dtype)
        self.slots = SlotAllocator(batch_size)
        self._drop_graphs()

    def clear_kv_cache(self) -> None:
        for block in self.blocks:
            block.mixer.cache = None
        self.slots = None
        self._drop_graphs()

    def reset_caches(self) -> None:
        for t in self.state_tensors():
            t.zero_()

    def _apply(self, fn, recurse: bool = True):
        self._drop_graphs()
        return super()._apply(fn, recurse)

    def state_tensors(self) -> List[torch.Tensor]:
        out: List[torch.Tensor] = []
        for b in self.blocks:
            c = b.mixer.cache
            if c is not None:
                out.extend([c.latents] if hasattr(c, "latents") else [c.keys, c.values])
        return out

    # ---- weights ----------------------------------------------------------------------------------------------------
    def reset_parameters(self, seed: int = 1234, std: float = 0.02) -> None:
        """Random weights for benchmarks and smoke runs: N(0, std) matrices, unit norms, zero biases and sinks, a head-mixing matrix
        near the identity, and a sum over depth that passes the newest result on."""
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for name, p in self.named_parameters():
            leaf = name.rsplit(".", 1)[-1]
            if leaf == "talk":
                p.data.copy_(torch.eye(p.shape[0], device=p.device) + torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, 0.05, generator=gen))
            elif leaf == "dwa":
                p.data.zero_()
                p.data[-1] = 1.0
            elif leaf == "sink" and isinstance(self.get_submodule(name.rsplit(".", 1)[0]), TalkingHeadsAttention):
                p.data.fill_(float(self.get_submodule(name.rsplit(".", 1)[0]).spec.sink_logit))     # a constant of the design
            elif "norm" in leaf:
                p.data.fill_(1.0)
            elif p.dim() == 1:
                p.data.zero_()
            else:
                p.data.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=gen))

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Fill the parameters from the checkpoint's tensors: ``embed``, ``final.norm``, ``head`` and per layer i ``l<i>.norm1|norm1b|
        norm2|norm2b|dwa``, the mixer under ``l<i>.mix.`` (latent: ``dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o`` and ``sink``, a borrowing layer
        without ``dkv``; attention: ``q|k|v`` with ``.b`` biases, ``q.norm|k.norm|talk|o``) and ``l<i>.mlp.up|down``.  Projections that
        read the same input are stored fused."""
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

        put(self.embed, take("embed"))
        put(self.final_norm, take("final.norm"))
        put(self.head, take("head"))
        for i, block in enumerate(self.blocks):
            p, mx = f"l{i}.", block.mixer
            put(block.norm_1, take(p + "norm1"))
            put(block.norm_1b, take(p + "norm1b"))
            put(block.dwa, take(p + "dwa"))
            q = p + "mix."
            if isinstance(mx, TalkingHeadsAttention):
                put(mx.w_qkv, torch.cat([take(q + "q"), take(q + "k"), take(q + "v")], dim=0))
                put(mx.b_qkv, torch.cat([take(q + "q.b"), take(q + "k.b"), take(q + "v.b")], dim=0))
                put(mx.q_norm, take(q + "q.norm"))
                put(mx.k_norm, take(q + "k.norm"))
                put(mx.talk, take(q + "talk"))
                if mx.sink is not None:
                    mx.sink.data.fill_(float(mx.spec.sink_logit))
                put(mx.w_o, take(q + "o"))
            else:
                rows = [take(q + "dq")] + ([take(q + "dkv")] if mx.owns_latent else []) + ([take(q + "g")] if mx.gate_cols else [])
                put(mx.w_down, torch.cat(rows, dim=0))
                put(mx.q_norm, take(q + "dq.norm"))
                if mx.owns_latent:
                    put(mx.kv_norm, take(q + "dkv.norm"))
                put(mx.w_uq, take(q + "uq"))
                put(mx.w_ukv, torch.cat([take(q + "uk"), take(q + "uv")], dim=0))
                if mx.sink is not None:
                    put(mx.sink, take(q + "sink"))
                put(mx.w_o, take(q + "o"))
            if block.mlp is None:
                used.update(n for n in (p + "norm2", p + "norm2b") if n in tensors)   # a layer without feed-forward has no use for them
                continue
            put(block.norm_2, take(p + "norm2"))
            put(block.norm_2b, take(p + "norm2b"))
            put(block.mlp.w_up, take(p + "mlp.up"))
            put(block.mlp.w_down, take(p + "mlp.down"))
        extra = sorted(set(tensors) - used)
        if extra:
            raise KeyError(f"unexpected tensors in the checkpoint: {extra[:6]}")

    # ---- one step ---------------------------------------------------------------------------------------------------
    def _run(self, tokens: torch.Tensor, batch: RaggedBatch, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """tokens int32 (n,) -> fp32 logits (rows wanted or n, vocab)"""
        c, eps, groups = self.config, self.config.norm_eps, self.config.norm_groups
        n, d, L = tokens.numel(), c.n_embd, len(self.blocks)
        with self._true_fp32():
            stack = torch.empty((L + 1, n, d), dtype=torch.float32, device=tokens.device)   # X_0 .. X_L of this step's rows
            _, act = K.embed_pos(tokens, None, self.embed, None, 1.0, x_out=stack[0])
            cur = stack[0]
            hand = [torch.empty((n, d), dtype=torch.float32, device=tokens.device) for _ in range(min(L, 2))]
            first = self.blocks[0].norm_1 if L else self.final_norm
            K.depth_residual(cur, cur, eps, groups, pre_w=first, act=act)
            shared: Dict[int, torch.Tensor] = {}
            for i, block in enumerate(self.blocks):
                nxt = self.blocks[i + 1].norm_1 if i + 1 < L else self.final_norm
                own, new = stack[i + 1], hand[i & 1]
                y = block.mixer(act, batch, shared)
                if block.mlp is not None:
                    K.depth_residual(cur, own, eps, groups, y=y, post_w=block.norm_1b, pre_w=block.norm_2, act=act)
                    K.depth_residual(own, own, eps, groups, y=block.mlp(act), post_w=block.norm_2b, stack=stack, m=i + 2, depth_w=block.dwa, avg=new,
                                     pre_w=nxt, act=act)
                else:
                    K.depth_residual(cur, own, eps, groups, y=y, post_w=block.norm_1b, stack=stack, m=i + 2, depth_w=block.dwa, avg=new, pre_w=nxt,
                                     act=act)
                cur = new
                if self.trace is not None:
                    self.trace.append(cur.clone())
            xn = act if want_rows is None else K.gather_rows(act, want_rows)
            return K.scale_f32(F.linear(xn, self.head), 1.0)

    @torch.inference_mode()
    def step(self, tokens: Sequence[int], seqs: Sequence[Tuple[int, int, int]], want: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One step over a ragged batch.  `tokens`: the new tokens of all sequences, sequence after sequence; `seqs`: per sequence
        (cache slot, position of its first new token, number of new tokens); `want`: indices into `tokens` of the rows whose logits
        are returned (default: all).  Returns fp32 (rows, vocab).  Every sequence's earlier positions must be in its slot already
        (a reused slot needs no clearing: nothing beyond a sequence's own positions is read)."""
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        dev, L = self.device, self.max_seq_length
        n = len(tokens)
        if n == 0 or n != sum(s[2] for s in seqs):
            raise ValueError("step: the sequence lengths must add up to the number of tokens (> 0)")
        row_pos, row_slot, seq_meta, seq_state, ctx_rows = [], [], [], [], []
        first = 0
        for slot, start, length in seqs:
            if not 0 <= slot < self.slots.capacity or length <= 0 or start < 0 or start + length > L:
                raise ValueError(f"step: sequence (slot {slot}, start {start}, length {length}) does not fit {self.slots.capacity} slots of {L}")
            row_pos.extend(range(start, start + length))
            row_slot.extend([slot] * length)
            seq_meta.extend((first, length, start, len(ctx_rows)))
            seq_state.extend((first, length, start, slot))
            ctx_rows.extend(range(slot * L, slot * L + start + length))
            first += length
        S = len(seqs)
        decode = all(s[2] == 1 for s in seqs)
        # the two per-sequence tables first: the kernels read their rows as 16-byte words
        i32 = torch.tensor(seq_meta + seq_state + list(tokens) + row_pos + row_slot, dtype=torch.int32).to(dev, non_blocking=True)
        cache_rows = [s * L + p for s, p in zip(row_slot, row_pos)]
        nw = 0 if want is None else len(want)
        i64 = torch.tensor(cache_rows + (list(want) if want is not None else []) + ([] if decode else ctx_rows), dtype=torch.int64).to(dev, non_blocking=True)
        t0 = 8 * S
        batch = RaggedBatch(row_pos=i32[t0 + n : t0 + 2 * n], row_slot=i32[t0 + 2 * n :], cache_rows=i64[:n], decode=decode,
                            context_hint=max(row_pos) + 1, max_q_len=max(s[2] for s in seqs), seqs=i32[: 4 * S].view(S, 4),
                            seq_state=i32[4 * S : t0].view(S, 4), ctx_rows=None if decode else i64[n + nw :])
        return self._run(i32[t0 : t0 + n], batch, i64[n : n + nw] if want is not None else None)

    def forward(self, idx: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """idx (B, T) token ids, batch row b = cache slot b, all rows at the positions `input_pos` (T,), as ``GPT.forward``.
        Returns fp32 logits (B, T, vocab).  T = 1 runs without any host synchronisation (CUDA-graph capturable)."""
        B, T = idx.shape
        if input_pos is None:
            raise TypeError("Fizadra runs over its caches: pass input_pos")
        if self.slots is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        if B > self.slots.capacity:
            raise ValueError(f"batch of {B} rows, but only {self.slots.capacity} cache slots")
        dev, L = idx.device, self.max_seq_length
        const = self.__dict__.get("_const")
        if const is None or const[0].numel() < B or const[0].device != dev:
            slots = torch.arange(max(B, self.slots.capacity), dtype=torch.int32, device=dev)
            const = self.__dict__["_const"] = (slots, slots.to(torch.int64) * L, torch.ones_like(slots))
        ar = const[0][:B]
        if T == 1:
            pos32 = input_pos.to(torch.int32).expand(B).contiguous()
            batch = RaggedBatch(row_pos=pos32, row_slot=ar, cache_rows=const[1][:B] + input_pos.to(torch.int64), decode=True, context_hint=L,
                                seq_state=torch.stack([ar, const[2][:B], pos32, ar], dim=1).contiguous())
            return self._run(idx.reshape(B).to(torch.int32), batch, None).view(B, 1, -1)
        start = int(input_pos[0])   # host read: sizes the context of the prompt's attention
        if start + T > L:
            raise ValueError(f"Cannot forward sequence of length {start + T}, max seq length is only {L}.")
        pos32 = input_pos.to(torch.int32)
        ctx = start + T
        batch = RaggedBatch(
            row_pos=pos32.repeat(B), row_slot=ar.repeat_interleave(T),
            cache_rows=(const[1][:B, None] + input_pos.to(torch.int64)[None, :]).reshape(-1), decode=False, context_hint=ctx,
            seqs=torch.tensor([(b * T, T, start, b * ctx) for b in range(B)], dtype=torch.int32).to(dev),
            seq_state=torch.tensor([(b * T, T, start, b) for b in range(B)], dtype=torch.int32).to(dev),
            ctx_rows=(const[1][:B, None] + torch.arange(ctx, device=dev)[None, :]).reshape(-1), max_q_len=T)
        return self._run(idx.reshape(B * T).to(torch.int32), batch, None).view(B, T, -1)
