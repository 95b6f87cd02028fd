"""Serving several requests over one model: the slot-managed cache, ragged steps, batched greedy / sampled generation, and
the replay of a recorded trace of steps.

``Session`` owns what a set of live requests needs: the model's caches (grown when more requests are live than there are
slots), one cache slot and the number of cached tokens per request.  ``Session.step`` is the one step function: every entry
brings the next tokens of a request, all entries run as one ragged batch (the model's ``step``), finished requests give their
slots back; the model is any that serves sequences from slots (``ragged.SlotServed`` with a ``step``: Pomipel, Lefalix).  ``generate_batch`` schedules prompts through it (prefill together, then one token per live request and step,
shorter requests leaving the batch early); ``Replayer`` feeds it recorded steps instead of sampled tokens.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from lit_gpt_b200 import kernels as K


class Session:
    def __init__(self, model: Any, slots: int = 4, max_seq_length: Optional[int] = None) -> None:
        self.model = model
        if max_seq_length is not None:
            model.max_seq_length = max_seq_length
        model.set_kv_cache(batch_size=max(1, slots))
        self.live: Dict[Any, List[int]] = {}    # request id -> [slot, cached tokens]

    def _grow(self) -> None:
        """Twice the slots, the live requests' caches and states carried over (slot numbers stay)."""
        model = self.model
        old = model.state_tensors()
        taken = {slot for slot, _ in self.live.values()}
        capacity = model.slots.capacity
        model.set_kv_cache(batch_size=2 * capacity)
        for new, prev in zip(model.state_tensors(), old):
            new[:capacity].copy_(prev)
        model.slots._free = [s for s in range(2 * capacity) if s not in taken]

    def step(self, entries: Sequence[Tuple[Any, Sequence[int], Optional[Sequence[int]]]], end: Iterable[Any] = ()) -> Optional[torch.Tensor]:
        """entries: (request id, its next tokens, places among them whose logits are wanted or None for all).  Returns the
        wanted logits, fp32 (rows, vocab), in the order of the entries -- None when nothing is wanted."""
        model = self.model
        tokens: List[int] = []
        seqs: List[Tuple[int, int, int]] = []
        want: List[int] = []
        for rid, toks, places in entries:
            if not toks:
                continue
            if rid not in self.live:
                if model.slots.in_use == model.slots.capacity:
                    self._grow()
                self.live[rid] = [model.slots.acquire(), 0]
            slot, cached = self.live[rid]
            places = range(len(toks)) if places is None else places
            want.extend(len(tokens) + int(p) for p in places)
            seqs.append((slot, cached, len(toks)))
            tokens.extend(int(t) for t in toks)
            self.live[rid][1] = cached + len(toks)
        logits = None
        if tokens:
            # rows nobody asks for still run (they fill the cache); without any wanted row the last one stands in and is dropped
            out = model.step(tokens, seqs, want if want else [len(tokens) - 1])
            logits = out if want else None
        for rid in end:
            state = self.live.pop(rid, None)
            if state is not None:
                model.slots.release(state[0])
        return logits


@torch.inference_mode()
def generate_batch(model: Any, prompts: Sequence[Sequence[int]], max_new_tokens: int, *, temperature: float = 0.0, top_k: Optional[int] = None,
                   eos_id: Optional[int] = None, session: Optional[Session] = None) -> List[List[int]]:
    """Generate up to `max_new_tokens` tokens for each prompt, all prompts as one batch: one ragged prefill step, then one token
    per live request and step; a request that produced `eos_id` or reached the cache's length leaves the batch and frees its
    slot.  Returns prompt + generated ids per request.  temperature 0: greedy."""
    from lit_gpt_b200.generate.base import _rng_for

    session = session if session is not None else Session(model, slots=len(prompts))
    dev = model.device
    out = [list(p) for p in prompts]
    ids = [("gen", i) for i in range(len(prompts))]
    token = torch.empty(1, dtype=torch.int64, device=dev)
    rng = _rng_for(dev) if temperature > 0.0 else None

    def draw(logits: torch.Tensor) -> List[int]:
        picked = []
        for r in range(logits.shape[0]):
            K.sample_(logits[r : r + 1], token, temperature, top_k, rng)
            picked.append(int(token))
        return picked

    live = list(range(len(prompts)))
    budget = [max_new_tokens] * len(prompts)
    nxt = draw(session.step([(ids[i], out[i], [len(out[i]) - 1]) for i in live])) if max_new_tokens > 0 else []
    while live:
        done = []
        for i, t in zip(live, nxt):
            out[i].append(t)
            budget[i] -= 1
            if budget[i] <= 0 or t == eos_id or len(out[i]) >= model.max_seq_length:
                done.append(i)
        live = [i for i in live if i not in done]
        if not live:
            session.step([], end=[ids[i] for i in done])
            break
        logits = session.step([(ids[i], [out[i][-1]], None) for i in live], end=[ids[i] for i in done])
        nxt = draw(logits)
    return out


class Replayer:
    """Feeds recorded steps ({"id", "tokens", "want"} entries, "end" lists) through a Session of the model in a directory."""

    def __init__(self, model_dir: Any, dtype: torch.dtype = torch.bfloat16, max_tokens: int = 0, device: Any = "cuda") -> None:
        from lit_gpt_b200.config import load_config, model_class

        config = load_config(Path(model_dir))
        cls = model_class(config)
        if not hasattr(cls, "step"):
            raise SystemExit(f"{cls.__name__} has no ragged step function: traces replay on models served through Session only")
        from lit_gpt_b200.checkpoint import load_registered

        self.model = load_registered(model_dir, dtype=dtype, device=device)
        bound = self.model.config.block_size
        if max_tokens and max_tokens < bound:
            # no request can be longer than what all live requests hold together: caches sized by position need no more than that
            self.model.max_seq_length = max_tokens
        slots = max(1, min(64, -(-max_tokens // self.model.max_seq_length))) if max_tokens else 2
        self.session = Session(self.model, slots=slots)

    def step(self, entries: Sequence[Dict[str, Any]], end: Iterable[Any] = ()) -> Optional[torch.Tensor]:
        return self.session.step([(e["id"], e.get("tokens", []), e.get("want", [])) for e in entries], end)
