"""Latent attention and its cache.

A latent-attention layer caches ONE vector of ``kv_rank`` numbers per position (the normalised down-projection of the
layer input) instead of keys and values; per head, keys and values are up-projections of that vector, and there is no
rotation.  Because only the latent is cached, a layer can be told to attend over the latents ANOTHER layer has cached
(``source``), with its own up-projections, queries and output projection.

Batches are ragged: a step carries the tokens of several sequences packed into one (n, d) matrix, described by a
``RaggedBatch`` (per row: cache slot and position; per sequence: first row, length, first position).  Prefill expands the
context's keys and values with one matrix product and runs the tiled kernel ``K.latent_prefill``; a step of single tokens
runs ``K.latent_decode``, which absorbs the up-projections and never materialises keys or values.

``RotaryLatentAttention`` is the variant with rotary positions: every head has `dim` unrotated and `rot_dim` rotated query / key
numbers; the rotated key part is ONE vector per position shared by all heads, rotated by its position and cached behind the
latent (cache rows are [latent | rotated key part]), so the absorbed decode only lengthens its dot products.  A learned sink
logit per head and a sigmoid output gate (per head or per output number, projected from the mixer's input) are options.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from .config import LatentMixerSpec, RotaryLatentSpec
from .ragged import RaggedBatch  # noqa: F401  (re-exported)

DECODE_KEYS_PER_SPLIT = 64
DECODE_MAX_SPLITS = 64


DECODE_TARGET_CTAS = 296   # two per SM


def decode_splits(context: int, rows: int = 1) -> int:
    """CTAs that share one (sequence, head tile) of a decode step over a context of at most `context` positions: 64-key ranges,
    but no more splits than it takes `rows` (sequences x head tiles) to fill the GPU twice."""
    return max(1, min(DECODE_MAX_SPLITS, -(-context // DECODE_KEYS_PER_SPLIT), max(1, DECODE_TARGET_CTAS // max(rows, 1))))


class LatentCache(nn.Module):
    """(slots, max_seq, kv_rank) latents of one layer; slot = one live sequence."""

    def __init__(self, slots: int, max_seq: int, kv_rank: int, device=None, dtype=None, extra: int = 0) -> None:
        """`extra`: numbers stored behind the latent in every row (a key part shared by the heads)."""
        super().__init__()
        self.register_buffer("latents", torch.zeros((slots, max_seq, kv_rank + extra), device=device, dtype=dtype), persistent=False)

    @property
    def rows(self) -> torch.Tensor:
        return self.latents.view(-1, self.latents.shape[-1])

    def reset_parameters(self) -> None:
        torch.nn.init.zeros_(self.latents)


class LatentAttention(nn.Module):
    def __init__(self, width: int, spec: LatentMixerSpec, eps: float, source: Optional["LatentAttention"] = None) -> None:
        super().__init__()
        self.spec, self.eps, self.width = spec, eps, width
        self.owns_latent = source is None
        self.__dict__["source"] = source if source is not None else self     # not a submodule: the owner registers its own cache
        H = spec.heads
        down_rows = spec.q_rank + (spec.kv_rank if self.owns_latent else 0)
        # fused down-projection: rows [0, q_rank) give the query latent, the rest (if any) the key-value latent
        self.w_down = nn.Parameter(torch.empty(down_rows, width), requires_grad=False)
        self.q_norm = nn.Parameter(torch.ones(spec.q_rank), requires_grad=False)
        self.kv_norm = nn.Parameter(torch.ones(spec.kv_rank), requires_grad=False) if self.owns_latent else None
        self.w_uq = nn.Parameter(torch.empty(H * spec.dim, spec.q_rank), requires_grad=False)
        # fused up-projection: rows [0, H * dim) keys, then H * vdim values
        self.w_ukv = nn.Parameter(torch.empty(H * (spec.dim + spec.vdim), spec.kv_rank), requires_grad=False)
        self.w_o = nn.Parameter(torch.empty(width, H * spec.vdim), requires_grad=False)
        self.cache: Optional[LatentCache] = None

    def build_cache(self, slots: int, max_seq: int, device=None, dtype=None) -> Optional[LatentCache]:
        return LatentCache(slots, max_seq, self.spec.kv_rank, device, dtype) if self.owns_latent else None

    @property
    def w_uk(self) -> torch.Tensor:
        return self.w_ukv[: self.spec.heads * self.spec.dim]

    @property
    def w_uv(self) -> torch.Tensor:
        return self.w_ukv[self.spec.heads * self.spec.dim :]

    def forward(self, h: torch.Tensor, batch: RaggedBatch, shared: Dict[int, torch.Tensor]) -> torch.Tensor:
        """h (n, width) in the matrix-product dtype -> (n, width).  `shared`: per-step scratch in which the owner of a latent
        leaves the gathered context for the layers that read it."""
        s, n = self.spec, h.shape[0]
        H = s.heads
        cache = self.source.cache
        if cache is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        down = F.linear(h, self.w_down)
        cq = torch.empty((n, s.q_rank), dtype=h.dtype, device=h.device)
        segs = [K.rms_seg(down[:, : s.q_rank], self.q_norm, cq, s.q_rank, False)]
        if self.owns_latent:   # the second half goes, normalised, straight into its cache rows
            segs.append(K.rms_seg(down[:, s.q_rank :], self.kv_norm, cache.rows, s.kv_rank, False, out_rows=batch.cache_rows))
        K.rms_rows(n, self.eps, *segs, in_dtype=h.dtype, out_dtype=h.dtype, device=h.device)
        q = F.linear(cq, self.w_uq)
        if batch.decode:
            tiles = -(-H // 16) if h.dtype == torch.bfloat16 and s.kv_rank % 32 == 0 and s.kv_rank <= 512 else H
            y = K.latent_decode(q, self.w_uk, self.w_uv, cache.latents, batch.row_slot, batch.row_pos, H, s.dim, s.vdim, s.scale,
                                decode_splits(batch.context_hint, n * tiles))
        else:
            key = id(self.source)
            ctx = shared.get(key)
            if ctx is None:
                ctx = shared[key] = K.gather_rows(cache.rows, batch.ctx_rows)
            kv = F.linear(ctx, self.w_ukv)
            y = K.latent_prefill(q, kv[:, : H * s.dim], kv[:, H * s.dim :], batch.seqs, batch.max_q_len, H, s.dim, s.vdim, s.scale)
        return F.linear(y, self.w_o)


class RotaryLatentAttention(nn.Module):
    """Latent attention with a rotated key part shared by the heads, optional sink and output gate (see the module text)."""

    def __init__(self, width: int, spec: RotaryLatentSpec, eps: float, source: Optional["RotaryLatentAttention"] = None) -> None:
        super().__init__()
        self.spec, self.eps, self.width = spec, eps, width
        self.owns_latent = source is None
        self.__dict__["source"] = source if source is not None else self     # not a submodule: the owner registers its own cache
        H = spec.heads
        self.gate_cols = {None: 0, "head": H, "element": H * spec.vdim}[spec.gate]
        self.kv_cols = spec.kv_rank + spec.rot_dim if self.owns_latent else 0
        # fused projection of the mixer's input: rows [0, q_rank) the query latent, then (own latents only) kv_rank latent rows and
        # rot_dim rows of the shared key part, then the gate rows
        self.w_down = nn.Parameter(torch.empty(spec.q_rank + self.kv_cols + self.gate_cols, width), requires_grad=False)
        self.q_norm = nn.Parameter(torch.ones(spec.q_rank), requires_grad=False)
        self.kv_norm = nn.Parameter(torch.ones(spec.kv_rank), requires_grad=False) if self.owns_latent else None
        self.w_uq = nn.Parameter(torch.empty(H * (spec.dim + spec.rot_dim), spec.q_rank), requires_grad=False)
        # fused up-projection: rows [0, H * dim) unrotated keys, then H * vdim values
        self.w_ukv = nn.Parameter(torch.empty(H * (spec.dim + spec.vdim), spec.kv_rank), requires_grad=False)
        self.sink = nn.Parameter(torch.zeros(H), requires_grad=False) if spec.sink else None
        self.w_o = nn.Parameter(torch.empty(width, H * spec.vdim), requires_grad=False)
        self.cache: Optional[LatentCache] = None
        self._freq_cache: dict = {}

    def build_cache(self, slots: int, max_seq: int, device=None, dtype=None) -> Optional[LatentCache]:
        return LatentCache(slots, max_seq, self.spec.kv_rank, device, dtype, extra=self.spec.rot_dim) if self.owns_latent else None

    def freq(self, device: torch.device) -> torch.Tensor:
        """Angular frequencies of the rotated pairs on `device` (fp32), made from the specification in double precision."""
        t = self._freq_cache.get(device)
        if t is None:
            t = self._freq_cache[device] = torch.tensor(self.spec.rot.frequencies(), dtype=torch.float32, device=device)
        return t

    @property
    def w_uk(self) -> torch.Tensor:
        return self.w_ukv[: self.spec.heads * self.spec.dim]

    @property
    def w_uv(self) -> torch.Tensor:
        return self.w_ukv[self.spec.heads * self.spec.dim :]

    def forward(self, h: torch.Tensor, batch: RaggedBatch, shared: Dict[int, torch.Tensor]) -> torch.Tensor:
        """h (n, width) in the matrix-product dtype -> (n, width)"""
        s, n = self.spec, h.shape[0]
        H, dn, dr, dv, r, qr = s.heads, s.dim, s.rot_dim, s.vdim, s.kv_rank, s.q_rank
        cache = self.source.cache
        if cache is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        down = F.linear(h, self.w_down)
        cq = torch.empty((n, qr), dtype=h.dtype, device=h.device)
        segs = [K.rms_seg(down[:, :qr], self.q_norm, cq, qr, False)]
        if self.owns_latent:   # the latent goes, normalised, straight into its cache rows
            segs.append(K.rms_seg(down[:, qr : qr + r], self.kv_norm, cache.rows[:, :r], r, False, out_rows=batch.cache_rows))
        K.rms_rows(n, self.eps, *segs, in_dtype=h.dtype, out_dtype=h.dtype, device=h.device)
        q = F.linear(cq, self.w_uq)
        fr, il, mag = self.freq(h.device), s.rot.interleaved, s.rot.magnitude
        turns = [K.rope_seg(q, q, H, dn + dr, freq=fr, rot_off=dn, rot_dims=dr, interleaved=il, mag=mag)]
        if self.owns_latent:   # the shared key part, rotated by its position, behind the latent
            turns.append(K.rope_seg(down[:, qr + r : qr + r + dr], cache.rows[:, r:], 1, dr, freq=fr, rot_dims=dr, interleaved=il, mag=mag,
                                    out_rows=batch.cache_rows))
        K.head_rope(n, batch.row_pos, self.eps, *turns, dtype=h.dtype, device=h.device)
        gate = down[:, qr + self.kv_cols :] if self.gate_cols else None
        if batch.decode:
            tiles = -(-H // 16) if h.dtype == torch.bfloat16 and r % 32 == 0 and dr % 32 == 0 and r <= 512 else H
            y = K.latent_decode(q, self.w_uk, self.w_uv, cache.latents, batch.row_slot, batch.row_pos, H, dn, dv, s.scale,
                                decode_splits(batch.context_hint, n * tiles), shared_dims=dr, sink=self.sink, gate=gate)
        else:
            key = id(self.source)
            ctx = shared.get(key)
            if ctx is None:
                ctx = shared[key] = K.gather_rows(cache.rows, batch.ctx_rows)
            kv = F.linear(ctx[:, :r], self.w_ukv)
            y = K.latent_prefill(q, kv[:, : H * dn], kv[:, H * dn :], batch.seqs, batch.max_q_len, H, dn + dr, dv, s.scale, k_shared=ctx[:, r:],
                                 sink=self.sink, gate=gate)
        return F.linear(y, self.w_o)
