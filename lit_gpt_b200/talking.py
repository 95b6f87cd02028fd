"""Grouped-head attention whose scores are mixed over the heads before the softmax ("talking heads"), over cached keys and values.

    q, k, v = W h + b;  q, k: per head x / sqrt(mean(x^2) + eps) * w (one weight vector for all query heads, one for all key heads),
              then rotary positions on the first rot.dims dimensions (pairs i, i + dims / 2 or 2i, 2i + 1 as the specification says);
    s_g(i, j)  = scale * q_g(i) . k_{g / (H / G)}(j);   s'_h = sum_g talk[h, g] s_g;
    p_h(i, j)  = exp(s'_h(i, j)) / (exp(sink) + sum_{j' <= i} exp(s'_h(i, j')))      sink = 0: an extra 1 in the denominator;
    out        = W_o concat_h(sum_j p_h(i, j) v_{h / (H / G)}(j)).

What a sequence keeps (``KeyValueCache``, one slot per live sequence): the normed, rotated keys and the values of all its positions.
The projections are vendor matrix products; norm + rotation + cache store (``K.head_rope``, one launch for q, k and v) and the
attention (``K.talk_attn``) are this library's kernels.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from .config import TalkingMixerSpec
from .latent import decode_splits
from .ragged import RaggedBatch


class KeyValueCache(nn.Module):
    """(slots, max_seq, G * dk) keys and (slots, max_seq, G * dv) values of one layer; slot = one live sequence."""

    def __init__(self, slots: int, max_seq: int, k_cols: int, v_cols: int, device=None, dtype=None) -> None:
        super().__init__()
        self.register_buffer("keys", torch.zeros((slots, max_seq, k_cols), device=device, dtype=dtype), persistent=False)
        self.register_buffer("values", torch.zeros((slots, max_seq, v_cols), device=device, dtype=dtype), persistent=False)

    @property
    def key_rows(self) -> torch.Tensor:
        return self.keys.view(-1, self.keys.shape[-1])

    @property
    def value_rows(self) -> torch.Tensor:
        return self.values.view(-1, self.values.shape[-1])


class TalkingHeadsAttention(nn.Module):
    def __init__(self, width: int, spec: TalkingMixerSpec, eps: float) -> None:
        super().__init__()
        self.spec, self.eps, self.width = spec, eps, width
        H, G, dk, dv = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        # fused projection: rows [0, H dk) queries, then G dk keys, then G dv values
        self.w_qkv = nn.Parameter(torch.empty((H + G) * dk + G * dv, width), requires_grad=False)
        self.b_qkv = nn.Parameter(torch.zeros((H + G) * dk + G * dv), requires_grad=False)
        self.q_norm = nn.Parameter(torch.ones(dk), requires_grad=False)
        self.k_norm = nn.Parameter(torch.ones(dk), requires_grad=False)
        self.talk = nn.Parameter(torch.eye(H), requires_grad=False)
        # the sink logit of every head (a constant of the design, kept as a tensor for the kernel); None: ordinary softmax
        self.sink = nn.Parameter(torch.full((H,), float(spec.sink_logit)), requires_grad=False) if spec.sink_logit is not None else None
        self.w_o = nn.Parameter(torch.empty(width, H * dv), requires_grad=False)
        self.cache: Optional[KeyValueCache] = None
        self._freq_cache: dict = {}

    def build_cache(self, slots: int, max_seq: int, device=None, dtype=None) -> KeyValueCache:
        s = self.spec
        return KeyValueCache(slots, max_seq, s.kv_heads * s.dim, s.kv_heads * s.vdim, device, dtype)

    def freq(self, device: torch.device) -> Optional[torch.Tensor]:
        rot = self.spec.rot
        if rot is None or rot.dims == 0:
            return None
        t = self._freq_cache.get(device)
        if t is None:
            t = self._freq_cache[device] = torch.tensor(rot.frequencies(), dtype=torch.float32, device=device)
        return t

    def forward(self, h: torch.Tensor, batch: RaggedBatch, shared=None) -> torch.Tensor:
        """h (n, width) in the matrix-product dtype -> (n, width)"""
        s, n, cache = self.spec, h.shape[0], self.cache
        if cache is None:
            raise TypeError("You need to call `set_kv_cache()` first")
        H, G, dk, dv = s.heads, s.kv_heads, s.dim, s.vdim
        qkv = F.linear(h, self.w_qkv, self.b_qkv)
        q, k, v = qkv[:, : H * dk], qkv[:, H * dk : (H + G) * dk], qkv[:, (H + G) * dk :]
        rot, fr = s.rot, self.freq(h.device)
        rd = rot.dims if fr is not None else 0
        il = rot.interleaved if fr is not None else True
        mag = rot.magnitude if fr is not None else 1.0
        K.head_rope(n, batch.row_pos, self.eps,
                    K.rope_seg(q, q, H, dk, norm_w=self.q_norm, freq=fr, rot_dims=rd, interleaved=il, mag=mag),
                    K.rope_seg(k, cache.key_rows, G, dk, norm_w=self.k_norm, freq=fr, rot_dims=rd, interleaved=il, mag=mag, out_rows=batch.cache_rows),
                    K.rope_seg(v, cache.value_rows, G, dv, out_rows=batch.cache_rows), dtype=h.dtype, device=h.device)
        splits = decode_splits(batch.context_hint, batch.seq_state.shape[0]) if batch.decode else 1
        y = K.talk_attn(q, cache.key_rows, cache.value_rows, batch.seq_state, batch.max_q_len, H, G, dk, dv, cache.keys.shape[1], s.scale, splits,
                        talk=self.talk, sink=self.sink, context=0 if batch.decode else batch.context_hint)
        return F.linear(y, self.w_o)
