"""Sliding-window attention with an attention sink, over a ring of cached keys and values.

    q, k, v = W h + b;  each channel then passes a short causal convolution over time (``K.short_conv``);
    q, k    : rotary positions on the first rot.dims dimensions (interleaved pairs), then x / sqrt(mean(x^2) + eps) per head;
    p_ij    = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij')),  s_ij = scale * q_i . k_j,  over 0 <= i - j < window;
    out     = W_o concat_h(sum_j p_ij v_j) + b_o.

What a sequence keeps between steps (``WindowState``, one slot per live sequence): the last conv - 1 projected rows (the
convolution's tail) and the keys and values of its last `ring` >= window positions, position p in ring row p % ring.  The
projections are vendor matrix products; convolution, rotation, norm (one kernel), attention and the ring update are this
library's kernels.

``GatedWindowAttention`` is the same attention over the same rings (``RingState``) without convolution, norm or sink, and with

    s_ij   -= r1_h ln(1 + r2_h (i - j))                      (optional distance bias, two learned numbers per head)
    out     = W_o (concat_h(sum_j p_ij v_j) * sigmoid(W_g h))  (gate per output number, or one per head)

optional biases on q, k, v and optional rotary positions on half-split pairs (``K.head_rope``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from .config import GatedWindowSpec, WindowMixerSpec
from .ragged import RaggedBatch


class WindowState(nn.Module):
    """Per slot: conv tail (conv - 1, columns of q | k | v) and key / value rings (ring, kv_heads * dim | vdim)."""

    def __init__(self, slots: int, spec: WindowMixerSpec, device=None, dtype=None) -> None:
        super().__init__()
        cols = spec.heads * spec.dim + spec.kv_heads * (spec.dim + spec.vdim)
        self.ring = spec.window
        self.register_buffer("tail", torch.zeros((slots, max(spec.conv - 1, 1), cols), device=device, dtype=dtype), persistent=False)
        self.register_buffer("k_ring", torch.zeros((slots, self.ring, spec.kv_heads * spec.dim), device=device, dtype=dtype), persistent=False)
        self.register_buffer("v_ring", torch.zeros((slots, self.ring, spec.kv_heads * spec.vdim), device=device, dtype=dtype), persistent=False)

    def tensors(self):
        return [self.tail, self.k_ring, self.v_ring]


class WindowAttention(nn.Module):
    def __init__(self, width: int, spec: WindowMixerSpec, eps: float) -> None:
        super().__init__()
        self.spec, self.eps, self.width = spec, eps, width
        H, G, dk, dv = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        self.cols = H * dk + G * dk + G * dv
        # fused projection: rows [0, H dk) queries, then G dk keys, then G dv values; the convolution weights follow the same order
        self.w_qkv = nn.Parameter(torch.empty(self.cols, width), requires_grad=False)
        self.b_qkv = nn.Parameter(torch.zeros(self.cols), requires_grad=False)
        self.conv = nn.Parameter(torch.empty(self.cols, spec.conv), requires_grad=False)
        self.sink = nn.Parameter(torch.zeros(H), requires_grad=False)
        self.w_o = nn.Parameter(torch.empty(width, H * dv), requires_grad=False)
        self.b_o = nn.Parameter(torch.zeros(width), requires_grad=False)
        self._freq_cache: dict = {}

    def inv_freq(self, device: torch.device) -> Optional[torch.Tensor]:
        """Angular frequencies of the rotated pairs on `device`, in double precision (the kernel reduces position * frequency
        before the fp32 sine); made from the specification, so no cast or move of the module touches them."""
        rot = self.spec.rot
        if rot is None or rot.dims == 0:
            return None
        t = self._freq_cache.get(device)
        if t is None:
            t = self._freq_cache[device] = torch.tensor(rot.frequencies(), dtype=torch.float64, device=device)
        return t

    def build_state(self, slots: int, device=None, dtype=None) -> WindowState:
        return WindowState(slots, self.spec, device, dtype)

    def forward(self, h: torch.Tensor, batch: RaggedBatch, state: WindowState) -> torch.Tensor:
        """h (n, width) in the matrix-product dtype -> (n, width)"""
        s, n = self.spec, h.shape[0]
        H, G, dk, dv = s.heads, s.kv_heads, s.dim, s.vdim
        qkv = F.linear(h, self.w_qkv, self.b_qkv)
        out = torch.empty((n, self.cols), dtype=h.dtype, device=h.device)
        q, k, v = out[:, : H * dk], out[:, H * dk : (H + G) * dk], out[:, (H + G) * dk :]
        rot = s.rot
        rd = rot.dims if rot is not None else 0
        mag = rot.magnitude if rot is not None else 1.0
        cw, fr = self.conv, self.inv_freq(h.device)
        groups = [
            K.conv_group(cw[: H * dk], q, 0, H, dk, post=1, rot_dims=rd, inv_freq=fr, rot_mscale=mag, eps=self.eps),
            K.conv_group(cw[H * dk : (H + G) * dk], k, H * dk, G, dk, post=1, rot_dims=rd, inv_freq=fr, rot_mscale=mag, eps=self.eps),
            K.conv_group(cw[(H + G) * dk :], v, (H + G) * dk, G, dv),
        ]
        K.short_conv(qkv, groups, s.conv, state.tail, batch.seq_state, batch.row_seq)
        y = K.window_attn(q, k, v, state.k_ring, state.v_ring, self.sink, batch.seq_state, batch.row_seq, batch.max_q_len, H, G, dk, dv,
                          s.window, s.scale, from_start=batch.identity_ctx)
        return F.linear(y, self.w_o, self.b_o)


class RingState(nn.Module):
    """Per slot: key / value rings (ring, kv_heads * dim | vdim) of a sequence's last `ring` positions."""

    def __init__(self, slots: int, ring: int, k_cols: int, v_cols: int, device=None, dtype=None) -> None:
        super().__init__()
        self.ring = ring
        self.register_buffer("k_ring", torch.zeros((slots, ring, k_cols), device=device, dtype=dtype), persistent=False)
        self.register_buffer("v_ring", torch.zeros((slots, ring, v_cols), device=device, dtype=dtype), persistent=False)

    def tensors(self):
        return [self.k_ring, self.v_ring]


class GatedWindowAttention(nn.Module):
    def __init__(self, width: int, spec: GatedWindowSpec, eps: float = 0.0) -> None:
        super().__init__()
        self.spec, self.eps, self.width = spec, eps, width
        H, G, dk, dv = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        self.gate_cols = 0 if spec.gate is None else (H if spec.gate == "head" else H * dv)
        self.cols = H * dk + G * dk + G * dv + self.gate_cols
        # fused projection: rows [0, H dk) queries, then G dk keys, G dv values, then the gate's rows
        self.w_in = nn.Parameter(torch.empty(self.cols, width), requires_grad=False)
        self.b_in = nn.Parameter(torch.zeros(self.cols), requires_grad=False) if spec.bias else None
        self.r1 = nn.Parameter(torch.zeros(H), requires_grad=False) if spec.distance else None
        self.r2 = nn.Parameter(torch.zeros(H), requires_grad=False) if spec.distance else None
        self.w_o = nn.Parameter(torch.empty(width, H * dv), requires_grad=False)
        self._freq_cache: dict = {}

    def freq(self, device: torch.device) -> Optional[torch.Tensor]:
        """Angular frequencies of the rotated pairs on `device` (fp32; made from the specification, so no cast of the module touches them)."""
        rot = self.spec.rot
        if rot is None or rot.dims == 0:
            return None
        t = self._freq_cache.get(device)
        if t is None:
            t = self._freq_cache[device] = torch.tensor(rot.frequencies(), dtype=torch.float32, device=device)
        return t

    def build_state(self, slots: int, device=None, dtype=None) -> RingState:
        s = self.spec
        return RingState(slots, s.window, s.kv_heads * s.dim, s.kv_heads * s.vdim, device, dtype)

    def forward(self, h: torch.Tensor, batch: RaggedBatch, state: RingState) -> torch.Tensor:
        """h (n, width) in the matrix-product dtype -> (n, width)"""
        s, n = self.spec, h.shape[0]
        H, G, dk, dv = s.heads, s.kv_heads, s.dim, s.vdim
        proj = F.linear(h, self.w_in, self.b_in)
        q, k, v = proj[:, : H * dk], proj[:, H * dk : (H + G) * dk], proj[:, (H + G) * dk : (H + G) * dk + G * dv]
        gate = proj[:, (H + G) * dk + G * dv :] if self.gate_cols else None
        fr = self.freq(h.device)
        if fr is not None:
            rot = s.rot
            K.head_rope(n, batch.row_pos, self.eps,
                        K.rope_seg(q, q, H, dk, freq=fr, rot_dims=rot.dims, interleaved=rot.interleaved, mag=rot.magnitude),
                        K.rope_seg(k, k, G, dk, freq=fr, rot_dims=rot.dims, interleaved=rot.interleaved, mag=rot.magnitude),
                        dtype=h.dtype, device=h.device)
        y = K.window_attn(q, k, v, state.k_ring, state.v_ring, None, batch.seq_state, batch.row_seq, batch.max_q_len, H, G, dk, dv, s.window,
                          s.scale, from_start=batch.identity_ctx, dist=(self.r1, self.r2) if s.distance else None, gate=gate,
                          gate_per_head=s.gate == "head")
        return F.linear(y, self.w_o)
