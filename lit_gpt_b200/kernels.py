"""Tensor-level wrappers over the C ABI (``include/b200gpt.h``): argument checking, output allocation, workspaces.

Every function launches on torch's current CUDA stream and never synchronises, so calls are capturable in a CUDA
graph.  CUDA tensors only — no CPU path exists (``B200Error`` is raised instead).
"""
from __future__ import annotations

import ctypes
import functools
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch._dynamo

from . import _cabi as C
from ._cabi import ACT_GELU, ACT_GELU_TANH, ACT_RELU2, ACT_SILU  # noqa: F401  (activation kinds of activation_ / glu)

QTYPES = {"nf4": C.Q_NF4, "fp4": C.Q_FP4, "int4": C.Q_INT4}
_workspaces: Dict[Tuple[str, int], torch.Tensor] = {}


def _ws(kind: str, device: torch.device, nbytes: int) -> torch.Tensor:
    """Persistent zero-initialised workspace per (kind, device).  Split-K counters inside are self-cleaning."""
    key = (kind, device.index if device.index is not None else torch.cuda.current_device())
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise C.B200Error(f"workspace '{kind}' must be allocated before CUDA-graph capture (run one eager step first)")
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _bf16c(t: Optional[torch.Tensor], name: str) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != torch.bfloat16:
        raise C.B200Error(f"{name} must be bfloat16 (got {t.dtype}); the kernels compute in bf16 with fp32 accumulation")
    return t if t.is_contiguous() else t.contiguous()


# ---------------------------------------------------------------------------------------------------------
# quantisation
# ---------------------------------------------------------------------------------------------------------
def quantize_4bit(w: torch.Tensor, quant_type: str = "nf4", blocksize: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (packed uint8 [(numel+1)//2, 1], absmax fp32 [ceil(numel/blocksize)]) — bitsandbytes Params4bit layout."""
    C.require_cuda(w)
    if w.dtype not in C.DTYPE_CODE:
        raise C.B200Error(f"quantize_4bit: unsupported dtype {w.dtype}")
    w = w.contiguous()
    n = w.numel()
    packed = torch.empty(((n + 1) // 2, 1), dtype=torch.uint8, device=w.device)
    absmax = torch.empty(((n + blocksize - 1) // blocksize,), dtype=torch.float32, device=w.device)
    C.check(C.load().b200_quantize_4bit(w.data_ptr(), C.DTYPE_CODE[w.dtype], n, blocksize, QTYPES[quant_type],
                                        packed.data_ptr(), absmax.data_ptr(), C.stream_ptr(w.device)), "quantize_4bit")
    return packed, absmax


def dequantize_4bit(packed: torch.Tensor, absmax: torch.Tensor, shape, dtype: torch.dtype = torch.bfloat16,
                    quant_type: str = "nf4", blocksize: int = 64) -> torch.Tensor:
    C.require_cuda(packed, absmax)
    out = torch.empty(tuple(shape), dtype=dtype, device=packed.device)
    C.check(C.load().b200_dequantize_4bit(packed.data_ptr(), absmax.data_ptr(), out.numel(), blocksize, QTYPES[quant_type],
                                          out.data_ptr(), C.DTYPE_CODE[dtype], C.stream_ptr(packed.device)), "dequantize_4bit")
    return out


_dynamic_map_cache: Dict[int, torch.Tensor] = {}


def dynamic_map(device: torch.device) -> torch.Tensor:
    """bitsandbytes' 256-entry signed 8-bit "dynamic" code (functional.create_dynamic_map(signed=True, 7, 8)), sorted."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _dynamic_map_cache:
        import numpy as np

        f32 = np.float32
        data = []
        for i in range(7):
            items = int(2 ** i + 1)
            b = np.linspace(0.1, 1, items, dtype=f32)
            means = ((b[:-1] + b[1:]) / f32(2.0)).astype(f32)
            scale = 10 ** (-6 + i)
            data += (scale * means.astype(np.float64)).tolist() + (-scale * means.astype(np.float64)).tolist()
        data += [0, 1.0]
        data += [0] * (256 - len(data))
        data.sort()
        _dynamic_map_cache[key] = torch.tensor(np.array(data, dtype=f32), device=device)
    return _dynamic_map_cache[key]


def double_quant_absmax(absmax: torch.Tensor, offset: Optional[float] = None):
    """-> (q uint8 [n], absmax2 fp32 [ceil(n/256)], offset float, absmax_dequantised fp32 [n])  (SURVEY Q2)."""
    C.require_cuda(absmax)
    absmax = absmax.contiguous().float()
    n = absmax.numel()
    if offset is None:
        offset = float(absmax.mean())
    q = torch.empty(n, dtype=torch.uint8, device=absmax.device)
    a2 = torch.empty((n + 255) // 256, dtype=torch.float32, device=absmax.device)
    deq = torch.empty_like(absmax)
    code = dynamic_map(absmax.device)
    C.check(C.load().b200_double_quant_absmax(absmax.data_ptr(), n, code.data_ptr(), offset, q.data_ptr(), a2.data_ptr(), deq.data_ptr(),
                                              C.stream_ptr(absmax.device)), "double_quant_absmax")
    return q, a2, offset, deq


def dequant_absmax(qabs: torch.Tensor, absmax2: torch.Tensor, offset: float) -> torch.Tensor:
    """Load-time inverse of ``double_quant_absmax`` for pre-quantized checkpoints: fp32 absmax = code[q] * absmax2[i // 256]
    + offset with the kernel's two separate roundings (csrc/quantize.cu), so a reloaded module streams identical statistics."""
    C.require_cuda(qabs, absmax2)
    code = dynamic_map(qabs.device)
    n = qabs.numel()
    m = absmax2.float().repeat_interleave(256)[:n]
    return (code[qabs.long()] * m + torch.tensor(float(offset), dtype=torch.float32, device=qabs.device)).contiguous()


def int4_fuse_scale_zero(scales: torch.Tensor, qzeros: torch.Tensor) -> torch.Tensor:
    """Load-time rebuild of the kernel-side ``sz`` tensor, int32 (N, G) = half2{scale, zero} (low half: fp16 scale bits, high
    half: the 4-bit zero-point as fp16), from the checkpoint tensors of ``quantize_int4``.  Bit-exact to the quantizer's own."""
    N, G = scales.shape
    shifts = torch.arange(0, 32, 4, device=qzeros.device, dtype=torch.int32)
    z = ((qzeros.to(torch.int32).unsqueeze(-1) >> shifts) & 0xF).reshape(N, -1)[:, :G]
    lo = scales.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    hi = z.to(torch.float16).view(torch.int16).to(torch.int32) & 0xFFFF
    return (lo | (hi << 16)).contiguous()


# ---------------------------------------------------------------------------------------------------------
# bnb.int8 (LLM.int8())
# ---------------------------------------------------------------------------------------------------------
def quantize_int8(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (CB int8 (N, K), SCB fp32 (N)) — Linear8bitLt's row-wise weight quantisation (oracle/quant_ref.py:312-320)."""
    C.require_cuda(w)
    if w.dim() != 2 or w.dtype not in C.DTYPE_CODE:
        raise C.B200Error(f"quantize_int8 expects a 2-D floating-point weight (got {tuple(w.shape)}, {w.dtype})")
    w = w.contiguous()
    N, K = w.shape
    cb = torch.empty((N, K), dtype=torch.int8, device=w.device)
    scb = torch.empty((N,), dtype=torch.float32, device=w.device)
    C.check(C.load().b200_quantize_int8(w.data_ptr(), C.DTYPE_CODE[w.dtype], N, K, cb.data_ptr(), scb.data_ptr(),
                                        C.stream_ptr(w.device)), "quantize_int8")
    return cb, scb


def dequantize_int8(cb: torch.Tensor, scb: torch.Tensor, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    C.require_cuda(cb, scb)
    N, K = cb.shape
    out = torch.empty((N, K), dtype=dtype, device=cb.device)
    C.check(C.load().b200_dequantize_int8(cb.data_ptr(), scb.data_ptr(), N, K, out.data_ptr(), C.DTYPE_CODE[dtype],
                                          C.stream_ptr(cb.device)), "dequantize_int8")
    return out


def linear_int8(x: torch.Tensor, cb: torch.Tensor, scb: torch.Tensor, bias: Optional[torch.Tensor] = None,
                threshold: float = 6.0) -> torch.Tensor:
    """LLM.int8() forward: x (..., K) fp16 -> (..., N) fp16 (MatMul8bitLt inference path, oracle/quant_ref.py:326-345)."""
    C.require_cuda(x, cb, scb, bias)
    if x.dtype != torch.float16:
        raise C.B200Error(f"linear_int8 computes in fp16 like bitsandbytes (got {x.dtype}); cast the activation first")
    N, K = cb.shape
    if x.shape[-1] != K:
        raise C.B200Error(f"linear_int8: activation has {x.shape[-1]} features, weight expects {K}")
    x2 = x.reshape(-1, K)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    M = x2.shape[0]
    y = torch.empty((M, N), dtype=torch.float16, device=x.device)
    if M == 0:
        return y.reshape(*x.shape[:-1], N)
    if bias is not None and bias.dtype != torch.float16:
        bias = bias.to(torch.float16)
    lib = C.load()
    ws = _ws("int8", x.device, int(lib.b200_linear_int8_workspace_bytes(M, K)))
    a = C.LinearInt8Args(x=x2.data_ptr(), cb=cb.data_ptr(), scb=scb.data_ptr(), bias=None if bias is None else bias.data_ptr(),
                         y=y.data_ptr(), M=M, N=N, K=K, threshold=float(threshold), workspace=ws.data_ptr(),
                         workspace_bytes=ws.numel())
    C.check(lib.b200_linear_int8(ctypes.byref(a), C.stream_ptr(x.device)), "linear_int8")
    return y.reshape(*x.shape[:-1], N)


def quantize_int4(w: torch.Tensor, group: int = 128):
    """-> (qweight uint32-as-int32 (N, ceil(K/8)), scales fp16 (N, G), qzeros int32 (N, ceil(G/8)), sz int32 (N, G))."""
    C.require_cuda(w)
    if w.dim() != 2:
        raise C.B200Error("quantize_int4 expects a 2-D (out_features, in_features) weight")
    w = w.contiguous()
    N, K = w.shape
    G = (K + group - 1) // group
    qweight = torch.empty((N, (K + 7) // 8), dtype=torch.int32, device=w.device)
    scales = torch.empty((N, G), dtype=torch.float16, device=w.device)
    qzeros = torch.empty((N, (G + 7) // 8), dtype=torch.int32, device=w.device)
    sz = torch.empty((N, G), dtype=torch.int32, device=w.device)
    C.check(C.load().b200_quantize_int4(w.data_ptr(), C.DTYPE_CODE[w.dtype], N, K, group, qweight.data_ptr(), scales.data_ptr(),
                                        qzeros.data_ptr(), sz.data_ptr(), C.stream_ptr(w.device)), "quantize_int4")
    return qweight, scales, qzeros, sz


def dequantize_int4(qweight, scales, qzeros, K: int, group: int = 128, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    C.require_cuda(qweight, scales, qzeros)
    N = qweight.shape[0]
    out = torch.empty((N, K), dtype=dtype, device=qweight.device)
    C.check(C.load().b200_dequantize_int4(qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), N, K, group, out.data_ptr(),
                                          C.DTYPE_CODE[dtype], C.stream_ptr(qweight.device)), "dequantize_int4")
    return out


# ---------------------------------------------------------------------------------------------------------
# fused dequant-GEMV (batch <= 16)
# ---------------------------------------------------------------------------------------------------------
def qgemv(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, N: int, K: int, quant_type: str = "nf4",
          blocksize: int = 64, *, bias: Optional[torch.Tensor] = None, delta: Optional[torch.Tensor] = None,
          x_out: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-5,
          residual: Optional[torch.Tensor] = None, packed2: Optional[torch.Tensor] = None,
          scale2: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = epilogue(prologue(x) @ dequant(W).T); see b200_qgemv in include/b200gpt.h.  x: (..., K) with <= 16 rows."""
    C.require_cuda(x, packed, scale)
    x = _bf16c(x, "x")
    lead = x.shape[:-1]
    batch = x.numel() // K
    if x.shape[-1] != K:
        raise C.B200Error(f"qgemv: x has {x.shape[-1]} features, weight expects {K}")
    epilogue = C.EPI_SWIGLU if packed2 is not None else (C.EPI_RESIDUAL if residual is not None else C.EPI_STORE)
    y = out if out is not None else torch.empty((*lead, N), dtype=torch.bfloat16, device=x.device)
    nbytes = C.load().b200_qgemv_workspace_bytes()
    ws = _ws("qgemv", x.device, nbytes)
    delta, residual, bias, norm_weight = _bf16c(delta, "delta"), _bf16c(residual, "residual"), _bf16c(bias, "bias"), _bf16c(norm_weight, "norm_weight")
    args = C.QGemvArgs(
        packed=packed.data_ptr(), scale=scale.data_ptr(), packed2=C.ptr(packed2), scale2=C.ptr(scale2),
        qtype=QTYPES[quant_type], blocksize=blocksize, N=N, K=K, x=x.data_ptr(), delta=C.ptr(delta), x_out=C.ptr(x_out),
        norm_weight=C.ptr(norm_weight), norm_eps=norm_eps, batch=batch, epilogue=epilogue, bias=C.ptr(bias),
        residual=C.ptr(residual), y=y.data_ptr(), workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    C.check(C.load().b200_qgemv(ctypes.byref(args), C.stream_ptr(x.device)), "qgemv")
    return y


# ---------------------------------------------------------------------------------------------------------
# tiled layout + streaming GEMV (the decode hot path)
# ---------------------------------------------------------------------------------------------------------
def tiled_bytes(N: int, K: int, quant_type: str = "nf4") -> int:
    """Size of the tiled buffer for an (N, K) matrix; 0 when the layout does not cover the shape."""
    return int(C.load().b200_tiled_bytes(N, K, QTYPES[quant_type]))


def tile_4bit(packed: torch.Tensor, scale: torch.Tensor, N: int, K: int, quant_type: str = "nf4", blocksize: int = 64,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reference-layout (packed, absmax) or (qweight, sz) -> flat uint8 tiled buffer (csrc/tile.cu)."""
    C.require_cuda(packed, scale)
    nbytes = tiled_bytes(N, K, quant_type)
    if nbytes == 0:
        raise C.B200Error(f"tile_4bit: shape ({N}, {K}) is not covered by the tiled layout for {quant_type}")
    if out is None:
        out = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
    C.check(C.load().b200_tile_4bit(packed.data_ptr(), scale.data_ptr(), N, K, QTYPES[quant_type], blocksize, out.data_ptr(),
                                    C.stream_ptr(packed.device)), "tile_4bit")
    return out


def untile_4bit(tiled: torch.Tensor, N: int, K: int, quant_type: str = "nf4", blocksize: int = 64):
    """Inverse of tile_4bit -> (packed, scale) in the reference layout, bit for bit."""
    C.require_cuda(tiled)
    if quant_type == "int4":
        packed = torch.empty((N, K // 8), dtype=torch.int32, device=tiled.device)
        scale = torch.empty((N, K // blocksize), dtype=torch.int32, device=tiled.device)
    else:
        packed = torch.empty((N * K // 2, 1), dtype=torch.uint8, device=tiled.device)
        scale = torch.empty((N * K // blocksize,), dtype=torch.float32, device=tiled.device)
    C.check(C.load().b200_untile_4bit(tiled.data_ptr(), N, K, QTYPES[quant_type], blocksize, packed.data_ptr(), scale.data_ptr(),
                                      C.stream_ptr(tiled.device)), "untile_4bit")
    return packed, scale


def qgemv_tiled(x: torch.Tensor, tiled: torch.Tensor, N: int, K: int, quant_type: str = "nf4", blocksize: int = 64, *,
                bias: Optional[torch.Tensor] = None, bias2: Optional[torch.Tensor] = None, delta: Optional[torch.Tensor] = None,
                x_out: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-5,
                residual: Optional[torch.Tensor] = None, tiled2: Optional[torch.Tensor] = None,
                prefetch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                tp: Optional["C.TpHandoff"] = None, fold: int = 1, kv_hint: Optional[tuple] = None,
                attn: Optional[dict] = None) -> torch.Tensor:
    """y = epilogue(prologue(x) @ dequant(W).T) over tiled matrices; see b200_qgemv_tiled in include/b200gpt.h.
    ``tp``: tensor-parallel hand-off over peer memory (lit_gpt_b200/p2p.py builds it).  ``fold``: the tiled buffer is
    the (N / fold, fold * K) view of the flat 4-bit storage (shards whose K is not a multiple of the block)."""
    C.require_cuda(x, tiled)
    x = _bf16c(x, "x")
    if x.shape[-1] != K:
        raise C.B200Error(f"qgemv_tiled: x has {x.shape[-1]} features, weight expects {K}")
    lead = x.shape[:-1]
    batch = x.numel() // K
    epilogue = C.EPI_SWIGLU if tiled2 is not None else (C.EPI_RESIDUAL if residual is not None else C.EPI_STORE)
    y = out if out is not None else torch.empty((*lead, N), dtype=torch.bfloat16, device=x.device)
    delta, residual, bias, bias2, norm_weight = (_bf16c(delta, "delta"), _bf16c(residual, "residual"), _bf16c(bias, "bias"),
                                                 _bf16c(bias2, "bias2"), _bf16c(norm_weight, "norm_weight"))
    ws = _ws("qgemv_tiled", x.device, C.load().b200_qgemv_tiled_workspace_bytes())
    hint = None
    if kv_hint is not None:  # (k_cache, v_cache, pos): L2 prefetch of the filled cache rows for the attention step that follows
        kc, vc, pos = kv_hint
        hint = C.KvHint(k=kc.data_ptr(), v=vc.data_ptr(), pos=pos.data_ptr(), pos_is_int64=int(pos.dtype == torch.int64),
                        chunks=kc.shape[0] * kc.shape[1], chunk_stride=kc.shape[2] * kc.shape[3] * kc.element_size(),
                        row_bytes=kc.shape[3] * kc.element_size(), max_rows=kc.shape[2])
    at = None
    if attn is not None:  # the decode-attention step fused into this (QKV) launch: y is its input, attn["out"] its output
        kc, vc, pos, cos, sin = attn["k_cache"], attn["v_cache"], attn["pos"], attn["cos"], attn["sin"]
        at = C.AttnDecodeArgs(
            qkv=y.data_ptr(), cos=cos.data_ptr(), sin=sin.data_ptr(), table_dtype=_table_code(cos), table_preselected=0,
            rope_n_elem=attn["rope_n_elem"], pos=pos.data_ptr(), pos_is_int64=int(pos.dtype == torch.int64), k_cache=kc.data_ptr(),
            v_cache=vc.data_ptr(), out=attn["out"].data_ptr(), batch=kc.shape[0], n_head=attn["n_head"], n_groups=attn["n_groups"],
            head_size=attn["head_size"], max_seq=kc.shape[2], num_splits=0, workspace=None, workspace_bytes=0)
    args = C.QGemvTiledArgs(
        tiled=tiled.data_ptr(), tiled2=C.ptr(tiled2), qtype=QTYPES[quant_type], blocksize=blocksize, N=N, K=K, x=x.data_ptr(),
        delta=C.ptr(delta), x_out=C.ptr(x_out), norm_weight=C.ptr(norm_weight), norm_eps=norm_eps, batch=batch, epilogue=epilogue,
        bias=C.ptr(bias), bias2=C.ptr(bias2), residual=C.ptr(residual), y=y.data_ptr(), prefetch=C.ptr(prefetch),
        prefetch_bytes=0 if prefetch is None else prefetch.numel() * prefetch.element_size(),
        workspace=ws.data_ptr(), workspace_bytes=ws.numel(), tp=None if tp is None else ctypes.pointer(tp), fold=fold,
        kv_hint=None if hint is None else ctypes.pointer(hint), attn=None if at is None else ctypes.addressof(at))
    C.check(C.load().b200_qgemv_tiled(ctypes.byref(args), C.stream_ptr(x.device)), "qgemv_tiled")
    return y


@functools.lru_cache(maxsize=None)
def qgemv_attn_fusable(N: int, K: int, quant_type: str, n_head: int, n_groups: int, head_size: int, rope_n_elem: int, max_seq: int) -> bool:
    """Whether b200_qgemv_tiled can run the decode attention of (n_head, n_groups, head_size) fused into the QKV GEMV (dry run)."""
    at = C.AttnDecodeArgs(qkv=256, cos=256, sin=256, table_dtype=0, table_preselected=0, rope_n_elem=rope_n_elem, pos=256,
                          pos_is_int64=1, k_cache=256, v_cache=256, out=256, batch=1, n_head=n_head, n_groups=n_groups,
                          head_size=head_size, max_seq=max_seq, num_splits=0, workspace=None, workspace_bytes=0)
    args = C.QGemvTiledArgs(qtype=QTYPES[quant_type], blocksize=128 if quant_type == "int4" else 64, N=N, K=K, batch=1,
                            epilogue=C.EPI_STORE, attn=ctypes.addressof(at))
    return bool(C.load().b200_qgemv_tiled_supported(ctypes.byref(args)))


@functools.lru_cache(maxsize=None)
def _qgemv_tiled_supported(N: int, K: int, quant_type: str, batch: int, swiglu: bool, fold: int) -> bool:
    args = C.QGemvTiledArgs(qtype=QTYPES[quant_type], blocksize=128 if quant_type == "int4" else 64, N=N, K=K, batch=batch,
                            epilogue=C.EPI_SWIGLU if swiglu else C.EPI_STORE, tiled2=256 if swiglu else None, fold=fold)  # dry run: pointers are not dereferenced
    return bool(C.load().b200_qgemv_tiled_supported(ctypes.byref(args)))


@torch._dynamo.assume_constant_result
def qgemv_tiled_supported(N: int, K: int, quant_type: str, batch: int, swiglu: bool = False, fold: int = 1) -> bool:
    """Whether b200_qgemv_tiled runs (batch, K) x (N, K) on a streaming kernel (its shared-memory plan covers the
    activation rows); asked up front so that the caller can pick the generic GEMV / the prefill GEMM instead.
    A pure function of the shape: a constant while tracing (no graph break)."""
    if not 1 <= batch <= 16:
        return False
    return _qgemv_tiled_supported(int(N), int(K), quant_type, int(batch), bool(swiglu), int(fold))


def tp_gather(h: "C.TpHandoff", batch: int, n_per_rank: int, device: torch.device) -> torch.Tensor:
    """All-gather of a row-sharded Linear's outputs over the peer-memory slots -> (batch, world * n_per_rank) bf16."""
    out = torch.empty((batch, h.world * n_per_rank), dtype=torch.bfloat16, device=device)
    ws = _ws("qgemv_tiled", device, C.load().b200_qgemv_tiled_workspace_bytes())
    C.check(C.load().b200_tp_gather(ctypes.byref(h), batch, n_per_rank, out.data_ptr(), ws.data_ptr(), C.stream_ptr(device)), "tp_gather")
    return out


def check_gemv_errors(device: torch.device) -> None:
    """Raise if a GEMV kernel on `device` gave up a bounded wait (a tensor-parallel peer that never delivered its
    packets, a stream-K partner CTA): synchronizes the current stream.  Called by generate() at its sync points."""
    key = ("qgemv_tiled", device.index if device.index is not None else torch.cuda.current_device())
    ws = _workspaces.get(key)
    if ws is None:
        return
    code = ctypes.c_uint(0)
    with torch.cuda.device(device):
        C.check(C.load().b200_qgemv_tiled_error(ws.data_ptr(), C.stream_ptr(device), ctypes.byref(code)), "qgemv_tiled_error")
    if code.value:
        what = {1: "a stream-K partner CTA", 2: "a tensor-parallel peer"}.get(code.value, f"code {code.value}")
        raise C.B200Error(f"dequant-GEMV: {what} did not deliver within the bounded wait; the output of this step is invalid")


def qgemv_tiled_tune(depth: int = 0, ctas_per_sm: int = 0, l2_prefetch: bool = True) -> None:
    C.load().b200_qgemv_tiled_tune(depth, ctas_per_sm, int(l2_prefetch))


# ---------------------------------------------------------------------------------------------------------
# norm / embedding / argmax
# ---------------------------------------------------------------------------------------------------------
def qgemm(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, N: int, K: int, quant_type: str = "nf4", blocksize: int = 64,
          bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Prefill GEMM y (M, N) = x (M, K) . dequant(W)^T on tcgen05 / TMEM (reference-layout packed weights + scales).
    Raises NotImplementedError for shapes the kernel does not cover (K not a multiple of the block, N % 8 != 0)."""
    C.require_cuda(x, packed, scale, bias)
    x = _bf16c(x, "x")
    bias = _bf16c(bias, "bias")
    M = x.numel() // K
    if x.numel() != M * K:
        raise C.B200Error("qgemm: x does not hold whole rows of length K")
    y = out if out is not None else torch.empty(tuple(x.shape[:-1]) + (N,), dtype=torch.bfloat16, device=x.device)
    need = C.load().b200_qgemm_workspace_bytes(M, N, K)   # fp32 partial sums of a one-tile prompt split over k ranges; 0 otherwise
    ws = _ws("qgemm", x.device, need) if need else None
    args = C.QGemmArgs(packed=packed.data_ptr(), scale=scale.data_ptr(), qtype=QTYPES[quant_type], blocksize=blocksize, M=M, N=N, K=K,
                       x=x.data_ptr(), bias=C.ptr(bias), y=y.data_ptr(), workspace=C.ptr(ws), workspace_bytes=0 if ws is None else ws.numel())
    C.check(C.load().b200_qgemm(ctypes.byref(args), C.stream_ptr(x.device)), "qgemm")
    return y


def qgemm_tune(mt3: bool = True) -> None:
    """development switch: 384-token tiles for long prompts (default) or the 256-token tiles of round 1"""
    C.check(C.load().b200_qgemm_tune(1 if mt3 else 0), "qgemm_tune")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, delta: Optional[torch.Tensor] = None,
            sum_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    C.require_cuda(x, weight)
    x, weight, delta = _bf16c(x, "x"), _bf16c(weight, "weight"), _bf16c(delta, "delta")
    dim = x.shape[-1]
    y = torch.empty_like(x)
    C.check(C.load().b200_rmsnorm(x.data_ptr(), C.ptr(delta), weight.data_ptr(), eps, y.data_ptr(), C.ptr(sum_out),
                                  x.numel() // dim, dim, C.stream_ptr(x.device)), "rmsnorm")
    return y


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """silu(a) * b with the reference's bf16 rounding points (model.py:715), one kernel."""
    C.require_cuda(a, b)
    a, b = _bf16c(a, "a"), _bf16c(b, "b")
    if a.shape != b.shape:
        raise C.B200Error("swiglu: shape mismatch")
    y = torch.empty_like(a)
    C.check(C.load().b200_swiglu(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), C.stream_ptr(a.device)), "swiglu")
    return y


def embedding(idx: torch.Tensor, wte: torch.Tensor) -> torch.Tensor:
    C.require_cuda(idx, wte)
    wte = _bf16c(wte, "wte")
    if idx.dtype not in (torch.int64, torch.int32):
        raise C.B200Error(f"embedding: idx must be int32/int64 (got {idx.dtype})")
    idx = idx.contiguous()
    out = torch.empty((*idx.shape, wte.shape[1]), dtype=torch.bfloat16, device=wte.device)
    C.check(C.load().b200_embedding(idx.data_ptr(), int(idx.dtype == torch.int64), wte.data_ptr(), out.data_ptr(), idx.numel(),
                                    wte.shape[1], wte.shape[0], C.stream_ptr(wte.device)), "embedding")
    return out


def argmax_(logits: torch.Tensor, token_out: torch.Tensor, pos_inout: Optional[torch.Tensor] = None, vocab: Optional[int] = None,
            history: Optional[torch.Tensor] = None) -> None:
    """token_out[b] = argmax(logits[b, :vocab]); optionally pos_inout[0] += 1 and history[pos] = token (on device)."""
    if history is not None and history.dtype != token_out.dtype:
        raise C.B200Error("argmax_: history must have the dtype of token_out")
    C.require_cuda(logits, token_out)
    logits = _bf16c(logits, "logits")
    V = logits.shape[-1]
    batch = logits.numel() // V
    C.check(C.load().b200_argmax(logits.data_ptr(), batch, vocab or V, V, token_out.data_ptr(), int(token_out.dtype == torch.int64),
                                 C.ptr(pos_inout), int(pos_inout is not None and pos_inout.dtype == torch.int64),
                                 C.ptr(history), 0 if history is None else history.numel(),
                                 C.stream_ptr(logits.device)), "argmax")


def new_rng_state(device: torch.device, seed: Optional[int] = None) -> torch.Tensor:
    """Device-side Philox state for ``sample_``: int64[2] = (seed, offset).  The seed defaults to torch's current seed, so
    ``seed_everything`` (generate/base.py:140) makes the draws reproducible."""
    seed = (torch.initial_seed() if seed is None else int(seed)) & 0x7FFFFFFFFFFFFFFF  # torch's default seed is a full uint64
    return torch.tensor([seed, 0], dtype=torch.int64, device=device)


def sample_(logits: torch.Tensor, token_out: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
            rng_state: Optional[torch.Tensor] = None, pos_inout: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
            noise: Optional[torch.Tensor] = None) -> None:
    """token_out[0] = one draw from softmax(top_k(logits[0, -1]) / temperature) (generate/base.py:22-41), on the device;
    optionally pos_inout[0] += 1 and history[pos] = token like ``argmax_``.  ``noise``: Exp(1) values to use instead of Philox."""
    C.require_cuda(logits, token_out)
    if logits.dtype not in (torch.bfloat16, torch.float32):
        raise C.B200Error(f"sample_: logits must be bf16 or fp32 (got {logits.dtype})")
    V = logits.shape[-1]
    row = (logits[0, -1] if logits.dim() == 3 else logits[0] if logits.dim() == 2 else logits).contiguous()  # base.py:31
    if history is not None and history.dtype != token_out.dtype:
        raise C.B200Error("sample_: history must have the dtype of token_out")
    if temperature > 0.0 and rng_state is None and noise is None:
        raise C.B200Error("sample_: temperature > 0 needs rng_state (K.new_rng_state) or noise")
    if rng_state is not None and (rng_state.dtype != torch.int64 or rng_state.numel() != 2 or not rng_state.is_cuda):
        raise C.B200Error("sample_: rng_state must be a CUDA int64[2] tensor")
    if noise is not None:
        noise = noise.to(torch.float32).contiguous()
        if noise.numel() != V:
            raise C.B200Error("sample_: noise must hold one value per vocabulary entry")
    C.check(C.load().b200_sample(row.data_ptr(), C.DTYPE_CODE[row.dtype], V, float(temperature), int(top_k or 0), C.ptr(rng_state), C.ptr(noise),
                                 token_out.data_ptr(), int(token_out.dtype == torch.int64), C.ptr(pos_inout),
                                 int(pos_inout is not None and pos_inout.dtype == torch.int64), C.ptr(history),
                                 0 if history is None else history.numel(), C.stream_ptr(logits.device)), "sample")


# ---------------------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------------------
def _table_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return C.F32
    if t.dtype == torch.bfloat16:
        return C.BF16
    raise C.B200Error(f"cos/sin tables must be fp32 or bf16 (got {t.dtype})")


def attn_decode(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor,
                v_cache: torch.Tensor, n_head: int, n_groups: int, head_size: int, rope_n_elem: int,
                num_splits: int = 0, table_preselected: bool = False) -> torch.Tensor:
    """Fused RoPE + cache append + split-K decode attention for one token per sequence.

    qkv (B, 1, (H+2G)*hs) or (B, (H+2G)*hs); cos/sin: the model's FULL tables (max_seq, rope_n_elem); pos: device int
    scalar tensor (input_pos); caches (B, G, max_seq, hs) bf16, updated in place.  Returns (B, H*hs)."""
    C.require_cuda(qkv, cos, sin, pos, k_cache, v_cache)
    qkv = _bf16c(qkv, "qkv")
    B = k_cache.shape[0]
    max_seq = k_cache.shape[2]
    if k_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise C.B200Error("kv cache must be contiguous bfloat16 (B, n_query_groups, max_seq, head_size)")
    if qkv.numel() != B * (n_head + 2 * n_groups) * head_size:
        raise C.B200Error("attn_decode: qkv does not hold exactly one token per cached sequence")
    if pos.dtype not in (torch.int64, torch.int32) or pos.numel() != 1:
        raise C.B200Error("attn_decode: pos must be a single int32/int64 device scalar")
    cos, sin = cos.contiguous(), sin.contiguous()
    out = torch.empty((B, n_head * head_size), dtype=torch.bfloat16, device=qkv.device)
    lib = C.load()
    max_splits = 64
    ws = _ws("attn", qkv.device, lib.b200_attn_decode_workspace_bytes(B, n_head, head_size, max_splits))
    args = C.AttnDecodeArgs(
        qkv=qkv.data_ptr(), cos=cos.data_ptr(), sin=sin.data_ptr(), table_dtype=_table_code(cos), table_preselected=int(table_preselected), rope_n_elem=rope_n_elem,
        pos=pos.data_ptr(), pos_is_int64=int(pos.dtype == torch.int64), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(),
        out=out.data_ptr(), batch=B, n_head=n_head, n_groups=n_groups, head_size=head_size, max_seq=max_seq,
        num_splits=num_splits, workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    C.check(lib.b200_attn_decode(ctypes.byref(args), C.stream_ptr(qkv.device)), "attn_decode")
    return out


def rope_kv_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, n_head: int, n_groups: int, head_size: int, rope_n_elem: int,
                   table_preselected: bool = False) -> torch.Tensor:
    """Prefill: RoPE q/k for T tokens at positions pos[0..T), write k/v into the GQA-native caches, return roped q
    as (B, H, T, hs)."""
    C.require_cuda(qkv, cos, sin, pos, k_cache, v_cache)
    qkv = _bf16c(qkv, "qkv")
    B, T = qkv.shape[0], qkv.shape[1]
    if pos.numel() != T:
        raise C.B200Error("rope_kv_append: pos must have one entry per token")
    cos, sin, pos = cos.contiguous(), sin.contiguous(), pos.contiguous()
    q = torch.empty((B, n_head, T, head_size), dtype=torch.bfloat16, device=qkv.device)
    C.check(C.load().b200_rope_kv_append(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), _table_code(cos), int(table_preselected), rope_n_elem,
                                         pos.data_ptr(), int(pos.dtype == torch.int64), k_cache.data_ptr(), v_cache.data_ptr(),
                                         q.data_ptr(), B, T, n_head, n_groups, head_size, k_cache.shape[2],
                                         C.stream_ptr(qkv.device)), "rope_kv_append")
    return q


def attn_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Prefill attention (reference ``scaled_dot_product_attention``, lit_gpt/model.py:658-665, cached call): q (B, H, T, hs)
    roped, caches (B, G, Tmax, hs) already extended; row t sees cache positions <= pos[t].  Returns (B, T, H * hs)."""
    C.require_cuda(q, k_cache, v_cache, pos)
    q = _bf16c(q, "q")
    if k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16 or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise C.B200Error("attn_prefill: caches must be contiguous bf16")
    B, H, T, hs = q.shape
    G, Tmax = k_cache.shape[1], k_cache.shape[2]
    if pos.numel() != T:
        raise C.B200Error("attn_prefill: pos must have one entry per token")
    pos = pos.contiguous()
    y = torch.empty((B, T, H * hs), dtype=torch.bfloat16, device=q.device)
    C.check(C.load().b200_attn_prefill(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), int(pos.dtype == torch.int64),
                                       y.data_ptr(), B, T, H, G, hs, Tmax, float(scale if scale is not None else hs ** -0.5),
                                       C.stream_ptr(q.device)), "attn_prefill")
    return y


def attn_decode_tune(force_scalar: bool = False) -> bool:
    """Test knob: route grouped-query shapes through the scalar decode-attention kernel; returns the previous setting."""
    return bool(C.load().b200_attn_decode_tune(int(force_scalar)))


def set_pdl(enabled: bool) -> bool:
    return bool(C.load().b200_set_pdl(int(enabled)))


def launch_count() -> int:
    return int(C.load().b200_launch_count())


def qgemv_tune(ksteps: int = 0, ctas_per_sm: int = 0, force_generic: bool = False) -> None:
    C.load().b200_qgemv_tune(ksteps, ctas_per_sm, int(force_generic))



# ---------------------------------------------------------------------------------------------------------
# fp32 residual stream, latent attention, sparse experts (csrc/resid.cu, latent.cu, moe.cu).  `T` below is the
# matrix-product dtype of a model: bfloat16 or float32; these wrappers load only the core library (C.load_core).
# ---------------------------------------------------------------------------------------------------------
def _code(t: torch.Tensor) -> int:
    if t.dtype not in (torch.bfloat16, torch.float32):
        raise C.B200Error(f"expected a bfloat16 or float32 tensor (got {t.dtype})")
    return C.DTYPE_CODE[t.dtype]


def embed_pos(tokens: torch.Tensor, pos: Optional[torch.Tensor], embed: torch.Tensor, pos_table: Optional[torch.Tensor], scale: float,
              x_out: Optional[torch.Tensor] = None):
    """tokens, pos int32 (n,) -> (x fp32 (n, d), act T (n, d)) with x = embed[tokens] * scale + pos_table[pos]; without a
    position table (pos None) x = embed[tokens] * scale.  `x_out`: a contiguous fp32 (n, d) tensor to receive x."""
    C.require_cuda(tokens, pos, embed, pos_table)
    if tokens.dtype != torch.int32 or (pos is not None and pos.dtype != torch.int32) or (pos is None and pos_table is not None):
        raise C.B200Error("embed_pos: tokens and pos must be int32")
    n, d = tokens.numel(), embed.shape[1]
    if x_out is not None and (x_out.dtype != torch.float32 or not x_out.is_contiguous() or x_out.numel() != n * d or not x_out.is_cuda):
        raise C.B200Error("embed_pos: x_out must be a contiguous fp32 (n, d) CUDA tensor")
    x = x_out if x_out is not None else torch.empty((n, d), dtype=torch.float32, device=embed.device)
    act = torch.empty((n, d), dtype=embed.dtype, device=embed.device)
    C.check(C.load_core().b200_embed_pos(tokens.data_ptr(), C.ptr(pos), embed.data_ptr(), C.ptr(pos_table), float(scale), x.data_ptr(),
                                         act.data_ptr(), n, d, embed.shape[0], 0 if pos_table is None else pos_table.shape[0], _code(embed),
                                         C.stream_ptr(embed.device)), "embed_pos")
    return x, act


def _seg(inp: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, d: int, plus_one: bool, in_rows=None, out_rows=None) -> "C.RmsRowsSeg":
    if inp.stride(-1) != 1 or out.stride(-1) != 1 or not weight.is_contiguous():
        raise C.B200Error("rms_rows: rows must be contiguous")
    for idx in (in_rows, out_rows):
        if idx is not None and (idx.dtype != torch.int64 or not idx.is_contiguous()):
            raise C.B200Error("rms_rows: row indices must be contiguous int64")
    return C.RmsRowsSeg(inp=inp.data_ptr(), weight=weight.data_ptr(), out=out.data_ptr(), in_rows=C.ptr(in_rows), out_rows=C.ptr(out_rows),
                        ld_in=inp.stride(-2), ld_out=out.stride(-2), d=d, plus_one=int(plus_one))


def rms_rows(rows: int, eps: float, *segs: "C.RmsRowsSeg", in_dtype: torch.dtype, out_dtype: torch.dtype, device: torch.device) -> None:
    """One launch normalising `rows` rows of one or two segments built by ``rms_seg`` (statistics in fp32)."""
    arr = (C.RmsRowsSeg * len(segs))(*segs)
    C.check(C.load_core().b200_rms_rows(arr, len(segs), rows, float(eps), C.DTYPE_CODE[in_dtype], C.DTYPE_CODE[out_dtype], C.stream_ptr(device)),
            "rms_rows")


rms_seg = _seg


def residual_norm_add(y: torch.Tensor, weight: torch.Tensor, eps: float, x: torch.Tensor, act: torch.Tensor) -> None:
    """x (fp32, in place) += y / rms(y) * (1 + weight); act = T(x)."""
    C.require_cuda(y, weight, x, act)
    if x.dtype != torch.float32 or not (y.is_contiguous() and x.is_contiguous() and act.is_contiguous()) or act.dtype != y.dtype:
        raise C.B200Error("residual_norm_add: x must be fp32, y and act of one dtype, all contiguous")
    d = y.shape[-1]
    C.check(C.load_core().b200_residual_norm_add(y.data_ptr(), weight.data_ptr(), float(eps), x.data_ptr(), act.data_ptr(), y.numel() // d, d,
                                                 _code(y), C.stream_ptr(y.device)), "residual_norm_add")


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    C.require_cuda(src, rows)
    if not src.is_contiguous() or rows.dtype not in (torch.int64, torch.int32) or not rows.is_contiguous():
        raise C.B200Error("gather_rows: contiguous source and int64 / int32 rows")
    d = src.shape[-1]
    dst = torch.empty((rows.numel(), d), dtype=src.dtype, device=src.device)
    C.check(C.load_core().b200_gather_rows(src.data_ptr(), rows.data_ptr(), int(rows.dtype == torch.int64), dst.data_ptr(), rows.numel(), d, _code(src),
                                           C.stream_ptr(src.device)), "gather_rows")
    return dst


def sqrelu_(x: torch.Tensor) -> torch.Tensor:
    """x = relu(x)^2 in place."""
    C.require_cuda(x)
    if not x.is_contiguous():
        raise C.B200Error("sqrelu_: contiguous tensor")
    C.check(C.load_core().b200_sqrelu(x.data_ptr(), x.numel(), _code(x), C.stream_ptr(x.device)), "sqrelu")
    return x


def scale_f32(t: torch.Tensor, scale: float) -> torch.Tensor:
    C.require_cuda(t)
    t = t.contiguous()
    out = torch.empty(t.shape, dtype=torch.float32, device=t.device)
    C.check(C.load_core().b200_scale_f32(t.data_ptr(), float(scale), out.data_ptr(), t.numel(), _code(t), C.stream_ptr(t.device)), "scale_f32")
    return out


LATENT_PREFILL_MMA = True   # tests switch it off to reach the any-size kernel with tensor-core-sized heads


def _gate_mode(gate: Optional[torch.Tensor], n_head: int, dv: int) -> int:
    """0: no gate, 1: one column per head, 2: one column per output number."""
    if gate is None:
        return 0
    if gate.stride(-1) != 1 or gate.shape[-1] not in (n_head, n_head * dv):
        raise C.B200Error("output gate: rows of one number per head or per output number, unit inner stride")
    return 2 if gate.shape[-1] == n_head * dv and dv > 1 else 1


def latent_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seqs: torch.Tensor, max_q_len: int, n_head: int, dk: int, dv: int,
                   scale: float, *, k_shared: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ragged causal attention over explicit keys and values.  q (n, H * dk); k (m, H * dk) and v (m, H * dv) may be column
    slices of one buffer; seqs int32 (S, 4) = first query row, query rows, position of the first query row, row of position 0 in
    k / v.  Optional: `k_shared` (m, dk2), a key part shared by all heads that meets the last dk2 numbers of every query head (k is
    then (m, H * (dk - dk2))); `sink` (H,), a logit per head in the denominator only; `gate` (n, H) or (n, H * dv), whose sigmoid
    multiplies the output."""
    C.require_cuda(q, k, v, seqs, k_shared, sink, gate)
    if k_shared is not None and (k_shared.dtype != q.dtype or k_shared.stride(-1) != 1):
        raise C.B200Error("latent_prefill: the shared key part must have the queries' dtype and unit inner stride")
    if (sink is not None and (sink.dtype != q.dtype or not sink.is_contiguous())) or (gate is not None and gate.dtype != q.dtype):
        raise C.B200Error("latent_prefill: sink and gate must have the queries' dtype")
    plain = k_shared is None and sink is None and gate is None
    if seqs.dtype != torch.int32 or seqs.dim() != 2 or seqs.shape[1] != 4 or not seqs.is_contiguous():
        raise C.B200Error("latent_prefill: seqs must be contiguous int32 (S, 4)")
    if not (q.dtype == k.dtype == v.dtype) or q.stride(-1) != 1 or k.stride(-1) != 1 or v.stride(-1) != 1:
        raise C.B200Error("latent_prefill: q, k, v of one dtype with unit inner stride")
    out = torch.empty((q.shape[0], n_head * dv), dtype=q.dtype, device=q.device)
    if (plain and q.dtype == torch.bfloat16 and dk == dv and dk in (64, 128) and not (q.stride(0) | k.stride(0) | v.stride(0)) & 7
            and not (q.data_ptr() | k.data_ptr() | v.data_ptr() | seqs.data_ptr()) & 15 and LATENT_PREFILL_MMA):
        # tensor-core tiles of the GQA models' prefill kernel, over the packed operands
        C.check(C.load_core().b200_attn_prefill_ragged(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), seqs.data_ptr(),
                                                       seqs.shape[0], max_q_len, out.data_ptr(), out.stride(0), n_head, dk, float(scale),
                                                       C.stream_ptr(q.device)), "attn_prefill_ragged")
        return out
    gm = _gate_mode(gate, n_head, dv)
    if (k_shared is not None and q.dtype == torch.bfloat16 and LATENT_PREFILL_MMA and dv in (64, 128) and dk - k_shared.shape[-1] == dv
            and k_shared.shape[-1] in (64, 128) and not (q.stride(0) | k.stride(0) | v.stride(0) | k_shared.stride(0)) & 7
            and not (q.data_ptr() | k.data_ptr() | v.data_ptr() | k_shared.data_ptr() | seqs.data_ptr()) & 15):
        # tensor-core tiles with the shared key part as extra columns of the score product
        C.check(C.load_core().b200_attn_prefill_shared(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), k_shared.data_ptr(),
                                                       k_shared.stride(0), k_shared.shape[-1], seqs.data_ptr(), seqs.shape[0], max_q_len, out.data_ptr(),
                                                       out.stride(0), n_head, dv, float(scale), C.ptr(sink), C.ptr(gate),
                                                       0 if gate is None else gate.stride(0), gm, C.stream_ptr(q.device)), "attn_prefill_shared")
        return out
    args = C.LatentPrefillArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), ldq=q.stride(0), ldk=k.stride(0), ldv=v.stride(0),
                               ldo=out.stride(0), seqs=seqs.data_ptr(), n_seqs=seqs.shape[0], max_q_len=max_q_len, n_head=n_head, dk=dk, dv=dv,
                               scale=float(scale), dtype=_code(q), k2=C.ptr(k_shared), ldk2=0 if k_shared is None else k_shared.stride(0),
                               dk2=0 if k_shared is None else k_shared.shape[-1], sink=C.ptr(sink), gate=C.ptr(gate),
                               ldg=0 if gate is None else gate.stride(0), gate_mode=_gate_mode(gate, n_head, dv))
    C.check(C.load_core().b200_latent_prefill(ctypes.byref(args), C.stream_ptr(q.device)), "latent_prefill")
    return out


def latent_decode(q: torch.Tensor, w_uk: torch.Tensor, w_uv: torch.Tensor, cache: torch.Tensor, row_slot: torch.Tensor, row_pos: torch.Tensor,
                  n_head: int, dk: int, dv: int, scale: float, n_split: int, *, shared_dims: int = 0, sink: Optional[torch.Tensor] = None,
                  gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query row per sequence over the cached latents (slots, max_seq, r); row b reads positions 0 .. row_pos[b] of slot
    row_slot[b].  Returns (B, H * dv).  With `shared_dims` = dk2 > 0 a cache row is [r latent | dk2 shared key part] and a query
    head [dk | dk2] numbers; `sink` and `gate` as in ``latent_prefill``."""
    C.require_cuda(q, w_uk, w_uv, cache, row_slot, row_pos, sink, gate)
    if (sink is not None and (sink.dtype != q.dtype or not sink.is_contiguous())) or (gate is not None and gate.dtype != q.dtype):
        raise C.B200Error("latent_decode: sink and gate must have the queries' dtype")
    if row_slot.dtype != torch.int32 or row_pos.dtype != torch.int32:
        raise C.B200Error("latent_decode: row_slot and row_pos must be int32")
    if not (q.dtype == w_uk.dtype == w_uv.dtype == cache.dtype) or not (w_uk.is_contiguous() and w_uv.is_contiguous() and cache.is_contiguous()):
        raise C.B200Error("latent_decode: one dtype, contiguous weights and cache")
    B, r, max_seq = q.shape[0], cache.shape[-1] - shared_dims, cache.shape[1]
    lib = C.load_core()
    ws = _ws("latent", q.device, lib.b200_latent_decode_workspace_bytes(B, n_head, r + shared_dims, n_split))
    out = torch.empty((B, n_head * dv), dtype=q.dtype, device=q.device)
    args = C.LatentDecodeArgs(q=q.data_ptr(), w_uk=w_uk.data_ptr(), w_uv=w_uv.data_ptr(), cache=cache.data_ptr(), out=out.data_ptr(), ldq=q.stride(0),
                              ldo=out.stride(0), slot_stride=cache.stride(0), row_slot=row_slot.data_ptr(), row_pos=row_pos.data_ptr(), batch=B,
                              n_head=n_head, dk=dk, dv=dv, r=r, max_seq=max_seq, n_split=n_split, scale=float(scale), dtype=_code(q),
                              workspace=ws.data_ptr(), workspace_bytes=ws.numel(), dk2=shared_dims, sink=C.ptr(sink), gate=C.ptr(gate),
                              ldg=0 if gate is None else gate.stride(0), gate_mode=_gate_mode(gate, n_head, dv))
    C.check(lib.b200_latent_decode(ctypes.byref(args), C.stream_ptr(q.device)), "latent_decode")
    return out


def latent_decode_tune(force_any_size_kernel: bool = False) -> bool:
    """Test knob: keep bf16 decode attention on the any-size kernel; returns the previous setting."""
    return bool(C.load_core().b200_latent_decode_tune(int(force_any_size_kernel)))


def moe_route(x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], top: int, n_group: int, keep: int,
              softmax: bool = False, group_max: bool = False, topk_softmax: bool = False, bias: bool = False):
    """-> (ids int32 (n, top), weights fp32 (n, top)); see b200_moe_route.  softmax: scores are a softmax over all experts
    instead of sigmoids; group_max: a group ranks by its largest score instead of the sum of its two largest; topk_softmax: the
    largest raw logits are chosen and weighted by a softmax among those few; bias: `correction` is a bias inside the logit."""
    C.require_cuda(x, w_router, correction)
    n, d = x.shape
    E = w_router.shape[0]
    ids = torch.empty((n, top), dtype=torch.int32, device=x.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=x.device)
    C.check(C.load_core().b200_moe_route(x.data_ptr(), w_router.data_ptr(), C.ptr(correction), ids.data_ptr(), wts.data_ptr(), n, d, E, top, n_group,
                                         keep, (C.ROUTE_SOFTMAX if softmax else 0) | (C.ROUTE_GROUP_MAX if group_max else 0)
                                         | (C.ROUTE_TOPK_SOFTMAX if topk_softmax else 0) | (C.ROUTE_BIAS if bias else 0), _code(x),
                                         C.stream_ptr(x.device)), "moe_route")
    return ids, wts


MOE_GEMV_MAX_PAIRS = 64   # up to this many (token, choice) pairs the experts run as weight-streaming GEMVs


def moe_experts(x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, gated: bool = False,
                limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """out[t] = sum_k wts[t, k] * W_down[ids[t, k]] relu(W_up[ids[t, k]] x[t])^2 with stacked weights (E, ff, d) / (E, d, ff);
    gated: W_up is (E, 2 ff, d), gate rows first, and the hidden vector is silu(gate) * up -- or, with limit > 0, the clamped form
    g sigmoid(alpha g) (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit)."""
    C.require_cuda(x, ids, wts, w_up, w_down)
    n, d = x.shape
    E, ff, top = w_up.shape[0], w_down.shape[2], ids.shape[1]
    lib, st, code = C.load_core(), C.stream_ptr(x.device), _code(x)
    out = torch.empty((n, d), dtype=x.dtype, device=x.device)
    if n * top <= MOE_GEMV_MAX_PAIRS:
        hidden = torch.empty((n * top, ff), dtype=x.dtype, device=x.device)
        C.check(lib.b200_moe_gemv(x.data_ptr(), ids.data_ptr(), wts.data_ptr(), w_up.data_ptr(), w_down.data_ptr(), hidden.data_ptr(), out.data_ptr(),
                                  n, top, d, ff, (2 if limit > 0 else 1) if gated else 0, float(limit), float(alpha), code, st), "moe_gemv")
        return out
    plan = moe_plan(ids, E)
    up_rows = 2 * ff if gated else ff
    hidden = torch.empty((n * top, up_rows), dtype=x.dtype, device=x.device)
    C.check(lib.b200_moe_gemm(x.data_ptr(), x.stride(0), plan.slot_token.data_ptr(), w_up.data_ptr(), hidden.data_ptr(), up_rows,
                              plan.expert_off.data_ptr(), plan.tile_off.data_ptr(), n * top, E, up_rows, d, 0 if gated else 1, code, st), "moe_gemm(up)")
    if gated:
        hidden = glu_clamped(hidden, limit, alpha) if limit > 0 else glu(hidden, C.ACT_SILU)
    y = torch.empty((n * top, d), dtype=x.dtype, device=x.device)
    C.check(lib.b200_moe_gemm(hidden.data_ptr(), ff, None, w_down.data_ptr(), y.data_ptr(), d, plan.expert_off.data_ptr(), plan.tile_off.data_ptr(),
                              n * top, E, d, ff, 0, code, st), "moe_gemm(down)")
    return moe_combine(y, plan, wts)


class MoEPlan:
    """The (token, choice) pairs of a step sorted by expert: rows [expert_off[e], expert_off[e + 1]) belong to expert e;
    slot_token[row] is the token of a sorted row, slot_of[t * top + k] the row of a pair (all int32, on the device)."""

    __slots__ = ("expert_off", "tile_off", "slot_token", "slot_of", "tokens", "top")


def moe_plan(ids: torch.Tensor, n_expert: int) -> MoEPlan:
    n, top = ids.shape
    E = n_expert
    meta = torch.empty(2 * (E + 1) + 2 * n * top, dtype=torch.int32, device=ids.device)
    plan = MoEPlan()
    plan.tokens, plan.top = n, top
    plan.expert_off, plan.tile_off = meta[: E + 1], meta[E + 1 : 2 * (E + 1)]
    plan.slot_token, plan.slot_of = meta[2 * (E + 1) : 2 * (E + 1) + n * top], meta[2 * (E + 1) + n * top :]
    C.check(C.load_core().b200_moe_plan(ids.data_ptr(), n, top, E, plan.expert_off.data_ptr(), plan.tile_off.data_ptr(), plan.slot_token.data_ptr(),
                                        plan.slot_of.data_ptr(), C.stream_ptr(ids.device)), "moe_plan")
    return plan


def moe_combine(y: torch.Tensor, plan: MoEPlan, wts: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_k wts[t, k] * y[slot_of[t, k]] (fp32 sum in the order of k)."""
    d = y.shape[-1]
    out = torch.empty((plan.tokens, d), dtype=y.dtype, device=y.device)
    C.check(C.load_core().b200_moe_combine(y.data_ptr(), plan.slot_of.data_ptr(), wts.data_ptr(), out.data_ptr(), plan.tokens, plan.top, d, _code(y),
                                           C.stream_ptr(y.device)), "moe_combine")
    return out


# ---------------------------------------------------------------------------------------------------------
# sequence-state mechanisms: sandwich-normed residual, short convolutions, gated delta rule, windowed attention over a ring
# (csrc/resid.cu, shortconv.cu, delta.cu, window_attn.cu).  A step's rows are described by ``seqs`` int32 (S, 4) = first row,
# rows, first position, state slot, and ``row_seq`` int32 (n,).
# ---------------------------------------------------------------------------------------------------------
def sandwich_residual(x: torch.Tensor, y0: torch.Tensor, post_w: Optional[torch.Tensor], eps: float, *, w0: Optional[torch.Tensor] = None,
                      y1: Optional[torch.Tensor] = None, w1: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None,
                      pre_w: Optional[torch.Tensor] = None, act: Optional[torch.Tensor] = None) -> None:
    """x (fp32, in place) += norm(y) * post_w [+ extra]; act = T(norm(x) * pre_w).  y = y0, or with y1 the mean of the two branches
    each normed with its weight (w0, w1)."""
    C.require_cuda(x, y0, y1, post_w, extra, pre_w, act)
    if x.dtype != torch.float32 or not x.is_contiguous() or not y0.is_contiguous() or (y1 is not None and not y1.is_contiguous()):
        raise C.B200Error("sandwich_residual: x must be contiguous fp32, the branches contiguous")
    if extra is not None and (extra.dtype != torch.float32 or not extra.is_contiguous()):
        raise C.B200Error("sandwich_residual: extra must be contiguous fp32")
    d = x.shape[-1]
    args = C.SandwichArgs(y0=y0.data_ptr(), w0=C.ptr(w0), y1=C.ptr(y1), w1=C.ptr(w1), post_w=C.ptr(post_w), extra=C.ptr(extra), pre_w=C.ptr(pre_w),
                          x=x.data_ptr(), act=C.ptr(act), rows=x.numel() // d, d=d, eps=float(eps), dtype=_code(y0))
    C.check(C.load_core().b200_sandwich_residual(ctypes.byref(args), C.stream_ptr(x.device)), "sandwich_residual")


def activation_(x: torch.Tensor, kind: int) -> torch.Tensor:
    """In place: C.ACT_GELU (erf), C.ACT_GELU_TANH, C.ACT_SILU, C.ACT_RELU2."""
    C.require_cuda(x)
    if not x.is_contiguous():
        raise C.B200Error("activation_: contiguous tensor")
    C.check(C.load_core().b200_activation(x.data_ptr(), x.numel(), kind, _code(x), C.stream_ptr(x.device)), "activation")
    return x


def glu(x: torch.Tensor, kind: int) -> torch.Tensor:
    """x (rows, 2 ff) = [gate | up] -> act(gate) * up (rows, ff)."""
    C.require_cuda(x)
    if not x.is_contiguous() or x.shape[-1] % 2:
        raise C.B200Error("glu: contiguous rows of even length")
    ff = x.shape[-1] // 2
    out = torch.empty(x.shape[:-1] + (ff,), dtype=x.dtype, device=x.device)
    C.check(C.load_core().b200_glu(x.data_ptr(), out.data_ptr(), x.numel() // (2 * ff), ff, kind, _code(x), C.stream_ptr(x.device)), "glu")
    return out


def xielu_(x: torch.Tensor, params: torch.Tensor) -> torch.Tensor:
    """In place: z > 0: softplus(p) z^2 + z / 2; z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2, with (p, q) = params."""
    C.require_cuda(x, params)
    if not x.is_contiguous() or params.dtype != x.dtype or params.numel() != 2 or not params.is_contiguous():
        raise C.B200Error("xielu_: contiguous tensor, two parameters in its dtype")
    C.check(C.load_core().b200_xielu(x.data_ptr(), x.numel(), params.data_ptr(), _code(x), C.stream_ptr(x.device)), "xielu")
    return x


def glu_clamped(x: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """x (rows, 2 ff) = [gate | up] -> g sigmoid(alpha g) (u + 1) (rows, ff), g = min(gate, limit), u = clamp(up, -limit, limit)."""
    C.require_cuda(x)
    if not x.is_contiguous() or x.shape[-1] % 2:
        raise C.B200Error("glu_clamped: contiguous rows of even length")
    ff = x.shape[-1] // 2
    out = torch.empty(x.shape[:-1] + (ff,), dtype=x.dtype, device=x.device)
    C.check(C.load_core().b200_glu_clamped(x.data_ptr(), out.data_ptr(), x.numel() // (2 * ff), ff, float(limit), float(alpha), _code(x),
                                           C.stream_ptr(x.device)), "glu_clamped")
    return out


def scaled_residual(x: torch.Tensor, *, y0: Optional[torch.Tensor] = None, s0: Optional[torch.Tensor] = None, y1: Optional[torch.Tensor] = None,
                    y2: Optional[torch.Tensor] = None, s1: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None,
                    row_add: Optional[torch.Tensor] = None, cast: Optional[torch.Tensor] = None, norm: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                    act: Optional[torch.Tensor] = None) -> None:
    """x (fp32 (rows, d), in place) += y0 * s0 + (y1 + y2) * s1 + extra + row_add; cast = T(x); act = T(tanh(alpha x) * w + b) with
    norm = (alpha, w, b).  y*, s* (d numbers), row_add (d numbers), cast and act share the matrix-product dtype; extra is fp32 rows."""
    alpha, nw, nb = norm if norm is not None else (None, None, None)
    C.require_cuda(x, y0, s0, y1, y2, s1, extra, row_add, cast, alpha, nw, nb, act)
    if x.dtype != torch.float32 or not x.is_contiguous() or (extra is not None and (extra.dtype != torch.float32 or not extra.is_contiguous())):
        raise C.B200Error("scaled_residual: the stream and extra must be contiguous fp32")
    typed = [t for t in (y0, s0, y1, y2, s1, row_add, cast, alpha, nw, nb, act) if t is not None]
    if not typed or any(t.dtype != typed[0].dtype or not t.is_contiguous() for t in typed):
        raise C.B200Error("scaled_residual: branches, scales, norm and outputs in one dtype, contiguous")
    if norm is not None and act is None:
        raise C.B200Error("scaled_residual: the norm needs somewhere to go")
    d = x.shape[-1]
    args = C.ScaledResidualArgs(y0=C.ptr(y0), s0=C.ptr(s0), y1=C.ptr(y1), y2=C.ptr(y2), s1=C.ptr(s1), extra=C.ptr(extra), row_add=C.ptr(row_add),
                                x=x.data_ptr(), cast=C.ptr(cast), alpha=C.ptr(alpha), nw=C.ptr(nw), nb=C.ptr(nb), act=C.ptr(act) if norm is not None else None,
                                rows=x.numel() // d, d=d, dtype=_code(typed[0]))
    C.check(C.load_core().b200_scaled_residual(ctypes.byref(args), C.stream_ptr(x.device)), "scaled_residual")


def conv_group(w: torch.Tensor, out: torch.Tensor, col0: int, heads: int, dim: int, *, act: int = 0, post: int = 0, rot_dims: int = 0,
               inv_freq: Optional[torch.Tensor] = None, rot_mscale: float = 1.0, post_scale: float = 1.0, eps: float = 0.0) -> "C.ConvGroup":
    """One group of heads for ``short_conv``: act 0 none / 1 silu; post 0 none / 1 rotate + RMS norm / 2 unit vector."""
    if not w.is_contiguous() or out.stride(-1) != 1 or out.dtype not in (w.dtype, torch.float32):
        raise C.B200Error("conv_group: contiguous weights, output rows in the model dtype or fp32")
    if inv_freq is not None and (inv_freq.dtype != torch.float64 or inv_freq.numel() < rot_dims // 2 or not inv_freq.is_cuda):
        raise C.B200Error("conv_group: inv_freq must be a CUDA float64 tensor of rot_dims / 2 entries")
    return C.ConvGroup(w=w.data_ptr(), out=out.data_ptr(), ld_out=out.stride(-2), inv_freq=C.ptr(inv_freq), col0=col0, heads=heads, dim=dim,
                       act=act, post=post, rot_dims=rot_dims, out_f32=int(out.dtype == torch.float32 and w.dtype != torch.float32),
                       rot_mscale=float(rot_mscale), post_scale=float(post_scale), eps=float(eps))


def short_conv(inp: torch.Tensor, groups: Sequence["C.ConvGroup"], taps: int, tail: Optional[torch.Tensor], seqs: torch.Tensor,
               row_seq: torch.Tensor) -> None:
    """Causal convolution over `taps` positions on the first tail.shape[-1] columns of inp (rows, cols), per group of heads with
    its activation and per-head step; tail (slots, taps - 1, conv_cols) holds what earlier steps left, and is updated."""
    C.require_cuda(inp, tail, seqs, row_seq)
    if inp.stride(-1) != 1 or seqs.dtype != torch.int32 or row_seq.dtype != torch.int32 or not seqs.is_contiguous():
        raise C.B200Error("short_conv: unit inner stride, int32 seqs and row_seq")
    if tail is not None and (tail.dtype != inp.dtype or not tail.is_contiguous()):
        raise C.B200Error("short_conv: the tail must be contiguous in the model dtype")
    lib, st = C.load_core(), C.stream_ptr(inp.device)
    arr = (C.ConvGroup * len(groups))(*groups)
    cols = sum(g.heads * g.dim for g in groups) if tail is None else tail.shape[-1]
    stride = 0 if tail is None else tail.stride(0)
    C.check(lib.b200_short_conv(inp.data_ptr(), inp.stride(0), arr, len(groups), taps, C.ptr(tail), stride, cols, seqs.data_ptr(), row_seq.data_ptr(),
                                inp.shape[0], _code(inp), st), "short_conv")
    if tail is not None and taps > 1:
        C.check(lib.b200_conv_tail_update(inp.data_ptr(), inp.stride(0), tail.data_ptr(), stride, cols, taps, seqs.data_ptr(), seqs.shape[0],
                                          _code(inp), st), "conv_tail_update")


def delta_rule_state_floats(dk: int, dv: int) -> int:
    """fp32 numbers one head's state takes in the kernel's own order."""
    return int(C.load_core().b200_delta_rule_state_floats(dk, dv))


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta_in: torch.Tensor, decay_in: torch.Tensor, a_log: torch.Tensor,
               dt_bias: torch.Tensor, state: torch.Tensor, seqs: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int,
               channel_decay: bool, max_rows: int = 0) -> torch.Tensor:
    """Gated delta rule over the step's rows; state (slots, floats) fp32 is read (unless the sequence starts at 0) and written.
    q, k (n, kv_heads * dk), v (n, heads * dv) fp32; beta_in (n, heads), decay_in (n, heads [* dk]) raw projections; max_rows: the
    longest sequence's rows in this step (picks the launch shape).  -> fp32 (n, heads * dv)"""
    C.require_cuda(q, k, v, beta_in, decay_in, a_log, dt_bias, state, seqs)
    if not (q.dtype == k.dtype == v.dtype == state.dtype == torch.float32) or seqs.dtype != torch.int32 or not seqs.is_contiguous():
        raise C.B200Error("delta_rule: q, k, v and the state are fp32, seqs int32")
    if beta_in.dtype != decay_in.dtype or a_log.dtype != beta_in.dtype or dt_bias.dtype != beta_in.dtype:
        raise C.B200Error("delta_rule: projections and parameters in one dtype")
    for t in (q, k, v, beta_in, decay_in):
        if t.stride(-1) != 1:
            raise C.B200Error("delta_rule: unit inner strides")
    if state.stride(0) < heads * delta_rule_state_floats(dk, dv) or not state.is_contiguous():
        raise C.B200Error("delta_rule: the state slots are too small")
    out = torch.empty((q.shape[0], heads * dv), dtype=torch.float32, device=q.device)
    args = C.DeltaRuleArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), ldq=q.stride(0), ldk=k.stride(0), ldv=v.stride(0),
                           beta_in=beta_in.data_ptr(), ld_beta=beta_in.stride(0), decay_in=decay_in.data_ptr(), ld_decay=decay_in.stride(0),
                           a_log=a_log.data_ptr(), dt_bias=dt_bias.data_ptr(), state=state.data_ptr(), state_slot_stride=state.stride(0),
                           out=out.data_ptr(), ldo=out.stride(0), seqs=seqs.data_ptr(), n_seqs=seqs.shape[0], heads=heads, kv_heads=kv_heads,
                           dk=dk, dv=dv, channel_decay=int(channel_decay), dtype=_code(beta_in), max_rows=int(max_rows))
    C.check(C.load_core().b200_delta_rule(ctypes.byref(args), C.stream_ptr(q.device)), "delta_rule")
    return out


GATE_SILU, GATE_SIGMOID = 1, 2


def gated_rms_heads(o: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, heads: int, dv: int, gate: int, eps: float) -> torch.Tensor:
    """o fp32 (n, heads * dv), z (n, heads * dv) raw gate projection -> T (n, heads * dv): per-head RMS norm * weight * gate(z)."""
    C.require_cuda(o, z, weight)
    if o.dtype != torch.float32 or o.stride(-1) != 1 or z.stride(-1) != 1 or z.dtype != weight.dtype:
        raise C.B200Error("gated_rms_heads: o fp32, gate and weight in the model dtype")
    out = torch.empty((o.shape[0], heads * dv), dtype=z.dtype, device=o.device)
    C.check(C.load_core().b200_gated_rms_heads(o.data_ptr(), o.stride(0), z.data_ptr(), z.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0),
                                               o.shape[0], heads, dv, gate, float(eps), _code(z), C.stream_ptr(o.device)), "gated_rms_heads")
    return out


WINDOW_PREFILL_MMA = True   # tests switch it off to run whole prompts with tensor-core-sized heads on the any-size kernel


def window_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_ring: torch.Tensor, v_ring: torch.Tensor, sink: Optional[torch.Tensor],
                seqs: torch.Tensor, row_seq: torch.Tensor, max_q_len: int, n_head: int, n_kv_head: int, dk: int, dv: int, window: int,
                scale: float, from_start: bool = False, *, dist: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                gate: Optional[torch.Tensor] = None, gate_per_head: bool = False) -> torch.Tensor:
    """Sliding-window attention with a sink over this step's k / v rows and the rings (slots, ring, G * dk | dv) of earlier
    positions; afterwards the step's rows enter the rings.  -> (n, n_head * dv).  from_start: every sequence of the step begins
    at position 0, so nothing is read from the rings -- bf16 prompts with 64- or 128-wide heads then run on the tensor-core tiles
    of the prefill kernel the other models use.  dist = (r1, r2), n_head numbers each: score -= r1 ln(1 + r2 (i - j)).  gate: raw
    projections of the rows (n, n_head) with gate_per_head, else (n, n_head * dv); the output is multiplied by their sigmoid."""
    r1, r2 = dist if dist is not None else (None, None)
    C.require_cuda(q, k, v, k_ring, v_ring, sink, seqs, row_seq, r1, r2, gate)
    if dist is not None and not (r1.dtype == r2.dtype == q.dtype and r1.numel() == r2.numel() == n_head and r1.is_contiguous() and r2.is_contiguous()):
        raise C.B200Error("window_attn: the distance bias is two contiguous vectors of n_head numbers in the operands' dtype")
    if gate is not None and (gate.dtype != q.dtype or gate.stride(-1) != 1 or gate.shape[-1] != (n_head if gate_per_head else n_head * dv)):
        raise C.B200Error("window_attn: the gate is (rows, n_head) or (rows, n_head * dv) in the operands' dtype with a unit inner stride")
    gate_mode = 0 if gate is None else (1 if gate_per_head else 2)
    ldg = 0 if gate is None else gate.stride(0)
    if not (q.dtype == k.dtype == v.dtype == k_ring.dtype == v_ring.dtype) or not (k_ring.is_contiguous() and v_ring.is_contiguous()):
        raise C.B200Error("window_attn: one dtype, contiguous rings")
    if q.stride(-1) != 1 or k.stride(-1) != 1 or v.stride(-1) != 1 or seqs.dtype != torch.int32 or not seqs.is_contiguous():
        raise C.B200Error("window_attn: unit inner strides, int32 seqs")
    ring = k_ring.shape[1]
    out = torch.empty((q.shape[0], n_head * dv), dtype=q.dtype, device=q.device)
    lib, st = C.load_core(), C.stream_ptr(q.device)
    if (from_start and max_q_len > 1 and WINDOW_PREFILL_MMA and q.dtype == torch.bfloat16 and dk == dv and dk in (64, 128)
            and not (q.stride(0) | k.stride(0) | v.stride(0)) & 7 and not (q.data_ptr() | k.data_ptr() | v.data_ptr() | seqs.data_ptr()) & 15):
        C.check(lib.b200_attn_prefill_window_ex(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), seqs.data_ptr(),
                                                seqs.shape[0], max_q_len, out.data_ptr(), out.stride(0), n_head, n_kv_head, dk, float(scale), window,
                                                C.ptr(sink), C.ptr(r1), C.ptr(r2), C.ptr(gate), ldg, gate_mode, st), "attn_prefill_window")
        C.check(lib.b200_ring_store(k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), k_ring.data_ptr(), v_ring.data_ptr(), ring, n_kv_head * dk,
                                    n_kv_head * dv, seqs.data_ptr(), row_seq.data_ptr(), q.shape[0], _code(q), st), "ring_store")
        return out
    # the any-size kernels store the step's rows into the rings themselves (single rows: inside the attention kernel)
    args = C.WindowAttnArgs(row_seq=row_seq.data_ptr(), rows=q.shape[0], q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(),
                            ldq=q.stride(0), ldk=k.stride(0), ldv=v.stride(0), ldo=out.stride(0), k_ring=k_ring.data_ptr(), v_ring=v_ring.data_ptr(), sink=C.ptr(sink), seqs=seqs.data_ptr(),
                            n_seqs=seqs.shape[0], max_q_len=max_q_len, ring=ring, n_head=n_head, n_kv_head=n_kv_head, dk=dk, dv=dv, window=window,
                            scale=float(scale), dtype=_code(q), dist_r1=C.ptr(r1), dist_r2=C.ptr(r2), gate=C.ptr(gate), ldg=ldg, gate_mode=gate_mode)
    C.check(lib.b200_window_attn(ctypes.byref(args), st), "window_attn")
    return out


def window_attn_tune(force_tiled_kernel: bool = False) -> bool:
    """Test knob: keep single-row steps on the tiled kernel; returns the previous setting."""
    return bool(C.load_core().b200_window_attn_tune(int(force_tiled_kernel)))


# grouped norms with an average over depth, per-head rotation, attention with scores mixed over the heads
# (csrc/depth.cu, rope.cu, talk_attn.cu)
# ---------------------------------------------------------------------------------------------------------
def depth_residual(x_in: torch.Tensor, x_out: torch.Tensor, eps: float, groups: int, *, y: Optional[torch.Tensor] = None,
                   post_w: Optional[torch.Tensor] = None, stack: Optional[torch.Tensor] = None, m: int = 0, depth_w: Optional[torch.Tensor] = None,
                   avg: Optional[torch.Tensor] = None, pre_w: Optional[torch.Tensor] = None, act: Optional[torch.Tensor] = None) -> None:
    """x_out (fp32) = x_in + gnorm(y) * post_w (without y: x_in itself); avg (fp32) = sum_{j < m} depth_w[j] X_j with X_j = stack[j] for
    j < m - 1 and X_{m-1} = x_out; act = T(gnorm(avg, or x_out) * pre_w).  gnorm divides each of `groups` equal consecutive pieces of
    a row by its own root mean square.  `stack` (layers, rows, d) fp32; y, the weights and act share the matrix-product dtype."""
    C.require_cuda(x_in, x_out, y, post_w, stack, depth_w, avg, pre_w, act)
    for t in (x_in, x_out, stack, avg):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise C.B200Error("depth_residual: the stream, the stack and the average must be contiguous fp32")
    ref = y if y is not None else (act if act is not None else depth_w)
    for t in (y, post_w, depth_w, pre_w, act):
        if t is not None and (t.dtype != ref.dtype or not t.is_contiguous()):
            raise C.B200Error("depth_residual: branch, weights and act must be contiguous and of one dtype")
    d = x_in.shape[-1]
    rows = x_in.numel() // d
    if avg is not None and (depth_w is None or depth_w.numel() < m or m < 1 or (m > 1 and (stack is None or stack.shape[0] < m - 1))):
        raise C.B200Error("depth_residual: the average over m results needs m weights and m - 1 earlier results")
    args = C.DepthResidualArgs(y=C.ptr(y), post_w=C.ptr(post_w), x_in=x_in.data_ptr(), x_out=x_out.data_ptr(), stack=C.ptr(stack),
                               stack_stride=0 if stack is None else stack.stride(0), depth_w=C.ptr(depth_w), avg=C.ptr(avg), pre_w=C.ptr(pre_w),
                               act=C.ptr(act), rows=rows, d=d, groups=groups, m=m, eps=float(eps), dtype=C.DTYPE_CODE[ref.dtype])
    C.check(C.load_core().b200_depth_residual(ctypes.byref(args), C.stream_ptr(x_in.device)), "depth_residual")


def rope_seg(inp: torch.Tensor, out: torch.Tensor, heads: int, dim: int, *, norm_w: Optional[torch.Tensor] = None, freq: Optional[torch.Tensor] = None,
             rot_off: int = 0, rot_dims: int = 0, interleaved: bool = True, mag: float = 1.0, out_rows: Optional[torch.Tensor] = None,
             in_stride: Optional[int] = None, out_stride: Optional[int] = None) -> "C.HeadRopeSeg":
    """One group of `heads` heads of `dim` numbers for ``head_rope``: `inp` / `out` are 2-d views (rows, columns) whose first column
    is the group's first head; heads lie `in_stride` / `out_stride` (default dim) numbers apart.  freq: fp32 (rot_dims / 2,)."""
    if inp.stride(-1) != 1 or out.stride(-1) != 1 or inp.dtype != out.dtype:
        raise C.B200Error("head_rope: rows of one dtype with unit inner stride")
    if freq is not None and (freq.dtype != torch.float32 or not freq.is_contiguous() or freq.numel() < rot_dims // 2):
        raise C.B200Error("head_rope: frequencies must be contiguous fp32, one per rotated pair")
    if out_rows is not None and (out_rows.dtype != torch.int64 or not out_rows.is_contiguous()):
        raise C.B200Error("head_rope: row indices must be contiguous int64")
    return C.HeadRopeSeg(inp=inp.data_ptr(), out=out.data_ptr(), norm_w=C.ptr(norm_w), freq=C.ptr(freq) if rot_dims else None, out_rows=C.ptr(out_rows),
                         ld_in=inp.stride(-2), ld_out=out.stride(-2), heads=heads, dim=dim, in_stride=dim if in_stride is None else in_stride,
                         out_stride=dim if out_stride is None else out_stride, rot_off=rot_off, rot_dims=rot_dims, interleaved=int(interleaved),
                         mag=float(mag))


def head_rope(rows: int, row_pos: torch.Tensor, eps: float, *segs: "C.HeadRopeSeg", dtype: torch.dtype, device: torch.device) -> None:
    """One launch over `rows` rows for up to three groups of heads built by ``rope_seg``: per head an optional weighted RMS norm, the
    rotation of a run of its dimensions by the row's position, and the move to its destination (in place, dense, or cache rows)."""
    if row_pos.dtype != torch.int32 or not row_pos.is_contiguous():
        raise C.B200Error("head_rope: positions must be contiguous int32")
    arr = (C.HeadRopeSeg * len(segs))(*segs)
    C.check(C.load_core().b200_head_rope(arr, len(segs), row_pos.data_ptr(), rows, float(eps), C.DTYPE_CODE[dtype], C.stream_ptr(device)), "head_rope")


TALK_PREFILL_MMA = True          # tests switch it off to reach the any-size kernel with tensor-core-sized heads
TALK_PREFILL_MMA_MIN_ROWS = 32   # shorter portions stay on the any-size kernel
TALK_PREFILL_PLANE_BYTES = 8 << 30


def talk_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seqs: torch.Tensor, max_q_len: int, n_head: int, n_kv_head: int, dk: int,
              dv: int, max_seq: int, scale: float, n_split: int = 1, *, talk: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None,
              context: int = 0) -> torch.Tensor:
    """Causal attention over cached keys and values whose scores are mixed over the heads by `talk` (H, H) before the softmax, with an
    optional sink logit per head.  q (n, H * dk); k_cache / v_cache: 2-d views (slots * max_seq, G * dk | G * dv) of the cache rows;
    seqs int32 (S, 4) = first row, rows, first position, cache slot.  Returns (n, H * dv).  With `context` (an upper bound of any row's
    position + 1), bf16 prompts with dk = dv in {64, 128} run on the tensor-core tiles over fp32 score planes."""
    C.require_cuda(q, k_cache, v_cache, seqs, talk, sink)
    n = q.shape[0]
    s_ld = -(-max(context, 1) // 64) * 64
    lib = C.load_core()
    if (context > 0 and TALK_PREFILL_MMA and q.dtype == torch.bfloat16 and k_cache.dtype == v_cache.dtype == torch.bfloat16
            and dk == dv and dk in (64, 128) and n_head <= 64 and max_q_len >= TALK_PREFILL_MMA_MIN_ROWS
            and seqs.dtype == torch.int32 and seqs.is_contiguous() and q.stride(-1) == k_cache.stride(-1) == v_cache.stride(-1) == 1
            and not (q.stride(0) | k_cache.stride(0) | v_cache.stride(0)) & 7
            and not (q.data_ptr() | k_cache.data_ptr() | v_cache.data_ptr() | seqs.data_ptr()) & 15
            and all(t is None or (t.dtype == torch.bfloat16 and t.is_contiguous()) for t in (talk, sink))):
        plane = lib.b200_attn_prefill_mixed_plane_floats(seqs.shape[0], max_q_len, s_ld)
        if n_head * plane * 4 <= TALK_PREFILL_PLANE_BYTES:
            planes = torch.empty((n_head, plane), dtype=torch.float32, device=q.device)
            out = torch.empty((n, n_head * dv), dtype=q.dtype, device=q.device)
            C.check(lib.b200_attn_prefill_mixed(q.data_ptr(), q.stride(0), k_cache.data_ptr(), k_cache.stride(0), v_cache.data_ptr(), v_cache.stride(0),
                                                seqs.data_ptr(), seqs.shape[0], max_q_len, max_seq, C.ptr(talk), C.ptr(sink), out.data_ptr(), out.stride(0),
                                                n_head, n_kv_head, dk, float(scale), planes.data_ptr(), s_ld, C.stream_ptr(q.device)), "attn_prefill_mixed")
            return out
    ws = _ws("talk", q.device, lib.b200_talk_attn_workspace_bytes(n, n_head, dv, n_split))
    out = torch.empty((n, n_head * dv), dtype=q.dtype, device=q.device)
    args = C.TalkAttnArgs(q=q.data_ptr(), ldq=q.stride(0), k_cache=k_cache.data_ptr(), ldk=k_cache.stride(0), v_cache=v_cache.data_ptr(),
                          ldv=v_cache.stride(0), talk=C.ptr(talk), sink=C.ptr(sink), out=out.data_ptr(), ldo=out.stride(0), seqs=seqs.data_ptr(),
                          n_seqs=seqs.shape[0], max_q_len=max_q_len, rows=n, n_head=n_head, n_kv_head=n_kv_head, dk=dk, dv=dv, max_seq=max_seq,
                          n_split=n_split, scale=float(scale), dtype=_code(q), workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    C.check(lib.b200_talk_attn(ctypes.byref(args), C.stream_ptr(q.device)), "talk_attn")
    return out
