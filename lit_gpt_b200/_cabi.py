"""ctypes binding of ``libb200gpt.so`` — the ONLY way the Python package reaches the kernels.

There is no fallback: if the library is missing and cannot be built, importing any kernel raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libb200gpt.so")

BF16, F16, F32 = 0, 1, 2
Q_NF4, Q_FP4, Q_INT4 = 0, 1, 2
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
DTYPE_CODE = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32}


class LinearInt8Args(ctypes.Structure):  # mirrors b200_linear_int8_args
    _fields_ = [("x", c_void_p), ("cb", c_void_p), ("scb", c_void_p), ("bias", c_void_p), ("y", c_void_p),
                ("M", c_int64), ("N", c_int64), ("K", c_int64), ("threshold", c_float), ("workspace", c_void_p),
                ("workspace_bytes", c_size_t)]


class QGemvArgs(ctypes.Structure):
    _fields_ = [
        ("packed", c_void_p), ("scale", c_void_p), ("packed2", c_void_p), ("scale2", c_void_p),
        ("qtype", c_int), ("blocksize", c_int), ("N", c_int64), ("K", c_int64),
        ("x", c_void_p), ("delta", c_void_p), ("x_out", c_void_p), ("norm_weight", c_void_p),
        ("norm_eps", c_float), ("batch", c_int), ("epilogue", c_int),
        ("bias", c_void_p), ("residual", c_void_p), ("y", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


class TpHandoff(ctypes.Structure):  # mirrors b200_tp_handoff
    _fields_ = [("world", c_int), ("rank", c_int), ("peer_y", c_void_p * 8), ("reduced", c_void_p), ("reserved", c_void_p * 7), ("send_seq", c_void_p),
                ("slots", c_void_p), ("slot_stride", c_int64), ("recv_seq", c_void_p), ("recv_done", c_void_p)]


class KvHint(ctypes.Structure):
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("pos", c_void_p), ("pos_is_int64", c_int), ("chunks", c_int),
                ("chunk_stride", c_int64), ("row_bytes", c_int), ("max_rows", c_int)]


class QGemvTiledArgs(ctypes.Structure):
    _fields_ = [
        ("tiled", c_void_p), ("tiled2", c_void_p), ("qtype", c_int), ("blocksize", c_int), ("N", c_int64), ("K", c_int64),
        ("x", c_void_p), ("delta", c_void_p), ("x_out", c_void_p), ("norm_weight", c_void_p),
        ("norm_eps", c_float), ("batch", c_int), ("epilogue", c_int),
        ("bias", c_void_p), ("bias2", c_void_p), ("residual", c_void_p), ("y", c_void_p),
        ("prefetch", c_void_p), ("prefetch_bytes", c_int64), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("tp", ctypes.POINTER(TpHandoff)), ("kv_hint", ctypes.POINTER(KvHint)), ("attn", c_void_p), ("fold", c_int),
    ]


class AttnDecodeArgs(ctypes.Structure):
    _fields_ = [
        ("qkv", c_void_p), ("cos", c_void_p), ("sin", c_void_p), ("table_dtype", c_int), ("table_preselected", c_int), ("rope_n_elem", c_int),
        ("pos", c_void_p), ("pos_is_int64", c_int), ("k_cache", c_void_p), ("v_cache", c_void_p), ("out", c_void_p),
        ("batch", c_int), ("n_head", c_int), ("n_groups", c_int), ("head_size", c_int), ("max_seq", c_int),
        ("num_splits", c_int), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


class QGemmArgs(ctypes.Structure):
    _fields_ = [
        ("packed", c_void_p), ("scale", c_void_p), ("qtype", c_int), ("blocksize", c_int),
        ("M", c_int64), ("N", c_int64), ("K", c_int64), ("x", c_void_p), ("bias", c_void_p), ("y", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


class RmsRowsSeg(ctypes.Structure):  # mirrors b200_rms_rows_seg
    _fields_ = [("inp", c_void_p), ("weight", c_void_p), ("out", c_void_p), ("in_rows", c_void_p), ("out_rows", c_void_p),
                ("ld_in", c_int64), ("ld_out", c_int64), ("d", c_int), ("plus_one", c_int)]


class LatentPrefillArgs(ctypes.Structure):  # mirrors b200_latent_prefill_args
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p),
                ("ldq", c_int64), ("ldk", c_int64), ("ldv", c_int64), ("ldo", c_int64), ("seqs", c_void_p),
                ("n_seqs", c_int), ("max_q_len", c_int), ("n_head", c_int), ("dk", c_int), ("dv", c_int),
                ("scale", c_float), ("dtype", c_int),
                ("k2", c_void_p), ("ldk2", c_int64), ("dk2", c_int), ("sink", c_void_p), ("gate", c_void_p), ("ldg", c_int64), ("gate_mode", c_int)]


class LatentDecodeArgs(ctypes.Structure):  # mirrors b200_latent_decode_args
    _fields_ = [("q", c_void_p), ("w_uk", c_void_p), ("w_uv", c_void_p), ("cache", c_void_p), ("out", c_void_p),
                ("ldq", c_int64), ("ldo", c_int64), ("slot_stride", c_int64), ("row_slot", c_void_p), ("row_pos", c_void_p),
                ("batch", c_int), ("n_head", c_int), ("dk", c_int), ("dv", c_int), ("r", c_int), ("max_seq", c_int), ("n_split", c_int),
                ("scale", c_float), ("dtype", c_int), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
                ("dk2", c_int), ("sink", c_void_p), ("gate", c_void_p), ("ldg", c_int64), ("gate_mode", c_int)]


class DepthResidualArgs(ctypes.Structure):  # mirrors b200_depth_residual_args
    _fields_ = [("y", c_void_p), ("post_w", c_void_p), ("x_in", c_void_p), ("x_out", c_void_p), ("stack", c_void_p), ("stack_stride", c_int64),
                ("depth_w", c_void_p), ("avg", c_void_p), ("pre_w", c_void_p), ("act", c_void_p), ("rows", c_int64), ("d", c_int), ("groups", c_int),
                ("m", c_int), ("eps", c_float), ("dtype", c_int)]


class HeadRopeSeg(ctypes.Structure):  # mirrors b200_head_rope_seg
    _fields_ = [("inp", c_void_p), ("out", c_void_p), ("norm_w", c_void_p), ("freq", c_void_p), ("out_rows", c_void_p), ("ld_in", c_int64),
                ("ld_out", c_int64), ("heads", c_int), ("dim", c_int), ("in_stride", c_int), ("out_stride", c_int), ("rot_off", c_int),
                ("rot_dims", c_int), ("interleaved", c_int), ("mag", c_float)]


class TalkAttnArgs(ctypes.Structure):  # mirrors b200_talk_attn_args
    _fields_ = [("q", c_void_p), ("ldq", c_int64), ("k_cache", c_void_p), ("ldk", c_int64), ("v_cache", c_void_p), ("ldv", c_int64),
                ("talk", c_void_p), ("sink", c_void_p), ("out", c_void_p), ("ldo", c_int64), ("seqs", c_void_p), ("n_seqs", c_int),
                ("max_q_len", c_int), ("rows", c_int64), ("n_head", c_int), ("n_kv_head", c_int), ("dk", c_int), ("dv", c_int), ("max_seq", c_int),
                ("n_split", c_int), ("scale", c_float), ("dtype", c_int), ("workspace", c_void_p), ("workspace_bytes", c_size_t)]


class SandwichArgs(ctypes.Structure):  # mirrors b200_sandwich_args
    _fields_ = [("y0", c_void_p), ("w0", c_void_p), ("y1", c_void_p), ("w1", c_void_p), ("post_w", c_void_p), ("extra", c_void_p),
                ("pre_w", c_void_p), ("x", c_void_p), ("act", c_void_p), ("rows", c_int64), ("d", c_int), ("eps", c_float), ("dtype", c_int)]


class ConvGroup(ctypes.Structure):  # mirrors b200_conv_group
    _fields_ = [("w", c_void_p), ("out", c_void_p), ("ld_out", c_int64), ("inv_freq", c_void_p), ("col0", c_int), ("heads", c_int), ("dim", c_int),
                ("act", c_int), ("post", c_int), ("rot_dims", c_int), ("out_f32", c_int), ("rot_mscale", c_float), ("post_scale", c_float),
                ("eps", c_float)]


class DeltaRuleArgs(ctypes.Structure):  # mirrors b200_delta_rule_args
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("ldq", c_int64), ("ldk", c_int64), ("ldv", c_int64),
                ("beta_in", c_void_p), ("ld_beta", c_int64), ("decay_in", c_void_p), ("ld_decay", c_int64), ("a_log", c_void_p),
                ("dt_bias", c_void_p), ("state", c_void_p), ("state_slot_stride", c_int64), ("out", c_void_p), ("ldo", c_int64),
                ("seqs", c_void_p), ("n_seqs", c_int), ("heads", c_int), ("kv_heads", c_int), ("dk", c_int), ("dv", c_int),
                ("channel_decay", c_int), ("dtype", c_int), ("max_rows", c_int)]


class WindowAttnArgs(ctypes.Structure):  # mirrors b200_window_attn_args
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p), ("ldq", c_int64), ("ldk", c_int64), ("ldv", c_int64),
                ("ldo", c_int64), ("k_ring", c_void_p), ("v_ring", c_void_p), ("sink", c_void_p), ("seqs", c_void_p), ("n_seqs", c_int),
                ("max_q_len", c_int), ("ring", c_int), ("n_head", c_int), ("n_kv_head", c_int), ("dk", c_int), ("dv", c_int), ("window", c_int),
                ("scale", c_float), ("dtype", c_int), ("row_seq", c_void_p), ("rows", c_int64), ("dist_r1", c_void_p), ("dist_r2", c_void_p),
                ("gate", c_void_p), ("ldg", c_int64), ("gate_mode", c_int)]


class ScaledResidualArgs(ctypes.Structure):  # mirrors b200_scaled_residual_args
    _fields_ = [("y0", c_void_p), ("s0", c_void_p), ("y1", c_void_p), ("y2", c_void_p), ("s1", c_void_p), ("extra", c_void_p), ("row_add", c_void_p),
                ("x", c_void_p), ("cast", c_void_p), ("alpha", c_void_p), ("nw", c_void_p), ("nb", c_void_p), ("act", c_void_p), ("rows", c_int64),
                ("d", c_int), ("dtype", c_int)]


ROUTE_SOFTMAX, ROUTE_GROUP_MAX, ROUTE_TOPK_SOFTMAX, ROUTE_BIAS = 1, 2, 4, 8
ACT_GELU, ACT_GELU_TANH, ACT_SILU, ACT_RELU2 = 0, 1, 2, 3

# Entry points of the sources every model needs (library state, norms, sampling) and of the fp32-residual / latent-attention /
# expert kernels: `load_core()` can serve them from a library built from those sources alone.
_CORE_SOURCES = ("api.cu", "norm.cu", "sample.cu", "resid.cu", "latent.cu", "moe.cu", "attn_prefill.cu", "shortconv.cu", "delta.cu", "window_attn.cu",
                 "depth.cu", "rope.cu", "talk_attn.cu")
_CORE_SIGNATURES = {
    "b200_embed_pos": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_rms_rows": (c_int, [ctypes.POINTER(RmsRowsSeg), c_int, c_int64, c_float, c_int, c_int, c_void_p]),
    "b200_residual_norm_add": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "b200_gather_rows": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "b200_sqrelu": (c_int, [c_void_p, c_int64, c_int, c_void_p]),
    "b200_scale_f32": (c_int, [c_void_p, c_float, c_void_p, c_int64, c_int, c_void_p]),
    "b200_latent_prefill": (c_int, [ctypes.POINTER(LatentPrefillArgs), c_void_p]),
    "b200_attn_prefill_ragged": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_int,
                                         c_float, c_void_p]),
    "b200_attn_prefill_shared": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int, c_int,
                                         c_void_p, c_int64, c_int, c_int, c_float, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200_latent_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200_latent_decode": (c_int, [ctypes.POINTER(LatentDecodeArgs), c_void_p]),
    "b200_latent_decode_tune": (c_int, [c_int]),
    "b200_moe_route": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_moe_plan": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_moe_gemm": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                              c_void_p]),
    "b200_moe_gemv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_float, c_float,
                              c_int, c_void_p]),
    "b200_moe_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_sandwich_residual": (c_int, [ctypes.POINTER(SandwichArgs), c_void_p]),
    "b200_activation": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p]),
    "b200_glu": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_xielu": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p]),
    "b200_glu_clamped": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_float, c_float, c_int, c_void_p]),
    "b200_scaled_residual": (c_int, [ctypes.POINTER(ScaledResidualArgs), c_void_p]),
    "b200_short_conv": (c_int, [c_void_p, c_int64, ctypes.POINTER(ConvGroup), c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int,
                                c_void_p]),
    "b200_conv_tail_update": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_int, c_void_p]),
    "b200_delta_rule_state_floats": (c_int64, [c_int, c_int]),
    "b200_delta_rule": (c_int, [ctypes.POINTER(DeltaRuleArgs), c_void_p]),
    "b200_gated_rms_heads": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_float, c_int,
                                     c_void_p]),
    "b200_window_attn": (c_int, [ctypes.POINTER(WindowAttnArgs), c_void_p]),
    "b200_window_attn_tune": (c_int, [c_int]),
    "b200_depth_residual": (c_int, [ctypes.POINTER(DepthResidualArgs), c_void_p]),
    "b200_head_rope": (c_int, [ctypes.POINTER(HeadRopeSeg), c_int, c_void_p, c_int64, c_float, c_int, c_void_p]),
    "b200_attn_prefill_mixed_plane_floats": (c_size_t, [c_int, c_int, c_int64]),
    "b200_attn_prefill_mixed": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_int64, c_int, c_int, c_int, c_float, c_void_p, c_int64, c_void_p]),
    "b200_talk_attn_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int]),
    "b200_talk_attn": (c_int, [ctypes.POINTER(TalkAttnArgs), c_void_p]),
    "b200_attn_prefill_window": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_int,
                                         c_int, c_float, c_int, c_void_p, c_void_p]),
    "b200_attn_prefill_window_ex": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_int,
                                            c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200_ring_store": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int64, c_int,
                                c_void_p]),
}
_CORE_SHARED = ("b200_abi_version", "b200_last_error", "b200_device_info", "b200_set_pdl", "b200_launch_count", "b200_rmsnorm", "b200_swiglu",
                "b200_embedding", "b200_argmax", "b200_sample", "b200_attn_prefill")

_SIGNATURES = {
    "b200_abi_version": (c_int, []),
    "b200_last_error": (c_char_p, []),
    "b200_device_info": (c_int, [ctypes.POINTER(c_int)] * 3),
    "b200_set_pdl": (c_int, [c_int]),
    "b200_launch_count": (c_int64, []),
    "b200_qgemv_tune": (c_int, [c_int, c_int, c_int]),
    "b200_quantize_4bit": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_dequantize_4bit": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p]),
    "b200_double_quant_absmax": (c_int, [c_void_p, c_int64, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_p2p_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "b200_p2p_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "b200_p2p_close": (c_int, [c_void_p]),
    "b200_p2p_free": (c_int, [c_void_p]),
    "b200_quantize_int8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "b200_dequantize_int8": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "b200_linear_int8_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "b200_linear_int8": (c_int, [ctypes.POINTER(LinearInt8Args), c_void_p]),
    "b200_quantize_int4": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200_dequantize_int4": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_int, c_void_p]),
    "b200_qgemv_workspace_bytes": (c_size_t, []),
    "b200_qgemv": (c_int, [ctypes.POINTER(QGemvArgs), c_void_p]),
    "b200_tiled_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "b200_tile_4bit": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200_untile_4bit": (c_int, [c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_qgemv_tiled": (c_int, [ctypes.POINTER(QGemvTiledArgs), c_void_p]),
    "b200_qgemv_tiled_workspace_bytes": (c_size_t, []),
    "b200_qgemv_tiled_tune": (c_int, [c_int, c_int, c_int]),
    "b200_qgemv_tiled_trace": (c_int, [c_void_p, c_int]),
    "b200_qgemv_tiled_supported": (c_int, [ctypes.POINTER(QGemvTiledArgs)]),
    "b200_qgemv_tiled_error": (c_int, [c_void_p, c_void_p, ctypes.POINTER(ctypes.c_uint)]),
    "b200_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "b200_attn_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200_attn_decode": (c_int, [ctypes.POINTER(AttnDecodeArgs), c_void_p]),
    "b200_attn_decode_tune": (c_int, [c_int]),
    "b200_attn_decode_noalloc": (c_int, [ctypes.POINTER(AttnDecodeArgs), c_void_p]),
    "b200_attn_decode_noalloc_max_bytes": (c_size_t, []),
    "b200_rope_kv_append": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_attn_prefill": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_float, c_void_p]),
    "b200_tp_gather": (c_int, [ctypes.POINTER(TpHandoff), c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "b200_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "b200_embedding": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "b200_argmax": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int64, c_void_p]),
    "b200_sample": (c_int, [c_void_p, c_int, c_int64, c_float, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int64,
                            c_void_p]),
    "b200_qgemm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "b200_qgemm": (c_int, [ctypes.POINTER(QGemmArgs), c_void_p]),
    "b200_qgemm_tune": (c_int, [c_int]),
}

_SIGNATURES.update(_CORE_SIGNATURES)

_lib = None
_core = None
CORE_LIB_PATH = os.path.join(_PKG, "lib", "libb200gpt_core.so")


class B200Error(RuntimeError):
    pass


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load libb200gpt.so (building it in-tree with nvcc when absent).  Raises if neither is possible."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise B200Error(f"{LIB_PATH} is missing: run `python -m lit_gpt_b200.build`")
        from .build import build_library

        build_library()
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch, which must be loud
        fn.restype = res
        fn.argtypes = args
    if lib.b200_abi_version() != 1:
        raise B200Error(f"libb200gpt ABI version {lib.b200_abi_version()} != 1")
    _lib = lib
    return lib


def _bind(lib: ctypes.CDLL, names) -> ctypes.CDLL:
    for name in names:
        res, args = _SIGNATURES[name]
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.b200_abi_version() != 1:
        raise B200Error(f"libb200gpt ABI version {lib.b200_abi_version()} != 1")
    return lib


def load_core() -> ctypes.CDLL:
    """The library for models that need none of the quantized-weight kernels: the full library when it is already loaded or
    built and current, else ``libb200gpt_core.so``, built in-tree from ``_CORE_SOURCES`` alone (seconds instead of the minute
    the GEMV / GEMM sources take)."""
    global _core
    if _core is not None:
        return _core
    from .build import build_library, library_is_current

    if _lib is not None or library_is_current():
        _core = load()
        return _core
    path = build_library(sources_subset=_CORE_SOURCES, out=CORE_LIB_PATH)
    _core = _bind(ctypes.CDLL(path), list(_CORE_SIGNATURES) + list(_CORE_SHARED))
    return _core


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = (_lib or _core or load()).b200_last_error().decode(errors="replace")
        if rc == 3:
            raise NotImplementedError(f"{what}: {msg}")
        raise B200Error(f"{what} failed (code {rc}): {msg}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device | None = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise B200Error("b200gpt kernels run on CUDA tensors only; there is no CPU fallback")
