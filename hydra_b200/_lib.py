"""ctypes binding of the C ABI declared in ``include/hydra_b200.h``.

The shared library is the product: there is no Python or CPU fallback behind these calls.  If the library is
missing it is built once with nvcc (``hydra_b200.build``); if that is impossible the import of any op fails
with an error that says so.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

from . import build as _build

c_i32, c_i64, c_f32, c_vp, c_sz = C.c_int, C.c_int64, C.c_float, C.c_void_p, C.c_size_t

HB200_F32, HB200_BF16, HB200_F16 = 0, 1, 2
ATTN_NO_ROPE, ATTN_NO_QK_NORM, ATTN_NO_CONVS, ATTN_NO_QK_MEAN, ATTN_NO_VALUE_SHIFT = 1, 2, 4, 8, 16   # hb200_model.attn_disable
MASK_AS_REFERENCE, MASK_INTENDED = 0, 1        # hb200_attention_masked_gqa / hb200_ccgqa_forward_masked mask modes
EPI_STORE, EPI_RESID, EPI_SWIGLU, EPI_SCATTER_ADD = 0, 1, 2, 3


class BlockWeights(C.Structure):
    _fields_ = [(n, c_vp) for n in (
        "norm1_w", "norm2_w", "final_norm_w", "w_qkv", "w_o", "w1_qk", "w2_q", "w2_k", "key_temperature",
        "w_gate_up", "w_down", "mor_w", "mor_b", "rec", "mod_wn", "mod_b")] + [("attn_logit_bound", c_f32),
                                                                               ("w_gate_up_n", c_vp), ("gate_up_bias", c_vp)]


class Model(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "vocab", "dim", "n_blocks", "n_rec", "n_heads", "n_kv_heads", "head_dim", "ffn_hidden",
        "min_depth", "adaptive", "max_seq_len", "gemm_impl")] + [
        (n, c_f32) for n in ("mod_capacity", "norm_eps", "residual_scale", "output_scale")] + [
        ("tok_emb", c_vp), ("norm_w", c_vp), ("rope_cos", c_vp), ("rope_sin", c_vp),
        ("blocks", C.POINTER(BlockWeights)), ("profile", c_vp), ("lm_head", c_vp), ("static_routing", C.c_int32), ("mor_rampup", c_f32),
        ("attn_disable", C.c_int32), ("conv_ksize", C.c_int32)]


class LaunchRecord(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("kind", "block", "rec", "m", "n", "k")]


KERNEL_KINDS = ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "gemm_lm_head", "rms_norm", "pre_attention",
                "attention", "mor_score", "select", "norm_gather", "embed", "other")


class Taps(C.Structure):
    _fields_ = [("depths", c_vp), ("mod_idx", c_vp), ("mod_scores", c_vp), ("router_logits", c_vp),
                ("mlp_rows", c_vp), ("block_out", c_vp), ("force_routing", C.c_int32)]


class DecodeState(C.Structure):
    _fields_ = [("batch", C.c_int32), ("capacity", C.c_int32), ("kcache", c_vp), ("vcache", c_vp), ("halo", c_vp),
                ("vshift", c_vp), ("scores", c_vp), ("pos", c_vp), ("tokens", c_vp), ("history", c_vp)]


# name -> (restype, argtypes); mirrors include/hydra_b200.h one to one
SIGNATURES = {
    "hb200_version": (c_i32, []),
    "hb200_last_error": (C.c_char_p, []),
    "hb200_rms_norm": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i32, c_f32, c_i32, c_i32, c_vp]),
    "hb200_rope": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_i64, c_i64, c_i64, c_i32, c_i32, c_vp]),
    "hb200_qk_norm": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i32, c_f32, c_f32, c_i32, c_i32, c_vp]),
    "hb200_swiglu": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i32, c_i64, c_i64, c_i32, c_vp]),
    "hb200_gemm_bf16": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i64, c_i64, c_i64, c_i32, c_vp, c_f32,
                                c_vp, c_vp, c_i32, c_vp, c_vp]),
    "hb200_gemm_skinny_bf16": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i64, c_i64, c_i64, c_i32, c_vp, c_f32,
                                       c_vp, c_vp, c_vp, c_vp]),
    "hb200_interleave_gate_up": (c_i32, [c_vp, c_vp, c_i32, c_i32, c_vp]),
    "hb200_repack_conv_weight": (c_i32, [c_vp, c_vp, c_i32, c_i32, c_vp]),
    "hb200_ccgqa_pre_attention": (c_i32, [c_vp] * 10 + [c_i32] * 5 + [c_vp, c_vp]),
    "hb200_ccgqa_pre_attention_ablated": (c_i32, [c_vp] * 10 + [c_i32] * 7 + [c_vp, c_vp]),
    "hb200_repack_conv_weight_k": (c_i32, [c_vp, c_vp, c_i32, c_i32, c_i32, c_vp]),
    "hb200_attention_causal_gqa": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_f32, c_f32,
                                           c_vp, c_vp]),
    "hb200_mod_topk_select": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp]),
    "hb200_mor_depths": (c_i32, [c_vp, c_vp, c_i64, c_i32, c_i32, c_vp]),
    "hb200_argmax_rows": (c_i32, [c_vp, c_i64, c_i32, c_i64, c_vp, c_vp]),
    "hb200_cross_entropy_rows": (c_i32, [c_vp, c_vp, c_i64, c_i32, c_i64, c_i64, c_vp, c_vp]),
    "hb200_sample_rows": (c_i32, [c_vp, c_i64, c_i32, c_i64, c_f32, c_i32, c_f32, c_vp, c_vp, c_vp]),
    "hb200_embed": (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_f32, c_vp]),
    "hb200_model_workspace_bytes": (c_sz, [C.POINTER(Model), c_i32, c_i32]),
    "hb200_model_forward": (c_i32, [C.POINTER(Model), c_vp, c_i32, c_i32, c_vp, c_sz, c_vp, c_i64, c_vp,
                                    C.POINTER(Taps), c_vp, c_vp]),
    "hb200_block_forward": (c_i32, [C.POINTER(Model), c_i32, c_vp, c_vp, c_i32, c_i32, c_vp, c_sz,
                                    C.POINTER(Taps), c_vp, c_vp]),
    "hb200_ccgqa_forward": (c_i32, [C.POINTER(Model), c_i32, c_vp, c_vp, c_i32, c_i32, c_vp, c_sz, c_vp, c_vp]),
    "hb200_decode_workspace_bytes": (c_sz, [C.POINTER(Model), c_i32]),
    "hb200_model_prefill_cached": (c_i32, [C.POINTER(Model), c_vp, c_i32, c_i32, c_vp, c_sz, C.POINTER(DecodeState),
                                           c_vp, c_i64, c_vp, c_vp]),
    "hb200_model_decode_step": (c_i32, [C.POINTER(Model), C.POINTER(DecodeState), c_vp, c_sz, c_vp, c_i64, c_vp, c_vp]),
    "hb200_ccgqa_forward_masked": (c_i32, [C.POINTER(Model), c_i32, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_sz, c_vp,
                                           c_vp]),
    "hb200_attention_masked_gqa": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_f32,
                                           c_vp]),
    "hb200_ccgqa_forward_static_max_bytes": (c_sz, []),
    "hb200_ccgqa_forward_static": (c_i32, [C.POINTER(Model), c_i32, c_vp, c_vp, c_i32, c_i32, c_vp, c_vp]),
    "hb200_profile_create": (c_vp, [c_i32]),
    "hb200_profile_destroy": (None, [c_vp]),
    "hb200_profile_reset": (c_i32, [c_vp]),
    "hb200_profile_read": (c_i32, [c_vp, C.POINTER(LaunchRecord), C.POINTER(c_f32), c_i32]),
}

_lib = None
_lock = threading.Lock()


class Hb200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def lib() -> C.CDLL:
    """The loaded shared library (built on first use if it is missing or stale)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB_PATH
        if not os.path.exists(path) or (_build.is_stale() and os.environ.get("HB200_NO_REBUILD", "0") != "1"):
            try:
                _build.build()
            except Exception as e:  # pragma: no cover - depends on the toolchain of the host
                if not os.path.exists(path):
                    raise ImportError(
                        f"hydra_b200: the CUDA extension {path} is missing and could not be built ({e}). "
                        "There is no fallback path; run `python -m hydra_b200.build` on a machine with nvcc.") from e
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError here means header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = handle
        return _lib


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = lib().hb200_last_error()
        raise Hb200Error(f"{what or 'hb200 call'} failed with status {status}: {msg.decode() if msg else ''}")
