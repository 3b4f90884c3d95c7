"""CCGQAAttention module, drop-in for the reference's (hydra/attention/backends/ccgqa/attention.py:67-331).

Same constructor arguments, attributes, parameter names (``qkv_proj.weight``, ``o_proj.weight``,
``q_conv.conv{1,2}.weight``, ``k_conv.conv{1,2}.weight``, ``key_temperature``), non-persistent RoPE buffers
(``cos_cached`` / ``sin_cached``) and helper methods (``_init_rope``, ``_apply_rope``), so a reference
``state_dict`` loads unchanged and ``HydraMoRBlock`` can hold it.  ``forward`` runs four launches of the CUDA
extension: qkv GEMM (tcgen05), fused pre-attention kernel, causal GQA attention, output GEMM (tcgen05).

Arithmetic: bf16 storage, fp32 accumulation; an fp32/fp16 input is converted to bf16 and the result converted
back.  CUDA only.  Inference only (no autograd through the kernels).  ``forward(x, mask)`` with a padding mask
([B, S], 1 = valid) runs a CUDA-core attention kernel and by default computes what the reference computes there (see
``mask_semantics``).  The ``use_*`` ablation switches are honoured (a stage that is off selects a CUDA-core kernel);
so does a ``conv_kernel_size`` other than 3; sizes above 8 raise NotImplementedError.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.nn as nn

from .. import _lib, kernels
from .._pack import PackedBlock, PackedModel


class ConvSequence(nn.Module):
    """Parameter holder with the layout of the reference's OptimizedConvSequence
    (hydra/attention/backends/ccgqa/kernels/fused_conv.py:16-37): a grouped k=3 Conv1d then a dense k=3 Conv1d,
    both without bias.  The convolutions themselves run inside the fused pre-attention kernel."""

    def __init__(self, channels: int, groups1: int, groups2: int, kernel_size: int = 3):
        super().__init__()
        self.channels = channels
        self.kernel_size = kernel_size
        self.conv1 = nn.Conv1d(channels, channels, kernel_size=kernel_size, padding=0, groups=groups1, bias=False)
        self.conv2 = nn.Conv1d(channels, channels, kernel_size=kernel_size, padding=0, groups=groups2, bias=False)


class CCGQAAttention(nn.Module):
    def __init__(self, dim: int, n_heads: int = 16, n_kv_heads: int = 4, compression_factor: int = 4,
                 max_seq_len: int = 8192, use_rope: bool = True, use_qk_norm: bool = True, use_convs: bool = True,
                 use_qk_mean: bool = True, use_value_shift: bool = True, conv_kernel_size: int = 3,
                 use_fused_kernel: bool = True):
        super().__init__()
        self.dim = dim
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads
        self.n_groups = n_heads // n_kv_heads
        self.compression_factor = compression_factor
        self.use_rope, self.use_qk_norm, self.use_convs = use_rope, use_qk_norm, use_convs
        self.use_qk_mean, self.use_value_shift = use_qk_mean, use_value_shift
        self.use_fused_kernel = use_fused_kernel
        self.latent_dim = dim // compression_factor
        self.head_dim = self.latent_dim // n_heads
        self.kv_dim = n_kv_heads * self.head_dim
        assert self.latent_dim % n_heads == 0, f"latent_dim {self.latent_dim} must be divisible by n_heads {n_heads}"
        assert self.head_dim % 2 == 0, f"head_dim {self.head_dim} must be even for RoPE (splits into pairs)"
        if use_convs and not 1 <= conv_kernel_size <= 8:
            raise NotImplementedError("hydra_b200 CCGQAAttention implements conv kernel sizes 1 to 8")
        # the reference's ablation switches: a stage that is off selects the CUDA-core pre-attention kernel
        self._attn_disable = ((0 if use_rope else _lib.ATTN_NO_ROPE) | (0 if use_qk_norm else _lib.ATTN_NO_QK_NORM) |
                              (0 if use_convs else _lib.ATTN_NO_CONVS) | (0 if use_qk_mean else _lib.ATTN_NO_QK_MEAN) |
                              (0 if use_value_shift else _lib.ATTN_NO_VALUE_SHIFT))
        self.qkv_proj = nn.Linear(dim, self.latent_dim + 2 * self.kv_dim, bias=False)
        self.o_proj = nn.Linear(self.latent_dim, dim, bias=False)
        self.output_scale = float(os.environ.get("HYDRA_CCGQA_OUTPUT_SCALE", "1.0"))
        if use_convs:                            # as in the reference, a module without convolutions has no conv parameters
            self.q_conv = ConvSequence(self.latent_dim, n_heads, 1, conv_kernel_size)
            self.k_conv = ConvSequence(self.kv_dim, n_kv_heads, 1, conv_kernel_size)
        self.key_temperature = nn.Parameter(torch.full((1,), float(self.head_dim ** 0.5)))
        self._init_rope(max_seq_len)
        self.scale = self.head_dim ** -0.5
        self.max_seq_len = max_seq_len
        # forward(x, mask): "reference" = what the reference module computes when it is handed a padding mask - its boolean
        # mask is True for future and padded keys (attention.py:269-283) and SDPA lets True keys take part, so a query
        # uses the keys after it and the padded ones; "intended" = causal over the valid keys, as its comments describe
        self.mask_semantics = os.environ.get("HYDRA_B200_MASK_SEMANTICS", "reference").strip().lower()
        self._packed: Optional[PackedModel] = None
        self._packed_key = None

    # -- RoPE cache, same construction as attention.py:160-185 ------------------------------------------------
    def _init_rope(self, max_seq_len: int) -> None:
        hd = self.head_dim
        freqs = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
        ang = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), freqs)
        mode = os.environ.get("HYDRA_ROPE_CACHE_DTYPE", "").strip().lower()
        dt = torch.bfloat16 if mode in {"bf16", "bfloat16"} else (
            torch.float16 if mode in {"fp16", "float16", "half"} else torch.float32)
        self.register_buffer("cos_cached", ang.cos().to(dt)[None, None], persistent=False)
        self.register_buffer("sin_cached", ang.sin().to(dt)[None, None], persistent=False)
        self._packed = None

    def _apply_rope(self, x: torch.Tensor, seq_len: int) -> torch.Tensor:
        """x [B, heads, S, head_dim] -> rotated (attention.py:187-199), through the fused RoPE kernel."""
        return kernels.fused_rope(x, self.cos_cached[:, :, :seq_len, :], self.sin_cached[:, :, :seq_len, :])

    # -- device-side weights -----------------------------------------------------------------------------------
    def _pack(self, device: torch.device) -> PackedModel:
        key = (device, self.cos_cached.shape[2]) + tuple((p.data_ptr(), p._version) for p in self.parameters())
        if self._packed is None or self._packed_key != key:
            sd = {k: v for k, v in self.state_dict().items()}
            blk = PackedBlock(sd, "", device, attention_only=True, head_dim=self.head_dim)
            self._packed = PackedModel(
                vocab=8, dim=self.dim, n_rec=1, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                head_dim=self.head_dim, ffn_hidden=8, min_depth=0, adaptive=False,
                max_seq_len=self.cos_cached.shape[2], mod_capacity=1.0, norm_eps=1e-6, residual_scale=1.0,
                output_scale=self.output_scale, blocks=[blk], tok_emb=None, norm_w=None, device=device,
                attn_disable=self._attn_disable)
            self._packed_key = key
        return self._packed

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        """Accept the reference's older checkpoint layouts (attention.py:333-383): separate ``q_down`` / ``k_down`` /
        ``v_down`` (/ ``v_shift_down``) projections are concatenated into ``qkv_proj``; flat ``q_conv1`` ...
        ``k_conv2`` become ``q_conv.conv1`` ... ``k_conv.conv2``."""
        for stem in ("q", "k"):
            for n in ("1", "2"):
                for suffix in ("weight", "bias"):
                    old, new = f"{prefix}{stem}_conv{n}.{suffix}", f"{prefix}{stem}_conv.conv{n}.{suffix}"
                    if old in state_dict:
                        val = state_dict.pop(old)
                        if suffix == "weight" and new not in state_dict:
                            state_dict[new] = val
        q_key, qkv_key = prefix + "q_down.weight", prefix + "qkv_proj.weight"
        if q_key in state_dict and qkv_key not in state_dict:
            parts = [state_dict.pop(q_key), state_dict.pop(prefix + "k_down.weight"),
                     state_dict.pop(prefix + "v_down.weight")]
            vs = prefix + "v_shift_down.weight"
            if vs in state_dict:
                parts.append(state_dict.pop(vs))
            state_dict[qkv_key] = torch.cat(parts, dim=0)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if torch.is_grad_enabled() and x.requires_grad:
            # the kernels are forward-only and the result carries no grad_fn: a training step through this module would
            # silently get zero gradient for everything upstream of it
            raise RuntimeError("hydra_b200 CCGQAAttention is inference only (no autograd through its kernels): wrap the "
                               "call in torch.no_grad(), or uninstall() before training")
        if not x.is_cuda:
            raise RuntimeError("hydra_b200 CCGQAAttention runs on CUDA tensors only (there is no CPU fallback)")
        B, S, D = x.shape
        if D != self.dim:
            raise ValueError(f"expected last dim {self.dim}, got {D}")
        pm = self._pack(x.device)
        xb = x.detach().to(torch.bfloat16).contiguous()
        y = torch.empty_like(xb)
        if B * S == 0:
            return y.to(x.dtype)
        ws = pm.workspace(B, S)
        if mask is not None:
            # mask [B, S], 1 = valid token, 0 = padding (attention.py:269-283); see ``mask_semantics``
            if tuple(mask.shape) != (B, S):
                raise ValueError(f"mask must be [batch, seq_len] = {(B, S)}, got {tuple(mask.shape)}")
            modes = {"reference": _lib.MASK_AS_REFERENCE, "intended": _lib.MASK_INTENDED}
            if self.mask_semantics not in modes:
                raise ValueError(f"mask_semantics must be 'reference' or 'intended', got {self.mask_semantics!r}")
            valid = (mask.to(x.device) != 0).to(torch.uint8).contiguous()
            with kernels._on(x.device):
                _lib.check(_lib.lib().hb200_ccgqa_forward_masked(
                    C.byref(pm.struct), 0, xb.data_ptr(), y.data_ptr(), valid.data_ptr(), modes[self.mask_semantics], B, S,
                    ws.data_ptr(), ws.numel(), pm.err_flag.data_ptr(), kernels._stream(x.device)), "ccgqa_forward_masked")
            return y if x.dtype == torch.bfloat16 else y.to(x.dtype)
        with kernels._on(x.device):
            _lib.check(_lib.lib().hb200_ccgqa_forward(C.byref(pm.struct), 0, xb.data_ptr(), y.data_ptr(), B, S,
                                                      ws.data_ptr(), ws.numel(), pm.err_flag.data_ptr(),
                                                      kernels._stream(x.device)), "ccgqa_forward")
        return y if x.dtype == torch.bfloat16 else y.to(x.dtype)
