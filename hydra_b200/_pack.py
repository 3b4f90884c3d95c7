"""Weight preparation shared by the attention module and the whole-model executor: reference ``state_dict``
tensors -> the device layouts the kernels read (bf16 GEMM operands, repacked conv weights, interleaved
gate_up rows, fp32 norm gains / router vectors / RoPE tables), plus the ctypes structs that point at them."""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, List, Optional

import torch

from . import _lib

Tensor = torch.Tensor


def rope_tables(max_seq_len: int, head_dim: int, device, theta: float = 10000.0):
    """fp32 cos/sin [max_seq_len, head_dim/2], computed exactly as the reference builds its cache
    (hydra/attention/backends/ccgqa/attention.py:160-185): on the CPU in fp32, then moved."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    ang = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), inv)
    return ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous()


def _bf16(t: Tensor, device) -> Tensor:
    return t.detach().to(device=device, dtype=torch.bfloat16).contiguous()


def _f32(t: Tensor, device) -> Tensor:
    return t.detach().to(device=device, dtype=torch.float32).contiguous()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def repack_conv(w: Tensor, device) -> Tensor:
    """Conv1d weight [C_out, C_in/groups, K] -> bf16 [C_out, K*C_in/groups], (co, j*cin+ci) = w[co, ci, j]."""
    src = _bf16(w, device)
    co, ci, ks = src.shape
    if not 1 <= ks <= 8:
        raise NotImplementedError(f"conv kernel size {ks}: the pre-attention kernels are built for kernel sizes 1 to 8")
    out = torch.empty((co, ks * ci), dtype=torch.bfloat16, device=device)
    _lib.check(_lib.lib().hb200_repack_conv_weight_k(src.data_ptr(), out.data_ptr(), co, ci, ks, _stream(device)),
               "repack_conv_weight")
    return out


def interleave_gate_up(w: Tensor, device) -> Tensor:
    """gate_up.weight [2F, D] -> bf16 rows interleaved in groups of 8 (8 gate rows, 8 up rows, ...)."""
    src = _bf16(w, device)
    F2, K = src.shape
    out = torch.empty_like(src)
    _lib.check(_lib.lib().hb200_interleave_gate_up(src.data_ptr(), out.data_ptr(), F2 // 2, K, _stream(device)),
               "interleave_gate_up")
    return out


class PackedBlock:
    """Device tensors of one HydraMoRBlock (kept alive here) and the matching C struct."""

    def __init__(self, sd: Dict[str, Tensor], pre: str, device, *, attention_only: bool = False, plain: bool = False,
                 head_dim: Optional[int] = None, fold_norm: bool = False):
        """plain: a HydraBlock (blocks.py:33-70) - attention and one MLP pass, no routers, no recursion offsets, no exit
        norm; expressed as a one-recursion block with a zero offset."""
        a = pre if attention_only else pre + "attention."
        t: Dict[str, Optional[Tensor]] = {}
        t["w_qkv"] = _bf16(sd[a + "qkv_proj.weight"], device)
        t["w_o"] = _bf16(sd[a + "o_proj.weight"], device)
        if a + "q_conv.conv1.weight" in sd:
            t["w1_qk"] = torch.cat([repack_conv(sd[a + "q_conv.conv1.weight"], device),
                                    repack_conv(sd[a + "k_conv.conv1.weight"], device)], dim=0).contiguous()
            t["w2_q"] = repack_conv(sd[a + "q_conv.conv2.weight"], device)
            t["w2_k"] = repack_conv(sd[a + "k_conv.conv2.weight"], device)
            self.conv_ksize = int(sd[a + "q_conv.conv1.weight"].shape[-1])
        else:                                   # a module built with use_convs=False has no conv parameters
            if head_dim is None:
                raise KeyError(f"{a}q_conv.conv1.weight is missing (a module without convolutions must state its head_dim)")
            t["w1_qk"] = t["w2_q"] = t["w2_k"] = None
            self.conv_ksize = 3
        t["key_temperature"] = _f32(sd[a + "key_temperature"], device).reshape(1)
        for k in ("norm1_w", "norm2_w", "final_norm_w", "w_gate_up", "w_down", "mor_w", "mor_b", "rec",
                  "mod_wn", "mod_b"):
            t[k] = None
        if not attention_only:
            t["norm1_w"] = _f32(sd[pre + "norm1.weight"], device)
            t["norm2_w"] = _f32(sd[pre + "norm2.weight"], device)
            t["w_gate_up"] = interleave_gate_up(sd[pre + "mlp.gate_up.weight"], device)
            t["w_down"] = _bf16(sd[pre + "mlp.down.weight"], device)
        if plain:
            t["rec"] = torch.zeros((1, t["norm1_w"].numel()), dtype=torch.float32, device=device)
        elif not attention_only:
            t["final_norm_w"] = _f32(sd[pre + "final_norm.weight"], device)
            t["mor_w"] = _f32(sd[pre + "mor_router.router.weight"], device).reshape(-1)
            t["mor_b"] = _f32(sd[pre + "mor_router.router.bias"], device).reshape(1)
            rb = sd[pre + "mor_executor.recursion_bias"]
            re = sd[pre + "mor_executor.recursion_embed.weight"]
            # the reference adds bias then embedding to the hidden state in its dtype; one fp32 vector here
            t["rec"] = (_f32(rb, device).reshape(re.shape[0], -1) + _f32(re, device)).contiguous()
            mk = pre + "mod_mlp_wrapper.mod_router.router."
            if mk + "weight" in sd:
                # Linear(norm(x)) = rsqrt(..) * sum x_d * (gain_d * w_d): fold the norm gain into the router weight
                t["mod_wn"] = (_f32(sd[mk + "weight"], device).reshape(-1) * t["norm2_w"]).contiguous()
                t["mod_b"] = _f32(sd[mk + "bias"], device).reshape(1)
        # optional: the pre-MLP norm folded into the first MLP contraction: norm(x + rec; g) W^T = inv_rms * (x W'^T +
        # rec W'^T) with W' = W diag(g) (rounded to bf16 once, here) and the per-recursion bias rec W'^T in fp32.  With
        # these the executor contracts the routed rows of the hidden state directly instead of a normalised copy.
        t["w_gate_up_n"] = t["gate_up_bias"] = None
        if fold_norm and not attention_only and t["rec"] is not None:
            wf = _f32(sd[pre + "mlp.gate_up.weight"], device) * t["norm2_w"][None, :]
            wn = wf.to(torch.bfloat16)
            F2 = wn.shape[0]
            orow = torch.arange(F2, device=device)
            grp, r16 = orow // 16, orow % 16
            srow = torch.where(r16 < 8, grp * 8 + r16, F2 // 2 + grp * 8 + (r16 - 8))     # interleaved row -> source row
            t["w_gate_up_n"] = interleave_gate_up(wn, device)
            t["gate_up_bias"] = (t["rec"] @ wn.float().T)[:, srow].contiguous()            # [R, 2F], interleaved order
            del wf, wn
        self.tensors = t
        # q is a unit vector and |k| = |key_temperature| after the fused pre-attention kernel (RoPE is a rotation), so
        # |q.k| / sqrt(hd) <= |temperature| / sqrt(hd); 2% slack covers the bf16 rounding of q and k
        hd = head_dim if head_dim is not None else sd[a + "q_conv.conv1.weight"].shape[1]
        temp = abs(float(sd[a + "key_temperature"].detach().float().reshape(-1)[0].item()))
        self.attn_logit_bound = max(temp, 1e-3) / math.sqrt(hd) * 1.02
        self.struct = _lib.BlockWeights(**{k: (v.data_ptr() if v is not None else None) for k, v in t.items()},
                                        attn_logit_bound=self.attn_logit_bound)


class PackedModel:
    """hb200_model struct + everything it points to."""

    def __init__(self, *, vocab: int, dim: int, n_rec: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 ffn_hidden: int, min_depth: int, adaptive: bool, max_seq_len: int, mod_capacity: float,
                 norm_eps: float, residual_scale: float, output_scale: float, blocks: List[PackedBlock],
                 tok_emb: Optional[Tensor], norm_w: Optional[Tensor], device, gemm_impl: int = 0,
                 lm_head: Optional[Tensor] = None, static_routing: bool = False, mor_rampup: float = 0.0,
                 attn_disable: int = 0):
        self.blocks = blocks
        self.block_array = (_lib.BlockWeights * len(blocks))(*[b.struct for b in blocks])
        self.cos, self.sin = rope_tables(max_seq_len, head_dim, device)
        self.tok_emb, self.norm_w, self.lm_head = tok_emb, norm_w, lm_head
        self.out_proj = lm_head if lm_head is not None else tok_emb      # weight of the output projection
        self.struct = _lib.Model(
            vocab=vocab, dim=dim, n_blocks=len(blocks), n_rec=n_rec, n_heads=n_heads, n_kv_heads=n_kv_heads,
            head_dim=head_dim, ffn_hidden=ffn_hidden, min_depth=min_depth, adaptive=int(adaptive),
            max_seq_len=max_seq_len, gemm_impl=gemm_impl, mod_capacity=mod_capacity, norm_eps=norm_eps,
            residual_scale=residual_scale, output_scale=output_scale,
            tok_emb=tok_emb.data_ptr() if tok_emb is not None else None,
            norm_w=norm_w.data_ptr() if norm_w is not None else None,
            rope_cos=self.cos.data_ptr(), rope_sin=self.sin.data_ptr(),
            blocks=C.cast(self.block_array, C.POINTER(_lib.BlockWeights)),
            lm_head=lm_head.data_ptr() if lm_head is not None else None, static_routing=int(bool(static_routing)),
            mor_rampup=float(mor_rampup), attn_disable=int(attn_disable),
            conv_ksize=blocks[0].conv_ksize if blocks else 3)
        if any(b.conv_ksize != blocks[0].conv_ksize for b in blocks):
            raise ValueError("blocks with different conv kernel sizes")
        self._ws: Dict[tuple, Tensor] = {}
        self.device = device
        self.err_flag = torch.zeros(1, dtype=torch.int32, device=device)

    def resize_rope(self, max_seq_len: int) -> None:
        """Grow the RoPE tables (never shrinks them); the old tables stay alive until the stream has drained."""
        if max_seq_len <= self.struct.max_seq_len:
            return
        torch.cuda.current_stream(self.device).synchronize()
        self.cos, self.sin = rope_tables(max_seq_len, self.struct.head_dim, self.device)
        self.struct.rope_cos, self.struct.rope_sin = self.cos.data_ptr(), self.sin.data_ptr()
        self.struct.max_seq_len = max_seq_len

    def workspace(self, B: int, S: int) -> Tensor:
        """A workspace of at least hb200_model_workspace_bytes(B, S); one buffer is kept and grown on demand, so a
        generation loop whose sequence grows by one token per step does not reallocate every step."""
        n = _lib.lib().hb200_model_workspace_bytes(C.byref(self.struct), B, S)
        ws = self._ws.get("buf")
        if ws is None or ws.numel() < n:
            self._ws.clear()
            ws = torch.empty(n, dtype=torch.uint8, device=self.device)
            self._ws["buf"] = ws
        return ws

    def reserve(self, B: int, S: int) -> None:
        """Allocate the workspace for the largest [B, S] that will be run."""
        self.workspace(B, S)

    def check_device_errors(self) -> None:
        """Synchronises and raises if a bounded in-kernel wait ran out during an earlier call."""
        if int(self.err_flag.item()) != 0:
            self.err_flag.zero_()
            raise _lib.Hb200Error("a bounded wait inside a GEMM kernel ran out (status HB200_ERR_DEVICE_WAIT); "
                                  "the results of that call are undefined")
