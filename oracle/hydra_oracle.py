"""CPU oracle for the HYDRA inference forward hot path.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared
against; it is never the thing that is shipped or measured as the product.  Only
the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import it.

It restates, in plain CPU PyTorch arithmetic (fp32 by default, fp64 on request),
the algorithm of the reference's eval-mode forward.  Every function cites the
reference file:line (paths relative to the reference project root) whose
behaviour it follows.  Parity of this restatement is PINNED: the fixtures under
``tests/golden/`` were produced by importing and running the reference itself
(``tests/golden/make_golden.py``), and ``tests/test_oracle_golden.py`` checks
every function here against them.

Third-party arithmetic on the path (PyTorch ATen, pinned by the reference only as
``torch>=2.0.0``): ``torch.topk`` tie order and SDPA summation order are not
pinned by any reference test; with fp32 scores ties do not occur in practice.

Parameters are passed as a flat dict that uses the reference's ``state_dict`` key
names (``layers.{i}.attention.qkv_proj.weight`` ...), so the same dict can be
loaded from a reference checkpoint.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

Tensor = torch.Tensor


# ----------------------------------------------------------------------------
# configuration
# ----------------------------------------------------------------------------
@dataclass
class HydraConfig:
    """Shape of a HydraModel (hydra/model/framework/model.py:180-215)."""

    vocab_size: int = 50257
    dim: int = 512
    n_mor_blocks: int = 2
    recursions_per_block: int = 2
    n_heads: int = 8
    n_kv_heads: int = 2
    compression_factor: int = 4
    mlp_ratio: float = 2.67
    max_seq_len: int = 512
    mod_capacity: float = 0.75
    mor_min_depth: int = 0
    adaptive: bool = True
    output_scale: float = 1.0        # HYDRA_CCGQA_OUTPUT_SCALE, attention.py:129-130
    residual_scale: float = 0.5      # blocks.py:491
    norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    hidden_dim: Optional[int] = None  # override of the MLP width (op-level tests)
    attn_off: tuple = ()             # attention stages switched off in every block (ATTENTION_STAGES): what blocks built as
                                     # HydraMoRBlock(..., use_convs=False, ...) compute (blocks.py:482-490 hands the use_*
                                     # kwargs to the attention factory; HydraModel itself forwards none of them)
    static_routing: bool = False     # static_routing_mode (model.py:202): dense compute with soft routing weights
    mor_rampup_scale: float = 1.0    # MoR curriculum (blocks.py:731-757): strictly between 0 and 1 the block returns
                                     # scale * adaptive + (1 - scale) * fixed-depth; <= 0 is the fixed-depth path

    @property
    def latent_dim(self) -> int:
        return self.dim // self.compression_factor

    @property
    def head_dim(self) -> int:
        return self.latent_dim // self.n_heads

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def ffn_hidden(self) -> int:
        # blocks.py:501-503: int(dim*ratio) rounded up to a multiple of 256
        if self.hidden_dim is not None:
            return self.hidden_dim
        h = int(self.dim * self.mlp_ratio)
        return ((h + 255) // 256) * 256

    def block_has_mod(self, i: int) -> bool:
        # model.py:283,296: MoD wraps the MLP only in interior blocks
        return (0 < i < self.n_mor_blocks - 1) and self.mod_capacity is not None and self.mod_capacity > 0


# ----------------------------------------------------------------------------
# exported fused-op semantics  (hydra/kernels/fused_ops.py)
# ----------------------------------------------------------------------------
def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """x * rsqrt(mean(x^2) + eps) * w   (fused_ops.py:1196-1205, layers/common.py:106-118)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * weight


def ada_rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """Unconditioned AdaRMSNorm (layers/common.py:153-160); same formula as rms_norm."""
    ms = x.pow(2).mean(dim=-1, keepdim=True)
    return (x * torch.rsqrt(ms + eps)) * weight


def rope_tables(seq_len: int, head_dim: int, theta: float = 10000.0) -> Tuple[Tensor, Tensor]:
    """fp32 cos/sin tables [S, hd/2]  (attention.py:160-185)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Interleaved-pair rotary embedding on x [B,H,S,hd]  (fused_ops.py:300-306,
    attention.py:194-199).  cos/sin: [S,hd/2] or [1,1,>=S,hd/2]."""
    S = x.shape[2]
    if cos.dim() == 4:
        cos, sin = cos[0, 0], sin[0, 0]
    cos = cos[:S].to(x.dtype)
    sin = sin[:S].to(x.dtype)
    xe, xo = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = xe * cos - xo * sin
    out[..., 1::2] = xe * sin + xo * cos
    return out


def l2_normalize(x: Tensor, eps: float = 1e-12) -> Tensor:
    """F.normalize(p=2, dim=-1): x / max(||x||, eps)  (attention.py:260-262)."""
    n = x.pow(2).sum(dim=-1, keepdim=True).sqrt().clamp_min(eps)
    return x / n


def qk_norm(q: Tensor, k: Tensor, scale: float, temperature: float = 1.0) -> Tuple[Tensor, Tensor]:
    """Exported fused_qk_norm semantics, PyTorch path (fused_ops.py:587-596)."""
    return l2_normalize(q) * scale, l2_normalize(k) * scale * temperature


def qk_norm_rsqrt(q: Tensor, k: Tensor, scale: float, temperature: float = 1.0) -> Tuple[Tensor, Tensor]:
    """Exported fused_qk_norm semantics, device-kernel formula x*rsqrt(sum x^2 + 1e-8)*scale
    (fused_ops.py:350-369)."""
    qn = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-8) * scale
    kn = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-8) * scale * temperature
    return qn, kn


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """silu(gate) * up  (fused_ops.py:881-883)."""
    return gate * torch.sigmoid(gate) * up


# ----------------------------------------------------------------------------
# CCGQA attention  (hydra/attention/backends/ccgqa/attention.py:201-331)
# ----------------------------------------------------------------------------
def causal_conv_k3(x: Tensor, w: Tensor, groups: int) -> Tensor:
    """One causal Conv1d (cross-correlation, left zero padding of K - 1, no bias); K = 3 in every model of the reference,
    other sizes through the module's ``conv_kernel_size``.

    x [B,S,C]; w [C, C/groups, K]   (kernels/fused_conv.py:22-37,48-57).
    y[t, c] = sum_j sum_{c' in group(c)} w[c, c', j] * x[t-(K-1)+j, c'],  x[<0] := 0.
    """
    B, S, C = x.shape
    K = w.shape[-1]
    cg = C // groups
    xp = torch.cat([x.new_zeros(B, K - 1, C), x], dim=1)       # [B, S+K-1, C]
    y = x.new_zeros(B, S, C)
    for g in range(groups):
        xs = xp[:, :, g * cg:(g + 1) * cg]                     # [B, S+K-1, cg]
        wg = w[g * cg:(g + 1) * cg]                            # [cg_out, cg_in, K]
        acc = 0
        for j in range(K):
            acc = acc + xs[:, j:j + S, :] @ wg[:, :, j].transpose(0, 1)
        y[:, :, g * cg:(g + 1) * cg] = acc
    return y


def conv_sequence(x: Tensor, w1: Tensor, w2: Tensor, groups1: int) -> Tensor:
    """Grouped k=3 causal conv then dense k=3 causal conv (fused_conv.py:39-62).
    The second conv pads the FIRST conv's output with zeros (it does not see conv1
    evaluated on padded input)."""
    return causal_conv_k3(causal_conv_k3(x, w1, groups1), w2, 1)


ATTENTION_STAGES = ("rope", "qk_norm", "convs", "qk_mean", "value_shift")


def ccgqa_pre_attention(qkv: Tensor, p: Dict[str, Tensor], pre: str, cfg: HydraConfig,
                        cos: Tensor, sin: Tensor, off=()) -> Tuple[Tensor, Tensor, Tensor]:
    """Everything between qkv_proj and SDPA (attention.py:208-266).

    qkv [B,S,lat+2*kvd] -> q [B,H,S,hd], k [B,KV,S,hd], v [B,KV,S,hd].
    ``off``: names from ATTENTION_STAGES that are switched off (the module's ``use_*`` arguments, attention.py:74-160).
    """
    assert set(off) <= set(ATTENTION_STAGES), off
    B, S, _ = qkv.shape
    lat, kvd, H, KV, hd = cfg.latent_dim, cfg.kv_dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    q0 = qkv[..., :lat]
    k0 = qkv[..., lat:lat + kvd]
    half = kvd // 2
    # value shift, split by channel index (attention.py:211-220)
    v = qkv.new_zeros(B, S, kvd)
    v[..., :half] = qkv[..., lat + kvd:lat + kvd + half]
    v[:, 1:, half:] = qkv[:, :-1, lat + kvd + half:]
    if "value_shift" in off:
        v = qkv[..., lat + kvd:].clone()
    # conv sequences (attention.py:228-231)
    if "convs" in off:
        q1, k1 = q0, k0
    else:
        q1 = conv_sequence(q0, p[pre + "q_conv.conv1.weight"], p[pre + "q_conv.conv2.weight"], H)
        k1 = conv_sequence(k0, p[pre + "k_conv.conv1.weight"], p[pre + "k_conv.conv2.weight"], KV)
    # QK-mean coupling (attention.py:233-246)
    if "qk_mean" in off:
        q2, k2 = q1, k1
    elif H // KV == 1:
        m = 0.5 * (q0 + k0)
        q2, k2 = q1 + m, k1 + m
    else:
        qm = q0.reshape(B, S, H, hd).mean(dim=2)
        km = k0.reshape(B, S, KV, hd).mean(dim=2)
        q2 = (q1.reshape(B, S, H, hd) + 0.5 * km.unsqueeze(2)).reshape(B, S, lat)
        k2 = (k1.reshape(B, S, KV, hd) + 0.5 * qm.unsqueeze(2)).reshape(B, S, kvd)
    q = q2.reshape(B, S, H, hd).transpose(1, 2)
    k = k2.reshape(B, S, KV, hd).transpose(1, 2)
    v = v.reshape(B, S, KV, hd).transpose(1, 2)
    # L2 norm, key temperature (attention.py:260-262)
    if "qk_norm" not in off:
        q = l2_normalize(q)
        k = l2_normalize(k) * p[pre + "key_temperature"].to(k.dtype)
    # RoPE after the norm (attention.py:264-266)
    if "rope" not in off:
        q = rope(q, cos, sin)
        k = rope(k, cos, sin)
    return q.contiguous(), k.contiguous(), v.contiguous()


def causal_gqa_attention(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """softmax_causal(q k^T / sqrt(hd)) v with q-head h using kv-head h // (H/KV)
    (attention.py:288-327; SDPA default scale).  Returns [B,H,S,hd]."""
    B, H, S, hd = q.shape
    KV = k.shape[1]
    G = H // KV
    kk = k.repeat_interleave(G, dim=1)
    vv = v.repeat_interleave(G, dim=1)
    s = (q @ kk.transpose(-1, -2)) * (1.0 / math.sqrt(hd))
    mask = torch.ones(S, S, dtype=torch.bool).triu(1)
    s = s.masked_fill(mask, float("-inf"))
    pr = torch.softmax(s, dim=-1)
    return pr @ vv


def masked_gqa_attention(q: Tensor, k: Tensor, v: Tensor, mask: Tensor, semantics: str = "reference") -> Tensor:
    """Attention with a padding mask [B,S] (1 = valid token, 0 = padding); query i may use key j where
      "reference": j > i or key j is padding - what CCGQAAttention.forward(x, mask) computes: it builds a boolean mask that
                   is True for future and padded keys (attention.py:269-283) and F.scaled_dot_product_attention reads True
                   as "takes part";
      "intended":  j <= i and key j is valid - what the comments there describe.
    A query with no usable key gives zeros (SDPA's result for a fully masked row)."""
    B, H, S, hd = q.shape
    G = H // k.shape[1]
    kk = k.repeat_interleave(G, dim=1)
    vv = v.repeat_interleave(G, dim=1)
    s = (q @ kk.transpose(-1, -2)) * (1.0 / math.sqrt(hd))
    future = torch.ones(S, S, dtype=torch.bool).triu(1)[None, None]
    pad = (mask == 0).view(B, 1, 1, S)
    if semantics == "reference":
        allowed = future | pad
    elif semantics == "intended":
        allowed = ~future & ~pad
    else:
        raise ValueError(f"unknown mask semantics {semantics!r}")
    s = s.masked_fill(~allowed, float("-inf"))
    pr = torch.softmax(s, dim=-1)
    pr = torch.where(allowed.any(dim=-1, keepdim=True), pr, torch.zeros_like(pr))
    return pr @ vv


def ccgqa_forward(x: Tensor, p: Dict[str, Tensor], pre: str, cfg: HydraConfig, mask: Optional[Tensor] = None,
                  mask_semantics: str = "reference", off=()) -> Tensor:
    """CCGQAAttention.forward (attention.py:201-331): causal, or with a padding mask (see masked_gqa_attention; the
    projections, convolutions and the value shift run over padded positions unchanged)."""
    B, S, _ = x.shape
    cos, sin = rope_tables(S, cfg.head_dim, cfg.rope_theta)
    cos, sin = cos.to(x.dtype), sin.to(x.dtype)
    qkv = x @ p[pre + "qkv_proj.weight"].transpose(0, 1)
    q, k, v = ccgqa_pre_attention(qkv, p, pre, cfg, cos, sin, off)
    o = causal_gqa_attention(q, k, v) if mask is None else masked_gqa_attention(q, k, v, mask, mask_semantics)
    o = o.transpose(1, 2).reshape(B, S, cfg.latent_dim)
    return (o @ p[pre + "o_proj.weight"].transpose(0, 1)) * cfg.output_scale


# ----------------------------------------------------------------------------
# routing
# ----------------------------------------------------------------------------
def mod_k(seq_len: int, capacity: float) -> int:
    """k = max(1, min(L, int(L * clamp(cap, 1e-4, 1))))  (mixture_of_depths.py:179-181)."""
    cap = float(min(max(capacity, 1e-4), 1.0))
    return max(1, min(seq_len, int(seq_len * cap)))


def mod_select(scores: Tensor, capacity: float) -> Tensor:
    """Ascending indices of the top-k scores of each row  (mixture_of_depths.py:187,
    blocks.py:261).  scores [B,L] -> int64 [B,k]."""
    k = mod_k(scores.shape[1], capacity)
    _, idx = torch.topk(scores, k, dim=-1)
    idx, _ = torch.sort(idx, dim=1)
    return idx


def mor_depths(logits: Tensor, n_rec: int, min_depth: int = 0) -> Tuple[Tensor, Tensor]:
    """Router logits -> (int64 depths, probs)  (mixture_of_recursions.py:268-289)."""
    sq = torch.tanh(logits / 2.0) * 3.0
    probs = torch.sigmoid(sq)
    if min_depth > 0:
        cont = min_depth + probs * (n_rec - 1 - min_depth)
    else:
        cont = probs * (n_rec - 1)
    depths = torch.round(cont).long().clamp(min_depth, n_rec - 1)
    return depths, probs


def swiglu_mlp(z: Tensor, w_gate_up: Tensor, w_down: Tensor) -> Tensor:
    """down(silu(gate) * up), [gate|up] = gate_up(z).chunk(2)  (layers/common.py:224-230)."""
    gu = z @ w_gate_up.transpose(0, 1)
    F_ = w_gate_up.shape[0] // 2
    return swiglu(gu[..., :F_], gu[..., F_:]) @ w_down.transpose(0, 1)


@dataclass
class RoutingTaps:
    """Routing decisions of one forward, for parity checks and forced replays."""

    depths: List[Tensor] = field(default_factory=list)                 # per block [B,L] int64
    router_logits: List[Tensor] = field(default_factory=list)          # per block [B,L]
    mod_indices: Dict[Tuple[int, int], Tensor] = field(default_factory=dict)  # (block, rec) -> [B,k]
    mod_scores: Dict[Tuple[int, int], Tensor] = field(default_factory=dict)   # (block, rec) -> [B,L]
    block_out: List[Tensor] = field(default_factory=list)              # per block [B,L,D]
    mlp_rows: Dict[Tuple[int, int], int] = field(default_factory=dict) # (block, rec) -> rows whose MLP result is used


def static_block_forward(x: Tensor, p: Dict[str, Tensor], i: int, cfg: HydraConfig,
                         taps: Optional[RoutingTaps] = None) -> Tensor:
    """HydraMoRBlock with ``static_routing_mode`` (the model flag is honoured in eval as well): every token runs every
    recursion and the routers only weight the results.
    MoD wrapper (blocks.py:190-241): ``mlp(u) * q + u * (1 - q)``, q = sigmoid(clamp(score(u), -10, 10)), u the
    normalised MLP input.  MoR executor (mixture_of_recursions.py:482-558): ``cur += delta`` for all tokens each
    recursion; output = sum_r w_r * cur_r with w_r = exp(-(d - r)^2) / (sum_j exp(-(d - j)^2) + 1e-8),
    d = sigmoid(3 tanh(l / 2)) * (R - 1) (min_depth plays no part).  Fixed-depth blocks (blocks.py:593-606) only get
    the MoD mixing."""
    pre = f"layers.{i}."
    R = cfg.recursions_per_block
    B, L, D = x.shape
    a = ada_rms_norm(x, p[pre + "norm1.weight"], cfg.norm_eps)
    h = x + cfg.residual_scale * ccgqa_forward(a, p, pre + "attention.", cfg, off=cfg.attn_off)
    if cfg.adaptive:
        logits = h @ p[pre + "mor_router.router.weight"].reshape(-1) + p[pre + "mor_router.router.bias"]
        d = torch.sigmoid(torch.tanh(logits / 2.0) * 3.0) * (R - 1)
        wts = torch.exp(-((d.unsqueeze(0) - torch.arange(R, dtype=h.dtype).view(-1, 1, 1)) ** 2))
        wts = wts / (wts.sum(dim=0, keepdim=True) + 1e-8)
    else:
        logits = h.new_zeros(B, L)
    if taps is not None:
        taps.router_logits.append(logits.clone())
    rec_bias = p[pre + "mor_executor.recursion_bias"].reshape(R, D)
    rec_embed = p[pre + "mor_executor.recursion_embed.weight"]
    cur = h
    out = torch.zeros_like(h)
    for r in range(R):
        u = ada_rms_norm(cur + rec_bias[r] + rec_embed[r], p[pre + "norm2.weight"], cfg.norm_eps)
        delta = swiglu_mlp(u, p[pre + "mlp.gate_up.weight"], p[pre + "mlp.down.weight"])
        if cfg.block_has_mod(i):
            mp = pre + "mod_mlp_wrapper.mod_router.router."
            scores = u @ p[mp + "weight"].reshape(-1) + p[mp + "bias"]
            q = torch.sigmoid(scores.clamp(-10.0, 10.0)).unsqueeze(-1)
            delta = delta * q + u * (1 - q)
            if taps is not None:
                taps.mod_scores[(i, r)] = scores.clone()
        if taps is not None:
            taps.mlp_rows[(i, r)] = B * L
        cur = cur + delta
        if cfg.adaptive:
            out = out + wts[r].unsqueeze(-1) * cur
    y = rms_norm(out if cfg.adaptive else cur, p[pre + "final_norm.weight"], cfg.norm_eps)
    if taps is not None:
        taps.block_out.append(y.clone())
    return y


def mor_block_forward(x: Tensor, p: Dict[str, Tensor], i: int, cfg: HydraConfig,
                      taps: Optional[RoutingTaps] = None,
                      forced: Optional[RoutingTaps] = None) -> Tensor:
    """HydraMoRBlock._forward_mor in eval with MoD hard routing enabled
    (blocks.py:608-632, 243-269; mixture_of_recursions.py:426-480).

    ``forced`` replays another run's depths / MoD index lists instead of computing
    them, so numerical error can be separated from routing flips.
    """
    if cfg.adaptive and cfg.mor_rampup_scale < 1.0:
        # HydraMoRBlock.forward (blocks.py:645-657): both paths are whole block forwards (attention included)
        import dataclasses
        s_ = float(cfg.mor_rampup_scale)
        fixed_cfg = dataclasses.replace(cfg, adaptive=False, mor_rampup_scale=1.0)
        # before the ramp starts the fixed path is the whole block: its MoD routing is what taps record / forced replays
        fixed = mor_block_forward(x, p, i, fixed_cfg, taps if s_ <= 0.0 else None, forced if s_ <= 0.0 else None)
        if s_ <= 0.0:
            return fixed
        adaptive = mor_block_forward(x, p, i, dataclasses.replace(cfg, mor_rampup_scale=1.0), taps, forced)
        y = s_ * adaptive + (1.0 - s_) * fixed
        if taps is not None:
            taps.block_out[-1] = y.clone()
        return y
    if cfg.static_routing:
        if forced is not None:
            raise ValueError("static routing makes no routing decisions to replay")
        return static_block_forward(x, p, i, cfg, taps)
    pre = f"layers.{i}."
    R = cfg.recursions_per_block
    B, L, D = x.shape
    a = ada_rms_norm(x, p[pre + "norm1.weight"], cfg.norm_eps)
    att = ccgqa_forward(a, p, pre + "attention.", cfg, off=cfg.attn_off)
    h = x + cfg.residual_scale * att
    if cfg.adaptive:
        logits = h @ p[pre + "mor_router.router.weight"].reshape(-1) + p[pre + "mor_router.router.bias"]
        depths, _ = mor_depths(logits, R, cfg.mor_min_depth)
        if forced is not None:
            depths = forced.depths[i].to(torch.int64)
    else:
        # _forward_fixed (blocks.py:593-606) == every token at the maximum depth
        logits = h.new_zeros(B, L)
        depths = torch.full((B, L), R - 1, dtype=torch.int64)
    if taps is not None:
        taps.depths.append(depths.clone())
        taps.router_logits.append(logits.clone())
    rec_bias = p[pre + "mor_executor.recursion_bias"].reshape(R, D)
    rec_embed = p[pre + "mor_executor.recursion_embed.weight"]
    has_mod = cfg.block_has_mod(i)
    cur = h
    out = torch.zeros_like(h)
    for r in range(R):
        active = (depths >= r)
        exits = (depths == r)
        u = ada_rms_norm(cur + rec_bias[r] + rec_embed[r], p[pre + "norm2.weight"], cfg.norm_eps)
        if has_mod:
            mp = pre + "mod_mlp_wrapper.mod_router.router."
            scores = u @ p[mp + "weight"].reshape(-1) + p[mp + "bias"]
            idx = mod_select(scores, cfg.mod_capacity)
            if forced is not None:
                idx = forced.mod_indices[(i, r)].to(torch.int64)
            if taps is not None:
                taps.mod_indices[(i, r)] = idx.clone()
                taps.mod_scores[(i, r)] = scores.clone()
            gidx = idx.unsqueeze(-1).expand(-1, -1, D)
            sel = torch.gather(u, 1, gidx)
            delta = torch.zeros_like(u)
            delta.scatter_(1, gidx, swiglu_mlp(sel, p[pre + "mlp.gate_up.weight"], p[pre + "mlp.down.weight"]))
            if taps is not None:
                selmask = torch.zeros(B, L, dtype=torch.bool)
                selmask.scatter_(1, idx, True)
                taps.mlp_rows[(i, r)] = int((selmask & active).sum())
        else:
            delta = swiglu_mlp(u, p[pre + "mlp.gate_up.weight"], p[pre + "mlp.down.weight"])
            if taps is not None:
                taps.mlp_rows[(i, r)] = int(active.sum())
        cur = cur + delta * active.unsqueeze(-1).to(h.dtype)
        out = out + cur * exits.unsqueeze(-1).to(h.dtype)
    y = rms_norm(out, p[pre + "final_norm.weight"], cfg.norm_eps)
    if taps is not None:
        taps.block_out.append(y.clone())
    return y


def embed(ids: Tensor, p: Dict[str, Tensor], cfg: HydraConfig) -> Tensor:
    """Clamp ids into range, gather rows, scale by sqrt(dim)  (model.py:51-73,427)."""
    ids = ids.clamp(0, cfg.vocab_size - 1)
    return p["tok_emb.weight"][ids] * math.sqrt(cfg.dim)


def model_forward(ids: Tensor, p: Dict[str, Tensor], cfg: HydraConfig,
                  taps: Optional[RoutingTaps] = None,
                  forced: Optional[RoutingTaps] = None,
                  return_hidden: bool = False) -> Tensor:
    """HydraModel.forward, eval, return_losses=False  (model.py:408-506)."""
    h = embed(ids, p, cfg)
    for i in range(cfg.n_mor_blocks):
        h = mor_block_forward(h, p, i, cfg, taps, forced)
    h = rms_norm(h, p["norm.weight"], cfg.norm_eps)
    if return_hidden:
        return h
    w_out = p["output.weight"] if "output.weight" in p else p["tok_emb.weight"]
    return h @ w_out.transpose(0, 1)


def base_block_forward(x: Tensor, p: Dict[str, Tensor], i: int, cfg: HydraConfig) -> Tensor:
    """HydraBlock.forward (blocks.py:68-70): h = x + attn(norm1 x); h + mlp(norm2 h).  No routing, no residual
    scale, no exit norm."""
    pre = f"layers.{i}."
    h = x + ccgqa_forward(rms_norm(x, p[pre + "norm1.weight"], cfg.norm_eps), p, pre + "attention.", cfg, off=cfg.attn_off)
    return h + swiglu_mlp(rms_norm(h, p[pre + "norm2.weight"], cfg.norm_eps), p[pre + "mlp.gate_up.weight"],
                          p[pre + "mlp.down.weight"])


def base_model_forward(ids: Tensor, p: Dict[str, Tensor], cfg: HydraConfig, taps: Optional[list] = None) -> Tensor:
    """HydraBaseModel.forward (model.py:140-159): the routing-free baseline; cfg.n_mor_blocks is its n_layers.
    `taps`, if given, receives every block's output."""
    h = embed(ids, p, cfg)
    for i in range(cfg.n_mor_blocks):
        h = base_block_forward(h, p, i, cfg)
        if taps is not None:
            taps.append(h)
    h = rms_norm(h, p["norm.weight"], cfg.norm_eps)
    w_out = p["output.weight"] if "output.weight" in p else p["tok_emb.weight"]
    return h @ w_out.transpose(0, 1)


def greedy_generate(prompt_ids: Tensor, p: Dict[str, Tensor], cfg: HydraConfig, max_new_tokens: int,
                    return_margins: bool = False):
    """Greedy form of the reference's generation loop (diagnostics/eval_checkpoint.py:127-160): the full forward is
    re-run on the whole sequence for every new token (the reference has no KV cache); next token = argmax of the
    last position's logits (its sampler with temperature -> 0, top-k/top-p off).  With ``return_margins`` also the
    gap between the best and second-best logit at every step."""
    seq = prompt_ids.clone()
    margins = []
    for _ in range(max_new_tokens):
        logits = model_forward(seq, p, cfg)[:, -1, :]
        top2 = logits.topk(2, dim=-1).values
        margins.append(top2[:, 0] - top2[:, 1])
        seq = torch.cat([seq, logits.argmax(dim=-1, keepdim=True)], dim=1)
    if return_margins:
        return seq, torch.stack(margins, dim=1)
    return seq


def sample_filter(logits: Tensor, temperature: float, top_k: int, top_p: float) -> Tensor:
    """The filtering of the reference's sampler (diagnostics/eval_checkpoint.py:133-151) on [B, V] logits: divide by
    the temperature, remove what lies below the k-th largest value (``top_k > 0``; ties with it stay), then in
    descending order remove a token iff the probability mass up to and including its predecessor exceeds ``top_p``
    (the first always stays).  Removed entries are -inf.  Equal logits are ordered by ascending token id."""
    x = logits.to(torch.float32) / temperature
    if top_k > 0:
        kth = torch.topk(x, min(int(top_k), x.shape[-1]))[0][..., -1, None]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, sorted_idx = torch.sort(x, descending=True, stable=True)
        cum = torch.cumsum(torch.softmax(sorted_logits, dim=-1), dim=-1)
        rem = cum > top_p
        rem[..., 1:] = rem[..., :-1].clone()
        rem[..., 0] = False
        x = x.masked_fill(rem.scatter(1, sorted_idx, rem), float("-inf"))
    return x


def sample_next_token(logits: Tensor, temperature: float, top_k: int, top_p: float, uniforms: Tensor) -> Tensor:
    """One draw per row from softmax(sample_filter(...)) (eval_checkpoint.py:153-155).  The reference draws with
    torch.multinomial; this draw is the inverse CDF in descending-logit order (equal logits by ascending id) at
    ``uniforms`` [B] in [0, 1): the first token whose cumulative probability exceeds the uniform number.
    ``temperature <= 0`` or ``top_k == 1``: the argmax (lowest id among equal maxima)."""
    if not temperature > 0.0 or top_k == 1:
        m = logits.max(dim=-1, keepdim=True).values
        return (logits == m).to(torch.int64).argmax(dim=-1)
    x = sample_filter(logits, temperature, top_k, top_p)
    sx, si = torch.sort(x, descending=True, stable=True)
    cdf = torch.cumsum(torch.softmax(sx.to(torch.float64), dim=-1), dim=-1)
    kept = torch.isfinite(sx).sum(dim=-1)
    j = (cdf > uniforms.to(torch.float64)[:, None]).to(torch.int64).argmax(dim=-1)
    j = torch.minimum(j, kept - 1)
    miss = ~(cdf > uniforms.to(torch.float64)[:, None]).any(dim=-1)      # rounding left the last cdf entry below u
    j = torch.where(miss, kept - 1, j)
    return si.gather(1, j[:, None])[:, 0]


# ----------------------------------------------------------------------------
# cached (incremental) decode - NOT in the reference
# ----------------------------------------------------------------------------
class DecodeCache:
    """Per-block state that lets one new token be processed without re-running the sequence.

    The reference has no KV cache and no decode path (its generation helper re-runs the whole forward,
    diagnostics/eval_checkpoint.py:127-160), so this restatement is pinned only against the re-forward itself:
    with mod_capacity = 1.0 cached decode is mathematically the same computation (every operation of the eval
    forward is causal except MoD's top-k over the sequence) and tests require equality up to fp32 rounding.  With
    capacity < 1 it is an approximation by construction: a past token's MoD selection is frozen at the value it had
    when that token was the newest one.

    Per block: post-RoPE keys and value-shifted values of every position (the latent-space KV cache), the
    pre-conv q|k rows of the last four positions (causal conv halo: conv1 o conv2 reach back four tokens), the
    previous position's v_shift half, and - for MoD blocks - the router score of every cached position per
    recursion."""

    def __init__(self, cfg: HydraConfig, batch: int):
        self.cfg, self.batch, self.pos = cfg, batch, 0
        nb = cfg.n_mor_blocks
        self.k = [None] * nb        # [B, KV, pos, hd]
        self.v = [None] * nb
        self.halo = [None] * nb     # [B, 4, lat+kvd], oldest first
        self.vshift = [None] * nb   # [B, kvd/2]
        self.scores = {}            # (block, rec) -> [B, pos]


def _qk_finish(q1, k1, q0, k0, p, pre, cfg, positions):
    """QK-mean coupling, L2 norm, temperature, RoPE for rows at the given absolute positions (attention.py:233-266).
    q1,k1: conv outputs [B,n,lat]/[B,n,kvd]; q0,k0: pre-conv rows."""
    B, n, _ = q1.shape
    H, KV, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    if H // KV == 1:
        m = 0.5 * (q0 + k0)
        q2, k2 = q1 + m, k1 + m
    else:
        qm = q0.reshape(B, n, H, hd).mean(dim=2)
        km = k0.reshape(B, n, KV, hd).mean(dim=2)
        q2 = (q1.reshape(B, n, H, hd) + 0.5 * km.unsqueeze(2)).reshape(B, n, -1)
        k2 = (k1.reshape(B, n, KV, hd) + 0.5 * qm.unsqueeze(2)).reshape(B, n, -1)
    q = l2_normalize(q2.reshape(B, n, H, hd).transpose(1, 2))
    k = l2_normalize(k2.reshape(B, n, KV, hd).transpose(1, 2)) * p[pre + "key_temperature"].to(k2.dtype)
    cos, sin = rope_tables(int(positions.max()) + 1, hd, cfg.rope_theta)
    cos, sin = cos[positions].to(q.dtype), sin[positions].to(q.dtype)

    def rot(x):
        xe, xo = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = xe * cos - xo * sin
        out[..., 1::2] = xe * sin + xo * cos
        return out

    return rot(q), rot(k)


def cached_prefill(ids: Tensor, p: Dict[str, Tensor], cfg: HydraConfig) -> Tuple[Tensor, DecodeCache]:
    """Full eval forward of the prompt (identical to model_forward) that also fills a DecodeCache.
    Returns (logits [B,S,V], cache)."""
    B, S = ids.shape
    cache = DecodeCache(cfg, B)
    lat, kvd = cfg.latent_dim, cfg.kv_dim
    taps = RoutingTaps()
    h = embed(ids, p, cfg)
    for i in range(cfg.n_mor_blocks):
        pre = f"layers.{i}.attention."
        a = ada_rms_norm(h, p[f"layers.{i}.norm1.weight"], cfg.norm_eps)
        qkv = a @ p[pre + "qkv_proj.weight"].transpose(0, 1)
        cos, sin = rope_tables(S, cfg.head_dim, cfg.rope_theta)
        _, k, v = ccgqa_pre_attention(qkv, p, pre, cfg, cos, sin)
        cache.k[i], cache.v[i] = k.clone(), v.clone()
        halo = qkv.new_zeros(B, 4, lat + kvd)
        n = min(4, S)
        halo[:, 4 - n:] = qkv[:, S - n:, :lat + kvd]
        cache.halo[i] = halo
        cache.vshift[i] = qkv[:, -1, lat + kvd + kvd // 2:].clone()
        h = mor_block_forward(h, p, i, cfg, taps)
    for key, sc in taps.mod_scores.items():
        cache.scores[key] = sc.clone()
    cache.pos = S
    hN = rms_norm(h, p["norm.weight"], cfg.norm_eps)
    return hN @ p.get("output.weight", p["tok_emb.weight"]).transpose(0, 1), cache


def cached_decode_step(tokens: Tensor, p: Dict[str, Tensor], cfg: HydraConfig, cache: DecodeCache) -> Tensor:
    """One new token per sequence at position cache.pos.  tokens int64 [B] -> logits [B, V]; appends to the cache."""
    B = tokens.shape[0]
    t = cache.pos
    lat, kvd, H, KV, hd = cfg.latent_dim, cfg.kv_dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    R, D = cfg.recursions_per_block, cfg.dim
    if cfg.adaptive and cfg.mor_rampup_scale < 1.0:
        if cfg.mor_rampup_scale > 0.0:
            raise ValueError("cached decode inside the MoR ramp-up blend is not defined (two block outputs per step)")
        import dataclasses
        cfg = dataclasses.replace(cfg, adaptive=False, mor_rampup_scale=1.0)   # before the ramp: the fixed-depth path
    x = embed(tokens.view(B, 1), p, cfg)[:, 0]                               # [B, D]
    for i in range(cfg.n_mor_blocks):
        pre = f"layers.{i}."
        ap = pre + "attention."
        a = ada_rms_norm(x, p[pre + "norm1.weight"], cfg.norm_eps)
        qkv = a @ p[ap + "qkv_proj.weight"].transpose(0, 1)                  # [B, lat+2kvd]
        half = kvd // 2
        v_new = torch.cat([qkv[:, lat + kvd:lat + kvd + half], cache.vshift[i]], dim=1)   # [B, kvd]
        win = torch.cat([cache.halo[i], qkv[:, None, :lat + kvd]], dim=1)    # positions t-4 .. t
        # conv1 on the window: its last three rows (positions t-2 .. t) see their full receptive field
        y1q = causal_conv_k3(win[..., :lat], p[ap + "q_conv.conv1.weight"], H)[:, 2:]
        y1k = causal_conv_k3(win[..., lat:], p[ap + "k_conv.conv1.weight"], KV)[:, 2:]
        c2q = sum(y1q[:, j] @ p[ap + "q_conv.conv2.weight"][:, :, j].transpose(0, 1) for j in range(3))
        c2k = sum(y1k[:, j] @ p[ap + "k_conv.conv2.weight"][:, :, j].transpose(0, 1) for j in range(3))
        q, k = _qk_finish(c2q[:, None], c2k[:, None], qkv[:, None, :lat], qkv[:, None, lat:lat + kvd], p, ap, cfg,
                          torch.tensor([t]))
        cache.k[i] = torch.cat([cache.k[i], k], dim=2)
        cache.v[i] = torch.cat([cache.v[i], v_new.reshape(B, KV, 1, hd)], dim=2)
        cache.halo[i] = win[:, 1:].clone()
        cache.vshift[i] = qkv[:, lat + kvd + half:].clone()
        # one query against all cached keys (causal by construction)
        G = H // KV
        kk = cache.k[i].repeat_interleave(G, dim=1)
        vv = cache.v[i].repeat_interleave(G, dim=1)
        sc = (q @ kk.transpose(-1, -2)) * (1.0 / math.sqrt(hd))            # [B,H,1,t+1]
        o = (torch.softmax(sc, dim=-1) @ vv).transpose(1, 2).reshape(B, lat)
        h = x + cfg.residual_scale * (o @ p[ap + "o_proj.weight"].transpose(0, 1)) * cfg.output_scale
        if cfg.adaptive:
            logit = h @ p[pre + "mor_router.router.weight"].reshape(-1) + p[pre + "mor_router.router.bias"]
            depth, _ = mor_depths(logit, R, cfg.mor_min_depth)
        else:
            depth = torch.full((B,), R - 1, dtype=torch.int64)
        rec = p[pre + "mor_executor.recursion_bias"].reshape(R, D) + p[pre + "mor_executor.recursion_embed.weight"]
        cur = h
        if cfg.static_routing:
            # static routing is causal throughout (no top-k over the sequence): the cached step is the forward of the
            # newest position, exactly (static_block_forward)
            if cfg.adaptive:
                d = torch.sigmoid(torch.tanh(logit / 2.0) * 3.0) * (R - 1)
                wts = torch.exp(-((d.unsqueeze(0) - torch.arange(R, dtype=h.dtype).view(-1, 1)) ** 2))
                wts = wts / (wts.sum(dim=0, keepdim=True) + 1e-8)
            out = torch.zeros_like(h)
            for r in range(R):
                u = ada_rms_norm(cur + rec[r], p[pre + "norm2.weight"], cfg.norm_eps)
                delta = swiglu_mlp(u, p[pre + "mlp.gate_up.weight"], p[pre + "mlp.down.weight"])
                if cfg.block_has_mod(i):
                    mp = pre + "mod_mlp_wrapper.mod_router.router."
                    qq = torch.sigmoid((u @ p[mp + "weight"].reshape(-1) + p[mp + "bias"]).clamp(-10.0, 10.0))[:, None]
                    delta = delta * qq + u * (1 - qq)
                cur = cur + delta
                if cfg.adaptive:
                    out = out + wts[r][:, None] * cur
            x = rms_norm(out if cfg.adaptive else cur, p[pre + "final_norm.weight"], cfg.norm_eps)
            continue
        for r in range(R):
            u = ada_rms_norm(cur + rec[r], p[pre + "norm2.weight"], cfg.norm_eps)
            use = depth >= r
            if cfg.block_has_mod(i):
                mp = pre + "mod_mlp_wrapper.mod_router.router."
                s_new = u @ p[mp + "weight"].reshape(-1) + p[mp + "bias"]                 # [B]
                old = cache.scores[(i, r)]                                               # [B, t]
                kk_ = mod_k(t + 1, cfg.mod_capacity)
                # top-k over positions 0..t with the newest position losing ties
                selected = (old >= s_new[:, None]).sum(dim=1) < kk_
                cache.scores[(i, r)] = torch.cat([old, s_new[:, None]], dim=1)
                use = use & selected
            delta = swiglu_mlp(u, p[pre + "mlp.gate_up.weight"], p[pre + "mlp.down.weight"])
            cur = cur + delta * use[:, None].to(cur.dtype)
        x = rms_norm(cur, p[pre + "final_norm.weight"], cfg.norm_eps)
    cache.pos = t + 1
    hN = rms_norm(x, p["norm.weight"], cfg.norm_eps)
    return hN @ p.get("output.weight", p["tok_emb.weight"]).transpose(0, 1)


def cached_generate(prompt_ids: Tensor, p: Dict[str, Tensor], cfg: HydraConfig, max_new_tokens: int,
                    return_logits: bool = False):
    """Greedy generation with the decode cache: prefill the prompt, then one cached step per new token."""
    logits, cache = cached_prefill(prompt_ids, p, cfg)
    seq = prompt_ids.clone()
    last = logits[:, -1]
    all_last = [last]
    for n in range(max_new_tokens):
        nxt = last.argmax(dim=-1)
        seq = torch.cat([seq, nxt[:, None]], dim=1)
        if n + 1 < max_new_tokens:
            last = cached_decode_step(nxt, p, cfg, cache)
            all_last.append(last)
    if return_logits:
        return seq, torch.stack(all_last, dim=1)
    return seq


# ----------------------------------------------------------------------------
# seeded random-init weights with the reference's distributions
# ----------------------------------------------------------------------------
def init_params(cfg: HydraConfig, seed: int = 0, dtype: torch.dtype = torch.float32,
                round_to_bf16: bool = True, perturb: bool = False) -> Dict[str, Tensor]:
    """Random-init weights drawn from the distributions the reference uses
    (model.py:351-374; mixture_of_recursions.py:380-384; base.py:16-19;
    attention.py:147): Linear/Embedding/Conv1d N(0,0.02), o_proj and down scaled by
    1/sqrt(2*NB*R), norm gains 1, recursion_bias 0, recursion_embed N(0,0.02),
    key_temperature sqrt(hd), MoR router bias logit(0.2+0.3*i/max(1,NB-1)) (depth
    scale 1), MoD router bias logit(capacity).

    The draw ORDER is this file's own (the reference's constructor consumes its RNG
    differently), so these are "seeded random-init weights of that architecture",
    not a bit-copy of ``HydraModel(...)`` at the same seed.  ``perturb`` moves the
    norm gains, recursion biases and router weights off their init values so every
    term of the forward is exercised.  ``round_to_bf16`` makes every value exactly
    representable in bf16, so the bf16 device path starts from identical bits.
    """
    g = torch.Generator().manual_seed(seed)
    D, lat, kvd, H, KV, hd = cfg.dim, cfg.latent_dim, cfg.kv_dim, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    F_, R, NB = cfg.ffn_hidden, cfg.recursions_per_block, cfg.n_mor_blocks
    res = 1.0 / math.sqrt(2 * NB * R)

    def nrm(*shape, std=0.02, mean=0.0):
        return torch.randn(*shape, generator=g) * std + mean

    def logit(pr):
        pr = min(max(pr, 1e-4), 1 - 1e-4)
        return math.log(pr / (1 - pr))

    p: Dict[str, Tensor] = {}
    p["tok_emb.weight"] = nrm(cfg.vocab_size, D)
    for i in range(NB):
        pre = f"layers.{i}."
        p[pre + "attention.qkv_proj.weight"] = nrm(lat + 2 * kvd, D)
        p[pre + "attention.o_proj.weight"] = nrm(D, lat) * res
        p[pre + "attention.q_conv.conv1.weight"] = nrm(lat, hd, 3)
        p[pre + "attention.q_conv.conv2.weight"] = nrm(lat, lat, 3)
        p[pre + "attention.k_conv.conv1.weight"] = nrm(kvd, hd, 3)
        p[pre + "attention.k_conv.conv2.weight"] = nrm(kvd, kvd, 3)
        p[pre + "attention.key_temperature"] = torch.full((1,), float(hd ** 0.5))
        p[pre + "norm1.weight"] = nrm(D, std=0.1, mean=1.0) if perturb else torch.ones(D)
        p[pre + "norm2.weight"] = nrm(D, std=0.1, mean=1.0) if perturb else torch.ones(D)
        p[pre + "final_norm.weight"] = nrm(D, std=0.1, mean=1.0) if perturb else torch.ones(D)
        p[pre + "mlp.gate_up.weight"] = nrm(2 * F_, D)
        p[pre + "mlp.down.weight"] = nrm(D, F_) * res
        p[pre + "mor_router.router.weight"] = nrm(1, D, std=0.2 if perturb else 0.02)
        p[pre + "mor_router.router.bias"] = torch.tensor([logit(0.2 + 0.3 * i / max(1, NB - 1))])
        p[pre + "mor_executor.recursion_bias"] = (nrm(R, 1, 1, D, std=0.05) if perturb
                                                  else torch.zeros(R, 1, 1, D))
        p[pre + "mor_executor.recursion_embed.weight"] = nrm(R, D)
        if cfg.block_has_mod(i):
            mp = pre + "mod_mlp_wrapper.mod_router.router."
            p[mp + "weight"] = nrm(1, D, std=0.2 if perturb else 0.02)
            p[mp + "bias"] = torch.tensor([logit(cfg.mod_capacity)])
    p["norm.weight"] = nrm(D, std=0.1, mean=1.0) if perturb else torch.ones(D)
    if round_to_bf16:
        p = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in p.items()}
    return {k: v.to(dtype) for k, v in p.items()}


def cast_params(p: Dict[str, Tensor], dtype: torch.dtype) -> Dict[str, Tensor]:
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in p.items()}


def config_from_state_dict(sd: Dict[str, Tensor], *, n_heads: int, n_kv_heads: int,
                           compression_factor: int = 4, mod_capacity: float = 0.75,
                           max_seq_len: int = 2048, mor_min_depth: int = 0) -> HydraConfig:
    """Recover the shape fields that a reference state_dict determines."""
    V, D = sd["tok_emb.weight"].shape
    nb = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
    R = sd["layers.0.mor_executor.recursion_embed.weight"].shape[0]
    F_ = sd["layers.0.mlp.down.weight"].shape[1]
    return HydraConfig(vocab_size=V, dim=D, n_mor_blocks=nb, recursions_per_block=R, n_heads=n_heads,
                       n_kv_heads=n_kv_heads, compression_factor=compression_factor,
                       max_seq_len=max_seq_len, mod_capacity=mod_capacity, mor_min_depth=mor_min_depth,
                       hidden_dim=F_)


def eval_loss(ids: Tensor, p: Dict[str, Tensor], cfg: HydraConfig, reduction: str = "mean") -> Tensor:
    """The loss of the reference's evaluation helper (diagnostics/eval_checkpoint.py:168-193): the model on
    ``ids[:, :-1]``, F.cross_entropy against ``ids[:, 1:]`` (sum over tokens there; "mean" divides by their number,
    which is what the helper returns at the end)."""
    logits = model_forward(ids[:, :-1], p, cfg)
    tgt = ids[:, 1:].clamp(0, cfg.vocab_size - 1)
    nll = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt.reshape(-1), reduction="none")
    if reduction == "none":
        return nll.view(tgt.shape)
    return nll.sum() if reduction == "sum" else nll.mean()
