"""Whole-model executor: HydraModel.forward in eval (hydra/model/framework/model.py:408-506) as one call
into the CUDA extension, fed from a reference ``state_dict`` (key layout: ``tok_emb.weight``,
``layers.{i}.attention.*``, ``layers.{i}.{norm1,norm2,final_norm}.weight``, ``layers.{i}.mlp.*``,
``layers.{i}.mor_router.router.*``, ``layers.{i}.mor_executor.*``,
``layers.{i}.mod_mlp_wrapper.mod_router.router.*``, ``norm.weight``).

Routing is the reference's eval behaviour with MoD enabled (hard top-k at ``mod_capacity`` in the interior
blocks) and MoR dynamic depth routing; routing decisions stay on the device.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import _lib, kernels
from ._pack import PackedBlock, PackedModel, _bf16, _f32
from .sampling import cross_entropy_rows, sample_rows

Tensor = torch.Tensor


@dataclass
class Taps:
    """Routing decisions and per-block outputs of one forward (device tensors)."""

    depths: Tensor            # int32 [NB, B*S]
    mod_idx: Tensor           # int32 [NB, R, B, k]  ascending positions (valid for blocks that carry MoD)
    mod_scores: Tensor        # fp32  [NB, R, B*S]
    router_logits: Tensor     # fp32  [NB, B*S]
    mlp_rows: Tensor          # int32 [NB, R] rows whose MLP result was used
    block_out: Optional[Tensor] = None   # bf16 [NB, B*S, D]


def mod_k(seq_len: int, capacity: float) -> int:
    """k = max(1, min(L, int(L * clamp(cap, 1e-4, 1))))  (hydra/routing/mixture_of_depths.py:179-181)."""
    cap = float(min(max(capacity, 1e-4), 1.0))
    return max(1, min(seq_len, int(seq_len * cap)))


def random_state_dict(*, vocab_size: int = 50257, dim: int, n_mor_blocks: int, recursions_per_block: int, n_heads: int,
                      n_kv_heads: int, compression_factor: int = 4, mlp_ratio: float = 2.67,
                      mod_capacity: float = 0.5, seed: int = 0, device="cuda") -> Dict[str, Tensor]:
    """Seeded random-init weights of a HydraModel architecture, generated on `device`, with the reference's
    key names and init distributions (hydra/model/framework/model.py:351-374: Linear / Embedding / Conv1d
    N(0, 0.02), o_proj and down scaled by 1/sqrt(2*blocks*recursions), norm gains 1, recursion_bias 0,
    recursion_embed N(0, 0.02), key_temperature sqrt(head_dim); depth-router bias
    logit(0.2 + 0.3*i/(blocks-1)) and MoD-router bias logit(capacity), hydra/routing/base.py:16-19).
    Synthetic stand-in for a checkpoint; the draw order is this function's own."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    lat = dim // compression_factor
    hd = lat // n_heads
    kvd = n_kv_heads * hd
    F = ((int(dim * mlp_ratio) + 255) // 256) * 256
    R, NB = recursions_per_block, n_mor_blocks
    res = 1.0 / math.sqrt(2 * NB * R)

    def nrm(*shape, std=0.02):
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std

    def logit(p):
        p = min(max(p, 1e-4), 1 - 1e-4)
        return math.log(p / (1 - p))

    sd: Dict[str, Tensor] = {"tok_emb.weight": nrm(vocab_size, dim), "norm.weight": torch.ones(dim, device=dev)}
    for i in range(NB):
        pre = f"layers.{i}."
        sd[pre + "attention.qkv_proj.weight"] = nrm(lat + 2 * kvd, dim)
        sd[pre + "attention.o_proj.weight"] = nrm(dim, lat) * res
        sd[pre + "attention.q_conv.conv1.weight"] = nrm(lat, hd, 3)
        sd[pre + "attention.q_conv.conv2.weight"] = nrm(lat, lat, 3)
        sd[pre + "attention.k_conv.conv1.weight"] = nrm(kvd, hd, 3)
        sd[pre + "attention.k_conv.conv2.weight"] = nrm(kvd, kvd, 3)
        sd[pre + "attention.key_temperature"] = torch.full((1,), float(hd ** 0.5), device=dev)
        for n in ("norm1", "norm2", "final_norm"):
            sd[pre + n + ".weight"] = torch.ones(dim, device=dev)
        sd[pre + "mlp.gate_up.weight"] = nrm(2 * F, dim)
        sd[pre + "mlp.down.weight"] = nrm(dim, F) * res
        sd[pre + "mor_router.router.weight"] = nrm(1, dim)
        sd[pre + "mor_router.router.bias"] = torch.tensor([logit(0.2 + 0.3 * i / max(1, NB - 1))], device=dev)
        sd[pre + "mor_executor.recursion_bias"] = torch.zeros(R, 1, 1, dim, device=dev)
        sd[pre + "mor_executor.recursion_embed.weight"] = nrm(R, dim)
        if 0 < i < NB - 1 and mod_capacity and mod_capacity > 0:
            sd[pre + "mod_mlp_wrapper.mod_router.router.weight"] = nrm(1, dim)
            sd[pre + "mod_mlp_wrapper.mod_router.router.bias"] = torch.tensor([logit(mod_capacity)], device=dev)
    return sd


def random_base_state_dict(*, vocab_size: int = 50257, dim: int, n_layers: int, n_heads: int, n_kv_heads: int,
                           compression_factor: int = 4, mlp_ratio: float = 2.67, seed: int = 0,
                           device="cuda") -> Dict[str, Tensor]:
    """Seeded random-init weights of a HydraBaseModel (model.py:82-138: Linear / Embedding / Conv1d N(0, 0.02), o_proj and
    down scaled by 1/sqrt(2*n_layers), norm gains 1, key_temperature sqrt(head_dim)); the draw order is this function's."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    lat = dim // compression_factor
    hd = lat // n_heads
    kvd = n_kv_heads * hd
    F = ((int(dim * mlp_ratio) + 255) // 256) * 256
    res = 1.0 / math.sqrt(2 * n_layers)

    def nrm(*shape, std=0.02):
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std

    sd: Dict[str, Tensor] = {"tok_emb.weight": nrm(vocab_size, dim), "norm.weight": torch.ones(dim, device=dev)}
    for i in range(n_layers):
        pre = f"layers.{i}."
        sd[pre + "attention.qkv_proj.weight"] = nrm(lat + 2 * kvd, dim)
        sd[pre + "attention.o_proj.weight"] = nrm(dim, lat) * res
        sd[pre + "attention.q_conv.conv1.weight"] = nrm(lat, hd, 3)
        sd[pre + "attention.q_conv.conv2.weight"] = nrm(lat, lat, 3)
        sd[pre + "attention.k_conv.conv1.weight"] = nrm(kvd, hd, 3)
        sd[pre + "attention.k_conv.conv2.weight"] = nrm(kvd, kvd, 3)
        sd[pre + "attention.key_temperature"] = torch.full((1,), float(hd ** 0.5), device=dev)
        sd[pre + "norm1.weight"] = torch.ones(dim, device=dev)
        sd[pre + "norm2.weight"] = torch.ones(dim, device=dev)
        sd[pre + "mlp.gate_up.weight"] = nrm(2 * F, dim)
        sd[pre + "mlp.down.weight"] = nrm(dim, F) * res
    return sd


def create_hydra_model(vocab_size: int = 50257, dim: int = 2048, n_mor_blocks: int = 8, recursions_per_block: int = 4,
                       n_heads: int = 32, n_kv_heads: int = 4, compression_factor: int = 4, mlp_ratio: float = 2.67,
                       max_seq_len: int = 8192, mod_capacity: float = 0.5, adaptive: bool = True, seed: int = 0,
                       device="cuda", **ignored) -> "HydraB200Model":
    """``hydra.model.framework.factory.create_hydra_model`` (factory.py:11-50, same arguments and defaults; the
    training-only ones - aux_loss_weight, warm-ups, depth scaling - are accepted and ignored): a seeded random-init
    model of that architecture on this backend."""
    sd = random_state_dict(vocab_size=vocab_size, dim=dim, n_mor_blocks=n_mor_blocks,
                           recursions_per_block=recursions_per_block, n_heads=n_heads, n_kv_heads=n_kv_heads,
                           compression_factor=compression_factor, mlp_ratio=mlp_ratio, mod_capacity=mod_capacity,
                           seed=seed, device=device)
    return HydraB200Model(sd, n_heads=n_heads, n_kv_heads=n_kv_heads, compression_factor=compression_factor,
                          max_seq_len=max_seq_len, mod_capacity=mod_capacity, adaptive=adaptive, device=device)


def create_base_model(spec, seed: int = 0, device="cuda") -> "HydraB200BaseModel":
    """``create_base_model(spec)`` (factory.py:53-66): the routing-free baseline from an object with the reference's
    spec attributes (vocab_size, dim, n_layers, n_heads, n_kv_heads, compression_factor, mlp_ratio, max_seq_len), same
    defaults; seeded random init."""
    kw = dict(vocab_size=getattr(spec, "vocab_size", 50257), dim=getattr(spec, "dim", 1344),
              n_layers=getattr(spec, "n_layers", 24), n_heads=getattr(spec, "n_heads", 21),
              n_kv_heads=getattr(spec, "n_kv_heads", 3), compression_factor=getattr(spec, "compression_factor", 4),
              mlp_ratio=getattr(spec, "mlp_ratio", 2.67))
    sd = random_base_state_dict(seed=seed, device=device, **kw)
    if not getattr(spec, "tie_weights", True):
        g = torch.Generator(device=torch.device(device)).manual_seed(seed + 1)
        sd["output.weight"] = torch.randn(kw["vocab_size"], kw["dim"], generator=g, device=device) * 0.02
    return HydraB200BaseModel(sd, n_heads=kw["n_heads"], n_kv_heads=kw["n_kv_heads"],
                              compression_factor=kw["compression_factor"],
                              max_seq_len=getattr(spec, "max_seq_len", 8192), device=device)


# the reference's backward-compatible names (factory.py:69-71)
create_ccgqa_model = create_base_model
create_ccgqa_mod_mor_model = create_hydra_model


def normalize_state_dict(obj) -> Dict[str, Tensor]:
    """Checkpoint payload -> flat state_dict with the current key names.

    Accepts what the reference writes and what its evaluation helper reads
    (diagnostics/eval_checkpoint.py:93-99, hydra/training/checkpointing.py:99-192): a bare state_dict or a dict
    holding it under ``"model"`` / ``"model_state_dict"`` / ``"state_dict"``; ``_orig_mod.`` prefixes left by
    torch.compile are stripped; the older attention layouts (attention.py:333-383: ``q_down``/``k_down``/``v_down``
    (+``v_shift_down``) and flat ``q_conv1`` ... ``k_conv2``) are folded into ``qkv_proj`` / ``q_conv.conv1`` ...;
    MoD bookkeeping buffers are dropped, and so is ``output.weight`` when it is the tied embedding (same storage or
    equal values); an untied projection (``tie_weights=False``, model.py:343-349) is kept."""
    sd = obj
    if isinstance(obj, dict):
        for key in ("model", "model_state_dict", "state_dict"):
            if key in obj and isinstance(obj[key], dict):
                sd = obj[key]
                break
    out: Dict[str, Tensor] = {}
    for k, v in sd.items():
        if not torch.is_tensor(v):
            continue
        while k.startswith("_orig_mod.") or k.startswith("module."):
            k = k.split(".", 1)[1]
        out[k] = v
    prefixes = sorted({k[: -len("q_down.weight")] for k in out if k.endswith("attention.q_down.weight")})
    for pre in prefixes:
        if pre + "qkv_proj.weight" not in out:
            parts = [out.pop(pre + "q_down.weight"), out.pop(pre + "k_down.weight"), out.pop(pre + "v_down.weight")]
            if pre + "v_shift_down.weight" in out:
                parts.append(out.pop(pre + "v_shift_down.weight"))
            out[pre + "qkv_proj.weight"] = torch.cat(parts, dim=0)
    for k in list(out):
        for stem in ("q", "k"):
            for n in ("1", "2"):
                old = f"attention.{stem}_conv{n}.weight"
                if k.endswith(old):
                    out.setdefault(k[: -len(old)] + f"attention.{stem}_conv.conv{n}.weight", out.pop(k))
    for k in list(out):
        if k.endswith("._aux_loss") or ".mod_mlp_wrapper.mlp." in k:
            out.pop(k)
    if "output.weight" in out and "tok_emb.weight" in out:
        o, e = out["output.weight"], out["tok_emb.weight"]
        if o.data_ptr() == e.data_ptr() or (o.shape == e.shape and o.device == e.device and torch.equal(o, e)):
            out.pop("output.weight")
    return out


_BLOCK_KEYS = (
    "attention.qkv_proj.weight", "attention.o_proj.weight", "attention.q_conv.conv1.weight",
    "attention.q_conv.conv2.weight", "attention.k_conv.conv1.weight", "attention.k_conv.conv2.weight",
    "attention.key_temperature", "norm1.weight", "norm2.weight", "final_norm.weight", "mlp.gate_up.weight",
    "mlp.down.weight", "mor_router.router.weight", "mor_router.router.bias", "mor_executor.recursion_bias",
    "mor_executor.recursion_embed.weight", "mod_mlp_wrapper.mod_router.router.weight",
    "mod_mlp_wrapper.mod_router.router.bias")
# RoPE tables / masks that older checkpoints saved; recomputed here
_IGNORED_SUFFIXES = ("cos_cached", "sin_cached", "causal_mask")


def check_state_dict_is_consumed(sd: Dict[str, Tensor]) -> None:
    """Refuse weights this executor would silently drop.  A reference model built with ``moe_enabled`` runs its
    ``moe_layers`` after the scheduled blocks (model.py:431-503); the MoE feed-forward is not part of this backend, so a
    state_dict that carries ``moe_layers.*`` would give plausible but wrong logits.  Any other key that no kernel reads is
    reported the same way."""
    moe = sorted(k for k in sd if k.startswith("moe_layers.") or ".moe_layers." in k)
    if moe:
        raise NotImplementedError(
            f"the state_dict carries {len(moe)} mixture-of-experts tensors ({moe[0]} ...): HydraModel(moe_enabled=True) "
            "runs those layers inside its forward and this backend does not implement them")
    unknown = []
    for k in sd:
        if k in ("tok_emb.weight", "norm.weight", "output.weight"):
            continue
        # bookkeeping buffers of the reference (step counters, routing statistics, the loss tracker's running means):
        # every one of them is registered under a name with a leading underscore, no parameter is
        if k.endswith(_IGNORED_SUFFIXES) or k.rsplit(".", 1)[-1].startswith("_"):
            continue
        if k.startswith("layers."):
            rest = k.split(".", 2)[2] if k.count(".") >= 2 else ""
            if rest in _BLOCK_KEYS:
                continue
        unknown.append(k)
    if unknown:
        raise KeyError(f"state_dict keys that this backend does not consume (refusing to drop them silently): "
                       f"{sorted(unknown)[:8]}{' ...' if len(unknown) > 8 else ''}")


def _untied_output(sd: Dict[str, Tensor], dev) -> Optional[Tensor]:
    """bf16 copy of an untied output projection left in a normalised state_dict, or None when the projection is tied."""
    o = sd.get("output.weight")
    if o is None:
        return None
    if tuple(o.shape) != tuple(sd["tok_emb.weight"].shape):
        raise ValueError(f"output.weight {tuple(o.shape)} does not match tok_emb.weight {tuple(sd['tok_emb.weight'].shape)}")
    return _bf16(o, dev)


def _pad_after_eos(seq: Tensor, prompt_len: int, eos_token_id: Optional[int]) -> Tensor:
    """Overwrite what follows the first generated ``eos_token_id`` of each row with that token (no-op for None)."""
    if eos_token_id is None or seq.shape[1] <= prompt_len:
        return seq
    gen = seq[:, prompt_len:]
    after = (gen == eos_token_id).to(torch.int32).cumsum(dim=1) > 0          # from the first end-of-text token on
    gen[after] = eos_token_id
    return seq


def load_checkpoint(path: str, **model_kwargs) -> "HydraB200Model":
    """Build a HydraB200Model from a checkpoint file written by the reference's trainer (``torch.save`` payload with the
    weights under ``"model"``).  Head counts and routing settings are not stored in the weights: pass ``n_heads``,
    ``n_kv_heads`` and, unless the defaults apply, ``mod_capacity`` / ``mor_min_depth`` / ``max_seq_len``."""
    payload = torch.load(path, map_location="cpu", weights_only=False)
    return HydraB200Model(normalize_state_dict(payload), **model_kwargs)


class HydraB200Model:
    """Inference-only HYDRA model on one B200.

    Args mirror ``HydraModel`` (model.py:180-215) where they affect the eval forward; shapes that the
    ``state_dict`` determines (vocab, dim, blocks, recursions, MLP width) are read from it.
    """

    def __init__(self, state_dict: Dict[str, Tensor], *, n_heads: int, n_kv_heads: int, compression_factor: int = 4,
                 max_seq_len: int = 2048, mod_capacity: float = 0.5, mor_min_depth: int = 0, adaptive: bool = True,
                 device: str | torch.device = "cuda", norm_eps: float = 1e-6, gemm_impl: int = 0,
                 static_routing_mode: bool = False, mor_rampup_scale: float = 1.0, use_rope: bool = True,
                 use_qk_norm: bool = True, use_convs: bool = True, use_qk_mean: bool = True, use_value_shift: bool = True,
                 fold_norm: bool = False):
        """fold_norm: fold the pre-MLP norm into the first MLP contraction (``hb200_block_weights.w_gate_up_n``): the
        routed rows of the hidden state are gathered by the GEMM itself and no normalised copy is written.  Off by
        default: with the gather done by cp.async the contraction loses more than the copy costs (measured)."""
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("HydraB200Model needs a CUDA device (there is no CPU fallback)")
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        sd = normalize_state_dict(state_dict)
        check_state_dict_is_consumed(sd)
        V, D = sd["tok_emb.weight"].shape
        nb = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
        R = sd["layers.0.mor_executor.recursion_embed.weight"].shape[0]
        F = sd["layers.0.mlp.down.weight"].shape[1]
        lat = D // compression_factor
        hd = lat // n_heads
        self.vocab_size, self.dim, self.n_mor_blocks, self.recursions_per_block = V, D, nb, R
        self.effective_layers = nb * R
        self.n_heads, self.n_kv_heads, self.head_dim, self.ffn_hidden = n_heads, n_kv_heads, hd, F
        self.max_seq_len, self.mod_capacity, self.mor_min_depth, self.adaptive = max_seq_len, mod_capacity, mor_min_depth, adaptive
        # static_routing_mode (model.py:202; the reference honours it in eval too): dense compute, soft routing weights
        self.static_routing_mode = bool(static_routing_mode)
        # MoR curriculum scale (HydraMoRBlock.get_mor_rampup_scale, blocks.py:645-657): 1 = adaptive routing, <= 0 = the
        # fixed-depth path, in between every block returns scale * adaptive + (1 - scale) * fixed (forward / prefill only)
        self.mor_rampup_scale = float(mor_rampup_scale)
        if adaptive and self.mor_rampup_scale <= 0.0:
            adaptive = self.adaptive = False
        self.device = dev
        # the attention modules' ablation switches: HydraMoRBlock hands use_* kwargs to the attention factory
        # (blocks.py:482-490); HydraModel itself forwards none, so these only matter for a model assembled from such blocks
        self.attn_disable = ((0 if use_rope else _lib.ATTN_NO_ROPE) | (0 if use_qk_norm else _lib.ATTN_NO_QK_NORM) |
                             (0 if use_convs else _lib.ATTN_NO_CONVS) | (0 if use_qk_mean else _lib.ATTN_NO_QK_MEAN) |
                             (0 if use_value_shift else _lib.ATTN_NO_VALUE_SHIFT))
        with kernels._on(dev):
            blocks = [PackedBlock(sd, f"layers.{i}.", dev, head_dim=hd, fold_norm=fold_norm) for i in range(nb)]
            self.has_mod = [b.tensors["mod_wn"] is not None for b in blocks]
            self.packed = PackedModel(
                vocab=V, dim=D, n_rec=R, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=hd, ffn_hidden=F,
                min_depth=mor_min_depth, adaptive=adaptive, max_seq_len=max_seq_len, mod_capacity=mod_capacity,
                norm_eps=norm_eps, residual_scale=0.5,
                output_scale=float(os.environ.get("HYDRA_CCGQA_OUTPUT_SCALE", "1.0")), blocks=blocks,
                tok_emb=_bf16(sd["tok_emb.weight"], dev), norm_w=_f32(sd["norm.weight"], dev), device=dev,
                gemm_impl=gemm_impl, lm_head=_untied_output(sd, dev), static_routing=self.static_routing_mode,
                mor_rampup=self.mor_rampup_scale if 0.0 < self.mor_rampup_scale < 1.0 else 0.0,
                attn_disable=self.attn_disable)
        # rows of the logits buffer start on 128-byte boundaries: the output projection's stores then cover whole memory
        # sectors (with rows padded to 16 bytes only, its launch took 5.75 ms instead of 5.14 at 65536 x 50257)
        self.ld_logits = (V + 63) // 64 * 64
        self._logits: Optional[Tensor] = None
        self.last_taps: Optional[Taps] = None
        # forward(reuse_buffer=True) replays a CUDA graph of the launch sequence from the second call of a shape on (the
        # executor never synchronises with the host: row counts stay on the device); HB200_PREFILL_GRAPH=0 switches it off
        self.use_graph = os.environ.get("HB200_PREFILL_GRAPH", "1").strip() != "0"
        self._graphs: Dict[tuple, tuple] = {}
        self._graph_seen: Dict[tuple, int] = {}

    # -- reference-compatible conveniences ----------------------------------------------------------------------
    def eval(self):
        return self

    def set_global_step(self, step: int) -> None:
        """The reference enables MoD hard routing in eval only after its warm-up step
        (hydra/model/framework/blocks.py:136-140); here it is always enabled, so this is a no-op."""

    @staticmethod
    def reference_kwargs(model) -> dict:
        """Constructor arguments read off a reference ``HydraModel`` instance: shape attributes, routing settings, and
        the curriculum state its blocks are in (static routing, MoR ramp-up scale)."""
        if getattr(model, "moe_enabled", False) and len(getattr(model, "moe_layers", ())) > 0:
            raise NotImplementedError("this HydraModel was built with moe_enabled=True: its forward runs "
                                      f"{len(model.moe_layers)} mixture-of-experts layers (model.py:431-503) that this "
                                      "backend does not implement")
        # MoD hard routing is on only once the wrapper's warm-up has passed (blocks.py:140,162-186: `_mod_enabled`, set
        # by set_global_step); before that every token goes through the MLP, which is capacity 1.0 here
        wrappers = [l.mod_mlp_wrapper for l in model.layers if getattr(l, "mod_mlp_wrapper", None) is not None]
        mod_on = bool(wrappers) and all(getattr(w_, "_mod_enabled", False) for w_ in wrappers)
        attn = model.layers[0].attention
        switches = {name: bool(getattr(attn, name, True))
                    for name in ("use_rope", "use_qk_norm", "use_convs", "use_qk_mean", "use_value_shift")}
        return dict(**{k: v for k, v in switches.items() if not v},       # only the ones that are off
                    n_heads=model.n_heads, n_kv_heads=model.n_kv_heads, compression_factor=model.compression_factor,
                    max_seq_len=model.max_seq_len, mod_capacity=model.mod_capacity if mod_on else 1.0,
                    mor_min_depth=getattr(model, "mor_min_depth", 0), adaptive=model.adaptive,
                    static_routing_mode=bool(getattr(model, "static_routing_mode", False)),
                    mor_rampup_scale=float(model.layers[0].get_mor_rampup_scale())
                    if hasattr(model.layers[0], "get_mor_rampup_scale") else 1.0)

    @classmethod
    def from_reference(cls, model, **overrides) -> "HydraB200Model":
        """Build from a reference ``HydraModel`` instance (reads its shape attributes and state_dict)."""
        kw = cls.reference_kwargs(model)
        kw.update(overrides)
        return cls(model.state_dict(), **kw)

    # -- forward ---------------------------------------------------------------------------------------------------
    def _alloc_taps(self, B: int, S: int, block_out: bool) -> Taps:
        NB, R, T = self.n_mor_blocks, self.recursions_per_block, B * S
        k = mod_k(S, self.mod_capacity)
        d = self.device
        return Taps(depths=torch.zeros((NB, T), dtype=torch.int32, device=d),
                    mod_idx=torch.zeros((NB, R, B, k), dtype=torch.int32, device=d),
                    mod_scores=torch.zeros((NB, R, T), dtype=torch.float32, device=d),
                    router_logits=torch.zeros((NB, T), dtype=torch.float32, device=d),
                    mlp_rows=torch.zeros((NB, R), dtype=torch.int32, device=d),
                    block_out=torch.zeros((NB, T, self.dim), dtype=torch.bfloat16, device=d) if block_out else None)

    def forward(self, ids: Tensor, mask: Optional[Tensor] = None, return_losses: bool = False, *, taps: bool = False,
                forced: Optional[Taps] = None, block_out: bool = False, logits: bool = True, hidden: bool = False,
                reuse_buffer: bool = False):
        """ids int64 [B, S] on this model's device -> logits bf16 [B, S, vocab] (a view of a buffer whose rows are
        padded to a multiple of 64 columns, i.e. 128 bytes).  Every call returns a tensor of its own, as the reference does;
        ``reuse_buffer=True`` writes into one buffer kept by the model instead (the next such call of the same shape
        overwrites it) - for benchmark and generation loops that want no allocation per step.

        ``mask`` is accepted and ignored, exactly as the reference does: ``HydraModel.forward(x, mask)`` hands it to
        its blocks, and both block types drop it before the attention call (blocks.py:645-657, model.py:143-159).

        taps=True records routing decisions in ``self.last_taps``; ``forced`` replays the decisions of an earlier
        run (its ``depths`` and ``mod_idx``).  hidden=True returns the post-norm hidden state instead/as well.
        """
        if return_losses:
            raise NotImplementedError("return_losses=True is the training path (auxiliary routing losses); this is the "
                                      "inference forward, HydraModel.forward(x, return_losses=False)")
        if not ids.is_cuda or ids.device != self.device:
            raise RuntimeError(f"ids must be on {self.device} (there is no CPU fallback)")
        if ids.dim() != 2:
            raise ValueError("ids must be [batch, seq_len]")
        B, S = ids.shape
        ids = ids.to(torch.int64).contiguous()
        pm = self.packed
        ws = pm.workspace(B, S)
        T = B * S
        out = None
        if logits and reuse_buffer:
            if self._logits is None or self._logits.shape[0] != T:
                self._logits = None
                self._logits = torch.empty((T, self.ld_logits), dtype=torch.bfloat16, device=self.device)
            out = self._logits
        elif logits:
            out = torch.empty((T, self.ld_logits), dtype=torch.bfloat16, device=self.device)
        hid = torch.empty((T, self.dim), dtype=torch.bfloat16, device=self.device) if hidden else None
        tp = None
        tstruct = None
        if forced is not None:
            tp = Taps(depths=forced.depths.contiguous(), mod_idx=forced.mod_idx.contiguous(),
                      mod_scores=torch.zeros_like(forced.mod_scores), router_logits=torch.zeros_like(forced.router_logits),
                      mlp_rows=torch.zeros_like(forced.mlp_rows),
                      block_out=torch.zeros((self.n_mor_blocks, T, self.dim), dtype=torch.bfloat16, device=self.device)
                      if block_out else None)
        elif taps or block_out:
            tp = self._alloc_taps(B, S, block_out)
        if tp is not None:
            tstruct = _lib.Taps(depths=tp.depths.data_ptr(), mod_idx=tp.mod_idx.data_ptr(),
                                mod_scores=tp.mod_scores.data_ptr(), router_logits=tp.router_logits.data_ptr(),
                                mlp_rows=tp.mlp_rows.data_ptr(),
                                block_out=tp.block_out.data_ptr() if tp.block_out is not None else None,
                                force_routing=1 if forced is not None else 0)
        def launch(ids_):
            with kernels._on(self.device):
                _lib.check(_lib.lib().hb200_model_forward(
                    C.byref(pm.struct), ids_.data_ptr(), B, S, ws.data_ptr(), ws.numel(),
                    out.data_ptr() if out is not None else None, self.ld_logits,
                    hid.data_ptr() if hid is not None else None, C.byref(tstruct) if tstruct is not None else None,
                    pm.err_flag.data_ptr(), kernels._stream(self.device)), "model_forward")

        graphable = (self.use_graph and logits and reuse_buffer and not hidden and tp is None and
                     getattr(self, "_profile", None) is None and not torch.cuda.is_current_stream_capturing())
        if graphable:
            # the launch sequence of a shape is fixed (no host decision depends on device data), so it is captured
            # once - after one ordinary call has set the kernels' attributes and sized the buffers - and replayed
            key = (B, S)
            entry = self._graphs.get(key)
            if entry is not None and entry[2:] != (ws.data_ptr(), out.data_ptr()):
                entry = None                                   # a buffer was re-allocated: the captured pointers are stale
                self._graphs.pop(key, None)
            if entry is None and self._graph_seen.get(key, 0) >= 1:
                static_ids = ids.clone()
                graph = torch.cuda.CUDAGraph()
                torch.cuda.current_stream(self.device).synchronize()
                with torch.cuda.graph(graph):
                    launch(static_ids)
                entry = (graph, static_ids, ws.data_ptr(), out.data_ptr())
                while len(self._graphs) >= 8:                   # a handful of shapes at most: drop the oldest capture
                    self._graphs.pop(next(iter(self._graphs)))
                self._graphs[key] = entry
            if entry is not None:
                entry[1].copy_(ids)
                entry[0].replay()
            else:
                self._graph_seen[key] = self._graph_seen.get(key, 0) + 1
                launch(ids)
        else:
            launch(ids)
        self.last_taps = tp
        lg = out[:, :self.vocab_size].view(B, S, self.vocab_size) if out is not None else None
        if hidden and logits:
            return lg, hid.view(B, S, self.dim)
        if hidden:
            return hid.view(B, S, self.dim)
        return lg

    __call__ = forward

    def eval_loss(self, ids: Tensor, targets: Optional[Tensor] = None, reduction: str = "mean",
                  ignore_index: int = -100):
        """Next-token cross-entropy as the reference's evaluation helper computes it (diagnostics/eval_checkpoint.py:
        168-193): with ``targets=None`` the model runs on ``ids[:, :-1]`` and is scored against ``ids[:, 1:]``;
        otherwise ``targets`` [B, S] pairs with ``ids`` [B, S] (``ignore_index`` entries do not count).
        ``reduction``: "mean" (over counted tokens), "sum", or "none" (fp32 [B, S] per-token losses)."""
        if reduction not in ("mean", "sum", "none"):
            raise ValueError(f"unknown reduction {reduction!r}")
        if targets is None:
            if ids.shape[1] < 2:
                raise ValueError("eval_loss needs at least two tokens per sequence")
            ids, targets = ids[:, :-1], ids[:, 1:]
        if tuple(targets.shape) != tuple(ids.shape):
            raise ValueError("targets must have the shape of ids")
        B, S = ids.shape
        lg = self.forward(ids)
        padded = lg.as_strided((B * S, self.ld_logits), (self.ld_logits, 1))      # the rows with their padding columns
        nll = cross_entropy_rows(padded, targets.to(self.device).reshape(-1), vocab=self.vocab_size,
                                 ignore_index=ignore_index)
        if reduction == "none":
            return nll.view(B, S)
        total = nll.sum()
        if reduction == "sum":
            return total
        return total / (targets != ignore_index).sum().clamp(min=1).to(total.dtype)

    def resize_rope_cache(self, new_max_seq_len: int) -> None:
        """HydraModel.resize_rope_cache (model.py:376-392): longer sequences than the model was built for.  The tables
        only ever grow; ``max_seq_len`` takes the new value, as in the reference."""
        new_max_seq_len = int(new_max_seq_len)
        with kernels._on(self.device):
            self.packed.resize_rope(new_max_seq_len)
        self.max_seq_len = new_max_seq_len

    def forward_hidden(self, ids: Tensor) -> Tensor:
        """Post-norm hidden states [B, S, dim] (HydraModel.forward_hidden, model.py:508-520)."""
        return self.forward(ids, logits=False, hidden=True)

    def prefill(self, ids_host: Tensor, out_host: Optional[Tensor] = None) -> Tensor:
        """End-to-end prefill from host memory: copies ids [B, S] (ideally pinned) to the device, runs the full
        forward (all logits are computed and stay resident in HBM), and returns the last position's logits
        [B, vocab] in host memory - what a decoder needs next."""
        ids = ids_host.to(self.device, non_blocking=True)
        lg = self.forward(ids, reuse_buffer=True)
        last = lg[:, -1, :]
        if out_host is None:
            out_host = torch.empty(last.shape, dtype=last.dtype, pin_memory=True)
        out_host.copy_(last, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host

    def generate(self, prompt_ids: Tensor, max_new_tokens: int, mode: str = "reforward", use_graph: bool = True,
                 temperature: Optional[float] = None, top_k: int = 50, top_p: float = 0.9,
                 generator: Optional[torch.Generator] = None, eos_token_id: Optional[int] = None) -> Tensor:
        """Generation.  ``mode="reforward"`` (default) is the reference's way; ``mode="cached"`` runs
        :meth:`generate_cached` (latent-space KV cache; an addition the reference does not have).
        ``temperature=None`` (default) chooses greedily; a number turns on the reference's sampler
        (diagnostics/eval_checkpoint.py:133-155: temperature, ``top_k``, ``top_p``; its defaults are 0.8 / 50 / 0.9)
        with uniform numbers drawn from ``generator`` (:func:`hydra_b200.sampling.sample_rows`).
        ``eos_token_id``: the reference's helper stops its single sequence at the first end-of-text token
        (eval_checkpoint.py:158-160); a batch advances in lockstep here, so every sequence runs the full length and
        whatever follows a sequence's first end-of-text token is overwritten with that token.

        Re-forward: the whole sequence is run through the model again for every new
        token (diagnostics/eval_checkpoint.py:127-160 re-forwards ``generated`` each step; the reference has no KV
        cache).  Exact with respect to the eval forward, including MoD's top-k over the growing sequence, at O(S^2)
        cost.  Only the last position is projected to the vocabulary.  Deterministic form of the reference's sampler
        (temperature -> 0): next token = argmax of the last position's logits.
        prompt_ids int64 [B, P] on this device -> int64 [B, P + max_new_tokens]."""
        if mode == "cached":
            seq = self.generate_cached(prompt_ids, max_new_tokens, use_graph=use_graph, temperature=temperature,
                                       top_k=top_k, top_p=top_p, generator=generator)
            return _pad_after_eos(seq, prompt_ids.shape[1], eos_token_id)
        if mode != "reforward":
            raise ValueError(f"unknown generation mode {mode!r} (use 'reforward' or 'cached')")
        if not prompt_ids.is_cuda or prompt_ids.device != self.device:
            raise RuntimeError(f"prompt_ids must be on {self.device} (there is no CPU fallback)")
        B, P = prompt_ids.shape
        total = P + int(max_new_tokens)
        if total > self.max_seq_len:
            raise ValueError(f"prompt + new tokens = {total} exceeds max_seq_len {self.max_seq_len}")
        seq = torch.empty((B, total), dtype=torch.int64, device=self.device)
        seq[:, :P] = prompt_ids
        self.packed.reserve(B, total)
        ld = self.ld_logits
        last_logits = torch.empty((B, ld), dtype=torch.bfloat16, device=self.device)
        nxt = torch.empty((B,), dtype=torch.int64, device=self.device)
        lib = _lib.lib()
        for cur in range(P, total):
            hid = self.forward(seq[:, :cur], logits=False, hidden=True)            # [B, cur, D]
            last = hid[:, -1, :].contiguous()
            with kernels._on(self.device):
                st = kernels._stream(self.device)
                _lib.check(lib.hb200_gemm_bf16(last.data_ptr(), self.packed.out_proj.data_ptr(), last_logits.data_ptr(),
                                               B, self.vocab_size, self.dim, self.dim, self.dim, ld, _lib.EPI_STORE,
                                               None, 1.0, None, None, self.packed.struct.gemm_impl,
                                               self.packed.err_flag.data_ptr(), st), "lm_head (last position)")
                if temperature is None:
                    _lib.check(lib.hb200_argmax_rows(last_logits.data_ptr(), B, self.vocab_size, ld, nxt.data_ptr(), st),
                               "argmax_rows")
                else:
                    sample_rows(last_logits, temperature, top_k, top_p, generator=generator, vocab=self.vocab_size,
                                out=nxt)
            seq[:, cur] = nxt
        return _pad_after_eos(seq, P, eos_token_id)

    # -- cached decode -----------------------------------------------------------------------------------------------
    def new_decode_session(self, batch: int, capacity: int) -> "DecodeSession":
        """Device state for ``batch`` sequences of up to ``capacity`` positions (prompt + generated)."""
        if self.adaptive and 0.0 < getattr(self, "mor_rampup_scale", 1.0) < 1.0:
            raise NotImplementedError("cached decode is not built for a MoR ramp-up scale between 0 and 1 "
                                      "(use mode='reforward')")
        if getattr(self, "attn_disable", 0) or self.packed.blocks[0].conv_ksize != 3:
            raise NotImplementedError("cached decode is not built for attention modules with a stage switched off or a "
                                      "conv kernel size other than 3 (use mode='reforward')")
        return DecodeSession(self, batch, capacity)

    def generate_cached(self, prompt_ids: Tensor, max_new_tokens: int, use_graph: bool = True,
                        return_logits: bool = False, temperature: Optional[float] = None, top_k: int = 50,
                        top_p: float = 0.9, generator: Optional[torch.Generator] = None):
        """Generation (greedy, or sampled when ``temperature`` is a number) with the latent-space KV cache: one prefill of the prompt, then one decode step per new
        token that touches only the newest position.  With ``mod_capacity == 1`` a step computes what the re-forward
        computes for that position; with capacity < 1 a past token's MoD selection stays as decided when that token was
        the newest (the re-forward re-decides it over the longer sequence), so the two modes may diverge.
        With ``use_graph`` the launch sequence of one step is captured once into a CUDA graph and replayed.
        prompt_ids int64 [B, P] on this device -> int64 [B, P + max_new_tokens] (and, if asked, the bf16 logits
        [B, max_new_tokens, vocab] each choice was made from)."""
        if not prompt_ids.is_cuda or prompt_ids.device != self.device:
            raise RuntimeError(f"prompt_ids must be on {self.device} (there is no CPU fallback)")
        B, P = prompt_ids.shape
        n_new = int(max_new_tokens)
        total = P + n_new
        if total > self.max_seq_len:
            raise ValueError(f"prompt + new tokens = {total} exceeds max_seq_len {self.max_seq_len}")
        sess = self.new_decode_session(B, total)
        keep = [] if return_logits else None
        if n_new > 0:
            sess.prefill(prompt_ids)
            if temperature is not None:
                sess.resample(temperature, top_k, top_p, generator=generator)
            if keep is not None:
                keep.append(sess.last_logits[:, :self.vocab_size].clone())
            for _ in range(n_new - 1):
                sess.step(use_graph=use_graph)
                if temperature is not None:
                    sess.resample(temperature, top_k, top_p, generator=generator)
                if keep is not None:
                    keep.append(sess.last_logits[:, :self.vocab_size].clone())
            seq = sess.history[:, :total].clone()
        else:
            seq = prompt_ids.clone()
        self.check_device_errors()
        if return_logits:
            return seq, (torch.stack(keep, dim=1) if keep else None)
        return seq

    def check_device_errors(self) -> None:
        self.packed.check_device_errors()

    # -- per-launch timing (CUDA events recorded by the executor around every kernel it enqueues) ------------------
    def enable_profile(self, capacity: int = 4096) -> None:
        h = _lib.lib().hb200_profile_create(int(capacity))
        if not h:
            raise _lib.Hb200Error("could not create the launch recorder")
        self._profile, self._profile_cap = h, int(capacity)
        self.packed.struct.profile = h

    def disable_profile(self) -> None:
        if getattr(self, "_profile", None):
            self.packed.struct.profile = None
            _lib.lib().hb200_profile_destroy(self._profile)
            self._profile = None

    def read_profile(self, reset: bool = True) -> List[dict]:
        """One dict per recorded launch (kind, block, rec, m, n, k, ms); waits for the device first (the events of the
        last launches must have completed before their times can be read)."""
        torch.cuda.synchronize(self.device)
        cap = self._profile_cap
        recs = (_lib.LaunchRecord * cap)()
        ms = (C.c_float * cap)()
        n = _lib.lib().hb200_profile_read(self._profile, recs, ms, cap)
        if n < 0:
            _lib.check(n, "profile_read")
        if n > cap:
            raise _lib.Hb200Error(f"the launch recorder holds {cap} records but {n} launches were made since the last "
                                  "read: the breakdown would be truncated (enable_profile with a larger capacity)")
        out = [dict(kind=_lib.KERNEL_KINDS[recs[i].kind], block=recs[i].block, rec=recs[i].rec, m=recs[i].m,
                    n=recs[i].n, k=recs[i].k, ms=float(ms[i])) for i in range(min(n, cap))]
        if reset:
            _lib.lib().hb200_profile_reset(self._profile)
        return out

    def get_routing_stats(self) -> dict:
        """Rows whose MLP result was used per (block, recursion) in the last tapped forward."""
        if self.last_taps is None:
            return {}
        return {"mlp_rows": self.last_taps.mlp_rows.cpu().tolist()}


class HydraB200BaseModel(HydraB200Model):
    """``HydraBaseModel`` (hydra/model/framework/model.py:82-160): the routing-free baseline - ``n_layers`` plain
    pre-norm blocks (``HydraBlock``, blocks.py:33-70: ``h = x + attn(norm1 x)``, ``h + mlp(norm2 h)``), final RMSNorm,
    tied output projection.  Runs on the same executor as the routed model: every block is a one-recursion block with
    a zero recursion offset, full residual scale, no routers and no exit norm.  ``state_dict`` keys:
    ``tok_emb.weight``, ``layers.{i}.attention.*``, ``layers.{i}.{norm1,norm2}.weight``, ``layers.{i}.mlp.*``,
    ``norm.weight``, and ``output.weight`` when the projection is untied."""

    def __init__(self, state_dict: Dict[str, Tensor], *, n_heads: int, n_kv_heads: int, compression_factor: int = 4,
                 max_seq_len: int = 2048, device: str | torch.device = "cuda", norm_eps: float = 1e-6,
                 gemm_impl: int = 0):
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("HydraB200BaseModel needs a CUDA device (there is no CPU fallback)")
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        sd = normalize_state_dict(state_dict)
        check_state_dict_is_consumed(sd)
        V, D = sd["tok_emb.weight"].shape
        nb = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
        F = sd["layers.0.mlp.down.weight"].shape[1]
        lat = D // compression_factor
        hd = lat // n_heads
        self.vocab_size, self.dim, self.n_mor_blocks, self.recursions_per_block = V, D, nb, 1
        self.n_layers = nb
        self.n_heads, self.n_kv_heads, self.head_dim, self.ffn_hidden = n_heads, n_kv_heads, hd, F
        self.max_seq_len, self.mod_capacity, self.mor_min_depth, self.adaptive = max_seq_len, 1.0, 0, False
        self.device = dev
        with kernels._on(dev):
            blocks = [PackedBlock(sd, f"layers.{i}.", dev, plain=True) for i in range(nb)]
            self.has_mod = [False] * nb
            self.packed = PackedModel(
                vocab=V, dim=D, n_rec=1, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=hd, ffn_hidden=F,
                min_depth=0, adaptive=False, max_seq_len=max_seq_len, mod_capacity=1.0, norm_eps=norm_eps,
                residual_scale=1.0, output_scale=float(os.environ.get("HYDRA_CCGQA_OUTPUT_SCALE", "1.0")),
                blocks=blocks, tok_emb=_bf16(sd["tok_emb.weight"], dev), norm_w=_f32(sd["norm.weight"], dev),
                device=dev, gemm_impl=gemm_impl, lm_head=_untied_output(sd, dev))
        self.ld_logits = (V + 63) // 64 * 64
        self._logits = None
        self.last_taps = None
        self.use_graph = os.environ.get("HB200_PREFILL_GRAPH", "1").strip() != "0"
        self._graphs = {}
        self._graph_seen = {}

    @staticmethod
    def reference_kwargs(model) -> dict:
        """Constructor arguments read off a reference ``HydraBaseModel`` instance (it keeps them on its attention modules)."""
        attn = model.layers[0].attention
        return dict(n_heads=attn.n_heads, n_kv_heads=attn.n_kv_heads, compression_factor=attn.compression_factor,
                    max_seq_len=int(attn.cos_cached.shape[-2]))   # [1, 1, S, hd/2] in the reference, [S, hd/2] here

    @classmethod
    def from_reference(cls, model, **overrides) -> "HydraB200BaseModel":
        """Build from a reference ``HydraBaseModel`` instance."""
        kw = cls.reference_kwargs(model)
        kw.update(overrides)
        return cls(model.state_dict(), **kw)


class DecodeSession:
    """Caches and bookkeeping of a batch of sequences decoded in lockstep (``hb200_decode_state``).

    ``prefill(prompt)`` runs the eval forward of the prompt and fills the caches; every ``step()`` then consumes the
    token chosen by the previous call and chooses the next one greedily.  ``history`` [B, capacity] int64 holds the
    token of every position; ``last_logits`` [B, ld] bf16 the logits of the latest choice."""

    def __init__(self, model: HydraB200Model, batch: int, capacity: int):
        if capacity > model.max_seq_len:
            raise ValueError(f"capacity {capacity} exceeds max_seq_len {model.max_seq_len}")
        self.model, self.batch, self.capacity = model, int(batch), int(capacity)
        dev = model.device
        nb, R, KV, hd = model.n_mor_blocks, model.recursions_per_block, model.n_kv_heads, model.head_dim
        lat, kvd = model.n_heads * hd, KV * hd
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.kcache = torch.zeros((nb, batch, KV, capacity, hd), **bf)
        self.vcache = torch.zeros((nb, batch, KV, capacity, hd), **bf)
        self.halo = torch.zeros((nb, batch, 4, lat + kvd), **bf)
        self.vshift = torch.zeros((nb, batch, kvd // 2), **bf)
        self.scores = torch.zeros((nb, R, batch, capacity), dtype=torch.float32, device=dev)
        self.pos_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.history = torch.zeros((batch, capacity), dtype=torch.int64, device=dev)
        self.last_logits = torch.zeros((batch, model.ld_logits), **bf)
        self.struct = _lib.DecodeState(
            batch=batch, capacity=capacity, kcache=self.kcache.data_ptr(), vcache=self.vcache.data_ptr(),
            halo=self.halo.data_ptr(), vshift=self.vshift.data_ptr(), scores=self.scores.data_ptr(),
            pos=self.pos_dev.data_ptr(), tokens=self.tokens.data_ptr(), history=self.history.data_ptr())
        n = _lib.lib().hb200_decode_workspace_bytes(C.byref(model.packed.struct), batch)
        self.workspace = torch.empty(max(int(n), 1), dtype=torch.uint8, device=dev)
        self.pos = 0            # host mirror of *pos
        self._graph = None
        self._eager_steps = 0

    def prefill(self, prompt_ids: Tensor) -> None:
        m = self.model
        B, P = prompt_ids.shape
        if B != self.batch or P < 1 or P > self.capacity:
            raise ValueError(f"prompt shape {tuple(prompt_ids.shape)} does not fit batch {self.batch} / capacity {self.capacity}")
        ids = prompt_ids.contiguous()
        ws = m.packed.workspace(B, P)
        with kernels._on(m.device):
            _lib.check(_lib.lib().hb200_model_prefill_cached(
                C.byref(m.packed.struct), ids.data_ptr(), B, P, ws.data_ptr(), ws.numel(), C.byref(self.struct),
                self.last_logits.data_ptr(), m.ld_logits, m.packed.err_flag.data_ptr(), kernels._stream(m.device)),
                "model_prefill_cached")
        self.pos = P
        self._graph = None

    def resample(self, temperature: float = 0.8, top_k: int = 50, top_p: float = 0.9,
                 uniforms: Optional[Tensor] = None, generator: Optional[torch.Generator] = None) -> Tensor:
        """Replace the greedy choice made by the latest ``prefill`` / ``step`` with a draw from ``last_logits``
        (the reference's sampler, :func:`hydra_b200.sampling.sample_rows`): the next ``step`` processes the drawn
        tokens, and ``history`` records them.  Returns the tokens (the session's own buffer)."""
        if self.pos < 1 or self.pos >= self.capacity:
            raise RuntimeError("resample() needs a prefill first and room for the chosen token in the history")
        sample_rows(self.last_logits, temperature, top_k, top_p, uniforms=uniforms, generator=generator,
                    vocab=self.model.vocab_size, out=self.tokens)
        self.history[:, self.pos] = self.tokens
        return self.tokens

    def _launch_step(self) -> None:
        m = self.model
        _lib.check(_lib.lib().hb200_model_decode_step(
            C.byref(m.packed.struct), C.byref(self.struct), self.workspace.data_ptr(), self.workspace.numel(),
            self.last_logits.data_ptr(), m.ld_logits, m.packed.err_flag.data_ptr(), kernels._stream(m.device)),
            "model_decode_step")

    def step(self, use_graph: bool = False) -> None:
        """Process ``tokens`` at position ``pos`` and choose the next token.  The first step always launches
        directly (one-time kernel attribute setup must not happen inside a capture); later steps replay a graph
        of the identical launch sequence when ``use_graph`` is set."""
        if self.pos >= self.capacity:
            raise RuntimeError(f"decode cache is full ({self.capacity} positions)")
        m = self.model
        with kernels._on(m.device):
            if not use_graph or self._eager_steps == 0:
                self._launch_step()
                self._eager_steps += 1
            else:
                if self._graph is None:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        self._launch_step()
                    self._graph = g
                self._graph.replay()
        self.pos += 1
