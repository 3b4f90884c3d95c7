"""Readers for the golden fixtures written by tests/golden/make_golden.py."""
from __future__ import annotations

import os
from typing import Dict, Tuple

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bits_to_f32(a: np.ndarray) -> torch.Tensor:
    """uint16 bf16 bit patterns -> fp32 tensor with the same values."""
    t = torch.from_numpy(a.astype(np.int32))
    return (t << 16).to(torch.int32).view(torch.float32)


def load(name: str) -> Dict[str, np.ndarray]:
    with np.load(os.path.join(GOLDEN_DIR, name)) as z:
        return {k: z[k] for k in z.files}


def tensor(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.uint16:
        return bits_to_f32(a)
    return torch.from_numpy(np.ascontiguousarray(a))


def weights(fx: Dict[str, np.ndarray], prefix: str = "") -> Dict[str, torch.Tensor]:
    """All 'w:<state_dict key>' entries as fp32 tensors keyed by prefix + key."""
    return {prefix + k[2:]: tensor(v).to(torch.float32) for k, v in fx.items() if k.startswith("w:")}


def attention_fixture(name: str):
    from oracle.hydra_oracle import HydraConfig
    fx = load(name)
    dim, H, KV, B, S = (int(v) for v in fx["meta"])
    cfg = HydraConfig(dim=dim, n_heads=H, n_kv_heads=KV, max_seq_len=S)
    return fx, cfg, weights(fx, "attn.")


def ablated_attention_fixture(name: str):
    """(fx, cfg, [(stages that are off, weights with the 'attn.' prefix, reference output y), ...]); the variants with
    another conv kernel size have every stage on and show it in the shape of their conv weights."""
    fx, cfg, _ = attention_fixture(name)
    out = []
    for i, names in enumerate(fx["variants"].tolist()):
        pre = f"v{i}:w:"
        w = {"attn." + k[len(pre):]: tensor(v).to(torch.float32) for k, v in fx.items() if k.startswith(pre)}
        out.append((tuple(n for n in names.split(",") if not n.startswith("ksize=")), w, torch.from_numpy(fx[f"v{i}:y"])))
    return fx, cfg, out


def model_fixture(name: str):
    from oracle.hydra_oracle import HydraConfig
    fx = load(name)
    vocab, dim, NB, R, H, KV, B, S = (int(v) for v in fx["meta"])
    cfg = HydraConfig(vocab_size=vocab, dim=dim, n_mor_blocks=NB, recursions_per_block=R, n_heads=H,
                      n_kv_heads=KV, max_seq_len=S, mod_capacity=float(fx["cap"][0]),
                      hidden_dim=int(fx["ffn_hidden"][0]),
                      static_routing=bool(int(fx["static"][0])) if "static" in fx else False,
                      mor_rampup_scale=float(fx["rampup"][0]) if "rampup" in fx else 1.0)
    return fx, cfg, weights(fx)
