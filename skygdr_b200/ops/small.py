"""Small fused decoder ops (skygdr_b200/csrc/kernels/fused_ops.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from .._ext import load
from .kv_cache import PagedKVPool


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(x) * w; with ``residual``: residual += x in place, y = rmsnorm(residual) * w."""
    if out is None:
        out = torch.empty_like(x)
    load().rmsnorm(x, residual, w, out, eps)
    return out


def rope_inv_freq(theta: float, device, head_dim: int = 128) -> torch.Tensor:
    return (1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).to(device)


def rope_append(qkv: torch.Tensor, q_norm, k_norm, pool: PagedKVPool, layer: int, inv_freq: torch.Tensor,
                block_table: torch.Tensor, positions: torch.Tensor, q_heads: int, eps: float = 1e-6,
                seq_ids: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-head QK-norm, rotary embedding, q -> q_out [tokens][q_heads][128], k/v -> paged cache."""
    tokens = positions.numel()
    if q_out is None:
        q_out = torch.empty((tokens, q_heads, 128), dtype=torch.bfloat16, device=qkv.device)
    bs, ls, ks = pool.strides
    if pool.layout == "hnd":
        hs, ts = pool.data.stride(3), pool.data.stride(4)
    else:
        ts, hs = pool.data.stride(3), pool.data.stride(4)
    load().rope_append(qkv, q_norm, k_norm, q_out, pool.layer_base(layer), inv_freq, block_table, positions, seq_ids, bs, ks,
                       hs, ts, q_heads, pool.geom.kv_heads, eps)
    return q_out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty((*gate_up.shape[:-1], gate_up.shape[-1] // 2), dtype=gate_up.dtype, device=gate_up.device)
    load().silu_mul(gate_up, out)
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, row_ss: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gathers table rows. ``row_ss`` (fp32 [slots][>= tokens]): slot 0 receives every gathered row's sum of squares and the other
    slots are zeroed, ready for the GEMM epilogues that accumulate into them."""
    if out is None:
        out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    load().embedding(ids, table, out, row_ss)
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    load().argmax(logits, out)
    return out
