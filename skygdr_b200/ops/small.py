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


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gathers table rows."""
    if out is None:
        out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    load().embedding(ids, table, out)
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    load().argmax(logits, out)
    return out


def sample(logits: torch.Tensor, temperature: float, seed: int, positions: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Draws one token per row from softmax(logits / temperature) (Gumbel-max over hashed noise, one pass, no normalisation).
    Deterministic for a given (seed, positions): ``positions`` (int32, one per row) makes a replayed CUDA graph draw fresh
    noise every step, since a sequence's position advances. Greedy decoding is ``argmax``."""
    if out is None:
        out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    load().sample(logits, out, float(temperature), int(seed) & 0xFFFFFFFF, positions)
    return out


def sample_noise_reference(seed: int, positions: torch.Tensor, rows: int, vocab: int) -> torch.Tensor:
    """The uniform numbers the sampling kernel hashes out of (seed, position, row, column), restated with integer tensor
    arithmetic: fp32 [rows][vocab] in (0, 1). ``sample_reference`` builds the kernel's decision from them."""
    M = 0xFFFFFFFF
    r = torch.arange(rows, dtype=torch.int64)[:, None]
    c = torch.arange(vocab, dtype=torch.int64)[None, :]
    pos = positions.to(torch.int64).cpu()[:rows, None]
    h = ((seed & M) * 0x9E3779B1 & M) ^ (((pos + 0x7F4A7C15) & M) * 0x85EBCA77 & M) ^ (((r + 0x165667B1) & M) * 0xC2B2AE3D & M) \
        ^ (((c + 0x27D4EB2F) & M) * 0x9E3779B1 & M)
    h = h ^ (h >> 16)
    h = (h * 0x85EBCA6B) & M
    h = h ^ (h >> 13)
    h = (h * 0xC2B2AE35) & M
    h = h ^ (h >> 16)
    return ((h >> 8).to(torch.float32) + 0.5) * (1.0 / 16777216.0)


def sample_reference(logits: torch.Tensor, temperature: float, seed: int, positions: Optional[torch.Tensor] = None):
    """(token ids, perturbed values) of the Gumbel-max rule on the CPU in fp32: the oracle of ``sample``."""
    rows, vocab = logits.shape
    pos = positions if positions is not None else torch.zeros(rows, dtype=torch.int32)
    u = sample_noise_reference(seed, pos, rows, vocab)
    v = logits.float().cpu() * (1.0 / temperature) - torch.log(-torch.log(u))
    return v.argmax(-1).int(), v
