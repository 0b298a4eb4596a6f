"""Seeded synthetic inputs for the parity tests (TEST INFRASTRUCTURE ONLY).

Values come from a counter-based hash (splitmix64) followed by Box-Muller in float64, so a
(seed, shape) pair yields the same tensor on every machine and library version -- the committed
golden vectors under ``tests/golden/`` store only seeds and outputs.

The distributions follow the benchmark configurations: N(0,1) queries/keys/values, a fraction of
"planted" key positions aligned with the scoring query so that the top-k is well separated, and
optional fixed outlier channels.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import numpy as np
import torch

from . import tokenselect_oracle as orc

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def hash_u64(seed: int, stream: int, n: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([seed * 1000003 + stream], dtype=np.uint64))[0]
        return _splitmix64(np.arange(n, dtype=np.uint64) + base)


def uniform(seed: int, stream: int, n: int) -> np.ndarray:
    """float64 uniforms in (0, 1)."""
    return ((hash_u64(seed, stream, n) >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)


def normal(seed: int, stream: int, shape) -> torch.Tensor:
    """fp32 N(0,1) tensor of ``shape``."""
    n = int(np.prod(shape))
    u1 = uniform(seed, 2 * stream, n)
    u2 = uniform(seed, 2 * stream + 1, n)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return torch.from_numpy(z.astype(np.float32).reshape(shape))


def permutation(seed: int, stream: int, n: int) -> torch.Tensor:
    return torch.from_numpy(np.argsort(hash_u64(seed, stream, n), kind="stable").astype(np.int64))


@dataclasses.dataclass
class LayerCase:
    """One layer's tensors for one request, in the serving stack's paged layout."""
    q: torch.Tensor              # [Hq*D]      un-rotated query of the token being decoded
    k_pool: torch.Tensor         # [rows, Hkv, D]
    v_pool: torch.Tensor         # [rows, Hkv, D]
    req_to_token: torch.Tensor   # [max_reqs, max_ctx] int32: logical position -> pool row
    req_pool_idx: int
    n_tokens: int                # counts the token being decoded; its K/V are already in the pool
    planted: torch.Tensor        # logical positions of the planted keys


def make_layer_case(seed: int, n_tokens: int, hq: int, hkv: int, d: int, n_init: int, n_local: int,
                    rope_base: float, rope_scale: float = 1.0, gqa_map: str = "mod",
                    dtype: torch.dtype = torch.float32, planted_frac: float = 0.01,
                    planted_gain: float = 3.0, outlier_channels: int = 0, outlier_gain: float = 8.0,
                    pool_rows: Optional[int] = None, max_reqs: int = 2, req_pool_idx: int = 1,
                    max_ctx: Optional[int] = None, permute_slots: bool = True) -> LayerCase:
    """N(0,1) ``q, K, V``; ``planted_frac`` of the candidate positions get
    ``K[p, kv] += planted_gain * q_hat`` where ``q_hat`` is the unit vector of the rotated scoring
    query of the lowest-numbered query head paired with ``kv`` under ``gqa_map``;
    ``outlier_channels`` fixed channels per head are multiplied by ``outlier_gain`` in K and V.
    Pool rows are a seeded permutation so paging is exercised."""
    pool_rows = pool_rows or (n_tokens + 64)
    max_ctx = max_ctx or n_tokens + 8
    q = normal(seed, 1, (hq, d))
    k = normal(seed, 2, (n_tokens, hkv, d))
    v = normal(seed, 3, (n_tokens, hkv, d))
    if outlier_channels:
        ch = permutation(seed, 7, d)[:outlier_channels]
        k[:, :, ch] *= outlier_gain
        v[:, :, ch] *= outlier_gain
    q = q.to(dtype)
    q_rot = orc.rotate_scoring_query(q, n_local, rope_base, rope_scale).float()
    nc = max(n_tokens - n_init - n_local, 0)
    n_plant = int(round(planted_frac * nc))
    planted = (permutation(seed, 4, nc)[:n_plant] + n_init) if n_plant else torch.zeros(0, dtype=torch.int64)
    for kv in range(hkv):
        h0 = min(h for h in range(hq) if orc.scoring_kv_head(h, hq, hkv, gqa_map) == kv)
        q_hat = q_rot[h0] / q_rot[h0].norm()
        k[planted, kv, :] += planted_gain * q_hat
    rows = permutation(seed, 5, pool_rows)[:n_tokens] if permute_slots else torch.arange(n_tokens)
    k_pool = normal(seed, 8, (pool_rows, hkv, d)).to(dtype)     # unused rows hold noise, not zeros
    v_pool = normal(seed, 9, (pool_rows, hkv, d)).to(dtype)
    k_pool[rows] = k.to(dtype)
    v_pool[rows] = v.to(dtype)
    rtt = torch.full((max_reqs, max_ctx), -1, dtype=torch.int32)
    rtt[req_pool_idx, :n_tokens] = rows.to(torch.int32)
    return LayerCase(q=q.reshape(-1), k_pool=k_pool, v_pool=v_pool, req_to_token=rtt,
                     req_pool_idx=req_pool_idx, n_tokens=n_tokens, planted=planted)


def make_chunk_queries(seed: int, case: LayerCase, lq: int, hq: int, d: int, spread: float = 0.5) -> torch.Tensor:
    """Queries of a prefill chunk ``[lq, hq*d]``: the case's query plus ``spread`` x N(0,1) per token, so
    that the chunk's mean fingerprint keeps a direction (the mean of independent queries would be ~0)."""
    noise = normal(seed, 11, (lq, hq * d))
    return (case.q.float().view(1, -1) + spread * noise).to(case.q.dtype)


@dataclasses.dataclass
class AttentionCase:
    """Inputs of one sparse-attention call: a request's pools plus an attended row list."""
    q: torch.Tensor              # [Hq*D] un-rotated decode query (the last listed token's)
    q_chunk: torch.Tensor        # [Lq, Hq*D] un-rotated queries of a prefill chunk closing the list
    k_pool: torch.Tensor         # [rows, Hkv, D]
    v_pool: torch.Tensor
    slots: torch.Tensor          # [n] int32 pool rows in list order


def make_attention_case(seed: int, n_list: int, lq: int, hq: int, hkv: int, d: int,
                        dtype: torch.dtype = torch.bfloat16, pool_rows: Optional[int] = None) -> AttentionCase:
    """N(0,1) pools of ``pool_rows`` rows and a list of ``n_list`` distinct rows in a seeded order (what a
    selected index set looks like after the slot map: unordered pool rows).  ``q`` is the decode query,
    ``q_chunk`` the ``lq`` queries of a prefill chunk whose own rows are the last ``lq`` of the list."""
    pool_rows = pool_rows or (n_list + 97)
    q = normal(seed, 21, (hq * d,)).to(dtype)
    q_chunk = (q.float().view(1, -1) + 0.5 * normal(seed, 22, (max(lq, 1), hq * d))).to(dtype)
    k_pool = normal(seed, 23, (pool_rows, hkv, d)).to(dtype)
    v_pool = normal(seed, 24, (pool_rows, hkv, d)).to(dtype)
    slots = permutation(seed, 25, pool_rows)[:n_list].to(torch.int32)
    return AttentionCase(q=q, q_chunk=q_chunk, k_pool=k_pool, v_pool=v_pool, slots=slots)
