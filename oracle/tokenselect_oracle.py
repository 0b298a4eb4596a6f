"""CPU oracle for TokenSelect's decode-time selection + sparse paged attention.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA path: it may be imported
by the test-suite, by the smoke check and by the benchmark's CPU-baseline / reference legs and
by nothing else.  The product (``tokenselect_b200``) never imports it and has no CPU fallback.

It restates, in plain torch/numpy on the CPU, the algorithm of the reference file
``patcher/token_retrieval.py``.  Every function cites the reference lines it follows.

Parity pin: the reference ships no tests or golden vectors.  The pin used here is the
reference module itself, executed verbatim on the CPU (``oracle/reference_verbatim.py``), whose
outputs are committed under ``tests/golden/`` and compared with this restatement by
``tests/test_oracle_golden.py``.  The attention half (the third-party FlashInfer wrappers the reference
calls, ``:746-772`` and ``:802-823``) is pinned to outputs of that library taken on a B200 with the
reference's call-site arguments (``tests/golden/flashinfer_attention.npz``, made by
``tests/golden/make_flashinfer_golden.py``, compared in ``tests/test_oracle_flashinfer.py``).

Two arithmetic modes exist for the vote vector:

* ``logits_dtype=torch.float32`` -- the mode the CUDA path is built to (fp32 logits and votes).
* ``logits_dtype=torch.bfloat16`` -- what the reference really does (its logits buffer is bf16
  even for an fp32 model, ``token_retrieval.py:345-347``); only used to reproduce the
  reference-verbatim golden vectors bit for bit.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

FLAG_DENSE = 0      # guard hit: attend to every token      (token_retrieval.py:376-378)
FLAG_RECOMPUTE = 1  # scores recomputed this step           (token_retrieval.py:395-417)
FLAG_REUSE = 2      # cached index set reused               (token_retrieval.py:418-420)


# --------------------------------------------------------------------------------------
# RoPE                                                     token_retrieval.py:56-114
# --------------------------------------------------------------------------------------
def rope_inv_freq(head_dim: int, base: float) -> torch.Tensor:
    """fp32 inverse frequencies, same expression as token_retrieval.py:73-82."""
    return 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """token_retrieval.py:112-114."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin rows for fp32 ``positions``; table construction of token_retrieval.py:92-96."""
    freqs = torch.outer(positions.to(torch.float32), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_scoring_query(q: torch.Tensor, n_local: int, rope_base: float, rope_scale: float) -> torch.Tensor:
    """Scoring query: rotate ``q [Hq, D]`` at the fixed position ``n_local * rope_scale`` in fp32
    and round back to ``q.dtype`` (token_retrieval.py:380-388 with :98-107; the position is
    multiplied by the scale at :93)."""
    inv_freq = rope_inv_freq(q.shape[-1], rope_base)
    pos = torch.tensor([n_local * rope_scale], dtype=torch.float32)
    cos, sin = rope_cos_sin(pos, inv_freq)
    return ((q.float() * cos) + (rotate_half(q).float() * sin)).to(q.dtype)


def rotate_chunk_queries(q: torch.Tensor, n_local: int, rope_base: float, rope_scale: float) -> torch.Tensor:
    """Prefill chunk ``q [Lq, Hq, D]``: query i is rotated at position ``(n_local + i) * rope_scale`` and
    rounded to ``q.dtype`` (token_retrieval.py:380-388: ``position_ids = arange(n_local, n_local + Lq)``)."""
    lq = q.shape[0]
    inv_freq = rope_inv_freq(q.shape[-1], rope_base)
    pos = torch.arange(n_local, n_local + lq, dtype=torch.float32) * rope_scale
    cos, sin = rope_cos_sin(pos, inv_freq)                               # [Lq, D]
    return ((q.float() * cos[:, None, :]) + (rotate_half(q).float() * sin[:, None, :])).to(q.dtype)


def chunk_fingerprint(q: torch.Tensor, n_local: int, rope_base: float, rope_scale: float,
                      fixed_order: bool = True) -> torch.Tensor:
    """Scoring query of a prefill chunk: the mean over the chunk of the rotated, rounded queries
    (token_retrieval.py:392, ``torch.mean(query, dim=0)``), ``[Hq, D]`` in ``q.dtype``.  ``fixed_order``
    fixes what torch leaves open: 128 fp32 partial sums (partial s takes queries s, s+128, ... in ascending
    order); lane j of 32 joins its four partials as ``((j + (j+32)) + (j+64)) + (j+96)``; an XOR butterfly
    (16, 8, 4, 2, 1) joins the lanes; one fp32 division by the chunk length, one rounding to the dtype;
    otherwise ``torch.mean`` itself is called."""
    rot = rotate_chunk_queries(q, n_local, rope_base, rope_scale)
    if not fixed_order:
        return torch.mean(rot.view(rot.shape[0], -1), dim=0).view(rot.shape[1:])
    rot32 = rot.float().numpy()
    p128 = np.zeros((128,) + tuple(rot.shape[1:]), dtype=np.float32)
    for i in range(rot.shape[0]):
        p128[i % 128] = p128[i % 128] + rot32[i]
    part = ((p128[0:32] + p128[32:64]) + p128[64:96]) + p128[96:128]
    lanes = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        part = part + part[lanes ^ o]
    return torch.from_numpy(part[0] / np.float32(rot.shape[0])).to(q.dtype)


# --------------------------------------------------------------------------------------
# scoring, soft vote, top-k                                 token_retrieval.py:166-261, 338-373
# --------------------------------------------------------------------------------------
def scoring_kv_head(h: int, hq: int, hkv: int, gqa_map: str) -> int:
    """KV head paired with query head ``h`` while scoring.  The reference uses
    ``h % num_kv_heads`` (token_retrieval.py:202); ``div`` is the conventional ``h // group``."""
    if gqa_map == "mod":
        return h % hkv
    if gqa_map == "div":
        return h // (hq // hkv)
    raise ValueError(gqa_map)


def score_logits(q_rot: torch.Tensor, k_pool: torch.Tensor, slots: torch.Tensor, gqa_map: str = "mod") -> torch.Tensor:
    """``logit[h, t] = sum_d q_rot[h, d] * k_pool[slots[t], kv(h), d]`` in fp32, no scaling
    (token_retrieval.py:195-231).  ``q_rot [Hq, D]``, ``k_pool [rows, Hkv, D]`` -> ``[Hq, Nc]``."""
    hq, _ = q_rot.shape
    hkv = k_pool.shape[1]
    rows = k_pool[slots.long()].float()                      # [Nc, Hkv, D]
    out = torch.empty((hq, rows.shape[0]), dtype=torch.float32)
    qf = q_rot.float()
    for h in range(hq):
        out[h] = rows[:, scoring_kv_head(h, hq, hkv, gqa_map), :] @ qf[h]
    return out


def soft_vote(logits: torch.Tensor, logits_dtype: torch.dtype = torch.float32,
              truncate: bool = False) -> torch.Tensor:
    """Per-head softmax over tokens, summed over heads (token_retrieval.py:361).  With
    ``logits_dtype=bfloat16`` the logits are first narrowed to the reference's bf16 buffer
    (token_retrieval.py:345-347) and every op runs on bf16 tensors as the reference does.
    ``truncate=True`` narrows by dropping the low 16 bits, which is what Triton's CPU interpreter
    does on the store at token_retrieval.py:231 (a compiled Triton kernel rounds to nearest)."""
    if logits_dtype == torch.bfloat16 and truncate:
        logits = (logits.float().contiguous().view(torch.int32) & ~0xFFFF).view(torch.float32)
    return torch.softmax(logits.to(logits_dtype), dim=-1).sum(dim=0)


def max_pool_votes(votes: torch.Tensor, kernel_size: int) -> torch.Tensor:
    """Optional sliding max (token_retrieval.py:366-369).  Even sizes shorten the vector by one."""
    if kernel_size <= 0:
        return votes
    return torch.nn.functional.max_pool1d(
        votes.unsqueeze(0), kernel_size=kernel_size, padding=(kernel_size - 1) // 2, stride=1
    ).squeeze(0)


def topk_sorted(votes: torch.Tensor, k: int, deterministic: bool = True) -> torch.Tensor:
    """Indices of the ``k`` largest votes in ascending order (token_retrieval.py:371-372).
    ``deterministic=True`` breaks exact ties by lowest index (the CUDA path's rule);
    ``False`` calls ``torch.topk`` exactly as the reference does."""
    if deterministic:
        v = votes.float().numpy()
        order = np.argsort(-v, kind="stable")[:k]
        return torch.from_numpy(np.sort(order).astype(np.int64))
    idx = torch.topk(votes, k, dim=-1).indices
    return torch.sort(idx).values


def retrieval_positions(n_tokens: int, n_init: int, n_local: int, topk_cand: torch.Tensor) -> torch.Tensor:
    """``init || top-k || local`` logical positions (token_retrieval.py:429-446)."""
    return torch.cat(
        [torch.arange(0, n_init), topk_cand.long() + n_init, torch.arange(n_tokens - n_local, n_tokens)]
    )


# --------------------------------------------------------------------------------------
# selection cache                                           token_retrieval.py:394-421
# --------------------------------------------------------------------------------------
def cosine_terms_fixed_order(q: np.ndarray, c: np.ndarray) -> np.ndarray:
    """fp32 ``(q.c, |q|^2, |c|^2)`` in the fixed order the CUDA path uses, so that reuse
    decisions can be replayed bit for bit: 32 strided partial sums (element ``j + 32*i`` goes
    to partial ``j``, ascending ``i``, one rounding per multiply and per add), then an XOR
    butterfly over the 32 partials with offsets 16, 8, 4, 2, 1."""
    q = q.astype(np.float32).reshape(-1)
    c = c.astype(np.float32).reshape(-1)
    assert q.size == c.size and q.size % 32 == 0
    q2 = q.reshape(-1, 32)
    c2 = c.reshape(-1, 32)
    acc = np.zeros((3, 32), dtype=np.float32)
    for i in range(q2.shape[0]):
        acc[0] = acc[0] + q2[i] * c2[i]
        acc[1] = acc[1] + q2[i] * q2[i]
        acc[2] = acc[2] + c2[i] * c2[i]
    lanes = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        acc = acc + acc[:, lanes ^ off]
    return acc[:, 0].copy()


def cosine_terms_fixed_order_batch(q: np.ndarray, c: np.ndarray) -> np.ndarray:
    """:func:`cosine_terms_fixed_order` for a batch of (query, cached query) pairs ``[B, n]`` at once (same
    order of operations per pair, hence the same bits); returns ``[B, 3]``.  Used to replay the reuse
    decisions of many layers per step (token_retrieval.py:394-421 keeps one cached query per layer)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    c = np.ascontiguousarray(c, dtype=np.float32)
    assert q.shape == c.shape and q.ndim == 2 and q.shape[1] % 32 == 0
    bsz = q.shape[0]
    q2 = q.reshape(bsz, -1, 32)
    c2 = c.reshape(bsz, -1, 32)
    acc = np.zeros((3, bsz, 32), dtype=np.float32)
    for i in range(q2.shape[1]):
        acc[0] = acc[0] + q2[:, i] * c2[:, i]
        acc[1] = acc[1] + q2[:, i] * q2[:, i]
        acc[2] = acc[2] + c2[:, i] * c2[:, i]
    lanes = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        acc = acc + acc[:, :, lanes ^ off]
    return np.ascontiguousarray(acc[:, :, 0].T)


def cosine_from_terms(terms: np.ndarray) -> np.float32:
    """``dot / (sqrt(qq) * sqrt(cc))`` with every operation rounded to fp32."""
    dot, qq, cc = (np.float32(t) for t in terms)
    den = np.float32(np.sqrt(qq) * np.sqrt(cc))
    if den == np.float32(0):
        return np.float32(0)
    return np.float32(dot / den)


def cache_says_recompute(cos: np.float32, theta: float) -> bool:
    """Strict ``<`` as in token_retrieval.py:397-400, threshold held in fp32."""
    return bool(np.float32(cos) < np.float32(theta))


# --------------------------------------------------------------------------------------
# sparse paged decode attention                             token_retrieval.py:815-825
# --------------------------------------------------------------------------------------
def sparse_attention(
    q: torch.Tensor,          # [Hq, D] un-rotated
    k_pool: torch.Tensor,     # [rows, Hkv, D]
    v_pool: torch.Tensor,     # [rows, Hkv, D]
    slots: torch.Tensor,      # [n] pool rows in list order
    sm_scale: float,
    rope_base: float,
    rope_scale: float = 1.0,
    logit_cap: float = 0.0,
    compute_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """Decode attention over ``slots`` as the reference's third-party decode wrapper computes it
    in its Llama-RoPE mode (call site token_retrieval.py:815-823): the query is rotated at
    position ``n-1``, the j-th listed key at position ``j``, rotate-half pairing, frequencies
    divided by ``rope_scale``; logits times ``sm_scale``; soft-cap ``cap*tanh(x/cap)`` only when
    ``cap > 0``; softmax; values un-rotated; KV head ``h // group``.  Returns ``[Hq, D]`` in
    ``compute_dtype`` (fp32 by default; fp64 gives the truth used for tolerance checks)."""
    hq, d = q.shape
    hkv = k_pool.shape[1]
    group = hq // hkv
    n = slots.numel()
    inv_freq = rope_inv_freq(d, rope_base) / rope_scale
    kpos = torch.arange(n, dtype=torch.float32)
    qpos = torch.tensor([n - 1], dtype=torch.float32)
    if compute_dtype == torch.float64:
        inv64 = inv_freq.double()
        fk = torch.outer(kpos.double(), inv64)
        fq = torch.outer(qpos.double(), inv64)
        cos_k, sin_k = torch.cat((fk, fk), -1).cos(), torch.cat((fk, fk), -1).sin()
        cos_q, sin_q = torch.cat((fq, fq), -1).cos(), torch.cat((fq, fq), -1).sin()
    else:
        cos_k, sin_k = rope_cos_sin(kpos, inv_freq)
        cos_q, sin_q = rope_cos_sin(qpos, inv_freq)
    qf = q.to(compute_dtype)
    q_rot = qf * cos_q.to(compute_dtype) + rotate_half(qf) * sin_q.to(compute_dtype)          # [Hq, D]
    ks = k_pool[slots.long()].to(compute_dtype)                                              # [n, Hkv, D]
    vs = v_pool[slots.long()].to(compute_dtype)
    k_rot = ks * cos_k.to(compute_dtype)[:, None, :] + rotate_half(ks) * sin_k.to(compute_dtype)[:, None, :]
    out = torch.empty((hq, d), dtype=compute_dtype)
    for h in range(hq):
        kv = h // group
        s = (k_rot[:, kv, :] @ q_rot[h]) * sm_scale
        if logit_cap > 0:
            s = logit_cap * torch.tanh(s / logit_cap)
        p = torch.softmax(s, dim=0)
        out[h] = p @ vs[:, kv, :]
    return out


def sparse_prefill_attention(
    q: torch.Tensor,          # [Lq, Hq, D] un-rotated queries of the chunk (the last Lq tokens of the list)
    k_pool: torch.Tensor,     # [rows, Hkv, D]
    v_pool: torch.Tensor,
    slots: torch.Tensor,      # [n] pool rows in list order; the chunk's own rows are the last Lq
    sm_scale: float,
    rope_base: float,
    rope_scale: float = 1.0,
    logit_cap: float = 0.0,
    compute_dtype: torch.dtype = torch.float32,
    operand_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Causal attention of a prefill chunk over ``slots`` as the reference's third-party paged prefill
    wrapper computes it in its Llama-RoPE mode with ``causal=True`` (call site
    token_retrieval.py:746-772): with ``n`` listed keys and ``Lq`` queries, query i sits at position
    ``n - Lq + i`` and sees the listed keys ``j <= n - Lq + i``; key j is rotated at position j; the
    rest as in :func:`sparse_attention`.  Returns ``[Lq, Hq, D]``.  ``operand_dtype`` (e.g. bf16) rounds the
    rotated queries and keys to that type before the dot products, which is what the library's tensor-core
    prefill kernel does with bf16 inputs; ``None`` keeps them exact (the truth used for tolerances)."""
    lq, hq, d = q.shape
    hkv = k_pool.shape[1]
    group = hq // hkv
    n = slots.numel()
    inv_freq = rope_inv_freq(d, rope_base) / rope_scale
    kpos = torch.arange(n, dtype=torch.float32)
    qpos = torch.arange(n - lq, n, dtype=torch.float32)
    if compute_dtype == torch.float64:
        inv64 = inv_freq.double()
        fk, fq = torch.outer(kpos.double(), inv64), torch.outer(qpos.double(), inv64)
        cos_k, sin_k = torch.cat((fk, fk), -1).cos(), torch.cat((fk, fk), -1).sin()
        cos_q, sin_q = torch.cat((fq, fq), -1).cos(), torch.cat((fq, fq), -1).sin()
    else:
        cos_k, sin_k = rope_cos_sin(kpos, inv_freq)
        cos_q, sin_q = rope_cos_sin(qpos, inv_freq)
    qf = q.to(compute_dtype)
    q_rot = qf * cos_q.to(compute_dtype)[:, None, :] + rotate_half(qf) * sin_q.to(compute_dtype)[:, None, :]
    ks = k_pool[slots.long()].to(compute_dtype)
    vs = v_pool[slots.long()].to(compute_dtype)
    k_rot = ks * cos_k.to(compute_dtype)[:, None, :] + rotate_half(ks) * sin_k.to(compute_dtype)[:, None, :]
    if operand_dtype is not None:
        q_rot = q_rot.float().to(operand_dtype).to(compute_dtype)
        k_rot = k_rot.float().to(operand_dtype).to(compute_dtype)
    visible = torch.arange(n)[None, :] <= (n - lq + torch.arange(lq))[:, None]       # [Lq, n]
    out = torch.empty((lq, hq, d), dtype=compute_dtype)
    for h in range(hq):
        kv = h // group
        s = (q_rot[:, h, :] @ k_rot[:, kv, :].T) * sm_scale                           # [Lq, n]
        if logit_cap > 0:
            s = logit_cap * torch.tanh(s / logit_cap)
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=1) @ vs[:, kv, :]
    return out


# --------------------------------------------------------------------------------------
# whole decode layer for a ragged batch, with per-request state
# --------------------------------------------------------------------------------------
@dataclasses.dataclass
class OracleConfig:
    n_layers: int
    hq: int                       # query heads on this rank (all heads when tp == 1)
    hkv: int                      # KV heads on this rank
    head_dim: int
    n_init: int
    n_local: int
    top_k: int
    rope_base: float
    rope_scale: float = 1.0
    similarity_threshold: float = 0.9
    query_cache: bool = False     # the reference ships with it off (token_retrieval.py:918)
    gqa_map: str = "mod"
    kernel_size: int = -1
    sm_scale: Optional[float] = None
    logit_cap: float = 0.0
    logits_dtype: torch.dtype = torch.float32
    logits_truncate: bool = False     # reproduce the Triton interpreter's bf16 narrowing
    deterministic_topk: bool = True

    @property
    def n_sel(self) -> int:
        return self.n_init + self.top_k + self.n_local


@dataclasses.dataclass
class _CacheEntry:
    valid: bool = False
    fingerprint: Optional[np.ndarray] = None     # fp32 copy of the rounded scoring query
    topk_positions: Optional[torch.Tensor] = None  # logical positions (already + n_init)


class DecodeOracle:
    """Per-request decode state and one-layer step (token_retrieval.py:264-449, 777-825).

    ``tp_ranks`` > 1 emulates KV-head tensor parallelism: query and KV heads are split into
    contiguous groups, each group scores with its *local* head map (token_retrieval.py:357, :462),
    the vote vectors are summed (token_retrieval.py:363-364) and every group attends with its own
    heads over the common index set."""

    def __init__(self, cfg: OracleConfig, tp_ranks: int = 1):
        self.cfg = cfg
        self.tp = tp_ranks
        self.cache: Dict[Tuple[int, int], _CacheEntry] = {}
        self.retrieval_count: Dict[int, int] = {}
        self.skip_count: Dict[int, int] = {}

    def reset_request(self, req_slot: int) -> None:
        """A new request id gets fresh state (token_retrieval.py:147-163, :322-327)."""
        for key in [k for k in self.cache if k[0] == req_slot]:
            del self.cache[key]
        self.retrieval_count[req_slot] = 0
        self.skip_count[req_slot] = 0

    # -- votes over candidates of one request ------------------------------------------------
    def votes(self, q_rot: torch.Tensor, k_pool: torch.Tensor, cand_slots: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        total = None
        hq_r, hkv_r = cfg.hq // self.tp, cfg.hkv // self.tp
        for r in range(self.tp):
            lg = score_logits(
                q_rot[r * hq_r:(r + 1) * hq_r], k_pool[:, r * hkv_r:(r + 1) * hkv_r, :], cand_slots, cfg.gqa_map
            )
            v = soft_vote(lg, cfg.logits_dtype, cfg.logits_truncate)
            total = v if total is None else total + v
        return total

    # -- selection for one request -----------------------------------------------------------
    def select(self, layer: int, req_slot: int, q: torch.Tensor, k_pool: torch.Tensor,
               slot_row: torch.Tensor, n_tokens: int,
               scoring_query: Optional[torch.Tensor] = None) -> Tuple[int, torch.Tensor, dict]:
        """Returns ``(flag, logical positions, info)`` for one request (token_retrieval.py:375-449).
        ``q [Hq, D]`` un-rotated; ``slot_row`` is the request's row of the position->slot map.  A prefill
        chunk passes its fingerprint as ``scoring_query`` (already rotated and averaged, :380-392)."""
        cfg = self.cfg
        info: dict = {}
        if cfg.n_sel >= n_tokens:                                   # :376-378
            return FLAG_DENSE, torch.arange(n_tokens), info
        if scoring_query is not None:
            q_rot = scoring_query
        else:
            q_rot = rotate_scoring_query(q, cfg.n_local, cfg.rope_base, cfg.rope_scale)   # :380-388
        info["q_rot"] = q_rot
        recompute = True
        entry = self.cache.setdefault((req_slot, layer), _CacheEntry())
        if cfg.query_cache:
            self.retrieval_count[req_slot] = self.retrieval_count.get(req_slot, 0) + 1   # :421
            if entry.valid:
                hq_r = cfg.hq // self.tp
                terms = np.zeros(3, dtype=np.float32)
                for r in range(self.tp):     # per-rank partial sums, then summed like an all-reduce
                    sl = slice(r * hq_r, (r + 1) * hq_r)
                    terms = terms + cosine_terms_fixed_order(
                        q_rot[sl].float().numpy(), entry.fingerprint[sl])
                cos = cosine_from_terms(terms)
                info["cos"] = float(cos)
                recompute = cache_says_recompute(cos, cfg.similarity_threshold)   # :396-400
        if recompute:
            cand_slots = slot_row[cfg.n_init: n_tokens - cfg.n_local]             # :424-426
            v = self.votes(q_rot, k_pool, cand_slots)
            v = max_pool_votes(v, cfg.kernel_size)                                # :366-369
            info["votes"] = v
            topk_cand = topk_sorted(v, cfg.top_k, cfg.deterministic_topk)         # :371-372
            topk_pos = topk_cand.long() + cfg.n_init                              # :433
            if cfg.query_cache:                                                   # :415-417
                entry.valid = True
                entry.fingerprint = q_rot.float().numpy().copy()
                entry.topk_positions = topk_pos.clone()
            flag = FLAG_RECOMPUTE
        else:
            topk_pos = entry.topk_positions                                       # :419
            self.skip_count[req_slot] = self.skip_count.get(req_slot, 0) + 1      # :420
            flag = FLAG_REUSE
        pos = torch.cat([torch.arange(0, cfg.n_init), topk_pos,
                         torch.arange(n_tokens - cfg.n_local, n_tokens)])         # :436-446
        return flag, pos, info

    # -- one layer, ragged batch ----------------------------------------------------------------
    def decode_layer(self, layer: int, q: torch.Tensor, k_new: Optional[torch.Tensor],
                     v_new: Optional[torch.Tensor], out_cache_loc: Optional[torch.Tensor],
                     k_pool: torch.Tensor, v_pool: torch.Tensor, req_to_token: torch.Tensor,
                     req_pool_indices: torch.Tensor, seq_lens: torch.Tensor,
                     attn_dtype: torch.dtype = torch.float32) -> dict:
        """One decode step of one layer (token_retrieval.py:777-825).  ``q [bs, Hq*D]``;
        ``k_new, v_new [bs, Hkv*D]`` are written to the pools at ``out_cache_loc`` first
        (token_retrieval.py:844-850); ``seq_lens`` count the token being decoded."""
        cfg = self.cfg
        bs = q.shape[0]
        if k_new is not None:
            k_pool[out_cache_loc.long()] = k_new.view(bs, cfg.hkv, cfg.head_dim).to(k_pool.dtype)
            v_pool[out_cache_loc.long()] = v_new.view(bs, cfg.hkv, cfg.head_dim).to(v_pool.dtype)
        sm_scale = cfg.sm_scale if cfg.sm_scale is not None else cfg.head_dim ** -0.5
        outs, flags, positions, slots_out, infos = [], [], [], [], []
        for b in range(bs):
            n = int(seq_lens[b])
            row = req_to_token[int(req_pool_indices[b])]
            qb = q[b].view(cfg.hq, cfg.head_dim)
            flag, pos, info = self.select(layer, int(req_pool_indices[b]), qb, k_pool, row, n)
            sl = row[pos.long()]                                                 # :448
            hq_r, hkv_r = cfg.hq // self.tp, cfg.hkv // self.tp
            o = torch.cat([
                sparse_attention(qb[r * hq_r:(r + 1) * hq_r], k_pool[:, r * hkv_r:(r + 1) * hkv_r],
                                 v_pool[:, r * hkv_r:(r + 1) * hkv_r], sl, sm_scale, cfg.rope_base,
                                 cfg.rope_scale, cfg.logit_cap, attn_dtype)
                for r in range(self.tp)], dim=0)
            outs.append(o.reshape(-1))
            flags.append(flag)
            positions.append(pos)
            slots_out.append(sl)
            infos.append(info)
        return {"out": torch.stack(outs), "flags": flags, "positions": positions,
                "slots": slots_out, "info": infos}


    # -- one prefill chunk of one request ------------------------------------------------------------
    def extend_chunk(self, layer: int, req_slot: int, q: torch.Tensor, k_new: Optional[torch.Tensor],
                     v_new: Optional[torch.Tensor], out_cache_loc: Optional[torch.Tensor],
                     k_pool: torch.Tensor, v_pool: torch.Tensor, slot_row: torch.Tensor, n_tokens: int,
                     attn_dtype: torch.dtype = torch.float32,
                     scoring_query: Optional[torch.Tensor] = None) -> dict:
        """One chunk (at most 512 tokens, token_retrieval.py:716-724, :917) of a prefill, one layer
        (:726-775).  ``q [Lq, Hq*D]``; the chunk's K/V rows are stored first (:726-734) and
        ``n_tokens`` counts them; selection uses the chunk's fingerprint (:736-738, :392); a request
        with ``n_sel >= n_tokens`` attends to all its tokens (:741-744); causal attention over the
        list (:760-772)."""
        cfg = self.cfg
        lq = q.shape[0]
        if k_new is not None:
            k_pool[out_cache_loc.long()] = k_new.view(lq, cfg.hkv, cfg.head_dim).to(k_pool.dtype)
            v_pool[out_cache_loc.long()] = v_new.view(lq, cfg.hkv, cfg.head_dim).to(v_pool.dtype)
        qh = q.view(lq, cfg.hq, cfg.head_dim)
        fp = scoring_query if scoring_query is not None else \
            chunk_fingerprint(qh, cfg.n_local, cfg.rope_base, cfg.rope_scale)
        flag, pos, info = self.select(layer, req_slot, None, k_pool, slot_row, n_tokens, scoring_query=fp)
        info["fingerprint"] = fp
        sl = slot_row[pos.long()]
        sm_scale = cfg.sm_scale if cfg.sm_scale is not None else cfg.head_dim ** -0.5
        hq_r, hkv_r = cfg.hq // self.tp, cfg.hkv // self.tp
        o = torch.cat([
            sparse_prefill_attention(qh[:, r * hq_r:(r + 1) * hq_r], k_pool[:, r * hkv_r:(r + 1) * hkv_r],
                                     v_pool[:, r * hkv_r:(r + 1) * hkv_r], sl, sm_scale, cfg.rope_base,
                                     cfg.rope_scale, cfg.logit_cap, attn_dtype)
            for r in range(self.tp)], dim=1)
        return {"out": o.reshape(lq, -1), "flag": flag, "positions": pos, "slots": sl, "info": info}


# --------------------------------------------------------------------------------------
# parity rule for index sets
# --------------------------------------------------------------------------------------
def index_sets_match(got: np.ndarray, want: np.ndarray, votes: np.ndarray, k: int,
                     rel_tol: float = 1e-4) -> Tuple[bool, str]:
    """Selected candidate sets must be equal, except that an index in the symmetric difference is
    accepted when its vote lies within ``rel_tol`` (relative) of the k-th largest vote.
    ``got``/``want`` are candidate indices (into ``votes``)."""
    got_s, want_s = set(int(x) for x in got), set(int(x) for x in want)
    if len(got_s) != len(got) or len(got_s) != k:
        return False, f"selection has {len(got_s)} unique of {len(got)}; expected {k}"
    diff = got_s ^ want_s
    if not diff:
        return True, "identical"
    v = votes.astype(np.float64)
    kth = np.sort(v)[::-1][k - 1]
    bad = [i for i in diff if abs(v[i] - kth) > rel_tol * max(abs(kth), 1e-300)]
    if bad:
        return False, f"{len(bad)} of {len(diff)} differing indices lie outside the tie band (kth={kth:.6e})"
    return True, f"{len(diff)} differing indices, all inside the tie band"
