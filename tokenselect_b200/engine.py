"""Host side of the decode-time selection + sparse attention path.

``TokenSelectEngine`` owns one C-ABI handle (workspace + per-request selection cache on one GPU) and
turns torch tensors into ``ts_decode_args``.  It plays the role of the reference's
``ReqToTokenRetriever`` / ``TokenRetriever`` pair (patcher/token_retrieval.py:117-163, :264-449)
together with the decode branch of the patched attention forward (:777-825); all arithmetic runs in
the CUDA library.  There is no fallback path: without the library or without a GPU, construction fails.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Dict, Optional, Sequence

import torch

from . import _lib
from ._lib import TsExtendArgs, TsConfig, TsDecodeArgs, check


@dataclasses.dataclass
class TokenSelectConfig:
    """Knobs.  The first block keeps the reference's YAML / ``patch()`` names
    (config/*.yaml ``model.*``, token_retrieval.py:885-894)."""
    rope_base: float = 1e6
    rope_scale: float = 1.0
    rope_model: str = "ROPE_LLAMA"
    max_n_tokens: int = 1048576
    top_k: int = 2048
    n_init: int = 128
    n_local: int = 512
    kernel_size: int = -1
    # constants of the reference made explicit
    query_cache: bool = False              # QUERY_CACHE, hard-wired off at :918
    similarity_threshold: float = 0.9      # :313-315, held in fp32 here
    gqa_map: str = "mod"                   # scoring pairs head h with KV head h % Hkv (:202)
    # model geometry of this tensor-parallel rank
    n_layers: int = 32
    num_q_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    dtype: torch.dtype = torch.bfloat16
    sm_scale: Optional[float] = None       # RadixAttention.scaling (:818)
    logit_cap: float = 0.0                 # RadixAttention.logit_cap (:819)
    # capacity
    max_reqs: int = 8                      # rows of req_to_token
    max_batch: int = 8
    max_total_tokens: Optional[int] = None  # sum of sequence lengths in one batch
    tp_rank: int = 0
    tp_size: int = 1
    plain_score: bool = False              # diagnostic: plain-load scoring kernel for bf16 too
    score_path: str = "auto"               # "auto" | "direct" (keys to registers) | "staged" (bulk copies to smem)
    tp_fused: bool = True                  # tp_size > 1: sum the votes inside the kernel through peer memory
    prefill_chunk: int = 512               # PREFILL_CHUNK_SIZE (:917); 0: no prefill workspace
    extra_flags: int = 0                   # further TS_CFG_* diagnostic bits, passed through
    wait_limit_us: int = 0                 # bound of every device-side wait in microseconds; 0: one second

    @property
    def n_sel(self) -> int:
        return self.n_init + self.top_k + self.n_local

    @classmethod
    def from_yaml(cls, path: str, **overrides) -> "TokenSelectConfig":
        """Read the ``model:`` block of a reference-style YAML file (config/llama-token-retrieval.yaml)."""
        import yaml
        with open(path) as f:
            model = (yaml.safe_load(f) or {}).get("model", {})
        names = {f.name for f in dataclasses.fields(cls)}
        kw = {k: v for k, v in model.items() if k in names}
        kw.update(overrides)
        return cls(**kw)


def rotary_tables(cfg: TokenSelectConfig):
    """cos/sin tables built on the host exactly as the reference's RotaryEmbedding builds them
    (token_retrieval.py:73-96): fp32 inverse frequencies, fp32 outer product with the positions.
    Returns ``(score [D/2, 2], attn [n_sel+1, D/2, 2])``: the scoring query sits at position
    ``n_local * rope_scale`` (:93, :380-388); attention positions 0..n_sel use frequencies divided by
    ``rope_scale`` (:820-822)."""
    d = cfg.head_dim
    inv_freq = 1.0 / (cfg.rope_base ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang_s = torch.outer(torch.tensor([cfg.n_local * cfg.rope_scale], dtype=torch.float32), inv_freq)[0]
    score = torch.stack((ang_s.cos(), ang_s.sin()), dim=-1).contiguous()
    ang_a = torch.outer(torch.arange(cfg.n_sel + 1, dtype=torch.float32), inv_freq / cfg.rope_scale)
    attn = torch.stack((ang_a.cos(), ang_a.sin()), dim=-1).contiguous()
    return score, attn


def chunk_rotary_table(cfg: TokenSelectConfig) -> torch.Tensor:
    """cos/sin of the positions a prefill chunk's queries are rotated at before they are averaged into
    the chunk's fingerprint: ``position_ids = arange(n_local, n_local + Lq)`` times ``rope_scale``
    (token_retrieval.py:380-388 with :92-96).  ``[prefill_chunk, D/2, 2]`` fp32, built with the same torch
    expressions as :func:`rotary_tables`."""
    d = cfg.head_dim
    inv_freq = 1.0 / (cfg.rope_base ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    pos = torch.arange(cfg.n_local, cfg.n_local + cfg.prefill_chunk, dtype=torch.float32) * cfg.rope_scale
    ang = torch.outer(pos, inv_freq)
    return torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class TokenSelectEngine:
    """One handle of the CUDA library on the current device."""

    def __init__(self, cfg: TokenSelectConfig, device: Optional[torch.device] = None,
                 process_group=None):
        if not torch.cuda.is_available():
            raise RuntimeError("tokenselect_b200 needs a CUDA device; there is no CPU path")
        self.lib = _lib.load()
        self.cfg = cfg
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.group = process_group
        if cfg.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be bfloat16 or float32")
        max_total = cfg.max_total_tokens or cfg.max_batch * cfg.max_n_tokens
        score_cs, attn_cs = rotary_tables(cfg)
        self._tables = (score_cs, attn_cs)        # keep the host memory alive during ts_create
        c = TsConfig()
        c.struct_size = C.sizeof(TsConfig)
        c.device = self.device.index or 0
        c.n_layers, c.hq, c.hkv, c.head_dim = cfg.n_layers, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        c.dtype = _lib.TS_DTYPE_BF16 if cfg.dtype == torch.bfloat16 else _lib.TS_DTYPE_F32
        c.n_init, c.n_local, c.top_k, c.kernel_size = cfg.n_init, cfg.n_local, cfg.top_k, cfg.kernel_size
        c.query_cache = 1 if cfg.query_cache else 0
        c.similarity_threshold = cfg.similarity_threshold
        c.gqa_map = {"mod": _lib.TS_GQA_MOD, "div": _lib.TS_GQA_DIV}[cfg.gqa_map]
        c.rope_base, c.rope_scale = float(cfg.rope_base), float(cfg.rope_scale)
        c.sm_scale = cfg.sm_scale if cfg.sm_scale is not None else cfg.head_dim ** -0.5
        c.logit_cap = cfg.logit_cap
        c.max_reqs, c.max_batch, c.max_ctx = cfg.max_reqs, cfg.max_batch, cfg.max_n_tokens
        c.max_total_tokens = max_total
        c.tp_rank, c.tp_size = cfg.tp_rank, cfg.tp_size
        c.flags = (_lib.TS_CFG_PLAIN_SCORE if cfg.plain_score else 0) | {"auto": 0, "direct": 2, "staged": 4}[cfg.score_path] | int(cfg.extra_flags)
        c.prefill_chunk = int(cfg.prefill_chunk) if (cfg.tp_size == 1 or (cfg.tp_fused and not cfg.query_cache)) else 0
        c.wait_limit_us = int(cfg.wait_limit_us)
        c.score_cos_sin = score_cs.data_ptr()
        c.attn_cos_sin = attn_cs.data_ptr()
        self._c = c
        ws = C.c_size_t()
        check(self.lib.ts_query_workspace(C.byref(c), C.byref(ws)), "ts_query_workspace")
        self.workspace_bytes = ws.value
        ve = C.c_int64()
        check(self.lib.ts_vote_buffer_elems(C.byref(c), C.byref(ve)), "ts_vote_buffer_elems")
        self.vote_elems = ve.value
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(self.lib.ts_create(C.byref(c), C.byref(self._h)), "ts_create")
        self.tp_votes = self.tp_cos = None
        self.fused_tp = False
        self.chunk_cs = chunk_rotary_table(cfg).to(self.device) if c.prefill_chunk > 0 else None
        if cfg.tp_size > 1:
            self.tp_votes = torch.zeros(self.vote_elems, dtype=torch.float32, device=self.device)
            self.tp_cos = torch.zeros(cfg.max_batch * 4, dtype=torch.float32, device=self.device)
            if cfg.tp_fused and not cfg.query_cache:
                self._attach_peers()
        self._rids: Dict[int, object] = {}

    def _attach_peers(self) -> None:
        """Give the library every rank's exchange buffer (torch symmetric memory over NVLink) so that the
        selection kernel can sum the ranks' votes itself instead of the host calling all_reduce between
        two kernels (token_retrieval.py:363-364).  Needs an initialised NCCL process group."""
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized():
            return
        import torch.distributed._symmetric_memory as symm_mem
        group = self.group if self.group is not None else dist.group.WORLD
        self._symm = symm_mem.empty(self.symmetric_bytes(), dtype=torch.uint8, device=self.device)
        self._symm.zero_()
        handle = symm_mem.rendezvous(self._symm, group)
        ptrs = [int(x) for x in handle.buffer_ptrs]
        if len(ptrs) != self.cfg.tp_size or handle.rank != self.cfg.tp_rank:
            raise RuntimeError("symmetric-memory group does not match tp_rank / tp_size")
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)                 # every buffer is zeroed before anyone raises a flag
        self.attach_peer_buffers(ptrs)
        self._symm_handle = handle

    def symmetric_bytes(self) -> int:
        """Bytes of peer-visible, zero-filled memory every rank provides for the in-kernel vote exchange."""
        nbytes = C.c_size_t()
        check(self.lib.ts_tp_symmetric_bytes(C.byref(self._c), C.byref(nbytes)), "ts_tp_symmetric_bytes")
        return nbytes.value

    def attach_peer_buffers(self, ptrs: Sequence[int]) -> None:
        """Hand the library the device addresses of ALL ranks' exchange buffers, in rank order
        (``ts_tp_attach_peers``); from then on ``decode_layer`` sums the votes inside the selection kernel."""
        arr = (C.c_uint64 * len(ptrs))(*[int(x) for x in ptrs])
        check(self.lib.ts_tp_attach_peers(self._h, arr, len(ptrs)), "ts_tp_attach_peers", self._h)
        self.fused_tp = True

    # ------------------------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self.lib.ts_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------------------------------
    def bind_requests(self, rids: Sequence[object], req_pool_indices: Sequence[int]) -> None:
        """Tell the engine which request id occupies which request slot.  A slot whose id changed
        gets fresh selection-cache state, as a new ``rid`` gets a fresh TokenRetriever in the
        reference (token_retrieval.py:147-163)."""
        for rid, slot in zip(rids, req_pool_indices):
            slot = int(slot)
            if self._rids.get(slot, None) != rid:
                self._rids[slot] = rid
                self.reset_request(slot)

    def reset_request(self, req_slot: int) -> None:
        check(self.lib.ts_reset_request(self._h, int(req_slot), self._stream()), "ts_reset_request", self._h)

    def counters(self, req_slot: int):
        """(retrieval_count, skip_count) of a request slot (token_retrieval.py:150-161)."""
        a, b = C.c_uint64(), C.c_uint64()
        check(self.lib.ts_get_counters(self._h, int(req_slot), C.byref(a), C.byref(b), self._stream()),
              "ts_get_counters", self._h)
        return a.value, b.value

    def last_error(self):
        code, detail = C.c_int32(), C.c_int32()
        check(self.lib.ts_last_error(self._h, C.byref(code), C.byref(detail)), "ts_last_error", self._h)
        return code.value, detail.value

    def raise_on_device_error(self) -> None:
        code, detail = self.last_error()
        if code != 0:
            raise _lib.TokenSelectError(code, "device-side error", f"detail={detail}")

    @property
    def launch_count(self) -> int:
        n = C.c_uint64()
        check(self.lib.ts_launch_count(self._h, C.byref(n)), "ts_launch_count")
        return n.value

    STAGES = ("prepare", "select", "select_tp_b", "attend_split", "attend_merge", "extend_prep", "extend_gather",
              "extend_attend")

    def timing_begin(self, max_launches: int = 65536) -> None:
        """Record a CUDA-event pair around every kernel of this handle until ``timing_end``."""
        check(self.lib.ts_timing_begin(self._h, int(max_launches)), "ts_timing_begin", self._h)

    def timing_end(self) -> dict:
        """``{stage: (total_ms, launches)}`` since ``timing_begin`` (synchronises the device)."""
        ms = (C.c_double * 8)()
        n = (C.c_uint64 * 8)()
        check(self.lib.ts_timing_end(self._h, ms, n), "ts_timing_end", self._h)
        return {name: (ms[i], n[i]) for i, name in enumerate(self.STAGES)}

    def debug_read(self, which: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(numel, dtype=dtype)
        check(self.lib.ts_debug_read(self._h, which, out.data_ptr(), out.numel() * out.element_size()),
              "ts_debug_read", self._h)
        return out

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    # ------------------------------------------------------------------------------------------
    def _args(self, layer, q, k_new, v_new, out_cache_loc, k_pool, v_pool, req_to_token,
              req_pool_indices, seq_lens, out, debug) -> TsDecodeArgs:
        cfg = self.cfg
        bs = q.shape[0]
        hd = cfg.num_q_heads * cfg.head_dim
        kd = cfg.num_kv_heads * cfg.head_dim
        for name, t, dt in (("q", q, cfg.dtype), ("k_pool", k_pool, cfg.dtype), ("v_pool", v_pool, cfg.dtype),
                            ("req_to_token", req_to_token, torch.int32),
                            ("req_pool_indices", req_pool_indices, torch.int32),
                            ("seq_lens", seq_lens, torch.int32), ("out", out, cfg.dtype)):
            if not t.is_cuda or t.dtype != dt:
                raise ValueError(f"{name}: expected a CUDA tensor of {dt}, got {t.device} {t.dtype}")
        if q.numel() != bs * hd or not q.is_contiguous() or not out.is_contiguous() or out.numel() != bs * hd:
            raise ValueError("q/out must be contiguous [batch, num_q_heads*head_dim]")
        if not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.shape != v_pool.shape:
            raise ValueError("pools must be contiguous [rows, num_kv_heads, head_dim] of equal shape")
        if k_pool[0].numel() != kd:
            raise ValueError("pool row size does not match num_kv_heads*head_dim")
        if req_to_token.dim() != 2 or req_to_token.stride(1) != 1:
            raise ValueError("req_to_token must be [max_reqs, max_ctx] with unit inner stride")
        a = TsDecodeArgs()
        a.struct_size = C.sizeof(TsDecodeArgs)
        a.layer, a.batch = int(layer), int(bs)
        a.q = q.data_ptr()
        if k_new is not None:
            for name, t in (("k", k_new), ("v", v_new)):
                if not t.is_cuda or t.dtype != cfg.dtype or not t.is_contiguous() or t.numel() != bs * kd:
                    raise ValueError(f"{name}: expected contiguous CUDA [batch, num_kv_heads*head_dim] {cfg.dtype}")
            if out_cache_loc is None or out_cache_loc.dtype != torch.int32 or not out_cache_loc.is_cuda:
                raise ValueError("out_cache_loc must be a CUDA int32 tensor")
            a.k_new, a.v_new, a.out_cache_loc = k_new.data_ptr(), v_new.data_ptr(), out_cache_loc.data_ptr()
        a.k_pool, a.v_pool, a.pool_rows = k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0]
        a.req_to_token, a.req_to_token_stride = req_to_token.data_ptr(), req_to_token.stride(0)
        a.req_pool_indices, a.seq_lens = req_pool_indices.data_ptr(), seq_lens.data_ptr()
        a.out = out.data_ptr()
        a.tp_votes, a.tp_cos = _ptr(self.tp_votes), _ptr(self.tp_cos)
        if debug is not None:                      # any subset of the four inspection outputs
            a.dbg_sel_slots = _ptr(debug.get("slots"))
            a.dbg_sel_pos = _ptr(debug.get("positions"))
            a.dbg_sel_count = _ptr(debug.get("count"))
            a.dbg_flags = _ptr(debug.get("flags"))
        a.stream = self._stream()
        return a

    def new_debug_buffers(self, batch: int) -> dict:
        n = self.cfg.n_sel
        z = lambda *s: torch.zeros(*s, dtype=torch.int32, device=self.device)  # noqa: E731
        return {"slots": z(batch, n), "positions": z(batch, n), "count": z(batch), "flags": z(batch)}

    def decode_layer(self, layer: int, q: torch.Tensor, k_new: Optional[torch.Tensor],
                     v_new: Optional[torch.Tensor], out_cache_loc: Optional[torch.Tensor],
                     k_pool: torch.Tensor, v_pool: torch.Tensor, req_to_token: torch.Tensor,
                     req_pool_indices: torch.Tensor, seq_lens: torch.Tensor,
                     out: Optional[torch.Tensor] = None, debug: Optional[dict] = None,
                     vote_elems: Optional[int] = None) -> torch.Tensor:
        """One decode step of one layer for a ragged batch: append ``k_new, v_new`` at
        ``out_cache_loc`` (token_retrieval.py:844-854), select (:375-449), attend (:815-825).
        ``seq_lens`` count the token being decoded.  Enqueues on the current stream; no host sync.
        With ``tp_size > 1`` the fp32 vote vector (and the three cosine terms when the selection cache
        is on) are all-reduced over ``process_group`` between the library's three stages
        (:363-364); ``vote_elems`` bounds the reduced prefix (default: the whole buffer)."""
        if out is None:
            out = torch.empty_like(q)
        a = self._args(layer, q, k_new, v_new, out_cache_loc, k_pool, v_pool, req_to_token,
                       req_pool_indices, seq_lens, out, debug)
        if self.cfg.tp_size == 1 or self.fused_tp:
            check(self.lib.ts_decode_layer(self._h, C.byref(a)), "ts_decode_layer", self._h)
            return out
        import torch.distributed as dist
        check(self.lib.ts_tp_prepare(self._h, C.byref(a)), "ts_tp_prepare", self._h)
        if self.cfg.query_cache:
            dist.all_reduce(self.tp_cos[: 4 * q.shape[0]], op=dist.ReduceOp.SUM, group=self.group)
        check(self.lib.ts_tp_score_vote(self._h, C.byref(a)), "ts_tp_score_vote", self._h)
        n = self.vote_elems if vote_elems is None else min(int(vote_elems), self.vote_elems)
        dist.all_reduce(self.tp_votes[:n], op=dist.ReduceOp.SUM, group=self.group)
        check(self.lib.ts_tp_select_attend(self._h, C.byref(a)), "ts_tp_select_attend", self._h)
        return out

    def extend_chunk(self, layer: int, q: torch.Tensor, k_new: Optional[torch.Tensor],
                     v_new: Optional[torch.Tensor], out_cache_loc: Optional[torch.Tensor],
                     k_pool: torch.Tensor, v_pool: torch.Tensor, req_to_token: torch.Tensor,
                     req_pool_index: int, seq_len: int, out: Optional[torch.Tensor] = None,
                     debug: Optional[dict] = None) -> torch.Tensor:
        """One chunk (at most ``prefill_chunk`` tokens) of one request's prefill, one layer: one iteration of
        the chunk loop at token_retrieval.py:716-775.  ``q [Lq, Hq*D]``, ``k_new, v_new [Lq, Hkv*D]`` are
        stored at ``out_cache_loc [Lq]`` first; ``seq_len`` counts the request's tokens including this
        chunk.  Returns ``[Lq, Hq*D]``.  ``debug`` may hold int32 tensors ``slots, positions [n_sel]``,
        ``count, flags [1]`` and ``fingerprint [Hq*D]`` (model dtype)."""
        cfg = self.cfg
        if self.chunk_cs is None:
            raise ValueError("prefill needs prefill_chunk > 0 (and, with tp_size > 1, the in-kernel vote exchange)")
        lq = q.shape[0]
        hd, kd = cfg.num_q_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
        if out is None:
            out = torch.empty_like(q)
        for name, t, dt in (("q", q, cfg.dtype), ("k_pool", k_pool, cfg.dtype), ("v_pool", v_pool, cfg.dtype),
                            ("req_to_token", req_to_token, torch.int32), ("out", out, cfg.dtype)):
            if not t.is_cuda or t.dtype != dt:
                raise ValueError(f"{name}: expected a CUDA tensor of {dt}, got {t.device} {t.dtype}")
        if q.numel() != lq * hd or not q.is_contiguous() or not out.is_contiguous() or out.numel() != lq * hd:
            raise ValueError("q/out must be contiguous [chunk, num_q_heads*head_dim]")
        if not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.shape != v_pool.shape:
            raise ValueError("pools must be contiguous [rows, num_kv_heads, head_dim] of equal shape")
        if req_to_token.dim() != 2 or req_to_token.stride(1) != 1:
            raise ValueError("req_to_token must be [max_reqs, max_ctx] with unit inner stride")
        a = TsExtendArgs()
        a.struct_size = C.sizeof(TsExtendArgs)
        a.layer, a.chunk_len, a.req_pool_index, a.seq_len = int(layer), int(lq), int(req_pool_index), int(seq_len)
        a.q = q.data_ptr()
        if k_new is not None:
            for name, t in (("k", k_new), ("v", v_new)):
                if not t.is_cuda or t.dtype != cfg.dtype or not t.is_contiguous() or t.numel() != lq * kd:
                    raise ValueError(f"{name}: expected contiguous CUDA [chunk, num_kv_heads*head_dim] {cfg.dtype}")
            if out_cache_loc is None or out_cache_loc.dtype != torch.int32 or not out_cache_loc.is_cuda \
                    or out_cache_loc.numel() != lq or not out_cache_loc.is_contiguous():
                raise ValueError("out_cache_loc must be a contiguous CUDA int32 tensor [chunk]")
            a.k_new, a.v_new, a.out_cache_loc = k_new.data_ptr(), v_new.data_ptr(), out_cache_loc.data_ptr()
        a.k_pool, a.v_pool, a.pool_rows = k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0]
        a.req_to_token, a.req_to_token_stride = req_to_token.data_ptr(), req_to_token.stride(0)
        a.chunk_cos_sin = self.chunk_cs.data_ptr()
        a.out = out.data_ptr()
        if debug is not None:
            a.dbg_sel_slots = debug["slots"].data_ptr()
            a.dbg_sel_pos = debug["positions"].data_ptr()
            a.dbg_sel_count = debug["count"].data_ptr()
            a.dbg_flags = debug["flags"].data_ptr()
            if "fingerprint" in debug:
                a.dbg_fingerprint = debug["fingerprint"].data_ptr()
        a.stream = self._stream()
        check(self.lib.ts_extend_chunk(self._h, C.byref(a)), "ts_extend_chunk", self._h)
        return out

    # The three tensor-parallel stages one by one, for callers that run the exchange themselves
    # (e.g. several ranks' engines driven from one process).  ``args`` comes from ``build_args``.
    def build_args(self, layer, q, k_new, v_new, out_cache_loc, k_pool, v_pool, req_to_token,
                   req_pool_indices, seq_lens, out, debug=None) -> TsDecodeArgs:
        return self._args(layer, q, k_new, v_new, out_cache_loc, k_pool, v_pool, req_to_token,
                          req_pool_indices, seq_lens, out, debug)

    def tp_prepare(self, args: TsDecodeArgs) -> None:
        check(self.lib.ts_tp_prepare(self._h, C.byref(args)), "ts_tp_prepare", self._h)

    def tp_score_vote(self, args: TsDecodeArgs) -> None:
        check(self.lib.ts_tp_score_vote(self._h, C.byref(args)), "ts_tp_score_vote", self._h)

    def tp_select_attend(self, args: TsDecodeArgs) -> None:
        check(self.lib.ts_tp_select_attend(self._h, C.byref(args)), "ts_tp_select_attend", self._h)

    @staticmethod
    def vote_elems_for(seq_lens_host: Sequence[int], n_init: int, n_local: int) -> int:
        """Upper bound of the vote-vector prefix in use for these sequence lengths."""
        total = 0
        for n in seq_lens_host:
            nc = max(int(n) - n_init - n_local, 0)
            total += (nc + 127) // 128 * 128
        return total


def attend_rows_static(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, rows: torch.Tensor,
                       out: torch.Tensor, sm_scale: float, rope_base: float, rope_scale: float = 1.0,
                       logit_cap: float = 0.0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of one request over the listed pool rows through ``ts_attend_rows_static``, the entry
    point for callers that are not allowed to allocate device memory (a serving loop or callback that must
    stay off the allocator, or a process whose memory another component owns in full): it needs no engine, writes its
    intermediate results to a fixed array inside the library and allocates nothing.  ``out`` must be
    supplied by the caller for the same reason.  At most ``4 MiB / (heads * (head_dim + 2) * 4)`` chunks
    of 32 rows; calls that overlap on the GPU race on the shared array, so keep them on one stream."""
    lib = _lib.load()
    if rows.dtype != torch.int32 or not rows.is_cuda or not rows.is_contiguous():
        raise ValueError("rows must be a contiguous CUDA int32 tensor")       # int64 rows would be read as (value, 0) pairs
    for name, t in (("q", q), ("k_pool", k_pool), ("v_pool", v_pool), ("out", out)):
        if not t.is_cuda or not t.is_contiguous() or t.dtype != q.dtype:
            raise ValueError(f"{name}: expected a contiguous CUDA tensor of {q.dtype}")
    if q.dtype not in (torch.bfloat16, torch.float32) or k_pool.dim() != 3 or k_pool.shape != v_pool.shape:
        raise ValueError("q must be bf16 or fp32; pools must be [rows, num_kv_heads, head_dim] of equal shape")
    if status is not None and (status.dtype != torch.int32 or not status.is_cuda):
        raise ValueError("status must be a CUDA int32 tensor")
    hq = q.numel() // k_pool.shape[2]
    a = _lib.TsAttendStaticArgs()
    a.struct_size = C.sizeof(_lib.TsAttendStaticArgs)
    a.dtype = _lib.TS_DTYPE_BF16 if q.dtype == torch.bfloat16 else _lib.TS_DTYPE_F32
    a.hq, a.hkv, a.head_dim, a.count = hq, k_pool.shape[1], k_pool.shape[2], rows.numel()
    a.q, a.k_pool, a.v_pool, a.pool_rows = q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0]
    a.rows, a.out = rows.data_ptr(), out.data_ptr()
    a.sm_scale, a.logit_cap, a.rope_base, a.rope_scale = sm_scale, logit_cap, float(rope_base), float(rope_scale)
    a.status = None if status is None else status.data_ptr()
    a.stream = torch.cuda.current_stream(q.device).cuda_stream
    check(lib.ts_attend_rows_static(C.byref(a)), "ts_attend_rows_static")
    return out
