"""Run the reference's own selection code, unmodified, on the CPU (TEST INFRASTRUCTURE ONLY).

The reference module ``patcher/token_retrieval.py`` cannot be imported as shipped: it imports a
serving stack (``sglang`` 0.2.13, old ``vllm`` modules) that is not installed.  Its selection math
(``RotaryEmbedding``, ``TokenRetriever``, the Triton scoring kernel) needs none of that, so this
loader pre-seeds ``sys.modules`` with inert stand-ins for those imports, switches Triton to its
CPU interpreter and imports the file from where it lies.  Nothing of the reference is copied.

Limits: the interpreter only handles fp32 tensors here (bf16 gives NaN), the selection-cache
branch of the reference raises (it calls ``get_topk_tokens`` with a missing argument,
``token_retrieval.py:411-413``), and one call takes seconds -- it is an oracle, never a timed
baseline.

Used by ``tests/golden/make_golden.py`` to produce the committed golden vectors and, when the
reference checkout is present, by ``tests/test_oracle_golden.py`` to re-check them live.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from typing import Optional
from unittest import mock

import torch

# where the reference checkout lives: the environment variable, else a sibling "reference" directory of the repository
DEFAULT_REFERENCE_ROOT = os.environ.get(
    "TOKENSELECT_REFERENCE_ROOT",
    os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
_STUBBED = [
    "sglang", "sglang.srt", "sglang.srt.managers", "sglang.srt.managers.schedule_batch",
    "sglang.srt.model_executor", "sglang.srt.model_executor.forward_batch_info",
    "sglang.srt.model_executor.model_runner",
    "vllm", "vllm.config", "vllm.model_executor", "vllm.model_executor.layers",
    "vllm.model_executor.layers.rotary_embedding", "vllm.model_executor.model_loader",
    "vllm.model_executor.model_loader.loader", "vllm.model_executor.model_loader.utils",
]
_module = None


def available(root: str = DEFAULT_REFERENCE_ROOT) -> bool:
    return os.path.isfile(os.path.join(root, "patcher", "token_retrieval.py"))


def load(root: str = DEFAULT_REFERENCE_ROOT):
    """Import the reference module with stand-ins for the absent serving stack."""
    global _module
    if _module is not None:
        return _module
    os.environ["TRITON_INTERPRET"] = "1"
    if "triton" in sys.modules:
        raise RuntimeError("triton was imported before TRITON_INTERPRET=1 could be set")
    saved = {name: sys.modules.get(name) for name in _STUBBED}
    try:
        for name in _STUBBED:
            sys.modules[name] = mock.MagicMock(name=name)
        path = os.path.join(root, "patcher", "token_retrieval.py")
        spec = importlib.util.spec_from_file_location("_tokenselect_reference", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for name, old in saved.items():
            if old is None:
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = old
    _module = mod
    return mod


class _FakePool:
    """The only pool method the selection code calls (token_retrieval.py:288-291)."""

    def __init__(self, k_pool: torch.Tensor):
        self._k = k_pool

    def get_key_buffer(self, layer_id: int) -> torch.Tensor:
        return self._k


def retrieval_indices(q: torch.Tensor, k_pool: torch.Tensor, slot_row: torch.Tensor, n_tokens: int,
                      hq: int, hkv: int, head_dim: int, n_init: int, n_local: int, top_k: int,
                      rope_base: float, rope_scale: float = 1, kernel_size: int = -1,
                      root: str = DEFAULT_REFERENCE_ROOT) -> Optional[torch.Tensor]:
    """Reference ``TokenRetriever.retrieval_indices`` (token_retrieval.py:375-449) for one decode
    query ``q [Hq*D]`` or one prefill chunk ``q [Lq, Hq*D]`` (fp32) of a request whose ``n_tokens``
    positions map to ``slot_row``.
    The module globals are set as ``patch()`` sets them (token_retrieval.py:907-918).
    Returns the int32 slot list, or None when the reference falls back to dense attention."""
    ref = load(root)
    assert q.dtype == torch.float32 and k_pool.dtype == torch.float32, "interpreter path is fp32 only"
    ref.ROPE_BASE, ref.ROPE_SCALE, ref.ROPE_MODE = rope_base, rope_scale, "ROPE_LLAMA"
    ref.MAX_N_TOKENS, ref.TOP_K, ref.N_INIT, ref.N_Local = int(slot_row.numel()), top_k, n_init, n_local
    ref.KERNEL_SIZE = kernel_size
    ref.QUERY_ROTATE, ref.PREFILL_CHUNK_SIZE, ref.QUERY_CACHE = True, 512, False
    rope = ref.RotaryEmbedding(head_dim, rope_base, rope_scale, "cpu")
    retriever = ref.TokenRetriever(
        num_layers=1, head_dim=head_dim, num_heads=hq, num_kv_heads=hkv, fingerprint_dim=hkv * head_dim,
        max_num_tokens=int(slot_row.numel()), dtype=torch.float32, device="cpu",
        token_to_kv_pool=_FakePool(k_pool), rotary_embedding=rope)
    retriever.add_k_cache(slot_row[:n_tokens].to(torch.int32), 0)
    with torch.no_grad():
        return retriever.retrieval_indices(q.reshape(-1, hq * head_dim), 0, n_init, n_local, top_k)
