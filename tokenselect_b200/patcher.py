"""Drop-in surface of the reference's patcher for the decode and chunked-prefill path.

The reference monkey-patches a serving stack that is not a dependency here.  This module keeps the
names, argument meaning and error behaviour of the pieces that path touches
(patcher/token_retrieval.py):

* ``patch(...)``                      -- the knob entry point (:885-921); stores module-level knobs.
* ``ForwardMode``, ``InputMetadata``  -- the metadata fields the patched forward reads (:519-532).
* ``ReqToTokenPool``, ``TokenToKVPool`` -- the paged layout: page size 1, ``req_to_token[req, pos]``
  is a pool row, K and V buffers of ``[rows, kv_heads, head_dim]`` per layer (:170, :599-601, :847-848).
* ``ReqToTokenRetriever``             -- per-request state keyed by request id (:117-163).
* ``RadixAttention.forward(q, k, v, input_metadata)`` -- the patched forward (:827-842): stores the
  new K/V, selects, attends, returns ``[batch, heads*head_dim]``; in EXTEND mode it runs the chunked
  prefill of one request (:703-775).

A serving stack integrates by constructing one ``ReqToTokenRetriever`` per model runner (as
PatchedModelRunner does at :458-469) and assigning ``RadixAttention.forward`` /
``patched_radix_attention_forward`` onto its attention class (as :868-875 does).
"""
from __future__ import annotations

import dataclasses
import enum
from typing import List, Optional, Sequence

import torch

from .engine import TokenSelectConfig, TokenSelectEngine

# knobs written by patch(), same names as the reference's module globals (:29-39)
ROPE_BASE = -1
ROPE_SCALE = -1
ROPE_MODE = ""
MAX_N_TOKENS = -1
TOP_K = -1
N_INIT = -1
N_Local = -1
PREFILL_CHUNK_SIZE = -1
QUERY_ROTATE = False
QUERY_CACHE = False
KERNEL_SIZE = -1
SIMILARITY_THRESHOLD = 0.9
GQA_MAP = "mod"


def patch(rope_base=1e6, rope_scale=1, rope_model="ROPE_LLAMA", max_n_tokens=1024, top_k=16, n_init=1,
          n_local=16, kernel_size=-1, *, query_cache=False, similarity_threshold=0.9, gqa_map="mod"):
    """Same positional knobs and defaults as the reference's ``patch`` (:885-894).  The keyword-only
    extras expose what the reference hard-codes: ``QUERY_CACHE`` (:918), the 0.9 threshold (:313-315)
    and the scoring head map (:202)."""
    global ROPE_BASE, ROPE_SCALE, ROPE_MODE, MAX_N_TOKENS, TOP_K, N_INIT, N_Local, KERNEL_SIZE
    global QUERY_ROTATE, QUERY_CACHE, PREFILL_CHUNK_SIZE, SIMILARITY_THRESHOLD, GQA_MAP
    if rope_model != "ROPE_LLAMA":
        raise NotImplementedError("only the ROPE_LLAMA positional mode is implemented")
    ROPE_BASE, ROPE_SCALE, ROPE_MODE = rope_base, rope_scale, rope_model
    MAX_N_TOKENS, TOP_K, N_INIT, N_Local, KERNEL_SIZE = max_n_tokens, top_k, n_init, n_local, kernel_size
    QUERY_ROTATE, PREFILL_CHUNK_SIZE = True, 512
    QUERY_CACHE, SIMILARITY_THRESHOLD, GQA_MAP = bool(query_cache), float(similarity_threshold), gqa_map


class ForwardMode(enum.IntEnum):
    PREFILL = enum.auto()
    EXTEND = enum.auto()
    DECODE = enum.auto()


class ReqToTokenPool:
    """``req_to_token [size, max_context_len] int32``: logical position -> pool row (:599-601)."""

    def __init__(self, size: int, max_context_len: int, device="cuda"):
        self.size = size
        self.max_context_len = max_context_len
        self.req_to_token = torch.zeros((size, max_context_len), dtype=torch.int32, device=device)


class TokenToKVPool:
    """Per-layer K and V buffers ``[size, kv_heads, head_dim]`` (:170, :847-848)."""

    def __init__(self, size: int, dtype: torch.dtype, head_num: int, head_dim: int, layer_num: int,
                 device="cuda"):
        self.size = size
        self.k_buffer = [torch.zeros((size, head_num, head_dim), dtype=dtype, device=device) for _ in range(layer_num)]
        self.v_buffer = [torch.zeros((size, head_num, head_dim), dtype=dtype, device=device) for _ in range(layer_num)]

    def get_key_buffer(self, layer_id: int) -> torch.Tensor:
        return self.k_buffer[layer_id]

    def get_value_buffer(self, layer_id: int) -> torch.Tensor:
        return self.v_buffer[layer_id]

    def get_kv_buffer(self, layer_id: int):
        return self.k_buffer[layer_id], self.v_buffer[layer_id]


class ReqToTokenRetriever:
    """Per-request selection state, keyed by request id (:117-163).  The reference supports one
    running request (:130); here every request slot of the batch has its own state."""

    def __init__(self, num_layers, head_dim, num_heads, num_kv_heads, max_num_tokens, dtype,
                 max_reqs: int = 8, max_batch: int = 8, max_total_tokens: Optional[int] = None,
                 sm_scale: Optional[float] = None, logit_cap: float = 0.0, tp_rank: int = 0,
                 tp_size: int = 1, process_group=None, device=None, engine_factory=None):
        if TOP_K < 0:
            raise RuntimeError("call patch(...) before building the model runner")
        cfg = TokenSelectConfig(
            rope_base=ROPE_BASE, rope_scale=ROPE_SCALE, rope_model=ROPE_MODE, max_n_tokens=max_num_tokens,
            top_k=TOP_K, n_init=N_INIT, n_local=N_Local, kernel_size=KERNEL_SIZE, query_cache=QUERY_CACHE,
            similarity_threshold=SIMILARITY_THRESHOLD, gqa_map=GQA_MAP, n_layers=num_layers,
            num_q_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, dtype=dtype,
            sm_scale=sm_scale, logit_cap=logit_cap, max_reqs=max_reqs, max_batch=max_batch,
            max_total_tokens=max_total_tokens, tp_rank=tp_rank, tp_size=tp_size)
        self.config = cfg
        if engine_factory is not None:
            self.engine = engine_factory(cfg)
        else:
            self.engine = TokenSelectEngine(cfg, device=device, process_group=process_group)

    def get_token_retriever(self, req_ids: Sequence[object], req_pool_indices: Sequence[int]) -> TokenSelectEngine:
        """New request id in a slot -> fresh state for that slot (:147-163)."""
        self.engine.bind_requests(req_ids, req_pool_indices)
        return self.engine


@dataclasses.dataclass
class InputMetadata:
    """The fields of the serving stack's batch metadata that the patched forward reads (:519-532)."""
    forward_mode: ForwardMode
    batch_size: int
    req_pool_indices: torch.Tensor        # [batch] int32
    seq_lens: torch.Tensor                # [batch] int32, counting the token being decoded
    req_to_token_pool: ReqToTokenPool
    token_to_kv_pool: TokenToKVPool
    out_cache_loc: torch.Tensor           # [batch] int32
    token_retriever: TokenSelectEngine = None
    seq_lens_cpu: Optional[List[int]] = None   # optional host copy; bounds the tensor-parallel message
    # EXTEND only (host values, so that the chunk loop needs no device sync): the request's slot and the
    # number of its tokens already in the cache before this forward (prefix_lens of the serving stack)
    req_pool_indices_cpu: Optional[List[int]] = None
    extend_prefix_lens_cpu: Optional[List[int]] = None


def patched_radix_attention_forward(self, q, k, v, input_metadata: InputMetadata):
    """Replacement for ``RadixAttention.forward`` (:827-842).  ``q [batch, heads*head_dim]``,
    ``k, v [batch, kv_heads*head_dim]`` un-rotated (the patched model skips its own rotary layer,
    :856-866, :878-881)."""
    if k is not None:
        assert v is not None
        k = k.view(-1, self.tp_k_head_num * self.qk_head_dim)
        v = v.view(-1, self.tp_v_head_num * self.v_head_dim)
    if input_metadata.forward_mode == ForwardMode.DECODE:
        eng = input_metadata.token_retriever
        k_pool, v_pool = input_metadata.token_to_kv_pool.get_kv_buffer(self.layer_id)
        ve = None
        if input_metadata.seq_lens_cpu is not None:
            ve = eng.vote_elems_for(input_metadata.seq_lens_cpu, eng.cfg.n_init, eng.cfg.n_local)
        o = eng.decode_layer(
            self.layer_id, q.contiguous().view(-1, self.tp_q_head_num * self.head_dim),
            None if k is None else k.contiguous(), None if v is None else v.contiguous(),
            input_metadata.out_cache_loc, k_pool, v_pool, input_metadata.req_to_token_pool.req_to_token,
            input_metadata.req_pool_indices, input_metadata.seq_lens, vote_elems=ve)
        return o.view(-1, self.tp_q_head_num * self.head_dim)
    if input_metadata.forward_mode == ForwardMode.EXTEND:
        return patched_radix_attention_extend_forward(self, q, k, v, input_metadata)
    raise NotImplementedError("ForwardMode.PREFILL is not a mode of the patched stack (:834-841)")


def patched_radix_attention_extend_forward(self, q, k, v, input_metadata: InputMetadata):
    """Replacement for ``patched_radix_attention_extend_forward_flashinfer`` (:703-775): the new tokens of
    ONE request (the reference asserts a single request, :130, :526-528) go through the layer in chunks of
    ``PREFILL_CHUNK_SIZE`` (:716-724); every chunk stores its K/V, selects with its fingerprint and runs
    causal attention over the selected list."""
    if input_metadata.batch_size != 1:
        raise NotImplementedError("prefill handles one request per forward, as the reference does")
    if input_metadata.req_pool_indices_cpu is None or input_metadata.extend_prefix_lens_cpu is None:
        raise ValueError("EXTEND needs req_pool_indices_cpu and extend_prefix_lens_cpu (host values)")
    eng = input_metadata.token_retriever
    chunk = PREFILL_CHUNK_SIZE if PREFILL_CHUNK_SIZE > 0 else eng.cfg.prefill_chunk
    hd = self.tp_q_head_num * self.head_dim
    q = q.contiguous().view(-1, hd)
    total = q.shape[0]
    req = int(input_metadata.req_pool_indices_cpu[0])
    prefix = int(input_metadata.extend_prefix_lens_cpu[0])
    k_pool, v_pool = input_metadata.token_to_kv_pool.get_kv_buffer(self.layer_id)
    outputs = torch.empty_like(q)
    for start in range(0, total, chunk):
        end = min(start + chunk, total)
        eng.extend_chunk(
            self.layer_id, q[start:end], None if k is None else k[start:end].contiguous(),
            None if v is None else v[start:end].contiguous(),
            None if k is None else input_metadata.out_cache_loc[start:end].contiguous(), k_pool, v_pool,
            input_metadata.req_to_token_pool.req_to_token, req, prefix + end, out=outputs[start:end])
    return outputs


class RadixAttention:
    """Attribute surface of the serving stack's attention layer that the patched forward reads
    (:708, :754-756, :795, :816-819, :832-833)."""

    def __init__(self, num_heads: int, head_dim: int, scaling: float, num_kv_heads: int, layer_id: int,
                 logit_cap: float = -1):
        self.tp_q_head_num = num_heads
        self.tp_k_head_num = num_kv_heads
        self.tp_v_head_num = num_kv_heads
        self.head_dim = head_dim
        self.qk_head_dim = head_dim
        self.v_head_dim = head_dim
        self.scaling = scaling
        self.layer_id = layer_id
        self.logit_cap = logit_cap if logit_cap is not None and logit_cap > 0 else 0
        self.sliding_window_size = -1

    forward = patched_radix_attention_forward

    def __call__(self, q, k, v, input_metadata):
        return self.forward(q, k, v, input_metadata)


# ---------------------------------------------------------------------------------------------
# Installers: the three patch groups of the reference, applied to whatever classes a serving stack
# hands in.  The reference imports SGLang 0.2.13 and patches its classes in place (:452-472, :475-568,
# :868-883); that package is not a dependency here, so the installers take the module objects (or
# stand-ins with the same attributes) as arguments.  ``install()`` looks the real modules up.
# ---------------------------------------------------------------------------------------------
def patched_meta_attention_forward(self, positions, hidden_states, input_metadata):
    """Attention module forward without its own rotary embedding (:856-866): q and k reach the patched
    ``RadixAttention.forward`` un-rotated; the rotation happens inside the selection and attention kernels."""
    qkv, _ = self.qkv_proj(hidden_states)
    q, k, v = qkv.split([self.q_size, self.kv_size, self.kv_size], dim=-1)
    attn_output = self.attn(q, k, v, input_metadata)
    output, _ = self.o_proj(attn_output)
    return output


def patch_attention(model):
    """Equivalent of ``patch_attention`` (:700, :868-876): every layer's attention module loses its rotary
    step and its ``attn`` object gets the patched forward.  Returns the model."""
    for layer in model.model.layers:
        layer.self_attn.__class__.forward = patched_meta_attention_forward
        layer.self_attn.attn.__class__.forward = patched_radix_attention_forward
    return model


def patch_rotary_embedding(rotary_embedding_module):
    """``get_rope`` returns None, as at :878-881: the model must not rotate q and k itself."""
    def patched_rotary_embedding_get_rope(*args, **kwargs):
        return None
    rotary_embedding_module.get_rope = patched_rotary_embedding_get_rope
    return rotary_embedding_module


def patch_model_runner(model_runner_module, engine_factory=None):
    """Equivalent of ``patch_model_runner`` (:452-472): ``ModelRunner`` is replaced by a subclass whose
    constructor also builds the per-runner ``req_to_token_retriever`` from ``model_config`` (layers, head_dim,
    attention heads and this rank's KV heads) and the ``patch()`` knobs.  ``engine_factory`` replaces the CUDA
    engine in tests without a GPU."""
    base = model_runner_module.ModelRunner

    class PatchedModelRunner(base):
        def __init__(self, **kwargs):
            super().__init__(**kwargs)
            mc = self.model_config
            tp_size = getattr(self, "tp_size", 1)
            self.req_to_token_retriever = ReqToTokenRetriever(
                mc.num_hidden_layers, mc.head_dim, mc.num_attention_heads // tp_size, mc.get_num_kv_heads(tp_size),
                MAX_N_TOKENS, self.dtype,
                max_reqs=int(self.req_to_token_pool.req_to_token.shape[0]),
                max_batch=int(getattr(self, "max_running_requests", 8) or 8),
                max_total_tokens=int(getattr(self, "max_total_num_tokens", 0)) or None,
                tp_rank=getattr(self, "tp_rank", 0), tp_size=tp_size, engine_factory=engine_factory)

    model_runner_module.ModelRunner = PatchedModelRunner
    return PatchedModelRunner


def patch_input_metadata(forward_batch_info_module):
    """Equivalent of ``patch_input_metadata`` (:475-568): ``InputMetadata.from_schedule_batch`` additionally
    binds the batch's request ids to their request slots (a new id in a slot gets fresh selection state,
    :147-163) and carries the runner's engine as ``token_retriever``.  No third-party attention wrappers are
    planned and no sequence lengths are copied to the host (:570-625 is not needed: the kernels read
    ``req_to_token`` directly)."""
    base = forward_batch_info_module.InputMetadata

    class PatchedInputMetadata(base):
        token_retriever = None

        @classmethod
        def from_schedule_batch(cls, model_runner, batch, forward_mode):
            ret = super().from_schedule_batch(model_runner, batch, forward_mode)
            slots = batch.req_pool_indices.tolist() if hasattr(batch.req_pool_indices, "tolist") else list(batch.req_pool_indices)
            ret.token_retriever = model_runner.req_to_token_retriever.get_token_retriever(
                [r.rid for r in batch.reqs], slots)
            ret.req_pool_indices_cpu = slots
            if getattr(forward_mode, "name", str(forward_mode)) != "DECODE":
                ret.extend_prefix_lens_cpu = [len(r.prefix_indices) for r in batch.reqs]
            return ret

    forward_batch_info_module.InputMetadata = PatchedInputMetadata
    return PatchedInputMetadata


def install():
    """Apply the three patch groups to an installed SGLang (the reference pins 0.2.13, README.md:42).  Raises
    ImportError when it is absent."""
    import sglang.srt.model_executor.forward_batch_info as fbi
    import sglang.srt.model_executor.model_runner as mr
    from sglang.srt.layers import rotary_embedding as rot       # noqa: F401  (location in 0.2.13: vllm's module)
    patch_input_metadata(fbi)
    patch_model_runner(mr)
    patch_rotary_embedding(rot)
