"""CPU-only checks: the C-ABI library builds, loads and exports every declared symbol; host-side
configuration, rotation tables and knob plumbing.  No kernel is launched here."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from oracle import tokenselect_oracle as orc
from tokenselect_b200 import _lib, build, patcher
from tokenselect_b200.engine import TokenSelectConfig, TokenSelectEngine, rotary_tables

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="session", autouse=True)
def built_library():
    build.build_library()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tokenselect_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ts_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_library):
    names = _declared_symbols()
    assert len(names) >= 15
    assert set(names) == set(_lib.EXPORTS)
    for n in names:
        assert hasattr(built_library, n), n
    assert built_library.ts_abi_version() == _lib.TS_ABI_VERSION
    assert built_library.ts_status_string(0) == b"ok"
    assert b"slot" in built_library.ts_status_string(6) or b"row" in built_library.ts_status_string(6)


def _cfg(**kw):
    c = _lib.TsConfig()
    c.struct_size = C.sizeof(_lib.TsConfig)
    c.n_layers, c.hq, c.hkv, c.head_dim, c.dtype = 32, 32, 8, 128, 0
    c.n_init, c.n_local, c.top_k, c.kernel_size = 128, 512, 2048, -1
    c.rope_base, c.rope_scale, c.sm_scale = 5e5, 1.0, 128 ** -0.5
    c.max_reqs, c.max_batch, c.max_ctx, c.max_total_tokens = 4, 1, 1 << 17, 1 << 17
    c.tp_rank, c.tp_size = 0, 1
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def test_workspace_query_and_validation(built_library):
    ws = C.c_size_t()
    assert built_library.ts_query_workspace(C.byref(_cfg()), C.byref(ws)) == 0
    # logits (fp32, 32 heads) dominate: ~128 B per candidate
    assert 16 << 20 < ws.value < 256 << 20
    ve = C.c_int64()
    assert built_library.ts_vote_buffer_elems(C.byref(_cfg()), C.byref(ve)) == 0
    assert ve.value >= (1 << 17)
    for bad, status in ((dict(struct_size=8), 1), (dict(hq=30), 1), (dict(head_dim=96), 2), (dict(dtype=5), 2),
                        (dict(hq=32, hkv=2), 2), (dict(max_batch=100000), 1), (dict(tp_rank=2), 1),
                        (dict(n_local=0), 1), (dict(rope_base=0.0), 1)):
        assert built_library.ts_query_workspace(C.byref(_cfg(**bad)), C.byref(ws)) == status, bad
    h = C.c_void_p()
    assert built_library.ts_create(C.byref(_cfg(hq=30)), C.byref(h)) == 1
    assert built_library.ts_reset_request(None, 0, None) == 1
    assert built_library.ts_decode_layer(None, None) == 1


def test_symmetric_buffer_size_follows_the_exchange_form(built_library):
    """Peer-visible memory per rank: flag pad + two vote buffers; up to four ranks add two push areas of
    tp_size x capacity 8-byte pairs (votes pushed with their exchange number), unless TS_CFG_TP_PULL."""
    def nbytes(**kw):
        n = C.c_size_t()
        assert built_library.ts_tp_symmetric_bytes(C.byref(_cfg(**kw)), C.byref(n)) == 0
        return n.value
    ve = C.c_int64()
    assert built_library.ts_vote_buffer_elems(C.byref(_cfg(hq=4, hkv=1, tp_size=8)), C.byref(ve)) == 0
    cap = ve.value
    pull8 = nbytes(hq=4, hkv=1, tp_size=8)
    assert pull8 == 2 * 8 * 256 * 4 + 2 * cap * 4                      # flags [2][8][256] + votes [2][cap]
    assert nbytes(hq=8, hkv=2, tp_size=4, flags=2048) == pull8         # pull forced: same layout at any degree
    push4, push2 = nbytes(hq=8, hkv=2, tp_size=4), nbytes(hq=16, hkv=4, tp_size=2)
    assert 0 <= push4 - pull8 - 2 * 4 * cap * 8 < 256                  # + [2][4][cap] pairs, 256-byte aligned
    assert 0 <= push2 - pull8 - 2 * 2 * cap * 8 < 256


def test_struct_layout_matches_header():
    """Compile a one-line C program against the header and compare sizeof with the ctypes mirror."""
    import subprocess
    import tempfile
    src = ('#include "tokenselect_b200.h"\n#include <stdio.h>\n#include <stddef.h>\n'
           'int main(){printf("%zu %zu %zu %zu %zu %zu %zu\\n", sizeof(ts_config), sizeof(ts_decode_args),'
           ' offsetof(ts_config, rope_base), offsetof(ts_decode_args, stream), sizeof(ts_extend_args),'
           ' offsetof(ts_extend_args, chunk_cos_sin), offsetof(ts_config, prefill_chunk));'
           'printf("%zu %zu\\n", offsetof(ts_config, wait_limit_us), offsetof(ts_config, score_cos_sin));return 0;}\n')
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "s.c"), "w").write(src)
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), os.path.join(d, "s.c"), "-o",
                               os.path.join(d, "s")])
        a, b, c, e, x, y, z, w, v = map(int, subprocess.check_output([os.path.join(d, "s")]).split())
    assert a == C.sizeof(_lib.TsConfig) and b == C.sizeof(_lib.TsDecodeArgs)
    assert c == _lib.TsConfig.rope_base.offset and e == _lib.TsDecodeArgs.stream.offset
    assert x == C.sizeof(_lib.TsExtendArgs) and y == _lib.TsExtendArgs.chunk_cos_sin.offset
    assert z == _lib.TsConfig.prefill_chunk.offset
    assert w == _lib.TsConfig.wait_limit_us.offset and v == _lib.TsConfig.score_cos_sin.offset


def test_rotation_tables_match_oracle_bitwise():
    cfg = TokenSelectConfig(rope_base=5e5, n_init=16, n_local=64, top_k=256, head_dim=128)
    score, attn = rotary_tables(cfg)
    inv = orc.rope_inv_freq(128, 5e5)
    cos, sin = orc.rope_cos_sin(torch.tensor([64.0]), inv)
    assert torch.equal(score[:, 0], cos[0, :64]) and torch.equal(score[:, 1], sin[0, :64])
    cos, sin = orc.rope_cos_sin(torch.arange(cfg.n_sel + 1, dtype=torch.float32), inv)
    assert torch.equal(attn[..., 0], cos[:, :64]) and torch.equal(attn[..., 1], sin[:, :64])
    assert attn.shape == (cfg.n_sel + 1, 64, 2)
    # prefill chunk: positions n_local, n_local + 1, ... (token_retrieval.py:380-388)
    from tokenselect_b200.engine import chunk_rotary_table
    table = chunk_rotary_table(cfg)
    cos, sin = orc.rope_cos_sin(torch.arange(64, 64 + cfg.prefill_chunk, dtype=torch.float32), inv)
    assert torch.equal(table[..., 0], cos[:, :64]) and torch.equal(table[..., 1], sin[:, :64])


def test_config_from_reference_style_yaml(tmp_path):
    p = tmp_path / "llama.yaml"
    p.write_text("model:\n  type: token-retrieval\n  path: some/model\n  rope_base: 500000\n  rope_scale: 1\n"
                 "  n_init: 128\n  n_local: 512\n  top_k: 2048\n  max_n_tokens: 1048576\nmax_len: 1048576\n"
                 "chunk_size: 8192\ndtype: bfloat16\n")
    cfg = TokenSelectConfig.from_yaml(str(p), query_cache=True)
    assert (cfg.rope_base, cfg.n_init, cfg.n_local, cfg.top_k, cfg.max_n_tokens) == (500000, 128, 512, 2048, 1048576)
    assert cfg.query_cache and cfg.n_sel == 2688 and cfg.kernel_size == -1


def test_patch_sets_reference_knobs():
    patcher.patch(rope_base=5e5, rope_scale=1, max_n_tokens=4096, top_k=64, n_init=4, n_local=32, kernel_size=5)
    assert (patcher.ROPE_BASE, patcher.TOP_K, patcher.N_INIT, patcher.N_Local, patcher.KERNEL_SIZE) == \
        (5e5, 64, 4, 32, 5)
    assert patcher.QUERY_ROTATE is True and patcher.QUERY_CACHE is False and patcher.PREFILL_CHUNK_SIZE == 512
    with pytest.raises(NotImplementedError):
        patcher.patch(rope_model="ROPE_OTHER")


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_engine_refuses_to_run_without_a_gpu():
    with pytest.raises(RuntimeError, match="CUDA"):
        TokenSelectEngine(TokenSelectConfig())


def test_vote_prefix_bound():
    assert TokenSelectEngine.vote_elems_for([131072], 128, 512) == (131072 - 640 + 127) // 128 * 128
    assert TokenSelectEngine.vote_elems_for([100, 700, 641], 128, 512) == 128 + 128


def test_installers_patch_stand_in_serving_classes():
    """The three patch groups (patcher/token_retrieval.py:452-472, :475-568, :868-883) applied to stand-ins with
    the attributes the reference reads: the patched runner builds the per-runner state from model_config and
    the patch() knobs, the patched metadata binds request ids to slots and carries the engine, the patched
    attention classes route DECODE and EXTEND to it.  No GPU: a recording engine stands in for the CUDA one."""
    import types
    from tokenselect_b200 import patcher
    patcher.patch(rope_base=5e5, max_n_tokens=4096, top_k=256, n_init=16, n_local=64)
    calls = []

    class FakeEngine:
        def __init__(self, cfg):
            self.cfg = cfg
            self.bound = []

        def bind_requests(self, rids, slots):
            self.bound.append((list(rids), list(slots)))

        def decode_layer(self, layer, q, k, v, loc, kp, vp, rtt, ridx, lens, vote_elems=None):
            calls.append(("decode", layer, tuple(q.shape)))
            return torch.zeros_like(q)

        def extend_chunk(self, layer, q, k, v, loc, kp, vp, rtt, req, seq_len, out=None):
            calls.append(("extend", layer, q.shape[0], req, seq_len))
            out.zero_()
            return out

        @staticmethod
        def vote_elems_for(lens, n_init, n_local):
            return 0

    class ModelConfig:
        num_hidden_layers, head_dim, num_attention_heads = 2, 128, 8

        @staticmethod
        def get_num_kv_heads(tp_size):
            return 2 // tp_size

    class ModelRunner:
        def __init__(self, **kw):
            self.model_config, self.tp_size, self.tp_rank, self.dtype = ModelConfig(), 1, 0, torch.bfloat16
            self.req_to_token_pool = patcher.ReqToTokenPool(4, 512, device="cpu")
            self.token_to_kv_pool = patcher.TokenToKVPool(1024, torch.bfloat16, 2, 128, 2, device="cpu")
            self.max_total_num_tokens = 1024

    class InputMetadata(patcher.InputMetadata):
        @classmethod
        def from_schedule_batch(cls, model_runner, batch, forward_mode):
            return cls(forward_mode=forward_mode, batch_size=len(batch.reqs), req_pool_indices=batch.req_pool_indices,
                       seq_lens=batch.seq_lens, req_to_token_pool=model_runner.req_to_token_pool,
                       token_to_kv_pool=model_runner.token_to_kv_pool, out_cache_loc=batch.out_cache_loc)

    mr_mod, fbi_mod, rot_mod = types.SimpleNamespace(ModelRunner=ModelRunner), types.SimpleNamespace(InputMetadata=InputMetadata), \
        types.SimpleNamespace(get_rope=lambda *a, **k: object())
    patcher.patch_model_runner(mr_mod, engine_factory=FakeEngine)
    patcher.patch_input_metadata(fbi_mod)
    patcher.patch_rotary_embedding(rot_mod)
    assert rot_mod.get_rope(128, 128, 4096, 1e6) is None
    runner = mr_mod.ModelRunner()
    cfg = runner.req_to_token_retriever.config
    assert (cfg.n_layers, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim) == (2, 8, 2, 128)
    assert (cfg.top_k, cfg.n_init, cfg.n_local, cfg.max_n_tokens, cfg.max_reqs) == (256, 16, 64, 4096, 4)

    class Attn:                                            # the serving stack's RadixAttention
        tp_q_head_num, tp_k_head_num, tp_v_head_num, head_dim, qk_head_dim, v_head_dim, layer_id = 8, 2, 2, 128, 128, 128, 1

        def __call__(self, q, k, v, md):
            return self.forward(q, k, v, md)

    class SelfAttn:                                        # the model's attention module
        q_size, kv_size = 8 * 128, 2 * 128

        def __init__(self):
            self.attn = Attn()
            self.qkv_proj = lambda h: (torch.cat([h, h[:, :512]], dim=-1), None)
            self.o_proj = lambda a: (a, None)

    model = types.SimpleNamespace(model=types.SimpleNamespace(layers=[types.SimpleNamespace(self_attn=SelfAttn())]))
    patcher.patch_attention(model)
    req = types.SimpleNamespace(rid="r-17", prefix_indices=[])
    batch = types.SimpleNamespace(reqs=[req], req_pool_indices=torch.tensor([3], dtype=torch.int32),
                                  seq_lens=torch.tensor([700], dtype=torch.int32),
                                  out_cache_loc=torch.tensor([5], dtype=torch.int32))
    md = fbi_mod.InputMetadata.from_schedule_batch(runner, batch, patcher.ForwardMode.DECODE)
    assert md.token_retriever is runner.req_to_token_retriever.engine and md.token_retriever.bound == [(["r-17"], [3])]
    out = model.model.layers[0].self_attn.forward(None, torch.zeros(1, 1024, dtype=torch.bfloat16), md)
    assert out.shape == (1, 1024) and calls[-1] == ("decode", 1, (1, 1024))
    batch.out_cache_loc = torch.arange(600, dtype=torch.int32)
    md = fbi_mod.InputMetadata.from_schedule_batch(runner, batch, patcher.ForwardMode.EXTEND)
    out = model.model.layers[0].self_attn.forward(None, torch.zeros(600, 1024, dtype=torch.bfloat16), md)
    assert out.shape == (600, 1024)
    assert calls[-2:] == [("extend", 1, 512, 3, 512), ("extend", 1, 88, 3, 600)]      # chunks of 512 (:716-724, :917)
