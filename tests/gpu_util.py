"""Helpers shared by the GPU parity tests: build an engine for a seeded case, run one layer step
through the C ABI and through the CPU oracle, and compare."""
from __future__ import annotations

import numpy as np
import torch

from oracle import synth
from oracle import tokenselect_oracle as orc
from tokenselect_b200 import TokenSelectConfig, TokenSelectEngine


def make_engine(hq, hkv, d, n_init, n_local, top_k, rope_base, dtype, n_layers=1, max_ctx=None,
                max_reqs=4, max_batch=4, max_total=None, rope_scale=1.0, **kw) -> TokenSelectEngine:
    cfg = TokenSelectConfig(rope_base=rope_base, rope_scale=rope_scale, max_n_tokens=max_ctx or 1 << 18, top_k=top_k,
                            n_init=n_init, n_local=n_local, n_layers=n_layers, num_q_heads=hq, num_kv_heads=hkv,
                            head_dim=d, dtype=dtype, max_reqs=max_reqs, max_batch=max_batch,
                            max_total_tokens=max_total or (max_batch * (max_ctx or 1 << 18)), **kw)
    return TokenSelectEngine(cfg)


def oracle_config(eng: TokenSelectEngine, **kw) -> orc.OracleConfig:
    c = eng.cfg
    return orc.OracleConfig(c.n_layers, c.num_q_heads, c.num_kv_heads, c.head_dim, c.n_init, c.n_local, c.top_k,
                            c.rope_base, c.rope_scale, c.similarity_threshold, c.query_cache, c.gqa_map,
                            c.kernel_size, c.sm_scale, c.logit_cap, **kw)


def run_gpu(eng: TokenSelectEngine, layer, q, k_pool, v_pool, rtt, req_idx, seq_lens, k_new=None, v_new=None,
            loc=None):
    """All arguments are CPU tensors; returns (out, debug dict) as CPU tensors."""
    dev = eng.device
    bs = q.shape[0]
    dbg = eng.new_debug_buffers(bs)
    kp, vp = k_pool.to(dev), v_pool.to(dev)
    out = eng.decode_layer(
        layer, q.to(dev), None if k_new is None else k_new.to(dev), None if v_new is None else v_new.to(dev),
        None if loc is None else loc.to(device=dev, dtype=torch.int32), kp, vp, rtt.to(dev),
        req_idx.to(device=dev, dtype=torch.int32), seq_lens.to(device=dev, dtype=torch.int32), debug=dbg)
    torch.cuda.synchronize()
    eng.raise_on_device_error()
    res = {k: v.cpu() for k, v in dbg.items()}
    res["k_pool"], res["v_pool"] = kp.cpu(), vp.cpu()
    return out.cpu(), res


def logits_columns_to_heads(eng: TokenSelectEngine) -> np.ndarray:
    """Column c of the library's logit rows is kv_head*group + j; return head index per column."""
    c = eng.cfg
    group = c.num_q_heads // c.num_kv_heads
    cols = []
    for kv in range(c.num_kv_heads):
        for j in range(group):
            cols.append(kv + c.num_kv_heads * j if c.gqa_map == "mod" else kv * group + j)
    return np.array(cols)


def check_selection(eng, res, b, oracle_pos, oracle_votes, n_tokens):
    """Index-set parity rule: identical to the oracle except inside the 1e-4 relative tie band of the
    k-th vote; strictly ascending; windows exact."""
    c = eng.cfg
    cnt = int(res["count"][b])
    assert cnt == c.n_sel
    pos = res["positions"][b, :cnt].numpy()
    assert np.all(np.diff(pos) > 0), "positions must be strictly ascending"
    assert np.array_equal(pos[: c.n_init], np.arange(c.n_init))
    assert np.array_equal(pos[c.n_init + c.top_k:], np.arange(n_tokens - c.n_local, n_tokens))
    want = oracle_pos.numpy()
    got_c = pos[c.n_init: c.n_init + c.top_k] - c.n_init
    want_c = want[c.n_init: c.n_init + c.top_k] - c.n_init
    ok, why = orc.index_sets_match(got_c, want_c, oracle_votes.double().numpy(), c.top_k, rel_tol=1e-4)
    assert ok, why
    return pos


def case_tensors(case: synth.LayerCase):
    return (case.q[None].contiguous(), case.k_pool, case.v_pool, case.req_to_token,
            torch.tensor([case.req_pool_idx]), torch.tensor([case.n_tokens]))
