"""Prefill chunks through the C ABI (``ts_extend_chunk``) against the CPU oracle: the chunk's K/V rows in
the pools, the fingerprint bit for bit, the selected index set, and the causal attention output."""
import numpy as np
import pytest
import torch

from oracle import synth
from oracle import tokenselect_oracle as orc
from tests import gpu_util as gu
from tokenselect_b200 import patcher

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32

# name, seed, N (incl. chunk), chunk, Hq, Hkv, D, n_init, n_local, top_k, base, dtype, attention tolerance
SHAPES = [
    ("llama_8k_full_chunk", 31, 8192, 512, 32, 8, 128, 128, 512, 1024, 5e5, BF16, 2e-2),
    ("qwen_4k_full_chunk", 32, 4096, 512, 28, 4, 128, 128, 512, 512, 1e6, BF16, 2e-2),
    ("gqa4_chunk64", 33, 2048, 64, 8, 2, 128, 16, 64, 256, 5e5, BF16, 2e-2),
    ("partial_chunk37", 34, 1500, 37, 8, 2, 128, 16, 64, 256, 5e5, BF16, 2e-2),
    ("chunk_is_whole_request_dense", 35, 300, 300, 8, 2, 128, 16, 64, 256, 5e5, BF16, 2e-2),
    ("dense_with_prefix", 36, 330, 64, 8, 2, 128, 16, 64, 256, 5e5, BF16, 2e-2),
    ("fp32_check_mode", 37, 2048, 64, 8, 2, 128, 16, 64, 256, 5e5, F32, 1e-5),
    ("head_dim64_plain_path", 38, 1024, 48, 4, 4, 64, 8, 64, 128, 1e4, BF16, 2e-2),
    ("one_kv_head", 39, 3000, 128, 4, 1, 128, 16, 128, 256, 5e5, BF16, 2e-2),
]


def _chunk_case(seed, n, lq, hq, hkv, d, n_init, n_local, base, dtype):
    case = synth.make_layer_case(seed, n, hq, hkv, d, n_init, n_local, base, dtype=dtype)
    qc = synth.make_chunk_queries(seed, case, lq, hq, d)
    row = case.req_to_token[case.req_pool_idx]
    loc = row[n - lq:n].clone()
    # the chunk's K/V rows arrive with the call: take them out of the pools and pass them as k_new, v_new
    k_new = case.k_pool[loc.long()].reshape(lq, -1).clone()
    v_new = case.v_pool[loc.long()].reshape(lq, -1).clone()
    k_before, v_before = case.k_pool.clone(), case.v_pool.clone()
    k_before[loc.long()] = 0
    v_before[loc.long()] = 0
    return case, qc, loc, k_new, v_new, k_before, v_before


@pytest.mark.parametrize("shape", SHAPES, ids=[s[0] for s in SHAPES])
def test_chunk_matches_oracle(shape):
    name, seed, n, lq, hq, hkv, d, n_init, n_local, top_k, base, dtype, tol = shape
    case, qc, loc, k_new, v_new, k_before, v_before = _chunk_case(seed, n, lq, hq, hkv, d, n_init, n_local, base, dtype)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, top_k, base, dtype, max_ctx=n + 8, max_batch=1,
                         prefill_chunk=512)
    dev = eng.device
    dbg = eng.new_debug_buffers(1)
    dbg["fingerprint"] = torch.zeros(hq * d, dtype=dtype, device=dev)
    kp, vp = k_before.to(dev), v_before.to(dev)
    out = eng.extend_chunk(0, qc.to(dev), k_new.to(dev), v_new.to(dev), loc.to(dev), kp, vp,
                           case.req_to_token.to(dev), case.req_pool_idx, n, debug=dbg)
    torch.cuda.synchronize()
    eng.raise_on_device_error()
    res = {k: v.cpu() for k, v in dbg.items()}
    # the chunk's rows are in the pools (token_retrieval.py:726-734)
    assert torch.equal(kp.cpu(), case.k_pool) and torch.equal(vp.cpu(), case.v_pool)
    # fingerprint: rotation at n_local + t, rounding, fixed-order mean -- bit for bit
    want_fp = orc.chunk_fingerprint(qc.view(lq, hq, d), n_local, base, 1.0)
    assert torch.equal(res["fingerprint"].view(hq, d), want_fp)
    o = orc.DecodeOracle(gu.oracle_config(eng))
    ref = o.extend_chunk(0, case.req_pool_idx, qc, None, None, None, case.k_pool, case.v_pool,
                         case.req_to_token[case.req_pool_idx], n, attn_dtype=torch.float64)
    assert int(res["flags"][0]) == ref["flag"]
    cnt = int(res["count"][0])
    if ref["flag"] == orc.FLAG_DENSE:
        assert cnt == n and torch.equal(res["positions"][0, :n], torch.arange(n, dtype=torch.int32))
    else:
        gu.check_selection(eng, res, 0, ref["positions"], ref["info"]["votes"], n)
    sl = res["slots"][0, :cnt]
    assert torch.equal(sl, case.req_to_token[case.req_pool_idx][res["positions"][0, :cnt].long()])
    # attention over the list the GPU selected (equal to the oracle's up to the tie band)
    sm_scale = d ** -0.5
    want = orc.sparse_prefill_attention(qc.view(lq, hq, d), case.k_pool, case.v_pool, sl, sm_scale, base, 1.0, 0.0,
                                        torch.float64).reshape(lq, -1)
    err = (out.cpu().double() - want).abs().max().item()
    assert err <= tol, err


def test_prefill_loop_through_the_patched_forward_then_decode():
    """A 1300-token prompt goes through ``RadixAttention.forward`` in EXTEND mode (three chunks: the first
    attends densely, the other two select), then one DECODE step; both against the oracle.  As in the
    reference's shipped configurations the local window is as long as a chunk."""
    hq, hkv, d, n_init, n_local, top_k, base, n = 8, 2, 128, 16, 512, 256, 5e5, 1300
    patcher.patch(rope_base=base, rope_scale=1, max_n_tokens=n + 64, top_k=top_k, n_init=n_init, n_local=n_local)
    dev = torch.device("cuda")
    case = synth.make_layer_case(41, n + 1, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    qs = synth.normal(41, 12, (n + 1, hq * d)).to(BF16) * 0.5 + case.q.view(1, -1)
    row = case.req_to_token[case.req_pool_idx]
    k_tok = case.k_pool[row[:n + 1].long()].reshape(n + 1, -1)
    v_tok = case.v_pool[row[:n + 1].long()].reshape(n + 1, -1)
    retr = patcher.ReqToTokenRetriever(1, d, hq, hkv, n + 64, BF16, max_reqs=2, max_batch=1)
    eng = retr.get_token_retriever(["r0"], [case.req_pool_idx])
    rtp = patcher.ReqToTokenPool(2, case.req_to_token.shape[1])
    rtp.req_to_token.copy_(case.req_to_token)
    kvp = patcher.TokenToKVPool(case.k_pool.shape[0], BF16, hkv, d, 1)
    attn = patcher.RadixAttention(hq, d, d ** -0.5, hkv, 0)
    meta = patcher.InputMetadata(
        forward_mode=patcher.ForwardMode.EXTEND, batch_size=1,
        req_pool_indices=torch.tensor([case.req_pool_idx], dtype=torch.int32, device=dev),
        seq_lens=torch.tensor([n], dtype=torch.int32, device=dev), req_to_token_pool=rtp, token_to_kv_pool=kvp,
        out_cache_loc=row[:n].to(dev), token_retriever=eng, req_pool_indices_cpu=[case.req_pool_idx],
        extend_prefix_lens_cpu=[0])
    out = attn(qs[:n].to(dev), k_tok[:n].to(dev), v_tok[:n].to(dev), meta)
    torch.cuda.synchronize()
    eng.raise_on_device_error()
    # oracle: the same chunk loop
    o = orc.DecodeOracle(gu.oracle_config(eng))
    kp, vp = torch.zeros_like(case.k_pool), torch.zeros_like(case.v_pool)
    flags = []
    for start in range(0, n, 512):
        end = min(start + 512, n)
        ref = o.extend_chunk(0, case.req_pool_idx, qs[start:end], k_tok[start:end], v_tok[start:end],
                             row[start:end], kp, vp, row, end, attn_dtype=torch.float64)
        flags.append(ref["flag"])
        err = (out[start:end].cpu().double() - ref["out"]).abs().max().item()
        assert err <= 2e-2, (start, err)
    assert flags == [orc.FLAG_DENSE, orc.FLAG_RECOMPUTE, orc.FLAG_RECOMPUTE]
    assert torch.equal(kvp.get_key_buffer(0).cpu(), kp) and torch.equal(kvp.get_value_buffer(0).cpu(), vp)
    # one decode step on top of the prefilled cache
    meta.forward_mode = patcher.ForwardMode.DECODE
    meta.seq_lens = torch.tensor([n + 1], dtype=torch.int32, device=dev)
    meta.out_cache_loc = row[n:n + 1].to(dev)
    od = attn(qs[n:n + 1].to(dev), k_tok[n:n + 1].to(dev), v_tok[n:n + 1].to(dev), meta)
    torch.cuda.synchronize()
    eng.raise_on_device_error()
    ref = o.decode_layer(0, qs[n:n + 1], k_tok[n:n + 1], v_tok[n:n + 1], row[n:n + 1], kp, vp, case.req_to_token,
                         torch.tensor([case.req_pool_idx]), torch.tensor([n + 1]), attn_dtype=torch.float64)
    assert (od.cpu().double() - ref["out"]).abs().max().item() <= 2e-2


def test_extend_argument_checks():
    eng = gu.make_engine(8, 2, 128, 16, 64, 256, 5e5, BF16, max_ctx=4096, max_batch=1, prefill_chunk=128)
    dev = eng.device
    kp = torch.zeros(4096, 2, 128, dtype=BF16, device=dev)
    rtt = torch.zeros(4, 4096, dtype=torch.int32, device=dev)
    q = torch.zeros(256, 8 * 128, dtype=BF16, device=dev)
    from tokenselect_b200._lib import TokenSelectError
    with pytest.raises(TokenSelectError) as e:          # chunk longer than the workspace was created for
        eng.extend_chunk(0, q, None, None, None, kp, kp.clone(), rtt, 1, 2000)
    assert e.value.status == 4
    with pytest.raises(TokenSelectError) as e:          # sequence shorter than the chunk
        eng.extend_chunk(0, q[:64], None, None, None, kp, kp.clone(), rtt, 1, 10)
    assert e.value.status == 1
    eng2 = gu.make_engine(8, 2, 128, 16, 64, 256, 5e5, BF16, max_ctx=4096, max_batch=1, prefill_chunk=0)
    with pytest.raises(ValueError):
        eng2.extend_chunk(0, q[:64], None, None, None, kp, kp.clone(), rtt, 1, 100)


def test_selection_cache_across_chunks_and_decode():
    """Selection cache on: two consecutive chunks with similar queries and a decode step.  The reuse
    decisions (cosine of the new scoring query against the cached fingerprint, fixed fp32 order) and the
    emitted positions must equal the oracle's."""
    hq, hkv, d, n_init, n_local, top_k, base = 8, 2, 128, 16, 64, 256, 5e5
    n_total, lq = 2200, 64
    case = synth.make_layer_case(51, n_total, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, top_k, base, BF16, max_ctx=n_total + 8, max_batch=1,
                         prefill_chunk=512, query_cache=True, similarity_threshold=0.9)
    dev = eng.device
    eng.reset_request(case.req_pool_idx)
    o = orc.DecodeOracle(gu.oracle_config(eng))
    o.reset_request(case.req_pool_idx)
    kp, vp, rtt = case.k_pool.to(dev), case.v_pool.to(dev), case.req_to_token.to(dev)
    row = case.req_to_token[case.req_pool_idx]
    q1 = synth.make_chunk_queries(51, case, lq, hq, d, spread=0.3)
    q2 = synth.make_chunk_queries(52, case, lq, hq, d, spread=0.3)      # same direction, other noise
    q3 = -q1                                                             # opposite direction
    flags = []
    for step, (qc, n) in enumerate(((q1, 2000), (q2, 2064), (q3, 2128))):
        dbg = eng.new_debug_buffers(1)
        eng.extend_chunk(0, qc.to(dev), None, None, None, kp, vp, rtt, case.req_pool_idx, n, debug=dbg)
        torch.cuda.synchronize()
        eng.raise_on_device_error()
        ref = o.extend_chunk(0, case.req_pool_idx, qc, None, None, None, case.k_pool, case.v_pool, row, n)
        res = {k: v.cpu() for k, v in dbg.items()}
        assert int(res["flags"][0]) == ref["flag"], (step, ref["info"].get("cos"))
        flags.append(ref["flag"])
        if ref["flag"] == orc.FLAG_RECOMPUTE:
            gu.check_selection(eng, res, 0, ref["positions"], ref["info"]["votes"], n)
            # keep the oracle's cached set equal to the GPU's (they may differ inside the tie band)
            o.cache[(case.req_pool_idx, 0)].topk_positions = res["positions"][0, n_init:n_init + top_k].long().clone()
        else:
            assert torch.equal(res["positions"][0, : eng.cfg.n_sel].long(), ref["positions"].long())
    assert flags == [orc.FLAG_RECOMPUTE, orc.FLAG_REUSE, orc.FLAG_RECOMPUTE]
    assert eng.counters(case.req_pool_idx) == (3, 1)


@pytest.mark.parametrize("dtype,tol", [(BF16, 2e-2), (F32, 1e-5)], ids=["bf16", "fp32"])
def test_rope_scale_and_soft_cap_decode_and_chunk(dtype, tol):
    """rope_scale != 1 (scoring position n_local * scale, attention frequencies / scale) and a logit soft
    cap, through a decode step and a prefill chunk of the same request."""
    hq, hkv, d, n_init, n_local, top_k, base, n, lq = 8, 2, 128, 16, 64, 256, 5e5, 2500, 96
    scale, cap = 4.0, 20.0
    case = synth.make_layer_case(71, n, hq, hkv, d, n_init, n_local, base, rope_scale=scale, dtype=dtype)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, top_k, base, dtype, max_ctx=n + 8, max_batch=1,
                         rope_scale=scale, logit_cap=cap, prefill_chunk=512)
    o = orc.DecodeOracle(gu.oracle_config(eng))
    row = case.req_to_token[case.req_pool_idx]
    # decode
    out, res = gu.run_gpu(eng, 0, *gu.case_tensors(case))
    flag, pos, info = o.select(0, case.req_pool_idx, case.q.view(hq, d), case.k_pool, row, n)
    gu.check_selection(eng, res, 0, pos, info["votes"], n)
    sl = res["slots"][0, : eng.cfg.n_sel]
    want = orc.sparse_attention(case.q.view(hq, d), case.k_pool, case.v_pool, sl, d ** -0.5, base, scale, cap,
                                torch.float64).reshape(-1)
    assert (out[0].double() - want).abs().max().item() <= tol
    # prefill chunk
    dev = eng.device
    qc = synth.make_chunk_queries(71, case, lq, hq, d)
    dbg = eng.new_debug_buffers(1)
    dbg["fingerprint"] = torch.zeros(hq * d, dtype=dtype, device=dev)
    out2 = eng.extend_chunk(0, qc.to(dev), None, None, None, case.k_pool.to(dev), case.v_pool.to(dev),
                            case.req_to_token.to(dev), case.req_pool_idx, n, debug=dbg)
    torch.cuda.synchronize()
    eng.raise_on_device_error()
    res2 = {k: v.cpu() for k, v in dbg.items()}
    assert torch.equal(res2["fingerprint"].view(hq, d), orc.chunk_fingerprint(qc.view(lq, hq, d), n_local, base, scale))
    ref = o.extend_chunk(0, case.req_pool_idx, qc, None, None, None, case.k_pool, case.v_pool, row, n)
    gu.check_selection(eng, res2, 0, ref["positions"], ref["info"]["votes"], n)
    sl2 = res2["slots"][0, : eng.cfg.n_sel]
    want2 = orc.sparse_prefill_attention(qc.view(lq, hq, d), case.k_pool, case.v_pool, sl2, d ** -0.5, base, scale, cap,
                                         torch.float64).reshape(lq, -1)
    assert (out2.cpu().double() - want2).abs().max().item() <= tol


@pytest.mark.parametrize("flags", [8, 16, 512], ids=["mma_sync_kernel", "four_threads_per_row", "narrow_key_blocks"])
def test_diagnostic_attention_variants_agree(flags):
    """The diagnostic variants of the prefill attention (TS_CFG_EXTEND_MMA_SYNC, TS_CFG_EXTEND_FOUR_PER_ROW,
    TS_CFG_EXTEND_NARROW_BLOCKS) against the oracle on a full chunk and a tail chunk."""
    hq, hkv, d, n_init, n_local, top_k, base = 8, 2, 128, 16, 512, 256, 5e5
    for seed, n, lq in ((91, 3000, 512), (92, 2100, 77)):
        case = synth.make_layer_case(seed, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
        qc = synth.make_chunk_queries(seed, case, lq, hq, d)
        eng = gu.make_engine(hq, hkv, d, n_init, n_local, top_k, base, BF16, max_ctx=n + 8, max_batch=1,
                             prefill_chunk=512, extra_flags=flags)
        dev = eng.device
        dbg = eng.new_debug_buffers(1)
        out = eng.extend_chunk(0, qc.to(dev), None, None, None, case.k_pool.to(dev), case.v_pool.to(dev),
                               case.req_to_token.to(dev), case.req_pool_idx, n, debug=dbg)
        torch.cuda.synchronize()
        eng.raise_on_device_error()
        sl = dbg["slots"][0, : int(dbg["count"][0])].cpu()
        want = orc.sparse_prefill_attention(qc.view(lq, hq, d), case.k_pool, case.v_pool, sl, d ** -0.5, base, 1.0, 0.0,
                                            torch.float64).reshape(lq, -1)
        assert (out.cpu().double() - want).abs().max().item() <= 2e-2
