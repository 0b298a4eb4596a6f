"""CUDA path against the CPU oracle, through the C ABI, on seeded inputs.

Tolerances (from the parity rules of this path):
  * selected index set: identical to the oracle except indices whose vote lies within 1e-4
    (relative) of the k-th vote; ascending order; init / local windows exact;
  * attention output: <= 2e-2 absolute for bf16, <= 1e-5 absolute in fp32 check mode;
  * scoring-query rotation: bit-exact; logits: 2e-3 absolute (fp32 summation order).
"""
import numpy as np
import pytest
import torch

from oracle import synth
from oracle import tokenselect_oracle as orc
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu

BF16, F32 = torch.bfloat16, torch.float32
ATTN_TOL = {BF16: 2e-2, F32: 1e-5}

# name, hq, hkv, d, N, n_init, n_local, top_k, rope_base, dtype, extra engine kwargs
SHAPES = [
    ("llama_tp1_bf16", 32, 8, 128, 8192, 128, 512, 1024, 5e5, BF16, {}),
    ("qwen_tp1_bf16", 28, 4, 128, 4096, 128, 512, 512, 1e6, BF16, {}),
    ("llama_tp4_bf16", 8, 2, 128, 3000, 16, 64, 256, 5e5, BF16, {}),
    ("llama_tp8_bf16", 4, 1, 128, 5000, 16, 64, 256, 5e5, BF16, {}),
    ("qwen_tp4_bf16", 7, 1, 128, 3001, 16, 64, 300, 1e6, BF16, {}),
    ("divmap_bf16", 8, 2, 128, 2500, 16, 64, 256, 5e5, BF16, {"gqa_map": "div"}),
    # the two bf16 scoring paths forced against their default row sizes
    ("direct_llama_tp1", 32, 8, 128, 8192, 128, 512, 1024, 5e5, BF16, {"score_path": "direct"}),
    ("direct_qwen_tp1", 28, 4, 128, 4096, 128, 512, 512, 1e6, BF16, {"score_path": "direct"}),
    ("direct_llama_tp4", 8, 2, 128, 3000, 16, 64, 256, 5e5, BF16, {"score_path": "direct"}),
    ("direct_llama_tp8", 4, 1, 128, 5000, 16, 64, 256, 5e5, BF16, {"score_path": "direct"}),
    ("plain_bf16", 8, 2, 128, 2048, 16, 64, 256, 5e5, BF16, {"plain_score": True}),
    # the general selection kernel followed by the stand-alone attention kernels (TS_CFG_SPLIT_ATTEND) at shapes
    # that default to the single layer-step kernel
    ("split_attend_llama_tp1", 32, 8, 128, 8192, 128, 512, 1024, 5e5, BF16, {"extra_flags": 256}),
    ("split_attend_qwen_tp4", 7, 1, 128, 3001, 16, 64, 300, 1e6, BF16, {"extra_flags": 256}),
    ("softcap_bf16", 8, 2, 128, 1500, 16, 64, 256, 5e5, BF16, {"logit_cap": 30.0}),
    ("fp32_check", 32, 8, 128, 8192, 128, 512, 1024, 5e5, F32, {}),
    ("fp32_d64_mha", 4, 4, 64, 1024, 8, 32, 128, 1e4, F32, {}),
    ("softcap_fp32", 8, 2, 128, 1500, 16, 64, 256, 5e5, F32, {"logit_cap": 30.0}),
]


@pytest.mark.parametrize("shape", SHAPES, ids=[s[0] for s in SHAPES])
def test_layer_step_matches_oracle(shape):
    name, hq, hkv, d, n, n_init, n_local, k, base, dtype, kw = shape
    seed = 100 + SHAPES.index(shape)
    case = synth.make_layer_case(seed, n, hq, hkv, d, n_init, n_local, base, dtype=dtype,
                                 gqa_map=kw.get("gqa_map", "mod"))
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, dtype, max_ctx=n + 8, **kw)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    out, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens)

    o = orc.DecodeOracle(gu.oracle_config(eng))
    ref = o.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens)
    info = ref["info"][0]
    assert int(res["flags"][0]) == orc.FLAG_RECOMPUTE == ref["flags"][0]

    # scoring query: bit-exact
    nc = n - n_init - n_local
    q_rot = eng.debug_read(0, hq * d, dtype)
    assert torch.equal(q_rot.view(hq, d), info["q_rot"]), "rotated scoring query differs"

    # logits
    lg = eng.debug_read(1, nc * hq, F32).view(nc, hq).numpy()
    want_lg = orc.score_logits(info["q_rot"], kp, rtt[case.req_pool_idx][n_init: n - n_local], eng.cfg.gqa_map)
    cols = gu.logits_columns_to_heads(eng)
    np.testing.assert_allclose(lg, want_lg.numpy()[cols].T, rtol=1e-5, atol=2e-3)

    # votes
    votes = eng.debug_read(2, nc, F32).numpy()
    np.testing.assert_allclose(votes, info["votes"].numpy(), rtol=2e-3, atol=1e-30)
    assert abs(votes.sum() - hq) < 1e-2 * hq

    # selection
    pos = gu.check_selection(eng, res, 0, ref["positions"][0], info["votes"], n)
    slots = res["slots"][0, : eng.cfg.n_sel]
    assert torch.equal(slots, rtt[case.req_pool_idx][torch.from_numpy(pos).long()])

    # attention over the rows the CUDA path selected
    want = orc.sparse_attention(q.view(hq, d), kp, vp, slots, eng.cfg.sm_scale or d ** -0.5, base, 1.0,
                                eng.cfg.logit_cap, torch.float64).reshape(-1)
    err = (out[0].double() - want).abs().max().item()
    assert err <= ATTN_TOL[dtype], f"attention error {err}"
    if np.array_equal(pos, ref["positions"][0].numpy()):
        err2 = (out[0].float() - ref["out"][0]).abs().max().item()
        assert err2 <= ATTN_TOL[dtype] + 1e-6


def _multi_request(seed, lens, hq, hkv, d, dtype, pool_rows, max_ctx, max_reqs, req_slots):
    """Several requests sharing one pool, rows scattered by a seeded permutation."""
    perm = synth.permutation(seed, 50, pool_rows)
    k_pool = synth.normal(seed, 51, (pool_rows, hkv, d)).to(dtype)
    v_pool = synth.normal(seed, 52, (pool_rows, hkv, d)).to(dtype)
    rtt = torch.full((max_reqs, max_ctx), -1, dtype=torch.int32)
    at = 0
    for n, slot in zip(lens, req_slots):
        rtt[slot, :n] = perm[at: at + n].to(torch.int32)
        at += n
    q = synth.normal(seed, 53, (len(lens), hq * d)).to(dtype)
    return q, k_pool, v_pool, rtt


@pytest.mark.parametrize("dtype,flags", [(BF16, 0), (BF16, 1024), (F32, 0)], ids=["bf16", "bf16_inline_attention", "fp32"])
def test_ragged_batch_with_dense_requests(dtype, flags):
    """Requests of different lengths in one call, some below the guard (attend to everything), at
    the guard boundary (N == n_sel and N == n_sel + 1), and one shorter than n_init.  Batches take the
    selection kernel followed by the attention kernels by default; TS_CFG_INLINE_ATTEND (1024) keeps the
    attention inside the layer-step kernel."""
    hq, hkv, d, n_init, n_local, k, base = 8, 2, 128, 16, 64, 256, 5e5
    n_sel = n_init + k + n_local
    lens = [2000, n_sel, n_sel + 1, 5, 1177, 40]
    slots = [3, 0, 5, 1, 2, 4]
    q, kp, vp, rtt = _multi_request(7, lens, hq, hkv, d, dtype, 6000, 2100, 6, slots)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, dtype, max_ctx=2100, max_reqs=6, max_batch=6,
                         extra_flags=flags)
    ridx, sl = torch.tensor(slots), torch.tensor(lens)
    out, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, sl)
    ref = orc.DecodeOracle(gu.oracle_config(eng)).decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, sl)
    for b, n in enumerate(lens):
        assert int(res["flags"][b]) == ref["flags"][b]
        if ref["flags"][b] == orc.FLAG_DENSE:
            assert int(res["count"][b]) == n
            assert torch.equal(res["positions"][b, :n], torch.arange(n, dtype=torch.int32))
            assert torch.equal(res["slots"][b, :n], rtt[slots[b], :n])
        else:
            gu.check_selection(eng, res, b, ref["positions"][b], ref["info"][b]["votes"], n)
        cnt = int(res["count"][b])
        want = orc.sparse_attention(q[b].view(hq, d), kp, vp, res["slots"][b, :cnt], d ** -0.5, base, 1.0, 0.0,
                                    torch.float64).reshape(-1)
        assert (out[b].double() - want).abs().max().item() <= ATTN_TOL[dtype]


def test_exact_ties_take_lowest_positions():
    """All candidate keys equal -> all votes equal -> the k lowest candidate positions win."""
    hq, hkv, d, n_init, n_local, k, base, n = 8, 2, 128, 16, 64, 256, 5e5, 3000
    case = synth.make_layer_case(11, n, hq, hkv, d, n_init, n_local, base, dtype=BF16, planted_frac=0.0)
    rows = case.req_to_token[case.req_pool_idx][:n].long()
    case.k_pool[rows] = case.k_pool[rows[0]].clone()
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    out, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens)
    pos = res["positions"][0, : eng.cfg.n_sel]
    assert torch.equal(pos[: n_init + k], torch.arange(n_init + k, dtype=torch.int32))
    assert torch.isfinite(out.float()).all()


def test_pairwise_ties_break_by_position():
    """Every candidate key appears twice (positions p and p + Nc/2): votes tie in pairs, and where the
    k-th vote's pair straddles the boundary the lower position must be the one taken."""
    hq, hkv, d, n_init, n_local, k, base = 8, 2, 128, 16, 64, 255, 5e5
    nc = 2000
    n = n_init + nc + n_local
    case = synth.make_layer_case(12, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    row = case.req_to_token[case.req_pool_idx]
    lo = row[n_init: n_init + nc // 2].long()
    hi = row[n_init + nc // 2: n_init + nc].long()
    case.k_pool[hi] = case.k_pool[lo]
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    _, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens)
    ref = orc.DecodeOracle(gu.oracle_config(eng)).decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens)
    votes = eng.debug_read(2, nc, F32).numpy()
    assert np.array_equal(votes[: nc // 2], votes[nc // 2:]), "duplicated keys must give identical votes"
    got = res["positions"][0, n_init: n_init + k].numpy() - n_init
    # exact rule on the CUDA path's own votes: sort by (-vote, position)
    order = np.lexsort((np.arange(nc), -votes.astype(np.float64)))[:k]
    assert np.array_equal(got, np.sort(order))
    gu.check_selection(eng, res, 0, ref["positions"][0], ref["info"][0]["votes"], n)


@pytest.mark.parametrize("ks", [5, 6, 1, 32])
def test_vote_max_pool(ks):
    hq, hkv, d, n_init, n_local, k, base, n = 8, 2, 128, 16, 64, 256, 5e5, 2048
    case = synth.make_layer_case(20 + ks, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8, kernel_size=ks)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    _, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens)
    ref = orc.DecodeOracle(gu.oracle_config(eng)).decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens)
    pooled = ref["info"][0]["votes"]
    nc = n - n_init - n_local
    assert pooled.numel() == (nc if ks % 2 else nc - 1)
    got = eng.debug_read(2, pooled.numel(), F32).numpy()
    np.testing.assert_allclose(got, pooled.numpy(), rtol=2e-3, atol=1e-30)
    # max-pooling creates runs of equal votes; compare with the exact rule on the CUDA path's own votes
    sel = res["positions"][0, n_init: n_init + k].numpy() - n_init
    order = np.lexsort((np.arange(got.size), -got.astype(np.float64)))[:k]
    assert np.array_equal(sel, np.sort(order))


def test_kv_append_then_attend():
    """k_new / v_new are written to the pools at out_cache_loc before selection and attention."""
    hq, hkv, d, n_init, n_local, k, base, n = 8, 2, 128, 16, 64, 256, 5e5, 1500
    case = synth.make_layer_case(31, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    loc = rtt[case.req_pool_idx, n - 1: n].clone()
    k_new = synth.normal(31, 60, (1, hkv * d)).to(BF16)
    v_new = synth.normal(31, 61, (1, hkv * d)).to(BF16)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8)
    out, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens, k_new, v_new, loc)
    assert torch.equal(res["k_pool"][loc.long()].reshape(1, -1), k_new)
    assert torch.equal(res["v_pool"][loc.long()].reshape(1, -1), v_new)
    kp2, vp2 = kp.clone(), vp.clone()
    ref = orc.DecodeOracle(gu.oracle_config(eng)).decode_layer(0, q, k_new, v_new, loc, kp2, vp2, rtt, ridx, lens)
    gu.check_selection(eng, res, 0, ref["positions"][0], ref["info"][0]["votes"], n)
    want = orc.sparse_attention(q.view(hq, d), kp2, vp2, res["slots"][0, : eng.cfg.n_sel], d ** -0.5, base, 1.0,
                                0.0, torch.float64).reshape(-1)
    assert (out[0].double() - want).abs().max().item() <= ATTN_TOL[BF16]


def test_bad_pool_row_is_reported_not_dereferenced():
    hq, hkv, d, n_init, n_local, k, base, n = 8, 2, 128, 16, 64, 256, 5e5, 1200
    case = synth.make_layer_case(41, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    rtt = rtt.clone()
    rtt[case.req_pool_idx, 500] = kp.shape[0] + 123
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8)
    dev = eng.device
    eng.decode_layer(0, q.to(dev), None, None, None, kp.to(dev), vp.to(dev), rtt.to(dev),
                     ridx.to(device=dev, dtype=torch.int32), lens.to(device=dev, dtype=torch.int32))
    torch.cuda.synchronize()
    code, detail = eng.last_error()
    assert code == 6 and detail == kp.shape[0] + 123
    # the error word is cleared by the read; the handle keeps working
    out, _ = gu.run_gpu(eng, 0, q, kp, vp, case.req_to_token, ridx, lens)
    assert torch.isfinite(out.float()).all()


def test_workspace_capacity_is_checked_on_the_device():
    hq, hkv, d, n_init, n_local, k, base, n = 8, 2, 128, 16, 64, 256, 5e5, 3000
    case = synth.make_layer_case(42, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8, max_batch=1, max_total=1024)
    dev = eng.device
    eng.decode_layer(0, q.to(dev), None, None, None, kp.to(dev), vp.to(dev), rtt.to(dev),
                     ridx.to(device=dev, dtype=torch.int32), lens.to(device=dev, dtype=torch.int32))
    torch.cuda.synchronize()
    code, _ = eng.last_error()
    assert code == 4


def test_invalid_arguments_are_rejected_on_the_host():
    eng = gu.make_engine(8, 2, 128, 16, 64, 256, 5e5, BF16, max_ctx=4096, max_batch=2)
    dev = eng.device
    q = torch.zeros(3, 8 * 128, dtype=BF16, device=dev)
    pool = torch.zeros(64, 2, 128, dtype=BF16, device=dev)
    rtt = torch.zeros(4, 4096, dtype=torch.int32, device=dev)
    idx = torch.zeros(3, dtype=torch.int32, device=dev)
    from tokenselect_b200 import TokenSelectError
    with pytest.raises(TokenSelectError) as ei:
        eng.decode_layer(0, q, None, None, None, pool, pool.clone(), rtt, idx, idx)   # batch 3 > max_batch 2
    assert ei.value.status == 4
    with pytest.raises(TokenSelectError):
        eng.decode_layer(7, q[:1], None, None, None, pool, pool.clone(), rtt, idx[:1], idx[:1])  # layer out of range
    with pytest.raises(ValueError):
        eng.decode_layer(0, q[:1].float(), None, None, None, pool, pool.clone(), rtt, idx[:1], idx[:1])


@pytest.mark.parametrize("gain", [6.0, 20.0], ids=["peaked", "very_peaked"])
def test_underflowing_votes(gain):
    """A query scaled until almost every softmax term underflows: most votes are denormal or exactly zero.
    Votes in the normal fp32 range must select exactly as in the oracle; where the k-th vote itself is
    denormal or zero, the two evaluations (division folded into the exponent here, exp then divide in the
    oracle) may disagree only among candidates whose oracle vote is below 2^-120, and zeros are taken from
    the lowest positions."""
    hq, hkv, d, n_init, n_local, k, base, n = 8, 2, 128, 16, 64, 256, 5e5, 3000
    case = synth.make_layer_case(61, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    case.q.mul_(gain)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8)
    out, res = gu.run_gpu(eng, 0, *gu.case_tensors(case))
    o = orc.DecodeOracle(gu.oracle_config(eng))
    flag, pos, info = o.select(0, case.req_pool_idx, case.q.view(hq, d), case.k_pool,
                               case.req_to_token[case.req_pool_idx], n)
    votes = info["votes"].double().numpy()
    got = res["positions"][0, n_init:n_init + k].numpy() - n_init
    want = pos[n_init:n_init + k].numpy() - n_init
    assert int(res["count"][0]) == eng.cfg.n_sel and np.all(np.diff(got) > 0)
    kth = np.sort(votes)[::-1][k - 1]
    diff = set(got.tolist()) ^ set(want.tolist())
    tiny = 2.0 ** -120
    if kth >= tiny:
        ok, why = orc.index_sets_match(got, want, votes, k, rel_tol=1e-4)
        assert ok, why
    else:
        assert all(votes[i] < tiny for i in diff), sorted(votes[list(diff)])[-3:]
        # everything in the normal range is in
        assert set(np.nonzero(votes >= tiny)[0].tolist()) <= set(got.tolist())
    assert torch.isfinite(out.float()).all()


def test_phase_stamps_only_with_the_diagnostic_flag():
    """TS_CFG_PHASE_STAMPS (32): CTA 0 records nanosecond timestamps at the selection kernel's phase boundaries,
    read back with ts_debug_read(3).  Without the flag the kernels read no timer and the slots stay zero; the
    results are the same either way."""
    hq, hkv, d, n_init, n_local, top_k, base, n = 8, 2, 128, 16, 64, 256, 5e5, 3000
    case = synth.make_layer_case(97, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    outs = []
    for flags in (0, 32):
        eng = gu.make_engine(hq, hkv, d, n_init, n_local, top_k, base, BF16, max_ctx=n + 8, max_batch=1,
                             extra_flags=flags)
        out, dbg = gu.run_gpu(eng, 0, *gu.case_tensors(case))
        eng.raise_on_device_error()
        ts = eng.debug_read(3, 64, torch.int64)
        if flags == 0:
            assert int(ts.abs().sum()) == 0
        else:
            phase = ts[:9]                        # start, plan, score, barrier, vote, barrier, filter, barrier, emit
            assert int(phase.min()) > 0 and bool((phase[1:] >= phase[:-1]).all())
        outs.append((out, dbg["slots"]))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
