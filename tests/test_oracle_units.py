"""Unit checks of the CPU oracle itself (no GPU)."""
import numpy as np
import pytest
import torch

from oracle import synth
from oracle import tokenselect_oracle as orc


def test_fixed_order_cosine_terms_are_close_to_float64():
    q = synth.normal(1, 1, (4096,)).numpy()
    c = (0.9 * torch.from_numpy(q) + 0.3 * synth.normal(1, 2, (4096,))).numpy()
    t = orc.cosine_terms_fixed_order(q, c)
    want = np.array([np.dot(q.astype(np.float64), c), np.dot(q.astype(np.float64), q), np.dot(c.astype(np.float64), c)])
    np.testing.assert_allclose(t, want, rtol=1e-5)
    cos = orc.cosine_from_terms(t)
    assert abs(float(cos) - want[0] / np.sqrt(want[1] * want[2])) < 1e-6
    assert orc.cache_says_recompute(np.float32(0.89999), 0.9) and not orc.cache_says_recompute(np.float32(0.9), 0.9)


@pytest.mark.parametrize("ks,expect", [(5, 20), (6, 19), (12, 19), (32, 19), (1, 20), (-1, 20), (0, 20)])
def test_max_pool_length(ks, expect):
    v = torch.arange(20, dtype=torch.float32)
    assert orc.max_pool_votes(v, ks).numel() == expect


def test_topk_ties_prefer_low_positions():
    v = torch.tensor([1.0, 3.0, 3.0, 2.0, 3.0, 0.5])
    assert orc.topk_sorted(v, 2).tolist() == [1, 2]
    assert orc.topk_sorted(v, 4).tolist() == [1, 2, 3, 4]


def test_guard_and_union_layout():
    cfg = orc.OracleConfig(1, 4, 2, 64, 4, 8, 16, 1e4)
    o = orc.DecodeOracle(cfg)
    c = synth.make_layer_case(9, 29, 4, 2, 64, 4, 8, 1e4)
    flag, pos, _ = o.select(0, 1, c.q.view(4, 64), c.k_pool, c.req_to_token[1], 28)
    assert flag == orc.FLAG_DENSE and pos.tolist() == list(range(28))
    flag, pos, info = o.select(0, 1, c.q.view(4, 64), c.k_pool, c.req_to_token[1], 29)
    assert flag == orc.FLAG_RECOMPUTE and pos.numel() == 28 and info["votes"].numel() == 17
    assert pos[:4].tolist() == [0, 1, 2, 3] and pos[-8:].tolist() == list(range(21, 29))


def test_tp_emulation_matches_single_rank_when_one_kv_head_per_rank_uses_div_map():
    """With one KV head per rank the rank-local `%` map equals the conventional `//` map."""
    c = synth.make_layer_case(10, 1500, 8, 4, 64, 8, 32, 1e4)
    a = orc.DecodeOracle(orc.OracleConfig(1, 8, 4, 64, 8, 32, 128, 1e4), tp_ranks=4)
    b = orc.DecodeOracle(orc.OracleConfig(1, 8, 4, 64, 8, 32, 128, 1e4, gqa_map="div"))
    _, pa, _ = a.select(0, 1, c.q.view(8, 64), c.k_pool, c.req_to_token[1], 1500)
    _, pb, _ = b.select(0, 1, c.q.view(8, 64), c.k_pool, c.req_to_token[1], 1500)
    assert torch.equal(pa, pb)


def test_selection_cache_rule():
    cfg = orc.OracleConfig(1, 4, 2, 64, 4, 8, 16, 1e4, query_cache=True, similarity_threshold=0.9)
    o = orc.DecodeOracle(cfg)
    c = synth.make_layer_case(11, 200, 4, 2, 64, 4, 8, 1e4)
    q = c.q.view(4, 64)
    f1, p1, _ = o.select(0, 1, q, c.k_pool, c.req_to_token[1], 199)
    f2, p2, i2 = o.select(0, 1, q * 1.5, c.k_pool, c.req_to_token[1], 200)      # same direction -> reuse
    f3, _, _ = o.select(0, 1, -q, c.k_pool, c.req_to_token[1], 200)            # opposite -> recompute
    assert (f1, f2, f3) == (orc.FLAG_RECOMPUTE, orc.FLAG_REUSE, orc.FLAG_RECOMPUTE)
    assert torch.equal(p1[4:20], p2[4:20]) and p2[-1] == 199 and abs(i2["cos"] - 1.0) < 1e-5
    assert o.retrieval_count[1] == 3 and o.skip_count[1] == 1
    o.reset_request(1)
    f4, _, _ = o.select(0, 1, q, c.k_pool, c.req_to_token[1], 200)
    assert f4 == orc.FLAG_RECOMPUTE and o.retrieval_count[1] == 1


def test_prefill_attention_rows_equal_decode_attention_on_prefixes():
    """Query i of a chunk sees the listed keys up to its own position, rotated as a decode query at that
    position would be: row i of the causal chunk attention equals decode attention over the list prefix."""
    torch.manual_seed(3)
    hq, hkv, d, n, lq = 4, 2, 64, 40, 7
    kp, vp = torch.randn(64, hkv, d), torch.randn(64, hkv, d)
    slots = torch.randperm(64)[:n].to(torch.int32)
    q = torch.randn(lq, hq, d)
    out = orc.sparse_prefill_attention(q, kp, vp, slots, d ** -0.5, 1e4, 1.0, 0.0, torch.float64)
    for i in (0, 3, lq - 1):
        want = orc.sparse_attention(q[i], kp, vp, slots[: n - lq + i + 1], d ** -0.5, 1e4, 1.0, 0.0, torch.float64)
        assert (out[i] - want).abs().max().item() < 1e-12


def test_chunk_fingerprint_fixed_order_matches_torch_mean():
    torch.manual_seed(4)
    q = torch.randn(100, 4, 64).bfloat16()
    a = orc.chunk_fingerprint(q, 16, 1e4, 1.0, True).float()
    b = orc.chunk_fingerprint(q, 16, 1e4, 1.0, False).float()
    # identical up to the last bf16 bit where the fp32 sums round differently
    assert (a - b).abs().max().item() <= 2 ** -8 * b.abs().max().item()
    one = orc.chunk_fingerprint(q[:1], 16, 1e4, 1.0, True)
    assert torch.equal(one, orc.rotate_scoring_query(q[0], 16, 1e4, 1.0))


def test_batched_fixed_order_cosine_terms_equal_the_single_pair_form_bitwise():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((5, 1024)).astype(np.float32)
    c = rng.standard_normal((5, 1024)).astype(np.float32)
    got = orc.cosine_terms_fixed_order_batch(q, c)
    for i in range(5):
        assert np.array_equal(got[i], orc.cosine_terms_fixed_order(q[i], c[i]))
