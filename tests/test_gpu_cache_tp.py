"""Selection cache, tensor-parallel split, golden vectors and full-size properties on the GPU."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import synth
from oracle import tokenselect_oracle as orc
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


def _ar1_queries(seed, steps, hq, d, rho, dtype):
    """q_t = rho*q_{t-1} + sqrt(1-rho^2)*eps_t, eps ~ N(0,1) per element."""
    eps = synth.normal(seed, 70, (steps, hq * d))
    q = torch.empty_like(eps)
    q[0] = eps[0]
    for t in range(1, steps):
        q[t] = rho * q[t - 1] + (1 - rho * rho) ** 0.5 * eps[t]
    return q.to(dtype)


_PAIRS = [(rho, theta) for rho in (0.80, 0.95, 0.99) for theta in (0.85, 0.90, 0.95)]


@pytest.mark.parametrize("dtype,rho,theta",
                         [(F32 if (rho, theta) in ((0.99, 0.95), (0.80, 0.90)) else BF16, rho, theta) for rho, theta in _PAIRS],
                         ids=[f"rho{int(r * 100)}_theta{int(t * 100)}" for r, t in _PAIRS])
def test_selection_cache_decisions_are_bit_exact(dtype, rho, theta):
    """Reuse / recompute decisions per (request, layer, step) equal the oracle's replay of the same
    fixed-order fp32 cosine, for every (rho, threshold) pair of the cache-stress configuration; the sequence
    grows by one token per step; two layers keep separate state.  A query sequence with a step inside the 1e-5
    band around the threshold (where fp32 and fp64 may disagree) is replaced by the next seed's, never skipped."""
    hq, hkv, d, n_init, n_local, k, base = 8, 2, 128, 16, 64, 256, 5e5
    n0, steps, layers = 1200, 20, 2
    case = synth.make_layer_case(55, n0 + steps, hq, hkv, d, n_init, n_local, base, dtype=dtype)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, dtype, n_layers=layers, max_ctx=n0 + steps + 8,
                         query_cache=True, similarity_threshold=theta)
    _, kp, vp, rtt, ridx, _ = gu.case_tensors(case)

    def run(seed):
        qs = _ar1_queries(seed, steps, hq, d, rho, dtype)
        o = orc.DecodeOracle(gu.oracle_config(eng))
        eng.reset_request(case.req_pool_idx)
        o.reset_request(case.req_pool_idx)
        reuse = checked = 0
        for t in range(steps):
            lens = torch.tensor([n0 + t])
            for layer in range(layers):
                q = (qs[t] if layer == 0 else -qs[t].flip(0))[None].contiguous()
                out, res = gu.run_gpu(eng, layer, q, kp, vp, rtt, ridx, lens)
                ref = o.decode_layer(layer, q, None, None, None, kp, vp, rtt, ridx, lens)
                cos = ref["info"][0].get("cos")
                if cos is not None and abs(cos - theta) < 1e-5:
                    return None                                # inside the band: try the next seed
                assert int(res["flags"][0]) == ref["flags"][0], f"seed {seed} step {t} layer {layer}: cos={cos}"
                checked += 1
                if ref["flags"][0] == orc.FLAG_REUSE:
                    reuse += 1
                    assert torch.equal(res["positions"][0, : eng.cfg.n_sel].long(), ref["positions"][0])
                else:
                    gu.check_selection(eng, res, 0, ref["positions"][0], ref["info"][0]["votes"], n0 + t)
                    # keep both caches on the same index set even if a tie-band index differs
                    o.cache[(case.req_pool_idx, layer)].topk_positions = \
                        res["positions"][0, n_init: n_init + k].long().clone()
                want = orc.sparse_attention(q.view(hq, d), kp, vp, res["slots"][0, : eng.cfg.n_sel], d ** -0.5, base,
                                            1.0, 0.0, torch.float64).reshape(-1)
                assert (out[0].double() - want).abs().max().item() <= (2e-2 if dtype == BF16 else 1e-5)
        retr, skips = eng.counters(case.req_pool_idx)
        assert retr == checked == o.retrieval_count[case.req_pool_idx]
        assert skips == reuse == o.skip_count[case.req_pool_idx]
        return reuse, qs

    done = None
    for seed in range(56, 64):
        done = run(seed)
        if done is not None:
            break
    assert done is not None, "eight query sequences in a row had a step inside the 1e-5 band"
    reuse, qs = done
    if rho >= 0.95 and theta <= 0.9:
        assert reuse > 0, "expected some reuse at this correlation"
    # a new request in the slot starts from scratch
    eng.reset_request(case.req_pool_idx)
    assert eng.counters(case.req_pool_idx) == (0, 0)
    _, res = gu.run_gpu(eng, 0, qs[steps - 1][None].contiguous(), kp, vp, rtt, ridx, torch.tensor([n0 + steps]))
    assert int(res["flags"][0]) == orc.FLAG_RECOMPUTE


@pytest.mark.parametrize("tp,hq,hkv", [(2, 8, 4), (4, 8, 4), (2, 28, 4)], ids=["tp2", "tp4_1kv", "qwen_tp2"])
def test_tensor_parallel_split_on_one_gpu(tp, hq, hkv):
    """The three-stage form with the exchange done by hand: `tp` engines (one per rank, all on this
    GPU) score their own heads, the vote vectors are summed, every rank selects from the sum.  All
    ranks must pick the same rows, equal to the oracle's emulation with rank-local head maps."""
    d, n_init, n_local, k, base, n = 128, 16, 64, 256, 5e5, 2600
    case = synth.make_layer_case(77, n, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
    hq_r, hkv_r = hq // tp, hkv // tp
    engs = [gu.make_engine(hq_r, hkv_r, d, n_init, n_local, k, base, BF16, max_ctx=n + 8, tp_rank=r, tp_size=tp,
                           query_cache=True) for r in range(tp)]
    dev = engs[0].device
    rtt_d = rtt.to(dev)
    ridx_d, lens_d = ridx.to(device=dev, dtype=torch.int32), lens.to(device=dev, dtype=torch.int32)
    outs, dbgs, args, keep = [], [], [], []
    for r, e in enumerate(engs):
        qr = q.view(1, hq, d)[:, r * hq_r:(r + 1) * hq_r].reshape(1, -1).contiguous().to(dev)
        kr = kp[:, r * hkv_r:(r + 1) * hkv_r].contiguous().to(dev)
        vr = vp[:, r * hkv_r:(r + 1) * hkv_r].contiguous().to(dev)
        out = torch.empty_like(qr)
        dbg = e.new_debug_buffers(1)
        keep.append((qr, kr, vr))
        outs.append(out)
        dbgs.append(dbg)
        args.append(e.build_args(0, qr, None, None, None, kr, vr, rtt_d, ridx_d, lens_d, out, dbg))
    for step in range(2):          # second step exercises the all-reduced cosine terms
        for e, a in zip(engs, args):
            e.tp_prepare(a)
        cos = sum(e.tp_cos for e in engs)
        for e in engs:
            e.tp_cos.copy_(cos)
        for e, a in zip(engs, args):
            e.tp_score_vote(a)
        votes = sum(e.tp_votes for e in engs)
        for e in engs:
            e.tp_votes.copy_(votes)
        for e, a in zip(engs, args):
            e.tp_select_attend(a)
        torch.cuda.synchronize()
        for e in engs:
            e.raise_on_device_error()
        flags = [int(dbg["flags"][0]) for dbg in dbgs]
        assert flags == [orc.FLAG_RECOMPUTE if step == 0 else orc.FLAG_REUSE] * tp
        for dbg in dbgs[1:]:
            assert torch.equal(dbg["slots"], dbgs[0]["slots"]), "ranks selected different rows"
    ocfg = orc.OracleConfig(1, hq, hkv, d, n_init, n_local, k, base)
    ref = orc.DecodeOracle(ocfg, tp_ranks=tp).decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens)
    res0 = {k_: v.cpu() for k_, v in dbgs[0].items()}
    gu.check_selection(engs[0], res0, 0, ref["positions"][0], ref["info"][0]["votes"], n)
    got = torch.cat([o.cpu().view(hq_r, d) for o in outs], dim=0).reshape(-1)
    want = torch.cat([
        orc.sparse_attention(q.view(hq, d)[r * hq_r:(r + 1) * hq_r], kp[:, r * hkv_r:(r + 1) * hkv_r],
                             vp[:, r * hkv_r:(r + 1) * hkv_r], res0["slots"][0, : engs[0].cfg.n_sel], d ** -0.5,
                             base, 1.0, 0.0, torch.float64) for r in range(tp)], dim=0).reshape(-1)
    assert (got.double() - want).abs().max().item() <= 2e-2


GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_selection.json")
with open(GOLDEN) as f:
    GOLDEN_CASES = [c for c in json.load(f)["cases"] if c["head_dim"] in (64, 128)]


@pytest.mark.parametrize("case", GOLDEN_CASES, ids=[c["name"] for c in GOLDEN_CASES])
def test_cuda_path_against_reference_golden(case):
    """fp32 check mode on the inputs the reference's own code was run on: same windows and order,
    >= 98 % of the reference's rows (its bf16 logit buffer moves a few indices at the k-th vote), and
    the dense fallback exactly where the reference returns None."""
    c = synth.make_layer_case(case["seed"], case["n_tokens"], case["hq"], case["hkv"], case["head_dim"],
                              case["n_init"], case["n_local"], case["rope_base"])
    eng = gu.make_engine(case["hq"], case["hkv"], case["head_dim"], case["n_init"], case["n_local"], case["top_k"],
                         case["rope_base"], F32, max_ctx=case["n_tokens"] + 8, kernel_size=case["kernel_size"])
    q, kp, vp, rtt, ridx, lens = gu.case_tensors(c)
    if "chunk" in case:            # a prefill chunk: selection with the chunk's fingerprint (ts_extend_chunk)
        qc = synth.make_chunk_queries(case["seed"], c, case["chunk"], case["hq"], case["head_dim"])
        dev = eng.device
        dbg = eng.new_debug_buffers(1)
        eng.extend_chunk(0, qc.to(dev), None, None, None, kp.to(dev), vp.to(dev), rtt.to(dev), c.req_pool_idx,
                         case["n_tokens"], debug=dbg)
        torch.cuda.synchronize()
        eng.raise_on_device_error()
        res = {k_: v.cpu() for k_, v in dbg.items()}
    else:
        _, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens)
    if case["slots"] is None:
        assert int(res["flags"][0]) == orc.FLAG_DENSE and int(res["count"][0]) == case["n_tokens"]
        return
    got = res["slots"][0, : eng.cfg.n_sel].tolist()
    want = case["slots"]
    assert len(got) == len(want)
    assert got[: case["n_init"]] == want[: case["n_init"]]
    assert got[-case["n_local"]:] == want[-case["n_local"]:]
    assert len(set(got) & set(want)) >= 0.98 * len(want)


def test_full_size_128k_properties_and_oracle():
    """Headline shape: 32/8 heads, 131072 tokens, top-k 2048, bf16, N(0,1) K/V with 1 % planted keys and
    4 outlier channels x8, generated on the device from a seed.  Checks the size-independent
    properties (count, order, uniqueness, windows, rows come from the request's own map) and, since
    the oracle still finishes in seconds at this size, the index-set rule and the attention output."""
    hq, hkv, d, n_init, n_local, k, base, n = 32, 8, 128, 128, 512, 2048, 5e5, 131072
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    rows = n + 1000
    kp = torch.randn(rows, hkv, d, generator=g, device=dev, dtype=torch.float32)
    vp = torch.randn(rows, hkv, d, generator=g, device=dev, dtype=torch.float32)
    ch = torch.randperm(d, generator=g, device=dev)[:4]
    kp[:, :, ch] *= 8
    vp[:, :, ch] *= 8
    q = torch.randn(1, hq * d, generator=g, device=dev, dtype=torch.float32).to(BF16)
    perm = torch.randperm(rows, generator=g, device=dev)[:n].to(torch.int32)
    rtt = torch.zeros(2, n + 8, dtype=torch.int32, device=dev)
    rtt[1, :n] = perm
    q_rot = orc.rotate_scoring_query(q.cpu().view(hq, d), n_local, base, 1.0).float().to(dev)
    planted = torch.randperm(n - n_init - n_local, generator=g, device=dev)[: (n // 100)] + n_init
    for kv in range(hkv):
        kp[perm[planted].long(), kv] += 3.0 * q_rot[kv] / q_rot[kv].norm()
    kp, vp = kp.to(BF16), vp.to(BF16)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8, max_reqs=2, max_batch=1)
    dbg = eng.new_debug_buffers(1)
    ridx = torch.tensor([1], dtype=torch.int32, device=dev)
    lens = torch.tensor([n], dtype=torch.int32, device=dev)
    out = eng.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens, debug=dbg)
    torch.cuda.synchronize()
    eng.raise_on_device_error()
    pos = dbg["positions"][0].cpu().numpy()
    slots = dbg["slots"][0].cpu()
    assert int(dbg["count"][0]) == n_init + k + n_local
    assert np.all(np.diff(pos) > 0)
    assert np.array_equal(pos[:n_init], np.arange(n_init))
    assert np.array_equal(pos[-n_local:], np.arange(n - n_local, n))
    assert torch.equal(slots, rtt[1].cpu()[torch.from_numpy(pos).long()])
    assert torch.isfinite(out.float()).all()
    # oracle at full size
    qc, kc, vc, rc = q.cpu(), kp.cpu(), vp.cpu(), rtt.cpu()
    ref = orc.DecodeOracle(gu.oracle_config(eng)).decode_layer(0, qc, None, None, None, kc, vc, rc,
                                                               torch.tensor([1]), torch.tensor([n]))
    res = {k_: v.cpu() for k_, v in dbg.items()}
    gu.check_selection(eng, res, 0, ref["positions"][0], ref["info"][0]["votes"], n)
    want = orc.sparse_attention(qc.view(hq, d), kc, vc, slots, d ** -0.5, base, 1.0, 0.0, torch.float64).reshape(-1)
    assert (out[0].cpu().double() - want).abs().max().item() <= 2e-2
