"""Tensor-parallel exchange protocol on CPU: two gloo ranks each score their own KV heads (oracle
arithmetic stands in for the kernels), all-reduce the fp32 vote vector and the three cosine terms, and
run the same deterministic top-k.  Every rank must end with the same index set, equal to the
single-process emulation, and must take the same reuse decision."""
import os
import socket
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import synth
from oracle import tokenselect_oracle as orc

HQ, HKV, D, N_INIT, N_LOCAL, K, BASE, N = 8, 4, 64, 8, 32, 128, 1e4, 1500


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = synth.make_layer_case(21, N, HQ, HKV, D, N_INIT, N_LOCAL, BASE)
        hq_r, hkv_r = HQ // world, HKV // world
        q = case.q.view(HQ, D)[rank * hq_r:(rank + 1) * hq_r]
        kp = case.k_pool[:, rank * hkv_r:(rank + 1) * hkv_r]
        row = case.req_to_token[case.req_pool_idx]
        results = []
        cached = None
        for step, scale in enumerate((1.0, 1.3, -1.0)):          # same direction -> reuse; flipped -> recompute
            q_rot = orc.rotate_scoring_query(q * scale, N_LOCAL, BASE, 1.0)
            recompute = True
            if cached is not None:
                terms = torch.from_numpy(orc.cosine_terms_fixed_order(q_rot.numpy(), cached["fp"]))
                dist.all_reduce(terms)                            # every rank decides on the same sums
                recompute = orc.cache_says_recompute(orc.cosine_from_terms(terms.numpy()), 0.9)
            if recompute:
                logits = orc.score_logits(q_rot, kp, row[N_INIT: N - N_LOCAL], "mod")   # rank-local head map
                votes = orc.soft_vote(logits)
                dist.all_reduce(votes)                            # token_retrieval.py:363-364
                top = orc.topk_sorted(votes, K) + N_INIT
                cached = {"fp": q_rot.numpy().copy(), "top": top}
            results.append((recompute, cached["top"].clone()))
        torch.save(results, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_agree_and_match_single_process_emulation(world):
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, port, d), nprocs=world, join=True)
        per_rank = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(world)]
    for r in range(1, world):
        for (f0, t0), (f1, t1) in zip(per_rank[0], per_rank[r]):
            assert f0 == f1 and torch.equal(t0, t1), "ranks diverged"
    assert [f for f, _ in per_rank[0]] == [True, False, True]
    case = synth.make_layer_case(21, N, HQ, HKV, D, N_INIT, N_LOCAL, BASE)
    cfg = orc.OracleConfig(1, HQ, HKV, D, N_INIT, N_LOCAL, K, BASE)
    _, pos, _ = orc.DecodeOracle(cfg, tp_ranks=world).select(0, 1, case.q.view(HQ, D), case.k_pool,
                                                            case.req_to_token[1], N)
    assert torch.equal(per_rank[0][0][1], pos[N_INIT: N_INIT + K])
