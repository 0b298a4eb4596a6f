"""The benchmark configurations that are parity cases rather than bench lines: the ragged continuous
batch (Qwen2-7B shape, 16 requests of log-uniform length joining and finishing at staggered steps) and the
1M-token, batch-4, one-KV-head-per-GPU shard.  Inputs are generated on the device from a seed; the oracle
runs on the CPU on the same tensors."""
import math

import numpy as np
import pytest
import torch

from oracle import tokenselect_oracle as orc
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _pools(gen, dev, rows, hkv, d):
    k = torch.randn(rows, hkv, d, generator=gen, device=dev, dtype=torch.float32)
    v = torch.randn(rows, hkv, d, generator=gen, device=dev, dtype=torch.float32)
    ch = torch.randperm(d, generator=gen, device=dev)[:4]
    k[:, :, ch] *= 8                   # outlier key channels; values stay unit-variance so the bf16 output
                                       # rounding stays inside the absolute attention tolerance
    return k, v


def _plant(k, rows_of_request, q_rot_first_heads, gen, n_init, n_local):
    n = rows_of_request.numel()
    nc = n - n_init - n_local
    if nc <= 0:
        return
    pick = torch.randperm(nc, generator=gen, device=k.device)[: max(1, n // 100)] + n_init
    for kv in range(k.shape[1]):
        u = q_rot_first_heads[kv]
        k[rows_of_request[pick].long(), kv] += 3.0 * u / u.norm()


def _check_request(eng, res, b, q_b, kp, vp, rtt_row, n, out_b, o, layer, slot):
    hq, d = eng.cfg.num_q_heads, eng.cfg.head_dim
    flag, pos, info = o.select(layer, slot, q_b.view(hq, d), kp, rtt_row, n)
    assert int(res["flags"][b]) == flag
    cnt = int(res["count"][b])
    if flag == orc.FLAG_DENSE:
        assert cnt == n and torch.equal(res["positions"][b, :n], torch.arange(n, dtype=torch.int32))
    else:
        gu.check_selection(eng, res, b, pos, info["votes"], n)
    sl = res["slots"][b, :cnt]
    assert torch.equal(sl, rtt_row[res["positions"][b, :cnt].long()])
    want = orc.sparse_attention(q_b.view(hq, d), kp, vp, sl, d ** -0.5, eng.cfg.rope_base, 1.0, 0.0,
                                torch.float64).reshape(-1)
    assert (out_b.double() - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("scale,flags", [(16, 0), (16, 1024), (1, 0)],
                         ids=["lengths_div16", "lengths_div16_inline_attention", "full_lengths"])
def test_ragged_continuous_batch_qwen_shape(scale, flags):
    """16 requests, lengths log-uniform in [16384, 262144] / scale from a seed; three scheduler steps in
    which requests finish and new ones join the freed slots (their cache state is reset).  Every request of
    every step is checked against the oracle at the reduced lengths; at full lengths the first and last
    request of each step are."""
    hq, hkv, d, n_init, n_local, k, base = 28, 4, 128, 128, 512, 2048, 1e6
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(77)
    rng = np.random.default_rng(5)
    max_reqs, bs = 20, 16
    lo, hi = 16384 // scale, 262144 // scale
    lens = [int(math.exp(rng.uniform(math.log(lo), math.log(hi)))) for _ in range(max_reqs)]
    if scale > 1:
        lens[3], lens[7] = n_init + k + n_local, 900          # one at the guard, one far below it
    total = sum(lens) + 3 * bs + 64
    max_ctx = max(lens) + 8
    kp, vp = _pools(g, dev, total, hkv, d)
    perm = torch.randperm(total, generator=g, device=dev).to(torch.int32)
    rtt = torch.zeros(max_reqs, max_ctx, dtype=torch.int32, device=dev)
    at = 0
    for r, n in enumerate(lens):
        rtt[r, :n + 3] = perm[at: at + n + 3]
        at += n + 3
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, n_layers=2, max_ctx=max_ctx, max_reqs=max_reqs,
                         max_batch=bs, max_total=sum(sorted(lens)[-bs:]) + 64, query_cache=True, extra_flags=flags)
    qs = torch.randn(3, max_reqs, hq * d, generator=g, device=dev).to(BF16)
    q_rot0 = orc.rotate_scoring_query(qs[0].cpu().view(max_reqs, hq, d), n_local, base, 1.0).float().to(dev)
    for r, n in enumerate(lens):
        _plant(kp, rtt[r, :n], q_rot0[r, :hkv], g, n_init, n_local)
    kp, vp = kp.to(BF16), vp.to(BF16)
    kc, vc, rc = kp.cpu(), vp.cpu(), rtt.cpu()
    o = orc.DecodeOracle(gu.oracle_config(eng))
    active = list(range(bs))                                   # request slot of each batch row
    cur = list(lens)
    rid = {s: ("req", s, 0) for s in active}
    eng.bind_requests([rid[s] for s in active], active)
    for s in active:
        o.reset_request(s)
    for step in range(3):
        if step == 1:                                          # two requests finish, two join in new slots
            for row, new_slot in ((2, 16), (9, 17)):
                active[row] = new_slot
                rid[new_slot] = ("req", new_slot, step)
                o.reset_request(new_slot)
        if step == 2:                                          # a finished slot is handed to a new request
            active[5] = 2
            rid[2] = ("req", 2, step)
            cur[2] = lens[2] // 2
            o.reset_request(2)
        eng.bind_requests([rid[s] for s in active], active)
        ridx = torch.tensor(active, dtype=torch.int32, device=dev)
        sl = torch.tensor([cur[s] for s in active], dtype=torch.int32, device=dev)
        q = qs[step if step < 2 else 0][active].contiguous()    # step 2 repeats step 0's queries: cache reuse
        for layer in range(2):
            dbg = eng.new_debug_buffers(bs)
            out = eng.decode_layer(layer, q, None, None, None, kp, vp, rtt, ridx, sl, debug=dbg)
            torch.cuda.synchronize()
            eng.raise_on_device_error()
            res = {k_: v.cpu() for k_, v in dbg.items()}
            outc, qc = out.cpu(), q.cpu()
            rows = range(bs) if scale > 1 else (0, bs - 1)
            for b in range(bs):
                s = active[b]
                if b in rows:
                    _check_request(eng, res, b, qc[b], kc, vc, rc[s], cur[s], outc[b], o, layer, s)
                else:                                           # keep the oracle's cache state in step
                    o.select(layer, s, qc[b].view(hq, d), kc, rc[s], cur[s])
                    if int(res["flags"][b]) == orc.FLAG_RECOMPUTE:
                        o.cache[(s, layer)].topk_positions = res["positions"][b, n_init:n_init + k].long().clone()
                if int(res["flags"][b]) == orc.FLAG_RECOMPUTE and b in rows:
                    o.cache[(s, layer)].topk_positions = res["positions"][b, n_init:n_init + k].long().clone()
        for s in active:
            cur[s] += 1


def test_one_million_tokens_batch4_one_kv_head_per_gpu():
    """The shard one GPU holds at tensor-parallel degree 8: 4 query heads, 1 KV head, four requests of
    1048576 tokens, top-k 4096, n_local 1024.  Properties for all four requests, oracle comparison for one."""
    hq, hkv, d, n_init, n_local, k, base, n = 4, 1, 128, 128, 1024, 4096, 5e5, 1048576
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(11)
    bs = 4
    total = bs * n + 64
    kp, vp = _pools(g, dev, total, hkv, d)
    perm = torch.randperm(total, generator=g, device=dev).to(torch.int32)
    rtt = torch.zeros(bs, n + 8, dtype=torch.int32, device=dev)
    for r in range(bs):
        rtt[r, :n] = perm[r * n:(r + 1) * n]
    q = torch.randn(bs, hq * d, generator=g, device=dev).to(BF16)
    q_rot = orc.rotate_scoring_query(q.cpu().view(bs, hq, d), n_local, base, 1.0).float().to(dev)
    for r in range(bs):
        _plant(kp, rtt[r, :n], q_rot[r, :hkv], g, n_init, n_local)
    kp, vp = kp.to(BF16), vp.to(BF16)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, BF16, max_ctx=n + 8, max_reqs=bs, max_batch=bs,
                         max_total=bs * (n + 8))
    ridx = torch.arange(bs, dtype=torch.int32, device=dev)
    sl = torch.full((bs,), n, dtype=torch.int32, device=dev)
    dbg = eng.new_debug_buffers(bs)
    out = eng.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, sl, debug=dbg)
    torch.cuda.synchronize()
    eng.raise_on_device_error()
    res = {k_: v.cpu() for k_, v in dbg.items()}
    n_sel = n_init + k + n_local
    for b in range(bs):
        pos = res["positions"][b].numpy()
        assert int(res["count"][b]) == n_sel and np.all(np.diff(pos) > 0)
        assert np.array_equal(pos[:n_init], np.arange(n_init)) and np.array_equal(pos[-n_local:], np.arange(n - n_local, n))
        assert torch.equal(res["slots"][b], rtt[b].cpu()[torch.from_numpy(pos).long()])
    assert torch.isfinite(out.float()).all()
    o = orc.DecodeOracle(gu.oracle_config(eng))
    b = 2
    _check_request(eng, res, b, q[b].cpu(), kp.cpu(), vp.cpu(), rtt[b].cpu(), n, out[b].cpu(), o, 0, b)
