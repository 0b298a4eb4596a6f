"""The decode calls enqueue on the current stream without synchronising or allocating, so a token's layer
loop can be captured once as a CUDA graph and replayed with new inputs written into the captured buffers.
Replays must equal the same calls launched from the host."""
import pytest
import torch

from oracle import synth
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def test_graph_replay_equals_host_launched_calls():
    hq, hkv, d, n_init, n_local, top_k, base, n, layers = 8, 2, 128, 16, 64, 256, 5e5, 3000, 2
    case = synth.make_layer_case(81, n + 4, hq, hkv, d, n_init, n_local, base, dtype=BF16)
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, top_k, base, BF16, n_layers=layers, max_ctx=n + 16, max_batch=1)
    dev = eng.device
    row = case.req_to_token[case.req_pool_idx]
    rtt = case.req_to_token.to(dev)
    ridx = torch.tensor([case.req_pool_idx], dtype=torch.int32, device=dev)
    # the last four tokens of the case arrive one per step: their K/V rows are passed with the call
    k_tok = case.k_pool[row[n:n + 4].long()].reshape(4, 1, -1).to(dev)
    v_tok = case.v_pool[row[n:n + 4].long()].reshape(4, 1, -1).to(dev)
    qs = (case.q.view(1, 1, -1) + 0.3 * synth.normal(81, 13, (4, layers, hq * d))).to(BF16).to(dev).unsqueeze(2)

    def pools():
        kp, vp = case.k_pool.clone(), case.v_pool.clone()
        kp[row[n:n + 4].long()] = 0
        vp[row[n:n + 4].long()] = 0
        return [kp.to(dev) for _ in range(layers)], [vp.to(dev) for _ in range(layers)]

    # host-launched reference run
    kps, vps = pools()
    want = []
    for t in range(4):
        lens = torch.tensor([n + t + 1], dtype=torch.int32, device=dev)
        loc = row[n + t:n + t + 1].to(dev)
        outs = [eng.decode_layer(li, qs[t, li], k_tok[t], v_tok[t], loc, kps[li], vps[li], rtt, ridx, lens)
                for li in range(layers)]
        want.append(torch.stack(outs).clone())
    torch.cuda.synchronize()
    eng.raise_on_device_error()

    # the same four steps as replays of one captured token
    kps, vps = pools()
    sq = torch.zeros(layers, 1, hq * d, dtype=BF16, device=dev)
    sk, sv = torch.zeros_like(k_tok[0]), torch.zeros_like(v_tok[0])
    sloc = torch.zeros(1, dtype=torch.int32, device=dev)
    slens = torch.full((1,), n + 1, dtype=torch.int32, device=dev)
    sout = torch.zeros(layers, 1, hq * d, dtype=BF16, device=dev)
    sq.copy_(qs[0]); sk.copy_(k_tok[0]); sv.copy_(v_tok[0]); sloc.copy_(row[n:n + 1].to(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for li in range(layers):
            eng.decode_layer(li, sq[li], sk, sv, sloc, kps[li], vps[li], rtt, ridx, slens, out=sout[li])
    for t in range(4):
        sq.copy_(qs[t]); sk.copy_(k_tok[t]); sv.copy_(v_tok[t])
        sloc.copy_(row[n + t:n + t + 1].to(dev))
        slens.fill_(n + t + 1)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(sout, want[t]), f"step {t}"
    eng.raise_on_device_error()
    assert torch.equal(kps[0].cpu(), case.k_pool) and torch.equal(vps[1].cpu(), case.v_pool)
