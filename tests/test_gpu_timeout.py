"""A bounded device-side wait that really runs out, on one GPU and without any fault: a tensor-parallel handle
of two ranks whose "peer" is a second, zero-filled buffer on the same GPU that never raises its flag.  The
selection kernel must give up after the configured limit, leave TS_ERR_DEVICE_TIMEOUT in the sticky error
word, return, and leave the GPU usable (the reference has no counterpart: its scripts kill a hung server,
scripts/infinitebench-mp-llama.sh:10)."""
import pytest
import torch

from oracle import synth
from oracle import tokenselect_oracle as orc
from tokenselect_b200 import TokenSelectConfig, TokenSelectEngine
from tokenselect_b200 import _lib

pytestmark = pytest.mark.gpu
HQ, HKV, D, N_INIT, N_LOCAL, K, BASE, N = 8, 2, 128, 16, 64, 256, 5e5, 3000
LIMIT_US = 2000
TS_ERR_DEVICE_TIMEOUT = 5


def _inputs(dev, hq, hkv):
    case = synth.make_layer_case(17, N, HQ, HKV, D, N_INIT, N_LOCAL, BASE, dtype=torch.bfloat16)
    q = case.q.view(1, HQ, D)[:, :hq].reshape(1, -1).contiguous().to(dev)
    kp, vp = case.k_pool[:, :hkv].contiguous().to(dev), case.v_pool[:, :hkv].contiguous().to(dev)
    ridx = torch.tensor([case.req_pool_idx], dtype=torch.int32, device=dev)
    lens = torch.tensor([N], dtype=torch.int32, device=dev)
    return case, q, kp, vp, case.req_to_token.to(dev), ridx, lens


def test_peer_flag_wait_runs_out_and_the_gpu_stays_usable():
    dev = torch.device("cuda:0")
    cfg = TokenSelectConfig(rope_base=BASE, max_n_tokens=N + 8, top_k=K, n_init=N_INIT, n_local=N_LOCAL, n_layers=1,
                            num_q_heads=HQ // 2, num_kv_heads=HKV // 2, head_dim=D, max_reqs=2, max_batch=1,
                            max_total_tokens=N + 8, tp_rank=0, tp_size=2, tp_fused=True, wait_limit_us=LIMIT_US)
    eng = TokenSelectEngine(cfg, device=dev)           # no process group: nothing is attached yet
    assert not eng.fused_tp
    nbytes = eng.symmetric_bytes()
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=dev)      # never flags, never votes
    eng.attach_peer_buffers([mine.data_ptr(), silent_peer.data_ptr()])
    case, q, kp, vp, rtt, ridx, lens = _inputs(dev, HQ // 2, HKV // 2)
    out = torch.zeros_like(q)
    # the same kernel once on a single-rank engine of the rank's shape: the first launch of a kernel in a process
    # loads it, which takes longer than the limit under test
    warm = TokenSelectEngine(TokenSelectConfig(rope_base=BASE, max_n_tokens=N + 8, top_k=K, n_init=N_INIT, n_local=N_LOCAL,
                                               n_layers=1, num_q_heads=HQ // 2, num_kv_heads=HKV // 2, head_dim=D, max_reqs=2,
                                               max_batch=1, max_total_tokens=N + 8), device=dev)
    warm.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens, out=out)
    torch.cuda.synchronize()
    warm.raise_on_device_error()
    warm.close()
    t0, t1, t2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    t0.record()
    eng.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens, out=out)       # returns: the wait is bounded
    t1.record()
    eng.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens, out=out)       # error word set: waits for nothing
    t2.record()
    torch.cuda.synchronize()
    first_ms, second_ms = t0.elapsed_time(t1), t1.elapsed_time(t2)
    code, detail = eng.last_error()
    assert code == TS_ERR_DEVICE_TIMEOUT and detail == 31, (code, detail)     # 30 + rank of the silent peer
    assert 0.5 * LIMIT_US * 1e-3 <= first_ms <= 8 * LIMIT_US * 1e-3, first_ms    # one limit, not one per wait site
    assert second_ms <= 0.5 * LIMIT_US * 1e-3, second_ms
    assert eng.last_error() == (0, 0)                                          # read-and-clear
    with pytest.raises(_lib.TokenSelectError):
        eng2 = TokenSelectEngine(TokenSelectConfig(num_q_heads=8, num_kv_heads=1, tp_rank=0, tp_size=16))
        del eng2
    eng.close()

    # the same GPU, a fresh single-rank engine: results still match the oracle
    cfg1 = TokenSelectConfig(rope_base=BASE, max_n_tokens=N + 8, top_k=K, n_init=N_INIT, n_local=N_LOCAL, n_layers=1,
                             num_q_heads=HQ, num_kv_heads=HKV, head_dim=D, max_reqs=2, max_batch=1,
                             max_total_tokens=N + 8)
    eng1 = TokenSelectEngine(cfg1, device=dev)
    case, q, kp, vp, rtt, ridx, lens = _inputs(dev, HQ, HKV)
    dbg = eng1.new_debug_buffers(1)
    out = eng1.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens, debug=dbg)
    torch.cuda.synchronize()
    eng1.raise_on_device_error()
    ocfg = orc.OracleConfig(1, HQ, HKV, D, N_INIT, N_LOCAL, K, BASE)
    _, pos, info = orc.DecodeOracle(ocfg).select(0, 1, case.q.view(HQ, D), case.k_pool, case.req_to_token[1], N)
    got = dbg["positions"][0].cpu()[N_INIT:N_INIT + K].numpy() - N_INIT
    ok, why = orc.index_sets_match(got, pos[N_INIT:N_INIT + K].numpy() - N_INIT, info["votes"].double().numpy(), K)
    assert ok, why
    ref = orc.sparse_attention(case.q.view(HQ, D), case.k_pool, case.v_pool, dbg["slots"][0].cpu(), D ** -0.5, BASE,
                               1.0, 0.0, torch.float64).reshape(-1)
    assert (out[0].cpu().double() - ref).abs().max().item() <= 2e-2
