"""Two real GPUs: the in-kernel tensor-parallel vote exchange (peer memory over NVLink) and the
host-driven NCCL form must both give every rank the same rows, equal to the oracle's emulation.
Skipped on boxes with fewer than two GPUs."""
import os
import socket
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from oracle import synth
from oracle import tokenselect_oracle as orc

pytestmark = pytest.mark.gpu
HQ, HKV, D, N_INIT, N_LOCAL, K, BASE, N = 8, 4, 128, 16, 64, 256, 5e5, 6000
LQ = 96


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fused, out_dir):
    import torch.distributed as dist
    from tokenselect_b200 import TokenSelectConfig, TokenSelectEngine
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        case = synth.make_layer_case(91, N, HQ, HKV, D, N_INIT, N_LOCAL, BASE, dtype=torch.bfloat16)
        hq_r, hkv_r = HQ // world, HKV // world
        cfg = TokenSelectConfig(rope_base=BASE, max_n_tokens=N + 8, top_k=K, n_init=N_INIT, n_local=N_LOCAL,
                                n_layers=1, num_q_heads=hq_r, num_kv_heads=hkv_r, head_dim=D, max_reqs=2,
                                max_batch=1, max_total_tokens=N + 8, tp_rank=rank, tp_size=world, tp_fused=fused)
        eng = TokenSelectEngine(cfg, device=dev)
        assert eng.fused_tp == fused
        q = case.q.view(1, HQ, D)[:, rank * hq_r:(rank + 1) * hq_r].reshape(1, -1).contiguous().to(dev)
        kp = case.k_pool[:, rank * hkv_r:(rank + 1) * hkv_r].contiguous().to(dev)
        vp = case.v_pool[:, rank * hkv_r:(rank + 1) * hkv_r].contiguous().to(dev)
        rtt = case.req_to_token.to(dev)
        ridx = torch.tensor([case.req_pool_idx], dtype=torch.int32, device=dev)
        lens = torch.tensor([N], dtype=torch.int32, device=dev)
        dbg = eng.new_debug_buffers(1)
        for _ in range(3):                                  # several calls: both flag parities get used
            out = eng.decode_layer(0, q, None, None, None, kp, vp, rtt, ridx, lens, debug=dbg)
        torch.cuda.synchronize()
        eng.raise_on_device_error()
        rec = {"slots": dbg["slots"].cpu(), "positions": dbg["positions"].cpu(), "out": out.cpu()}
        if fused:
            # one prefill chunk of LQ tokens closing the same request, heads split the same way
            qc = synth.make_chunk_queries(91, case, LQ, HQ, D).view(LQ, HQ, D)[:, rank * hq_r:(rank + 1) * hq_r]
            dbg2 = eng.new_debug_buffers(1)
            out2 = eng.extend_chunk(0, qc.reshape(LQ, -1).contiguous().to(dev), None, None, None, kp, vp, rtt,
                                    case.req_pool_idx, N, debug=dbg2)
            torch.cuda.synchronize()
            eng.raise_on_device_error()
            rec.update({"x_slots": dbg2["slots"].cpu(), "x_positions": dbg2["positions"].cpu(), "x_out": out2.cpu()})
        torch.save(rec, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fused", [True, False], ids=["in_kernel_sum", "nccl_all_reduce"])
def test_two_gpu_tensor_parallel(fused):
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, _free_port(), fused, d), nprocs=world, join=True)
        res = [torch.load(os.path.join(d, f"rank{r}.pt")) for r in range(world)]
    assert torch.equal(res[0]["slots"], res[1]["slots"]), "ranks selected different rows"
    case = synth.make_layer_case(91, N, HQ, HKV, D, N_INIT, N_LOCAL, BASE, dtype=torch.bfloat16)
    ocfg = orc.OracleConfig(1, HQ, HKV, D, N_INIT, N_LOCAL, K, BASE)
    _, pos, info = orc.DecodeOracle(ocfg, tp_ranks=world).select(0, 1, case.q.view(HQ, D), case.k_pool,
                                                                case.req_to_token[1], N)
    got = res[0]["positions"][0, N_INIT:N_INIT + K].numpy() - N_INIT
    want = pos[N_INIT:N_INIT + K].numpy() - N_INIT
    ok, why = orc.index_sets_match(got, want, info["votes"].double().numpy(), K)
    assert ok, why
    hq_r, hkv_r = HQ // world, HKV // world
    for r in range(world):
        ref = orc.sparse_attention(case.q.view(HQ, D)[r * hq_r:(r + 1) * hq_r], case.k_pool[:, r * hkv_r:(r + 1) * hkv_r],
                                   case.v_pool[:, r * hkv_r:(r + 1) * hkv_r], res[0]["slots"][0], D ** -0.5, BASE, 1.0,
                                   0.0, torch.float64).reshape(-1)
        assert (res[r]["out"][0].double() - ref).abs().max().item() <= 2e-2
    if fused:
        # the prefill chunk: same rows on both ranks, equal to the oracle's tensor-parallel emulation
        assert torch.equal(res[0]["x_slots"], res[1]["x_slots"]), "ranks selected different rows for the chunk"
        qc = synth.make_chunk_queries(91, case, LQ, HQ, D)
        ref = orc.DecodeOracle(ocfg, tp_ranks=world).extend_chunk(0, 1, qc, None, None, None, case.k_pool, case.v_pool,
                                                                  case.req_to_token[1], N, attn_dtype=torch.float64)
        got = res[0]["x_positions"][0, N_INIT:N_INIT + K].numpy() - N_INIT
        want = ref["positions"][N_INIT:N_INIT + K].numpy() - N_INIT
        ok, why = orc.index_sets_match(got, want, ref["info"]["votes"].double().numpy(), K)
        assert ok, why
        for r in range(world):
            want_o = orc.sparse_prefill_attention(
                qc.view(LQ, HQ, D)[:, r * hq_r:(r + 1) * hq_r], case.k_pool[:, r * hkv_r:(r + 1) * hkv_r],
                case.v_pool[:, r * hkv_r:(r + 1) * hkv_r], res[0]["x_slots"][0], D ** -0.5, BASE, 1.0, 0.0,
                torch.float64).reshape(LQ, -1)
            assert (res[r]["x_out"].double() - want_o).abs().max().item() <= 2e-2
