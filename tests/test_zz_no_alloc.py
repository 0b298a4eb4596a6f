"""The allocation-free attention entry point (``ts_attend_rows_static``) against the regular one and the oracle.

Some callers may not allocate device memory at the moment they need attention -- they run inside a
serving loop or callback that must stay clear of the allocator (an allocation can stall the device), or
all of the process's device memory was given to another component at start-up.  For them the library keeps the split kernel's partial
results in a fixed array of its own image instead of a workspace from ``ts_create``.  This test calls that
entry point through the C ABI twice in a row (the array keeps the previous call's contents, which must
not matter) and compares with the output of ``ts_decode_layer`` on the same rows and with the CPU oracle's
fp64 attention over those rows: 2e-2 absolute for bf16 as everywhere; 1e-4 in fp32 check mode -- not the
1e-5 of the table-driven kernels, because this entry point has no handle and therefore no host-built
rotation table: it evaluates cos/sin of position x frequency in the kernel, in fp32, with frequencies from
exp2 of an fp32 exponent, and at list positions in the thousands an angle off by a few fp32 ulps moves a
logit by ~1e-5.

Collected last on purpose: a failure here must not hide the results of the other tests.
"""
import pytest
import torch

from oracle import synth
from oracle import tokenselect_oracle as orc
from tests import gpu_util as gu
from tokenselect_b200.engine import attend_rows_static

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol,d,cap", [(torch.bfloat16, 2e-2, 128, 0.0), (torch.float32, 1e-4, 128, 0.0),
                                             (torch.bfloat16, 2e-2, 64, 0.0), (torch.float32, 1e-4, 128, 20.0)],
                         ids=["bf16", "fp32", "bf16_d64", "fp32_softcap"])
def test_static_scratch_attention_matches_regular_entry_point(dtype, tol, d, cap):
    hq, hkv, n_init, n_local, k, base = 8, 2, 16, 64, 256, 5e5
    sm_scale = d ** -0.5 if cap == 0.0 else 0.5          # large logits so that the cap bites
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, dtype, max_ctx=4096, logit_cap=cap, sm_scale=sm_scale)
    dev = eng.device
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for call, (seed, n) in enumerate(((61, 3000), (62, 1700))):       # two calls in a row, different lists
        case = synth.make_layer_case(seed, n, hq, hkv, d, n_init, n_local, base, dtype=dtype)
        q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
        want, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens)
        rows = res["slots"][0, : int(res["count"][0])].to(dev)
        kd, vd, qd = kp.to(dev), vp.to(dev), q[0].contiguous().to(dev)
        out = torch.empty_like(qd)                                    # the caller owns the output
        if call == 0:                                                 # first call on the device: module load, address look-up
            attend_rows_static(qd, kd, vd, rows, out, sm_scale, base, 1.0, cap, status)
            torch.cuda.synchronize()
        # No allocation by anyone during the call: the driver's free-memory figure sees a cudaMalloc inside the
        # library as well as one by torch (it may only grow here: Python can collect an engine of an earlier test
        # at any moment, which frees that engine's workspace); torch's own allocation count covers its caching
        # allocator.
        import gc
        gc.collect()
        free_before, _ = torch.cuda.mem_get_info(dev)
        count_before = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
        attend_rows_static(qd, kd, vd, rows, out, sm_scale, base, 1.0, cap, status)
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats(dev)["allocation.all.allocated"] == count_before
        assert torch.cuda.mem_get_info(dev)[0] >= free_before
        assert int(status.item()) == 0
        err = (out.float().cpu() - want[0].float()).abs().max().item()
        assert err <= tol, f"call {call}: max abs difference to ts_decode_layer {err}"
        ref = orc.sparse_attention(q[0].view(hq, d), kp, vp, rows.cpu(), sm_scale, base, 1.0, cap, torch.float64).reshape(-1)
        err = (out.double().cpu() - ref).abs().max().item()
        assert err <= tol, f"call {call}: max abs difference to the fp64 oracle {err}"


def test_static_scratch_reports_a_row_outside_the_pool():
    """A listed row outside [0, pool_rows) is read as row 0 and reported in the caller's status word; nothing faults."""
    hq, hkv, d, base = 8, 2, 128, 5e5
    dev = torch.device("cuda")
    a = synth.make_attention_case(71, 200, 0, hq, hkv, d)
    kd, vd, qd = a.k_pool.to(dev), a.v_pool.to(dev), a.q.to(dev)
    rows = a.slots.clone()
    rows[17] = kd.shape[0] + 5
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty_like(qd)
    attend_rows_static(qd, kd, vd, rows.to(dev), out, d ** -0.5, base, 1.0, 0.0, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 6                                    # TS_ERR_BAD_SLOT
    rows[17] = 0
    ref = orc.sparse_attention(a.q.view(hq, d), a.k_pool, a.v_pool, rows, d ** -0.5, base, 1.0, 0.0, torch.float64).reshape(-1)
    assert (out.double().cpu() - ref).abs().max().item() <= 2e-2
    with pytest.raises(ValueError):
        attend_rows_static(qd, kd, vd, rows.to(dev).long(), out, d ** -0.5, base)


def test_static_scratch_rejects_lists_beyond_its_fixed_array():
    from tokenselect_b200 import TokenSelectError
    dev = torch.device("cuda")
    hq, hkv, d = 32, 8, 128
    count = 8064 + 32                                                 # one chunk past the 4 MiB limit
    q = torch.zeros(hq * d, dtype=torch.bfloat16, device=dev)
    pool = torch.zeros(16, hkv, d, dtype=torch.bfloat16, device=dev)
    rows = torch.zeros(count, dtype=torch.int32, device=dev)
    with pytest.raises(TokenSelectError) as ei:
        attend_rows_static(q, pool, pool, rows, torch.empty_like(q), d ** -0.5, 5e5)
    assert ei.value.status == 4
    attend_rows_static(q, pool, pool, rows[:8064], torch.empty_like(q), d ** -0.5, 5e5)   # at the limit: accepted
    torch.cuda.synchronize()
