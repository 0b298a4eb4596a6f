"""The allocation-free attention entry point (``ts_attend_rows_static``) against the regular one.

Some callers may not allocate device memory at the moment they need attention -- they run inside a
serving loop or callback that must stay clear of the allocator (an allocation can stall the device), or
all of the process's device memory was given to another component at start-up.  For them the library keeps the split kernel's partial
results in a fixed array of its own image instead of a workspace from ``ts_create``.  This test calls that
entry point through the C ABI twice in a row (the array keeps the previous call's contents, which must
not matter) and compares with the output of ``ts_decode_layer`` on the same rows, within the tolerance the
other attention tests use (2e-2 absolute for bf16, 1e-5 in fp32 check mode is not claimed here because
cos/sin are evaluated in the kernel rather than read from the host-built tables: 1e-3).

Collected last on purpose: a failure here must not hide the results of the other tests.
"""
import pytest
import torch

from oracle import synth
from tests import gpu_util as gu
from tokenselect_b200.engine import attend_rows_static

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-3)], ids=["bf16", "fp32"])
def test_static_scratch_attention_matches_regular_entry_point(dtype, tol):
    hq, hkv, d, n_init, n_local, k, base = 8, 2, 128, 16, 64, 256, 5e5
    eng = gu.make_engine(hq, hkv, d, n_init, n_local, k, base, dtype, max_ctx=4096)
    dev = eng.device
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for call, (seed, n) in enumerate(((61, 3000), (62, 1700))):       # two calls in a row, different lists
        case = synth.make_layer_case(seed, n, hq, hkv, d, n_init, n_local, base, dtype=dtype)
        q, kp, vp, rtt, ridx, lens = gu.case_tensors(case)
        want, res = gu.run_gpu(eng, 0, q, kp, vp, rtt, ridx, lens)
        rows = res["slots"][0, : int(res["count"][0])].to(dev)
        kd, vd, qd = kp.to(dev), vp.to(dev), q[0].contiguous().to(dev)
        out = torch.empty_like(qd)                                    # the caller owns the output
        # torch's count of allocations made so far only grows; bytes in use would also move when Python
        # happens to collect tensors of earlier tests during the call
        before = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
        attend_rows_static(qd, kd, vd, rows, out, d ** -0.5, base, 1.0, 0.0, status)
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats(dev)["allocation.all.allocated"] == before
        assert int(status.item()) == 0
        err = (out.float().cpu() - want[0].float()).abs().max().item()
        assert err <= tol, f"call {call}: max abs difference {err}"


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
