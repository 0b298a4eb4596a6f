"""The bench's reference arm (CPU oracle timed on the host cores) and its byte accounting, on CPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.check_output([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--ctx", "4096",
                                   "--layers", "2", "--steps", "2", "--warmup", "1"], text=True, timeout=600)
    line = json.loads(out.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"]
    # one step is one decoded token (all layers), the counts printed are the counts really run, and the
    # workload string is the GPU arm's
    sys.path.insert(0, ROOT)
    import bench
    assert line["steps"] == 2 and line["warmup"] == 1
    assert line["config"]["workload"] == bench.workload_string(4096, 2)
    assert abs(line["ms_per_step"] * 1e-3 * line["value"] - 1.0) < 1e-6
    assert abs(line["us_per_layer"] * 2 - line["ms_per_step"] * 1e3) < 1e-3


def test_algorithmic_bytes_of_the_headline_shape():
    sys.path.insert(0, ROOT)
    import bench
    ab = bench.algorithmic_bytes(131072, 32, 8, 128)
    # key rows + row numbers + query + index list; K and V rows of the list + row numbers + query + output
    assert ab["select"] == 130432 * 2048 + 130432 * 4 + 32 * 128 * 2 + 2688 * 4
    assert ab["attend"] == 2 * 2688 * 2048 + 2688 * 4 + 2 * 32 * 128 * 2
    assert abs(ab["layer"] / 1e6 - 278.7) < 0.1


def test_attention_error_discounts_only_the_output_rounding():
    """The bench's attention check holds the error beyond the output's own bf16 rounding (half a bf16 step =
    2^-8 of the magnitude) to 2e-2: a large output rounded to bf16 passes, a small output that is off does not."""
    import torch
    sys.path.insert(0, ROOT)
    import bench
    ref = torch.tensor([13.037, -9.51, 0.3, 1e-3], dtype=torch.float64)
    rounded = ref.to(torch.bfloat16)
    err, beyond, ref_max = bench.attention_error(rounded, ref)
    assert err > 2e-2 and beyond <= 1e-6 and abs(ref_max - 13.037) < 1e-9        # pure rounding: nothing beyond it
    off = ref.clone()
    off[2] += 0.05
    err, beyond, _ = bench.attention_error(off, ref)
    assert abs(err - 0.05) < 1e-9 and beyond > 2e-2                               # an error of order-one outputs shows
    assert bench.attention_tolerance(1.3) == 2e-2 and abs(bench.attention_tolerance(10.0) - 5e-2) < 1e-12
