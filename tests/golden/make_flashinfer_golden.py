"""Generate ``tests/golden/flashinfer_attention.npz``: outputs of the third-party attention library the
reference calls (FlashInfer), run ON A GPU with the arguments of the reference's two call sites, on seeded
inputs.  The CPU oracle's ``sparse_attention`` / ``sparse_prefill_attention`` are held to these outputs by
``tests/test_oracle_flashinfer.py``.  TEST INFRASTRUCTURE: nothing of the product path imports FlashInfer.

    python tests/golden/make_flashinfer_golden.py [--out FILE]

Call sites mirrored (patcher/token_retrieval.py):
  decode  :802-823  wrapper planned with (indptr = [0, n], indices = the row list, last_page_len = [1],
                    Hq, Hkv, D, page size 1) and run with sm_scale, logits_soft_cap, rope_scale,
                    rope_theta, pos_encoding_mode = "ROPE_LLAMA" on q [1, Hq, D] and the (K, V) buffers;
  prefill :746-772  paged prefill wrapper planned with qo_indptr = [0, Lq] and the same list, run with
                    causal = True and the same rotation arguments on q [Lq, Hq, D].
The installed FlashInfer takes the rotation mode and scales at plan time instead of at run time; the
arithmetic requested is the same.  Only seeds, shapes and FlashInfer's outputs are stored; the inputs are
regenerated from the seed by ``oracle/synth.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import synth  # noqa: E402

# name, seed, listed rows, chunk length (0: decode only), Hq, Hkv, D, rope_base, rope_scale, logit_cap, sm_scale
CASES = [
    ("gqa4", 31, 700, 48, 8, 2, 128, 5e5, 1.0, 0.0, None),
    ("qwen_group7", 32, 520, 32, 28, 4, 128, 1e6, 1.0, 0.0, None),
    ("mha_d64", 33, 300, 40, 4, 4, 64, 1e4, 1.0, 0.0, None),
    ("rope_scale2", 34, 640, 48, 8, 2, 128, 5e5, 2.0, 0.0, None),
    ("softcap30", 35, 512, 32, 8, 2, 128, 5e5, 1.0, 30.0, 0.5),
    ("llama_list2688", 36, 2688, 0, 32, 8, 128, 5e5, 1.0, 0.0, None),
]


def run_case(dev, name, seed, n, lq, hq, hkv, d, base, scale, cap, sm):
    import flashinfer
    c = synth.make_attention_case(seed, n, lq, hq, hkv, d)
    sm_scale = d ** -0.5 if sm is None else sm
    kc, vc = c.k_pool.to(dev).unsqueeze(1).contiguous(), c.v_pool.to(dev).unsqueeze(1).contiguous()
    idx = c.slots.to(dev)
    indptr = torch.tensor([0, n], dtype=torch.int32, device=dev)
    last = torch.ones(1, dtype=torch.int32, device=dev)
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device=dev)
    common = dict(pos_encoding_mode="ROPE_LLAMA", logits_soft_cap=cap if cap > 0 else None, sm_scale=sm_scale,
                  rope_scale=scale, rope_theta=base, q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
    rec, arrays = {"name": name, "seed": seed, "n_list": n, "chunk": lq, "hq": hq, "hkv": hkv, "head_dim": d,
                   "rope_base": base, "rope_scale": scale, "logit_cap": cap, "sm_scale": sm_scale}, {}
    # decode: CUDA-core decode kernel where the head group is one it is built for, tensor-core path otherwise
    out = None
    for tc in (False, True):
        try:
            w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD", use_tensor_cores=tc)
            w.plan(indptr, idx, last, hq, hkv, d, 1, **common)
            out = w.run(c.q.to(dev).view(1, hq, d), (kc, vc))
            torch.cuda.synchronize()
            rec["decode_tensor_cores"] = tc
            break
        except Exception as e:                      # noqa: BLE001 (recorded, next variant tried)
            rec["decode_error_tc_%s" % tc] = repr(e)[:200]
    if out is None:
        raise RuntimeError(f"{name}: decode wrapper failed: {rec}")
    arrays[f"{name}__decode"] = out.float().cpu().numpy().reshape(hq, d)
    if lq > 0:
        qo = torch.tensor([0, lq], dtype=torch.int32, device=dev)
        w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
        w.plan(qo, indptr, idx, last, hq, hkv, d, 1, causal=True, **common)
        o = w.run(c.q_chunk.to(dev).view(lq, hq, d), (kc, vc))
        torch.cuda.synchronize()
        arrays[f"{name}__prefill"] = o.float().cpu().numpy().reshape(lq, hq, d)
    return rec, arrays


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "flashinfer_attention.npz"))
    args = ap.parse_args()
    import flashinfer
    dev = torch.device("cuda:0")
    records, arrays = [], {}
    for case in CASES:
        rec, arr = run_case(dev, *case)
        records.append(rec)
        arrays.update(arr)
        print(rec["name"], {k: v.shape for k, v in arr.items()}, flush=True)
    meta = {"flashinfer": flashinfer.__version__, "torch": torch.__version__,
            "gpu": torch.cuda.get_device_name(0), "cases": records}
    # bf16 outputs are stored as fp16-safe fp32 -> keep fp32, compressed
    np.savez_compressed(args.out, meta=np.array(json.dumps(meta)), **arrays)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
