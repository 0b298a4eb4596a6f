"""Generate ``tests/golden/reference_selection.json`` by running the reference's own selection
code (``patcher/token_retrieval.py``, unmodified, CPU, Triton interpreter) on seeded inputs.

    python tests/golden/make_golden.py [--reference-root DIR]

Only seeds, shapes and the reference's outputs are stored; the inputs are regenerated from the
seed by ``oracle/synth.py``.  The file committed beside this script was produced by this script.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import reference_verbatim as rv  # noqa: E402  (sets TRITON_INTERPRET before triton loads)
from oracle import synth  # noqa: E402

# name, seed, N, Hq, Hkv, D, n_init, n_local, top_k, rope_base, kernel_size
CASES = [
    ("tiny_gqa4", 3, 2048, 8, 2, 128, 16, 64, 256, 5e5, -1),
    ("tiny_mha", 4, 1024, 4, 4, 64, 8, 32, 128, 1e4, -1),
    ("llama_8k", 1, 8192, 32, 8, 128, 128, 512, 1024, 5e5, -1),
    ("qwen_4k", 2, 4096, 28, 4, 128, 128, 512, 512, 1e6, -1),
    ("guard_equal", 5, 336, 8, 2, 128, 16, 64, 256, 5e5, -1),      # n_sel == N -> dense
    ("guard_plus1", 6, 337, 8, 2, 128, 16, 64, 256, 5e5, -1),      # n_sel + 1 == N -> Nc = k + 1
    ("pool_odd5", 7, 2048, 8, 2, 128, 16, 64, 256, 5e5, 5),
    ("pool_even6", 8, 2048, 8, 2, 128, 16, 64, 256, 5e5, 6),
]

# prefill chunks: name, seed, N (tokens incl. the chunk), chunk length, Hq, Hkv, D, n_init, n_local, top_k, rope_base
CHUNK_CASES = [
    ("chunk_gqa4", 21, 2048, 64, 8, 2, 128, 16, 64, 256, 5e5),
    ("chunk_partial37", 22, 1500, 37, 8, 2, 128, 16, 64, 256, 5e5),
    ("chunk_llama_512", 23, 8192, 512, 32, 8, 128, 128, 512, 1024, 5e5),
    ("chunk_dense", 24, 300, 64, 8, 2, 128, 16, 64, 256, 5e5),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=rv.DEFAULT_REFERENCE_ROOT)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "reference_selection.json"))
    args = ap.parse_args()
    import torch
    records = []
    for name, seed, n, hq, hkv, d, n_init, n_local, top_k, base, ks in CASES:
        case = synth.make_layer_case(seed, n, hq, hkv, d, n_init, n_local, base)
        out = rv.retrieval_indices(case.q, case.k_pool, case.req_to_token[case.req_pool_idx], n, hq, hkv, d,
                                   n_init, n_local, top_k, base, 1, ks, root=args.reference_root)
        records.append({
            "name": name, "seed": seed, "n_tokens": n, "hq": hq, "hkv": hkv, "head_dim": d,
            "n_init": n_init, "n_local": n_local, "top_k": top_k, "rope_base": base, "kernel_size": ks,
            "slots": None if out is None else [int(x) for x in out.tolist()],
        })
        print(name, "dense" if out is None else len(out))
    for name, seed, n, lq, hq, hkv, d, n_init, n_local, top_k, base in CHUNK_CASES:
        case = synth.make_layer_case(seed, n, hq, hkv, d, n_init, n_local, base)
        qc = synth.make_chunk_queries(seed, case, lq, hq, d)
        out = rv.retrieval_indices(qc, case.k_pool, case.req_to_token[case.req_pool_idx], n, hq, hkv, d,
                                   n_init, n_local, top_k, base, 1, -1, root=args.reference_root)
        records.append({
            "name": name, "seed": seed, "n_tokens": n, "chunk": lq, "hq": hq, "hkv": hkv, "head_dim": d,
            "n_init": n_init, "n_local": n_local, "top_k": top_k, "rope_base": base, "kernel_size": -1,
            "slots": None if out is None else [int(x) for x in out.tolist()],
        })
        print(name, "dense" if out is None else len(out))
    with open(args.out, "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "torch": torch.__version__,
                   "source": "patcher/token_retrieval.py TokenRetriever.retrieval_indices, fp32, CPU, "
                             "TRITON_INTERPRET=1", "cases": records}, f)
    print("wrote", args.out)


if __name__ == "__main__":
    main()
