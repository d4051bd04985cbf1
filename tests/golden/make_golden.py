"""Regenerate ``naive_colsum_golden.npz`` from the reference implementation itself.

Run where a checkout of the reference is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [/path/to/reference]

It imports ``naive_colsum`` straight from the reference's ``flash_colsum/baselines.py``
(loaded by file path, so the reference's Triton kernels are not imported), feeds
it the seeded inputs of ``CASES`` upcast to fp32, and stores for each case the
fp32 output and a sha256 of the input bytes.  The tests regenerate the inputs
from the same seeds, check the digest, and compare the checkers with the stored
outputs; the reference checkout is not needed to run them.
"""

from __future__ import annotations

import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from flash_colsum_b200.inputs import Workload, make_inputs, digest  # noqa: E402

# name, B, H, Sq, Sk, D, dtype, causal, cls_len, outliers, key_is_query, seed
CASES = [
    Workload("c1_cpu_reference", 2, 4, 256, 256, 64, "fp32", seed=0),
    Workload("noncausal_fp16_tile_multiple", 2, 3, 128, 128, 64, "fp16", seed=1),
    Workload("noncausal_fp16_ragged_100", 2, 2, 100, 100, 64, "fp16", seed=2),
    Workload("noncausal_fp16_ragged_577", 1, 2, 577, 577, 64, "fp16", seed=3),
    Workload("noncausal_bf16_d128", 2, 2, 192, 192, 128, "bf16", seed=4),
    Workload("noncausal_key_is_query", 1, 4, 256, 256, 64, "fp16", key_is_query=True, seed=5),
    Workload("cls1_fp16_577", 3, 4, 577, 577, 64, "fp16", cls_len=1, seed=6),
    Workload("cls2_fp16", 1, 4, 300, 300, 64, "fp16", cls_len=2, seed=7),
    Workload("cls_longer_than_s", 2, 2, 40, 40, 64, "fp16", cls_len=64, seed=8),
    Workload("cls200_bf16_d128", 1, 2, 384, 384, 128, "bf16", cls_len=200, seed=9),
    Workload("causal_fp16_suffix_128_of_1024", 1, 4, 128, 1024, 128, "fp16", is_causal=True, seed=10),
    Workload("causal_fp16_ragged_q24_k200", 1, 3, 24, 200, 128, "fp16", is_causal=True, seed=11),
    Workload("causal_square_96", 1, 2, 96, 96, 64, "fp16", is_causal=True, seed=12),
    Workload("causal_keys_shorter_than_queries", 1, 2, 64, 40, 64, "fp16", is_causal=True, seed=13),
    Workload("causal_bf16_outlier_keys", 1, 4, 64, 2048, 128, "bf16", is_causal=True,
             key_outliers=True, seed=14),
    Workload("causal_q300_k700_d64", 1, 2, 300, 700, 64, "bf16", is_causal=True, seed=15),
    # head dimensions other than 64 and 128 (the reference's naive_colsum defines every D)
    Workload("noncausal_fp16_d32", 2, 3, 300, 300, 32, "fp16", seed=16),
    Workload("causal_bf16_d80", 1, 3, 200, 900, 80, "bf16", is_causal=True, seed=17),
    Workload("cls_fp16_d96", 2, 2, 577, 577, 96, "fp16", cls_len=1, seed=18),
    Workload("noncausal_fp16_d72", 1, 4, 577, 577, 72, "fp16", seed=19),
    Workload("causal_fp16_d8_long", 1, 2, 100, 2500, 8, "fp16", is_causal=True, seed=20),
    # fp32 inputs
    Workload("causal_fp32_d128", 1, 2, 128, 600, 128, "fp32", is_causal=True, seed=21),
    Workload("noncausal_fp32_d80", 2, 2, 260, 260, 80, "fp32", seed=22),
]


def load_reference(root: str):
    path = os.path.join(root, "flash_colsum", "baselines.py")
    spec = importlib.util.spec_from_file_location("_reference_baselines", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.naive_colsum


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    root = sys.argv[1]
    naive_colsum = load_reference(root)
    arrays, manifest = {}, []
    for w in CASES:
        q, k = make_inputs(w)
        out = naive_colsum(q.float(), k.float(), scale=None, is_causal=w.is_causal,
                           cls_len=w.cls_len)
        # also the reference run in the input dtype, as its own tests call it
        out_native = naive_colsum(q, k, scale=None, is_causal=w.is_causal, cls_len=w.cls_len)
        arrays[w.name] = out.to(torch.float32).numpy()
        arrays[w.name + "__native"] = out_native.to(torch.float32).numpy()
        manifest.append({**{f: getattr(w, f) for f in w.__dataclass_fields__},
                         "sha256": digest(q, k)})
        print(w.name, tuple(out.shape), float(out.sum()))
    np.savez_compressed(os.path.join(HERE, "naive_colsum_golden.npz"), **arrays)
    with open(os.path.join(HERE, "naive_colsum_golden.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": manifest}, f, indent=1)


if __name__ == "__main__":
    main()
