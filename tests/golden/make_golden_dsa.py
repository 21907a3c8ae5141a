"""Generates tests/golden/dsa_*.pt: outputs of the reference's OWN entry point for the DSA top-k indexer
(dsa_indexer/solution/python/dsa_topk_indexer.py::run, pure torch, the configured entry point of that definition)
on seeded inputs.  Run where the reference tree is available:

    python tests/golden/make_golden_dsa.py /path/to/reference

The inputs are regenerated from the stored seeds by oracle.dsa_oracle.make_inputs; only the reference's output
is stored.
"""
import importlib.util
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import dsa_oracle  # noqa: E402

CASES = {
    "dsa_small": dict(seq_lens=[0, 1, 63, 64, 65, 700], seed=1),
    "dsa_cut": dict(seq_lens=[2048, 2049, 3000, 5000], seed=2),
    "dsa_long": dict(seq_lens=[9000, 130], seed=3, weight_sign="positive"),
}


def main(ref_root):
    path = os.path.join(ref_root, "dsa_indexer", "solution", "python", "dsa_topk_indexer.py")
    spec = importlib.util.spec_from_file_location("ref_dsa_topk_indexer", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for name, kw in CASES.items():
        q, cache, w, sl, table = dsa_oracle.make_inputs(**kw)
        out = torch.empty(len(kw["seq_lens"]), dsa_oracle.TOPK, dtype=torch.int32)
        ref.run(q, cache, w, sl, table, out)
        torch.save({"make_inputs": kw, "topk_indices": out}, os.path.join(HERE, name + ".pt"))
        print(name, out.shape, int((out >= 0).sum()))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference"))
