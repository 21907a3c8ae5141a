"""Packs this library's sources into the ``solution.json`` the reference's harness consumes.

    python -m <package>.packaging.pack_solution [-o solution.json]

Counterpart of the reference's ``moe/scripts/pack_solution.py:34-86``, which hands its one source file
to the harness's packer.  That packer (``flashinfer_bench.agents.pack_solution_from_files``) is not
installed here, so this script writes the same document itself: the fields of the reference's own
``moe/solution.json`` — ``name``, ``definition``, ``author``, ``spec`` (language, target hardware, entry
point, dependencies, destination-passing style, binding), ``sources`` (path + content per file) and
``description``.

The harness compiles all ``sources`` in one flat directory, so the tree is flattened: every
translation unit of ``csrc/``, its two internal headers and ``include/syfi_moe.h`` land side by side,
``#include`` paths that climb directories are rewritten to the bare file name, and the tvm-ffi export
is renamed ``tvm_ffi_binding.cu`` (a CUDA-language solution compiles ``.cu`` files).  Only the files
listed in ``SOURCES`` are packed: what the single-GPU entry point needs.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys

try:
    import tomllib
except ImportError:  # pragma: no cover
    import tomli as tomllib

HERE = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.dirname(HERE)
REPO = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")

# (path in the repository, name in the flat solution directory)
SOURCES = [
    (os.path.join(CSRC, "tvm_ffi_binding.cc"), "tvm_ffi_binding.cu"),
    (os.path.join(CSRC, "api.cu"), "api.cu"),
    (os.path.join(CSRC, "router.cu"), "router.cu"),
    (os.path.join(CSRC, "permute.cu"), "permute.cu"),
    (os.path.join(CSRC, "grouped_gemm.cu"), "grouped_gemm.cu"),
    (os.path.join(CSRC, "grouped_gemm_pair.cu"), "grouped_gemm_pair.cu"),
    (os.path.join(CSRC, "combine.cu"), "combine.cu"),
    (os.path.join(CSRC, "ep_exchange.cu"), "ep_exchange.cu"),
    (os.path.join(CSRC, "prepack.cu"), "prepack.cu"),
    (os.path.join(CSRC, "moe_internal.h"), "moe_internal.h"),
    (os.path.join(CSRC, "ptx.cuh"), "ptx.cuh"),
    (os.path.join(REPO, "include", "syfi_moe.h"), "syfi_moe.h"),
]

_INCLUDE = re.compile(r'(#include\s+")(?:\.\./)+(?:[\w\-]+/)*([\w\-.]+")')


def flatten_includes(text: str) -> str:
    """``#include "../../include/syfi_moe.h"`` -> ``#include "syfi_moe.h"``."""
    return _INCLUDE.sub(r"\1\2", text)


def load_config(path: str | None = None) -> dict:
    with open(path or os.path.join(HERE, "config.toml"), "rb") as f:
        return tomllib.load(f)


def pack_solution(config: dict | None = None) -> dict:
    cfg = config or load_config()
    sol, build = cfg["solution"], cfg["build"]
    sources = []
    for src, name in SOURCES:
        with open(src) as f:
            sources.append({"path": name, "content": flatten_includes(f.read())})
    return {
        "name": sol["name"],
        "definition": sol["definition"],
        "author": sol["author"],
        "spec": {
            "language": build["language"],
            "target_hardware": list(build.get("target_hardware", ["cuda"])),
            "entry_point": build["entry_point"],
            "dependencies": [],
            "destination_passing_style": bool(build.get("destination_passing_style", True)),
            "binding": build.get("binding"),
        },
        "sources": sources,
        "description": "B200-native (sm_100a) fused FP8 block-scale DS-routing MoE layer: tcgen05 grouped GEMMs, "
                       "device-side scheduling, deterministic combine; compile every .cu for compute_100a.",
    }


def unpack_solution(doc: dict, directory: str) -> list[str]:
    """Writes ``sources`` into ``directory`` the way the harness's builder does; returns the paths."""
    os.makedirs(directory, exist_ok=True)
    paths = []
    for s in doc["sources"]:
        p = os.path.join(directory, s["path"])
        with open(p, "w") as f:
            f.write(s["content"])
        paths.append(p)
    return paths


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-o", "--output", default=os.path.join(HERE, "solution.json"))
    args = ap.parse_args()
    doc = pack_solution()
    with open(args.output, "w") as f:
        json.dump(doc, f, indent=2)
    print(f"solution packed: {args.output} ({len(doc['sources'])} sources, entry point {doc['spec']['entry_point']})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
