"""The packaging pair: config.toml + pack_solution (counterparts of the reference's moe/config.toml and
moe/scripts/pack_solution.py).  CPU only."""
import importlib
import json
import os
import shutil
import subprocess

import pytest

PKG = "mlsys-contest-syfi-agent-assisted_b200"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def packer():
    return importlib.import_module(PKG + ".packaging.pack_solution")


def test_config_names_the_reference_definition_and_binding(packer):
    cfg = packer.load_config()
    assert cfg["solution"]["definition"] == "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
    assert cfg["build"]["binding"] == "tvm-ffi" and cfg["build"]["language"] == "cuda"
    assert cfg["build"]["destination_passing_style"] is True
    assert cfg["build"]["entry_point"].endswith("::run_moe")


def test_solution_document_round_trips(packer, tmp_path):
    doc = packer.pack_solution()
    # same top-level fields as the reference's own solution.json
    assert set(doc) == {"name", "definition", "author", "spec", "sources", "description"}
    assert set(doc["spec"]) == {"language", "target_hardware", "entry_point", "dependencies",
                                "destination_passing_style", "binding"}
    again = json.loads(json.dumps(doc))
    assert again == doc
    names = [s["path"] for s in doc["sources"]]
    entry_file, entry_fn = doc["spec"]["entry_point"].split("::")
    assert entry_file in names and entry_fn == "run_moe"
    assert all("/" not in n for n in names)                       # flat directory
    # every source equals the repository file except for the flattened include paths
    for (src, name), packed in zip(packer.SOURCES, doc["sources"]):
        text = open(src).read()
        assert packed["path"] == name and packed["content"] == packer.flatten_includes(text)
        assert '#include "../' not in packed["content"]
    entry = next(s for s in doc["sources"] if s["path"] == entry_file)
    assert "TVM_FFI_DLL_EXPORT_TYPED_FUNC(run_moe" in entry["content"]
    # every quoted include resolves inside the flat directory
    import re
    for s in doc["sources"]:
        for inc in re.findall(r'#include\s+"([^"]+)"', s["content"]):
            assert inc in names, (s["path"], inc)
    paths = packer.unpack_solution(doc, str(tmp_path / "flat"))
    assert sorted(os.path.basename(p) for p in paths) == sorted(names)


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc")
def test_unpacked_headers_compile_from_the_flat_directory(packer, tmp_path):
    """A translation unit of the flat directory compiles without the repository's directory layout."""
    doc = packer.pack_solution()
    flat = str(tmp_path / "flat")
    packer.unpack_solution(doc, flat)
    proc = subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-c",
                           os.path.join(flat, "combine.cu"), "-o", os.path.join(flat, "combine.o")],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-2000:]
