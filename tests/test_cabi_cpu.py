"""The C-ABI library loads without a GPU, exports every symbol include/nerve_b200.h declares, parses and verifies
real compiler output, and fails loudly (not by falling back) when asked to compute without a device."""

import re
import shutil
from pathlib import Path

import pytest

from conftest import GOLDEN, PACKAGES, ROOT


def test_library_exports_every_declared_symbol():
    import llmoop_b200 as nb
    from llmoop_b200 import runtime

    header = (ROOT / "include" / "nerve_b200.h").read_text()
    declared = set(re.findall(r"\b(nerve_b200_[a-z0-9_]+)\s*\(", header))
    declared -= {"nerve_b200_output_callback"}
    assert declared == set(runtime.EXPORTED_SYMBOLS)
    lib = nb.library()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.nerve_b200_abi_version() == 1


@pytest.mark.parametrize("name", PACKAGES)
def test_golden_packages_validate_with_full_integrity_checks(name):
    import llmoop_b200 as nb

    ops, tensors = nb.validate_package(GOLDEN / name, 2)
    assert ops > 0 and tensors > 0


def test_integrity_failures_name_the_artifact(tmp_path):
    import llmoop_b200 as nb

    broken = tmp_path / "broken"
    shutil.copytree(GOLDEN / "tiny_int4_mtp_v16", broken)
    (broken / "tensors.json").write_text((broken / "tensors.json").read_text() + " ")
    with pytest.raises(nb.NerveError, match="tensors.json"):
        nb.validate_package(broken, 1)
    shutil.rmtree(broken)
    shutil.copytree(GOLDEN / "tiny_int4_mtp_v16", broken)
    weights = sorted((broken / "weights").glob("*.safetensors"))[3]
    weights.write_bytes(weights.read_bytes()[:-7])
    with pytest.raises(nb.NerveError, match="truncated"):
        nb.validate_package(broken, 1)


def test_a_tensor_index_that_promises_more_than_the_bytes_hold_is_rejected(tmp_path):
    """The kernels take their extents from the index's shapes, so a shape the stored bytes do not cover must stop
    the mount on the host (the reference: vulkan_distributed/planning.rs:582)."""
    import json

    import llmoop_b200 as nb

    def mutated(edit):
        package = tmp_path / "pkg"
        if package.exists():
            shutil.rmtree(package)
        shutil.copytree(GOLDEN / "tiny_int4_mtp_v16", package)
        index = json.loads((package / "tensors.json").read_text())
        edit(index["tensors"])
        (package / "tensors.json").write_text(json.dumps(index))
        return package

    def double_rows(name_filter):
        def edit(tensors):
            name = next(n for n, t in sorted(tensors.items()) if name_filter(n, t))
            for key in ("shape", "logical_shape"):
                if key in tensors[name]:
                    tensors[name][key][0] *= 2
        return edit

    quantized = lambda n, t: "quantization" in t
    scales = lambda n, t: n.endswith("weight_scale")
    norms = lambda n, t: "norm" in n and len(t["shape"]) == 1
    for edit in (double_rows(quantized), double_rows(scales), double_rows(norms)):
        with pytest.raises(nb.NerveError, match="does not match shape|bytes where"):
            nb.validate_package(mutated(edit), 0)

    def end_before_begin(tensors):
        name = sorted(tensors)[0]
        tensors[name]["data_offsets"] = [8, 4]
        tensors[name].pop("byte_count", None)
    with pytest.raises(nb.NerveError, match="end before they begin"):
        nb.validate_package(mutated(end_before_begin), 0)


def test_unknown_schema_and_ops_are_rejected(tmp_path):
    import json

    import llmoop_b200 as nb

    package = tmp_path / "pkg"
    shutil.copytree(GOLDEN / "tiny_int4_mtp_v16", package)
    manifest = json.loads((package / "vulkan_resident_package.json").read_text())
    manifest["component_executions"][0]["kernels"][0]["op"] = "gated_delta_step"
    (package / "vulkan_resident_package.json").write_text(json.dumps(manifest))
    with pytest.raises(nb.NerveError, match="no kernel for op"):
        nb.validate_package(package, 0)
    manifest["schema"] = "nerve.vulkan_resident_model_package.v2"
    (package / "vulkan_resident_package.json").write_text(json.dumps(manifest))
    with pytest.raises(nb.NerveError, match="unsupported package schema"):
        nb.validate_package(package, 0)


def test_mount_without_a_gpu_is_an_error_not_a_fallback():
    import torch

    import llmoop_b200 as nb

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(nb.NerveError):
        nb.Package(GOLDEN / "tiny_int4_mtp_v16", capacity_tokens=64)


def test_product_never_imports_the_oracle():
    for path in (ROOT / "llmoop_b200").rglob("*"):
        if path.suffix in (".py", ".cu", ".cpp", ".hpp", ".cuh", ".h"):
            text = path.read_text()
            assert "nerve_oracle" not in text and "oracle/" not in text, path


def test_reference_tiny_model_golden_equals_the_checked_in_fixture():
    """tests/golden/packages/reference_tiny_model was rebuilt from the generator formula with the reference
    compiler; its tensor index (names, shapes, file names, SHA-256 of every tensor) must equal the package the
    reference ships for its own runtime tests."""
    import json

    fixture = ROOT.parent / "reference" / "runtime-rs" / "test-fixtures" / "tiny_model"  # the reference checkout beside this repository
    if not fixture.exists():
        pytest.skip("reference checkout not present")
    ours = json.loads((GOLDEN / "reference_tiny_model" / "tensors.json").read_text())
    theirs = json.loads((fixture / "tensors.json").read_text())
    assert ours["tensors"] == theirs["tensors"]
    import llmoop_b200 as nb

    assert nb.validate_package(fixture, 2) == nb.validate_package(GOLDEN / "reference_tiny_model", 2) == (9, 11)
