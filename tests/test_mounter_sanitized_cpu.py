"""The mounter's host code (llmoop_b200/csrc/package.cpp) under AddressSanitizer and UndefinedBehaviorSanitizer,
without a GPU: tests/package_mount_cases.cpp opens packages with full verification and reads every tensor back.
Golden packages must pass; damaged copies (a truncated weights file, a flipped weight byte, a tensor index that
promises twice the rows, a manifest cut in the middle) must end in the mounter's own error message - never in a
sanitizer report or a crash (the reference rejects such packages with an error value too:
vulkan_distributed/planning.rs:582, package/specs.rs:35-46)."""

import json
import shutil
import subprocess
from pathlib import Path

import pytest

from conftest import GOLDEN, PACKAGES

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def sanitized_mounter(tmp_path_factory):
    out = tmp_path_factory.mktemp("mounter") / "package_mount_cases"
    command = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
               str(ROOT / "tests" / "package_mount_cases.cpp"), str(ROOT / "llmoop_b200" / "csrc" / "package.cpp"), "-o", str(out)]
    built = subprocess.run(command, capture_output=True, text=True)
    if built.returncode != 0 and "sanitize" in built.stderr and ("cannot find" in built.stderr or "unrecognized" in built.stderr):
        pytest.skip("the sanitizer runtimes are not installed")
    assert built.returncode == 0, built.stdout + built.stderr
    return out


def _run(binary, *directories):
    result = subprocess.run([str(binary), *[str(d) for d in directories]], capture_output=True, text=True)
    assert not result.stderr.strip(), result.stderr[-3000:]  # a sanitizer report goes to stderr
    return result.returncode, result.stdout.strip().splitlines()


def test_golden_packages_open_and_read_back_clean(sanitized_mounter):
    code, lines = _run(sanitized_mounter, *[GOLDEN / name for name in PACKAGES + ["reference_tiny_model"]])
    assert code == 0 and all(line.startswith("ok ") for line in lines) and len(lines) == len(PACKAGES) + 1, lines


def _weights_file(directory, tensor):
    index = json.loads((directory / "tensors.json").read_text())["tensors"]
    return directory / index[tensor]["source_file"]


def test_damaged_packages_end_in_an_error_message(sanitized_mounter, tmp_path):
    source = GOLDEN / "tiny_int4_mtp"
    tensor = "model.layers.0.mlp.down_proj.weight_packed"

    truncated = tmp_path / "truncated"
    shutil.copytree(source, truncated)
    path = _weights_file(truncated, tensor)
    path.write_bytes(path.read_bytes()[:-64])

    flipped = tmp_path / "flipped"
    shutil.copytree(source, flipped)
    path = _weights_file(flipped, tensor)
    blob = bytearray(path.read_bytes())
    blob[-1] ^= 0x5A
    path.write_bytes(bytes(blob))

    doubled = tmp_path / "doubled"
    shutil.copytree(source, doubled)
    index = json.loads((doubled / "tensors.json").read_text())
    index["tensors"][tensor]["shape"][0] *= 2
    index["tensors"][tensor]["logical_shape"][0] *= 2
    (doubled / "tensors.json").write_text(json.dumps(index))

    cut = tmp_path / "cut"
    shutil.copytree(source, cut)
    manifest = (cut / "vulkan_resident_package.json").read_text()
    (cut / "vulkan_resident_package.json").write_text(manifest[: len(manifest) // 2])

    code, lines = _run(sanitized_mounter, truncated, flipped, doubled, cut, source)
    assert code == 4, lines
    assert [line.split()[0] for line in lines] == ["error", "error", "error", "error", "ok"], lines
    assert all(len(line.split(":", 1)[1].strip()) > 10 for line in lines[:4]), lines  # each names what is wrong
