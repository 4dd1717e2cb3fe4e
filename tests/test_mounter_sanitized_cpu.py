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


def test_mutated_package_metadata_never_crashes_the_mounter(sanitized_mounter, tmp_path):
    """Seeded fuzzing of what the mounter parses: spans deleted or doubled, numbers replaced by zero, negative,
    2^32, 2^64 - 1 or the wrong type, strings replaced (other dtypes, paths outside the package, 5000 characters),
    files cut anywhere - in tensors.json, config.json, a lowered circuit and the manifest, with the manifest's integrity
    table brought up to date so that the mutation reaches the parser.  Every package must end as `ok` (a harmless
    mutation) or in an error message; the sanitizers must stay silent."""
    import hashlib
    import random
    import re

    rng = random.Random(7)
    source = GOLDEN / "tiny_int4_mtp"

    def mutate(text):
        kind = rng.randrange(6)
        if kind == 0:
            a = rng.randrange(len(text))
            return text[:a] + text[min(len(text), a + rng.randrange(1, 200)):]
        if kind == 1:
            match = rng.choice(list(re.finditer(r"-?\d+(\.\d+)?", text)))
            replacement = rng.choice(["-1", "0", "18446744073709551615", "9223372036854775808", "1e400", "4294967296", '""', "null", "[]", "7"])
            return text[:match.start()] + replacement + text[match.end():]
        if kind == 2:
            match = rng.choice(list(re.finditer(r'"[^"]*"', text)))
            replacement = rng.choice(['""', '"../../etc/passwd"', "123", "null", '"\\u0000"', '"' + "A" * 5000 + '"', '"BF16"', '"I32"', '"F8_E4M3"'])
            return text[:match.start()] + replacement + text[match.end():]
        if kind == 3:
            return text[:rng.randrange(len(text))]
        if kind == 4:
            a = rng.randrange(len(text))
            b = min(len(text), a + rng.randrange(1, 300))
            return text[:b] + text[a:b] + text[b:]
        a = rng.randrange(len(text))
        return text[:a] + rng.choice('{}[],:"0 ') + text[a + 1:]

    directories = []
    for index in range(160):
        directory = tmp_path / f"mutation_{index:03d}"
        shutil.copytree(source, directory)
        target = rng.choice(["tensors.json", "tensors.json", "config.json", "lowered/layer_00/circuit.json"])
        path = directory / target
        path.write_text(mutate(path.read_text()))
        manifest_path = directory / "vulkan_resident_package.json"
        manifest = json.loads(manifest_path.read_text())
        blob = path.read_bytes()
        if target in manifest["artifact_integrity"]["files"]:
            manifest["artifact_integrity"]["files"][target] = {"byte_count": len(blob), "sha256": hashlib.sha256(blob).hexdigest()}
        text = json.dumps(manifest)
        manifest_path.write_text(mutate(text) if rng.random() < 0.3 else text)
        directories.append(directory)
    _, lines = _run(sanitized_mounter, *directories)
    assert len(lines) == len(directories), "the mounter stopped early"
    assert all(line.startswith(("ok ", "error ")) for line in lines)
    assert sum(line.startswith("error ") for line in lines) >= len(lines) // 3  # the mutations do reach the checks


def test_mutated_weights_files_never_crash_the_mounter(sanitized_mounter, tmp_path):
    """The same for the safetensors files: header lengths of 0, 2^63, 2^64 - 1 or one off the file size, damaged header
    text, data offsets that are negative, reversed or far beyond the file, files cut anywhere or emptied."""
    import hashlib
    import random
    import struct

    rng = random.Random(3)
    source = GOLDEN / "tiny_int4_mtp"
    index = json.loads((source / "tensors.json").read_text())["tensors"]
    directories = []
    for number in range(80):
        directory = tmp_path / f"weights_{number:03d}"
        shutil.copytree(source, directory)
        relative = index[rng.choice(sorted(index))]["source_file"]
        path = directory / relative
        blob = bytearray(path.read_bytes())
        header_bytes = struct.unpack("<Q", blob[:8])[0]
        kind = rng.randrange(5)
        if kind == 0:
            blob[0:8] = struct.pack("<Q", rng.choice([0, 1, 7, 2 ** 63, 2 ** 64 - 1, len(blob), len(blob) + 1, len(blob) - 1, 2 ** 32]))
        elif kind == 1:
            blob[8 + rng.randrange(header_bytes)] = rng.choice(b'{}[]",:0 x')
        elif kind == 2:
            blob = blob[:rng.randrange(len(blob))]
        elif kind == 3:
            header = json.loads(bytes(blob[8:8 + header_bytes]))
            name = [key for key in header if key != "__metadata__"][0]
            header[name]["data_offsets"] = rng.choice([[0, 2 ** 62], [5, 3], [-1, 4], [0, 0], [2 ** 40, 2 ** 40 + 8]])
            text = json.dumps(header).encode()
            blob = bytearray(struct.pack("<Q", len(text)) + text + bytes(blob[8 + header_bytes:]))
        else:
            blob = bytearray()
        path.write_bytes(bytes(blob))
        manifest_path = directory / "vulkan_resident_package.json"
        manifest = json.loads(manifest_path.read_text())
        if relative in manifest["artifact_integrity"]["files"]:
            manifest["artifact_integrity"]["files"][relative] = {"byte_count": len(blob), "sha256": hashlib.sha256(bytes(blob)).hexdigest()}
            manifest_path.write_text(json.dumps(manifest))
        directories.append(directory)
    _, lines = _run(sanitized_mounter, *directories)
    assert len(lines) == len(directories), "the mounter stopped early"
    assert all(line.startswith(("ok ", "error ")) for line in lines)
    assert sum(line.startswith("error ") for line in lines) >= len(lines) // 3
