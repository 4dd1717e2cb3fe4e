"""Minimal safetensors reader/writer on raw bytes (no torch, no ml_dtypes).

The file format is: 8-byte little-endian header length N, N bytes of JSON
(`{name: {dtype, shape, data_offsets:[begin,end]}, "__metadata__": {...}}`),
then the concatenated tensor data.  Compiled NERVE packages store one tensor
per file under `weights/` with `__metadata__ = {format: "nerve", layout:
"row_major"}`; the runtime reads tensor bytes at `8 + N + data_offsets[0]`
(reference: runtime-rs/src/tensor_storage.rs:211-225).

Tensors are handled as (dtype string, shape, numpy uint8/uint16/int32/float32
array or raw bytes); BF16 is carried as uint16 bit patterns and F8_E4M3 as
uint8 bit patterns so that no rounding happens inside this module.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

DTYPE_BYTES = {
    "BF16": 2,
    "F16": 2,
    "F32": 4,
    "F8_E4M3": 1,
    "I32": 4,
    "I64": 8,
    "U8": 1,
    "I8": 1,
}

_NUMPY_CARRIER = {
    "BF16": np.uint16,
    "F16": np.float16,
    "F32": np.float32,
    "F8_E4M3": np.uint8,
    "I32": np.int32,
    "I64": np.int64,
    "U8": np.uint8,
    "I8": np.int8,
}


def carrier_dtype(dtype: str):
    return _NUMPY_CARRIER[dtype]


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """tensors: name -> (dtype, shape, array-or-bytes)."""
    header: dict = {}
    if metadata is not None:
        header["__metadata__"] = metadata
    offset = 0
    blobs = []
    for name, (dtype, shape, data) in tensors.items():
        raw = data if isinstance(data, (bytes, bytearray, memoryview)) else np.ascontiguousarray(data)
        count = 1
        for dim in shape:
            count *= int(dim)
        byte_count = count * DTYPE_BYTES[dtype]
        raw_len = len(raw) if isinstance(raw, (bytes, bytearray)) else raw.nbytes
        if raw_len != byte_count:
            raise ValueError(f"{name}: {raw_len} data bytes for {dtype}{list(shape)} ({byte_count})")
        header[name] = {
            "dtype": dtype,
            "shape": [int(d) for d in shape],
            "data_offsets": [offset, offset + byte_count],
        }
        offset += byte_count
        blobs.append(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for raw in blobs:
            if isinstance(raw, (bytes, bytearray, memoryview)):
                handle.write(raw)
            else:
                raw.tofile(handle)


def read_safetensors_header(path):
    with open(path, "rb") as handle:
        (length,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(length))
    return header, 8 + length


def read_safetensors(path) -> dict:
    """Returns name -> (dtype, shape, numpy array in the carrier dtype)."""
    header, base = read_safetensors_header(path)
    blob = Path(path).read_bytes()
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        array = np.frombuffer(blob, dtype=np.uint8, count=end - begin, offset=base + begin)
        array = array.view(carrier_dtype(entry["dtype"])).reshape(entry["shape"])
        out[name] = (entry["dtype"], tuple(entry["shape"]), array)
    return out


# --- bit-exact scalar-format helpers (numpy) ---------------------------------

def f32_to_bf16_bits(values) -> np.ndarray:
    """Round-to-nearest-even on the f32 bit pattern, no NaN special case:
    (bits + 0x7fff + lsb) >> 16."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    return ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(bits) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def _e4m3_table() -> np.ndarray:
    table = np.zeros(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exponent = (code >> 3) & 0xF
        mantissa = code & 0x7
        if exponent == 0xF and mantissa == 0x7:
            value = float("nan")
        elif exponent == 0:
            value = (mantissa / 8.0) * 2.0 ** -6
        else:
            value = (1.0 + mantissa / 8.0) * 2.0 ** (exponent - 7)
        table[code] = sign * value
    return table


E4M3_TO_F32 = _e4m3_table()


def f32_to_e4m3_bits(values) -> np.ndarray:
    """Round-to-nearest-even f32 -> e4m3fn with saturation to +-448."""
    x = np.ascontiguousarray(values, dtype=np.float32)
    sign = np.signbit(x)
    mag = np.minimum(np.abs(x).astype(np.float64), 448.0)
    exponent = np.floor(np.log2(np.maximum(mag, 2.0 ** -20)))
    exponent = np.maximum(exponent, -6.0)
    quantum = 2.0 ** (exponent - 3.0)
    scaled = np.rint(mag / quantum)  # numpy rint = ties-to-even
    mag_q = np.minimum(scaled * quantum, 448.0)
    # encode
    exponent_q = np.floor(np.log2(np.maximum(mag_q, 2.0 ** -20)))
    normal = mag_q >= 2.0 ** -6
    exponent_q = np.where(normal, exponent_q, -6.0)
    mantissa = np.where(normal, mag_q / 2.0 ** exponent_q - 1.0, mag_q / 2.0 ** -6) * 8.0
    code = np.where(normal, (exponent_q + 7.0) * 8.0 + mantissa, mantissa).astype(np.uint8)
    code = np.where(mag_q == 0.0, np.uint8(0), code)
    return (code | (sign.astype(np.uint8) << 7)).astype(np.uint8)
