"""Reading and writing safetensors checkpoints.

File layout and the checks follow the reference's reader (internal/safetensors/safetensors.go:42-165):
an 8-byte little-endian header length n (0 < n <= 100 MiB, n + 8 <= file size), a JSON object
name -> {dtype, shape, data_offsets}, ``__metadata__`` skipped, offsets checked against the file
size, byte count checked against shape x width.  A model folder holds ``model.safetensors`` or
the shards listed by ``model.safetensors.index.json``; shard names must be plain file names.

Tensors are returned as numpy views over a read-only memory map: BF16 as uint16 bit patterns,
F16 as float16, F32 as float32, integers as stored.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import numpy as np

_MAX_HEADER = 100 << 20

_DTYPES = {
    "BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4), "F64": (np.float64, 8),
    "I64": (np.int64, 8), "I32": (np.int32, 4), "I16": (np.int16, 2), "I8": (np.int8, 1),
    "U8": (np.uint8, 1), "BOOL": (np.uint8, 1),
}


class CheckpointError(ValueError):
    pass


@dataclass
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    file_index: int
    offset: int
    size: int


class Checkpoint:
    """The tensor index of a model folder; tensors are read lazily from memory maps."""

    def __init__(self, model_dir: str):
        self.dir = model_dir
        self.tensors: Dict[str, TensorEntry] = {}
        self._files: List[object] = []
        self._maps: List[mmap.mmap] = []
        names = ["model.safetensors"]
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(index_path):
            try:
                with open(index_path, "r") as f:
                    index = json.load(f)
                weight_map = index["weight_map"]
            except (OSError, ValueError, KeyError) as e:
                raise CheckpointError(f"safetensors: cannot parse {index_path}: {e}") from e
            names = []
            for shard in weight_map.values():
                if shard not in names:
                    names.append(shard)
        try:
            for name in names:
                if os.path.basename(name) != name:
                    raise CheckpointError(f"safetensors: shard {name!r} is not a plain file name")
                path = os.path.join(model_dir, name)
                try:
                    f = open(path, "rb")
                except OSError as e:
                    raise CheckpointError(f"safetensors: cannot open {path}: {e}") from e
                self._files.append(f)
                self._read_header(f, name, len(self._files) - 1)
        except Exception:
            self.close()
            raise

    def _read_header(self, f, name: str, file_index: int) -> None:
        size = os.fstat(f.fileno()).st_size
        head = f.read(8)
        if len(head) != 8:
            raise CheckpointError(f"safetensors: {name}: file of {size} bytes is too short for a header")
        (n,) = struct.unpack("<Q", head)
        if n == 0 or n > _MAX_HEADER or n + 8 > size:
            raise CheckpointError(f"safetensors: {name}: invalid header length {n} for a file of {size} bytes")
        raw = f.read(n)
        if len(raw) != n:
            raise CheckpointError(f"safetensors: {name}: truncated header")
        try:
            entries = json.loads(raw.decode("utf-8").rstrip(" "))
        except ValueError as e:
            raise CheckpointError(f"safetensors: {name}: cannot parse header: {e}") from e
        if not isinstance(entries, dict):
            raise CheckpointError(f"safetensors: {name}: header is not a JSON object")
        base = 8 + n
        self._maps.append(mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ))
        for tname, e in entries.items():
            if tname == "__metadata__":
                continue
            try:
                dtype, shape, off = e["dtype"], tuple(int(x) for x in e["shape"]), e["data_offsets"]
                lo, hi = int(off[0]), int(off[1])
                if len(off) != 2:
                    raise ValueError
            except (KeyError, TypeError, ValueError, IndexError):
                raise CheckpointError(f"safetensors: {name}: tensor {tname} has a malformed entry") from None
            if lo < 0 or hi < lo or base + hi > size:
                raise CheckpointError(f"safetensors: {name}: tensor {tname} has invalid data offsets "
                                      f"[{lo}, {hi}) for a file of {size} bytes")
            self.tensors[tname] = TensorEntry(tname, dtype, shape, file_index, base + lo, hi - lo)

    def has(self, name: str) -> bool:
        return name in self.tensors

    def names(self) -> List[str]:
        return sorted(self.tensors)

    def read(self, name: str) -> np.ndarray:
        """The tensor as a numpy view (BF16 as uint16 bits).  Raises if dtype or size is off."""
        e = self.tensors[name]
        if e.dtype not in _DTYPES:
            raise CheckpointError(f"safetensors: {name} has unsupported dtype {e.dtype}")
        np_dtype, width = _DTYPES[e.dtype]
        count = 1
        for d in e.shape:
            count *= d
        if e.size != count * width:
            raise CheckpointError(f"safetensors: {name} has dtype {e.dtype} and {e.size} bytes "
                                  f"for shape {list(e.shape)}")
        arr = np.frombuffer(self._maps[e.file_index], dtype=np_dtype, count=count, offset=e.offset)
        return arr.reshape(e.shape)

    def close(self) -> None:
        # numpy views may still reference the maps; they stay valid until garbage collected.
        for m in self._maps:
            try:
                m.close()
            except BufferError:
                pass
        self._maps = []
        for f in self._files:
            f.close()
        self._files = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def float32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, as internal/qwen3lm/lmtest/lmtest.go:136-140 does."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_float32(bits: np.ndarray) -> np.ndarray:
    """Exact widening (bits << 16), as internal/q8gemm/packed.go:178-179 does."""
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def write_safetensors(path: str, tensors: Mapping[str, Tuple[str, Sequence[int], np.ndarray]]) -> None:
    """Write one safetensors file.  ``tensors[name] = (dtype string, shape, array)``; a BF16 array is
    given as uint16 bit patterns.  Names are written in sorted order, the header padded with
    spaces to a multiple of 8 (internal/qwen3lm/lmtest/lmtest.go:106-131)."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        dtype, shape, arr = tensors[name]
        if dtype not in _DTYPES:
            raise CheckpointError(f"safetensors: cannot write dtype {dtype}")
        np_dtype, width = _DTYPES[dtype]
        count = 1
        for d in shape:
            count *= int(d)
        if arr.dtype != np_dtype or arr.size != count:
            raise CheckpointError(f"safetensors: {name}: array {arr.dtype}x{arr.size} does not match "
                                  f"{dtype} {list(shape)}")
        header[name] = {"dtype": dtype, "shape": [int(d) for d in shape],
                        "data_offsets": [offset, offset + count * width]}
        offset += count * width
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((-len(raw)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            f.write(np.ascontiguousarray(tensors[name][2]).tobytes())
