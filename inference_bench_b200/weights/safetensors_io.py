"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the raw little-endian tensor data.

Files are memory-mapped and tensors are handed out by name; a sharded checkpoint is described by
`model.safetensors.index.json` (`weight_map`: name -> file), as the reference reads it
(crates/specrt/src/weights.rs:112-141, 165-201).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

# safetensors dtype -> (numpy dtype of the stored bytes, bytes per element)
_STORED = {
    "F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2),
    "I32": (np.int32, 4), "I64": (np.int64, 8), "U8": (np.uint8, 1), "BOOL": (np.uint8, 1),
}
_TORCH_TO_ST = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32", torch.int64: "I64"}


class CheckpointError(ValueError):
    """A model folder's weight files cannot be read."""


@dataclass(frozen=True)
class StoredTensor:
    file: Path
    dtype: str
    shape: tuple[int, ...]
    begin: int  # absolute byte offsets inside the file
    end: int


class Checkpoint:
    """All tensors of a model folder by name, read lazily from memory maps."""

    def __init__(self, model_dir):
        self.dir = Path(model_dir)
        self.tensors: dict[str, StoredTensor] = {}
        self._maps: dict[Path, mmap.mmap] = {}
        for f in self._files():
            for name, st in _read_header(f).items():
                if name in self.tensors:
                    raise CheckpointError(f"tensor {name} appears in both {self.tensors[name].file.name} and {f.name}")
                self.tensors[name] = st

    def _files(self) -> list[Path]:
        index = self.dir / "model.safetensors.index.json"
        single = self.dir / "model.safetensors"
        if index.is_file():
            try:
                weight_map = json.loads(index.read_text())["weight_map"]
            except (json.JSONDecodeError, KeyError) as e:
                raise CheckpointError(f"{index} has no readable weight_map: {e}") from e
            files = sorted({self.dir / f for f in weight_map.values()})
            for f in files:
                if not f.is_file():
                    raise CheckpointError(f"{index.name} names {f.name}, which does not exist")
            return files
        if single.is_file():
            return [single]
        raise CheckpointError(f"{self.dir} has neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> list[str]:
        return sorted(self.tensors)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored: BF16 -> bfloat16, F32 -> float32, F16 -> float16, integers as stored."""
        st = self.tensors[name]
        mm = self._maps.get(st.file)
        if mm is None:
            with open(st.file, "rb") as fh:
                mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[st.file] = mm
        if st.dtype not in _STORED:
            raise CheckpointError(f"{name} is stored as {st.dtype}, which this engine does not read (no quantized formats)")
        np_dtype, size = _STORED[st.dtype]
        count = int(np.prod(st.shape)) if st.shape else 1
        if st.end - st.begin != count * size:
            raise CheckpointError(f"{name}: {st.end - st.begin} bytes stored, but shape {list(st.shape)} of {st.dtype} needs {count * size}")
        arr = np.frombuffer(mm, dtype=np_dtype, count=count, offset=st.begin).reshape(st.shape)
        t = torch.from_numpy(arr.copy())
        if st.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t

    def close(self) -> None:
        for mm in self._maps.values():
            mm.close()
        self._maps.clear()


def _read_header(path: Path) -> dict[str, StoredTensor]:
    with open(path, "rb") as fh:
        head = fh.read(8)
        if len(head) != 8:
            raise CheckpointError(f"{path} is too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = path.stat().st_size
        if n <= 0 or 8 + n > size:
            raise CheckpointError(f"{path} has a header length of {n} bytes, beyond its size {size}")
        try:
            header = json.loads(fh.read(n))
        except json.JSONDecodeError as e:
            raise CheckpointError(f"{path} has an unreadable header: {e}") from e
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        if not (0 <= lo <= hi and 8 + n + hi <= size):
            raise CheckpointError(f"{path}: tensor {name} has data offsets [{lo}, {hi}) outside the file")
        out[name] = StoredTensor(path, info["dtype"], tuple(int(s) for s in info["shape"]), 8 + n + lo, 8 + n + hi)
    return out


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Write CPU tensors (float32, float16, bfloat16, int32, int64) in name order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise CheckpointError(f"cannot store {name} of dtype {t.dtype}")
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((-len(text)) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for b in blobs:
            fh.write(b)
