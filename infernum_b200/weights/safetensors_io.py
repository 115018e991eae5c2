"""Reader and writer for the safetensors container.

Layout of a file: an unsigned 64-bit little-endian header length ``n``, ``n``
bytes of JSON mapping each tensor name to ``{"dtype", "shape",
"data_offsets": [begin, end]}`` (offsets relative to the end of the header),
then the raw little-endian tensor bytes.  The reference maps every
``*.safetensors`` file of a folder, sorted by name, into one name table
(infernum/src/weights/safetensors.rs:55-120); ``open_model_folder`` does the
same.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Sequence, Tuple

import torch

from ..errors import WeightError

_DTYPES = {
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int  # absolute byte offset in the file
    end: int
    file: "SafetensorsFile"

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    """One memory-mapped file and its table of tensors."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise WeightError(f"{path}: truncated (no header length)")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise WeightError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightError(f"{path}: header is not valid JSON: {exc}") from exc
        self.metadata = header.pop("__metadata__", {}) or {}
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            dtype_name = info.get("dtype")
            if dtype_name not in _DTYPES:
                raise WeightError(f"{path}: tensor {name!r} has unsupported dtype {dtype_name!r}")
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            entry = TensorEntry(name, _DTYPES[dtype_name], shape, base + begin, base + end, self)
            want = entry.numel() * torch.empty((), dtype=entry.dtype).element_size()
            if end - begin != want:
                raise WeightError(
                    f"{path}: tensor {name!r} spans {end - begin} bytes, its shape needs {want}"
                )
            if base + end > size:
                raise WeightError(f"{path}: tensor {name!r} reaches past the end of the file")
            self.entries[name] = entry

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only memory: clone or
        copy to the device before writing to it)."""
        e = self.entries[name]
        if e.numel() == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(self._map, dtype=e.dtype, count=e.numel(), offset=e.begin)
        return flat.view(e.shape)

    def close(self) -> None:
        # Tensors returned by read() keep the map alive through the buffer
        # protocol; closing is only attempted, never forced.
        try:
            if self._map is not None:
                self._map.close()
        except BufferError:
            pass
        self._fh.close()


def open_model_folder(folder: str) -> Dict[str, TensorEntry]:
    """Name table over every ``*.safetensors`` file of a folder, in sorted
    order; a name that appears twice keeps its last occurrence."""
    if os.path.isfile(folder):
        files = [folder]
    else:
        files = sorted(
            os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".safetensors")
        )
    if not files:
        raise WeightError(f"no .safetensors file in {folder}")
    table: Dict[str, TensorEntry] = {}
    for path in files:
        table.update(SafetensorsFile(path).entries)
    return table


def write_safetensors(
    path: str,
    specs: Sequence[Tuple[str, torch.dtype, Sequence[int]]],
    produce: Callable[[str], torch.Tensor],
    metadata: Dict[str, str] | None = None,
) -> None:
    """Write tensors one at a time: ``specs`` fixes names, dtypes and shapes
    (so the header can be written first) and ``produce(name)`` makes each
    tensor when its turn comes, which keeps a large model out of host memory."""
    header: Dict[str, dict] = {}
    offset = 0
    for name, dtype, shape in specs:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        header[name] = {
            "dtype": _NAMES[dtype],
            "shape": [int(s) for s in shape],
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, dtype, shape in specs:
            t = produce(name)
            if t.dtype != dtype or tuple(t.shape) != tuple(int(s) for s in shape):
                raise WeightError(
                    f"writer: tensor {name!r} came as {t.dtype} {tuple(t.shape)}, "
                    f"declared {dtype} {tuple(shape)}"
                )
            t = t.detach().contiguous().cpu()
            if t.numel():
                fh.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)


def save_tensors(path: str, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    specs = [(k, v.dtype, tuple(v.shape)) for k, v in tensors.items()]
    write_safetensors(path, specs, lambda name: tensors[name], metadata)


def tensor_names(entries: Iterable[TensorEntry]) -> List[str]:
    return [e.name for e in entries]
