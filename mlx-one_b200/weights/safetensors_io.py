"""Reading and writing safetensors files without a framework around them.

Format: 8 bytes little-endian header length, a JSON header that maps each tensor name to
{"dtype", "shape", "data_offsets"}, then the raw little-endian data. Files are mapped,
not read, so a tensor costs host memory only while it is copied to the device.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path
from typing import Iterator, Mapping

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {value: key for key, value in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors file."""


class SafetensorsFile:
    """A mapped safetensors file. ``entries`` maps names to (dtype, shape)."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._file = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
        (length,) = struct.unpack("<Q", self._file.read(8))
        if length <= 0 or 8 + length > size:
            raise SafetensorsError(f"{self.path}: header length {length} exceeds the file")
        try:
            header = json.loads(self._file.read(length))
        except ValueError as exc:
            raise SafetensorsError(f"{self.path}: header is not JSON: {exc}") from exc
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + length
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        self._header = header
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...]]] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: {name} has unsupported dtype {info['dtype']}")
            dtype, shape = _DTYPES[info["dtype"]], tuple(int(v) for v in info["shape"])
            begin, end = info["data_offsets"]
            count = 1
            for extent in shape:
                count *= extent
            if not (isinstance(begin, int) and isinstance(end, int) and 0 <= begin <= end
                    and end - begin == count * dtype.itemsize
                    and self._data_start + end <= size):
                raise SafetensorsError(f"{self.path}: {name} has inconsistent offsets")
            self.entries[name] = (dtype, shape)
        # the format wants the tensors' byte ranges side by side: none may share bytes
        ranges = sorted((info["data_offsets"][0], info["data_offsets"][1], name)
                        for name, info in header.items())
        for (_, before_end, before), (begin, _, name) in zip(ranges, ranges[1:]):
            if begin < before_end:
                raise SafetensorsError(f"{self.path}: {name} overlaps {before}")

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor that views the mapped file (copy it before the file closes)."""
        dtype, shape = self.entries[name]
        begin, end = self._header[name]["data_offsets"]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the map is read-only; so is its use
            return torch.frombuffer(view, dtype=dtype).reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        except BufferError:
            pass        # a tensor still views the map; the map goes with it
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def checkpoint_index(model_dir: str | Path) -> dict[str, str] | None:
    """``weight_map`` of ``model.safetensors.index.json`` (tensor name -> file name), or None
    if the folder has no index."""
    index = Path(model_dir) / "model.safetensors.index.json"
    if not index.is_file():
        return None
    try:
        value = json.loads(index.read_text()).get("weight_map")
    except (ValueError, AttributeError) as error:
        raise SafetensorsError(f"{index}: not a JSON object ({error})") from error
    if not isinstance(value, dict) or not value:
        raise SafetensorsError(f"{index}: a non-empty weight_map is required")
    if any(not isinstance(name, str) or not isinstance(file, str) for name, file in value.items()):
        raise SafetensorsError(f"{index}: weight_map must map tensor names to file names")
    return value


def checkpoint_files(model_dir: str | Path) -> list[Path]:
    """The safetensors files of a model folder, by the reference's rules
    (src/mlx_one/text/loading.py:571-610): one file, or the shards that
    ``model.safetensors.index.json`` names; several files without an index are refused, so are
    shards that are missing, lie outside the folder (also through a symbolic link) or are no
    safetensors files, and folders that hold pickle checkpoints only."""
    root = Path(model_dir)
    files = sorted(root.glob("*.safetensors"))
    if not files:
        pickled = list(root.glob("*.bin")) + list(root.glob("*.pt"))
        detail = "; pickle checkpoints (.bin, .pt) are not accepted" if pickled else ""
        raise FileNotFoundError(f"no safetensors file in {root}{detail}")
    weight_map = checkpoint_index(root)
    if weight_map is not None:
        files = sorted({root / name for name in weight_map.values()})
        for path in files:
            if path.parent != root or not path.is_file():
                raise FileNotFoundError(f"{path} is named by the index but is no file of {root}")
    elif len(files) != 1:
        raise SafetensorsError(f"{root} holds {len(files)} safetensors files and no index")
    inside = root.resolve()
    for path in files:
        if path.suffix != ".safetensors" or path.resolve().parent != inside:
            raise SafetensorsError(f"{path} is no safetensors file inside {root}")
    return files


def write_safetensors(path: str | Path, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> None:
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"{name}: dtype {tensor.dtype} cannot be stored")
        size = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(8 + len(blob)) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(blob)))
        out.write(blob)
        for name in order:
            tensor = tensors[name].detach().cpu().contiguous()
            out.write(tensor.view(torch.uint8).numpy().tobytes() if tensor.numel() else b"")
