"""Reader and writer of the safetensors file format.

The format: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` and the raw
little-endian tensor data.  The reference loads a converted ``model.pth`` with
``torch.load(mmap=True)`` (DELTA/Engine/utils.py:220); a model folder with
safetensors files takes its place here, read by memory map without a copy until
a tensor is sent to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import numpy as np
import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One open file: ``names()``, ``info(name)`` and ``tensor(name)`` (a CPU view)."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{self.path}: too short for a safetensors file")
        (hlen,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} does not fit the file of {size} bytes")
        try:
            self._header = json.loads(self._f.read(hlen).decode("utf-8"))
        except Exception as e:  # noqa: BLE001
            raise SafetensorsError(f"{self.path}: the header is not JSON: {e}") from None
        self._header.pop("__metadata__", None)
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for name, meta in self._header.items():
            if meta["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has the unknown dtype {meta['dtype']}")
            b, e = meta["data_offsets"]
            n = int(np.prod(meta["shape"])) if meta["shape"] else 1
            if e - b != n * torch.empty((), dtype=_DTYPES[meta["dtype"]]).element_size() or self._base + e > size:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has data offsets that do not fit its shape")

    def names(self) -> list[str]:
        return list(self._header)

    def info(self, name: str) -> tuple[tuple, torch.dtype]:
        m = self._header[name]
        return tuple(m["shape"]), _DTYPES[m["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        m = self._header[name]
        b, e = m["data_offsets"]
        dt = _DTYPES[m["dtype"]]
        if e == b:
            return torch.empty(m["shape"], dtype=dt)
        buf = memoryview(self._mm)[self._base + b:self._base + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the buffer is read-only; it is only read
            try:
                t = torch.frombuffer(buf, dtype=dt)
            except (ValueError, RuntimeError):  # data that does not start on a multiple of its element size
                t = torch.frombuffer(bytearray(buf), dtype=dt)
        return t.reshape(m["shape"])

    def close(self):
        # views handed out keep the map alive; it goes away with them
        self._f.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor]) -> None:
    """Writes CPU tensors under their names, in name order, data back to back."""
    header = {}
    offset = 0
    order = sorted(tensors)
    cpu = {}
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which the format does not hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        cpu[name] = t
        offset += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for name in order:
            t = cpu[name]
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))


def open_model_files(folder) -> list[SafetensorsFile]:
    """All safetensors files of a model folder (one ``model.safetensors`` or the
    shards named by ``model.safetensors.index.json``)."""
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [SafetensorsFile(folder / f) for f in files]
    single = folder / "model.safetensors"
    if single.is_file():
        return [SafetensorsFile(single)]
    found = sorted(folder.glob("*.safetensors"))
    if not found:
        raise SafetensorsError(f"no safetensors file in {folder}")
    return [SafetensorsFile(p) for p in found]
