"""Header-first safetensors reader/writer with hard limits.

A safetensors file is an 8-byte little-endian header length, a JSON header
``{name: {dtype, shape, data_offsets}, "__metadata__": {...}}`` and the raw payload.
The reader parses only the header, validates every entry against limits before any
payload byte is touched, and serves bounded range reads (a row range of one tensor),
which is what a sharded loader needs.  Parity: engine/crates/model/src/safetensors.rs:14-140,
231-259, 398-479 (Limits, Header::read, TensorFile::read_range, Index::parse).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1), "F8_E5M2": (torch.float8_e5m2, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class Limits:
    header_bytes: int = 256 << 20
    tensors: int = 2_000_000
    rank: int = 8
    shards: int = 4096
    name_bytes: int = 1024


NATIVE_READ_BYTES = 4 << 20      # ranges at least this large go through the native reader threads
READER_THREADS = 4


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    begin: int
    end: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]

    @property
    def itemsize(self) -> int:
        return _DTYPES[self.dtype][1]

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class Header:
    """Parsed and validated header of one file."""

    def __init__(self, tensors: dict, metadata: dict, data_start: int, file_size: int):
        self.tensors = tensors
        self.metadata = metadata
        self.data_start = data_start
        self.file_size = file_size

    @staticmethod
    def read(path: str, limits: Limits = Limits()) -> "Header":
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            raw = f.read(8)
            if len(raw) != 8:
                raise SafetensorsError(f"{path}: shorter than its length field")
            (hlen,) = struct.unpack("<Q", raw)
            if hlen > limits.header_bytes or 8 + hlen > size:
                raise SafetensorsError(f"{path}: header of {hlen} bytes exceeds the limit or the file")
            try:
                obj = json.loads(f.read(hlen))
            except (ValueError, UnicodeDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        if not isinstance(obj, dict):
            raise SafetensorsError(f"{path}: header is not an object")
        meta = obj.pop("__metadata__", {}) or {}
        if len(obj) > limits.tensors:
            raise SafetensorsError(f"{path}: {len(obj)} tensors exceed the limit")
        payload = size - 8 - hlen
        tensors = {}
        spans = []
        for name, ent in obj.items():
            if len(name.encode()) > limits.name_bytes:
                raise SafetensorsError(f"{path}: tensor name too long")
            try:
                dtype, shape, (b, e) = ent["dtype"], tuple(int(s) for s in ent["shape"]), ent["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: {name}: unsupported dtype {dtype}")
            if len(shape) > limits.rank or any(s < 0 for s in shape):
                raise SafetensorsError(f"{path}: {name}: bad shape {shape}")
            info = TensorInfo(name, dtype, shape, int(b), int(e))
            if info.begin < 0 or info.end < info.begin or info.end > payload:
                raise SafetensorsError(f"{path}: {name}: offsets outside the payload")
            if info.end - info.begin != info.numel * info.itemsize:
                raise SafetensorsError(f"{path}: {name}: byte length does not match shape")
            tensors[name] = info
            spans.append((info.begin, info.end))
        spans.sort()
        for (_, e0), (b1, _) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: overlapping tensors")
        return Header(tensors, meta, 8 + hlen, size)


class TensorFile:
    """One open shard; reads whole tensors or leading-dimension row ranges."""

    def __init__(self, path: str, limits: Limits = Limits()):
        self.path = path
        self.header = Header.read(path, limits)
        self._f = open(path, "rb")

    def close(self) -> None:
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def names(self):
        return self.header.tensors.keys()

    def info(self, name: str) -> TensorInfo:
        try:
            return self.header.tensors[name]
        except KeyError:
            raise SafetensorsError(f"{self.path}: no tensor {name!r}") from None

    def read_range(self, name: str, row0: int = 0, row1: int | None = None) -> torch.Tensor:
        """Rows [row0, row1) of the leading dimension (the whole tensor by default)."""
        info = self.info(name)
        if not info.shape:
            row0, row1, rows, row_bytes = 0, 1, 1, info.itemsize
            shape = ()
        else:
            rows = info.shape[0]
            row1 = rows if row1 is None else row1
            if not (0 <= row0 <= row1 <= rows):
                raise SafetensorsError(f"{name}: rows [{row0},{row1}) outside 0..{rows}")
            row_bytes = (info.numel // rows if rows else 0) * info.itemsize
            shape = (row1 - row0,) + info.shape[1:]
        nbytes = (row1 - row0) * row_bytes
        start = self.header.data_start + info.begin + row0 * row_bytes
        if nbytes >= NATIVE_READ_BYTES:
            from ..utils.native import host
            m = host()
            if m is not None:
                # reader threads fill a (pinned, when a GPU is present) staging tensor; no other host copy is made
                flat = torch.empty(nbytes, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
                try:
                    m.read_ranges(self.path, [start], [nbytes], [flat.data_ptr()], READER_THREADS, True)
                except RuntimeError as e:
                    raise SafetensorsError(f"{self.path}: {e}") from None
                return flat.view(info.torch_dtype).reshape(shape)
        self._f.seek(start)
        buf = bytearray(nbytes)
        got = self._f.readinto(buf)
        if got != nbytes:
            raise SafetensorsError(f"{self.path}: short read of {name}")
        flat = torch.frombuffer(buf, dtype=torch.uint8) if nbytes else torch.empty(0, dtype=torch.uint8)
        return flat.view(info.torch_dtype).reshape(shape)

    def read(self, name: str) -> torch.Tensor:
        return self.read_range(name)


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    """Write one safetensors file (tensors sorted by name, 8-byte aligned header)."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)


class Index:
    """``model.safetensors.index.json``: tensor name -> shard file."""

    def __init__(self, root: str, weight_map: dict, limits: Limits = Limits()):
        self.root = root
        self.weight_map = weight_map
        shards = sorted(set(weight_map.values()))
        if len(shards) > limits.shards:
            raise SafetensorsError("too many shards")
        for s in shards:
            if "/" in s or "\\" in s or s.startswith("."):
                raise SafetensorsError(f"shard name {s!r} leaves the checkpoint directory")
        self.shards = shards
        self._open: dict = {}
        self.limits = limits

    @staticmethod
    def parse(root: str, limits: Limits = Limits()) -> "Index":
        idx = os.path.join(root, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx, "rb") as f:
                obj = json.loads(f.read())
            wm = obj.get("weight_map")
            if not isinstance(wm, dict) or not all(isinstance(v, str) for v in wm.values()):
                raise SafetensorsError("index has no weight_map")
            return Index(root, dict(wm), limits)
        single = os.path.join(root, "model.safetensors")
        if os.path.exists(single):
            hdr = Header.read(single, limits)
            return Index(root, {n: "model.safetensors" for n in hdr.tensors}, limits)
        raise SafetensorsError(f"{root}: neither an index nor model.safetensors")

    def file(self, shard: str) -> TensorFile:
        if shard not in self._open:
            self._open[shard] = TensorFile(os.path.join(self.root, shard), self.limits)
        return self._open[shard]

    def names(self):
        return self.weight_map.keys()

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def info(self, name: str) -> TensorInfo:
        if name not in self.weight_map:
            raise SafetensorsError(f"checkpoint has no tensor {name!r}")
        return self.file(self.weight_map[name]).info(name)

    def read(self, name: str, row0: int = 0, row1: int | None = None) -> torch.Tensor:
        if name not in self.weight_map:
            raise SafetensorsError(f"checkpoint has no tensor {name!r}")
        return self.file(self.weight_map[name]).read_range(name, row0, row1)

    def inspect_shards(self) -> None:
        """Every tensor of the map must exist in its shard (header-only pass)."""
        for name, shard in self.weight_map.items():
            self.file(shard).info(name)

    def close(self) -> None:
        for f in self._open.values():
            f.close()
        self._open.clear()


def write_sharded(tensors: dict, root: str, max_shard_bytes: int = 4 << 30, metadata: dict | None = None) -> dict:
    """Split ``tensors`` into shards by size, write them and the index; returns the weight map."""
    os.makedirs(root, exist_ok=True)
    groups, cur, cur_bytes = [], {}, 0
    for name in sorted(tensors):
        nb = tensors[name].numel() * tensors[name].element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            groups.append(cur)
            cur, cur_bytes = {}, 0
        cur[name] = tensors[name]
        cur_bytes += nb
    if cur:
        groups.append(cur)
    wm = {}
    total = 0
    for i, g in enumerate(groups):
        fname = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
        save_file(g, os.path.join(root, fname), metadata)
        for n, t in g.items():
            wm[n] = fname
            total += t.numel() * t.element_size()
    with open(os.path.join(root, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": wm}, f, indent=1, sort_keys=True)
    return wm
