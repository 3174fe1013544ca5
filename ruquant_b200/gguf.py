"""GGUF v3 files holding W4A4 / W4A4H tensors: the container the reference's converter writes and its runtime loads.

Mirrors the reader of the reference's host side (src/gguf.rs:8-39 type table, 113-160 header walk): little-endian,
magic "GGUF", version 3 only, n_tensors and n_kv as u64, metadata values skipped by type, tensor infos (name, dims with
ne0 first, ggml type, offset relative to the data section), data section starting at the header's end rounded up to
`general.alignment` (32 when absent).  Types 44 / 45 are rows of 144-byte blocks of 256 codes, like Q4_K's geometry.

`Gguf.open(path)` maps the file; `weight(name)` puts one W4A4 / W4A4H tensor on the GPU, prepared for the kernels.
`write` is the small writer the tests and tools use to make such files (scalar and string metadata only).
"""
import mmap
import struct

import numpy as np

W4A4, W4A4H = 44, 45
F32, F16, BF16 = 0, 1, 30

# ggml type -> (elements per block, bytes per block), the types a converted model may contain (src/gguf.rs:16-39)
TYPE_LAYOUT = {
    0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 10: (256, 84), 11: (256, 110),
    12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292), 24: (1, 1), 25: (1, 2), 26: (1, 4), 30: (1, 2),
    44: (256, 144), 45: (256, 144),
}

# metadata value types: id -> struct format (fixed-size scalars)
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


class GgufError(ValueError):
    pass


class TensorInfo:
    def __init__(self, name, dims, ggml_type, offset):
        self.name, self.dims, self.type, self.offset = name, tuple(dims), ggml_type, offset

    @property
    def n_elements(self):
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def n_bytes(self):
        if self.type not in TYPE_LAYOUT:
            raise GgufError("%s: unsupported ggml type %d" % (self.name, self.type))
        blk, size = TYPE_LAYOUT[self.type]
        return self.n_elements // blk * size


class _Cursor:
    def __init__(self, buf):
        self.b, self.p = buf, 0

    def take(self, n):
        if self.p + n > len(self.b):
            raise GgufError("truncated GGUF header")
        v = self.b[self.p:self.p + n]
        self.p += n
        return v

    def unpack(self, fmt):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self):
        return bytes(self.take(self.unpack("<Q"))).decode("utf-8", "replace")

    def value(self, ty):
        """Parses scalars and strings; walks over arrays (returned as None)."""
        if ty in _SCALARS:
            return self.unpack(_SCALARS[ty])
        if ty == _STRING:
            return self.string()
        if ty == _ARRAY:
            et, n = self.unpack("<I"), self.unpack("<Q")
            for _ in range(n):
                self.value(et)
            return None
        raise GgufError("unknown GGUF value type %d" % ty)


class Gguf:
    def __init__(self, buf, path="<memory>"):
        c = _Cursor(buf)
        if bytes(c.take(4)) != b"GGUF":
            raise GgufError("%s: not a GGUF file" % path)
        version = c.unpack("<I")
        if version != 3:
            raise GgufError("%s: GGUF version %d, only 3 is supported" % (path, version))
        n_tensors, n_kv = c.unpack("<Q"), c.unpack("<Q")
        self.kv = {}
        for _ in range(n_kv):
            key = c.string()
            self.kv[key] = c.value(c.unpack("<I"))
        self.tensors = []
        for _ in range(n_tensors):
            name = c.string()
            nd = c.unpack("<I")
            dims = [c.unpack("<Q") for _ in range(nd)]
            ty, off = c.unpack("<I"), c.unpack("<Q")
            self.tensors.append(TensorInfo(name, dims, ty, off))
        align = self.alignment
        self.data_start = (c.p + align - 1) // align * align
        self.buf = buf
        self._by_name = {t.name: t for t in self.tensors}

    @classmethod
    def open(cls, path):
        with open(path, "rb") as f:
            m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return cls(memoryview(m), path)

    @property
    def alignment(self):
        a = self.kv.get("general.alignment")
        return int(a) if isinstance(a, int) and a > 0 else 32

    def info(self, name):
        if name not in self._by_name:
            raise KeyError(name)
        return self._by_name[name]

    def data(self, name):
        """The tensor's bytes as a read-only uint8 array over the mapped file."""
        t = self.info(name)
        start = self.data_start + t.offset
        if start + t.n_bytes > len(self.buf):
            raise GgufError("%s: data beyond the end of the file" % name)
        return np.frombuffer(self.buf, dtype=np.uint8, count=t.n_bytes, offset=start)

    def w4a4_tensors(self):
        """(name, type, K, N) of every 2-D W4A4 / W4A4H tensor: dims are (ne0 = K inputs, ne1 = N rows)."""
        return [(t.name, t.type, t.dims[0], t.dims[1]) for t in self.tensors if t.type in (W4A4, W4A4H) and len(t.dims) == 2]

    def weight(self, name, device="cuda", layouts=None):
        """Copies one W4A4 / W4A4H tensor to the GPU and prepares it (ruquant_b200.Weight)."""
        import torch
        import ruquant_b200 as rq
        t = self.info(name)
        if t.type not in (W4A4, W4A4H) or len(t.dims) != 2:
            raise GgufError("%s: not a 2-D W4A4 / W4A4H tensor" % name)
        blocks = torch.from_numpy(np.array(self.data(name))).to(device)
        return rq.Weight(blocks, t.type, t.dims[0], N=t.dims[1], layouts=rq.PREPACK_ALL if layouts is None else layouts)


def _kv_bytes(key, value):
    out = struct.pack("<Q", len(key.encode())) + key.encode()
    if isinstance(value, bool):
        return out + struct.pack("<I?", 7, value)
    if isinstance(value, int):
        return out + (struct.pack("<II", 4, value) if 0 <= value < 2 ** 32 else struct.pack("<Iq", 11, value))
    if isinstance(value, float):
        return out + struct.pack("<If", 6, value)
    if isinstance(value, str):
        v = value.encode()
        return out + struct.pack("<IQ", _STRING, len(v)) + v
    raise TypeError("metadata value of %s: only bool, int, float and str are written" % key)


def write(path, metadata, tensors, version=3):
    """metadata: {key: bool | int | float | str}; tensors: [(name, dims with ne0 first, ggml type, bytes-like)]."""
    align = int(metadata.get("general.alignment", 32))
    head = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(metadata))
    for k, v in metadata.items():
        head += _kv_bytes(k, v)
    offsets, off = [], 0
    for name, dims, ty, data in tensors:
        blk, size = TYPE_LAYOUT[ty]
        n = 1
        for d in dims:
            n *= d
        if len(memoryview(data).cast("B")) != n // blk * size:
            raise ValueError("%s: %d bytes given, %d expected" % (name, len(memoryview(data).cast("B")), n // blk * size))
        offsets.append(off)
        off = (off + n // blk * size + align - 1) // align * align
    for (name, dims, ty, _data), o in zip(tensors, offsets):
        head += struct.pack("<Q", len(name.encode())) + name.encode() + struct.pack("<I", len(dims))
        head += b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, o)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((len(head) + align - 1) // align * align - len(head)))
        pos = 0
        for (_name, _dims, _ty, data), o in zip(tensors, offsets):
            f.write(b"\0" * (o - pos))
            raw = memoryview(data).cast("B")
            f.write(raw)
            pos = o + len(raw)
