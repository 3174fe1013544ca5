"""GGUF v3 container for W4A4 / W4A4H tensors (host side, no GPU): layout rules of the reference's reader
(src/gguf.rs:8-39, 113-160) -- magic, version, alignment of the data section, type table, tensor offsets."""
import struct

import numpy as np
import pytest

from ruquant_b200 import gguf
from tests import inputs


def make_file(tmp_path, port, align=None, version=3):
    K, N = 1024, 8
    wf = inputs.normal_weights(N, K, 9100)
    w44 = port.quantize_weights(wf, 44)
    w45 = port.quantize_weights(wf, 45)
    norm = np.arange(K, dtype=np.float32)
    meta = {"general.architecture": "qwen3", "general.name": "tiny", "ruquant.act_group": 64, "ruquant.clip": 0.9,
            "flag": True}
    if align:
        meta["general.alignment"] = align
    path = str(tmp_path / "t.gguf")
    gguf.write(path, meta, [("blk.0.attn_norm.weight", (K,), gguf.F32, norm), ("blk.0.attn_q.weight", (K, N), gguf.W4A4, w44),
                            ("blk.0.ffn_down.weight", (K, N), gguf.W4A4H, w45)], version=version)
    return path, norm, w44, w45, K, N


@pytest.mark.parametrize("align", [None, 64, 4096])
def test_round_trip_and_alignment(tmp_path, port, align):
    path, norm, w44, w45, K, N = make_file(tmp_path, port, align)
    g = gguf.Gguf.open(path)
    a = align or 32
    assert g.alignment == a and g.data_start % a == 0
    assert g.kv["general.architecture"] == "qwen3" and g.kv["ruquant.act_group"] == 64 and g.kv["flag"] is True
    assert abs(g.kv["ruquant.clip"] - 0.9) < 1e-6
    assert [t.name for t in g.tensors] == ["blk.0.attn_norm.weight", "blk.0.attn_q.weight", "blk.0.ffn_down.weight"]
    assert all(t.offset % a == 0 for t in g.tensors)
    assert g.info("blk.0.attn_q.weight").n_bytes == N * (K // 256) * 144
    assert (g.data("blk.0.attn_norm.weight").view(np.float32) == norm).all()
    assert (g.data("blk.0.attn_q.weight") == w44.reshape(-1)).all()
    assert (g.data("blk.0.ffn_down.weight") == w45.reshape(-1)).all()
    assert g.w4a4_tensors() == [("blk.0.attn_q.weight", 44, K, N), ("blk.0.ffn_down.weight", 45, K, N)]


def test_rejections(tmp_path, port):
    path, *_ = make_file(tmp_path, port, version=2)
    with pytest.raises(gguf.GgufError, match="version 2"):
        gguf.Gguf.open(path)
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(gguf.GgufError, match="not a GGUF file"):
        gguf.Gguf.open(str(bad))
    # a tensor of a type outside the table: sized lazily, like the reference (error names the tensor and the type)
    head = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + struct.pack("<Q", 1) + b"x" + struct.pack("<IQIQ", 1, 256, 99, 0)
    odd = tmp_path / "odd.gguf"
    odd.write_bytes(head + b"\0" * 64)
    g = gguf.Gguf.open(str(odd))
    with pytest.raises(gguf.GgufError, match="unsupported ggml type 99"):
        g.info("x").n_bytes
    trunc = tmp_path / "trunc.gguf"
    trunc.write_bytes(open(path, "rb").read()[:40].replace(b"\x02\0\0\0", b"\x03\0\0\0", 1))
    with pytest.raises(gguf.GgufError, match="truncated"):
        gguf.Gguf.open(str(trunc))


def test_array_metadata_is_skipped(tmp_path):
    # key "tokens" = array of 3 strings, then a u32: the walk must land on the next key
    def s(x):
        return struct.pack("<Q", len(x)) + x
    head = b"GGUF" + struct.pack("<IQQ", 3, 0, 2)
    head += s(b"tokens") + struct.pack("<IIQ", 9, 8, 3) + s(b"a") + s(b"bc") + s(b"def")
    head += s(b"n") + struct.pack("<II", 4, 7)
    p = tmp_path / "arr.gguf"
    p.write_bytes(head)
    g = gguf.Gguf.open(str(p))
    assert g.kv["tokens"] is None and g.kv["n"] == 7 and g.tensors == []
