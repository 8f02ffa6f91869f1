"""Safetensors ingestion (vyre-safetensors/src/lib.rs:108-260, 871-907): header validation rules and the shard identity,
on files written here byte by byte (8-byte little-endian header length, JSON header, payload). CPU only."""
import hashlib
import json
import struct

import numpy as np
import pytest

import vyre_b200 as vb
from vyre_b200 import api, ffi


def write_shard(path, header: dict | bytes, payload: bytes = b""):
    raw = header if isinstance(header, bytes) else json.dumps(header, separators=(",", ":")).encode()
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(raw)) + raw + payload)
    return raw


def test_open_lists_tensors_in_name_order_with_absolute_ranges_and_identity(tmp_path):
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.arange(8, dtype=np.uint8)
    c = np.array([1.5, -2.0], dtype=np.float16)
    header = {
        "zeta.weight": {"dtype": "F32", "shape": [3, 4], "data_offsets": [8, 56]},
        "__metadata__": {"format": "pt", "nested": {"k": [1, 2, {"x": "y"}]}},
        "alpha": {"dtype": "U8", "shape": [8], "data_offsets": [0, 8]},
        "mid/f16": {"dtype": "F16", "shape": [2], "data_offsets": [56, 60]},
        "empty": {"dtype": "BF16", "shape": [0, 7], "data_offsets": [60, 60]},
    }
    p = tmp_path / "m.safetensors"
    raw = write_shard(p, header, b.tobytes() + a.tobytes() + c.tobytes())
    idx = api.SafetensorIndex.open(str(p))
    got = idx.tensors()
    assert [t["name"] for t in got] == ["alpha", "empty", "mid/f16", "zeta.weight"]
    start = 8 + len(raw)
    assert idx.tensor("zeta.weight") == {"name": "zeta.weight", "dtype": "F32", "shape": [3, 4], "file_range": (start + 8, start + 56), "index": 3}
    assert idx.tensor("empty")["file_range"] == (start + 60, start + 60)
    ident = idx.identity()
    assert ident["file_len"] == start + 60 and ident["data_start"] == start and len(ident["header_digest"]) == 32
    # the digest is BLAKE3 of the exact header bytes: a header that differs in one byte of whitespace has another identity
    p2 = tmp_path / "m2.safetensors"
    write_shard(p2, raw.replace(b'"alpha":', b'"alpha": '), b.tobytes() + a.tobytes() + c.tobytes())
    assert api.SafetensorIndex.open(str(p2)).identity()["header_digest"] != ident["header_digest"]
    assert api.SafetensorIndex.open(str(p)).identity()["header_digest"] == ident["header_digest"]
    # requirements (lib.rs:262-271)
    assert idx.require("zeta.weight", "F32", [3, 4])["index"] == 3
    for bad in [("zeta.weight", "F16", [3, 4]), ("zeta.weight", "F32", [4, 3]), ("zeta.weight", "F32", [12]), ("nope", "F32", [1])]:
        with pytest.raises(vb.BackendError) as e:
            idx.require(*bad)
        assert e.value.code == ffi.ERR_INVALID_PROGRAM and "Fix:" in str(e.value)


@pytest.mark.parametrize("name,make", [
    ("prefix", lambda: (b"\x01\x02\x03", None)),
    ("header longer than the file", lambda: (struct.pack("<Q", 100) + b"{}", None)),
    ("header above the limit", lambda: (struct.pack("<Q", 64 * 1024 * 1024 + 1) + b"{}", None)),
    ("not json", lambda: ({"raw": b"{nope}"}, b"")),
    ("trailing characters", lambda: ({"raw": b'{} x'}, b"")),
    ("duplicate name", lambda: ({"raw": b'{"a":{"dtype":"U8","shape":[1],"data_offsets":[0,1]},"a":{"dtype":"U8","shape":[1],"data_offsets":[1,2]}}'}, b"\0\0")),
    ("unknown dtype", lambda: ({"a": {"dtype": "U128", "shape": [1], "data_offsets": [0, 1]}}, b"\0")),
    ("missing field", lambda: ({"a": {"dtype": "U8", "shape": [1]}}, b"\0")),
    ("negative extent", lambda: ({"raw": b'{"a":{"dtype":"U8","shape":[-1],"data_offsets":[0,1]}}'}, b"\0")),
    ("range past the payload", lambda: ({"a": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]}}, b"\0\0")),
    ("start after end", lambda: ({"a": {"dtype": "U8", "shape": [0], "data_offsets": [2, 1]}}, b"\0\0")),
    ("byte length", lambda: ({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)),
    ("shape overflow", lambda: ({"a": {"dtype": "F64", "shape": [2**40, 2**40], "data_offsets": [0, 0]}}, b"")),
    ("overlap", lambda: ({"a": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]}, "b": {"dtype": "U8", "shape": [4], "data_offsets": [2, 6]}}, b"\0" * 6)),
    ("empty name", lambda: ({"": {"dtype": "U8", "shape": [1], "data_offsets": [0, 1]}}, b"\0")),
    ("long name", lambda: ({"n" * 4097: {"dtype": "U8", "shape": [1], "data_offsets": [0, 1]}}, b"\0")),
])
def test_invalid_shards_are_refused_with_a_fix(tmp_path, name, make):
    header, payload = make()
    p = tmp_path / "bad.safetensors"
    if payload is None:
        p.write_bytes(header)
    else:
        write_shard(p, header["raw"] if "raw" in header else header, payload)
    with pytest.raises(vb.BackendError) as e:
        api.SafetensorIndex.open(str(p))
    assert e.value.code == ffi.ERR_INVALID_PROGRAM and "Fix:" in str(e.value), name


def test_missing_file_and_adjacent_ranges(tmp_path):
    with pytest.raises(vb.BackendError, match="could not access"):
        api.SafetensorIndex.open(str(tmp_path / "absent.safetensors"))
    # ranges that touch are not an overlap; a long name of exactly 4096 bytes is accepted
    p = tmp_path / "ok.safetensors"
    write_shard(p, {"a": {"dtype": "I8", "shape": [2], "data_offsets": [0, 2]}, "n" * 4096: {"dtype": "I8", "shape": [2], "data_offsets": [2, 4]}},
                b"\1\2\3\4")
    assert len(api.SafetensorIndex.open(str(p)).tensors()) == 2


def test_reference_ingestion_fixtures(tmp_path):
    """vyre-safetensors/tests/ingestion.rs:49-161: the single-shard fixtures of the reference's own test, byte for byte."""
    header = (b'{"model.embed_tokens.weight":{"dtype":"BF16","shape":[2,2],"data_offsets":[0,8]},'
              b'"model.norm.weight":{"dtype":"BF16","shape":[2],"data_offsets":[8,12]}}')
    p = tmp_path / "model.safetensors"
    write_shard(p, header, bytes(12))
    idx = api.SafetensorIndex.open(str(p))  # :49-72 valid_bf16_tensors_have_exact_ranges_and_identity
    assert len(idx.tensors()) == 2
    emb = idx.tensor("model.embed_tokens.weight")
    assert emb["dtype"] == "BF16" and emb["shape"] == [2, 2] and emb["file_range"] == (8 + len(header), 16 + len(header))
    ident = idx.identity()
    assert ident["file_len"] == 8 + len(header) + 12 and ident["header_digest"] == vb.blake3(header)

    def refused(name, raw, payload, *needles):
        q = tmp_path / name
        if payload is None:
            q.write_bytes(raw)
        else:
            write_shard(q, raw, payload)
        with pytest.raises(vb.BackendError) as e:
            api.SafetensorIndex.open(str(q))
        for needle in needles:
            assert needle in str(e.value), (name, str(e.value))

    # :75-88 HeaderTooLarge { header_len: 64 MiB + 1, maximum: 64 MiB }
    refused("oversized.safetensors", struct.pack("<Q", 64 * 1024 * 1024 + 1), None, str(64 * 1024 * 1024 + 1), str(64 * 1024 * 1024))
    # :91-106 RangeOutOfBounds { name: weight, start: 0, end: 16, data_len: 12 }
    refused("truncated.safetensors", b'{"weight":{"dtype":"F32","shape":[4],"data_offsets":[0,16]}}', bytes(12), "weight", "16", "12")
    # :109-122 Overlap { left: a, right: b }
    refused("overlap.safetensors", b'{"a":{"dtype":"U8","shape":[8],"data_offsets":[0,8]},"b":{"dtype":"U8","shape":[8],"data_offsets":[4,12]}}',
            bytes(12), "`a`", "`b`")
    # :125-134 duplicate tensor name `weight`
    refused("duplicate.safetensors",
            b'{"weight":{"dtype":"U8","shape":[1],"data_offsets":[0,1]},"weight":{"dtype":"U8","shape":[1],"data_offsets":[1,2]}}', bytes(2),
            "duplicate tensor name `weight`")
    # :137-151 ByteLength { name: weight, actual: 6, expected: 8 }
    refused("wrong-length.safetensors", b'{"weight":{"dtype":"BF16","shape":[2,2],"data_offsets":[0,6]}}', bytes(6), "weight", "6", "8")
    # :154-161 malformed metadata
    refused("malformed.safetensors", b'{"weight": ', b"")
