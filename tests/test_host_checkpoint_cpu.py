"""The safetensors container of the host mirror, checked without a GPU against the layout
the reference writes (autograd/safetensors.go:30-98) and the rules its reader enforces
(autograd/safetensors_stream.go:28-96)."""
import json
import struct

import numpy as np
import pytest

from gograd_b200 import autograd as ag


def go_header(entries, metadata):
    """What Go's json.Marshal(map[string]any{...}) produces: keys sorted, struct fields in
    declaration order (dtype, shape, data_offsets), no spaces, <>& escaped."""
    items, offset = {}, 0
    for name in sorted(entries):
        a = entries[name]
        end = offset + a.size * 4
        items[name] = '{"dtype":"F32","shape":[%s],"data_offsets":[%d,%d]}' % (",".join(str(d) for d in a.shape), offset, end)
        offset = end
    if metadata is not None:
        def q(x):
            return json.dumps(x, ensure_ascii=False).replace("<", "\\u003c").replace(">", "\\u003e").replace("&", "\\u0026")
        items["__metadata__"] = "{" + ",".join(f"{q(k)}:{q(metadata[k])}" for k in sorted(metadata)) + "}"
    text = "{" + ",".join(f'"{k}":{items[k]}' for k in sorted(items)) + "}"
    raw = text.encode()
    raw += b" " * (-len(raw) % 8)
    return raw


def test_writer_layout_matches_the_reference(tmp_path):
    entries = {"v.0": np.arange(3, dtype=np.float32), "m.0": -np.arange(3, dtype=np.float32),
               "model.w": np.arange(6, dtype=np.float32).reshape(2, 3), "buffer.10": np.ones(1, np.float32)}
    metadata = {"format": "gograd-adamw", "version": "1", "optimizer": '{"Names":["a<b"],"LR":0.1}', "step_count": "3"}
    path = str(tmp_path / "state.safetensors")
    ag.safetensors_write(path, entries, metadata)
    raw = open(path, "rb").read()
    header = go_header(entries, metadata)
    assert raw[:8] == struct.pack("<Q", len(header))
    assert raw[8:8 + len(header)] == header and len(header) % 8 == 0
    payload = b"".join(entries[k].astype("<f4").tobytes() for k in sorted(entries))
    assert raw[8 + len(header):] == payload
    d = ag.safetensors_describe(path)
    assert d["metadata"] == metadata
    assert d["entries"]["model.w"]["shape"] == [2, 3] and d["entries"]["model.w"]["sum"] == 15.0
    assert sorted(d["entries"]) == sorted(entries)
    # no temporary file is left beside the target
    assert [p.name for p in tmp_path.iterdir()] == ["state.safetensors"]


def _file(header_text: bytes, payload: bytes) -> bytes:
    return struct.pack("<Q", len(header_text)) + header_text + payload


@pytest.mark.parametrize("name,blob,needle", [
    ("short", b"\x01\x02", "short safetensors file"),
    ("header_length", struct.pack("<Q", 1 << 40) + b"{}", "invalid safetensors header length"),
    ("dtype", _file(b'{"a":{"dtype":"F16","shape":[2],"data_offsets":[0,4]}}', b"\0" * 4), "incompatible dtype"),
    ("offsets", _file(b'{"a":{"dtype":"F32","shape":[2],"data_offsets":[0,4]}}', b"\0" * 8), "invalid offsets"),
    ("beyond_file", _file(b'{"a":{"dtype":"F32","shape":[2],"data_offsets":[0,8]}}', b"\0" * 4), "invalid"),
    ("overlap", _file(b'{"a":{"dtype":"F32","shape":[2],"data_offsets":[0,8]},"b":{"dtype":"F32","shape":[2],"data_offsets":[4,12]}}',
                      b"\0" * 12), "overlapping tensor ranges"),
    ("metadata", _file(b'{"__metadata__":{"k":1}}', b""), "invalid safetensors metadata"),
    ("json", _file(b'{"a":', b""), "invalid safetensors header"),
])
def test_reader_rejects_what_the_reference_rejects(tmp_path, name, blob, needle):
    path = tmp_path / f"{name}.safetensors"
    path.write_bytes(blob)
    with pytest.raises(ag.HostError) as e:
        ag.safetensors_describe(str(path))
    assert needle in str(e.value)


def test_empty_and_scalar_entries_round_trip(tmp_path):
    path = str(tmp_path / "x.safetensors")
    ag.safetensors_write(path, {"empty": np.zeros((0, 4), np.float32), "scalar": np.float32(2.5).reshape(())}, None)
    d = ag.safetensors_describe(path)
    assert d["entries"]["empty"]["shape"] == [0, 4] and d["entries"]["scalar"] == {"shape": [], "sum": 2.5}
    assert d["metadata"] == {}
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert b"__metadata__" not in raw[8:8 + hlen]


def test_grad_accumulator_bookkeeping():
    """GradAccumulator's counters and validation (autograd/accumulate.go:21-71, mirrored from
    autograd/accumulate_test.go:146-224): no device is involved."""
    for groups in (0, -1):
        with pytest.raises(ag.HostError, match="at least one micro-batch"):
            ag.GradAccumulator(groups)
    acc = ag.GradAccumulator(2)
    assert acc.Groups() == 2 and acc.Pending() == 0
    completes = []
    for micro in range(3):
        seed, complete = acc.MicroBatch()
        assert seed == np.float32(0.5)
        completes.append(complete)
    assert completes == [False, True, False] and acc.Pending() == 1
    acc.Reset()
    assert acc.Pending() == 0
    seed, complete = ag.GradAccumulator(3).MicroBatch()
    assert seed == np.float32(1) / np.float32(3) and not complete
    one = ag.GradAccumulator(1)
    assert one.MicroBatch() == (np.float32(1.0), True) and one.Pending() == 0
    broken = ag.GradAccumulator(2)
    broken._a.groups = 0
    with pytest.raises(ag.HostError, match="invalid gradient accumulator"):
        broken.MicroBatch()
    assert broken.Pending() == 0, "a failed call changes nothing"
