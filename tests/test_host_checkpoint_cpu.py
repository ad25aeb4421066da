"""The safetensors container of the host mirror, checked without a GPU against the layout
the reference writes (autograd/safetensors.go:30-98) and the rules its reader enforces
(autograd/safetensors_stream.go:28-96)."""
import json
import os
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


def _state_case():
    rng = np.random.default_rng(3)
    names = [f"layer{i}.w" for i in range(12)]          # twelve entries: "m.10" sorts before "m.2"
    shapes = [[3, 4], [5], [2, 2, 2], [1], [7], [6], [4, 4], [9], [10], [11], [2, 6], [13]]
    m = [rng.normal(0, 1, int(np.prod(s))).astype(np.float32) for s in shapes]
    v = [np.abs(rng.normal(0, 1, int(np.prod(s)))).astype(np.float32) for s in shapes]
    groups = [("decay", [0, 2, 4, 6, 8, 10], 1.0, 0.1), ("plain", [1, 3, 5, 7, 9, 11], 0.5, 0.0)]
    config = dict(step_count=17, lr=3e-4, weight_decay=0.1, beta1=0.9, beta2=0.95, eps=1e-8)
    return names, shapes, m, v, groups, config


def test_streamed_state_file_equals_the_one_written_from_memory(tmp_path):
    """The streaming writer produces the bytes of the in-memory writer; entries arrive in the file's
    own order (sorted names), whole or in pieces."""
    names, shapes, m, v, groups, c = _state_case()
    whole, streamed = str(tmp_path / "whole.safetensors"), str(tmp_path / "streamed.safetensors")
    ag.adamw_state_write(whole, names, shapes, m, v, c["step_count"], c["lr"], c["weight_decay"], c["beta1"], c["beta2"],
                         c["eps"], groups)
    stream = ag.AdamWStateStream(streamed, names, shapes, c["step_count"], c["lr"], c["weight_decay"], c["beta1"],
                                 c["beta2"], c["eps"], groups)
    order = []
    while True:
        nxt = stream.next()
        if nxt is None:
            break
        entry, remaining = nxt
        key, index = entry.split(".")
        values = (m if key == "m" else v)[int(index)]
        assert remaining == values.size
        order.append(entry)
        if values.size > 3:                                  # two pieces, as two owners of a straddling tensor would
            stream.append(entry, values[:3])
            assert stream.next() == (entry, values.size - 3)
            stream.append(entry, values[3:])
        else:
            stream.append(entry, values)
    stream.finish()
    assert order == sorted(order) and order[:4] == ["m.0", "m.1", "m.10", "m.11"]
    assert open(whole, "rb").read() == open(streamed, "rb").read()


def test_stream_rejects_wrong_order_and_incomplete_files(tmp_path):
    names, shapes, m, v, groups, c = _state_case()
    path = str(tmp_path / "broken.safetensors")
    args = (names, shapes, c["step_count"], c["lr"], c["weight_decay"], c["beta1"], c["beta2"], c["eps"], groups)
    stream = ag.AdamWStateStream(path, *args)
    with pytest.raises(ag.HostError, match="out of order"):
        stream.append("m.1", m[1])
    stream.append("m.0", m[0][:5])
    with pytest.raises(ag.HostError, match="too many values"):
        stream.append("m.0", m[0])
    with pytest.raises(ag.HostError, match="m.0 was not written"):
        stream.finish()
    assert [f for f in os.listdir(tmp_path) if not f.startswith("whole")] == [], "no file and no temporary left behind"
    stream = ag.AdamWStateStream(path, *args)
    stream.abort()
    assert os.listdir(tmp_path) == []
