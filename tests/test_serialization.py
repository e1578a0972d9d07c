"""State-dict round trips of quantized layers through the SafeTensors format, following the
reference writer's conventions (lucid/serialization/__init__.py:833-921, _safetensors.py)."""
import json
import struct

import numpy as np
import pytest
import torch

import lucid_b200 as lucid
from lucid_b200.serialization import SCALAR_KEYS_KEY, load_safetensors, safe_open, save_safetensors


def test_layout_matches_the_reference_writer(tmp_path):
    sd = {"w": torch.arange(6, dtype=torch.int8).reshape(2, 3), "s": torch.tensor(0.5),
          "p": torch.tensor([[-1, 2**31 - 1]], dtype=torch.int32), "h": torch.ones(3, dtype=torch.bfloat16)}
    path = tmp_path / "m.safetensors"
    save_safetensors(sd, path, metadata={"format": "lucid"})
    raw = path.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0 and raw[8:8 + n].rstrip(b" ").endswith(b"}")
    header = json.loads(raw[8:8 + n])
    assert list(header) == ["w", "s", "p", "h", "__metadata__"]  # insertion order, metadata last
    assert header["w"] == {"dtype": "I8", "shape": [2, 3], "data_offsets": [0, 6]}
    assert header["s"] == {"dtype": "F32", "shape": [1], "data_offsets": [6, 10]}  # zero-rank stored as (1,)
    assert header["p"]["dtype"] == "I32" and header["h"]["dtype"] == "BF16"
    assert header["__metadata__"] == {"format": "lucid", SCALAR_KEYS_KEY: '["s"]'}
    assert len(raw) == 8 + n + 6 + 4 + 8 + 6
    back = load_safetensors(path)
    assert list(back) == list(sd)
    for k in sd:
        assert back[k].dtype == sd[k].dtype and back[k].shape == sd[k].shape and torch.equal(back[k], sd[k])
    with safe_open(path) as f:
        assert f.metadata() == {"format": "lucid"} and f.keys() == list(sd)


def test_reads_files_of_other_writers(tmp_path):
    """Unsigned tensors widen, legacy comma-joined scalar keys are understood, unpadded headers load."""
    blobs = [np.array([0, 255], np.uint8).tobytes(), np.array([65535], np.uint16).tobytes(),
             np.array([4294967295], np.uint32).tobytes(), np.array([1.5], np.float32).tobytes()]
    header, off = {}, 0
    for name, code, shape, blob in (("a", "U8", [2], blobs[0]), ("b", "U16", [1], blobs[1]), ("c", "U32", [1], blobs[2]),
                                    ("x,y", "F32", [1], blobs[3])):
        header[name] = {"dtype": code, "shape": shape, "data_offsets": [off, off + len(blob)]}
        off += len(blob)
    header["__metadata__"] = {SCALAR_KEYS_KEY: "c"}  # legacy form
    enc = json.dumps(header).encode()
    path = tmp_path / "u.safetensors"
    path.write_bytes(struct.pack("<Q", len(enc)) + enc + b"".join(blobs))
    t = load_safetensors(path)
    assert t["a"].dtype is torch.int16 and t["a"].tolist() == [0, 255]
    assert t["b"].dtype is torch.int32 and t["b"].tolist() == [65535]
    assert t["c"].dtype is torch.int64 and t["c"].shape == () and int(t["c"]) == 4294967295
    assert t["x,y"].shape == (1,)
    bad = dict(header)
    bad["a"] = {"dtype": "U8", "shape": [3], "data_offsets": [0, 2]}
    enc = json.dumps(bad).encode()
    path.write_bytes(struct.pack("<Q", len(enc)) + enc + b"".join(blobs))
    with pytest.raises(ValueError, match="inconsistent"):
        load_safetensors(path)
    with pytest.raises(TypeError, match="strings to strings"):
        save_safetensors({}, path, metadata={"a": 1})
    with pytest.raises(ValueError, match="reserved"):
        save_safetensors({}, path, metadata={SCALAR_KEYS_KEY: "x"})
    with pytest.raises(TypeError, match="expected Tensor"):
        save_safetensors({"a": 1}, path)


@pytest.mark.gpu
def test_quantized_models_round_trip(tmp_path):
    """Static, dynamic, group-wise, recurrent and functional modules: state_dict -> file -> a
    freshly converted model gives the same bits; the packed group words keep their bit pattern."""
    import lucid_b200.nn.quantized as nnq
    import lucid_b200.quantization as Q
    from torch import nn

    torch.manual_seed(0)

    def build():
        torch.manual_seed(1)
        return nn.Sequential(nn.Linear(64, 128), nn.ReLU(), nn.Linear(128, 64))

    x = torch.randn(8, 64, device="cuda")
    prepared = Q.prepare(build()).cuda()
    prepared(x)
    static = Q.convert(prepared)
    dynamic = Q.quantize_dynamic(build())
    group = nnq.QuantizedLinearMLX.from_float(build()[0], bits=4, group_size=64)
    rnn = Q.quantize_dynamic(nn.ModuleDict({"rnn": nn.GRU(64, 32, batch_first=True)}))
    for i, (model, run) in enumerate(((static, lambda m: m(x)), (dynamic, lambda m: m(x)), (group, lambda m: m(x)),
                                      (rnn, lambda m: m["rnn"](x[None])[0]))):
        want = run(model)
        path = tmp_path / f"m{i}.safetensors"
        lucid.save(model.state_dict(), path)
        loaded = lucid.load(path)
        assert list(loaded) == list(model.state_dict())
        for k, v in model.state_dict().items():
            assert loaded[k].dtype == v.dtype and loaded[k].shape == v.shape and torch.equal(loaded[k], v.cpu())
        import copy

        fresh = copy.deepcopy(model)
        for b in fresh.buffers():
            b.zero_()
        fresh.load_state_dict(loaded)
        assert torch.equal(run(fresh), want)
    words = group.state_dict()["packed_weight"]
    assert words.dtype is torch.int32 and bool((words < 0).any())  # high code bits set: uint32 patterns in int32
