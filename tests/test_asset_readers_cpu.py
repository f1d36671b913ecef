"""ONNX initialiser reader, PyTorch checkpoint reader, finite scalar quantiser."""
import struct

import numpy as np
import pytest
import torch

from hartsyinference_b200.assets.onnx_reader import read_onnx_initializers
from hartsyinference_b200.assets.torch_checkpoint import load_torch_checkpoint
from hartsyinference_b200.audio.fsq import Fsq


def _vi(n: int) -> bytes:
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _ld(num: int, payload: bytes) -> bytes:
    return _vi((num << 3) | 2) + _vi(len(payload)) + payload


def _v(num: int, val: int) -> bytes:
    return _vi(num << 3) + _vi(val)


def _tensor_proto(name, dims, dtype, raw=None, floats=None, ints=None, int_field=5, packed_dims=True, external=None):
    b = _ld(1, b"".join(_vi(d) for d in dims)) if packed_dims else b"".join(_v(1, d) for d in dims)
    b += _v(2, dtype)
    if floats is not None:
        b += _ld(4, np.asarray(floats, "<f4").tobytes())
    if ints is not None:
        b += _ld(int_field, b"".join(_vi(i) for i in ints))
    b += _ld(8, name.encode())
    if raw is not None:
        b += _ld(9, raw)
    if external:
        for k, v in external.items():
            b += _ld(13, _ld(1, k.encode()) + _ld(2, v.encode()))
        b += _v(14, 1)
    return b


def test_onnx_initializers(tmp_path):
    w = np.arange(12, dtype="<f4").reshape(3, 4)
    h = np.asarray([1.5, -2.0], np.float16)
    ext = np.arange(6, dtype="<i2")
    (tmp_path / "weights.bin").write_bytes(b"\0" * 8 + ext.tobytes())
    bf = torch.tensor([1.0, -3.5, 0.15625], dtype=torch.bfloat16)
    inits = [
        _tensor_proto("dense.weight", [3, 4], 1, raw=w.tobytes()),
        _tensor_proto("typed.floats", [2, 2], 1, floats=[1, 2, 3, 4], packed_dims=False),
        _tensor_proto("ids", [3], 7, ints=[5, -1, 1 << 40], int_field=7),
        _tensor_proto("half.bits", [2], 10, ints=[int(x) for x in h.view(np.uint16)]),
        _tensor_proto("bf", [3], 16, raw=bf.view(torch.int16).numpy().tobytes()),
        _tensor_proto("scalar", [], 6, ints=[-7]),
        _tensor_proto("outside", [2, 3], 5, external={"location": "weights.bin", "offset": "8", "length": "12"}),
    ]
    node = _ld(1, _ld(1, b"x") + _ld(4, b"Relu"))                      # a node, skipped
    graph = node + _ld(2, b"g") + b"".join(_ld(5, t) for t in inits)
    model = _v(1, 8) + _ld(2, b"test") + _ld(7, graph) + _ld(8, _ld(1, b"") + _v(2, 17))
    (tmp_path / "m.onnx").write_bytes(model)
    t = read_onnx_initializers(tmp_path / "m.onnx")
    assert set(t) == {"dense.weight", "typed.floats", "ids", "half.bits", "bf", "scalar", "outside"}
    assert torch.equal(t["dense.weight"], torch.from_numpy(w.copy()))
    assert t["typed.floats"].tolist() == [[1, 2], [3, 4]]
    assert t["ids"].dtype == torch.int64 and t["ids"].tolist() == [5, -1, 1 << 40]
    assert t["half.bits"].dtype == torch.float16 and t["half.bits"].tolist() == [1.5, -2.0]
    assert t["bf"].dtype == torch.bfloat16 and torch.equal(t["bf"], bf)
    assert t["scalar"].shape == () and int(t["scalar"]) == -7
    assert t["outside"].dtype == torch.int16 and t["outside"].tolist() == [[0, 1, 2], [3, 4, 5]]
    (tmp_path / "bad.onnx").write_bytes(model[: len(model) // 2])        # cut in the middle of the graph
    with pytest.raises(ValueError):
        read_onnx_initializers(tmp_path / "bad.onnx")


def test_torch_checkpoint_reader(tmp_path):
    sd = {"a.weight": torch.randn(3, 4), "a.bias": torch.zeros(3), "blocks": [{"w": torch.ones(2)}, {"w": torch.ones(2) * 2}]}
    torch.save({"state_dict": sd, "epoch": 3}, tmp_path / "wrapped.pth")
    torch.save(sd, tmp_path / "plain.pt")
    for name in ("wrapped.pth", "plain.pt"):
        t = load_torch_checkpoint(tmp_path / name)
        assert set(t) == {"a.weight", "a.bias", "blocks.0.w", "blocks.1.w"}
        assert torch.equal(t["a.weight"], sd["a.weight"]) and t["blocks.1.w"].tolist() == [2, 2]

    class Evil:
        def __reduce__(self):
            return (print, ("executed",))
    import pickle
    (tmp_path / "evil.pt").write_bytes(pickle.dumps({"x": Evil()}))
    with pytest.raises(Exception):
        load_torch_checkpoint(tmp_path / "evil.pt")


def test_fsq_roundtrip():
    f = Fsq([8, 5, 5, 5])
    assert f.codebook_size == 1000
    idx = torch.arange(1000)
    codes = f.indices_to_codes(idx)
    assert codes.shape == (1000, 4) and codes.min() >= -1 and codes.max() <= 1
    assert torch.equal(f.codes_to_indices(codes), idx)
    z = torch.randn(64, 4, generator=torch.Generator().manual_seed(0)) * 3
    q = f.quantize(z)
    assert torch.equal(f.indices_to_codes(f.encode(z)), q)
    # odd level counts are symmetric around zero; quantisation keeps the sign of large inputs
    assert torch.equal(torch.sign(q[:, 1][z[:, 1].abs() > 1]), torch.sign(z[:, 1][z[:, 1].abs() > 1]))
    assert len(torch.unique(q[:, 0])) <= 8 and len(torch.unique(q[:, 1])) <= 5
