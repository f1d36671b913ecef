"""Checkpoint containers and codecs on CPU."""
import numpy as np
import pytest
import torch

from hartsyinference_b200.assets import gguf as G
from hartsyinference_b200.assets import safetensors as ST


def test_safetensors_roundtrip_and_sharded(tmp_path):
    a = {"w.a": torch.randn(5, 7), "w.b": torch.randn(3).to(torch.bfloat16), "w.c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "w.q": (torch.randn(4, 4) * 10).to(torch.float8_e4m3fn), "empty": torch.empty(0, 4)}
    ST.save_file(a, tmp_path / "x.safetensors", {"format": "pt", "note": 'quote " and \\ slash'})
    f = ST.SafeTensorsFile(tmp_path / "x.safetensors")
    assert set(f.keys()) == set(a)
    for k, v in a.items():
        got = f.get(k)
        assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape)
        assert torch.equal(got.view(torch.uint8), v.view(torch.uint8)) if v.numel() else True
    assert f.metadata["note"] == 'quote " and \\ slash'
    # cross-check with the reference implementation of the format when it is installed
    try:
        from safetensors.torch import load_file
        ref = load_file(str(tmp_path / "x.safetensors"))
        assert torch.equal(ref["w.a"], a["w.a"])
    except ImportError:
        pass
    ST.save_file({"p": torch.ones(2)}, tmp_path / "m-00001.safetensors")
    ST.save_file({"q": torch.zeros(2)}, tmp_path / "m-00002.safetensors")
    (tmp_path / "x.safetensors").unlink()
    ck = ST.ShardedCheckpoint(tmp_path)
    assert torch.equal(ck.get("p"), torch.ones(2)) and ck.get("nope") is None


def test_safetensors_rejects_garbage(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\xff" * 64)
    with pytest.raises(Exception):
        ST.SafeTensorsFile(p)


@pytest.mark.parametrize("name,tol", [("Q8_0", 0.01), ("Q4_0", 0.12), ("Q4_K", 0.08)])
def test_ggml_quant_dequant_roundtrip(name, tol):
    torch.manual_seed(0)
    x = torch.randn(8, 512)
    t = G.GGML_TYPES[name]
    raw = G.quantize(x, t)
    blk, nb = G.type_geometry(t)
    assert raw.numel() == x.numel() // blk * nb
    y = G.dequantize(raw, t, x.numel()).reshape(x.shape)
    rel = ((y - x).norm() / x.norm()).item()
    assert rel < tol, rel


def test_q8_0_matches_the_format_definition():
    # x = scale * q with scale = absmax / 127 stored as fp16, q = round(x / scale) clamped to +-127
    torch.manual_seed(1)
    x = torch.randn(64)
    raw = G.quantize(x, 8).numpy()
    for b in range(2):
        blk = raw[b * 34:(b + 1) * 34]
        d = np.frombuffer(blk[:2].tobytes(), dtype=np.float16)[0].astype(np.float32)
        q = np.frombuffer(blk[2:].tobytes(), dtype=np.int8).astype(np.float32)
        xs = x[b * 32:(b + 1) * 32].numpy()
        assert abs(d - np.abs(xs).max() / 127) < 1e-3 * max(1.0, d)
        assert np.abs(q * d - xs).max() <= d * 0.51 + 1e-3


def test_other_codecs_decode_hand_built_blocks():
    # Q4_1: y = q * d + m ; Q5_0: 5-bit value minus 16 ; IQ4_NL: table lookup
    d, m = np.float16(0.5), np.float16(-1.0)
    qs = np.arange(16, dtype=np.uint8) | (np.arange(16, dtype=np.uint8)[::-1] << 4)
    blk = d.tobytes() + m.tobytes() + qs.tobytes()
    y = G.dequantize(blk, 3, 32).numpy()
    assert np.allclose(y[:16], np.arange(16) * 0.5 - 1.0) and np.allclose(y[16:], np.arange(16)[::-1] * 0.5 - 1.0)
    qh = np.uint32(0xFFFF0000)
    blk5 = np.float16(1.0).tobytes() + qh.tobytes() + np.zeros(16, dtype=np.uint8).tobytes()
    y5 = G.dequantize(blk5, 6, 32).numpy()
    assert np.allclose(y5[:16], -16.0) and np.allclose(y5[16:], 0.0)
    blkn = np.float16(1.0).tobytes() + np.full(16, 0x0F, dtype=np.uint8).tobytes()
    yn = G.dequantize(blkn, 20, 32).numpy()
    assert np.allclose(yn[:16], 113.0) and np.allclose(yn[16:], -127.0)


def test_q6_k_and_q5_k_against_numpy_restatement():
    rng = np.random.default_rng(0)
    # Q6_K
    ql = rng.integers(0, 256, 128, dtype=np.uint8); qh = rng.integers(0, 256, 64, dtype=np.uint8)
    qli, qhi = ql.astype(np.int32), qh.astype(np.int32)
    sc = rng.integers(-32, 32, 16, dtype=np.int8); d = np.float16(0.01)
    blk = ql.tobytes() + qh.tobytes() + sc.tobytes() + d.tobytes()
    y = G.dequantize(blk, 14, 256).numpy()
    ref = np.zeros(256, dtype=np.float32)
    for n0 in (0, 1):
        for l in range(32):
            i_s = l // 16
            base = n0 * 128
            q_l, q_h, s = qli[n0 * 64:], qhi[n0 * 32:], sc[n0 * 8:].astype(np.int32)
            q1 = ((q_l[l] & 0xF) | (((q_h[l] >> 0) & 3) << 4)) - 32
            q2 = ((q_l[l + 32] & 0xF) | (((q_h[l] >> 2) & 3) << 4)) - 32
            q3 = ((q_l[l] >> 4) | (((q_h[l] >> 4) & 3) << 4)) - 32
            q4 = ((q_l[l + 32] >> 4) | (((q_h[l] >> 6) & 3) << 4)) - 32
            ref[base + l] = float(d) * s[i_s] * q1; ref[base + l + 32] = float(d) * s[i_s + 2] * q2
            ref[base + l + 64] = float(d) * s[i_s + 4] * q3; ref[base + l + 96] = float(d) * s[i_s + 6] * q4
    assert np.allclose(y, ref, atol=1e-5)


def test_gguf_write_read(tmp_path):
    torch.manual_seed(2)
    tensors = {"token_embd.weight": torch.randn(64, 256), "blk.0.attn_q.weight": torch.randn(256, 256),
               "output_norm.weight": torch.ones(256)}
    md = {"general.architecture": "llama", "llama.block_count": 1, "llama.embedding_length": 256,
          "llama.attention.head_count": 4, "llama.rope.freq_base": 10000.0, "general.name": "toy ✓",
          "tokenizer.ggml.tokens": ["a", "b", "c"], "tokenizer.ggml.scores": [0.5, 1.0, 2.0],
          "tokenizer.ggml.token_type": [1, 1, 1], "llama.use_thing": True}
    G.write_gguf(tmp_path / "t.gguf", md, tensors, quant={"blk.0.attn_q.weight": 12, "token_embd.weight": 8})
    f = G.GgufFile(tmp_path / "t.gguf")
    assert f.version == 3 and f.metadata["general.name"] == "toy ✓" and f.metadata["llama.block_count"] == 1
    assert f.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"] and f.metadata["llama.use_thing"] is True
    assert f.info("blk.0.attn_q.weight") == (12, (256, 256)) and f.info("output_norm.weight")[0] == 0
    q = f.get("blk.0.attn_q.weight")
    assert ((q - tensors["blk.0.attn_q.weight"]).norm() / tensors["blk.0.attn_q.weight"].norm()).item() < 0.08
    assert torch.equal(f.get("output_norm.weight"), tensors["output_norm.weight"])
    assert f.raw("token_embd.weight").numel() == 64 * 256 // 32 * 34
    from hartsyinference_b200.models.llm.config import from_gguf_metadata
    cfg = from_gguf_metadata(f.metadata)
    assert cfg.hidden_size == 256 and cfg.num_heads == 4 and cfg.vocab_size == 3


def test_views_keep_the_file_mapping_alive(tmp_path):
    """A view derived from a mapped tensor must stay readable after the reader object is gone."""
    import gc
    import torch
    from hartsyinference_b200.assets import gguf as G
    from hartsyinference_b200.assets.safetensors import SafeTensorsFile, save_file
    save_file({"a": torch.arange(1000, dtype=torch.float32)}, tmp_path / "x.safetensors")
    G.write_gguf(tmp_path / "x.gguf", {"general.architecture": "llama"}, {"a": torch.arange(1000, dtype=torch.float32).reshape(10, 100)})
    f = SafeTensorsFile(tmp_path / "x.safetensors")
    v = f.get("a").reshape(10, 100)[3:5]
    g = G.GgufFile(tmp_path / "x.gguf")
    w = g.get("a")[3:5]
    r = g.raw("a")[:16].view(torch.float32)
    del f, g
    gc.collect()
    assert v.sum().item() == w.sum().item() == float(torch.arange(300, 500).sum()) and r.tolist() == [0.0, 1.0, 2.0, 3.0]


def test_gguf_mxfp4_blocks(tmp_path):
    import torch
    from hartsyinference_b200.assets import gguf as G
    from hartsyinference_b200.assets.lowbit import E2M1
    assert G.type_geometry(G.MXFP4) == (32, 17)
    # one hand-made block: scale 2^1, element j = code j % 16 in the low nibbles, the reverse in the high ones
    lo = torch.arange(16, dtype=torch.uint8)
    hi = (15 - torch.arange(16)).to(torch.uint8)
    blk = torch.cat([torch.tensor([128], dtype=torch.uint8), lo | (hi << 4)])
    v = G.dequantize(blk, G.MXFP4, 32)
    table = torch.cat([E2M1, -E2M1]) * 2.0
    assert torch.equal(v[:16], table[lo.long()]) and torch.equal(v[16:], table[hi.long()])
    w = torch.randn(8, 64, generator=torch.Generator().manual_seed(0))
    packed = G.quantize(w, G.MXFP4)
    assert packed.numel() == 8 * 64 // 32 * 17
    back = G.dequantize(packed, G.MXFP4, w.numel()).reshape(w.shape)
    assert ((back - w).norm() / w.norm()) < 0.15
    G.write_gguf(tmp_path / "m.gguf", {"general.architecture": "llama"}, {"w": w}, quant={"w": G.MXFP4})
    f = G.GgufFile(tmp_path / "m.gguf")
    assert f.info("w")[0] == G.MXFP4 and torch.equal(f.get("w"), back)


def test_gguf_rejects_crafted_tensor_tables(tmp_path):
    """Offsets, dimensions and sizes that would wrap 64-bit arithmetic (and with it a naive bounds
    check), a negative dimension and data that starts past the end of the file are all refused at
    open instead of yielding a pointer outside the mapping."""
    import struct
    import pytest
    from hartsyinference_b200.assets import gguf as G
    from hartsyinference_b200.exceptions import HartsyInferenceError

    def s(text):
        b = text.encode()
        return struct.pack("<Q", len(b)) + b

    def build(dims, offset, ggml_type=0, pad=64):
        out = b"GGUF" + struct.pack("<IQQ", 3, 1, 0)            # version, tensors, metadata entries
        out += s("w") + struct.pack("<I", len(dims)) + b"".join(struct.pack("<q", d) for d in dims)
        out += struct.pack("<IQ", ggml_type, offset)
        out += b"\0" * ((-len(out)) % 32) + b"\0" * pad
        return out

    ok = tmp_path / "ok.gguf"
    ok.write_bytes(build([4, 4], 0))
    assert G.GgufFile(ok).get("w").shape == (4, 4)
    cases = {
        "wrapped_offset": build([4, 4], (1 << 64) - 32),
        "huge_offset": build([4, 4], 1 << 40),
        "negative_dim": build([-4, 4], 0),
        "zero_dim": build([0, 4], 0),
        "wrapping_dims": build([1 << 33, 1 << 33], 0),
        "too_big": build([1 << 20, 1 << 20], 0),
    }
    for name, blob in cases.items():
        p = tmp_path / f"{name}.gguf"
        p.write_bytes(blob)
        with pytest.raises(HartsyInferenceError):
            G.GgufFile(p)


def test_gguf_q3k_q8_1_q8_k_decoders():
    """Q3_K blocks against an independent statement of the format (the 6-bit scales recovered with
    the 32-bit mask arithmetic of the format's description), Q8_1 and Q8_K against their definition."""
    import ctypes as C
    import struct
    import numpy as np
    from hartsyinference_b200 import runtime
    fn = runtime.lib().b200_ggml_dequant
    fn.restype = C.c_int32
    rng = np.random.default_rng(0)

    def dequant(type_id, blocks, n):
        out = np.zeros(n, dtype=np.float32)
        rc = fn(type_id, blocks.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.POINTER(C.c_float)), C.c_int64(n))
        assert rc == 0
        return out

    nb = 5
    blk = rng.integers(0, 256, size=(nb, 110), dtype=np.uint8)
    for b in range(nb):
        blk[b, 108:110] = np.frombuffer(np.float16(rng.uniform(0.01, 0.1)).tobytes(), dtype=np.uint8)

    def ref_q3k(p):
        hm, qs, sc12 = p[:32], p[32:96], p[96:108]
        d = np.frombuffer(p[108:110].tobytes(), dtype=np.float16)[0].astype(np.float32)
        aux = list(struct.unpack("<3I", sc12.tobytes())) + [0]
        k1, k2 = 0x03030303, 0x0F0F0F0F
        tmp = aux[2]
        aux[2] = ((aux[0] >> 4) & k2) | (((tmp >> 4) & k1) << 4)
        aux[3] = ((aux[1] >> 4) & k2) | (((tmp >> 6) & k1) << 4)
        aux[0] = (aux[0] & k2) | (((tmp >> 0) & k1) << 4)
        aux[1] = (aux[1] & k2) | (((tmp >> 2) & k1) << 4)
        scales = np.frombuffer(struct.pack("<4I", *aux), dtype=np.int8).astype(np.int32) - 32
        y, i_s, m, q = [], 0, 1, 0
        for _ in range(2):
            shift = 0
            for _ in range(4):
                for part in (0, 16):
                    dl = d * scales[i_s]
                    i_s += 1
                    for l in range(16):
                        y.append(dl * (((int(qs[q + l + part]) >> shift) & 3) - (0 if hm[l + part] & m else 4)))
                shift += 2
                m <<= 1
            q += 32
        return np.array(y, dtype=np.float32)

    want = np.concatenate([ref_q3k(blk[b]) for b in range(nb)])
    assert np.array_equal(dequant(11, blk, nb * 256), want)
    # Q8_1: f16 scale, f16 sum, 32 int8
    b81 = np.zeros((3, 36), dtype=np.uint8)
    q81 = rng.integers(-127, 128, size=(3, 32)).astype(np.int8)
    for i in range(3):
        b81[i, 0:2] = np.frombuffer(np.float16(0.03 * (i + 1)).tobytes(), dtype=np.uint8)
        b81[i, 4:] = q81[i].view(np.uint8)
    got = dequant(9, b81, 96).reshape(3, 32)
    assert np.allclose(got, q81.astype(np.float32) * np.array([np.float16(0.03 * (i + 1)) for i in range(3)], dtype=np.float32)[:, None])
    # Q8_K: fp32 scale, 256 int8, 16 int16 block sums
    b8k = np.zeros((2, 292), dtype=np.uint8)
    q8k = rng.integers(-127, 128, size=(2, 256)).astype(np.int8)
    for i in range(2):
        b8k[i, 0:4] = np.frombuffer(np.float32(0.011 * (i + 1)).tobytes(), dtype=np.uint8)
        b8k[i, 4:260] = q8k[i].view(np.uint8)
    got = dequant(15, b8k, 512).reshape(2, 256)
    assert np.allclose(got, q8k.astype(np.float32) * np.array([0.011, 0.022], dtype=np.float32)[:, None])
