"""GGUF container and quant-codec tests (pattern: write -> read round trips and malformed-file rejection,
as in the reference's fs/ggml and fs/gguf test suites)."""
import struct

import numpy as np
import pytest
import torch

from ollama_b200.gguf import quants
from ollama_b200.gguf.reader import GGUFError, open_gguf
from ollama_b200.gguf.types import GGMLType, type_size, block_size, row_bytes
from ollama_b200.gguf.writer import WriteTensor, write_gguf


def test_roundtrip_kv_and_tensors(tmp_path):
    p = tmp_path / "a.gguf"
    w = torch.randn(4, 64)
    kv = {"general.architecture": "llama", "block_count": 2, "rope.freq_base": 10000.0, "general.name": "x",
          "tokenizer.ggml.tokens": ["a", "b", "c"], "tokenizer.ggml.scores": [0.0, 1.0, 2.0], "flag": True,
          "attention.head_count_kv": [1, 2]}
    write_gguf(p, kv, [WriteTensor("blk.1.w.weight", (64, 4), GGMLType.F32, w.numpy()),
                       WriteTensor("blk.0.w.weight", (64, 4), GGMLType.Q8_0, quants.quantize(w, GGMLType.Q8_0).numpy()),
                       WriteTensor("token_embd.weight", (64, 4), GGMLType.F16, w.half().numpy())])
    g = open_gguf(p)
    assert g.version == 3 and g.architecture == "llama"
    assert g.uint("block_count") == 2 and g.kv["llama.flag"] is True
    assert g.kv["tokenizer.ggml.tokens"] == ["a", "b", "c"]
    assert list(g.kv["llama.attention.head_count_kv"]) == [1, 2]
    assert list(g.tensors) == ["token_embd.weight", "blk.0.w.weight", "blk.1.w.weight"]  # block order, then name
    for ti in g.tensors.values():
        assert ti.offset % 32 == 0
    got = quants.dequantize_tensor(torch.from_numpy(g.tensor_bytes("blk.1.w.weight").copy()), GGMLType.F32, (4, 64))
    assert torch.equal(got, w)
    assert g.tensors["blk.0.w.weight"].torch_shape == (4, 64)
    g.close()


def test_rejects_malformed(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(GGUFError):
        open_gguf(p)
    p.write_bytes(b"GGUF" + struct.pack("<I", 9) + b"\0" * 64)
    with pytest.raises(GGUFError):
        open_gguf(p)
    # string length beyond the file
    p.write_bytes(b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1 << 40))
    with pytest.raises(GGUFError):
        open_gguf(p)
    # tensor data beyond end of file
    good = tmp_path / "g.gguf"
    write_gguf(good, {"general.architecture": "llama"}, [WriteTensor("a", (32,), GGMLType.F32, np.zeros(32, np.float32))])
    data = good.read_bytes()
    p.write_bytes(data[:-64])
    with pytest.raises(GGUFError):
        open_gguf(p)


def test_v2_and_big_endian_headers(tmp_path):
    def s(x, bo):
        b = x.encode()
        return struct.pack(bo + "Q", len(b)) + b
    for bo in ("<", ">"):
        body = b"GGUF" + struct.pack(bo + "IQQ", 2, 0, 1) + s("general.architecture", bo) + struct.pack(bo + "I", 8) + s("llama", bo)
        p = tmp_path / f"h{ord(bo)}.gguf"
        p.write_bytes(body + b"\0" * 64)
        g = open_gguf(p)
        assert g.version == 2 and g.architecture == "llama"


@pytest.mark.parametrize("t", [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q4_1, GGMLType.Q5_0, GGMLType.Q4_K, GGMLType.Q5_K,
                               GGMLType.Q6_K, GGMLType.MXFP4, GGMLType.F16, GGMLType.BF16])
def test_quant_roundtrip_error(t):
    torch.manual_seed(0)
    x = torch.randn(8, 512) * 0.02
    raw = quants.quantize(x, t)
    assert raw.numel() == 8 * row_bytes(t, 512)
    y = quants.dequantize_tensor(raw, t, (8, 512))
    rel = ((x - y).norm() / x.norm()).item()
    bound = {GGMLType.Q8_0: 0.01, GGMLType.Q4_0: 0.15, GGMLType.Q4_1: 0.12, GGMLType.Q5_0: 0.08, GGMLType.Q4_K: 0.10,
             GGMLType.Q5_K: 0.05, GGMLType.Q6_K: 0.03, GGMLType.MXFP4: 0.20, GGMLType.F16: 1e-3, GGMLType.BF16: 1e-2}[t]
    assert rel < bound, rel


def test_q8_0_exact_layout():
    x = torch.arange(-16, 16, dtype=torch.float32)
    raw = quants.quantize_q8_0(x).numpy()
    d = np.frombuffer(raw[:2].tobytes(), dtype=np.float16)[0]
    assert abs(float(d) - 16 / 127) < 1e-3
    q = raw[2:].view(np.int8)
    assert q[0] == -127 and q[16] == 0


def test_k_quant_scalar_decoders():
    """Decode Q4_K / Q6_K / Q2_K / Q3_K / Q5_K blocks with straightforward scalar loops and compare."""
    rng = np.random.default_rng(0)

    def half(b):
        return float(np.frombuffer(bytes(b), dtype=np.float16)[0])

    def k4(j, q):
        if j < 4:
            return q[j] & 63, q[j + 4] & 63
        return (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4), (q[j + 4] >> 4) | ((q[j] >> 6) << 4)

    for t in (GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.Q2_K, GGMLType.Q3_K):
        ts = type_size(t)
        blk = rng.integers(0, 256, ts, dtype=np.uint8)
        # keep the half-precision scales finite
        hpos = {GGMLType.Q4_K: [0, 2], GGMLType.Q5_K: [0, 2], GGMLType.Q6_K: [208], GGMLType.Q2_K: [80, 82], GGMLType.Q3_K: [108]}[t]
        for h in hpos:
            blk[h:h + 2] = np.frombuffer(np.float16(rng.uniform(0.01, 0.1)).tobytes(), dtype=np.uint8)
        y = np.zeros(256, np.float64)
        b = [int(v) for v in blk]
        if t == GGMLType.Q4_K:
            d, dmin, sc, qs = half(b[0:2]), half(b[2:4]), b[4:16], b[16:144]
            o = 0
            for j in range(4):
                s1, m1 = k4(2 * j, sc); s2, m2 = k4(2 * j + 1, sc)
                for l in range(32):
                    y[o + l] = d * s1 * (qs[32 * j + l] & 15) - dmin * m1
                    y[o + 32 + l] = d * s2 * (qs[32 * j + l] >> 4) - dmin * m2
                o += 64
        elif t == GGMLType.Q5_K:
            d, dmin, sc, qh, qs = half(b[0:2]), half(b[2:4]), b[4:16], b[16:48], b[48:176]
            o = 0
            for j in range(4):
                s1, m1 = k4(2 * j, sc); s2, m2 = k4(2 * j + 1, sc)
                for l in range(32):
                    y[o + l] = d * s1 * ((qs[32 * j + l] & 15) + (16 if qh[l] & (1 << (2 * j)) else 0)) - dmin * m1
                    y[o + 32 + l] = d * s2 * ((qs[32 * j + l] >> 4) + (16 if qh[l] & (2 << (2 * j)) else 0)) - dmin * m2
                o += 64
        elif t == GGMLType.Q6_K:
            ql, qh, sc, d = b[0:128], b[128:192], [v - 256 if v > 127 else v for v in b[192:208]], half(b[208:210])
            for n in range(2):
                for l in range(32):
                    i = l // 16
                    q1 = ((ql[64 * n + l] & 15) | (((qh[32 * n + l] >> 0) & 3) << 4)) - 32
                    q2 = ((ql[64 * n + l + 32] & 15) | (((qh[32 * n + l] >> 2) & 3) << 4)) - 32
                    q3 = ((ql[64 * n + l] >> 4) | (((qh[32 * n + l] >> 4) & 3) << 4)) - 32
                    q4 = ((ql[64 * n + l + 32] >> 4) | (((qh[32 * n + l] >> 6) & 3) << 4)) - 32
                    y[128 * n + l] = d * sc[8 * n + i] * q1
                    y[128 * n + l + 32] = d * sc[8 * n + i + 2] * q2
                    y[128 * n + l + 64] = d * sc[8 * n + i + 4] * q3
                    y[128 * n + l + 96] = d * sc[8 * n + i + 6] * q4
        elif t == GGMLType.Q2_K:
            scales, qs, d, dmin = b[0:16], b[16:80], half(b[80:82]), half(b[82:84])
            o, i = 0, 0
            for n in range(2):
                for j in range(4):
                    for half_ in range(2):
                        s = scales[i]; i += 1
                        for l in range(16):
                            y[o] = d * (s & 15) * ((qs[32 * n + 16 * half_ + l] >> (2 * j)) & 3) - dmin * (s >> 4)
                            o += 1
        elif t == GGMLType.Q3_K:
            hm, qs, sc, d = b[0:32], b[32:96], b[96:108], half(b[108:110])
            s16 = []
            for k in range(16):
                lo = (sc[k % 8] >> (4 * (k // 8))) & 15
                hi = (sc[8 + k % 4] >> (2 * (k // 4))) & 3
                s16.append((lo | (hi << 4)) - 32)
            o, i, m = 0, 0, 1
            for n in range(2):
                for j in range(4):
                    for half_ in range(2):
                        dl = d * s16[i]; i += 1
                        for l in range(16):
                            idx = 16 * half_ + l
                            y[o] = dl * (((qs[32 * n + idx] >> (2 * j)) & 3) - (0 if hm[idx] & m else 4))
                            o += 1
                    m <<= 1
        got = quants.dequantize(torch.from_numpy(blk.copy()), t).double().numpy()
        np.testing.assert_allclose(got, y, rtol=1e-5, atol=1e-6, err_msg=t.name)


def test_mxfp4_values():
    blk = np.zeros(17, np.uint8)
    blk[0] = 128            # scale 2
    blk[1] = 0x71           # low nibble 1 -> 0.5, high nibble 7 -> 6.0
    y = quants.dequantize(torch.from_numpy(blk), GGMLType.MXFP4)
    assert y[0].item() == 1.0 and y[16].item() == 12.0


@pytest.mark.parametrize("t", [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.MXFP4])
def test_native_codecs_match_the_tensor_op_codecs(t):
    """The C++ block codecs (native/codecs.cpp) decode to the same floats and encode to the same bytes as the torch codecs."""
    from ollama_b200.gguf import quants
    from ollama_b200.utils import hostlib
    if hostlib.lib() is None:
        pytest.skip("host library not built")
    g = torch.Generator().manual_seed(int(t))
    x = torch.randn(64, 1024, generator=g) * torch.rand(64, 1, generator=g) * 3
    x[3, :256] = 0.0                      # an all-zero block
    x[5, 100] = 70000.0                   # a scale beyond the half range
    raw = quants.quantize(x, t, native=False)
    a, b = quants.dequantize(raw, t, native=False), quants.dequantize(raw, t, native=True)
    ok = torch.isfinite(a)
    assert torch.equal(ok, torch.isfinite(b)) and torch.allclose(a[ok], b[ok], rtol=1e-6, atol=0)
    if hostlib.codec_supported(int(t), True):
        assert torch.equal(quants.quantize(x, t, native=True), raw)
    # garbage bytes (every bit pattern of the scale fields included) decode identically
    junk = torch.randint(0, 256, (raw.numel(),), dtype=torch.uint8, generator=g)
    a, b = quants.dequantize(junk, t, native=False), quants.dequantize(junk, t, native=True)
    ok = torch.isfinite(a)
    assert torch.equal(ok, torch.isfinite(b)) and torch.allclose(a[ok], b[ok], rtol=1e-6, atol=0)


def test_reader_survives_corrupted_files(tmp_path):
    """Random byte flips and truncations of a valid file (the reference fuzzes its reader the same way,
    fs/gguf/gguf_internal_test.go): the reader either opens the file or raises GGUFError, nothing else."""
    import random
    p = str(tmp_path / "a.gguf")
    write_gguf(p, {"general.architecture": "llama", "llama.block_count": 2, "tokenizer.ggml.tokens": ["a", "b", "c"], "x.arr": [1, 2, 3],
                   "general.name": "t"},
               [WriteTensor("a.weight", (32, 4), GGMLType.F32, np.zeros((4, 32), np.float32).tobytes()),
                WriteTensor("b.weight", (64,), GGMLType.Q8_0, bytes(68))])
    data = open(p, "rb").read()
    rnd = random.Random(0)
    q = str(tmp_path / "m.gguf")
    opened = 0
    for _ in range(800):
        b = bytearray(data)
        for _ in range(rnd.randint(1, 4)):
            b[rnd.randrange(0, min(len(b), 400))] = rnd.randrange(256)
        if rnd.random() < 0.2:
            b = b[:rnd.randrange(1, len(b))]
        with open(q, "wb") as f:
            f.write(b)
        try:
            g = open_gguf(q)
            for n in g.tensors:
                g.tensor_bytes(n)
            g.close()
            opened += 1
        except GGUFError:
            pass
    assert 0 < opened < 800


def test_host_helpers_are_clean_under_sanitizers():
    """The C++ codecs and the BPE merge loop, built with AddressSanitizer + UndefinedBehaviorSanitizer, on random blocks, on
    floats that include NaN / infinities / denormals, and on random merge tables (exerciser: ollama_b200/native/selftest.cc)."""
    import shutil
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    from ollama_b200.native.sanitize import run
    assert run() == 0
