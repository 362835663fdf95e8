"""Host compressors (the CPU data path and the oracle of the fused GPU kernels).

numpy restatements of the spec are the oracle; the code under test is the native
FP16Compressor / TopKCompressor (the reference's tests/test_compression.py:85-126 only
tested a Python re-implementation).
"""
import struct

import numpy as np
import pytest
import torch


def test_fp16_roundtrip_matches_numpy(native):
    x = torch.randn(10007) * 100
    blob = native._fp16_compress(x)
    assert len(blob) == 2 * x.numel()
    got = np.frombuffer(blob, dtype=np.float16)
    want = x.numpy().astype(np.float16)
    # normal range: identical bits (round to nearest even)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    back = native._fp16_decompress(blob, x.numel())
    assert torch.equal(back, torch.from_numpy(want.astype(np.float32)))


def test_fp16_special_values(native):
    x = torch.tensor([0.0, -0.0, float("inf"), -float("inf"), float("nan"), 65504.0, 65520.0, 1e-8, -1e-8, 6.2e-5])
    got = np.frombuffer(native._fp16_compress(x), dtype=np.float16)
    assert got[0] == 0 and np.signbit(got[1])
    assert np.isposinf(got[2]) and np.isneginf(got[3]) and np.isnan(got[4])
    assert got[5] == np.float16(65504.0) and np.isposinf(got[6])
    assert got[7] == 0 and got[8] == 0 and np.signbit(got[8])  # below the half-normal range: flushed to signed zero
    assert got[9] == np.float16(6.2e-5)  # smallest normals survive


def test_fp16_rejects_other_dtypes(native):
    with pytest.raises(RuntimeError):
        native._fp16_compress(torch.zeros(4, dtype=torch.int32))


def _unpack(blob):
    k = struct.unpack_from("<I", blob, 0)[0]
    rec = np.frombuffer(blob, dtype=np.dtype([("i", "<u4"), ("v", "<f4")]), offset=4, count=k)
    return k, rec["i"].astype(np.int64), rec["v"].copy()


def test_topk_wire_format_and_selection(native):
    g = torch.tensor([0.1, -5.0, 0.2, 4.0, -0.3, 3.0, 0.0, -2.0, 1.0, 0.5])
    c = native.TopKCompressor(0.3)
    assert c.k_for(10) == 3 and c.k_for(1) == 1 and c.k_for(3) == 1 and c.k_for(1000) == 300
    blob = c.compress(g, 1)
    assert len(blob) == 4 + 3 * 8
    k, idx, val = _unpack(blob)
    assert k == 3 and idx.tolist() == [1, 3, 5] and val.tolist() == [-5.0, 4.0, 3.0]
    dense = c.decompress(blob, 10)
    assert dense.tolist() == [0, -5.0, 0, 4.0, 0, 3.0, 0, 0, 0, 0]
    res = c.residual(1)
    assert torch.equal(res, torch.tensor([0.1, 0.0, 0.2, 0.0, -0.3, 0.0, 0.0, -2.0, 1.0, 0.5]))


def test_topk_error_feedback_eventually_sends_everything(native):
    n = 200
    c = native.TopKCompressor(0.05)
    g = torch.rand(n) + 0.1
    sent = torch.zeros(n)
    # a gradient of ones-ish, repeated: residuals grow until every index has been sent
    for _ in range(1000):
        k, idx, val = _unpack(c.compress(g, 0))
        sent[idx] += 1
        if (sent > 0).all():
            break
    assert (sent > 0).all(), "error feedback must surface every coordinate eventually"


def test_topk_residuals_are_keyed_by_bucket(native):
    c = native.TopKCompressor(0.5)
    a = torch.tensor([1.0, 2.0, 3.0, 4.0])
    b = torch.tensor([40.0, 30.0, 20.0, 10.0])
    c.compress(a, 11)
    c.compress(b, 22)
    assert c.residual(11).tolist() == [1.0, 2.0, 0.0, 0.0]
    assert c.residual(22).tolist() == [0.0, 0.0, 20.0, 10.0]
    assert c.residual_buffers() == 2
    c.reset_error_feedback()
    assert c.residual_buffers() == 0


def test_topk_conserves_mass(native):
    # sent + residual == sum of everything fed in
    n = 5000
    c = native.TopKCompressor(0.01)
    total_in = torch.zeros(n, dtype=torch.float64)
    total_sent = torch.zeros(n, dtype=torch.float64)
    for s in range(20):
        g = torch.randn(n, generator=torch.Generator().manual_seed(s))
        total_in += g.double()
        total_sent += c.decompress(c.compress(g, 0), n).double()
    assert torch.allclose(total_sent + c.residual(0).double(), total_in, atol=1e-4)


def test_topk_decompress_rejects_bad_payloads(native):
    c = native.TopKCompressor(0.5)
    bad_index = struct.pack("<IIf", 1, 99, 1.0)
    with pytest.raises(RuntimeError, match="out of range"):
        c.decompress(bad_index, 4)
    with pytest.raises(RuntimeError):
        c.decompress(struct.pack("<I", 3), 4)  # claims 3 entries, carries none
