"""Elementwise sm_100a kernels vs a plain PyTorch fp32/int reference.

Covers every hook the reference exposes for its Metal shaders
(accumulate, min, max, product, scale, accumulate_and_scale; reference
tests/test_local_kernels.py:66-337): all dtypes, unaligned sizes, unaligned base
pointers, 1 M elements and the integer averaging rules.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 7, 13, 97, 997, 4096, 1_000_003]
FLOATS = [torch.float32, torch.float16, torch.bfloat16, torch.float64]
INTS = [torch.int32, torch.int64, torch.uint8]


def _rand(n, dtype, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dtype.is_floating_point:
        return torch.randn(n, generator=g, dtype=torch.float32).to(dtype).to(dev)
    if dtype == torch.bool:
        return (torch.rand(n, generator=g) > 0.5).to(dev)
    hi = 7 if dtype == torch.uint8 else 1000
    lo = 0 if dtype == torch.uint8 else -1000
    return torch.randint(lo, hi, (n,), generator=g).to(dtype).to(dev)


def _ref_binary(a, b, op):
    if a.dtype == torch.bool:
        return (a | b) if op in ("sum", "max") else (a & b)
    wide = torch.float64 if a.dtype == torch.float64 else (torch.float32 if a.dtype.is_floating_point else torch.int64)
    x, y = a.to(wide), b.to(wide)
    r = {"sum": x + y, "min": torch.minimum(x, y), "max": torch.maximum(x, y), "product": x * y}[op]
    if a.dtype == torch.uint8:
        r = r % 256
    return r.to(a.dtype)


@pytest.mark.parametrize("dtype", FLOATS + INTS + [torch.bool])
@pytest.mark.parametrize("op", ["sum", "min", "max", "product"])
def test_binary_ops_match_reference(native, cuda_device, dtype, op):
    fn = {"sum": native._ew_accumulate_chunk, "min": native._ew_elementwise_min,
          "max": native._ew_elementwise_max, "product": native._ew_elementwise_product}[op]
    for n in SIZES:
        a = _rand(n, dtype, cuda_device, 1)
        b = _rand(n, dtype, cuda_device, 2)
        want = _ref_binary(a, b, op)
        got = fn(a.clone(), b)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"{op} {dtype} n={n}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int32])
def test_unaligned_base_pointer(native, cuda_device, dtype):
    # views that start 1 element into a buffer are not 16-byte aligned
    for n in (5, 1000, 65537):
        a_full = _rand(n + 1, dtype, cuda_device, 3)
        b_full = _rand(n + 1, dtype, cuda_device, 4)
        a, b = a_full[1:], b_full[1:]
        want = _ref_binary(a, b, "sum")
        head = a_full[0].clone()
        native._ew_accumulate_chunk(a, b)
        torch.cuda.synchronize()
        assert torch.equal(a, want)
        assert torch.equal(a_full[0], head), "wrote before the view"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64])
def test_scale_and_accumulate_scale_float(native, cuda_device, dtype):
    for n in SIZES:
        a = _rand(n, dtype, cuda_device, 5)
        b = _rand(n, dtype, cuda_device, 6)
        wide = torch.float64 if dtype == torch.float64 else torch.float32
        want = (a.to(wide) * 0.25).to(dtype)
        got = native._ew_scale_inplace(a.clone(), 0.25)
        assert torch.equal(got, want), f"scale {dtype} {n}"
        if dtype != torch.float64:
            want2 = ((a.to(torch.float32) + b.to(torch.float32)) * 0.5).to(dtype)
            got2 = native._ew_accumulate_and_scale(a.clone(), b, 0.5)
            assert torch.equal(got2, want2), f"accscale {dtype} {n}"


def test_integer_average_semantics(native, cuda_device):
    # i32 rounds to nearest (halves away from zero); i64 and u8 truncate towards zero.
    i32 = torch.tensor([7, -7, 5, -5, 1, 0, 10, -10], dtype=torch.int32, device=cuda_device)
    assert native._ew_scale_inplace(i32.clone(), 0.5).tolist() == [4, -4, 3, -3, 1, 0, 5, -5]
    i64 = torch.tensor([7, -7, 5, -5, 1, 0, 10, -10], dtype=torch.int64, device=cuda_device)
    assert native._ew_scale_inplace(i64.clone(), 0.5).tolist() == [3, -3, 2, -2, 0, 0, 5, -5]
    u8 = torch.tensor([7, 5, 1, 0, 255], dtype=torch.uint8, device=cuda_device)
    assert native._ew_scale_inplace(u8.clone(), 0.5).tolist() == [3, 2, 0, 0, 127]


def test_cast_roundtrip(native, cuda_device):
    x = torch.randn(100_003, device=cuda_device)
    for dt in (torch.float16, torch.bfloat16):
        y = native._cast(x, dt, 1.0)
        assert torch.equal(y, x.to(dt))
        z = native._cast(y, torch.float32, 2.0)
        assert torch.equal(z, y.float() * 2.0)


def test_metal_aliases_point_to_cuda_kernels(native):
    assert native._metal_accumulate_chunk is native._ew_accumulate_chunk
    assert native._metal_scale_inplace is native._ew_scale_inplace


def test_rejects_unsupported_dtype(native, cuda_device):
    a = torch.zeros(4, dtype=torch.int8, device=cuda_device)
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        native._ew_accumulate_chunk(a, a)
