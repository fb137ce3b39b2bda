"""npu_dynamic_quant on the GPU against the CPU oracle: bit-exact int8 values and fp32 scales."""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _check(capi, oracle, x, dev):
    q_ref, s_ref = oracle.dynamic_quant(x)
    q, s = capi.dynamic_quant(x.to(dev))
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))  # bitwise, -0.0 and all
    return q, s


def test_config1(capi, oracle, dev):
    x, _, _, _ = oracle.make_w8a8_inputs(128, 1024, 8, seed=1234)
    _check(capi, oracle, x, dev)


@pytest.mark.parametrize("shape", [(1, 8), (3, 8192), (1, 28672), (64, 14336), (257, 4096), (5, 100), (7, 33),
                                   (2, 40000), (1000, 16), (9, 2056), (130, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_shapes(capi, oracle, dev, shape, dtype):
    g = torch.Generator().manual_seed(shape[0] * 7919 + shape[1])
    x = (torch.randn(shape, generator=g) * 3).to(dtype)
    if shape[0] > 2:
        x[1].zero_()  # an all-zero token: scale 0, q 0
    _check(capi, oracle, x, dev)


def test_value_edge_cases(capi, oracle, dev):
    x = torch.zeros((6, 64), dtype=torch.bfloat16)
    x[0, :] = 1.0                      # every element is the maximum
    x[1, 3] = -65280.0                 # large magnitude, negative maximum
    x[2, 0] = 1e-30                    # tiny values: scale far below 1e-30 takes the exact-division branch
    x[2, 1] = -5e-31
    x[3, :] = torch.arange(64) * 0.5   # many exact .5 quotients: round-half-to-even
    x[3, 63] = 127.0
    x[4, 7] = 3.0
    x[4, 8] = 1.5
    _check(capi, oracle, x, dev)
    # quotients that sit next to rounding ties
    g = torch.Generator().manual_seed(5)
    base = torch.randint(-126, 127, (512, 256), generator=g).float() + 0.5
    base[:, 0] = 127.0
    _check(capi, oracle, base.to(torch.bfloat16), dev)
    _check(capi, oracle, (base * 0.37).to(torch.float16), dev)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_every_mantissa_against_every_maximum(capi, oracle, dev, dtype):
    """Short-mantissa inputs make exact ties x / scale = n + 1/2 common.  Row r has the maximum (128 + r) / 64
    and holds every 8-bit significand at eight exponents and both signs, so all ratios x / amax of two such
    numbers occur - ties, near ties and all; results must equal the IEEE divisions of the oracle bit for bit."""
    mant = torch.arange(128, 256, dtype=torch.float32)
    exps = torch.tensor([2.0 ** -e for e in range(6, 14)])
    vals = (mant[None, :] * exps[:, None]).reshape(-1)            # 1024 values in (0, 4)
    vals = torch.cat([vals, -vals])                                # 2048 columns
    rows = []
    for r in range(128):
        amax = (128 + r) / 64.0
        row = vals.clamp(-amax, amax).clone()
        row[0] = amax
        rows.append(row)
    x = torch.stack(rows).to(dtype)
    _check(capi, oracle, x, dev)
    # the same ratios at a scale whose reciprocal is not a power of two times a short number
    _check(capi, oracle, (x.float() * 0.7431).to(dtype), dev)
    _check(capi, oracle, (x.float() * 1.0e-3).to(dtype), dev)


def test_every_f16_significand_pair(capi, oracle, dev):
    """All 1024 f16 significands as the row maximum against all 1024 significands of x at eight exponents and
    both signs: with the quotient's significand independent of the exponents, this is every case the f16
    path can meet.  16.8 M elements, bit-exact against IEEE division."""
    mant = torch.arange(1024, 2048, dtype=torch.float32)                      # significands 1.0 .. 2 - 2^-10
    exps = torch.tensor([2.0 ** -e for e in range(9, 17)])
    vals = (mant[None, :] * exps[:, None]).reshape(-1)                         # 8192 values in (0, 4)
    vals = torch.cat([vals, -vals])                                            # 16384 columns
    amax = (mant / 512.0)[:, None]                                             # 1024 row maxima in [2, 4)
    x = torch.minimum(torch.maximum(vals[None, :], -amax), amax)
    x[:, 0] = amax[:, 0]
    _check(capi, oracle, x.to(torch.float16), dev)


def test_strided_rows_and_empty(capi, oracle, dev):
    lib = capi.lib()
    x = torch.randn((16, 256), dtype=torch.float32).to(torch.bfloat16)
    xd = x.to(dev)
    q = torch.zeros((16, 128), dtype=torch.int8, device=dev)
    s = torch.zeros(16, dtype=torch.float32, device=dev)
    # quantize the left half of every row: row stride 256, 128 columns
    capi.check(lib.qmm_dynamic_quant(xd.data_ptr(), capi.DTYPE_BF16, 16, 128, 256, q.data_ptr(), 128, s.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream), "qmm_dynamic_quant")
    q_ref, s_ref = oracle.dynamic_quant(x[:, :128].contiguous())
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    q0, s0 = capi.dynamic_quant(torch.zeros((0, 64), dtype=torch.bfloat16, device=dev))
    assert q0.shape == (0, 64) and s0.shape == (0,)
    q1, s1 = capi.dynamic_quant(torch.zeros((4, 0), dtype=torch.bfloat16, device=dev))
    assert q1.shape == (4, 0) and s1.cpu().tolist() == [0.0] * 4


def test_golden_fixture(capi, dev):
    g = np.load(GOLDEN / "w8a8_small.npz")
    x = torch.from_numpy(g["x_bits"]).view(torch.bfloat16)
    q, s = capi.dynamic_quant(x.to(dev))
    assert np.array_equal(q.cpu().numpy(), g["q"]) and np.array_equal(s.cpu().numpy(), g["s"])


def test_full_size_properties(capi, oracle, dev):
    """Prefill activation sizes [8192, 4096] and [8192, 14336]: oracle on a row sample, and for every row
    max|q| == 127, |x - q*scale| <= scale/2 (+ fp32 slack) and re-quantizing q*scale returns q."""
    for cols in (4096, 14336):
        g = torch.Generator(device=dev).manual_seed(cols)
        x = torch.randn((8192, cols), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        q, s = capi.dynamic_quant(x)
        rows = torch.arange(0, 8192, 37)
        q_ref, s_ref = oracle.dynamic_quant(x[rows.to(dev)].cpu())
        assert torch.equal(q[rows.to(dev)].cpu(), q_ref) and torch.equal(s[rows.to(dev)].cpu(), s_ref)
        assert torch.all(q.abs().amax(dim=1) == 127)
        err = (x.float() - q.float() * s[:, None]).abs()
        assert torch.all(err <= s[:, None] * 0.50002)  # half a step + fp32 rounding of x/s and q*s
        del x, err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", [8, 1024, 4096 + 8, 33])
def test_non_finite_rows(capi, oracle, dev, dtype, cols):
    """A row with an infinity: infinite scale, every element 0.  A row with a NaN: NaN scale, every element 0.
    Neighbouring rows are untouched (both the vector kernel and the any-alignment kernel)."""
    g = torch.Generator().manual_seed(cols)
    x = torch.randn((6, cols), generator=g).to(dtype)
    x[1, cols // 2] = float("inf")
    x[3, cols - 1] = float("nan")
    x[4, 0] = float("-inf")
    q_ref, s_ref = oracle.dynamic_quant(x)
    q, s = capi.dynamic_quant(x.to(dev))
    assert torch.equal(q.cpu(), q_ref)
    s, s_ref = s.cpu(), s_ref
    assert torch.isnan(s[3]) and torch.isnan(s_ref[3])
    keep = [0, 1, 2, 4, 5]
    assert torch.equal(s[keep], s_ref[keep]) and torch.isinf(s[1]) and torch.isinf(s[4])
    assert not q[1].any() and not q[3].any() and not q[4].any()
