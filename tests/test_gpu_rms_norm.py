"""npu_rms_norm and its fusion with npu_dynamic_quant on the GPU.

Parity: the oracle restates the reference's numpy golden (test/test_custom_ops/test_npu_rms_norm.py:10-18) and
is pinned to outputs of that golden itself (tests/golden/rms_norm_reference.npz).  The device sums a row's
squares in another order than numpy's pairwise mean, so rstd and y are compared with the reference test's own
tolerance (assertRtolEqual: 1e-4 for float32, 1e-3 for float16; bf16 outputs may differ by one unit in the
last place).  The quantization half is exact: q and scale equal dynamic_quant of the y the device produced,
bit for bit, in the oracle's arithmetic and in the unfused kernels'.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
RTOL = {torch.float32: 1e-4, torch.float16: 1e-3}


def _check_y(y, y_ref, oracle):
    if y.dtype == torch.bfloat16:
        assert oracle.bf16_ulp_distance(y.cpu(), y_ref).max().item() <= 1
    else:
        a, b = y.float().cpu().numpy(), y_ref.float().numpy()
        assert np.all(np.abs(a - b) <= RTOL[y.dtype] * np.abs(b) + 1e-30)


def test_reference_golden_vectors(capi, dev):
    """The reference's own golden outputs (float32, uniform(0, 100) as in its test), through the C ABI."""
    g = np.load(GOLDEN / "rms_norm_reference.npz")
    for name in ("a", "b", "c"):
        x, gamma = torch.from_numpy(g[f"{name}_x"]).to(dev), torch.from_numpy(g[f"{name}_gamma"]).to(dev)
        y, rstd = capi.rms_norm(x, gamma, 1e-6)
        assert y.dtype == torch.float32 and rstd.shape == g[f"{name}_rstd"].shape
        np.testing.assert_allclose(y.cpu().numpy(), g[f"{name}_y"], rtol=1e-4, atol=0)
        np.testing.assert_allclose(rstd.cpu().numpy(), g[f"{name}_rstd"], rtol=1e-4, atol=0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 8), (3, 200), (128, 1024), (64, 4096), (5, 12288), (7, 1000), (2, 3, 264),
                                   (16, 14336), (4, 32768 + 64), (9, 33)])
def test_rms_norm_against_oracle(capi, oracle, dev, shape, dtype):
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(shape, generator=g) * 3).to(dtype)
    gamma = (torch.rand(shape[-1], generator=g) + 0.5).to(dtype)
    y_ref, rstd_ref = oracle.rms_norm(x, gamma, 1e-6)
    y, rstd = capi.rms_norm(x.to(dev), gamma.to(dev), 1e-6)
    assert y.dtype == dtype and y.shape == x.shape and rstd.shape == rstd_ref.shape
    np.testing.assert_allclose(rstd.cpu().numpy(), rstd_ref.numpy(), rtol=1e-5)
    _check_y(y, y_ref, oracle)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 8), (3, 200), (128, 1024), (64, 4096), (16, 14336), (7, 1000), (2, 3, 264),
                                   (4, 32768 + 64), (9, 33)])
def test_fused_equals_composition(capi, oracle, dev, shape, dtype):
    g = torch.Generator().manual_seed(sum(shape) + 1)
    x = (torch.randn(shape, generator=g) * 3).to(dtype)
    x.view(-1, shape[-1])[0].zero_()  # a row of zeros: rstd = 1/sqrt(eps), y = 0, scale 0, q 0
    gamma = (torch.rand(shape[-1], generator=g) + 0.5).to(dtype)
    xd, gd = x.to(dev), gamma.to(dev)
    q, scale, rstd = capi.rms_norm_dynamic_quant(xd, gd, 1e-6)
    y, rstd_u = capi.rms_norm(xd, gd, 1e-6)
    q_u, scale_u = capi.dynamic_quant(y)
    assert q.dtype == torch.int8 and q.shape == x.shape and scale.shape == x.shape[:-1]
    assert torch.equal(rstd, rstd_u)
    assert torch.equal(q, q_u) and torch.equal(scale, scale_u)         # the unfused kernels, bit for bit
    q_o, scale_o = oracle.dynamic_quant(y.cpu())
    assert torch.equal(q.cpu(), q_o) and torch.equal(scale.cpu(), scale_o)  # the oracle's quantization of that y
    assert torch.all(q.view(-1, shape[-1])[0] == 0) and scale.reshape(-1)[0].item() == 0.0
    # and the whole chain against the oracle composition, to the tolerance of y
    q_ref, scale_ref, _ = oracle.rms_norm_dynamic_quant(x, gamma, 1e-6)
    assert (q.cpu().int() - q_ref.int()).abs().max().item() <= 1
    np.testing.assert_allclose(scale.cpu().numpy(), scale_ref.numpy(), rtol=2.0 ** -7)


def test_full_size(capi, oracle, dev):
    """8192 x 4096 bf16 (the prefill activation): properties over the whole output, oracle on a row sample."""
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn((8192, 4096), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    gamma = (torch.rand(4096, generator=g, device=dev) + 0.5).to(torch.bfloat16)
    q, scale, rstd = capi.rms_norm_dynamic_quant(x, gamma, 1e-6)
    assert int(q.int().abs().amax(dim=1).min().item()) == 127      # every row reaches full scale
    y, _ = capi.rms_norm(x, gamma, 1e-6)
    # |y - q * scale| <= scale / 2 up to the rounding of the fp32 quotient (127 * 2^-24 of a step)
    assert torch.all((y.double() - q.double() * scale.double()[:, None]).abs() <= scale.double()[:, None] / 2 * (1 + 1e-4))
    rows = torch.arange(0, 8192, 257)
    y_ref, rstd_ref = oracle.rms_norm(x[rows].cpu(), gamma.cpu(), 1e-6)
    assert oracle.bf16_ulp_distance(y[rows].cpu(), y_ref).max().item() <= 1
    np.testing.assert_allclose(rstd[rows].cpu().numpy(), rstd_ref.numpy(), rtol=1e-5)


def test_torch_ops(pkg, oracle, dev):
    import sys

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "ascend-python_b200"))
    try:
        import torch_npu
    finally:
        sys.path.pop(0)
    x = (torch.randn((2, 5, 512)) * 2).to(torch.float16)
    gamma = (torch.rand(512) + 0.5).to(torch.float16)
    y, rstd = torch_npu.npu_rms_norm(x.to(dev), gamma.to(dev))
    y_ref, rstd_ref = oracle.rms_norm(x, gamma, 1e-6)
    assert y.shape == (2, 5, 512) and rstd.shape == (2, 5, 1) and rstd.dtype == torch.float32
    _check_y(y, y_ref, oracle)
    q, scale, rstd2 = torch_npu.npu_rms_norm_dynamic_quant(x.to(dev), gamma.to(dev), 1e-6)
    assert q.shape == (2, 5, 512) and scale.shape == (2, 5) and torch.equal(rstd2, rstd)
    q_u, s_u = torch_npu.npu_dynamic_quant(y)
    assert torch.equal(q, q_u) and torch.equal(scale, s_u)
    with pytest.raises(RuntimeError, match="gamma should have the dtype"):
        torch_npu.npu_rms_norm(x.to(dev), gamma.float().to(dev))
    with pytest.raises(RuntimeError, match="trailing dimensions"):
        torch_npu.npu_rms_norm(x.to(dev), gamma[:256].to(dev))
