"""npu_weight_quant_batchmatmul on the GPU against the fp64 oracle.

Tolerance (floating point, stated here): the kernels may round the dequantized weight
W = (w + offset) * scale to the activation dtype before the tensor-core product and accumulate in
fp32, and the result is rounded once to the activation dtype.  For bf16 that is a relative error of
2^-9 per weight and per output; with independent roundings the accumulated error of an output stays
below 2^-7 * rms(row) with a wide margin, so the bound asserted is
    |y - y_ref| <= 2^-8 * |y_ref| + 2^-7 * rms(y_ref row)      (bf16; 2^-11 / 2^-10 for f16).
"""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _assert_close(y, y_ref, dtype):
    rel, rms_rel = (2.0 ** -8, 2.0 ** -7) if dtype == torch.bfloat16 else (2.0 ** -11, 2.0 ** -10)
    y = y.detach().float().cpu().numpy().astype(np.float64)
    rms = np.sqrt(np.mean(y_ref ** 2, axis=1, keepdims=True))
    bound = rel * np.abs(y_ref) + rms_rel * rms + 1e-30
    worst = np.max(np.abs(y - y_ref) / bound)
    assert worst <= 1.0, f"error is {worst:.2f}x the bound"


@pytest.mark.parametrize("tensor_cores", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 256, 64, 128), (4, 256, 64, 128), (16, 1024, 512, 128), (64, 2048, 1024, 128),
                                   (3, 512, 136, 64), (17, 384, 128, 32), (130, 512, 256, 128), (8, 512, 256, 512),
                                   (33, 4096, 7168, 128), (5, 8192, 2048 + 32, 128), (64, 1024, 4096, 1024),
                                   (9, 1024, 520, 64), (12, 256, 8, 256), (16, 2048, 1024 + 72, 128)])
def test_against_oracle(capi, oracle, dev, shape, dtype, tensor_cores):
    """tensor_cores=True passes the scratch buffer (where the operands allow it -- group a multiple of 64,
    16-byte pitches -- the register-operand MMA kernel up to 16 token rows and the tcgen05 kernel beyond);
    False withholds it, which selects the CUDA-core kernel."""
    M, K, N, group = shape
    x, packed, scale, offset = oracle.make_w4a16_inputs(M, K, N, seed=M + K + N, group=group, dtype=dtype)
    y_ref = oracle.weight_quant_batchmatmul(x, packed, scale, offset, antiquant_group_size=group)
    for _ in range(2):  # the second call reuses the scratch the first one left
        y = capi.weight_quant_batchmatmul(x.to(dev), packed.to(dev), scale.to(dev), offset.to(dev), group_size=group,
                                          use_workspace=tensor_cores)
        assert y.dtype == dtype and y.shape == (M, N)
        _assert_close(y, y_ref, dtype)


def test_bias_and_no_offset(capi, oracle, dev):
    x, packed, scale, offset = oracle.make_w4a16_inputs(5, 512, 256, seed=3)
    bias = torch.randn(256).to(torch.bfloat16)
    y_ref = oracle.weight_quant_batchmatmul(x, packed, scale, None, bias=bias, antiquant_group_size=128)
    y = capi.weight_quant_batchmatmul(x.to(dev), packed.to(dev), scale.to(dev), None, bias=bias.to(dev),
                                      group_size=128)
    _assert_close(y, y_ref, torch.bfloat16)


def test_golden_fixture(capi, dev):
    g = np.load(GOLDEN / "w4a16_small.npz")
    bf = lambda k: torch.from_numpy(g[k]).view(torch.bfloat16).to(dev)  # noqa: E731
    y = capi.weight_quant_batchmatmul(bf("x_bits"), torch.from_numpy(g["packed"]).to(dev), bf("scale_bits"),
                                      bf("offset_bits"), group_size=128)
    _assert_close(y, g["y"], torch.bfloat16)


@pytest.mark.parametrize("M", [1, 16, 64])
def test_decode_full_size(capi, oracle, dev, M):
    """K = 8192, N = 28672, group 128: oracle on a sample of 8-column groups, and linearity over the
    whole output: f(2x) == 2 f(x) exactly (scaling by two commutes with every rounding)."""
    K, N, group = 8192, 28672, 128
    g = torch.Generator(device=dev).manual_seed(M)
    x = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
    scale = torch.empty((K // group, N), device=dev).uniform_(5e-3, 2e-2, generator=g).to(torch.bfloat16)
    offset = torch.empty((K // group, N), device=dev).uniform_(-1, 1, generator=g).to(torch.bfloat16)
    y = capi.weight_quant_batchmatmul(x, packed, scale, offset, group_size=group)
    y2 = capi.weight_quant_batchmatmul(x * 2, packed, scale, offset, group_size=group)
    assert torch.equal(y2.float(), y.float() * 2)
    words = torch.arange(1, N // 8, 97, device=dev)
    cols = (words[:, None] * 8 + torch.arange(8, device=dev)[None, :]).reshape(-1)
    y_ref = oracle.weight_quant_batchmatmul(x.cpu(), packed[:, words].cpu(), scale[:, cols].cpu(),
                                            offset[:, cols].cpu(), antiquant_group_size=group)
    _assert_close(y[:, cols], y_ref, torch.bfloat16)
