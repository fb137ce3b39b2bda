"""Prepacked W4A16 path on the GPU: the layout pass round-trips bit-exactly, and the matmul over the
prepacked stream meets the same bound against the fp64 oracle as the stock entry point.

Tolerance (floating point, stated here).  The kernel rounds every weight W = fma(w, scale, offset*scale) once
to the activation dtype before the tensor-core product (a relative perturbation of at most u = 2^-9 for bf16,
2^-12 for f16), accumulates in fp32 and rounds the output once (u again).  The error of an output is therefore
a sum of K independent terms x[m,k] * dW[k,n]; its standard deviation is about 0.45 u * rss with
rss[m,n] = sqrt(sum_k (x[m,k] * W[k,n])^2), the natural scale of accumulated rounding error (a bound relative
to the row's rms would be too tight for columns whose scales are above average and too loose for the others).
The bound asserted is
    |y - y_ref| <= 2 u * |y_ref| + 8 u * rss[m,n]             (u = 2^-9 bf16, 2^-12 f16)
i.e. the output rounding plus about 18 standard deviations of the accumulated weight rounding.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rss(oracle, x, packed_w, scale, offset, group):
    W = oracle.antiquant_weight(packed_w, scale, offset, group)
    return np.sqrt((x.double().numpy() ** 2) @ (W ** 2))


def _assert_close(y, y_ref, rss, dtype):
    u = 2.0 ** -9 if dtype == torch.bfloat16 else 2.0 ** -12
    y = y.detach().float().cpu().numpy().astype(np.float64)
    bound = 2 * u * np.abs(y_ref) + 8 * u * rss + 1e-30
    worst = np.max(np.abs(y - y_ref) / bound)
    assert worst <= 1.0, f"error is {worst:.2f}x the bound"


@pytest.mark.parametrize("shape", [(128, 64, 128), (256, 136, 128), (1024, 4096, 256), (8192, 2048 + 32, 128),
                                   (384, 8, 384)])
def test_prepack_round_trip(capi, oracle, dev, shape):
    """unpack(prepack(w)) == w, and the scale / offset*scale rows of every block are what the layout says."""
    K, N, group = shape
    _, packed_w, scale, offset = oracle.make_w4a16_inputs(1, K, N, seed=K + N, group=group)
    buf = capi.w4a16_prepack(packed_w.to(dev), scale.to(dev), offset.to(dev), group_size=group)
    tiles, chunks = (N + 127) // 128, K // 128
    padded = 2 * ((chunks + 1) // 2)  # blocks along K come in pairs; an odd count is padded with a zero block
    assert buf.numel() == capi.w4a16_prepack_size(N, K, group) == tiles * padded * 8704
    back = capi.w4a16_unpack_weight(buf, N, K)
    assert torch.equal(back.cpu(), packed_w)
    blocks = buf.cpu().view(-1, 8704)
    so = blocks[:, 8192:].contiguous().view(torch.bfloat16).view(tiles, padded, 2, 128)
    s_ref = torch.zeros((padded, tiles * 128), dtype=torch.bfloat16)
    t_ref = torch.zeros_like(s_ref)
    rows = torch.arange(chunks) * 128 // group
    s_ref[:chunks, :N] = scale[rows]
    t_ref[:chunks, :N] = (offset[rows].float() * scale[rows].float()).to(torch.bfloat16)
    assert torch.equal(so[:, :, 0, :].permute(1, 0, 2).reshape(padded, -1), s_ref)
    assert torch.equal(so[:, :, 1, :].permute(1, 0, 2).reshape(padded, -1), t_ref)
    if padded > chunks:
        assert not blocks.view(tiles, padded, 8704)[:, chunks:].any()


def test_prepack_refusals(capi, dev):
    assert capi.w4a16_prepack_size(256, 192, 64) == 0      # K not a multiple of 128
    assert capi.w4a16_prepack_size(256, 256, 64) == 0      # group not a multiple of 128
    assert capi.w4a16_prepack_size(256, 512, 0) > 0        # per-channel: group = K
    w = torch.zeros((192, 32), dtype=torch.int32, device=dev)
    s = torch.ones((1, 256), dtype=torch.bfloat16, device=dev)
    with pytest.raises(capi.QmmError):
        capi.w4a16_prepack(w, s, None, group_size=0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 256, 64, 128), (2, 384, 200, 128), (2, 8192, 1024, 256), (4, 256, 128, 128), (16, 1024, 512, 128), (64, 2048, 1024, 128),
                                   (130, 512, 256, 128), (8, 512, 256, 512), (33, 4096, 7168, 128),
                                   (5, 8192, 2048 + 32, 128), (64, 1024, 4096, 1024), (12, 256, 8, 256),
                                   (16, 2048, 1024 + 72, 128), (48, 1152, 640, 384)])
def test_against_oracle(capi, oracle, dev, shape, dtype):
    M, K, N, group = shape
    x, packed_w, scale, offset = oracle.make_w4a16_inputs(M, K, N, seed=M + K + N, group=group, dtype=dtype)
    y_ref = oracle.weight_quant_batchmatmul(x, packed_w, scale, offset, antiquant_group_size=group)
    rss = _rss(oracle, x, packed_w, scale, offset, group)
    buf = capi.w4a16_prepack(packed_w.to(dev), scale.to(dev), offset.to(dev), group_size=group)
    for _ in range(2):  # the second call reuses the scratch the first one left
        y = capi.weight_quant_batchmatmul_prepacked(x.to(dev), buf, N)
        assert y.dtype == dtype and y.shape == (M, N)
        _assert_close(y, y_ref, rss, dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 256, 64, 128), (2, 384, 200, 128), (2, 8192, 1024, 256), (1, 4096, 7168, 128),
                                   (2, 1024, 4096, 1024)])
def test_one_or_two_tokens_meet_the_stock_tolerance(capi, oracle, dev, shape, dtype):
    """One or two tokens take the integer dot-product kernel, which never rounds a weight: it meets the bound of
    the stock-layout kernels, |y - y_ref| <= 2 u |y_ref| + 2^-7 (u / 2^-9) rms(row), not only the rss bound."""
    M, K, N, group = shape
    x, packed_w, scale, offset = oracle.make_w4a16_inputs(M, K, N, seed=M + K + N, group=group, dtype=dtype)
    y_ref = oracle.weight_quant_batchmatmul(x, packed_w, scale, offset, antiquant_group_size=group)
    buf = capi.w4a16_prepack(packed_w.to(dev), scale.to(dev), offset.to(dev), group_size=group)
    y = capi.weight_quant_batchmatmul_prepacked(x.to(dev), buf, N).float().cpu().numpy()
    u = 2.0 ** -9 if dtype == torch.bfloat16 else 2.0 ** -12
    rms = np.sqrt(np.mean(y_ref ** 2, axis=1, keepdims=True))
    assert np.all(np.abs(y - y_ref) <= 2 * u * np.abs(y_ref) + 2.0 ** -7 * (u / 2.0 ** -9) * rms + 1e-30)


def test_bias_and_no_offset(capi, oracle, dev):
    x, packed_w, scale, _ = oracle.make_w4a16_inputs(5, 512, 256, seed=3)
    bias = torch.randn(256).to(torch.bfloat16)
    y_ref = oracle.weight_quant_batchmatmul(x, packed_w, scale, None, bias=bias, antiquant_group_size=128)
    buf = capi.w4a16_prepack(packed_w.to(dev), scale.to(dev), None, group_size=128)
    y = capi.weight_quant_batchmatmul_prepacked(x.to(dev), buf, 256, bias=bias.to(dev))
    _assert_close(y, y_ref, _rss(oracle, x, packed_w, scale, None, 128), torch.bfloat16)


@pytest.mark.parametrize("M", [1, 2, 16, 64])
def test_decode_full_size(capi, oracle, dev, M):
    """K = 8192, N = 28672, group 128: oracle on a sample of 8-column groups, linearity over the whole output
    (f(2x) == 2 f(x) exactly: scaling by two commutes with every rounding), and run-to-run identity."""
    K, N, group = 8192, 28672, 128
    g = torch.Generator(device=dev).manual_seed(M)
    x = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    packed_w = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
    scale = torch.empty((K // group, N), device=dev).uniform_(5e-3, 2e-2, generator=g).to(torch.bfloat16)
    offset = torch.empty((K // group, N), device=dev).uniform_(-1, 1, generator=g).to(torch.bfloat16)
    buf = capi.w4a16_prepack(packed_w, scale, offset, group_size=group)
    assert torch.equal(capi.w4a16_unpack_weight(buf, N, K), packed_w)
    y = capi.weight_quant_batchmatmul_prepacked(x, buf, N)
    y_again = capi.weight_quant_batchmatmul_prepacked(x, buf, N)
    assert torch.equal(y, y_again)
    y2 = capi.weight_quant_batchmatmul_prepacked(x * 2, buf, N)
    assert torch.equal(y2.float(), y.float() * 2)
    words = torch.arange(1, N // 8, 97, device=dev)
    cols = (words[:, None] * 8 + torch.arange(8, device=dev)[None, :]).reshape(-1)
    y_ref = oracle.weight_quant_batchmatmul(x.cpu(), packed_w[:, words].cpu(), scale[:, cols].cpu(),
                                            offset[:, cols].cpu(), antiquant_group_size=group)
    rss = _rss(oracle, x.cpu(), packed_w[:, words].cpu(), scale[:, cols].cpu(), offset[:, cols].cpu(), group)
    _assert_close(y[:, cols], y_ref, rss, torch.bfloat16)
