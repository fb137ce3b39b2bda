"""The torch custom ops (torch.ops.npu.* / torch_npu.*) on CUDA tensors: same results as the C ABI
and the oracle, output shapes and dtypes, and the argument checks of the host functions."""
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
PKG_DIR = Path(__file__).resolve().parent.parent / "ascend-python_b200"


@pytest.fixture(scope="module")
def torch_npu(pkg):
    sys.path.insert(0, str(PKG_DIR))
    try:
        import torch_npu as mod
    finally:
        sys.path.pop(0)
    return mod


def test_dynamic_quant_then_quant_matmul(torch_npu, oracle, dev):
    x, w, scale, bias = oracle.make_w8a8_inputs(128, 1024, 1024, seed=1234)
    q_ref, s_ref = oracle.dynamic_quant(x)
    y_ref = oracle.quant_matmul(q_ref, w, scale, pertoken_scale=s_ref, bias=bias, output_dtype=torch.bfloat16)
    q, s = torch_npu.npu_dynamic_quant(x.to(dev))
    assert q.dtype == torch.int8 and s.dtype == torch.float32 and s.shape == (128,)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    y = torch_npu.npu_quant_matmul(q, w.to(dev), scale.to(dev), pertoken_scale=s, bias=bias.to(dev),
                                   output_dtype=torch.bfloat16)
    assert y.dtype == torch.bfloat16 and y.shape == (128, 1024)
    assert oracle.bf16_ulp_distance(y.cpu(), y_ref).max().item() <= 1
    acc = torch_npu.npu_quant_matmul(q, w.to(dev), scale.to(dev), output_dtype=torch.int32)
    assert torch.equal(acc.cpu(), oracle.quant_matmul(q_ref, w, None, output_dtype=torch.int32))
    # the transposed view of an [N,K] weight is consumed as stored
    wt = w.t().contiguous().to(dev)
    y_t = torch_npu.npu_quant_matmul(q, wt.t(), scale.to(dev), pertoken_scale=s, bias=bias.to(dev),
                                     output_dtype=torch.bfloat16)
    assert torch.equal(y_t, y)


def test_leading_dimensions(torch_npu, oracle, dev):
    x = torch.randn((2, 3, 256)).to(torch.bfloat16)
    q, s = torch_npu.npu_dynamic_quant(x.to(dev))
    q_ref, s_ref = oracle.dynamic_quant(x)
    assert q.shape == (2, 3, 256) and s.shape == (2, 3)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    w = torch.randint(-127, 128, (256, 64), dtype=torch.int8)
    scale = torch.rand(64) * 1e-2
    y = torch_npu.npu_quant_matmul(q, w.to(dev), scale.to(dev), pertoken_scale=s.reshape(-1),
                                   output_dtype=torch.float16)
    assert y.shape == (2, 3, 64)
    y_ref = oracle.quant_matmul(q_ref.reshape(6, 256), w, scale, pertoken_scale=s_ref.reshape(-1),
                                output_dtype=torch.float16)
    assert oracle.bf16_ulp_distance(y.reshape(6, 64).cpu(), y_ref).max().item() <= 1


def test_decode_shape_uses_cached_scratch(torch_npu, oracle, dev):
    g = torch.Generator().manual_seed(1)
    a = torch.randint(-127, 128, (8, 2048), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (2048, 3072), generator=g, dtype=torch.int8)
    scale = torch.rand(3072, generator=g) * 1e-2
    ref = oracle.quant_matmul(a, w, scale, output_dtype=torch.bfloat16)
    for _ in range(3):
        y = torch_npu.npu_quant_matmul(a.to(dev), w.to(dev), scale.to(dev), output_dtype=torch.bfloat16)
        assert oracle.bf16_ulp_distance(y.cpu(), ref).max().item() <= 1


def test_weight_quant_batchmatmul(torch_npu, oracle, dev):
    import numpy as np

    x, packed, scale, offset = oracle.make_w4a16_inputs(4, 512, 256, seed=2)
    y = torch_npu.npu_weight_quant_batchmatmul(x.to(dev), packed.to(dev), scale.to(dev), offset.to(dev),
                                               antiquant_group_size=128)
    y_ref = oracle.weight_quant_batchmatmul(x, packed, scale, offset, antiquant_group_size=128)
    rms = np.sqrt(np.mean(y_ref ** 2, axis=1, keepdims=True))
    assert np.all(np.abs(y.float().cpu().numpy() - y_ref) <= 2.0 ** -8 * np.abs(y_ref) + 2.0 ** -7 * rms)


def test_argument_checks(torch_npu, dev):
    q = torch.zeros((4, 64), dtype=torch.int8, device=dev)
    w = torch.zeros((64, 32), dtype=torch.int8, device=dev)
    s = torch.ones(32, device=dev)
    with pytest.raises(RuntimeError, match="K-axis"):
        torch_npu.npu_quant_matmul(q, torch.zeros((48, 32), dtype=torch.int8, device=dev), s,
                                   output_dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="int8"):
        torch_npu.npu_quant_matmul(q.float(), w, s, output_dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="offset"):
        torch_npu.npu_quant_matmul(q, w, s, offset=torch.zeros(32, device=dev), output_dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="output_dtype"):
        torch_npu.npu_quant_matmul(q, w, s, output_dtype=torch.float32)
    with pytest.raises(RuntimeError, match="pertoken_scale"):
        torch_npu.npu_quant_matmul(q, w, s, pertoken_scale=torch.ones(5, device=dev), output_dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="bfloat16 or float16"):
        torch_npu.npu_dynamic_quant(torch.zeros((2, 8), device=dev))
    with pytest.raises(RuntimeError, match="smooth_scales"):
        torch_npu.npu_dynamic_quant(torch.zeros((2, 8), dtype=torch.bfloat16, device=dev),
                                    smooth_scales=torch.ones(8, dtype=torch.bfloat16, device=dev))
    with pytest.raises(RuntimeError, match="not registered"):
        torch_npu.npu_mm_all_reduce_base(q, w, "no-such-communicator", dequant_scale=s)
    with pytest.raises(RuntimeError, match="reduce_op"):
        torch_npu.npu_mm_all_reduce_base(q, w, "c", reduce_op="max", dequant_scale=s)
    with pytest.raises(RuntimeError, match="2D"):
        torch_npu.npu_mm_all_reduce_base(q.reshape(2, 2, 64), w, "c", dequant_scale=s)


def test_weight_quant_batchmatmul_prepack_cache(torch_npu, capi, oracle, dev):
    """One or two token rows and more than eight: the operator prepacks the weight once (pointer-keyed cache) and
    runs the kernels over the prepacked stream; an in-place update of the weight invalidates the entry; three to
    eight rows keep the stock layout."""
    x, w, scale, offset = oracle.make_w4a16_inputs(16, 1024, 512, seed=9)
    _, w2, _, _ = oracle.make_w4a16_inputs(16, 1024, 512, seed=10)
    xd, wd, sd, od = x.to(dev), w.to(dev), scale.to(dev), offset.to(dev)
    y1 = torch_npu.npu_weight_quant_batchmatmul(xd, wd, sd, od, antiquant_group_size=128)
    direct = capi.weight_quant_batchmatmul_prepacked(xd, capi.w4a16_prepack(wd, sd, od, group_size=128), 512)
    assert torch.equal(y1, direct)
    assert torch.equal(torch_npu.npu_weight_quant_batchmatmul(xd, wd, sd, od, antiquant_group_size=128), y1)
    wd.copy_(w2.to(dev))  # same storage, new contents: the version counter moves, the entry is re-made
    y3 = torch_npu.npu_weight_quant_batchmatmul(xd, wd, sd, od, antiquant_group_size=128)
    direct3 = capi.weight_quant_batchmatmul_prepacked(xd, capi.w4a16_prepack(wd, sd, od, group_size=128), 512)
    assert torch.equal(y3, direct3) and not torch.equal(y3, y1)
    y_small = torch_npu.npu_weight_quant_batchmatmul(xd[:4], wd, sd, od, antiquant_group_size=128)
    assert torch.equal(y_small, capi.weight_quant_batchmatmul(xd[:4].contiguous(), wd, sd, od, group_size=128))
    y_one = torch_npu.npu_weight_quant_batchmatmul(xd[:1], wd, sd, od, antiquant_group_size=128)
    assert torch.equal(y_one, capi.weight_quant_batchmatmul_prepacked(
        xd[:1].contiguous(), capi.w4a16_prepack(wd, sd, od, group_size=128), 512))
    # a group the prepacked format does not cover (64) stays on the stock path and stays correct
    x5, w5, s5, o5 = oracle.make_w4a16_inputs(16, 512, 256, seed=11, group=64)
    y5 = torch_npu.npu_weight_quant_batchmatmul(x5.to(dev), w5.to(dev), s5.to(dev), o5.to(dev), antiquant_group_size=64)
    assert torch.equal(y5, capi.weight_quant_batchmatmul(x5.to(dev), w5.to(dev), s5.to(dev), o5.to(dev), group_size=64))


def test_quant_matmul_int8_output_and_offset(torch_npu, oracle, dev):
    """output_dtype=None (or torch.int8) is the requantized int8 output; offset applies to it alone."""
    g = torch.Generator().manual_seed(5)
    x1 = torch.randint(-127, 128, (2, 9, 256), generator=g, dtype=torch.int8)
    x2 = torch.randint(-127, 128, (256, 136), generator=g, dtype=torch.int8)
    scale = torch.empty(136).uniform_(1e-4, 4e-4, generator=g)
    offset = torch.empty(136).uniform_(-10, 10, generator=g)
    want = oracle.quant_matmul(x1.reshape(18, 256), x2, scale, offset=offset, output_dtype=torch.int8).reshape(2, 9, 136)
    got = torch_npu.npu_quant_matmul(x1.to(dev), x2.to(dev), scale.to(dev), offset=offset.to(dev))
    assert got.dtype == torch.int8 and got.shape == (2, 9, 136) and torch.equal(got.cpu(), want)
    got2 = torch_npu.npu_quant_matmul(x1.to(dev), x2.to(dev), scale.to(dev), offset=offset.to(dev),
                                      output_dtype=torch.int8)
    assert torch.equal(got2, got)
    with pytest.raises(RuntimeError, match="offset only applies to an int8 output"):
        torch_npu.npu_quant_matmul(x1.to(dev), x2.to(dev), scale.to(dev), offset=offset.to(dev),
                                   output_dtype=torch.bfloat16)
