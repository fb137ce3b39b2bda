"""npu_quant_matmul on the GPU through the C ABI: int32 accumulators bit-exact, bf16/f16 outputs
within 1 ulp of the fp32-epilogue oracle (they are produced by the same fp32 operations, so 0 ulp
is what the kernels deliver; the bound asserted is the contract's 1 ulp)."""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
ULP_TOL = 1  # bf16/f16 units in the last place


def _algos(capi, M):
    return [capi.ALGO_TILE, capi.ALGO_PAIR, capi.ALGO_SIMT] + ([capi.ALGO_STREAMK] if 1 <= M <= 128 else [])


def _make(oracle, M, K, N, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    scale = torch.empty(N).uniform_(1e-3, 1e-2, generator=g)
    pt = torch.empty(M).uniform_(1e-2, 5e-2, generator=g)
    bias = (torch.randn(N, generator=g) * 0.1).to(dtype)
    return a, w, scale, pt, bias


def _compare(capi, oracle, dev, a, w, scale, pt, bias, dtype, algo, transposed=False):
    ad = a.to(dev)
    wd = w.t().contiguous().to(dev).t() if transposed else w.to(dev)
    acc = capi.quant_matmul(ad, wd, None, output_dtype=torch.int32, algo=algo)
    assert torch.equal(acc.cpu(), oracle.quant_matmul(a, w, None, output_dtype=torch.int32))
    y = capi.quant_matmul(ad, wd, scale.to(dev), pertoken_scale=None if pt is None else pt.to(dev),
                          bias=None if bias is None else bias.to(dev), output_dtype=dtype, algo=algo)
    y_ref = oracle.quant_matmul(a, w, scale, pertoken_scale=pt, bias=bias, output_dtype=dtype)
    assert oracle.bf16_ulp_distance(y.cpu(), y_ref).max().item() <= ULP_TOL


def test_config1_all_kernels(capi, oracle, dev):
    """x bf16 [128,1024] -> dynamic quant -> int8 [1024,1024] weight, per-channel scale, bf16 bias and output."""
    x, w, scale, bias = oracle.make_w8a8_inputs(128, 1024, 1024, seed=1234)
    q_ref, s_ref = oracle.dynamic_quant(x)
    q, s = capi.dynamic_quant(x.to(dev))
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    y_ref = oracle.quant_matmul(q_ref, w, scale, pertoken_scale=s_ref, bias=bias, output_dtype=torch.bfloat16)
    acc_ref = oracle.quant_matmul(q_ref, w, None, output_dtype=torch.int32)
    for algo in _algos(capi, 128) + [capi.ALGO_AUTO]:
        acc = capi.quant_matmul(q, w.to(dev), None, output_dtype=torch.int32, algo=algo)
        assert torch.equal(acc.cpu(), acc_ref), f"algo {algo}"
        y = capi.quant_matmul(q, w.to(dev), scale.to(dev), pertoken_scale=s, bias=bias.to(dev),
                              output_dtype=torch.bfloat16, algo=algo)
        assert oracle.bf16_ulp_distance(y.cpu(), y_ref).max().item() <= ULP_TOL, f"algo {algo}"


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("shape", [(128, 128, 256), (128, 32, 256), (1, 16, 16), (200, 1040, 400), (129, 4096, 272),
                                   (1024, 512, 4352), (16, 8192, 1024), (100, 272, 1008), (333, 160, 48)])
def test_shapes_tcgen05(capi, oracle, dev, shape, transposed):
    M, K, N = shape
    a, w, scale, pt, bias = _make(oracle, M, K, N, seed=M + 31 * K + 977 * N)
    for algo in _algos(capi, M):
        _compare(capi, oracle, dev, a, w, scale, pt, bias, torch.bfloat16, algo, transposed)


@pytest.mark.parametrize("shape", [(37, 77, 53), (5, 1000, 9), (64, 100, 64), (1, 1, 1)])
def test_unaligned_shapes_take_the_simt_kernel(capi, oracle, dev, shape):
    M, K, N = shape
    a, w, scale, pt, bias = _make(oracle, M, K, N, seed=11 + M)
    for transposed in (False, True):
        _compare(capi, oracle, dev, a, w, scale, pt, bias, torch.bfloat16, capi.ALGO_AUTO, transposed)
    ad, wd = a.to(dev), w.to(dev)
    if K % 16 or N % 16:
        with pytest.raises(capi.QmmError, match="16-byte"):
            capi.quant_matmul(ad, wd, None, output_dtype=torch.int32, algo=capi.ALGO_TILE)


def test_epilogue_variants(capi, oracle, dev):
    a, w, scale, pt, bias = _make(oracle, 96, 256, 512, seed=4)
    for algo in _algos(capi, 96):
        _compare(capi, oracle, dev, a, w, scale, pt, bias.to(torch.float16), torch.float16, algo)  # f16 out + bias
        _compare(capi, oracle, dev, a, w, scale, None, None, torch.bfloat16, algo)                 # no pertoken/bias
        _compare(capi, oracle, dev, a, w, scale, pt, bias.float(), torch.bfloat16, algo)           # fp32 bias
        _compare(capi, oracle, dev, a, w, scale[:1].clone(), pt, None, torch.bfloat16, algo)       # scalar scale
        bias_i = torch.randint(-1000, 1000, (512,), dtype=torch.int32)
        acc = capi.quant_matmul(a.to(dev), w.to(dev), None, bias=bias_i.to(dev), output_dtype=torch.int32, algo=algo)
        assert torch.equal(acc.cpu(), oracle.quant_matmul(a, w, None, bias=bias_i, output_dtype=torch.int32))


def test_extreme_values_fill_the_accumulator(capi, oracle, dev):
    """All operands at -128/127 with K = 28672: |acc| reaches 4.7e8, still exact in int32."""
    M, K, N = 32, 28672, 256
    a = torch.full((M, K), -128, dtype=torch.int8)
    a[::2] = 127
    w = torch.full((K, N), -128, dtype=torch.int8)
    w[:, ::3] = 127
    for algo in _algos(capi, M):
        acc = capi.quant_matmul(a.to(dev), w.to(dev), None, output_dtype=torch.int32, algo=algo)
        assert torch.equal(acc.cpu(), oracle.quant_matmul(a, w, None, output_dtype=torch.int32))


def test_empty_dimensions(capi, dev):
    a = torch.zeros((0, 64), dtype=torch.int8, device=dev)
    w = torch.zeros((64, 32), dtype=torch.int8, device=dev)
    s = torch.ones(32, device=dev)
    assert capi.quant_matmul(a, w, s).shape == (0, 32)
    # K = 0: an empty sum, the epilogue of zeros
    a = torch.zeros((4, 0), dtype=torch.int8, device=dev)
    w = torch.zeros((0, 32), dtype=torch.int8, device=dev)
    bias = torch.arange(32, dtype=torch.float32, device=dev)
    y = capi.quant_matmul(a, w, s, bias=bias, output_dtype=torch.bfloat16)
    assert torch.equal(y.float().cpu(), torch.arange(32, dtype=torch.float32).repeat(4, 1))


def test_golden_fixture(capi, oracle, dev):
    g = np.load(GOLDEN / "w8a8_small.npz")
    q, w = torch.from_numpy(g["q"]).to(dev), torch.from_numpy(g["w"]).to(dev)
    scale, s = torch.from_numpy(g["scale"]).to(dev), torch.from_numpy(g["s"]).to(dev)
    bias = torch.from_numpy(g["bias_bits"]).view(torch.bfloat16).to(dev)
    for algo in _algos(capi, 8):
        acc = capi.quant_matmul(q, w, None, output_dtype=torch.int32, algo=algo)
        assert np.array_equal(acc.cpu().numpy(), g["acc"])
        y = capi.quant_matmul(q, w, scale, pertoken_scale=s, bias=bias, output_dtype=torch.bfloat16, algo=algo)
        y_ref = torch.from_numpy(g["y_bits"]).view(torch.bfloat16)
        assert oracle.bf16_ulp_distance(y.cpu(), y_ref).max().item() <= ULP_TOL
        yh = capi.quant_matmul(q, w, scale, pertoken_scale=s, output_dtype=torch.float16, algo=algo)
        yh_ref = torch.from_numpy(g["yh_bits"]).view(torch.float16)
        assert oracle.bf16_ulp_distance(yh.cpu(), yh_ref).max().item() <= ULP_TOL


def test_streamk_scratch_is_left_clean(capi, oracle, dev):
    """Two different problems back to back through the same scratch buffer, then the buffer is all zero."""
    for seed, (M, K, N) in enumerate([(33, 4096, 7168), (8, 1040, 1008), (128, 8192, 2048), (33, 4096, 7168)]):
        a, w, scale, pt, bias = _make(oracle, M, K, N, seed=seed)
        _compare(capi, oracle, dev, a, w, scale, pt, bias, torch.bfloat16, capi.ALGO_STREAMK)
    torch.cuda.synchronize()
    checked = 0
    for key, ws in capi._workspaces.items():
        if key[0] == "w8a8":  # the W4A16 scratch keeps its slot sums; only its counters return to zero
            assert int(ws.count_nonzero().item()) == 0
            checked += 1
    assert checked >= 1


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("shape", [(17, 2048, 256), (32, 8192, 2048), (100, 4096, 1008), (128, 28672, 512)])
def test_splitk(capi, oracle, dev, shape, transposed):
    """Few output tiles, long K: the tile kernel over K slices + the reduce kernel.  Integer sums are
    order-independent, so the result is the oracle's bit for bit; the scratch is zero afterwards."""
    M, K, N = shape
    a, w, scale, pt, bias = _make(oracle, M, K, N, seed=M + N)
    _compare(capi, oracle, dev, a, w, scale, pt, bias, torch.bfloat16, capi.ALGO_SPLITK, transposed)
    _compare(capi, oracle, dev, a, w, scale, None, bias.to(torch.float16), torch.float16, capi.ALGO_SPLITK, transposed)
    torch.cuda.synchronize()
    for key, ws in capi._workspaces.items():
        if key[0] == "w8a8":
            assert int(ws.count_nonzero().item()) == 0


def _checksums(a_dev, w_dev, acc_dev):
    """Checksum of checksums: column sums and row sums of the int32 result against
    (sum of rows of x1) @ x2 and x1 @ (sum of columns of x2), all in exact integer arithmetic."""
    col = acc_dev.sum(dim=0, dtype=torch.int64).cpu().numpy()
    row = acc_dev.sum(dim=1, dtype=torch.int64).cpu().numpy()
    a_sum = a_dev.sum(dim=0, dtype=torch.int64).cpu().numpy().astype(np.float64)
    w_sum = w_dev.sum(dim=1, dtype=torch.int64).cpu().numpy().astype(np.float64)
    # fp64 dot products of integers: every partial sum stays far below 2^53
    col_ref = a_sum @ w_dev.cpu().numpy().astype(np.float64)
    row_ref = a_dev.cpu().numpy().astype(np.float64) @ w_sum
    return np.array_equal(col.astype(np.float64), col_ref) and np.array_equal(row.astype(np.float64), row_ref)


@pytest.mark.parametrize("KN", [(4096, 6144), (4096, 28672), (4096, 4096), (14336, 4096)])
def test_prefill_full_size(capi, oracle, dev, KN):
    """The four M = 8192 prefill GEMMs of the 8B-class layer (QKV, gate/up, o_proj, down_proj): oracle on a sample of rows, exact integer checksums over the whole result,
    and the dequantized output of the sampled rows within 1 ulp."""
    K, N = KN
    M = 8192
    g = torch.Generator(device=dev).manual_seed(K + N)
    a = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
    w = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)
    scale = torch.empty(N, device=dev).uniform_(1e-3, 1e-2, generator=g)
    pt = torch.empty(M, device=dev).uniform_(1e-2, 5e-2, generator=g)
    acc = capi.quant_matmul(a, w, None, output_dtype=torch.int32, algo=capi.ALGO_AUTO)
    assert _checksums(a, w, acc)
    rows = torch.arange(5, M, 131, device=dev)
    acc_ref = oracle.quant_matmul(a[rows].cpu(), w.cpu(), None, output_dtype=torch.int32)
    assert torch.equal(acc[rows].cpu(), acc_ref)
    y = capi.quant_matmul(a, w, scale, pertoken_scale=pt, output_dtype=torch.bfloat16)
    y_ref = oracle.quant_matmul(a[rows].cpu(), w.cpu(), scale.cpu(), pertoken_scale=pt[rows].cpu(),
                                output_dtype=torch.bfloat16)
    assert oracle.bf16_ulp_distance(y[rows].cpu(), y_ref).max().item() <= ULP_TOL


@pytest.mark.parametrize("M", [1, 8, 32, 128])
@pytest.mark.parametrize("KN", [(8192, 28672), (28672, 8192)])
def test_decode_full_size(capi, oracle, dev, M, KN):
    """70B-class decode GEMMs: exact integer checksums over the whole result, oracle on a sample of columns."""
    K, N = KN
    g = torch.Generator(device=dev).manual_seed(M + K)
    a = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
    w = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)
    scale = torch.empty(N, device=dev).uniform_(1e-3, 1e-2, generator=g)
    pt = torch.empty(M, device=dev).uniform_(1e-2, 5e-2, generator=g)
    acc = capi.quant_matmul(a, w, None, output_dtype=torch.int32, algo=capi.ALGO_AUTO)
    assert _checksums(a, w, acc)
    cols = torch.arange(3, N, 61, device=dev)
    w_cols = w[:, cols].cpu()
    assert torch.equal(acc[:, cols].cpu(), oracle.quant_matmul(a.cpu(), w_cols, None, output_dtype=torch.int32))
    y = capi.quant_matmul(a, w, scale, pertoken_scale=pt, output_dtype=torch.bfloat16)
    y_ref = oracle.quant_matmul(a.cpu(), w_cols, scale[cols].cpu(), pertoken_scale=pt.cpu(),
                                output_dtype=torch.bfloat16)
    assert oracle.bf16_ulp_distance(y[:, cols].cpu(), y_ref).max().item() <= ULP_TOL


@pytest.mark.parametrize("shape", [(128, 1024, 1024), (1, 512, 264), (33, 4096, 520), (300, 257, 130), (2048, 2048, 1024)])
def test_int8_requantized_output(capi, oracle, dev, shape):
    """output_dtype = int8 with offset, per-token scale and int32 bias: bit-exact against the oracle's stated
    arithmetic (fp32, one rounding per operation, ties to even, saturation), for both weight layouts; two
    shapes in a row share the scratch."""
    M, K, N = shape
    g = torch.Generator().manual_seed(M + K + N)
    x1 = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    x2 = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    # results spread over about +-60 per standard deviation, so that the clamp to [-128, 127] is exercised
    scale = torch.empty(N).uniform_(0.5, 1.5, generator=g) * (60.0 / (5373.0 * K ** 0.5))
    offset = torch.empty(N).uniform_(-20, 20, generator=g)
    pt = torch.empty(M).uniform_(0.5, 2.0, generator=g)
    bias = torch.randint(-1000, 1000, (N,), generator=g, dtype=torch.int32)
    for kw in (dict(offset=offset, pertoken_scale=pt, bias=bias), dict(), dict(offset=offset[:1])):
        want = oracle.quant_matmul(x1, x2, scale, output_dtype=torch.int8, **kw)
        got = capi.quant_matmul_int8(x1.to(dev), x2.to(dev), scale.to(dev),
                                     **{k: v.to(dev) for k, v in kw.items()})
        assert got.dtype == torch.int8 and torch.equal(got.cpu(), want)
        assert want.min().item() == -128 or want.max().item() == 127  # the clamp is exercised
    wt = x2.t().contiguous().to(dev)
    got_t = capi.quant_matmul_int8(x1.to(dev), wt.t(), scale.to(dev), offset=offset.to(dev))
    assert torch.equal(got_t.cpu(), oracle.quant_matmul(x1, x2, scale, offset=offset, output_dtype=torch.int8))
