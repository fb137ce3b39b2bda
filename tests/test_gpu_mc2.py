"""npu_mm_reduce_scatter_base and npu_all_gather_base_mm on the GPU.

Parity: the oracle restates the reference's golden functions (test/test_custom_ops/test_mm_reduce_scatter_base.py:69-81,
test_all_gather_base_mm.py:72-78) and is pinned to their outputs (tests/golden/mc2_reference.npz).  The device
accumulates each rank's products in fp32 on the tensor cores (another order than the host BLAS), adds the ranks'
fp32 partials in rank order and rounds once, as the golden does.  Tolerance, stated here: the reference test's own
(assertEqual on float16 results: relative and absolute 1e-3); for bfloat16 one unit in the last place (2^-7
relative) with the same absolute term, which covers sums that cancel to nearly zero.  The gathered matrix is a copy
and must be identical.
"""
import ctypes
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
PKG_DIR = ROOT / "ascend-python_b200"
GOLDEN = Path(__file__).resolve().parent / "golden"


def _close(got, want):
    rtol = 1e-3 if want.dtype == torch.float16 else 2.0 ** -7
    return torch.allclose(got.float().cpu(), want.float(), rtol=rtol, atol=1e-3)


def _golden_module():
    spec = importlib.util.spec_from_file_location("make_mc2_golden", GOLDEN / "make_mc2_golden.py")
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    return mk


@pytest.fixture(scope="module")
def torch_npu(pkg):
    sys.path.insert(0, str(PKG_DIR))
    try:
        import torch_npu as mod
    finally:
        sys.path.pop(0)
    return mod


@pytest.fixture()
def solo(capi):
    lib = capi.lib()
    uid = ctypes.create_string_buffer(capi.UNIQUE_ID_BYTES)
    capi.check(lib.qmm_comm_unique_id(uid), "qmm_comm_unique_id")
    capi.check(lib.qmm_comm_init_rank(b"solo_mc2", uid, 1, 0), "qmm_comm_init_rank")
    yield "solo_mc2"
    capi.check(lib.qmm_comm_destroy(b"solo_mc2"), "qmm_comm_destroy")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(128, 512, 256), (16, 512, 256), (512, 1024, 768), (1000, 264, 520), (3, 40, 24),
                                   (130, 96, 136), (2048, 4096, 1024), (7, 5, 3)])
def test_single_rank_is_the_matmul(torch_npu, oracle, dev, solo, shape, dtype):
    """One rank: both operators are the bf16/f16 matmul alone (tcgen05 kernel for 16-byte aligned operands, CUDA
    cores otherwise), for a row-major x2 and for the transposed view of a row-major [N, K] matrix, with a bias."""
    M, K, N = shape
    g = torch.Generator().manual_seed(M + K + N)
    x1 = (torch.rand((M, K), generator=g) * 2 - 1).to(dtype)
    x2 = (torch.rand((K, N), generator=g) * 2 - 1).to(dtype)
    bias = (torch.rand(N, generator=g) - 0.5).to(dtype)
    want = oracle.mm_reduce_scatter([x1], [x2], 1, bias=bias)[0]
    got = torch_npu.npu_mm_reduce_scatter_base(x1.to(dev), x2.to(dev), solo, 1, reduce_op="sum", bias=bias.to(dev))
    assert got.dtype == dtype and got.shape == (M, N)
    assert _close(got, want)
    x2t = x2.t().contiguous().to(dev)  # [N, K] row-major; its transposed view is the K-major operand
    got_t = torch_npu.npu_mm_reduce_scatter_base(x1.to(dev), x2t.t(), solo, 1, bias=bias.to(dev))
    assert _close(got_t, want)
    outs, gathered = oracle.all_gather_mm([x1], [x2], 1)
    y, gout = torch_npu.npu_all_gather_base_mm(x1.to(dev), x2.to(dev), solo, 1)
    assert torch.equal(gout.cpu(), gathered) and _close(y, outs[0])
    y2, gnone = torch_npu.npu_all_gather_base_mm(x1.to(dev), x2.to(dev), solo, 1, gather_output=False)
    assert gnone.numel() == 0 and torch.equal(y2, y)


def test_argument_checks(torch_npu, dev, solo):
    a = torch.zeros((6, 8), dtype=torch.float16, device=dev)
    b = torch.zeros((8, 4), dtype=torch.float16, device=dev)
    with pytest.raises(RuntimeError, match="world_size should be greater than 0"):
        torch_npu.npu_mm_reduce_scatter_base(a, b, solo, 0)
    with pytest.raises(RuntimeError, match="Both inputs of mm are required to be 2D"):
        torch_npu.npu_mm_reduce_scatter_base(a[0], b, solo, 1)
    with pytest.raises(RuntimeError, match="The K-axis in the two inputs of Matmul must be equal"):
        torch_npu.npu_mm_reduce_scatter_base(a, b[:4], solo, 1)
    with pytest.raises(RuntimeError, match="does not match the size of communicator"):
        torch_npu.npu_mm_reduce_scatter_base(a, b, solo, 2)
    with pytest.raises(RuntimeError, match="not registered"):
        torch_npu.npu_all_gather_base_mm(a, b, "no-such-comm", 1)
    with pytest.raises(RuntimeError, match="gather_index=0"):
        torch_npu.npu_all_gather_base_mm(a, b, solo, 1, gather_index=1)
    with pytest.raises(RuntimeError, match="reduce_op"):
        torch_npu.npu_mm_reduce_scatter_base(a, b, solo, 1, reduce_op="max")


def _rank_main(rank, world, port, c2p):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(PKG_DIR))
    import torch.distributed as dist
    import torch_npu

    mk = _golden_module()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        hcom = torch_npu.get_comm_name()
        rs_x1, rs_x2, ag_x1, ag_x2 = mk.mc2_inputs(world)
        res = {}
        # the reference tests' own cases, twice in a row (the second call reuses the regions)
        for rep in range(2):
            res[f"rs{rep}"] = torch_npu.npu_mm_reduce_scatter_base(rs_x1[rank].to(dev), rs_x2[rank].to(dev), hcom, world,
                                                                   reduce_op="sum", bias=None, comm_turn=0).cpu()
            y, gth = torch_npu.npu_all_gather_base_mm(ag_x1[rank].to(dev), ag_x2[rank].to(dev), hcom, world)
            res[f"ag{rep}"], res[f"gather{rep}"] = y.cpu(), gth.cpu()
        # a larger bf16 case with a bias, operators interleaved with the allreduce operator (shared regions)
        g = torch.Generator().manual_seed(77)
        big_x1 = [(torch.rand((1024, 2048), generator=g) * 2 - 1).to(torch.bfloat16) for _ in range(world)]
        big_x2 = [(torch.rand((2048, 1536), generator=g) * 2 - 1).to(torch.bfloat16) for _ in range(world)]
        bias = (torch.rand(1536, generator=g) - 0.5).to(torch.bfloat16)
        res["big_rs"] = torch_npu.npu_mm_reduce_scatter_base(big_x1[rank].to(dev), big_x2[rank].to(dev), hcom, world,
                                                             bias=bias.to(dev)).cpu()
        y, _ = torch_npu.npu_all_gather_base_mm(big_x1[rank][:256].to(dev), big_x2[rank].to(dev), hcom, world,
                                                bias=bias.to(dev), gather_output=False)
        res["big_ag"] = y.cpu()
        torch.cuda.synchronize()
        c2p.put((rank, res))
        dist.barrier()
        torch_npu.destroy_comm(hcom)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,path", [(2, "peer"), (2, "nccl"), (4, "peer"), (8, "peer"), (8, "nccl")])
def test_multi_rank(oracle, pkg, world, path):
    """One process per GPU.  "peer": the matmul's epilogue stores fp32 rows into the owners' peer regions and the
    library's own kernels reduce / gather over NVLink; "nccl": ncclReduceScatter / ncclAllGather carry the exchange."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    mk = _golden_module()
    ctx = mp.get_context("spawn")
    c2p = ctx.Queue()
    port = 29800 + os.getpid() % 1000
    env = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    if path == "nccl":
        os.environ["QMM_ALLREDUCE"] = "nccl"
    try:
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, c2p)) for r in range(world)]
        for p in procs:
            p.start()
        results = {}
        for _ in range(world):
            rank, res = c2p.get(timeout=600)
            results[rank] = res
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        os.environ.clear()
        os.environ.update(env)
    rs_x1, rs_x2, ag_x1, ag_x2 = mk.mc2_inputs(world)
    rs_want = oracle.mm_reduce_scatter(rs_x1, rs_x2, world)
    ag_want, gathered = oracle.all_gather_mm(ag_x1, ag_x2, world)
    g = torch.Generator().manual_seed(77)
    big_x1 = [(torch.rand((1024, 2048), generator=g) * 2 - 1).to(torch.bfloat16) for _ in range(world)]
    big_x2 = [(torch.rand((2048, 1536), generator=g) * 2 - 1).to(torch.bfloat16) for _ in range(world)]
    bias = (torch.rand(1536, generator=g) - 0.5).to(torch.bfloat16)
    big_rs = oracle.mm_reduce_scatter(big_x1, big_x2, world, bias=bias)
    big_ag, _ = oracle.all_gather_mm([x[:256] for x in big_x1], big_x2, world, bias=bias)
    for r in range(world):
        for rep in range(2):
            assert results[r][f"rs{rep}"].shape == (128 // world, 256)
            assert _close(results[r][f"rs{rep}"], rs_want[r]), f"rank {r}"
            assert _close(results[r][f"ag{rep}"], ag_want[r]), f"rank {r}"
            assert torch.equal(results[r][f"gather{rep}"], gathered)
        assert _close(results[r]["big_rs"], big_rs[r])
        assert _close(results[r]["big_ag"], big_ag[r])
