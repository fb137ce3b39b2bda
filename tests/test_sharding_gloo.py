"""Multi-rank host logic on CPU: K sharding and the allreduce contract, with world_size-2 gloo ranks."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def test_k_shard_bounds(pkg):
    from ascend_python_b200.sharding import k_shard_bounds

    assert k_shard_bounds(28672, 2) == [0, 14336, 28672]
    assert k_shard_bounds(28672, 8) == [i * 3584 for i in range(9)]
    assert k_shard_bounds(1000, 3) == [0, 384, 640, 1000]  # 7 units of 128: 3+2+2, tail to the last rank
    assert k_shard_bounds(10, 4) == [0, 3, 6, 8, 10]
    assert k_shard_bounds(0, 2) == [0, 0, 0]
    for K in (1, 127, 128, 129, 4096, 28672, 12345):
        for W in (1, 2, 3, 4, 8):
            b = k_shard_bounds(K, W)
            assert b[0] == 0 and b[-1] == K and all(b[i] <= b[i + 1] for i in range(W))
    with pytest.raises(ValueError, match="world_size"):
        k_shard_bounds(16, 0)


def _rank_main(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    from __graft_entry__ import load_package
    from oracle import qmm_oracle as O

    load_package()
    from ascend_python_b200.sharding import shard_row_parallel

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, w, scale, bias = O.make_w8a8_inputs(24, 512, 40, seed=77)
        xs, ws = shard_row_parallel(x, w, world, rank)
        q8, s = O.dynamic_quant(xs.contiguous())  # every rank quantizes its own shard
        part = O.quant_matmul(q8, ws, scale, pertoken_scale=s, bias=bias if rank == 0 else None,
                              output_dtype=torch.bfloat16).float()
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        # gather every rank's quantized shard so that rank 0 can evaluate the oracle for the whole job
        gathered = [None] * world
        dist.all_gather_object(gathered, (q8, s))
        if rank == 0:
            x1_list = [g[0] for g in gathered]
            pt_list = [g[1] for g in gathered]
            w_list = [shard_row_parallel(x, w, world, r)[1] for r in range(world)]
            total, rounded = O.mm_all_reduce(x1_list, w_list, scale, pt_list, bias=bias, output_dtype=torch.bfloat16)
            q.put((np.array_equal(total, part.numpy()), float(np.abs(total).max())))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_row_parallel_allreduce_gloo_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    same, mag = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert same and mag > 0


def _mc2_rank_main(rank, world, port, q):
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    from make_mc2_golden import mc2_inputs

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rs_x1, rs_x2, ag_x1, ag_x2 = mc2_inputs(world)
        # reduce-scatter matmul: own operands only, one collective, rank r keeps rows [r * M/W, (r+1) * M/W)
        part = torch.matmul(rs_x1[rank].float(), rs_x2[rank].float())
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        rows = part.shape[0] // world
        rs_out = part[rank * rows:(rank + 1) * rows].to(torch.float16)
        # all-gather matmul: gather x1 in rank order, multiply by the rank's own x2
        pieces = [torch.empty_like(ag_x1[rank]) for _ in range(world)]
        dist.all_gather(pieces, ag_x1[rank])
        gathered = torch.cat(pieces)
        ag_out = torch.matmul(gathered.float(), ag_x2[rank].float()).to(torch.float16)
        q.put((rank, rs_out, ag_out, gathered))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_mc2_contract_against_reference_golden_gloo_world2():
    """Two gloo ranks carry out npu_mm_reduce_scatter_base and npu_all_gather_base_mm as distributed programs
    (each rank touches its own operands only; which rows a rank keeps, and the order of the gathered rows, are the
    operators' contract) and are compared with the outputs of the reference's own golden functions
    (tests/golden/mc2_reference.npz), at the reference tests' tolerance."""
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    from make_mc2_golden import mc2_inputs

    world = 2
    golden = np.load(ROOT / "tests" / "golden" / "mc2_reference.npz")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_mc2_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, rs_out, ag_out, gathered = q.get(timeout=120)
        got[rank] = (rs_out, ag_out, gathered)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    ag_x1 = mc2_inputs(world)[2]
    for r in range(world):
        rs_ref = torch.from_numpy(golden["rs2_out"][r]).view(torch.float16)
        ag_ref = torch.from_numpy(golden["ag2_out"][r]).view(torch.float16)
        assert got[r][0].shape == rs_ref.shape and got[r][1].shape == ag_ref.shape
        torch.testing.assert_close(got[r][0], rs_ref, rtol=1e-3, atol=1e-3)
        torch.testing.assert_close(got[r][1], ag_ref, rtol=1e-3, atol=1e-3)
        assert torch.equal(got[r][2], torch.cat(ag_x1))
