"""npu_mm_all_reduce_base: a single-rank communicator on one GPU, and 2/4/8 ranks (one process per
GPU; allreduce through peer memory or NCCL) when the box has that many GPUs.  The peer-memory path is also
held to the oracle bit for bit (same rank-order fp32 sum).  Tolerance after the allreduce: rtol 1e-2 against the
fp32 sum of the per-rank fp32 results (plus 1e-2 of the summed magnitudes as atol for cancellation)."""
import ctypes
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
PKG_DIR = ROOT / "ascend-python_b200"


def test_single_rank_communicator(capi, oracle, dev):
    """nranks = 1: the op is the matmul alone; chunking over M (comm_turn) must not change a bit."""
    sys.path.insert(0, str(PKG_DIR))
    try:
        import torch_npu
    finally:
        sys.path.pop(0)
    lib = capi.lib()
    uid = ctypes.create_string_buffer(capi.UNIQUE_ID_BYTES)
    capi.check(lib.qmm_comm_unique_id(uid), "qmm_comm_unique_id")
    capi.check(lib.qmm_comm_init_rank(b"solo", uid, 1, 0), "qmm_comm_init_rank")
    try:
        nr, rk = ctypes.c_int(-1), ctypes.c_int(-1)
        capi.check(lib.qmm_comm_info(b"solo", ctypes.byref(nr), ctypes.byref(rk)), "qmm_comm_info")
        assert (nr.value, rk.value) == (1, 0)
        assert lib.qmm_comm_init_rank(b"solo", uid, 1, 0) == 1  # name taken
        x, w, scale, bias = oracle.make_w8a8_inputs(640, 512, 768, seed=21)
        q_ref, s_ref = oracle.dynamic_quant(x)
        y_ref = oracle.quant_matmul(q_ref, w, scale, pertoken_scale=s_ref, bias=bias, output_dtype=torch.bfloat16)
        q, s = torch_npu.npu_dynamic_quant(x.to(dev))
        for turn in (0, 1, 3):
            y = torch_npu.npu_mm_all_reduce_base(q, w.to(dev), "solo", reduce_op="sum", bias=bias.to(dev),
                                                 dequant_scale=scale.to(dev), pertoken_scale=s, comm_turn=turn)
            assert y.dtype == torch.bfloat16 and y.shape == (640, 768)
            assert oracle.bf16_ulp_distance(y.cpu(), y_ref).max().item() <= 1
    finally:
        capi.check(lib.qmm_comm_destroy(b"solo"), "qmm_comm_destroy")
    assert lib.qmm_comm_destroy(b"solo") == 5  # not found any more


def test_missing_rank_times_out(capi, oracle, dev):
    """Failure detection without a fault: a two-rank communicator whose other rank never arrives.  Both
    regions are ordinary buffers of this GPU, nothing ever raises rank 1's "partial complete" flag, so the
    reduce kernel's bounded wait runs out (2 s), it records a status code and returns; the context stays
    usable and the next call of another operator is correct."""
    sys.path.insert(0, str(PKG_DIR))
    try:
        import torch_npu
    finally:
        sys.path.pop(0)
    lib = capi.lib()
    M, K, N = 256, 512, 512
    # adopted as a communicator handle but never used: the peer-memory path makes no NCCL call
    placeholder = ctypes.c_void_p(1)
    capi.check(lib.qmm_comm_register(b"half", placeholder, 2, 0), "qmm_comm_register")
    try:
        need = ctypes.c_size_t(0)
        capi.check(lib.qmm_comm_peer_memory_size(M, N, 2, ctypes.byref(need)), "qmm_comm_peer_memory_size")
        regions = [torch.zeros(need.value, dtype=torch.uint8, device=dev) for _ in range(2)]
        ptrs = (ctypes.c_void_p * 2)(*[r.data_ptr() for r in regions])
        capi.check(lib.qmm_comm_attach_peer_memory(b"half", ptrs, None, need.value), "qmm_comm_attach_peer_memory")
        x, w, scale, bias = oracle.make_w8a8_inputs(M, K, N, seed=77)
        q, s = torch_npu.npu_dynamic_quant(x.to(dev))
        torch_npu.npu_mm_all_reduce_base(q, w.to(dev), "half", reduce_op="sum", dequant_scale=scale.to(dev),
                                         pertoken_scale=s)
        torch.cuda.synchronize()  # returns after the wait limit, not never
        status = capi.device_status(reset=True)
        assert status & 0xffff0000 == 0x30000, f"expected the peer-wait timeout code, got {status:#x}"
        # the context is intact: a plain matmul right after is bit-exact
        q_ref, s_ref = oracle.dynamic_quant(x)
        acc_ref = oracle.quant_matmul(q_ref, w, scale, output_dtype=torch.int32)
        acc = capi.quant_matmul(q, w.to(dev), None, output_dtype=torch.int32)
        assert torch.equal(acc.cpu(), acc_ref)
    finally:
        capi.check(lib.qmm_comm_destroy(b"half"), "qmm_comm_destroy")


def _sample_rows(M, K, N):
    """Rows compared with the oracle: all of them, or 64 evenly spaced ones for the full-size configuration
    (whose CPU oracle would take minutes)."""
    return None if M * K * N <= 2 ** 36 else torch.arange(0, M, M // 64)


def _digest(t):
    """Order-dependent 64-bit checksum of a tensor's bits (for cross-rank identity of full outputs)."""
    v = t.contiguous().view(torch.int16).to(torch.int64)
    w = torch.arange(1, v.numel() + 1, device=v.device, dtype=torch.int64).view(v.shape)
    return int((v * w).sum().item())


def _rank_main(rank, world, port, shapes, c2p):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(PKG_DIR))
    import torch.distributed as dist
    import torch_npu
    from ascend_python_b200.sharding import shard_row_parallel
    from oracle import qmm_oracle as O

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        hcom = torch_npu.get_comm_name()
        for (M, K, N, turn) in shapes:
            x, w, scale, bias = O.make_w8a8_inputs(M, K, N, seed=M + K + N)
            xs, ws = shard_row_parallel(x, w, world, rank)
            q, s = torch_npu.npu_dynamic_quant(xs.contiguous().to(dev))
            y = torch_npu.npu_mm_all_reduce_base(q, ws.contiguous().to(dev), hcom, reduce_op="sum", bias=bias.to(dev),
                                                 dequant_scale=scale.to(dev), pertoken_scale=s, comm_turn=turn)
            torch.cuda.synchronize()
            rows = _sample_rows(M, K, N)
            if rows is None:
                c2p.put((rank, (M, K, N, turn), y.cpu(), q.cpu(), s.cpu(), _digest(y)))
            else:
                c2p.put((rank, (M, K, N, turn), y[rows].cpu(), q[rows].cpu(), s[rows].cpu(), _digest(y)))
        # Two calls of different shapes back to back, no host synchronisation in between: the second call's
        # partial area must not land where the first call's reduced rows are still being read by a peer.
        chain = [(256, 1024, 512), (2048, 4096, 1024)]
        outs = []
        ins = []
        for (M, K, N) in chain:
            x, w, scale, bias = O.make_w8a8_inputs(M, K, N, seed=M + K + N)
            xs, ws = shard_row_parallel(x, w, world, rank)
            ins.append((xs.contiguous().to(dev), ws.contiguous().to(dev), scale.to(dev), bias.to(dev)))
        torch.cuda.synchronize()
        for _ in range(3):
            for (xd, wd, sd, bd) in ins:
                q, s = torch_npu.npu_dynamic_quant(xd)
                outs.append(torch_npu.npu_mm_all_reduce_base(q, wd, hcom, reduce_op="sum", bias=bd, dequant_scale=sd,
                                                             pertoken_scale=s))
        torch.cuda.synchronize()
        for i, y in enumerate(outs):
            M, K, N = chain[i % 2]
            c2p.put((rank, ("chain", i, M, K, N), y.cpu(), None, None, _digest(y)))
        from ascend_python_b200 import capi
        c2p.put((rank, ("stats",), capi.comm_stats(hcom), None, None, ""))
        dist.barrier()
        torch_npu.destroy_comm(hcom)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,path", [(2, "peer"), (2, "peer_unfused"), (2, "multimem"), (2, "nccl"), (4, "peer"),
                                        (4, "multimem"), (8, "peer"), (8, "peer_unfused"), (8, "multimem")])
def test_multi_rank(oracle, pkg, world, path):
    """path "peer": calls with comm_turn == 0 reduce and gather through peer memory with plain peer loads inside
    the matmul kernel for prefill shapes (the default for two ranks; forced here for any rank count), in a kernel
    of its own otherwise; "peer_unfused": always in a kernel of its own; "multimem": the same with in-switch
    reduction / broadcast; "nccl" forces NCCL for every call."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from ascend_python_b200.sharding import shard_row_parallel

    # the last shape needs larger peer regions than the first ones allocated: the regions are re-made
    shapes = [(256, 1024, 512, 0), (2048, 4096, 1024, 2), (1000, 2048, 768, 3), (1000, 2048, 768, 0),
              (2048, 4096, 1024, 0), (3, 512, 264, 0), (4096, 512, 4352, 0)]
    if path in ("peer", "peer_unfused"):
        shapes.append((4096, 28672, 8192, 0))  # the row-parallel benchmark configuration itself, at full size
    ctx = mp.get_context("spawn")
    c2p = ctx.Queue()
    port = 29700 + os.getpid() % 1000
    env = dict(os.environ)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    if path == "peer_unfused":
        os.environ["QMM_PEER_FUSED"] = "0"
    elif path == "peer":
        os.environ["QMM_PEER_FUSED"] = "1"
    else:
        os.environ["QMM_ALLREDUCE"] = path
    bit_exact = path in ("peer", "peer_unfused")
    try:
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, shapes, c2p)) for r in range(world)]
        for p in procs:
            p.start()
        results = {}
        for _ in range(world * (len(shapes) + 7)):
            rank, key, y, q, s, digest = c2p.get(timeout=900)
            results[(rank, key)] = (y, q, s, digest)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        os.environ.clear()
        os.environ.update(env)
    for key in shapes:
        M, K, N, _ = key
        x, w, scale, bias = oracle.make_w8a8_inputs(M, K, N, seed=M + K + N)
        rows = _sample_rows(M, K, N)
        if rows is not None:
            x = x[rows]
        q_list = [results[(r, key)][1] for r in range(world)]
        s_list = [results[(r, key)][2] for r in range(world)]
        w_list = [shard_row_parallel(x, w, world, r)[1] for r in range(world)]
        # every rank quantized its own shard exactly like the oracle
        for r in range(world):
            q_ref, s_ref = oracle.dynamic_quant(shard_row_parallel(x, w, world, r)[0].contiguous())
            assert torch.equal(q_list[r], q_ref) and torch.equal(s_list[r], s_ref)
            assert results[(r, key)][3] == results[(0, key)][3], f"rank {r} holds another result than rank 0: {key}"
        total, rounded = oracle.mm_all_reduce(q_list, w_list, scale, s_list, bias=bias, output_dtype=torch.bfloat16)
        mag = sum(np.abs(oracle.quant_matmul(q_list[r], w_list[r], scale, pertoken_scale=s_list[r],
                                              output_dtype=torch.bfloat16).float().numpy()) for r in range(world))
        for r in range(world):
            y = results[(r, key)][0].float().numpy()
            assert np.all(np.abs(y - total) <= 1e-2 * np.abs(total) + 1e-2 * mag), f"rank {r} shape {key}"
            assert np.array_equal(y, results[(0, key)][0].float().numpy())  # all ranks hold the same result
        if bit_exact and key[3] == 0:
            # the library's own kernel adds the ranks' rounded partials in fp32 in rank order and rounds once,
            # which is the oracle's order: bit-exact, not just within the tolerance
            assert torch.equal(results[(0, key)][0].view(torch.int16), rounded.view(torch.int16)), f"shape {key}"
    # the back-to-back calls of alternating shapes: every repetition equals the oracle's rounded sum on every rank
    for i in range(6):
        M, K, N = [(256, 1024, 512), (2048, 4096, 1024)][i % 2]
        key = ("chain", i, M, K, N)
        x, w, scale, bias = oracle.make_w8a8_inputs(M, K, N, seed=M + K + N)
        q_list, s_list, w_list = [], [], []
        for r in range(world):
            xs, ws = shard_row_parallel(x, w, world, r)
            qr, sr = oracle.dynamic_quant(xs.contiguous())
            q_list.append(qr), s_list.append(sr), w_list.append(ws)
        total, rounded = oracle.mm_all_reduce(q_list, w_list, scale, s_list, bias=bias, output_dtype=torch.bfloat16)
        for r in range(world):
            y = results[(r, key)][0]
            if bit_exact:
                assert torch.equal(y.view(torch.int16), rounded.view(torch.int16)), f"rank {r} chained call {i}"
            else:
                assert np.all(np.abs(y.float().numpy() - total) <= 1e-2 * np.abs(total) + 2e-2 * np.abs(total).max())
            assert results[(r, key)][3] == results[(0, key)][3]
    # which kernels did the exchange: the fused matmul for the prefill-sized shapes of the default path only
    for r in range(world):
        st = results[(r, ("stats",))][0]
        if path == "peer":
            assert st["peer_fused_calls"] >= 10 and st["nccl_calls"] >= 2, st
        elif path == "nccl":
            assert st["peer_calls"] == 0, st
        else:
            assert st["peer_fused_calls"] == 0 and st["peer_calls"] > 0, st
