"""Call-site shim: the names existing callers use (``torch_npu.npu_quant_matmul(...)``)
bound to this build's ``torch.ops.npu.*`` operators on CUDA tensors.

It does not imitate the Ascend stack: there is no ``npu`` device, tensors live
on ``cuda``.  Put this package's parent directory on ``sys.path`` and
``import torch_npu``.

Communicators: the reference obtains a communicator name from the process
group (``group._get_backend(torch.device('npu')).get_hccl_comm_name(rank)``,
test/test_custom_ops/test_mm_reduce_scatter_base.py:29-33) and passes that
string as ``hcom``.  ``get_comm_name(group)`` is the counterpart here.
"""
from __future__ import annotations

import ctypes
import importlib.util
import sys
from pathlib import Path

import torch

_PKG_DIR = Path(__file__).resolve().parent.parent
_PKG_NAME = "ascend_python_b200"


def _load_pkg():
    if _PKG_NAME in sys.modules:
        return sys.modules[_PKG_NAME]
    spec = importlib.util.spec_from_file_location(_PKG_NAME, _PKG_DIR / "__init__.py",
                                                  submodule_search_locations=[str(_PKG_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[_PKG_NAME] = mod
    spec.loader.exec_module(mod)
    return mod


_pkg = _load_pkg()
_ops = _pkg.load_ops()
_capi = _pkg.capi


def npu_dynamic_quant(input, *, smooth_scales=None):
    return _ops.npu_dynamic_quant(input, smooth_scales=smooth_scales)


def npu_rms_norm(self, gamma, epsilon=1e-06):
    return _ops.npu_rms_norm(self, gamma, epsilon)


def npu_rms_norm_dynamic_quant(self, gamma, epsilon=1e-06):
    """npu_rms_norm fused with npu_dynamic_quant: (int8 values, per-token scale, rstd)."""
    return _ops.npu_rms_norm_dynamic_quant(self, gamma, epsilon)


def npu_quant_matmul(x1, x2, scale, *, offset=None, pertoken_scale=None, bias=None, output_dtype=None):
    return _ops.npu_quant_matmul(x1, x2, scale, offset=offset, pertoken_scale=pertoken_scale, bias=bias,
                                 output_dtype=output_dtype)


def npu_weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset=None, quant_scale=None,
                                 quant_offset=None, bias=None, antiquant_group_size=0):
    return _ops.npu_weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset, quant_scale, quant_offset,
                                             bias, antiquant_group_size)


def npu_mm_all_reduce_base(x1, x2, hcom, *, reduce_op="sum", bias=None, antiquant_scale=None, antiquant_offset=None,
                           x3=None, dequant_scale=None, pertoken_scale=None, antiquant_group_size=0, comm_turn=0):
    if comm_turn == 0 and x1.is_cuda:
        _ensure_peer_memory(hcom, x1.numel() // max(x1.shape[-1], 1), x2.shape[-1], x1.device)
    return _ops.npu_mm_all_reduce_base(x1, x2, hcom, reduce_op=reduce_op, bias=bias, antiquant_scale=antiquant_scale,
                                       antiquant_offset=antiquant_offset, x3=x3, dequant_scale=dequant_scale,
                                       pertoken_scale=pertoken_scale, antiquant_group_size=antiquant_group_size,
                                       comm_turn=comm_turn)


def npu_mm_reduce_scatter_base(self, x2, hcom, world_size, *, reduce_op="sum", bias=None, comm_turn=0):
    if self.is_cuda and world_size > 1:
        # first half of a region: the fp32 rows of all ranks that this rank will add up
        _ensure_peer_bytes(hcom, self.shape[0] * x2.shape[-1] * 4, self.device)
    return _ops.npu_mm_reduce_scatter_base(self, x2, hcom, world_size, reduce_op=reduce_op, bias=bias,
                                           comm_turn=comm_turn)


def npu_all_gather_base_mm(self, x2, hcom, world_size, *, bias=None, gather_index=0, gather_output=True, comm_turn=0):
    if self.is_cuda and world_size > 1:
        _ensure_peer_bytes(hcom, self.numel() * self.element_size(), self.device)  # this rank's shard of x1
    return _ops.npu_all_gather_base_mm(self, x2, hcom, world_size, bias=bias, gather_index=gather_index,
                                       gather_output=gather_output, comm_turn=comm_turn)


_comm_names = {}


def comm_name_for(group_name: str, world_size: int) -> str:
    """Deterministic registry name of a process group's communicator."""
    return f"qmm_comm_{group_name or 'default'}_{world_size}"


def get_comm_name(group=None) -> str:
    """Create (once) and register an NCCL communicator for ``group`` and return its name.

    Rank 0 of the group draws the NCCL unique id; it reaches the other ranks
    through the group's own object broadcast, so any backend works for the
    exchange.  Every rank must call this collectively, with its GPU current.
    """
    import torch.distributed as dist

    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialized")
    group = group if group is not None else dist.group.WORLD
    world_size = dist.get_world_size(group)
    rank = dist.get_rank(group)
    name = comm_name_for(getattr(group, "group_name", "") or str(id(group) if group is not dist.group.WORLD else ""),
                         world_size)
    if name in _comm_names:
        return name
    lib = _capi.lib()
    buf = ctypes.create_string_buffer(_capi.UNIQUE_ID_BYTES)
    if rank == 0:
        _capi.check(lib.qmm_comm_unique_id(buf), "qmm_comm_unique_id")
    payload = [bytes(buf.raw) if rank == 0 else None]
    src = dist.get_global_rank(group, 0) if group is not dist.group.WORLD else 0
    dist.broadcast_object_list(payload, src=src, group=group)
    uid = ctypes.create_string_buffer(payload[0], _capi.UNIQUE_ID_BYTES)
    _capi.check(lib.qmm_comm_init_rank(name.encode(), uid, world_size, rank), "qmm_comm_init_rank")
    _comm_names[name] = dict(group=group, world=world_size, rank=rank)
    return name


_peer_memory = {}  # communicator name -> dict(bytes, tensor, handle) or None when unavailable


def _ensure_peer_bytes(name: str, half_bytes: int, device) -> None:
    """Peer-mapped regions whose two halves hold at least ``half_bytes`` each (see _ensure_peer_memory)."""
    _ensure_peer_region(name, 65536 + 2 * ((int(half_bytes) + 255) // 256 * 256), device)


def _ensure_peer_memory(name: str, M: int, N: int, device) -> None:
    """Gives the communicator ``name`` peer-mapped regions large enough for an allreduce of [M, N]."""
    info = _comm_names.get(name)
    if not isinstance(info, dict):
        return
    need = ctypes.c_size_t(0)
    _capi.check(_capi.lib().qmm_comm_peer_memory_size(M, N, info["world"], ctypes.byref(need)),
                "qmm_comm_peer_memory_size")
    _ensure_peer_region(name, int(need.value), device)


def _ensure_peer_region(name: str, need_bytes: int, device) -> None:
    """Gives the communicator ``name`` peer-mapped regions of at least ``need_bytes``.

    The regions come from torch's symmetric memory (one allocation per rank, mapped by all ranks of
    the node); the library then reduces and gathers through NVLink loads instead of NCCL.  The first
    call, and any call that needs a larger region, is collective: all ranks reach it with the same
    size.  Where symmetric memory is not available the communicator stays on NCCL.
    QMM_ALLREDUCE = nccl | p2p | multimem forces a path; unset, peer memory with plain peer loads is used
    (measured on B200, M=4096, N=8192: 381 us against 424 us with NCCL on two GPUs, 250 us against 356 us on
    eight; in-switch reduction measured the same as plain loads, which keep the rank-order sum).
    """
    import os

    info = _comm_names.get(name)
    mode = os.environ.get("QMM_ALLREDUCE", "")
    if not isinstance(info, dict) or mode == "nccl":
        return
    world = info["world"]
    if world < 2 or world > 8:
        return
    lib = _capi.lib()
    cur = _peer_memory.get(name, {})
    if cur is None or (cur and cur["bytes"] >= need_bytes):
        return
    try:
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        nbytes = max(int(need_bytes), 32 << 20)
        nbytes = (nbytes + (2 << 20) - 1) // (2 << 20) * (2 << 20)
        if cur:
            _capi.check(lib.qmm_comm_attach_peer_memory(name.encode(), None, None, 0), "qmm_comm_attach_peer_memory")
            torch.cuda.synchronize(device)
        buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
        handle = symm.rendezvous(buf, info["group"])
        buf.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=info["group"])  # every region is zero before anyone raises a flag in it
        ptrs = (ctypes.c_void_p * world)(*[int(a) for a in handle.buffer_ptrs])
        # plain peer loads unless in-switch reduction is asked for
        mc = int(getattr(handle, "multicast_ptr", 0) or 0) if mode == "multimem" else 0
        _capi.check(lib.qmm_comm_attach_peer_memory(name.encode(), ptrs, ctypes.c_void_p(mc or None), nbytes),
                    "qmm_comm_attach_peer_memory")
        _peer_memory[name] = dict(bytes=nbytes, tensor=buf, handle=handle)
    except Exception as exc:  # symmetric memory missing or refused: NCCL carries the allreduce
        import warnings

        warnings.warn(f"peer memory for communicator {name} unavailable ({exc!r}); using NCCL")
        _peer_memory[name] = None


def destroy_comm(name: str) -> None:
    if _comm_names.pop(name, None):
        _peer_memory.pop(name, None)
        _capi.check(_capi.lib().qmm_comm_destroy(name.encode()), "qmm_comm_destroy")
