"""ctypes binding of the C ABI declared in ``include/qmm_b200.h``.

This is the thinnest possible host: it passes raw device pointers taken from
torch tensors to ``libqmm_b200.so``.  The torch custom ops (``op_plugin``) are
the production host; this module exists for tests, benchmarks and for callers
that have no torch dispatcher.  There is no fallback: if the library is not
built, loading raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libqmm_b200.so"

QMM_OK = 0
DTYPE_BF16, DTYPE_F16, DTYPE_F32, DTYPE_I32, DTYPE_NONE = 0, 1, 2, 3, -1
ALGO_AUTO, ALGO_TILE, ALGO_STREAMK, ALGO_SIMT, ALGO_PAIR, ALGO_SPLITK = 0, 1, 2, 3, 4, 5
UNIQUE_ID_BYTES = 128

# every symbol include/qmm_b200.h declares
EXPORTED_SYMBOLS = (
    "qmm_last_error", "qmm_version", "qmm_device_status", "qmm_dynamic_quant",
    "qmm_quant_matmul_workspace_size", "qmm_quant_matmul", "qmm_weight_quant_batchmatmul_workspace_size",
    "qmm_weight_quant_batchmatmul",
    "qmm_comm_unique_id", "qmm_comm_init_rank", "qmm_comm_register", "qmm_comm_info", "qmm_comm_destroy",
    "qmm_mm_all_reduce", "qmm_quant_matmul_decode_noalloc", "qmm_comm_peer_memory_size",
    "qmm_comm_attach_peer_memory",
    "qmm_w4a16_prepack_size", "qmm_w4a16_prepack", "qmm_w4a16_unpack_weight",
    "qmm_weight_quant_batchmatmul_prepacked_workspace_size", "qmm_weight_quant_batchmatmul_prepacked",
    "qmm_rms_norm", "qmm_rms_norm_dynamic_quant", "qmm_comm_stats", "qmm_int8_mma_peak", "qmm_noalloc_status",
    "qmm_mm_reduce_scatter_workspace_size", "qmm_mm_reduce_scatter", "qmm_all_gather_mm_workspace_size",
    "qmm_all_gather_mm", "qmm_quant_matmul_int8_workspace_size", "qmm_quant_matmul_int8",
)
NOALLOC_SCRATCH_BYTES = 16 << 20

_TORCH_TO_QMM = {torch.bfloat16: DTYPE_BF16, torch.float16: DTYPE_F16, torch.float32: DTYPE_F32,
                 torch.int32: DTYPE_I32}

_lib = None


class QmmError(RuntimeError):
    pass


def _export_nccl_path() -> None:
    """Point the library at the NCCL build torch itself uses (it binds NCCL with dlopen)."""
    import os

    if os.environ.get("QMM_NCCL_LIB"):
        return
    try:
        import nvidia.nccl  # type: ignore

        for base in nvidia.nccl.__path__:
            cand = Path(base) / "lib" / "libnccl.so.2"
            if cand.exists():
                os.environ["QMM_NCCL_LIB"] = str(cand)
                return
    except Exception:
        pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise QmmError(f"{LIB_PATH} is not built; run `python {_PKG / 'build.py'}` (there is no fallback path)")
        _export_nccl_path()
        L = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        c = ctypes
        L.qmm_last_error.restype = c.c_char_p
        L.qmm_version.restype = c.c_int
        L.qmm_device_status.argtypes = [c.c_int]
        L.qmm_dynamic_quant.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_int64, c.c_int64, c.c_void_p, c.c_int64,
                                        c.c_void_p, c.c_void_p]
        L.qmm_quant_matmul_workspace_size.argtypes = [c.c_int64, c.c_int64, c.c_int64, c.c_int,
                                                      c.POINTER(c.c_size_t)]
        L.qmm_quant_matmul.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_int64, c.c_void_p, c.c_int64,
                                       c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_int64, c.c_int64,
                                       c.c_int64, c.c_int64, c.c_int, c.c_void_p, c.c_size_t, c.c_void_p]
        L.qmm_quant_matmul_decode_noalloc.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_int64,
                                                      c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_int,
                                                      c.c_void_p, c.c_int, c.c_int64, c.c_int64, c.c_int64,
                                                      c.c_int64, c.c_void_p]
        L.qmm_quant_matmul_decode_noalloc.restype = c.c_int
        L.qmm_weight_quant_batchmatmul_workspace_size.argtypes = [c.c_int64, c.c_int64, c.c_int64, c.c_int64,
                                                                  c.POINTER(c.c_size_t)]
        L.qmm_weight_quant_batchmatmul_workspace_size.restype = c.c_int
        L.qmm_weight_quant_batchmatmul.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_void_p, c.c_int64, c.c_void_p,
                                                   c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_int64,
                                                   c.c_int64, c.c_int64, c.c_int64, c.c_void_p, c.c_size_t,
                                                   c.c_void_p]
        L.qmm_w4a16_prepack_size.argtypes = [c.c_int64, c.c_int64, c.c_int64, c.POINTER(c.c_size_t)]
        L.qmm_w4a16_prepack.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_int, c.c_int64, c.c_int64,
                                        c.c_int64, c.c_void_p, c.c_size_t, c.c_void_p]
        L.qmm_w4a16_unpack_weight.argtypes = [c.c_void_p, c.c_int64, c.c_int64, c.c_void_p, c.c_int64, c.c_void_p]
        L.qmm_weight_quant_batchmatmul_prepacked_workspace_size.argtypes = [c.c_int64, c.c_int64, c.c_int64,
                                                                            c.POINTER(c.c_size_t)]
        L.qmm_weight_quant_batchmatmul_prepacked.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_void_p, c.c_size_t,
                                                             c.c_void_p, c.c_void_p, c.c_int64, c.c_int64, c.c_int64,
                                                             c.c_int64, c.c_void_p, c.c_size_t, c.c_void_p]
        for name in ("qmm_w4a16_prepack_size", "qmm_w4a16_prepack", "qmm_w4a16_unpack_weight",
                     "qmm_weight_quant_batchmatmul_prepacked_workspace_size",
                     "qmm_weight_quant_batchmatmul_prepacked"):
            getattr(L, name).restype = c.c_int
        L.qmm_rms_norm.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_int64, c.c_int64, c.c_void_p, c.c_double,
                                   c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p]
        L.qmm_rms_norm.restype = c.c_int
        L.qmm_rms_norm_dynamic_quant.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_int64, c.c_int64, c.c_void_p,
                                                 c.c_double, c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p]
        L.qmm_rms_norm_dynamic_quant.restype = c.c_int
        L.qmm_int8_mma_peak.argtypes = [c.c_int, c.POINTER(c.c_double), c.POINTER(c.c_double), c.POINTER(c.c_double)]
        L.qmm_int8_mma_peak.restype = c.c_int
        L.qmm_noalloc_status.argtypes = [c.c_int]
        L.qmm_noalloc_status.restype = c.c_int
        L.qmm_mm_reduce_scatter_workspace_size.argtypes = [c.c_int64, c.c_int64, c.c_int64, c.c_int,
                                                           c.POINTER(c.c_size_t)]
        L.qmm_mm_reduce_scatter.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_void_p, c.c_int64, c.c_int64,
                                            c.c_void_p, c.c_void_p, c.c_int64, c.c_int64, c.c_int64, c.c_int64,
                                            c.c_char_p, c.c_char_p, c.c_int64, c.c_void_p, c.c_size_t, c.c_void_p]
        L.qmm_all_gather_mm_workspace_size.argtypes = [c.c_int64, c.c_int64, c.c_int64, c.c_int, c.POINTER(c.c_size_t)]
        L.qmm_all_gather_mm.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_void_p, c.c_int64, c.c_int64, c.c_void_p,
                                        c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_int64, c.c_int64, c.c_int64,
                                        c.c_char_p, c.c_int64, c.c_int64, c.c_void_p, c.c_size_t, c.c_void_p]
        for name in ("qmm_mm_reduce_scatter_workspace_size", "qmm_mm_reduce_scatter",
                     "qmm_all_gather_mm_workspace_size", "qmm_all_gather_mm"):
            getattr(L, name).restype = c.c_int
        L.qmm_quant_matmul_int8_workspace_size.argtypes = [c.c_int64, c.c_int64, c.c_int64, c.POINTER(c.c_size_t)]
        L.qmm_quant_matmul_int8_workspace_size.restype = c.c_int
        L.qmm_quant_matmul_int8.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_int64, c.c_void_p,
                                            c.c_int64, c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p,
                                            c.c_int64, c.c_int64, c.c_int64, c.c_int64, c.c_void_p, c.c_size_t,
                                            c.c_void_p]
        L.qmm_quant_matmul_int8.restype = c.c_int
        L.qmm_comm_unique_id.argtypes = [c.c_void_p]
        L.qmm_comm_init_rank.argtypes = [c.c_char_p, c.c_void_p, c.c_int, c.c_int]
        L.qmm_comm_register.argtypes = [c.c_char_p, c.c_void_p, c.c_int, c.c_int]
        L.qmm_comm_info.argtypes = [c.c_char_p, c.POINTER(c.c_int), c.POINTER(c.c_int)]
        L.qmm_comm_destroy.argtypes = [c.c_char_p]
        L.qmm_comm_stats.argtypes = [c.c_char_p] + [c.POINTER(c.c_int64)] * 4
        L.qmm_comm_stats.restype = c.c_int
        L.qmm_comm_peer_memory_size.argtypes = [c.c_int64, c.c_int64, c.c_int, c.POINTER(c.c_size_t)]
        L.qmm_comm_attach_peer_memory.argtypes = [c.c_char_p, c.POINTER(c.c_void_p), c.c_void_p, c.c_size_t]
        L.qmm_mm_all_reduce.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_int64, c.c_void_p,
                                        c.c_int64, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_int64,
                                        c.c_int64, c.c_int64, c.c_int64, c.c_char_p, c.c_char_p, c.c_int64,
                                        c.c_void_p, c.c_size_t, c.c_void_p]
        for name in ("qmm_dynamic_quant", "qmm_quant_matmul_workspace_size", "qmm_quant_matmul",
                     "qmm_weight_quant_batchmatmul", "qmm_comm_unique_id", "qmm_comm_init_rank",
                     "qmm_comm_register", "qmm_comm_info", "qmm_comm_destroy", "qmm_mm_all_reduce",
                     "qmm_device_status"):
            getattr(L, name).restype = c.c_int
        _lib = L
    return _lib


def check(rc: int, what: str) -> None:
    if rc != QMM_OK:
        raise QmmError(f"{what} failed with status {rc}: {lib().qmm_last_error().decode()}")


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def dtype_code(dt) -> int:
    return _TORCH_TO_QMM[dt]


def device_status(reset: bool = False) -> int:
    return lib().qmm_device_status(1 if reset else 0)


def dynamic_quant(x: torch.Tensor):
    """x: [..., cols] bf16/f16 CUDA tensor -> (int8 same shape, fp32 x.shape[:-1])."""
    assert x.is_cuda and x.stride(-1) == 1
    cols = x.shape[-1]
    rows = 1
    for d in x.shape[:-1]:
        rows *= d
    x2 = x.reshape(rows, cols)
    if x2.stride(-1) != 1 and x2.numel() > 0:
        x2 = x2.contiguous()
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    s = torch.empty((rows,), dtype=torch.float32, device=x.device)
    ld_x = x2.stride(0) if rows > 1 else max(cols, 1)
    with torch.cuda.device(x.device):
        check(lib().qmm_dynamic_quant(_ptr(x2), dtype_code(x.dtype), rows, cols, max(ld_x, cols), _ptr(q),
                                      max(cols, 1), _ptr(s), _stream()), "qmm_dynamic_quant")
    return q.reshape(x.shape), s.reshape(x.shape[:-1])


def quant_matmul_workspace_size(M: int, N: int, K: int, algo: int = ALGO_AUTO) -> int:
    n = ctypes.c_size_t(0)
    check(lib().qmm_quant_matmul_workspace_size(M, N, K, algo, ctypes.byref(n)), "qmm_quant_matmul_workspace_size")
    return int(n.value)


_workspaces = {}


def get_workspace(device, nbytes: int, kind: str = "w8a8") -> torch.Tensor | None:
    """Zero-initialised scratch, cached per (kernel family, device, stream); grown by reallocation.
    The families do not share a buffer: each relies on what it left behind itself."""
    if nbytes == 0:
        return None
    key = (kind, device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def quant_matmul(x1, x2, scale, pertoken_scale=None, bias=None, output_dtype=torch.bfloat16, algo=ALGO_AUTO,
                 out=None):
    """x1 int8 [M,K]; x2 int8 [K,N] (row-major or a transposed view); see qmm_quant_matmul."""
    assert x1.is_cuda and x1.dtype == torch.int8 and x2.dtype == torch.int8
    M, K = x1.shape
    K2, N = x2.shape
    assert K == K2
    if x1.stride(1) != 1 and K > 1:
        x1 = x1.contiguous()
    if x2.stride(0) != 1 and x2.stride(1) != 1:
        x2 = x2.contiguous()
    sk, sn = x2.stride(0), x2.stride(1)
    if N == 1 and sk != 1:
        sn = 1
    if K == 1 and sn != 1:
        sk = 1
    if out is None:
        out = torch.empty((M, N), dtype=output_dtype, device=x1.device)
    ws_bytes = quant_matmul_workspace_size(M, N, K, algo)
    ws = get_workspace(x1.device, ws_bytes)
    with torch.cuda.device(x1.device):
        check(lib().qmm_quant_matmul(
            _ptr(x1), max(x1.stride(0), K, 1) if M > 1 else max(K, 1), _ptr(x2), sk, sn,
            _ptr(scale), 0 if scale is None else scale.numel(), _ptr(pertoken_scale), _ptr(bias),
            DTYPE_NONE if bias is None else dtype_code(bias.dtype), _ptr(out), dtype_code(output_dtype),
            max(out.stride(0), N) if M > 1 else max(N, 1), M, N, K, algo, _ptr(ws), ws_bytes, _stream()),
            "qmm_quant_matmul")
    return out


def weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset=None, bias=None, group_size=0,
                             use_workspace=True):
    """x [M,K] bf16/f16; weight int32 [K, N/8]; scale/offset [K/group, N].
    use_workspace=False withholds the scratch, which selects the CUDA-core kernel."""
    assert x.is_cuda and weight.dtype == torch.int32
    M, K = x.shape
    N = weight.shape[1] * 8
    group = group_size if group_size > 0 else K
    x = x.contiguous()
    weight = weight.contiguous()
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    n = ctypes.c_size_t(0)
    check(lib().qmm_weight_quant_batchmatmul_workspace_size(M, N, K, group, ctypes.byref(n)),
          "qmm_weight_quant_batchmatmul_workspace_size")
    ws_bytes = int(n.value) if use_workspace else 0
    ws = get_workspace(x.device, ws_bytes, kind="w4a16")
    with torch.cuda.device(x.device):
        check(lib().qmm_weight_quant_batchmatmul(
            _ptr(x), dtype_code(x.dtype), K, _ptr(weight), weight.shape[1], _ptr(antiquant_scale.contiguous()),
            _ptr(None if antiquant_offset is None else antiquant_offset.contiguous()), group,
            _ptr(None if bias is None else bias.contiguous()), _ptr(out), N, M, N, K, _ptr(ws), ws_bytes, _stream()),
            "qmm_weight_quant_batchmatmul")
    return out


def w4a16_prepack_size(N: int, K: int, group: int) -> int:
    """Bytes of the prepacked form of a [K, N/8] int4 weight (0: this shape cannot be prepacked)."""
    n = ctypes.c_size_t(0)
    check(lib().qmm_w4a16_prepack_size(N, K, group, ctypes.byref(n)), "qmm_w4a16_prepack_size")
    return int(n.value)


def w4a16_prepack(weight, antiquant_scale, antiquant_offset=None, group_size=0):
    """weight int32 [K, N/8] + scale/offset [K/group, N] -> uint8 buffer in the k-major stream layout."""
    assert weight.is_cuda and weight.dtype == torch.int32
    K, N = weight.shape[0], weight.shape[1] * 8
    group = group_size if group_size > 0 else K
    nbytes = w4a16_prepack_size(N, K, group)
    if nbytes == 0:
        raise QmmError(f"W4A16 weights [K={K}, N={N}] with group {group} cannot be prepacked")
    weight = weight.contiguous()
    packed = torch.empty(nbytes, dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        check(lib().qmm_w4a16_prepack(_ptr(weight), weight.shape[1], _ptr(antiquant_scale.contiguous()),
                                      _ptr(None if antiquant_offset is None else antiquant_offset.contiguous()),
                                      dtype_code(antiquant_scale.dtype), group, N, K, _ptr(packed), nbytes, _stream()),
              "qmm_w4a16_prepack")
    return packed


def w4a16_unpack_weight(packed, N: int, K: int):
    """The stock int32 [K, N/8] words back out of a prepacked buffer."""
    w = torch.empty((K, N // 8), dtype=torch.int32, device=packed.device)
    with torch.cuda.device(packed.device):
        check(lib().qmm_w4a16_unpack_weight(_ptr(packed), N, K, _ptr(w), N // 8, _stream()), "qmm_w4a16_unpack_weight")
    return w


def weight_quant_batchmatmul_prepacked(x, packed, N: int, bias=None):
    """x [M,K] bf16/f16 (the dtype the weights were prepacked with); packed from w4a16_prepack."""
    assert x.is_cuda and packed.dtype == torch.uint8
    M, K = x.shape
    x = x.contiguous()
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    n = ctypes.c_size_t(0)
    check(lib().qmm_weight_quant_batchmatmul_prepacked_workspace_size(M, N, K, ctypes.byref(n)),
          "qmm_weight_quant_batchmatmul_prepacked_workspace_size")
    ws_bytes = int(n.value)
    ws = get_workspace(x.device, ws_bytes, kind="w4a16_prepacked")
    with torch.cuda.device(x.device):
        check(lib().qmm_weight_quant_batchmatmul_prepacked(
            _ptr(x), dtype_code(x.dtype), K, _ptr(packed), packed.numel(), _ptr(None if bias is None else bias.contiguous()),
            _ptr(out), N, M, N, K, _ptr(ws), ws_bytes, _stream()), "qmm_weight_quant_batchmatmul_prepacked")
    return out


def _rows_cols(x):
    cols = x.shape[-1]
    rows = 1
    for d in x.shape[:-1]:
        rows *= d
    return rows, cols


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, epsilon: float = 1e-6):
    """x [..., cols] bf16/f16/f32, gamma [cols] -> (y like x, rstd fp32 of shape x.shape[:-1] + (1,))."""
    assert x.is_cuda and gamma.dtype == x.dtype
    rows, cols = _rows_cols(x)
    x2 = x.reshape(rows, cols).contiguous()
    y = torch.empty_like(x2)
    rstd = torch.empty((rows,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().qmm_rms_norm(_ptr(x2), dtype_code(x.dtype), rows, cols, cols, _ptr(gamma.contiguous()), epsilon,
                                 _ptr(y), cols, _ptr(rstd), _stream()), "qmm_rms_norm")
    return y.reshape(x.shape), rstd.reshape(*x.shape[:-1], 1)


def rms_norm_dynamic_quant(x: torch.Tensor, gamma: torch.Tensor, epsilon: float = 1e-6):
    """Fused rms_norm + dynamic_quant: (q int8 like x, scale fp32 x.shape[:-1], rstd fp32 x.shape[:-1] + (1,))."""
    assert x.is_cuda and gamma.dtype == x.dtype
    rows, cols = _rows_cols(x)
    x2 = x.reshape(rows, cols).contiguous()
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device)
    scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
    rstd = torch.empty((rows,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().qmm_rms_norm_dynamic_quant(_ptr(x2), dtype_code(x.dtype), rows, cols, cols,
                                               _ptr(gamma.contiguous()), epsilon, _ptr(q), cols, _ptr(scale),
                                               _ptr(rstd), _stream()), "qmm_rms_norm_dynamic_quant")
    return q.reshape(x.shape), scale.reshape(x.shape[:-1]), rstd.reshape(*x.shape[:-1], 1)


def comm_stats(name: str) -> dict:
    """How many qmm_mm_all_reduce calls of communicator `name` took which allreduce path."""
    a, b, f, c = ctypes.c_int64(0), ctypes.c_int64(0), ctypes.c_int64(0), ctypes.c_int64(0)
    check(lib().qmm_comm_stats(name.encode(), ctypes.byref(a), ctypes.byref(b), ctypes.byref(f), ctypes.byref(c)),
          "qmm_comm_stats")
    return {"peer_calls": a.value, "peer_pushed_calls": b.value, "peer_fused_calls": f.value, "nccl_calls": c.value}


def int8_mma_peak(batches: int = 1024) -> dict:
    """Measured issue-rate ceiling of the int8 tensor pipe (see qmm_int8_mma_peak)."""
    a, b, c = ctypes.c_double(0), ctypes.c_double(0), ctypes.c_double(0)
    check(lib().qmm_int8_mma_peak(batches, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)), "qmm_int8_mma_peak")
    return {"ops_per_clk_per_sm": a.value, "tops": b.value, "sm_mhz": c.value}


def quant_matmul_int8(x1, x2, scale, offset=None, pertoken_scale=None, bias=None):
    """x1 int8 [M,K], x2 int8 [K,N] -> int8 [M,N] requantized (see qmm_quant_matmul_int8)."""
    assert x1.is_cuda and x1.dtype == torch.int8 and x2.dtype == torch.int8
    M, K = x1.shape
    N = x2.shape[1]
    x1 = x1.contiguous()
    if x2.stride(0) != 1 and x2.stride(1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((M, N), dtype=torch.int8, device=x1.device)
    n = ctypes.c_size_t(0)
    check(lib().qmm_quant_matmul_int8_workspace_size(M, N, K, ctypes.byref(n)), "qmm_quant_matmul_int8_workspace_size")
    ws = get_workspace(x1.device, int(n.value), kind="w8a8_int8")
    with torch.cuda.device(x1.device):
        check(lib().qmm_quant_matmul_int8(_ptr(x1), max(K, 1), _ptr(x2), x2.stride(0), x2.stride(1), _ptr(scale),
                                          scale.numel(), _ptr(offset), 0 if offset is None else offset.numel(),
                                          _ptr(pertoken_scale), _ptr(bias), _ptr(out), max(N, 1), M, N, K, _ptr(ws),
                                          int(n.value), _stream()), "qmm_quant_matmul_int8")
    return out
