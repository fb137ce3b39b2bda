"""CPU oracle for the quantized-matmul path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may import this module; no product code does.

PARITY UNPINNED.  The four operators restated here (``npu_dynamic_quant``,
``npu_quant_matmul``, ``npu_weight_quant_batchmatmul``,
``npu_mm_all_reduce_base``) do not exist in the reference snapshot and their
arithmetic lives in a closed device library that is not vendored, so the
reference holds no golden vector, known-answer test or fixture for them.  What
the reference does pin is the *style* of its golden computations, which this
file follows:

* ``test/test_custom_ops/test_mm_reduce_scatter_base.py:69-81`` — expected
  result of a matmul+collective op = fp32 CPU matmul per rank, summed over the
  ranks, cast to the output dtype;
* ``test/test_custom_ops/test_all_gather_base_mm.py:72-78`` — same, per-rank;
* ``test/test_custom_ops/test_npu_rms_norm.py:10-34`` — numpy golden
  (``supported_op_exec``) compared with the device op (``custom_op_exec``).

Three operators that DO exist in the reference are restated here too and ARE
pinned against outputs of the reference's own golden functions, executed from
the reference's test files (tests/golden/make_rms_norm_golden.py,
tests/golden/make_mc2_golden.py): ``rms_norm``, ``mm_reduce_scatter``,
``all_gather_mm``.

Every choice the reference leaves open is fixed here, once:

* dynamic quant: ``scale = amax / 127`` and ``q = rint(x / scale)`` with true
  IEEE fp32 divisions, round-half-to-even, clamp to [-128, 127]; a row whose
  amax is 0 gets scale 0 and q 0; amax propagates NaN and Inf into the scale,
  and a quotient that is NaN quantizes to 0.
* quant matmul: exact int32 accumulation; epilogue in fp32, one rounding per
  operation, in the order ``float(acc) * scale[n] * pertoken[m] + bias[n]``,
  then one round-to-nearest-even conversion to bf16/f16.  With
  ``output_dtype=int32`` the accumulator (+ int32 bias) is returned.
* W4A16: nibble j of packed word i along N holds column ``8*i + j`` as a
  two's complement 4-bit integer; ``W = (w + offset[g, n]) * scale[g, n]`` with
  ``g = k // group``; accumulation in fp64 (tolerance stated in the tests).
* matmul + allreduce: each rank's fp32-epilogue result is rounded to the
  output dtype, the rounded partials are summed in fp32 (bias on rank 0 only).

Algorithms restated from the task definition; functions cite the reference
test whose golden style they follow.
"""
from __future__ import annotations

import numpy as np
import torch

# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------


def _f32(t) -> np.ndarray:
    """torch (bf16/f16/f32) or numpy -> float32 numpy, exactly."""
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().to(torch.float32).numpy()
    return np.asarray(t, dtype=np.float32)


def _round_to(v: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """fp32 numpy -> torch tensor of `dtype` with round-to-nearest-even."""
    return torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32)).to(dtype)


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in units of the last place between two bf16/f16 tensors (same dtype)."""
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
    ia = a.cpu().contiguous().view(torch.int16).to(torch.int32)
    ib = b.cpu().contiguous().view(torch.int16).to(torch.int32)
    # map sign-magnitude to a monotonic integer line
    ia = torch.where(ia < 0, -(ia & 0x7FFF), ia)
    ib = torch.where(ib < 0, -(ib & 0x7FFF), ib)
    return (ia - ib).abs()


# ---------------------------------------------------------------------------
# npu_dynamic_quant
# ---------------------------------------------------------------------------


def dynamic_quant(x):
    """Per-token symmetric int8 quantization.

    Golden style: numpy ``supported_op_exec`` of
    test/test_custom_ops/test_npu_rms_norm.py:10-20 (fp32 numpy math on the
    host).  Returns (q int8 tensor of x's shape, scale fp32 of x.shape[:-1]).
    """
    xf = _f32(x)
    shape = xf.shape
    if xf.size == 0:
        return (torch.zeros(shape, dtype=torch.int8), torch.zeros(shape[:-1], dtype=torch.float32))
    xf = xf.reshape(-1, shape[-1])
    amax = np.max(np.abs(xf), axis=1).astype(np.float32)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    safe = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
    with np.errstate(all="ignore"):
        t = (xf / safe[:, None]).astype(np.float32)
    t = np.where(np.isnan(t), np.float32(0), t)  # Inf/Inf or anything/NaN: pinned to 0
    q = np.clip(np.rint(t), -128, 127)
    q = np.where(scale[:, None] == 0, 0, q).astype(np.int8)
    return torch.from_numpy(q.reshape(shape)), torch.from_numpy(scale.reshape(shape[:-1]))


# ---------------------------------------------------------------------------
# npu_rms_norm (+ the dynamic quantization that follows it in a decoder block)
# ---------------------------------------------------------------------------


def rms_norm(x, gamma, epsilon: float = 1e-6):
    """RMS normalisation; returns (y in x's dtype, rstd fp32 of shape x.shape[:-1] + (1,)).

    Restates the numpy golden of test/test_custom_ops/test_npu_rms_norm.py:10-18 operation by
    operation in float32 (``variance = mean(x**2, -1)``, ``std = sqrt(variance + eps)``,
    ``rstd = 1/std``, ``y = (x*rstd)*gamma``); 16-bit inputs are widened exactly first and y is
    rounded once to the input dtype.  tests/golden/rms_norm_reference.npz holds outputs of the
    reference's own function on seeded inputs (made by tests/golden/make_rms_norm_golden.py), and
    tests/test_oracle.py checks this function against them bit for bit: this oracle is pinned.
    """
    dtype = x.dtype if isinstance(x, torch.Tensor) else torch.float32
    xf, gf = _f32(x), _f32(gamma)
    variance = np.mean(np.power(xf, 2), axis=-1, keepdims=True)
    std = np.sqrt(variance + np.float32(epsilon))
    rstd = (1 / std).astype(np.float32)
    y = ((xf * rstd).astype(np.float32) * gf).astype(np.float32)
    return _round_to(y, dtype), torch.from_numpy(rstd)


def rms_norm_dynamic_quant(x, gamma, epsilon: float = 1e-6):
    """dynamic_quant(rms_norm(x)[0]): (q int8, scale fp32, rstd fp32) -- the composition the fused kernel
    must reproduce (the int8 values and scales bit for bit GIVEN the same y; y itself to the tolerance of
    rms_norm, whose row sum the device takes in another order)."""
    y, rstd = rms_norm(x, gamma, epsilon)
    q, scale = dynamic_quant(y)
    return q, scale, rstd


# ---------------------------------------------------------------------------
# npu_quant_matmul
# ---------------------------------------------------------------------------


def int8_matmul_exact(x1, x2) -> np.ndarray:
    """int8 [M,K] @ int8 [K,N] -> exact int32 (fp64 BLAS: |sum| < 2^53 for any K here)."""
    a = np.asarray(x1.cpu().numpy() if isinstance(x1, torch.Tensor) else x1).astype(np.float64)
    b = np.asarray(x2.cpu().numpy() if isinstance(x2, torch.Tensor) else x2).astype(np.float64)
    acc = a @ b
    assert np.all(np.abs(acc) < 2.0 ** 31), "int32 accumulator overflow"
    return acc.astype(np.int64).astype(np.int32)


def dequant_epilogue_f32(acc: np.ndarray, scale, pertoken_scale=None, bias=None) -> np.ndarray:
    """fp32 epilogue, one rounding per operation: float(acc)*scale[n]*pertoken[m] + bias[n]."""
    v = acc.astype(np.float32)
    s = _f32(scale).reshape(-1)
    v = (v * (s[None, :] if s.size > 1 else s[0])).astype(np.float32)
    if pertoken_scale is not None:
        v = (v * _f32(pertoken_scale).reshape(-1)[:, None]).astype(np.float32)
    if bias is not None:
        v = (v + _f32(bias).reshape(-1)[None, :]).astype(np.float32)
    return v


def quant_matmul(x1, x2, scale, *, offset=None, pertoken_scale=None, bias=None, output_dtype=torch.bfloat16):
    """W8A8 matmul + dequantization.

    Golden style: fp32 host matmul then cast to the output dtype
    (test/test_custom_ops/test_mm_reduce_scatter_base.py:74,79); the integer
    product is evaluated exactly instead of in fp32.
    """
    if offset is not None and output_dtype != torch.int8:
        raise ValueError("offset only applies to an int8 output")
    acc = int8_matmul_exact(x1, x2)
    if output_dtype == torch.int8:
        # requantized output (this build's stated choice; the operator is not in the reference snapshot):
        # v = float(acc + bias) * scale[n] (* pertoken[m]) (+ offset[n]) in fp32, one rounding per operation,
        # then round half to even and clamp to [-128, 127]
        if bias is not None:
            acc = acc + bias.cpu().numpy().astype(np.int32)[None, :]
        v = dequant_epilogue_f32(acc, scale, pertoken_scale, None)
        if offset is not None:
            o = _f32(offset).reshape(-1)
            v = (v + (o[None, :] if o.size > 1 else o[0])).astype(np.float32)
        return torch.from_numpy(np.clip(np.rint(v), -128, 127).astype(np.int8))
    if output_dtype == torch.int32:
        if bias is not None:
            acc = acc + bias.cpu().numpy().astype(np.int32)[None, :]
        return torch.from_numpy(acc)
    return _round_to(dequant_epilogue_f32(acc, scale, pertoken_scale, bias), output_dtype)


def quant_matmul_f32(x1, x2, scale, *, pertoken_scale=None, bias=None) -> np.ndarray:
    """The fp32-epilogue result before the final conversion (the '1 ulp' reference)."""
    return dequant_epilogue_f32(int8_matmul_exact(x1, x2), scale, pertoken_scale, bias)


# ---------------------------------------------------------------------------
# npu_weight_quant_batchmatmul (W4A16)
# ---------------------------------------------------------------------------


def pack_int4(w: np.ndarray) -> np.ndarray:
    """int values in [-8,7], shape [K,N] (N % 8 == 0) -> int32 [K, N/8]; nibble j = column 8*i+j."""
    w = np.asarray(w).astype(np.int64)
    K, N = w.shape
    assert N % 8 == 0 and w.min() >= -8 and w.max() <= 7
    u = (w & 0xF).reshape(K, N // 8, 8).astype(np.uint64)
    word = np.zeros((K, N // 8), dtype=np.uint64)
    for j in range(8):
        word |= u[:, :, j] << np.uint64(4 * j)
    return word.astype(np.uint32).view(np.int32)


def unpack_int4(packed) -> np.ndarray:
    """Inverse of pack_int4: int32 [K, N/8] -> int8 [K, N] with values in [-8,7]."""
    p = np.asarray(packed.cpu().numpy() if isinstance(packed, torch.Tensor) else packed).view(np.uint32)
    K, W = p.shape
    out = np.empty((K, W, 8), dtype=np.int8)
    for j in range(8):
        nib = ((p >> np.uint32(4 * j)) & np.uint32(0xF)).astype(np.int8)
        out[:, :, j] = np.where(nib >= 8, nib - 16, nib)
    return out.reshape(K, W * 8)


def antiquant_weight(packed, antiquant_scale, antiquant_offset, group: int) -> np.ndarray:
    """W[k,n] = (w[k,n] + offset[k//group, n]) * scale[k//group, n] in fp64."""
    w = unpack_int4(packed).astype(np.float64)
    K, N = w.shape
    g = group if group > 0 else K
    s = _f32(antiquant_scale).astype(np.float64).reshape(-1, N)
    s = np.repeat(s, g, axis=0)[:K]
    if antiquant_offset is not None:
        o = _f32(antiquant_offset).astype(np.float64).reshape(-1, N)
        w = w + np.repeat(o, g, axis=0)[:K]
    return w * s


def weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset=None, *, bias=None,
                             antiquant_group_size=0) -> np.ndarray:
    """x @ antiquant(weight) (+ bias) in fp64; callers compare with a stated tolerance.

    Golden style: host matmul in higher precision than the device op
    (test/test_custom_ops/test_all_gather_base_mm.py:72-78).
    """
    W = antiquant_weight(weight, antiquant_scale, antiquant_offset, antiquant_group_size)
    y = _f32(x).astype(np.float64) @ W
    if bias is not None:
        y = y + _f32(bias).astype(np.float64)[None, :]
    return y


# ---------------------------------------------------------------------------
# npu_mm_all_reduce_base
# ---------------------------------------------------------------------------


def mm_all_reduce(x1_list, x2_list, scale, pertoken_list, *, bias=None, output_dtype=torch.bfloat16):
    """Row-parallel W8A8 matmul + allreduce(sum).

    Follows test/test_custom_ops/test_mm_reduce_scatter_base.py:69-81 (matmul
    per rank on the host, sum over ranks, cast): here each rank's dequantized
    partial is first rounded to the output dtype, as the device op does, then
    the partials are summed in fp32.  Returns (fp32 sum as numpy, rounded tensor).
    """
    total = None
    for r, (a, b) in enumerate(zip(x1_list, x2_list)):
        pt = None if pertoken_list is None else pertoken_list[r]
        part = quant_matmul(a, b, scale, pertoken_scale=pt, bias=bias if r == 0 else None,
                            output_dtype=output_dtype).to(torch.float32).numpy()
        total = part if total is None else (total + part).astype(np.float32)
    return total, _round_to(total, output_dtype)


# ---------------------------------------------------------------------------
# npu_mm_reduce_scatter_base / npu_all_gather_base_mm (present in the reference, with tests)
# ---------------------------------------------------------------------------


def mm_reduce_scatter(x1_list, x2_list, world_size, *, bias=None):
    """Per-rank expected outputs of npu_mm_reduce_scatter_base.

    Restates ``_construct_excepted_result`` of test/test_custom_ops/test_mm_reduce_scatter_base.py:69-81:
    fp32 matmul per rank, partial results added in rank order in fp32, one cast to the input dtype, rows
    sliced by rank.  (``bias`` - not exercised by the reference test - is added to the fp32 sum once.)
    Pinned: tests/golden/mc2_reference.npz holds outputs of the reference's own function.
    """
    out = None
    for i in range(world_size):
        out_single = torch.matmul(x1_list[i].to(torch.float), x2_list[i].to(torch.float))
        out = out_single if out is None else torch.add(out, out_single)
    if bias is not None:
        out = out + bias.to(torch.float)[None, :]
    out = out.to(x1_list[0].dtype)
    index = x1_list[0].shape[0] // world_size
    return [out[index * i:index * (i + 1), :] for i in range(world_size)]


def all_gather_mm(x1_list, x2_list, world_size, *, bias=None):
    """(per-rank expected matmul outputs, gathered x1) of npu_all_gather_base_mm.

    Restates ``_construct_excepted_result`` of test/test_custom_ops/test_all_gather_base_mm.py:72-78:
    x1 of all ranks concatenated along the rows, fp32 matmul with the rank's own x2, one cast.
    Pinned by tests/golden/mc2_reference.npz like mm_reduce_scatter.
    """
    gather_out = torch.cat(x1_list)
    out_list = []
    for i in range(world_size):
        y = torch.matmul(gather_out.to(torch.float), x2_list[i].to(torch.float))
        if bias is not None:
            y = y + bias.to(torch.float)[None, :]
        out_list.append(y.to(gather_out.dtype))
    return out_list, gather_out


# ---------------------------------------------------------------------------
# seeded synthetic inputs (value distributions of the benchmark configurations)
# ---------------------------------------------------------------------------


def make_w8a8_inputs(M: int, K: int, N: int, seed: int, *, dtype=torch.bfloat16, with_bias=True):
    """x ~ N(0,1) in `dtype`; weight int8 uniform in [-127,127]; per-channel scale fp32
    uniform in [1e-3,1e-2]; bias ~ N(0,0.1) in `dtype`.  All from one seed."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g, dtype=torch.float32).to(dtype)
    w = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    scale = torch.empty(N, dtype=torch.float32).uniform_(1e-3, 1e-2, generator=g)
    bias = (torch.randn(N, generator=g, dtype=torch.float32) * 0.1).to(dtype) if with_bias else None
    return x, w, scale, bias


def make_w4a16_inputs(M: int, K: int, N: int, seed: int, *, group=128, dtype=torch.bfloat16):
    """x ~ N(0,1); int4 weights uniform in [-8,7] packed 8 per int32 along N; per-group
    scale uniform in [5e-3,2e-2] and offset uniform in [-1,1], both in `dtype`."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g, dtype=torch.float32).to(dtype)
    w = torch.randint(-8, 8, (K, N), generator=g, dtype=torch.int8)
    packed = torch.from_numpy(pack_int4(w.numpy()))
    ng = K // group
    scale = torch.empty((ng, N), dtype=torch.float32).uniform_(5e-3, 2e-2, generator=g).to(dtype)
    offset = torch.empty((ng, N), dtype=torch.float32).uniform_(-1.0, 1.0, generator=g).to(dtype)
    return x, packed, scale, offset


# ---------------------------------------------------------------------------
# the reference-style CPU path (timed as the CPU baseline)
# ---------------------------------------------------------------------------


def cpu_path_w8a8(x: torch.Tensor, w_f32: torch.Tensor, scale: torch.Tensor, bias, output_dtype=torch.bfloat16):
    """dynamic quant + W8A8 matmul + dequantization with multi-threaded torch CPU operators.

    This is the computation the reference's tests run on the host as their golden
    (``torch.matmul(x1.to(torch.float), x2.to(torch.float))``,
    test/test_custom_ops/test_mm_reduce_scatter_base.py:74): fp32 BLAS on int8-valued
    operands.  The product is evaluated in K chunks of 1024 so that every fp32 partial sum
    is an exact integer (1024 * 127 * 128 < 2^24) and the chunks are added in int32; the
    result equals ``quant_matmul(dynamic_quant(x), w, ...)`` bit for bit.
    `w_f32` is the int8 weight already converted to float32 (weights are static).
    """
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    s = amax / 127.0
    safe = torch.where(s == 0, torch.ones_like(s), s)
    q = torch.clamp(torch.round(xf / safe[:, None]), -128, 127)
    q = torch.where(s[:, None] == 0, torch.zeros_like(q), q)
    K = q.shape[1]
    acc = None
    for k0 in range(0, K, 1024):
        part = torch.matmul(q[:, k0:k0 + 1024], w_f32[k0:k0 + 1024]).to(torch.int32)
        acc = part if acc is None else acc + part
    v = acc.to(torch.float32) * scale[None, :]
    v = v * s[:, None]
    if bias is not None:
        v = v + bias.float()[None, :]
    return v.to(output_dtype), q.to(torch.int8), s
