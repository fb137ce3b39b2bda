"""The CPU oracle against hand-checkable cases, the committed golden fixtures
and the golden formula of the reference's own matmul+collective tests."""
import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def _bits16(t):
    return t.contiguous().view(torch.int16).numpy()


def _from_bits(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).view(dtype)


def test_dynamic_quant_hand_checked(oracle):
    # amax = 127 -> scale exactly 1 -> q = rint(x): ties go to even
    x = torch.tensor([[127.0, -127.0, 0.5, 1.5, 2.5, -0.5, -1.5, 3.0]], dtype=torch.bfloat16)
    q, s = oracle.dynamic_quant(x)
    assert s.tolist() == [1.0]
    assert q.tolist() == [[127, -127, 0, 2, 2, 0, -2, 3]]
    # amax = 254 -> scale 2 -> halves
    x = torch.tensor([[254.0, 1.0, 3.0, 5.0, -7.0]], dtype=torch.bfloat16)
    q, s = oracle.dynamic_quant(x)
    assert s.tolist() == [2.0]
    assert q.tolist() == [[127, 0, 2, 2, -4]]


def test_dynamic_quant_zero_row_and_shapes(oracle):
    x = torch.zeros((2, 3, 16), dtype=torch.float16)
    x[1, 2, 5] = -3.0
    q, s = oracle.dynamic_quant(x)
    assert q.shape == (2, 3, 16) and s.shape == (2, 3)
    assert s[0, 0].item() == 0.0 and q[0].abs().sum().item() == 0
    assert q[1, 2, 5].item() == -127 and s[1, 2].item() == np.float32(3.0) / np.float32(127.0)
    q, s = oracle.dynamic_quant(torch.zeros((4, 0), dtype=torch.bfloat16))
    assert q.shape == (4, 0) and s.shape == (4,)


def test_dynamic_quant_division_not_reciprocal(oracle):
    """The formula is a true division by scale; multiplying by 127/amax differs on some inputs."""
    x, _, _, _ = oracle.make_w8a8_inputs(128, 1024, 8, seed=1234)
    q, s = oracle.dynamic_quant(x)
    xf = x.float().numpy()
    amax = np.abs(xf).max(axis=1)
    recip = (np.float32(127.0) / amax).astype(np.float32)
    q_recip = np.clip(np.rint(xf * recip[:, None]), -128, 127).astype(np.int8)
    assert (q.numpy() != q_recip).sum() > 0
    assert np.abs(q.numpy().astype(np.int32) - q_recip.astype(np.int32)).max() <= 1


def _round_f32(fr):
    """Fraction -> nearest float32 (ties to even), exactly."""
    from fractions import Fraction

    if fr == 0:
        return np.float32(0.0)
    sign = -1 if fr < 0 else 1
    a = abs(fr)
    e = a.numerator.bit_length() - a.denominator.bit_length()
    if Fraction(2) ** e > a:
        e -= 1
    if e < -126:
        e = -126  # subnormal range: fixed exponent
    scaled = a / Fraction(2) ** (e - 23)  # integer significand with 24 bits when normal
    n = scaled.numerator // scaled.denominator
    rem = scaled - n
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and n % 2 == 1):
        n += 1
    return np.float32(sign * float(Fraction(n) * Fraction(2) ** (e - 23)))


def test_fma_division_equals_ieee_division():
    """The division the dynamic-quant kernel runs on the FMA pipe: y = RN(1/s), q0 = RN(x*y),
    r = RN(x - q0*s) (one fma), q1 = RN(q0 + r*y) (one fma).  q0 is within two ulps of x/s, r carries at most
    one rounding, so q0 + r*y differs from the exact quotient by less than 2^-21 ulp and q1 = RN(x/s) unless the
    quotient sits that close to a rounding boundary without being on it.  Checked here with exact rational
    arithmetic on the operands the kernel sees (s = amax/127 of a 16-bit-float row, |x| <= amax, exact and near
    ties x/s = n + 1/2 included); the GPU tests run every pair of bf16 / f16 significands."""
    from fractions import Fraction

    rng = np.random.default_rng(7)
    checked = 0
    for _ in range(60):
        amax = np.float32(torch.tensor(abs(rng.normal()) * 3 + 0.5).to(torch.bfloat16).float().item())
        s = np.float32(amax) / np.float32(127.0)
        if (s.view(np.uint32) & 0x7FFFFF) == 0x7FFFFF:
            continue  # the kernel takes true divisions for an all-ones significand
        y = np.float32(1.0) / s
        xs = torch.tensor(rng.uniform(-1, 1, 48) * float(amax)).to(torch.bfloat16).float().numpy()
        # plus values that make exact or near ties: (n + 1/2) * s rounded to bf16
        n = rng.integers(-126, 126, 16).astype(np.float32)
        ties = torch.tensor((n + 0.5) * s).to(torch.bfloat16).float().numpy()
        for x in np.concatenate([xs, ties]).astype(np.float32):
            q0 = np.float32(x * y)
            r = _round_f32(Fraction(float(x)) - Fraction(float(q0)) * Fraction(float(s)))
            q1 = _round_f32(Fraction(float(q0)) + Fraction(float(r)) * Fraction(float(y)))
            assert q1 == np.float32(x) / s, (x, s)
            checked += 1
    assert checked > 3000


def test_quant_matmul_hand_checked(oracle):
    x1 = torch.tensor([[1, -2, 3], [127, 127, 127]], dtype=torch.int8)
    x2 = torch.tensor([[1, 0], [0, 1], [-1, 127]], dtype=torch.int8)
    acc = oracle.quant_matmul(x1, x2, None, output_dtype=torch.int32)
    assert acc.tolist() == [[-2, 379], [0, 127 * 128]]
    scale = torch.tensor([0.5, 0.25])
    pt = torch.tensor([2.0, 1.0])
    bias = torch.tensor([1.0, -1.0], dtype=torch.bfloat16)
    y = oracle.quant_matmul(x1, x2, scale, pertoken_scale=pt, bias=bias, output_dtype=torch.bfloat16)
    # fp32 values -1, 188.5, 1, 4063 -> bf16 (8 significant bits): 188.5 ties to even 188, 4063 -> 4064
    assert y.float().tolist() == [[-1.0, 188.0], [1.0, 4064.0]]
    bias_i = torch.tensor([10, -10], dtype=torch.int32)
    acc_b = oracle.quant_matmul(x1, x2, None, bias=bias_i, output_dtype=torch.int32)
    assert acc_b.tolist() == [[8, 369], [10, 127 * 128 - 10]]


def test_int_accumulation_matches_torch_int_mm(oracle):
    g = torch.Generator().manual_seed(3)
    a = torch.randint(-128, 128, (32, 4096), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (4096, 24), generator=g, dtype=torch.int8)
    assert np.array_equal(oracle.int8_matmul_exact(a, b), torch._int_mm(a, b).numpy())


def test_reference_golden_formula(oracle):
    """The reference's matmul+collective golden (fp32 matmul per rank, sum over ranks, cast:
    test_mm_reduce_scatter_base.py:69-81) coincides with the oracle while the fp32 sums are exact
    (K <= 1024: K * 127^2 < 2^24), with unit scales."""
    ranks = 4
    g = torch.Generator().manual_seed(9)
    xs = [torch.randint(-127, 128, (16, 256), generator=g, dtype=torch.int8) for _ in range(ranks)]
    ws = [torch.randint(-127, 128, (256, 24), generator=g, dtype=torch.int8) for _ in range(ranks)]
    out, magnitude = None, None
    for a, b in zip(xs, ws):
        single = torch.matmul(a.to(torch.float), b.to(torch.float))
        out = single if out is None else torch.add(out, single)
        magnitude = single.abs() if magnitude is None else magnitude + single.abs()
    total, _ = oracle.mm_all_reduce(xs, ws, torch.ones(24), None, output_dtype=torch.bfloat16)
    # each rank's partial is rounded to bf16 (relative error <= 2^-9) before the sum
    assert np.all(np.abs(total - out.numpy()) <= magnitude.numpy() * 2.0 ** -8)
    acc = sum(oracle.int8_matmul_exact(a, b).astype(np.int64) for a, b in zip(xs, ws))
    assert np.array_equal(acc, out.numpy().astype(np.int64))


def test_int4_pack_roundtrip(oracle):
    g = np.random.default_rng(0)
    w = g.integers(-8, 8, size=(64, 48))
    packed = oracle.pack_int4(w)
    assert packed.shape == (64, 6) and packed.dtype == np.int32
    assert np.array_equal(oracle.unpack_int4(packed), w)
    # nibble j of word i is column 8*i+j
    w2 = np.zeros((1, 8), dtype=np.int64)
    w2[0] = [1, 2, 3, 4, 5, 6, 7, -1]
    assert oracle.pack_int4(w2).view(np.uint32)[0, 0] == 0xF7654321


def test_w4a16_hand_checked(oracle):
    w = np.array([[1, -2, 0, 0, 0, 0, 0, 0], [3, 4, 0, 0, 0, 0, 0, 0]])
    packed = torch.from_numpy(oracle.pack_int4(w))
    scale = torch.full((1, 8), 0.5, dtype=torch.bfloat16)
    offset = torch.full((1, 8), 1.0, dtype=torch.bfloat16)
    x = torch.tensor([[2.0, -1.0]], dtype=torch.bfloat16)
    y = oracle.weight_quant_batchmatmul(x, packed, scale, offset, antiquant_group_size=2)
    # W = (w + 1) * 0.5 ; y = 2*W[0] - W[1]
    assert y[0, 0] == 2 * 1.0 - 2.0 and y[0, 1] == 2 * (-0.5) - 2.5 and y[0, 2] == 2 * 0.5 - 0.5


def test_golden_w8a8_small(oracle):
    g = np.load(GOLDEN / "w8a8_small.npz")
    x = _from_bits(g["x_bits"], torch.bfloat16)
    q, s = oracle.dynamic_quant(x)
    assert np.array_equal(q.numpy(), g["q"]) and np.array_equal(s.numpy(), g["s"])
    w, scale = torch.from_numpy(g["w"]), torch.from_numpy(g["scale"])
    bias = _from_bits(g["bias_bits"], torch.bfloat16)
    assert np.array_equal(oracle.quant_matmul(q, w, scale, output_dtype=torch.int32).numpy(), g["acc"])
    y = oracle.quant_matmul(q, w, scale, pertoken_scale=s, bias=bias, output_dtype=torch.bfloat16)
    assert np.array_equal(_bits16(y), g["y_bits"])
    yh = oracle.quant_matmul(q, w, scale, pertoken_scale=s, output_dtype=torch.float16)
    assert np.array_equal(_bits16(yh), g["yh_bits"])


def test_golden_w4a16_small(oracle):
    g = np.load(GOLDEN / "w4a16_small.npz")
    packed = torch.from_numpy(g["packed"])
    assert np.array_equal(oracle.unpack_int4(packed), g["w_int"])
    y = oracle.weight_quant_batchmatmul(_from_bits(g["x_bits"], torch.bfloat16), packed,
                                        _from_bits(g["scale_bits"], torch.bfloat16),
                                        _from_bits(g["offset_bits"], torch.bfloat16), antiquant_group_size=128)
    assert np.array_equal(y, g["y"])


def test_golden_config1_digests(oracle):
    want = dict(line.split() for line in (GOLDEN / "config1_sha256.txt").read_text().splitlines())

    def sha(a):
        return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()

    x, w, scale, bias = oracle.make_w8a8_inputs(128, 1024, 1024, seed=1234)
    assert sha(_bits16(x)) == want["x"] and sha(w.numpy()) == want["w"]
    q, s = oracle.dynamic_quant(x)
    assert sha(q.numpy()) == want["q"] and sha(s.numpy()) == want["s"]
    acc = oracle.quant_matmul(q, w, scale, output_dtype=torch.int32)
    assert sha(acc.numpy()) == want["acc"]
    y = oracle.quant_matmul(q, w, scale, pertoken_scale=s, bias=bias, output_dtype=torch.bfloat16)
    assert sha(_bits16(y)) == want["y"]


def test_ulp_distance(oracle):
    a = torch.tensor([1.0, -1.0, 0.0, 2.0], dtype=torch.bfloat16)
    b = torch.tensor([1.0078125, -1.0078125, -0.0, 2.0], dtype=torch.bfloat16)
    assert oracle.bf16_ulp_distance(a, b).tolist() == [1, 1, 0, 0]


def test_rms_norm_pinned_to_reference_golden():
    """oracle.rms_norm against outputs of the reference's own numpy golden (executed from the reference's
    test file by tests/golden/make_rms_norm_golden.py): bit for bit."""
    from oracle import qmm_oracle as O

    g = np.load(GOLDEN / "rms_norm_reference.npz")
    for name in ("a", "b", "c"):
        y, rstd = O.rms_norm(torch.from_numpy(g[f"{name}_x"]), torch.from_numpy(g[f"{name}_gamma"]), 1e-6)
        assert np.array_equal(y.numpy(), g[f"{name}_y"]) and np.array_equal(rstd.numpy(), g[f"{name}_rstd"])


def test_rms_norm_dynamic_quant_composition():
    from oracle import qmm_oracle as O

    x = (torch.randn((6, 384), generator=torch.Generator().manual_seed(3)) * 2).to(torch.bfloat16)
    gamma = (torch.rand(384, generator=torch.Generator().manual_seed(4)) + 0.5).to(torch.bfloat16)
    q, s, rstd = O.rms_norm_dynamic_quant(x, gamma)
    y, rstd2 = O.rms_norm(x, gamma)
    q2, s2 = O.dynamic_quant(y)
    assert y.dtype == torch.bfloat16 and torch.equal(q, q2) and torch.equal(s, s2) and torch.equal(rstd, rstd2)
    assert rstd.shape == (6, 1)


def test_dynamic_quant_non_finite_rows():
    """Pinned choices: an infinite element gives an infinite scale (finite elements -> 0, the infinity itself
    -> 0 because Inf/Inf is NaN); a NaN gives a NaN scale and an all-zero row."""
    from oracle import qmm_oracle as O

    x = torch.tensor([[1.0, -2.0, float("inf"), 4.0], [1.0, float("nan"), -3.0, 0.5], [1.0, 2.0, -4.0, 0.0]]).to(torch.bfloat16)
    q, s = O.dynamic_quant(x)
    assert torch.isinf(s[0]) and torch.isnan(s[1]) and s[2].item() == np.float32(4.0) / np.float32(127.0)
    assert q[0].tolist() == [0, 0, 0, 0] and q[1].tolist() == [0, 0, 0, 0] and q[2].tolist() == [32, 64, -127, 0]


def test_mc2_oracles_pinned_to_reference_golden():
    """oracle.mm_reduce_scatter / all_gather_mm against outputs of the reference's own golden functions
    (executed from its test files by tests/golden/make_mc2_golden.py): bit for bit, 2, 4 and 8 ranks."""
    import importlib.util

    from oracle import qmm_oracle as O

    spec = importlib.util.spec_from_file_location("make_mc2_golden", GOLDEN / "make_mc2_golden.py")
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    g = np.load(GOLDEN / "mc2_reference.npz")
    for world in (2, 4, 8):
        rs_x1, rs_x2, ag_x1, ag_x2 = mk.mc2_inputs(world)
        rs = O.mm_reduce_scatter(rs_x1, rs_x2, world)
        ag, gathered = O.all_gather_mm(ag_x1, ag_x2, world)
        assert mk.digest(rs) == str(g[f"rs{world}_sha256"]) and mk.digest(ag) == str(g[f"ag{world}_sha256"])
        assert rs[0].shape == (128 // world, 256) and ag[0].shape == (16 * world, 256)
        assert torch.equal(gathered, torch.cat(ag_x1))
        if world < 8:
            for r in range(world):
                assert np.array_equal(rs[r].contiguous().view(torch.int16).numpy(), g[f"rs{world}_out"][r])
                assert np.array_equal(ag[r].contiguous().view(torch.int16).numpy(), g[f"ag{world}_out"][r])
