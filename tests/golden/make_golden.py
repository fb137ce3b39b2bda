"""Regenerates tests/golden/*.npz from the CPU oracle.

The reference holds no golden vectors for these operators (they are absent
from its snapshot), so the fixtures pin the ORACLE: any later change of its
arithmetic shows up as a fixture mismatch.  Inputs are seeded; outputs are
stored in full for the small cases and as SHA-256 digests for configuration 1
(x bf16 [128,1024], weight int8 [1024,1024]).

Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import qmm_oracle as O  # noqa: E402

OUT = Path(__file__).resolve().parent


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def small_w8a8():
    x, w, scale, bias = O.make_w8a8_inputs(8, 64, 32, seed=7)
    x[3].zero_()  # a zero row: scale 0, q 0
    q, s = O.dynamic_quant(x)
    acc = O.quant_matmul(q, w, scale, output_dtype=torch.int32)
    y = O.quant_matmul(q, w, scale, pertoken_scale=s, bias=bias, output_dtype=torch.bfloat16)
    yh = O.quant_matmul(q, w, scale, pertoken_scale=s, bias=None, output_dtype=torch.float16)
    np.savez(OUT / "w8a8_small.npz", x_bits=bits16(x), w=w.numpy(), scale=scale.numpy(), bias_bits=bits16(bias),
             q=q.numpy(), s=s.numpy(), acc=acc.numpy(), y_bits=bits16(y), yh_bits=bits16(yh))


def small_w4a16():
    x, packed, scale, offset = O.make_w4a16_inputs(4, 256, 64, seed=11, group=128)
    y = O.weight_quant_batchmatmul(x, packed, scale, offset, antiquant_group_size=128)
    np.savez(OUT / "w4a16_small.npz", x_bits=bits16(x), packed=packed.numpy(), scale_bits=bits16(scale),
             offset_bits=bits16(offset), w_int=O.unpack_int4(packed), y=y)


def config1_digests():
    x, w, scale, bias = O.make_w8a8_inputs(128, 1024, 1024, seed=1234)
    q, s = O.dynamic_quant(x)
    acc = O.quant_matmul(q, w, scale, output_dtype=torch.int32)
    y = O.quant_matmul(q, w, scale, pertoken_scale=s, bias=bias, output_dtype=torch.bfloat16)
    lines = [f"x {sha(bits16(x))}", f"w {sha(w.numpy())}", f"scale {sha(scale.numpy())}", f"bias {sha(bits16(bias))}",
             f"q {sha(q.numpy())}", f"s {sha(s.numpy())}", f"acc {sha(acc.numpy())}", f"y {sha(bits16(y))}"]
    (OUT / "config1_sha256.txt").write_text("\n".join(lines) + "\n")


if __name__ == "__main__":
    small_w8a8()
    small_w4a16()
    config1_digests()
    print("golden fixtures written to", OUT)
