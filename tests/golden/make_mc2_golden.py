"""Writes tests/golden/mc2_reference.npz: outputs of the REFERENCE's own golden functions for
npu_mm_reduce_scatter_base and npu_all_gather_base_mm on seeded inputs.

Both goldens are methods named ``_construct_excepted_result`` in the reference's test files
(test/test_custom_ops/test_mm_reduce_scatter_base.py:69-81, test_all_gather_base_mm.py:72-78).  The files
import torch_npu, which is not installable here, so the methods' source is taken out with ``ast`` and
executed unmodified with torch alone.  Shapes and value range are the reference tests' own (float16,
uniform(-1, 1), [128, 512] @ [512, 256] and [16, 512] @ [512, 256], 8 ranks), plus 2- and 4-rank cases.
The inputs are not stored: ``mc2_inputs`` regenerates them from the seed (the tests import it); the file
holds the reference's outputs, in full for 2 and 4 ranks and as SHA-256 digests for 8.

    python tests/golden/make_mc2_golden.py <path of the reference tree>
"""
import ast
import sys
from pathlib import Path

import numpy as np
import torch


def reference_method(path: Path, name: str):
    tree = ast.parse(path.read_text())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == name:
            ns = {"torch": torch}
            exec(compile(ast.Module(body=[node], type_ignores=[]), str(path), "exec"), ns)
            return ns[name]
    raise SystemExit(f"{name} not found in {path}")


SEED = 20240608


def mc2_inputs(world: int):
    """(rs_x1, rs_x2, ag_x1, ag_x2) lists of float16 tensors for `world` ranks, from the seed alone."""
    g = torch.Generator().manual_seed(SEED + world)
    u = lambda *shape: (torch.rand(shape, generator=g) * 2 - 1).to(torch.float16)  # noqa: E731
    rs_x1 = [u(128, 512) for _ in range(world)]
    rs_x2 = [u(512, 256) for _ in range(world)]
    ag_x1 = [u(16, 512) for _ in range(world)]
    ag_x2 = [u(512, 256) for _ in range(world)]
    return rs_x1, rs_x2, ag_x1, ag_x2


def digest(tensors) -> str:
    import hashlib

    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.int16).numpy().tobytes())
    return h.hexdigest()


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = Path(sys.argv[1]) / "test" / "test_custom_ops"
    rs = reference_method(ref / "test_mm_reduce_scatter_base.py", "_construct_excepted_result")
    ag = reference_method(ref / "test_all_gather_base_mm.py", "_construct_excepted_result")
    out = {}
    bits = lambda t: t.contiguous().view(torch.int16).numpy()  # noqa: E731
    for world in (2, 4, 8):
        rs_x1, rs_x2, ag_x1, ag_x2 = mc2_inputs(world)
        rs_exp = rs(None, rs_x1, rs_x2, world)
        ag_exp, gathered = ag(None, ag_x1, ag_x2, world)
        assert torch.equal(gathered, torch.cat(ag_x1))
        if world < 8:
            out[f"rs{world}_out"] = np.stack([bits(t) for t in rs_exp])
            out[f"ag{world}_out"] = np.stack([bits(t) for t in ag_exp])
        out[f"rs{world}_sha256"] = np.array(digest(rs_exp))
        out[f"ag{world}_sha256"] = np.array(digest(ag_exp))
    dst = Path(__file__).resolve().parent / "mc2_reference.npz"
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
