"""Writes tests/golden/rms_norm_reference.npz: outputs of the REFERENCE's own numpy golden for
npu_rms_norm on seeded inputs.

The golden lives in the reference's test file as a method (``TestNPURmsNorm.supported_op_exec``,
test/test_custom_ops/test_npu_rms_norm.py:10-18).  The file imports torch_npu at the top, which is not
installable here, so the method's source is taken out of the file with ``ast`` and executed unmodified
with numpy alone.  Run in a container that has the reference tree:

    python tests/golden/make_rms_norm_golden.py <path of the reference tree>
"""
import ast
import sys
from pathlib import Path

import numpy as np


def reference_golden(ref_root: Path):
    path = ref_root / "test" / "test_custom_ops" / "test_npu_rms_norm.py"
    tree = ast.parse(path.read_text())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "supported_op_exec":
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"np": np}
            exec(compile(mod, str(path), "exec"), ns)
            return lambda x, gamma: ns["supported_op_exec"](None, x, gamma)
    raise SystemExit(f"supported_op_exec not found in {path}")


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref_root = Path(sys.argv[1])
    golden = reference_golden(ref_root)
    rng = np.random.default_rng(20240607)
    out = {}
    # the reference test's distribution (uniform(0, 100), float32) at reduced sizes, plus a signed case
    for name, rows, cols, lo, hi in (("a", 8, 256, 0.0, 100.0), ("b", 1, 12288, 0.0, 100.0), ("c", 5, 200, -3.0, 3.0)):
        x = rng.uniform(lo, hi, [rows, cols]).astype(np.float32)
        gamma = rng.uniform(lo, hi, [cols]).astype(np.float32)
        y, rstd = golden(x, gamma)
        out[f"{name}_x"], out[f"{name}_gamma"], out[f"{name}_y"], out[f"{name}_rstd"] = x, gamma, y, rstd
    dst = Path(__file__).resolve().parent / "rms_norm_reference.npz"
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
