"""B200-native quantized-matmul operators behind the op-plugin operator API.

Layout of this package:

* ``csrc/``       hand-written sm_100a CUDA kernels and the C ABI (``include/qmm_b200.h``)
* ``op_plugin/``  C++ operator host code + yaml op registry (mirrors the reference's
                  ``op_plugin/ops`` + ``op_plugin/config``), registered as ``torch.ops.npu.*``
* ``codegen/``    yaml -> dispatch stubs + TORCH_LIBRARY registration
* ``torch_npu/``  call-site shim: ``torch_npu.npu_quant_matmul(...)`` etc.
* ``capi.py``     ctypes binding of the C ABI (tests, benchmarks)
* ``build.py``    in-tree build of ``lib/*.so``

The directory name contains a hyphen, so it is loaded by path (see
``__graft_entry__.load_package``) under the module name ``ascend_python_b200``.
"""
from . import capi  # noqa: F401


def load_ops():
    """Load the operator library; afterwards ``torch.ops.npu.npu_*`` exist.  Raises if it is not built."""
    from .ops_loader import load

    return load()
