"""The drop-in boundary without a GPU: the C-ABI library loads and exports every symbol the
header declares, argument validation answers with status codes and messages, the generated
torch-library registration carries the operator schemas, and the codegen reproduces the
reference's declaration style."""
import ctypes
import re
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
PKG_DIR = ROOT / "ascend-python_b200"


def test_library_exports_every_declared_symbol(capi):
    header = (ROOT / "include" / "qmm_b200.h").read_text()
    declared = set(re.findall(r"QMM_API\s+[\w\s\*]+?\b(qmm_\w+)\s*\(", header))
    assert declared == set(capi.EXPORTED_SYMBOLS)
    lib = capi.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.qmm_version() >= 100


def test_validation_needs_no_gpu(capi):
    lib = capi.lib()
    rc = lib.qmm_dynamic_quant(None, capi.DTYPE_BF16, -1, 4, 4, None, 4, None, None)
    assert rc == 1 and b"non-negative" in lib.qmm_last_error()
    rc = lib.qmm_dynamic_quant(None, capi.DTYPE_BF16, 0, 4, 4, None, 4, None, None)
    assert rc == 0  # empty input: nothing to launch
    n = ctypes.c_size_t(123)
    assert lib.qmm_quant_matmul_workspace_size(8, 256, 512, capi.ALGO_AUTO, ctypes.byref(n)) == 0
    assert n.value == 2 * 16 * 128 * 4 + 256  # two 128-column tiles x 16 padded rows of int32 + counters
    assert lib.qmm_quant_matmul_workspace_size(4096, 256, 512, capi.ALGO_AUTO, ctypes.byref(n)) == 0
    assert n.value == 0  # prefill shapes need no scratch
    rc = lib.qmm_quant_matmul(None, 8, None, 8, 1, None, 0, None, None, -1, None, 7, 8, 4, 8, 8, 0, None, 0, None)
    assert rc == 1 and b"output dtype" in lib.qmm_last_error()
    rc = lib.qmm_weight_quant_batchmatmul(None, capi.DTYPE_BF16, 8, None, 1, None, None, 128, None, None, 12, 1, 12,
                                          8, None, 0, None)
    assert rc == 1 and b"multiple of 8" in lib.qmm_last_error()
    nr, rk = ctypes.c_int(0), ctypes.c_int(0)
    rc = lib.qmm_comm_info(b"no-such-comm", ctypes.byref(nr), ctypes.byref(rk))
    assert rc == 5 and b"not registered" in lib.qmm_last_error()
    rc = lib.qmm_mm_all_reduce(None, 8, None, 8, 1, None, 8, None, None, -1, None, 0, 8, 4, 8, 8, b"c", b"max", 0,
                               None, 0, None)
    assert rc == 1 and b"reduce_op" in lib.qmm_last_error()
    # peer memory of the allreduce: the size is plain arithmetic (64 KiB of flags + two halves of equal size,
    # each large enough for the partials as [ranks][rows per rank rounded up to 32][N] and for the reduced
    # [M][N]; 16-bit elements, 256-byte rounding)
    need = ctypes.c_size_t(0)
    assert lib.qmm_comm_peer_memory_size(4096, 8192, 8, ctypes.byref(need)) == 0
    assert need.value == 65536 + 2 * 4096 * 8192 * 2
    assert lib.qmm_comm_peer_memory_size(1000, 768, 3, ctypes.byref(need)) == 0
    assert need.value == 65536 + 2 * max(3 * 352 * 768 * 2, 1000 * 768 * 2)
    assert lib.qmm_comm_peer_memory_size(-1, 8, 2, ctypes.byref(need)) == 1
    regions = (ctypes.c_void_p * 2)(None, None)
    rc = lib.qmm_comm_attach_peer_memory(b"no-such-comm", regions, None, 1 << 20)
    assert rc == 5 and b"not registered" in lib.qmm_last_error()
    # the prepacked W4A16 format: 8704-byte blocks of 128 columns x 128 k, an even number of blocks along K
    assert capi.w4a16_prepack_size(28672, 8192, 128) == 224 * 64 * 8704
    assert capi.w4a16_prepack_size(200, 384, 128) == 2 * 4 * 8704       # 200 -> 2 column tiles, 3 -> 4 blocks
    assert capi.w4a16_prepack_size(256, 256, 64) == 0                  # group below 128: not covered
    sizes = []
    for M in (1, 2, 16, 64):
        assert lib.qmm_weight_quant_batchmatmul_prepacked_workspace_size(M, 28672, 8192, ctypes.byref(n)) == 0
        assert n.value >= 65536 and n.value % 256 == 0
        sizes.append(n.value)
    assert sizes == sorted(sizes)
    assert lib.qmm_weight_quant_batchmatmul_prepacked_workspace_size(0, 28672, 8192, ctypes.byref(n)) == 0 and n.value == 0


def test_missing_library_fails_loudly(capi, monkeypatch):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", Path("/nonexistent/libqmm_b200.so"))
    with pytest.raises(capi.QmmError, match="no fallback"):
        capi.lib()


def test_ops_registered_with_reference_signatures(pkg):
    ops = pkg.load_ops()
    s = str(ops.npu_quant_matmul.default._schema)
    assert s == ("npu::npu_quant_matmul(Tensor x1, Tensor x2, Tensor scale, *, Tensor? offset=None, "
                 "Tensor? pertoken_scale=None, Tensor? bias=None, ScalarType? output_dtype=None) -> Tensor")
    assert "-> (Tensor, Tensor)" in str(ops.npu_dynamic_quant.default._schema)
    assert "str hcom" in str(ops.npu_mm_all_reduce_base.default._schema)
    assert 'str reduce_op="sum"' in str(ops.npu_mm_all_reduce_base.default._schema)
    assert "int antiquant_group_size=0" in str(ops.npu_weight_quant_batchmatmul.default._schema)
    # the reference's own entries, verbatim (op_plugin/config/v2r1/op_plugin_functions.yaml:2310-2313, :2113)
    assert str(ops.npu_mm_reduce_scatter_base.default._schema) == (
        'npu::npu_mm_reduce_scatter_base(Tensor self, Tensor x2, str hcom, int world_size, *, str reduce_op="sum", '
        "Tensor? bias=None, int comm_turn=0) -> Tensor")
    assert str(ops.npu_all_gather_base_mm.default._schema) == (
        "npu::npu_all_gather_base_mm(Tensor self, Tensor x2, str hcom, int world_size, *, Tensor? bias=None, "
        "int gather_index=0, bool gather_output=True, int comm_turn=0) -> (Tensor, Tensor)")
    assert str(ops.npu_rms_norm.default._schema) == \
        "npu::npu_rms_norm(Tensor self, Tensor gamma, float epsilon=9.9999999999999995e-07) -> (Tensor, Tensor)"
    # CUDA is the only backend: a CPU tensor has nowhere to go
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.npu_dynamic_quant(torch.zeros(2, 8, dtype=torch.bfloat16))


def test_torch_npu_shim_names(pkg):
    sys.path.insert(0, str(PKG_DIR))
    try:
        import torch_npu
    finally:
        sys.path.pop(0)
    for name in ("npu_dynamic_quant", "npu_quant_matmul", "npu_weight_quant_batchmatmul", "npu_mm_all_reduce_base",
                 "npu_mm_reduce_scatter_base", "npu_all_gather_base_mm", "npu_rms_norm", "npu_rms_norm_dynamic_quant",
                 "get_comm_name"):
        assert callable(getattr(torch_npu, name))
    assert torch_npu.comm_name_for("tp", 8) == "qmm_comm_tp_8"


def test_codegen_declarations(tmp_path):
    sys.path.insert(0, str(PKG_DIR))
    try:
        from codegen import gen_backend_stubs as gen
    finally:
        sys.path.pop(0)
    op = gen.parse_schema("npu_mm_reduce_scatter_base(Tensor self, Tensor x2, str hcom, int world_size, *, "
                          "str reduce_op='sum', Tensor? bias=None, int comm_turn=0) -> Tensor", "op_api")
    # declaration style of the reference's generated OpApiInterface.h
    assert op.signature(True) == ("at::Tensor npu_mm_reduce_scatter_base(const at::Tensor &self, const at::Tensor &x2, "
                                  "c10::string_view hcom, int64_t world_size, c10::string_view reduce_op=\"sum\", "
                                  "const c10::optional<at::Tensor> &bias=c10::nullopt, int64_t comm_turn=0)")
    op2 = gen.parse_schema("f(Tensor a, *, ScalarType? dt=None, bool flag=False, float eps=1e-6) -> (Tensor, Tensor)",
                           ["op_api"])
    assert op2.cpp_return() == "::std::tuple<at::Tensor,at::Tensor>"
    assert "c10::optional<at::ScalarType> dt=c10::nullopt" in op2.signature(True)
    assert "bool flag=false" in op2.signature(True) and "double eps=1e-6" in op2.signature(True)
    with pytest.raises(ValueError):
        gen.parse_schema("f(Dimname d) -> Tensor", "op_api")
    ops = gen.run(PKG_DIR / "op_plugin" / "config" / "op_plugin_functions.yaml", tmp_path)
    assert [o.name for o in ops] == ["npu_dynamic_quant", "npu_quant_matmul", "npu_weight_quant_batchmatmul",
                                     "npu_mm_all_reduce_base", "npu_rms_norm", "npu_rms_norm_dynamic_quant",
                                     "npu_mm_reduce_scatter_base", "npu_all_gather_base_mm"]
    lib_cpp = (tmp_path / "TorchLibrary.cpp").read_text()
    assert "TORCH_LIBRARY_FRAGMENT(npu, m)" in lib_cpp and "TORCH_LIBRARY_IMPL(npu, CUDA, m)" in lib_cpp
    assert "return op_api::npu_quant_matmul(x1, x2, scale, offset, pertoken_scale, bias, output_dtype);" in \
        (tmp_path / "OpInterface.cpp").read_text()
    bad = tmp_path / "bad.yaml"
    bad.write_text("official:\ncustom:\n")
    with pytest.raises(AssertionError, match="symint"):
        gen.parse_native_yaml(bad)
