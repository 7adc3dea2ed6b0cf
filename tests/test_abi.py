"""The C-ABI library loads on a machine without a GPU and exports every function that
include/mlel_b200.h declares (no compute is called here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "mlel_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlel_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(mlel):
    lib = mlel.lib()
    names = declared_functions()
    assert len(names) > 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_registry(mlel):
    names = mlel.tosa_op_names()
    assert len(names) == 66  # graph/graph_tosa_1_0_ext_inst.cpp:41-108
    assert mlel.ext_inst_set_registered("TOSA.001000.1")
    assert not mlel.ext_inst_set_registered("TOSA.000080.2")
    for op in ("CONV2D", "DEPTHWISE_CONV2D", "MATMUL", "RESCALE", "AVG_POOL2D", "MAX_POOL2D", "TABLE", "TRANSPOSE",
               "CONCAT", "CLAMP", "ADD", "SUB", "MUL", "REDUCE_SUM", "REDUCE_MAX", "CAST", "RESHAPE", "SLICE", "PAD"):
        assert op in names and mlel.tosa_op_supported(op)
    assert all(mlel.tosa_op_supported(op) for op in names)
    assert not mlel.tosa_op_supported("NOT_A_TOSA_OPERATOR")
    lib = mlel.lib()
    assert lib.mlel_tosa_lookup(b"TOSA.001000.1", b"CONV2D") == names.index("CONV2D")
    assert lib.mlel_tosa_lookup(b"TOSA.000080.2", b"CONV2D") == -1
    assert lib.mlel_tosa_lookup(b"TOSA.001000.1", b"NOT_A_TOSA_OPERATOR") == -1


def test_errors_are_status_codes_not_exceptions(mlel):
    p = mlel.Pipeline()
    a = p.bind_external(0, 0, mlel.I8, (1, 4, 4, 4))
    import pytest
    with pytest.raises(mlel.MlelError) as e:  # fp16 accumulate is not built: FEATURE_NOT_PRESENT
        w = p.composite_constant(__import__("numpy").zeros((4, 1, 1, 4), "int8"))
        b = p.composite_constant(__import__("numpy").zeros((4,), "int32"))
        o = p.make_tensor(mlel.I32, (1, 4, 4, 4))
        p.conv2d(a, o, w, b, [0] * 4, [1, 1], [1, 1], 0, 0, acc_type=2)
    assert e.value.status == -8
    with pytest.raises(mlel.MlelError) as e:
        p.lower_spvasm("this is not spir-v")
    assert e.value.status == -13
    with pytest.raises(mlel.MlelError):
        p.get_external(3, 3)
    with pytest.raises(mlel.MlelError):
        p.bind_external(0, 9, mlel.I8, (1, 2, 3, 4, 5, 6, 7))  # rank > 6


def test_library_has_no_oracle_dependency():
    import subprocess
    out = subprocess.run(["ldd", os.path.join(ROOT, "ai-ml-emulation-layer-for-vulkan_b200", "libmlel_b200.so")],
                         capture_output=True, text=True).stdout
    assert "oracle" not in out


def test_tuning_keys_and_values(mlel):
    """mlel_set_tuning takes exactly the documented keys and values; anything else is an error and changes nothing.
    (No GPU needed: the settings are read when a kernel is launched.)"""
    lib = mlel.lib()
    defaults = {b"pair_kernel": 1, b"pair_tile_pixels": 0, b"oc_tile_pixels": 0, b"oc_tile_rule": 3,
                b"dependent_launch": 1, b"tile_progress": 7}
    allowed = {b"pair_kernel": [0, 1, 2], b"pair_tile_pixels": [0, 128, 192, 256], b"oc_tile_pixels": [0, 128, 192, 256],
               b"oc_tile_rule": list(range(9)), b"dependent_launch": [0, 1], b"tile_progress": list(range(8))}
    refused = {b"pair_kernel": [-1, 3], b"pair_tile_pixels": [64, 100], b"oc_tile_pixels": [96, 512],
               b"oc_tile_rule": [9, -1], b"tile_progress": [8, -1]}
    try:
        for key, values in allowed.items():
            for v in values:
                assert lib.mlel_set_tuning(key, v) == 0, (key, v)
        for key, values in refused.items():
            for v in values:
                assert lib.mlel_set_tuning(key, v) != 0, (key, v)
        assert lib.mlel_set_tuning(b"no_such_key", 1) != 0
        assert lib.mlel_set_tuning(None, 1) != 0
    finally:
        for key, v in defaults.items():
            assert lib.mlel_set_tuning(key, v) == 0
