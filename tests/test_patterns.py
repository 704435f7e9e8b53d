"""The reference's decode-matmul pattern names as a table (host logic, CPU): the six base names
and the sixteen residual variants of python/tvm/relax/backend/contrib/cutlass.py:271-314,344-372,
and the attributes python/tvm/contrib/cutlass/build.py:742-775 derives from each."""
import pytest

from relax_b200 import patterns


def test_the_22_names_of_the_reference():
    assert patterns.BASE_PATTERNS == (
        "cutlass.decode_matmul", "cutlass.decode_matmul_bias", "cutlass.decode_matmul_cast",
        "cutlass.decode_matmul_cast_bias", "cutlass.decode_matmul_bias_gelu", "cutlass.decode_matmul_cast_bias_gelu")
    assert len(patterns.RESIDUAL_PATTERNS) == 16 and len(set(patterns.ALL_PATTERNS)) == 22
    # spot values written out by hand from the reference's construction
    assert "cutlass.decode_matmul_bias_residual_add" in patterns.RESIDUAL_PATTERNS
    assert "cutlass.decode_matmul_cast_bias_gelu_residual_multiply_relu" in patterns.RESIDUAL_PATTERNS
    assert not any(n.startswith("cutlass.decode_matmul_residual") for n in patterns.RESIDUAL_PATTERNS)
    assert not any(n.startswith("cutlass.decode_matmul_cast_residual") for n in patterns.RESIDUAL_PATTERNS)


@pytest.mark.parametrize("name,bias,act,binop,unop", [
    ("cutlass.decode_matmul", False, "identity", "", "identity"),
    ("cutlass.decode_matmul_cast", False, "identity", "", "identity"),
    ("cutlass.decode_matmul_bias", True, "identity", "", "identity"),
    ("cutlass.decode_matmul_cast_bias_gelu", True, "gelu", "", "identity"),
    ("cutlass.decode_matmul_bias_residual_add", True, "identity", "plus", "identity"),
    ("cutlass.decode_matmul_bias_gelu_residual_multiply", True, "gelu", "multiply", "identity"),
    ("cutlass.decode_matmul_cast_bias_residual_add_relu", True, "identity", "plus", "relu"),
    ("cutlass.decode_matmul_bias_gelu_residual_multiply_relu", True, "gelu", "multiply", "relu"),
])
def test_attributes_per_name(name, bias, act, binop, unop):
    a = patterns.PATTERN_TABLE[name]
    assert (a.bias, a.activation, a.binary_op, a.unary_op) == (bias, act, binop, unop)
    assert a.residual == (binop != "")
    assert a.cast == ("_cast" in name)


def test_a_relu_in_the_residual_postfix_is_not_the_activation():
    # build.py looks for the activation only between "matmul_" and "residual_"
    a = patterns.PATTERN_TABLE["cutlass.decode_matmul_bias_residual_add_relu"]
    assert a.activation == "identity" and a.unary_op == "relu"


def test_check_decode_matmul_scale_and_bias_shapes():
    ok = lambda **kw: patterns.check_decode_matmul(
        kw.get("lhs", (4, 64)), kw.get("ld", "float16"), (64, 64), kw.get("wd", "int8"), kw.get("s", (128,)),
        kw.get("sd", "float16"), kw.get("out", (4, 128)), kw.get("od", "float16"), kw.get("bias"))
    assert ok() and ok(s=(1, 128)) and ok(s=(1, 128), bias=(128,)) and ok(bias=(1, 128)) and ok(bias=(4, 128))
    assert ok(s=(2, 128))                       # (K // group_size, N)
    assert not ok(s=(1, 1, 128)) and not ok(s=(64,)) and not ok(bias=(2, 128))
    assert not ok(od="float32") and not ok(ld="float32") and not ok(wd="int32") and not ok(sd="float32")


def test_call_arguments_follow_the_annotator():
    c = patterns.call_arguments("cutlass.decode_matmul_bias", (2, 3, 64), (64, 64), (128,), (2, 3, 128), (1, 128))
    assert (c["m"], c["n"], c["k"], c["weight_bits"], c["group_size"], c["bias_stride"]) == (6, 128, 64, 4, -1, 0)
    c = patterns.call_arguments("cutlass.decode_matmul_bias", (64, 128), (128, 128), (2, 128), (64, 128), (64, 128))
    assert (c["m"], c["weight_bits"], c["group_size"], c["bias_stride"]) == (64, 8, 64, 128)
    with pytest.raises(ValueError):
        patterns.call_arguments("cutlass.decode_matmul", (4, 64), (64, 50), (128,), (4, 128))
