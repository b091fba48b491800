"""The StableHLO reader and dequant-chain matcher (host logic, no GPU).

Mirrors the reference's plan-shape tests, which parse the planner's JSON trace
to assert which route was chosen (tests/test_reduce_routing.py:55-62).
"""

import os

import pytest

from jax_metallib_b200 import _lib
from jax_metallib_b200.stablehlo import Executable, weight_only_linears_module

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures")


def load(name):
    return open(os.path.join(FIX, name)).read()


def fused(exe):
    return [t for t in exe.trace() if t["event"] == "fused"]


def test_config1_chain_becomes_one_kernel():
    exe = Executable(load("cfg1_w8a32.mlir"))
    assert (exe.num_args, exe.num_results, exe.num_steps) == (3, 1, 1)
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_w8a32_perchannel" and (f["M"], f["N"], f["K"]) == (32, 1024, 1024)
    assert f["ops_fused"] == 5  # convert, two broadcasts, multiply, dot_general
    assert exe.workspace_bytes == 0


def test_config1_spelling_variants_and_rank3_lhs():
    exe = Executable(load("cfg1_variant_reshape_swapped.mlir"))
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_w8a32_perchannel" and (f["M"], f["N"], f["K"]) == (32, 128, 256)


def test_config2_integer_dot_with_and_without_rescale():
    exe = Executable(load("cfg2_i8dot_rescale.mlir"))
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_i8i8_i32" and f["rescale"] is True and f["ops_fused"] == 8
    assert (f["M"], f["N"], f["K"]) == (2048, 4096, 4096) and exe.num_results == 2
    exe = Executable(load("cfg2_i8dot_only.mlir"))
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_i8i8_i32" and f["rescale"] is False
    # multiply order swapped (column scale first) is the same fused step
    text = load("cfg2_i8dot_rescale.mlir").replace("%4 = stablehlo.multiply %1, %3", "%4 = stablehlo.multiply %1, %6x") \
        .replace("%7 = stablehlo.multiply %4, %6 ", "%7 = stablehlo.multiply %4, %3 ").replace("%6x", "%6")
    lines = text.splitlines()
    # move the column broadcasts above the first multiply so that SSA order stays valid
    i4 = next(i for i, l in enumerate(lines) if l.strip().startswith("%4 ="))
    i5 = next(i for i, l in enumerate(lines) if l.strip().startswith("%5 ="))
    lines[i4], lines[i5], lines[i5 + 1] = lines[i5], lines[i5 + 1], lines[i4]
    (f,) = fused(Executable("\n".join(lines)))
    assert f["rescale"] is True


def test_config3_int4_chain():
    exe = Executable(load("cfg3_w4a16.mlir"))
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_w4a16_g128" and (f["M"], f["N"], f["K"]) == (4, 14336, 4096)
    assert f["ops_fused"] == 19
    assert exe.workspace_bytes == _lib.load().qmm_w4a16_g128_workspace_bytes(4, 14336, 4096)


def test_config5_bf16_activations():
    (f,) = fused(Executable(load("cfg5_w8a16.mlir")))
    assert f["kernel"] == "qmm_w8a16_perchannel" and (f["M"], f["N"], f["K"]) == (4096, 1024, 8192)
    # the trace says where the fused arithmetic departs from the program as written
    assert f["numerics"].startswith("f32_scale_in_epilogue")
    (f,) = fused(Executable(load("cfg1_w8a32.mlir")))
    assert f["numerics"] == "as_written"
    (f,) = fused(Executable(load("cfg3_w4a16.mlir")))
    assert f["numerics"].startswith("f32_group_sums")


@pytest.mark.parametrize("name,needle", [
    ("reject_unfused_add.mlir", "stablehlo.tanh"),
    ("reject_unsupported_op_after_unfused_chain.mlir", "stablehlo.negate"),
])
def test_unsupported_programs_fail_at_compile_time_naming_the_op(name, needle):
    with pytest.raises(_lib.QmmError) as e:
        Executable(load(name))
    assert e.value.status_name == "QMM_ERR_UNSUPPORTED" and needle in str(e.value)


def test_malformed_and_foreign_programs():
    with pytest.raises(_lib.QmmError) as e:
        Executable("module { }")
    assert e.value.status_name == "QMM_ERR_PARSE"
    with pytest.raises(_lib.QmmError) as e:
        Executable(load("cfg1_w8a32.mlir").replace("tensor<1024x1024xi8>) ->", "tensor<1024x1024xi8> ->"))
    assert e.value.status_name in ("QMM_ERR_PARSE", "QMM_ERR_UNSUPPORTED")
    # plain float dot: not on the path
    text = """module {
  func.func public @main(%arg0: tensor<8x16xf32>, %arg1: tensor<16x4xf32>) -> tensor<8x4xf32> {
    %0 = stablehlo.dot_general %arg0, %arg1, contracting_dims = [1] x [0] : (tensor<8x16xf32>, tensor<16x4xf32>) -> tensor<8x4xf32>
    return %0 : tensor<8x4xf32>
  }
}"""
    exe = Executable(text)  # runs, but as a standalone dot: the trace says so and why
    assert fused(exe) == [] and lib_fused_steps(exe) == 0
    (nf,) = [t for t in exe.trace() if t["event"] == "not_fused"]
    assert nf["op"] == "stablehlo.dot_general" and "plain float" in nf["reason"]
    # group size other than 128: no kernel fuses it, so the chain runs op by op and the trace names the reason
    exe = Executable(load("cfg3_w4a16.mlir").replace("32x128x14336", "64x64x14336").replace("32x14336", "64x14336"))
    assert lib_fused_steps(exe) == 0
    assert "group 128" in [t for t in exe.trace() if t.get("reason")][0]["reason"]


def lib_fused_steps(exe):
    return _lib.load().qmm_plan_num_fused_steps(exe._h)


def not_fused_ops(exe):
    return [t["op"] for t in exe.trace() if t["event"] == "not_fused"]


def test_a_chain_the_matcher_declines_runs_op_by_op_and_says_so():
    # the dequantised weight is also returned: fusing would lose it, so every op runs on its own
    exe = Executable(load("unfused_escaping_intermediate.mlir"))
    assert fused(exe) == [] and lib_fused_steps(exe) == 0 and exe.num_steps == 4
    assert not_fused_ops(exe) == ["stablehlo.dot_general", "stablehlo.convert", "stablehlo.broadcast_in_dim",
                                  "stablehlo.multiply"]
    reason = [t for t in exe.trace() if t["event"] == "not_fused" and "reason" in t][0]["reason"]
    assert "also used elsewhere" in reason
    assert exe.workspace_bytes >= 2 * 256 * 128 * 4  # the convert and broadcast results are temporaries
    # a [N, K] weight behind a transpose, and a dot that contracts the rhs on dimension 1
    exe = Executable(load("unfused_transposed_weight.mlir"))
    assert lib_fused_steps(exe) == 0 and "stablehlo.transpose" in not_fused_ops(exe)
    exe = Executable(load("unfused_contract_rhs_dim1.mlir"))
    assert lib_fused_steps(exe) == 0 and "stablehlo.dot_general" in not_fused_ops(exe)


def test_legacy_dot_trailing_convert_and_constants_fuse():
    exe = Executable(load("legacy_dot_w8a32.mlir"))
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_w8a32_perchannel" and (f["M"], f["N"], f["K"]) == (32, 128, 256)
    exe = Executable(load("cfg5_f32_accumulate_then_convert.mlir"))
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_w8a16_perchannel" and f["ops_fused"] == 6 and exe.num_steps == 1
    # weights and scales closed over as dense constants are arguments the plan owns; the bias add runs after
    exe = Executable(load("const_weight_bias_add.mlir"))
    (f,) = fused(exe)
    assert f["kernel"] == "qmm_w8a32_perchannel" and exe.num_args == 2 and exe.num_steps == 3
    assert not_fused_ops(exe) == ["stablehlo.broadcast_in_dim", "stablehlo.add"]
    exe = Executable(load("int8_result_wraps.mlir"))
    assert fused(exe) == [] and exe.num_steps == 1  # an i8-typed result: the standalone integer dot wraps it
    exe = Executable(load("unfused_slice_concat.mlir"))
    assert exe.num_steps == 5 and lib_fused_steps(exe) == 0


def test_constant_parsing_errors():
    bad = load("const_weight_bias_add.mlir").replace("[10, -11, 12]]", "[10, -11]]")
    with pytest.raises(_lib.QmmError) as e:
        Executable(bad)
    assert e.value.status_name == "QMM_ERR_PARSE" and "values" in str(e.value)
    hexed = load("const_weight_bias_add.mlir").replace(
        "dense<[[1, -2, 3], [4, 5, -6], [-7, 8, 9], [10, -11, 12]]>", 'dense<"0x01FE030405FAF908090AF50C">')
    assert Executable(hexed).num_args == 2


def test_a_layer_of_four_linears_is_four_fused_steps_with_introspection():
    text = weight_only_linears_module([(256, 512, 640, 0), (256, 512, 512, 0), (256, 512, 3584, 0), (256, 1792, 512, 1)])
    exe = Executable(text)
    assert (exe.num_args, exe.num_results, exe.num_steps) == (10, 4, 4)
    assert [(f["M"], f["N"], f["K"]) for f in fused(exe)] == [(256, 640, 512), (256, 512, 512), (256, 3584, 512),
                                                             (256, 512, 1792)]
    assert all(f["kernel"] == "qmm_w8a16_perchannel" for f in fused(exe))
    lib = _lib.load()
    import ctypes

    dt, rank = ctypes.c_int(), ctypes.c_int(8)
    dims = (ctypes.c_int64 * 8)()
    assert lib.qmm_plan_arg_info(exe._h, 1, ctypes.byref(dt), dims, ctypes.byref(rank)) == 0
    assert (dt.value, rank.value, dims[0], dims[1]) == (_lib.QMM_BF16, 2, 256, 1792)
    rank.value = 8
    assert lib.qmm_plan_result_info(exe._h, 2, ctypes.byref(dt), dims, ctypes.byref(rank)) == 0
    assert (dt.value, dims[0], dims[1]) == (_lib.QMM_BF16, 256, 3584)
    rank.value = 1  # too small for a rank-2 tensor
    assert lib.qmm_plan_result_info(exe._h, 2, ctypes.byref(dt), dims, ctypes.byref(rank)) != 0
    assert lib.qmm_plan_name(exe._h) == b"jit_layer"
    assert lib.qmm_plan_num_replicas(exe._h) == 1 and lib.qmm_plan_num_partitions(exe._h) == 1
    assert lib.qmm_plan_flops(exe._h) == 2.0 * 256 * (512 * (640 + 512 + 3584) + 1792 * 512)


# ---- the explicit custom_call route ---------------------------------------------------------------
def test_custom_call_route_builds_the_named_kernel():
    from jax_metallib_b200 import custom_call as cc

    text = cc.module_text(["tensor<256x512xbf16>", "tensor<512x384xi8>", "tensor<384xf32>"], "tensor<256x384xbf16>",
                          cc.backend_config("w8a16_perchannel"))
    exe = Executable(text)
    assert exe.num_steps == 1 and lib_fused_steps(exe) == 1 and fused(exe) == []
    (t,) = [t for t in exe.trace() if t["event"] == "custom_call"]
    assert t["kernel"] == "qmm_w8a16_perchannel" and (t["M"], t["N"], t["K"]) == (256, 384, 512)
    text = cc.module_text(["tensor<4x4096xbf16>", "tensor<2048x14336xui8>", "tensor<32x14336xbf16>", "tensor<32x14336xui4>"],
                          "tensor<4x14336xbf16>", cc.backend_config("w4a16_g128"))
    exe = Executable(text)
    assert exe.workspace_bytes >= _lib.load().qmm_w4a16_g128_workspace_bytes(4, 14336, 4096)
    text = cc.module_text(["tensor<4x4096xbf16>", "tensor<2048x14336xui8>", "tensor<32x14336xbf16>", "tensor<32x7168xui8>"],
                          "tensor<4x14336xbf16>", cc.backend_config("w4a16_g128", zeros_packed=True))
    assert Executable(text).num_steps == 1
    text = cc.module_text(["tensor<64x128xi8>", "tensor<128x256xui8>", "tensor<64xf32>", "tensor<256xf32>"],
                          "tensor<64x256xf32>", cc.backend_config("i8i8_i32"))
    assert [t["kernel"] for t in Executable(text).trace() if t["event"] == "custom_call"] == ["qmm_i8i8_i32"]


def test_custom_call_descriptor_is_validated_key_by_key():
    from jax_metallib_b200 import custom_call as cc

    types = (["tensor<32x64xf32>", "tensor<64x16xi8>", "tensor<16xf32>"], "tensor<32x16xf32>")

    def compile_with(config, target=None):
        text = cc.module_text(*types, config)
        if target:
            text = text.replace("@" + cc.TARGET, "@" + target)
        return Executable(text)

    assert compile_with(cc.backend_config("w8a32_perchannel")).num_steps == 1
    for config, needle in [
        ('{"version":2,"op":"w8a32_perchannel"}', "version"),
        ('{"version":1}', "needs the keys"),
        ('{"version":1,"op":"w8a32_perchannel","grid":4}', "unknown key"),
        ('{"version":1,"op":"gemm"}', "must be one of"),
        ('{"version":1,"op":"w8a32_perchannel","op":"x"}', "repeats"),
        ('[1]', "JSON object"),
        ('{"version":1,"op":"w8a16_perchannel"}', "expects"),  # operand types do not fit the named kernel
        ('{"version":1,"op":"w8a32_perchannel","pad":"' + "x" * 5000 + '"}', "4096"),
    ]:
        with pytest.raises(_lib.QmmError) as e:
            compile_with(config)
        assert needle in str(e.value), (config[:60], str(e.value))
    with pytest.raises(_lib.QmmError) as e:
        compile_with(cc.backend_config("w8a32_perchannel"), target="somebody.else")
    assert "somebody.else" in str(e.value) and e.value.status_name == "QMM_ERR_UNSUPPORTED"
    with pytest.raises(ValueError):
        cc.backend_config("w8a32_perchannel", zeros_packed=True)
    with pytest.raises(ValueError):
        cc.backend_config("dense")


# ---- counted while loops and views of stacked arguments ------------------------------------------
def test_scan_over_stacked_weights_is_unrolled_into_fused_steps_on_views():
    text = load("scan_two_layers_w8a16.mlir")
    exe = Executable(text)
    assert (exe.num_args, exe.num_results, exe.num_steps) == (3, 1, 2)
    fs = fused(exe)
    assert [f["kernel"] for f in fs] == ["qmm_w8a16_perchannel"] * 2 and not_fused_ops(exe) == []
    assert exe.workspace_bytes == 256 * 512 * 2  # only the activation carried between the two layers
    # more layers: the trip count comes from the loop's bound
    more = text.replace("tensor<2x512x512xi8>", "tensor<5x512x512xi8>").replace("tensor<2x512xf32>", "tensor<5x512xf32>") \
        .replace("%c_1 = stablehlo.constant dense<2> : tensor<i32>\n      %1 = stablehlo.compare  LT, %iterArg, %c_1",
                 "%c_1 = stablehlo.constant dense<5> : tensor<i32>\n      %1 = stablehlo.compare  LT, %iterArg, %c_1")
    assert Executable(more).num_steps == 5


def test_loops_that_are_not_counted_are_refused():
    text = load("scan_two_layers_w8a16.mlir")
    # the bound is an argument of the program: nothing to fold
    dyn = text.replace("%arg2: tensor<2x512xf32>)", "%arg2: tensor<2x512xf32>, %arg3: tensor<i32>)") \
        .replace("%1 = stablehlo.compare  LT, %iterArg, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>\n      stablehlo.return",
                 "%1 = stablehlo.compare  LT, %iterArg, %arg3,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>\n      stablehlo.return")
    with pytest.raises(_lib.QmmError) as e:
        Executable(dyn)
    assert e.value.status_name == "QMM_ERR_PARSE" and "counted" in str(e.value)
    long = text.replace("dense<2> : tensor<i32>\n      %1 = stablehlo.compare  LT, %iterArg, %c_1",
                        "dense<1000> : tensor<i32>\n      %1 = stablehlo.compare  LT, %iterArg, %c_1")
    with pytest.raises(_lib.QmmError) as e:
        Executable(long)
    assert "64 trips" in str(e.value)
