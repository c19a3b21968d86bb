"""The MLIR-text front end and the benchgc-compatible command line (host logic only)."""
import json

import pytest
import torch

from gc_b200 import benchgc, mlir_text


def test_mlp_module_text_round_trips_to_the_partition_the_c_api_takes():
    text = mlir_text.mlp_module(128, [512, 256], [True], "relu", "bf16")
    assert "linalg.matmul ins(%arg0, %arg1 : tensor<128x512xbf16>, tensor<512x256xbf16>)" in text
    assert "linalg.broadcast ins(%arg2 : tensor<256xbf16>)" in text and "dimensions = [0]" in text
    fn = mlir_text.parse_module(text)
    assert [a.type.shape for a in fn.args] == [(128, 512), (512, 256), (256,)]
    assert [o.name for o in fn.ops] == ["matmul", "add", "relu"]
    js, arg_ids, out_ids = mlir_text.to_partition(fn)
    g = json.loads(js)
    assert [n["kind"] for n in g["graph"]] == ["MatMul", "Add", "ReLU"]
    assert g["input_ports"] == [0, 1, 2] and arg_ids == [0, 1, 2] and g["output_ports"] == out_ids
    add = g["graph"][1]
    assert add["inputs"][1] == {"id": 2, "dtype": "bf16", "shape": [256]}           # the broadcast became numpy broadcast
    assert add["attrs"]["auto_broadcast"]["value"] == "numpy"


def test_four_layer_chain_argument_order_matches_the_pattern():
    # weights first, then the biases of the layers that have one (pattern/mlp.py:90-112)
    text = mlir_text.mlp_module(8, [16, 32, 16, 32, 16], [True, False, True, False], "relu", "f32")
    fn = mlir_text.parse_module(text)
    assert [a.type.shape for a in fn.args] == [(8, 16), (16, 32), (32, 16), (16, 32), (32, 16), (32,), (32,)]
    assert [o.name for o in fn.ops] == ["matmul", "add", "relu", "matmul", "relu", "matmul", "add", "relu", "matmul", "relu"]


def test_reference_interpretation_matches_torch_on_the_host():
    text = mlir_text.mlp_module(4, [8, 6, 5], [True, True], "relu", "f32")
    fn = mlir_text.parse_module(text)
    torch.manual_seed(0)
    t = {a.name: torch.randn(a.type.shape) for a in fn.args}
    (got,) = benchgc.ref_run(fn, t)
    h = torch.relu(t["%arg0"] @ t["%arg1"] + t["%arg3"])
    want = torch.relu(h @ t["%arg2"] + t["%arg4"])
    assert torch.equal(got, want)


def test_single_op_modules_and_transposes():
    T = mlir_text.TensorType
    text = mlir_text.matmul_module("matmul_transpose_b", T((1024, 512), "f32"), T((1024, 512), "f32"), T((1024, 1024), "f32"))
    fn = mlir_text.parse_module(text)
    assert fn.ops[0].attrs == {"transpose_a": False, "transpose_b": True}
    g = json.loads(mlir_text.to_partition(fn)[0])
    assert g["graph"][0]["attrs"]["transpose_b"] == {"type": "bool", "value": 1}
    with pytest.raises(mlir_text.ParseError):
        mlir_text.parse_module(mlir_text.matmul_module("matmul", T((4, 8), "f32"), T((9, 4), "f32"), T((4, 4), "f32")))
    with pytest.raises(mlir_text.Unimplemented):
        mlir_text.matmul_module("batch_matmul", T((2, 4, 8), "f32"), T((2, 8, 4), "f32"), T((2, 4, 4), "f32"))


@pytest.mark.parametrize("stmt, err", [
    ("%9 = linalg.exp ins(%arg0 : tensor<4x4xf32>) outs(%0 : tensor<4x4xf32>) -> tensor<4x4xf32>", mlir_text.Unimplemented),
    ("%9 = tensor.empty() : tensor<?x4xf32>", mlir_text.Unimplemented),
    ("%9 = linalg.add ins(%arg0, %nope : tensor<4x4xf32>, tensor<4x4xf32>) outs(%0 : tensor<4x4xf32>) -> tensor<4x4xf32>", mlir_text.ParseError),
])
def test_outside_the_subset_is_refused(stmt, err):
    text = "\n".join(["module {", "  func.func @entry(%arg0: tensor<4x4xf32>) -> tensor<4x4xf32> {",
                      "    %0 = tensor.empty() : tensor<4x4xf32>", "    " + stmt, "    return %9 : tensor<4x4xf32>", "  }", "}"])
    with pytest.raises(err):
        mlir_text.parse_module(text)


def test_matmul_without_zero_init_is_refused():
    text = "\n".join(["module {", "  func.func @entry(%arg0: tensor<4x4xf32>, %arg1: tensor<4x4xf32>) -> tensor<4x4xf32> {",
                      "    %0 = tensor.empty() : tensor<4x4xf32>",
                      "    %1 = linalg.matmul ins(%arg0, %arg1 : tensor<4x4xf32>, tensor<4x4xf32>) outs(%arg0 : tensor<4x4xf32>) -> tensor<4x4xf32>",
                      "    return %1 : tensor<4x4xf32>", "  }", "}"])
    with pytest.raises(mlir_text.Unimplemented):
        mlir_text.parse_module(text)


def test_default_fills_and_thresholds_follow_the_harness():
    flags = benchgc.build_parser().parse_args(["--driver", "linalg", "--case", "matmul", "--md", "0:32x128xbf16", "--md", "1:128x64xbf16",
                                               "--md", "2:32x64xbf16"])
    args = [benchgc.Arg(i) for i in range(3)]
    for md in flags.md:
        i, r = md.split(":", 1)
        args[int(i)].set_md(r)
    benchgc._defaults(flags, args, 2)
    assert args[0].fill_param == ["matmul", "src", "bf16", "bf16", "bf16", "128"]
    assert args[1].fill_param == ["matmul", "wei", "bf16", "bf16", "bf16", "128"]
    assert args[2].fill_type == "Z" and args[2].cmp_type == "P" and float(args[2].cmp_param[0]) == torch.finfo(torch.bfloat16).eps
    a = benchgc._fill(flags, args[0])
    w = benchgc._fill(flags, args[1])
    # integer-valued operands whose products and sums are exact in bf16's 8 digits
    assert a.dtype == torch.bfloat16 and torch.equal(a.float(), a.float().round()) and a.float().abs().max() <= 4
    assert torch.equal(w.float(), w.float().round()) and w.float().abs().max() <= 8
    assert (w != 0).float().mean() < 0.2          # density = 2^8 / 32 / 128
    # pattern defaults
    pf = benchgc.build_parser().parse_args(["--driver", "pattern", "--case", "mlp", "--dtype", "bf16"])
    pa = [benchgc.Arg(0), benchgc.Arg(1)]
    for x in pa:
        x.dtype, x.shape = "bf16", [4, 4]
    benchgc._defaults(pf, pa, 1)
    assert (pa[0].fill_type, pa[0].fill_param) == ("U", ["0", "1"]) and pa[1].cmp_param == ["0.05", "100.0"]
