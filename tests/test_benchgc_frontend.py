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
    js, arg_ids, out_ids, consts = mlir_text.to_partition(fn)
    assert consts == {}
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
    ("%9 = linalg.tanh ins(%arg0 : tensor<4x4xf32>) outs(%0 : tensor<4x4xf32>) -> tensor<4x4xf32>", mlir_text.Unimplemented),
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


def _llama2_reference(t, H):
    """The block in torch, op by op in each tensor's own dtype (what benchgc's evaluators compute)."""
    x, wo, res, _, g1, wg, wu, wd, eps, g2 = (t[f"%arg{i}"] for i in range(10))

    def rms(v, gamma):
        f = v.float()
        r = (torch.sum(torch.pow(f, 2.0), dim=[2]) / torch.full((1,), float(H))).reshape(f.shape[0], f.shape[1], 1)
        r = torch.pow(r + eps.reshape(1, 1, 1), -0.5)
        return gamma * (f * r).to(torch.bfloat16)

    r1 = res + torch.matmul(x.reshape(-1, H), wo.t()).reshape(x.shape)
    h = rms(r1, g1)
    gate = torch.matmul(h.reshape(-1, H), wg.t()).reshape(x.shape[0], x.shape[1], -1)
    one = torch.ones_like(gate)
    silu = (one / (one + torch.exp(torch.neg(gate)))) * gate
    up = torch.matmul(h.reshape(-1, H), wu.t()).reshape(gate.shape)
    r2 = r1 + torch.matmul((silu * up).reshape(-1, gate.shape[-1]), wd.t()).reshape(x.shape)
    return rms(r2, g2), r2


def test_llama2_decoder_block_in_linalg_form_lowers_to_a_partition():
    """The reference's own --driver mlir case (test/benchgc/cases/llama2.mlir) in small: collapse / expand_shape, copy as
    cast, powf by a splat, reduce with an add body, broadcasts along trailing dimensions, splat constants as operands."""
    B, S, H, I = 1, 8, 64, 96
    text = mlir_text.llama2_mlp_module(B, S, H, I)
    fn = mlir_text.parse_module(text)
    names = [o.name for o in fn.ops]
    assert names.count("matmul") == 4 and names.count("reshape") == 12 and names.count("reduce_sum") == 2 and names.count("pow") == 4
    assert names.count("cast") == 4 and names.count("neg") == 1 and names.count("exp") == 1
    js, arg_ids, out_ids, consts = mlir_text.to_partition(fn)
    g = json.loads(js)
    kinds = [n["kind"] for n in g["graph"]]
    for k in ("MatMul", "StaticReshape", "Typecast", "Pow", "ReduceSum", "Negate", "Exp", "Divide", "Multiply", "Add"):
        assert k in kinds, k
    assert sorted(v for v in consts.values()) == [(1.0, "bf16"), (float(H), "f32")]   # the splats used as operands
    assert 3 not in g["input_ports"]                       # %arg3 (an unused epsilon) is not a partition input
    assert len(out_ids) == 2
    # the host interpretation of the parsed module equals the block written directly in torch
    torch.manual_seed(0)
    t = {a.name: (torch.randn(a.type.shape) * (0.1 if a.type.rank == 2 else 1.0)).to(benchgc.compat.get_dtype(a.type.dtype)) for a in fn.args}
    t["%arg8"] = torch.full((1,), 1e-5)
    got = benchgc.ref_run(fn, t)
    want = _llama2_reference(t, H)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    # the partition compiles (host only)
    from gc_b200 import api
    plan = api.GraphCompiler().compile(js).plan()
    assert plan.count("step") >= 30


def test_the_reference_llama2_case_file_parses_when_the_checkout_is_present():
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.environ.get("GC_REFERENCE_DIR") or os.path.join(os.path.dirname(root), "reference")
    path = os.path.join(ref, "test", "benchgc", "cases", "llama2.mlir")
    if not os.path.exists(path):
        pytest.skip("reference checkout not present")
    fn = mlir_text.parse_module(open(path).read())
    mine = mlir_text.parse_module(mlir_text.llama2_mlp_module(1, 32, 4096, 11008))
    assert [o.name for o in fn.ops] == [o.name for o in mine.ops]                      # same op sequence as the generator's
    assert [a.type.shape for a in fn.args] == [a.type.shape for a in mine.args]
    js, _, out_ids, consts = mlir_text.to_partition(fn)
    assert len(out_ids) == 2 and len(consts) == 2


def test_attention_in_linalg_form_becomes_one_fused_partition():
    text = mlir_text.attention_module(4, 256, 128, 0.125)
    fn = mlir_text.parse_module(text)
    assert [o.name for o in fn.ops] == ["batch_matmul", "mul", "softmax", "batch_matmul"]
    js, arg_ids, out_ids, consts = mlir_text.to_partition(fn)
    g = json.loads(js)
    assert [n["kind"] for n in g["graph"]] == ["SDPA"] and consts == {}
    assert g["graph"][0]["attrs"]["scale"]["value"] == 0.125 and g["input_ports"] == [0, 1, 2]
    # a softmax that is not part of the pattern is refused
    lone = text.replace("linalg.batch_matmul ins(%6, %arg2", "linalg.batch_matmul ins(%4, %arg2")
    with pytest.raises(mlir_text.Unimplemented):
        mlir_text.to_partition(mlir_text.parse_module(lone))


def test_int8_matmul_in_linalg_form_becomes_one_quantized_partition():
    """linalg.quantized_matmul on ui8 activations and i8 weights, cast, per-channel scales and bias: BASELINE's int8
    configuration as a module; the chain folds into one QuantizedMatMul, the bare op gives its i32 accumulators."""
    text = mlir_text.quantized_matmul_module(64, 48, 32, src_zp=128)
    fn = mlir_text.parse_module(text)
    assert [o.name for o in fn.ops] == ["qmatmul", "cast", "mul", "add"]
    js, arg_ids, out_ids, consts = mlir_text.to_partition(fn)
    g = json.loads(js)
    assert [n["kind"] for n in g["graph"]] == ["QuantizedMatMul"] and consts == {}
    node = g["graph"][0]
    assert [t["dtype"] for t in node["inputs"]] == ["u8", "s8", "f32", "f32"] and node["attrs"]["src_zp"]["value"] == 128
    assert node["outputs"][0]["dtype"] == "f32" and g["input_ports"] == [0, 1, 2, 3]
    # the host interpretation: exact integer accumulators, then f32 arithmetic
    torch.manual_seed(0)
    t = {"%arg0": torch.randint(0, 256, (64, 32), dtype=torch.uint8), "%arg1": torch.randint(-127, 128, (32, 48), dtype=torch.int8),
         "%arg2": torch.rand(48) * 0.01, "%arg3": torch.rand(48)}
    (got,) = benchgc.ref_run(fn, t)
    acc = (t["%arg0"].int() - 128) @ t["%arg1"].int()
    assert torch.equal(got, acc.float() * t["%arg2"] + t["%arg3"])
    from gc_b200 import api
    assert "QuantizedMatMul" in api.GraphCompiler().compile(js).plan()
    # accumulators only
    fn2 = mlir_text.parse_module(mlir_text.quantized_matmul_module(64, 48, 32, src_zp=128, dequant=False))
    js2, _, _, _ = mlir_text.to_partition(fn2)
    g2 = json.loads(js2)
    assert [n["kind"] for n in g2["graph"]] == ["QuantizedMatMul"] and g2["graph"][0]["outputs"][0]["dtype"] == "s32"
    assert len(g2["graph"][0]["inputs"]) == 2
    assert "QuantizedMatMul" in api.GraphCompiler().compile(js2).plan()
    (acc2,) = benchgc.ref_run(fn2, t)
    assert torch.equal(acc2, acc)
