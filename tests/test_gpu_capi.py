"""The reference's C-API tests (test/dnnl/TestApiBasic.cpp, TestApiOps.cpp) restated against this
library, with HOST buffers exactly as the reference passes them, plus the MLP partitions of
BASELINE checked against the oracle and the benchgc golden outputs."""
import json

import numpy as np
import pytest
import torch

import oracle
from _util import assert_bf16_close, from_bits, tbits
from gc_b200 import api, partitions
from gc_b200 import benchgc_compat as bc

pytestmark = pytest.mark.gpu


def _t(i, dt, shape):
    return {"id": i, "dtype": dt, "shape": list(shape)}


def _run(graph, ins, outs, in_ports=None, out_ports=None, attrs=None):
    env = {"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "any", "graph": graph}
    if in_ports is not None:
        env["input_ports"] = in_ports
    if out_ports is not None:
        env["output_ports"] = out_ports
    gc = api.GraphCompiler()
    exe = gc.compile(json.dumps(env))
    exe.execute(ins, outs)
    exe.destroy()
    gc.destroy()


def _binary(kind, a, b, shape):
    out = np.empty(shape, np.float32)
    _run([{"kind": kind, "inputs": [_t(0, "f32", a.shape), _t(1, "f32", b.shape)], "outputs": [_t(2, "f32", shape)]}],
         {0: a, 1: b}, {2: out}, [0, 1], [2])
    return out


def test_basic_workflow_add():
    """TestApiBasic.basicWorkflow: 128-element f32 add, ctx.num_threads = 4."""
    a = np.zeros(128, np.float32); a[0] = 1.0
    b = np.arange(128, dtype=np.float32)
    out = np.empty(128, np.float32)
    gc = api.GraphCompiler(num_threads=4)
    exe = gc.compile(json.dumps({"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "any", "input_ports": [0, 1],
                                 "output_ports": [2],
                                 "graph": [{"kind": "Add", "inputs": [_t(0, "f32", [128]), _t(1, "f32", [128])],
                                            "outputs": [_t(2, "f32", [128])]}]}))
    exe.execute({1: b, 0: a}, {2: out})   # order differs from the argument order: matched by id
    assert np.array_equal(out, a + b)
    # the same call with its tensor structs built once: new data in the same buffers is picked up
    bound = exe.bind({0: a, 1: b}, {2: out})
    for k in (2.0, 3.0):
        a[1] = k
        bound.run()
        assert np.array_equal(out, a + b)


def test_ops_div_mul_sub():
    x = np.arange(64 * 32 * 32, dtype=np.float32).reshape(64, 32, 32)
    np.testing.assert_array_equal(_binary("Divide", x, x + 1, x.shape), x / (x + 1))
    v = np.arange(128, dtype=np.float32)
    np.testing.assert_array_equal(_binary("Multiply", v, v, v.shape), v * v)
    np.testing.assert_array_equal(_binary("Subtract", v, v * v, v.shape), v - v * v)


def test_ops_matmul_transpose_a_f32():
    """TestApiOps.matMul: out[512,64] = A[128,512]^T . B[128,64] + bias[64], exact in f32."""
    A = (np.arange(128)[:, None] + np.arange(512)[None, :]).astype(np.float32)
    B = (np.arange(128)[:, None] - np.arange(64)[None, :]).astype(np.float32)
    bias = np.arange(64, dtype=np.float32)
    out = np.empty((512, 64), np.float32)
    op = {"kind": "MatMul", "attrs": {"transpose_a": {"type": "bool", "value": 1}, "transpose_b": {"type": "bool", "value": 0}},
          "inputs": [_t(0, "f32", [128, 512]), _t(1, "f32", [128, 64]), _t(2, "f32", [64])], "outputs": [_t(3, "f32", [512, 64])]}
    _run([op], {0: A, 1: B, 2: bias}, {3: out}, [0, 1, 2], [3])
    want = np.empty((512, 64), np.float32)
    for i in range(0, 512, 37):
        for j in range(64):
            e = bias[j]
            for k in range(128):
                e += A[k, i] * B[k, j]
            want[i, j] = e
            assert out[i, j] == e
    assert np.array_equal(out, oracle.matmul_f32(A, B, bias, transA=True))


def test_ops_pow_relu_sigmoid_typecast_reduce():
    x = np.arange(64, dtype=np.float32)
    out = np.empty(64, np.float32)
    _run([{"kind": "Pow", "attrs": {"beta": {"type": "f32", "value": 2}}, "inputs": [_t(0, "f32", [64])], "outputs": [_t(1, "f32", [64])]}],
         {0: x}, {1: out})
    np.testing.assert_array_equal(out, x * x)
    x = (np.arange(128) - 64).astype(np.float32)
    out = np.empty(128, np.float32)
    _run([{"kind": "ReLU", "inputs": [_t(0, "f32", [128])], "outputs": [_t(1, "f32", [128])]}], {0: x}, {1: out})
    np.testing.assert_array_equal(out, np.maximum(x, 0))
    _run([{"kind": "Sigmoid", "inputs": [_t(0, "f32", [128])], "outputs": [_t(1, "f32", [128])]}], {0: x}, {1: out})
    want = 1.0 / (1.0 + np.exp(-x.astype(np.float32)))
    assert np.all(np.abs(out - want) <= 4 * np.spacing(want))  # ASSERT_FLOAT_EQ = 4 ulp
    xs = np.array([v / np.exp(-float(v)) for v in range(-64, 64)], np.float32)
    o16 = np.empty(128, np.float16)
    _run([{"kind": "Typecast", "inputs": [_t(0, "f32", [128])], "outputs": [_t(1, "f16", [128])]}], {0: xs}, {1: o16})
    with np.errstate(over="ignore"):
        assert np.array_equal(o16.view(np.uint16), xs.astype(np.float16).view(np.uint16))
    r = np.arange(16 * 64 * 32, dtype=np.float32).reshape(16, 64, 32)
    for kind, mean in (("ReduceSum", False), ("ReduceMean", True)):
        o = np.empty((16, 1, 32), np.float32)
        _run([{"kind": kind, "attrs": {"axes": {"type": "s64[]", "value": [1]}, "keep_dims": {"type": "bool", "value": 1}},
               "inputs": [_t(0, "f32", [16, 64, 32])], "outputs": [_t(1, "f32", [16, 1, 32])]}], {0: r}, {1: o})
        want = np.zeros((16, 32), np.float32)
        for y in range(64):
            want = want + r[:, y, :]
        if mean:
            want = want / np.float32(64)
        np.testing.assert_array_equal(o[:, 0, :], want)
    # long reductions run one block per output element; integer-valued data keeps every order exact
    big = (np.arange(6 * 5000, dtype=np.float32).reshape(6, 5000) % 97) - 48
    for kind, want in (("ReduceSum", big.sum(1)), ("ReduceMean", big.sum(1) / np.float32(5000))):
        o = np.empty((6,), np.float32)
        _run([{"kind": kind, "attrs": {"axes": {"type": "s64[]", "value": [-1]}},
               "inputs": [_t(0, "f32", [6, 5000])], "outputs": [_t(1, "f32", [6])]}], {0: big}, {1: o})
        np.testing.assert_array_equal(o, want.astype(np.float32))


def test_add_relu_bf16_broadcast_rounds_per_op():
    """bf16 elementwise ops are evaluated in f32 and rounded after each op (Pipeline.cpp:81-90)."""
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(4, 32, 28, generator=g).bfloat16(), torch.randn(28, generator=g).bfloat16()
    out = torch.empty(4, 32, 28, dtype=torch.bfloat16)
    graph = [{"kind": "Add", "attrs": {"auto_broadcast": {"type": "string", "value": "numpy"}},
              "inputs": [_t(0, "bf16", a.shape), _t(1, "bf16", b.shape)], "outputs": [_t(2, "bf16", a.shape)]},
             {"kind": "ReLU", "inputs": [_t(2, "bf16", a.shape)], "outputs": [_t(3, "bf16", a.shape)]}]
    _run(graph, {0: a, 1: b}, {3: out})
    assert torch.equal(out, torch.relu((a.float() + b.float()).bfloat16()))


@pytest.mark.parametrize("name", ["cfg1_mlp_bf16", "mlp_f32_32x16x64", "mpl_json_bf16", "mlp_bf16_ragged"])
@pytest.mark.parametrize("where", ["host", "device"])
def test_mlp_partitions_against_oracle_and_benchgc_golden(golden, name, where):
    meta, arrays = golden
    case = next(c for c in meta["cases"] if c["name"] == name)
    nl = len(case["hidden"]) - 1
    js, in_ids, out_id = partitions.mlp(case["batch"], case["hidden"], case["dtype"], case["has_bias"], case["act"],
                                        separate_add=(name == "mpl_json_bf16"))
    f = case["fills"]
    shapes = [(case["batch"], case["hidden"][0])] + [(case["hidden"][i], case["hidden"][i + 1]) for i in range(nl)] + \
             [(case["hidden"][i + 1],) for i in range(nl) if case["has_bias"][i]]
    kinds = ["src"] + ["w"] * nl + ["b"] * sum(case["has_bias"])
    tensors = [bc.fill_tensor(s, case["dtype"], f[k][0], f[k][1], i, case["seed"]) for i, (s, k) in enumerate(zip(shapes, kinds))]
    tdt = torch.bfloat16 if case["dtype"] == "bf16" else torch.float32
    out = torch.empty(case["batch"], case["hidden"][-1], dtype=tdt)
    if where == "device":
        tensors = [t.cuda() for t in tensors]
        out = out.cuda()
    exe = api.GraphCompiler().compile(js)
    exe.execute(dict(zip(in_ids, tensors)), {out_id: out})
    relu = case["act"] == "relu"
    ws, bs = tensors[1:1 + nl], tensors[1 + nl:]
    if case["dtype"] == "bf16":
        h = tbits(tensors[0])
        for W, b in zip(ws, bs):
            h, acc = oracle.linear_bf16(h, tbits(W), tbits(b), relu=relu, return_acc=True)
        mx, same = assert_bf16_close(tbits(out), h, max(case["hidden"]), what=name, pre=acc)
        assert_bf16_close(tbits(out), arrays[name + "_out"], max(case["hidden"]), what=name + " vs benchgc", pre=acc)
        ok, _ = bc.p2p(5e-2, 100.0, from_bits(arrays[name + "_out"]), out.cpu())
        assert ok
        print(f"{name} [{where}]: max_abs={mx:.4g} bit-identical={same:.5f}")
    else:
        h = tensors[0].cpu().numpy()
        for W, b in zip(ws, bs):
            h = oracle.matmul_f32(h, W.cpu().numpy(), b.cpu().numpy(), relu=relu)
        assert np.array_equal(out.cpu().numpy(), h)               # same accumulation order: bit-identical
        ok, _ = bc.p2p(1e-5, 100.0, torch.from_numpy(arrays[name + "_out"]), out.cpu())
        assert ok                                                    # the reference's own threshold


def test_quantized_matmul_partition_bit_exact():
    M, N, K = 256, 512, 384
    g = torch.Generator().manual_seed(5)
    A = torch.randint(0, 256, (M, K), generator=g, dtype=torch.uint8)
    W = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    scale = (torch.rand(N, generator=g) * 0.009 + 0.001)
    bias = torch.rand(N, generator=g) * 2 - 1
    js, ins, out_id = partitions.quantized_matmul(M, N, K, 128, bias=True, want_acc=True, constant_weights=True)
    out, acc = np.empty((M, N), np.float32), np.empty((M, N), np.int32)
    exe = api.GraphCompiler().compile(js)
    wacc, wout = oracle.linear_u8s8(A.numpy(), W.numpy(), scale.numpy(), bias.numpy(), zp_a=128)
    for _ in range(2):  # the second call reuses the cached constant weights and column sums
        out.fill(0); acc.fill(0)
        exe.execute({0: A.numpy(), 1: W.numpy(), 2: scale.numpy(), 3: bias.numpy()}, {4: out, 5: acc})
        assert np.array_equal(acc, wacc) and np.array_equal(out, wout)


def test_constant_tensors_are_cached_by_address_unless_switched_off():
    """A `property_type: constant` weight rewritten IN PLACE between two calls: resident (old) weights by default - the
    documented contract - and fresh weights with GC_B200_CONST_CACHE=0, as the reference re-reads them.  The switch is
    read once per process, so each setting runs in a process of its own."""
    import os
    import subprocess
    import sys

    code = r'''
import json, sys, numpy as np
from gc_b200 import api
M, N, K = 128, 64, 128
t = lambda i, s, c=False: dict({"id": i, "dtype": "f32", "shape": s}, **({"property_type": "constant"} if c else {}))
js = json.dumps({"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "strict", "graph": [
    {"kind": "MatMul", "inputs": [t(0, [M, K]), t(1, [K, N], True)], "outputs": [t(2, [M, N])]}]})
exe = api.GraphCompiler().compile(js)
A = np.ones((M, K), np.float32); W = np.ones((K, N), np.float32); out = np.empty((M, N), np.float32)
exe.execute({0: A, 1: W}, {2: out}); first = float(out[0, 0])
W *= 2.0
exe.execute({0: A, 1: W}, {2: out}); second = float(out[0, 0])
print(first, second)
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    got = {}
    for switch in ("1", "0"):
        env = dict(os.environ, GC_B200_CONST_CACHE=switch, PYTHONPATH=os.path.join(root, "graph-compiler_b200"))
        r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        got[switch] = tuple(float(x) for x in r.stdout.split()[-2:])
    assert got["1"] == (128.0, 128.0)   # cached by address: the rewritten buffer is not read again
    assert got["0"] == (128.0, 256.0)


def test_quantized_matmul_keeps_its_column_sums_across_calls_and_steps():
    """Device activations, constant host weights, and two temporaries after the matmul: the second call skips the
    column-sum kernel (the weights are resident), so the sums must have survived the first call's later steps."""
    import json

    M, N, K = 256, 512, 384
    g = torch.Generator().manual_seed(9)
    A = torch.randint(0, 256, (M, K), generator=g, dtype=torch.uint8)
    W = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    scale = (torch.rand(N, generator=g) * 0.009 + 0.001)
    t = lambda i, d, s, c=False: dict({"id": i, "dtype": d, "shape": s}, **({"property_type": "constant"} if c else {}))
    graph = [
        {"kind": "QuantizedMatMul", "attrs": {"src_zp": {"type": "s64", "value": 128}},
         "inputs": [t(0, "u8", [M, K]), t(1, "s8", [K, N], True), t(2, "f32", [N], True)], "outputs": [t(3, "f32", [M, N])]},
        {"kind": "Sigmoid", "inputs": [t(3, "f32", [M, N])], "outputs": [t(4, "f32", [M, N])]},
        {"kind": "Multiply", "inputs": [t(3, "f32", [M, N]), t(4, "f32", [M, N])], "outputs": [t(5, "f32", [M, N])]},
    ]
    js = json.dumps({"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "strict", "graph": graph})
    exe = api.GraphCompiler().compile(js)
    _, deq = oracle.linear_u8s8(A.numpy(), W.numpy(), scale.numpy(), None, zp_a=128)
    x = torch.from_numpy(deq)
    sig = 1.0 / (1.0 + torch.exp(-x))
    want = (x * sig).numpy()
    Ad = A.cuda()
    out = torch.empty(M, N, device="cuda")
    for call in range(3):
        out.zero_()
        exe.execute({0: Ad, 1: W.numpy(), 2: scale.numpy()}, {5: out})
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-6, atol=1e-6, err_msg=f"call {call}")


def test_mlp_chain_full_size_rows_against_oracle():
    """BASELINE configs[2]: 512 x (4096 -> 16384 -> 4096 -> 16384 -> 4096), N(0,0.02) weights, zero biases.
    Rows of the batch are independent, so the oracle recomputes a 16-row subset of the full-size run."""
    hidden = (4096, 16384, 4096, 16384, 4096)
    js, in_ids, out_id = partitions.mlp(512, hidden, "bf16", [True] * 4, "relu", constant_weights=True)
    X = bc.fill_tensor((512, 4096), "bf16", "N", (0, 1), 0).cuda()
    Ws = [bc.fill_tensor((hidden[i], hidden[i + 1]), "bf16", "N", (0, 0.02), 1 + i).cuda() for i in range(4)]
    Bs = [torch.zeros(hidden[i + 1], dtype=torch.bfloat16, device="cuda") for i in range(4)]
    out = torch.empty(512, 4096, dtype=torch.bfloat16, device="cuda")
    exe = api.GraphCompiler().compile(js)
    exe.execute(dict(zip(in_ids, [X] + Ws + Bs)), {out_id: out})
    rows = torch.tensor([0, 1, 17, 100, 127, 128, 129, 255, 256, 300, 383, 384, 400, 470, 510, 511])
    h = tbits(X[rows.cuda()])
    for W, b in zip(Ws, Bs):
        h = oracle.linear_bf16(h, tbits(W), tbits(b), relu=True)
    mx, same = assert_bf16_close(tbits(out[rows.cuda()]), h, 16384, what="mlp chain", floor_div=1.0)
    # every layer on its own (fed the oracle's activations) holds the single-layer rule
    h = tbits(X[rows.cuda()])
    from gc_b200 import lib
    for i, (W, b) in enumerate(zip(Ws, Bs)):
        got = lib.matmul_bf16(from_bits(h, "cuda"), W, b, relu=True)
        h = oracle.linear_bf16(h, tbits(W), tbits(b), relu=True)
        mxl, samel = assert_bf16_close(tbits(got), h, W.shape[0], what=f"mlp layer {i}")
        print(f"  layer {i}: max_abs={mxl:.4g} bit-identical={samel:.5f}")
    print(f"mlp chain 512x4096..: max_abs={mx:.4g} bit-identical={same:.5f}")


@pytest.mark.parametrize("layers", [1, 3])
def test_host_buffers_with_overlapped_copies_match_device_buffers(layers):
    """With host tensors and >= 512 rows the first / last MatMul run as two row blocks so that the host
    copies overlap the math; every output row must equal the device-tensor run of the same partition
    (same K order per row; K is short enough here that no block takes a different K split)."""
    batch, hidden = 1024, [256, 512, 384, 256][:layers + 1]
    js, in_ids, out_id = partitions.mlp(batch, hidden, "bf16", [True] * layers, "relu")
    g = torch.Generator().manual_seed(3)
    X = torch.randn(batch, hidden[0], generator=g).bfloat16()
    Ws = [(torch.randn(hidden[i], hidden[i + 1], generator=g) * 0.1).bfloat16() for i in range(layers)]
    Bs = [torch.randn(hidden[i + 1], generator=g).bfloat16() for i in range(layers)]
    exe = api.GraphCompiler().compile(js)
    out_h = torch.empty(batch, hidden[-1], dtype=torch.bfloat16).pin_memory()
    out_d = torch.empty(batch, hidden[-1], dtype=torch.bfloat16, device="cuda")
    exe.execute(dict(zip(in_ids, [X.pin_memory()] + Ws + Bs)), {out_id: out_h})
    exe.execute(dict(zip(in_ids, [t.cuda() for t in [X] + Ws + Bs])), {out_id: out_d})
    assert torch.equal(out_h, out_d.cpu())
    # and a second call with new activations in the same host buffers (staging buffers are reused)
    X2 = torch.randn(batch, hidden[0], generator=g).bfloat16()
    exe.execute(dict(zip(in_ids, [X2] + Ws + Bs)), {out_id: out_h})
    exe.execute(dict(zip(in_ids, [t.cuda() for t in [X2] + Ws + Bs])), {out_id: out_d})
    assert torch.equal(out_h, out_d.cpu())
    h = tbits(X2)
    for W, b in zip(Ws, Bs):
        h, acc = oracle.linear_bf16(h, tbits(W), tbits(b), relu=True, return_acc=True)
    assert_bf16_close(tbits(out_h), h, max(hidden), what="overlapped host path", pre=acc, floor_div=1.0 if layers > 1 else 16.0)


def _llama2_reference(t, eps):
    """The block of onednn-graph-llama2.mlir:5-45 on the host: bf16 ops are evaluated in f32 and rounded
    after every op (Pipeline.cpp:81-90), MatMul accumulates in f32 and rounds once, f32 ops stay f32."""
    r = lambda v: v.to(torch.bfloat16).to(torch.float32)                   # one bf16 rounding
    f = lambda v: v.to(torch.float32)
    mm = lambda a, w: r(f(a) @ f(w).t())

    def rmsnorm(h, gamma):
        c = f(h)
        rs = torch.pow(torch.pow(c, 2.0).mean(-1, keepdim=True) + eps, -0.5)
        return r(f(gamma) * r(c * rs))

    t7 = r(f(t["resid"]) + mm(t["x"], t["wo"]))
    t27 = rmsnorm(t7, t["g1"])
    t30 = mm(t27, t["w_gate"])
    t32 = r(r(torch.sigmoid(t30)) * t30)
    t36 = r(t32 * mm(t27, t["w_up"]))
    t39 = mm(t36, t["w_down"])
    t41 = r(t7 + t39)
    return rmsnorm(t41, t["g2"]), t41, t7.abs() + t39.abs()


@pytest.mark.parametrize("dims", [(1, 32, 512, 1024), (1, 32, 4096, 11008), (2, 40, 256, 384)])
def test_llama2_mlp_partition(dims):
    """RMSNorm + SiLU-gated MLP with three transpose_b MatMuls, all eleven reference op kinds but ReLU/Sub/Div."""
    B, S, H, I = dims
    js, ids, outs = partitions.llama2_mlp(B, S, H, I)
    g = torch.Generator().manual_seed(11)
    bf = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).bfloat16()
    t = {"x": bf(B, S, H), "wo": bf(H, H, scale=H ** -0.5), "resid": bf(B, S, H), "g1": bf(H) * 0.1 + 1, "w_gate": bf(I, H, scale=H ** -0.5),
         "w_up": bf(I, H, scale=H ** -0.5), "w_down": bf(H, I, scale=I ** -0.5), "g2": bf(H) * 0.1 + 1}
    t["g1"], t["g2"] = t["g1"].bfloat16(), t["g2"].bfloat16()
    eps = torch.tensor([1e-5], dtype=torch.float32)
    want_norm, want_res, add_operands = _llama2_reference(t, eps)
    exe = api.GraphCompiler().compile(js)
    ins = {ids[k]: v.cuda() for k, v in t.items()}
    ins[ids["eps"]] = eps.cuda()
    o_norm = torch.empty(B, S, H, dtype=torch.bfloat16, device="cuda")
    o_res = torch.empty(B, S, H, dtype=torch.bfloat16, device="cuda")
    exe.execute(ins, {outs[0]: o_norm, outs[1]: o_res})
    # The residual is bf16(t7 + bf16(matmul)): a 1-ulp flip of either rounded operand (any change of f32
    # summation order causes some) reaches the sum as up to two ulps — the double-rounding allowance of
    # assert_bf16_close with the operands' magnitudes as `pre`.  RMSNorm is scale-free: the normed output
    # inherits those two ulps and adds one per rounding of its two bf16 multiplies — four ulps of at most
    # 2^-7 relative each (pre = 3 |want|).
    for name, got, want, pre in (("residual", o_res, want_res, add_operands), ("normed", o_norm, want_norm, 3 * want_norm.abs())):
        mx, same = assert_bf16_close(tbits(got), tbits(want.bfloat16()), max(H, I), what=f"llama2 {name} {dims}", floor_div=1.0,
                                     pre=pre.numpy())
        print(f"llama2 {dims} {name}: max_abs={mx:.4g} bit-identical={same:.5f}")


def test_repeated_device_calls_replay_a_graph_with_identical_results():
    """From the third call with the same device addresses the launch list is replayed as a CUDA graph; results
    must equal those of an eager run (a first call on fresh addresses), and the launch counter keeps counting."""
    from gc_b200 import lib

    batch, hidden = 256, [256, 512, 256, 128]
    js, in_ids, out_id = partitions.mlp(batch, hidden, "bf16", [True] * 3, "relu")
    g = torch.Generator().manual_seed(5)
    X = torch.randn(batch, hidden[0], generator=g).bfloat16().cuda()
    Ws = [(torch.randn(hidden[i], hidden[i + 1], generator=g) * 0.1).bfloat16().cuda() for i in range(3)]
    Bs = [torch.randn(hidden[i + 1], generator=g).bfloat16().cuda() for i in range(3)]
    out = torch.empty(batch, hidden[-1], dtype=torch.bfloat16, device="cuda")
    exe = api.GraphCompiler().compile(js)
    per_call = []
    for it in range(5):
        X.copy_(torch.randn(batch, hidden[0], generator=g).bfloat16())
        l0 = lib.launch_count()
        exe.execute(dict(zip(in_ids, [X] + Ws + Bs)), {out_id: out})
        per_call.append(lib.launch_count() - l0)
        fresh_out = torch.empty_like(out)
        exe.execute(dict(zip(in_ids, [X.clone()] + Ws + Bs)), {out_id: fresh_out})   # new address: eager
        assert torch.equal(out, fresh_out), it
    assert len(set(per_call)) == 1 and per_call[0] == 3, per_call
    # asynchronous form on the caller's stream
    for it in range(4):
        X.copy_(torch.randn(batch, hidden[0], generator=g).bfloat16())
        exe.execute_on_stream(dict(zip(in_ids, [X] + Ws + Bs)), {out_id: out})
        torch.cuda.synchronize()
        fresh_out = torch.empty_like(out)
        exe.execute(dict(zip(in_ids, [X.clone()] + Ws + Bs)), {out_id: fresh_out})
        assert torch.equal(out, fresh_out), it
