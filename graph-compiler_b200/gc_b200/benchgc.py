"""benchgc-compatible command line for the B200 backend.

    python -m gc_b200.benchgc --driver pattern --case mlp --batch_size 128 --hidden_size_list 512x256 \
        --has_bias 1 --act_type relu --dtype bf16 [--mode C|P] [--fill i:T:params] [--cmp i:P:thr:zero%] [--seed s]
    python -m gc_b200.benchgc --driver linalg --case matmul --md 0:32x128xbf16 --md 1:128x64xbf16 --md 2:32x64xbf16
    python -m gc_b200.benchgc --driver mlir --case partition.mlir

Same flags, fills, comparison rules and result format as the reference's harness
(test/benchgc/src/benchgc/__main__.py:41-206 flags, :300-380 the two modes;
arg/__init__.py:94-153 fills; arg/compare.py:60-137 p2p; bench.py:33-60 timing),
for the subset of modules the matmul / MLP path covers.  Where the reference JIT-compiles
the module with `gc-cpu-pipeline`, this harness lowers the same MLIR text to a oneDNN-graph
partition and runs it through the C API on the GPU.  Mode C (host tensors in and out) compares
against a torch interpretation of the module on the host, as the reference's harness does
(test/benchgc/src/benchgc/linalg/*.py `ref_*`); mode P (arguments resident in device memory)
prints ``{"args":…, "compile_cost(ms)":…, "execute_cost(ms)":…}``.
"""
from __future__ import annotations

import argparse
import json
import sys
import timeit
from typing import Dict, List

import torch

from . import benchgc_compat as compat
from . import mlir_text

NO_VERBOSE, MODULE_VERBOSE, ARG_VERBOSE, COMPARE_VERBOSE = 0, 1, 2, 3


class Arg:
    """One entry-function argument or result (test/benchgc/src/benchgc/arg/arg.py)."""

    def __init__(self, index: int):
        self.index, self.dtype, self.shape = index, "", []
        self.fill_type, self.fill_param = "-", []
        self.cmp_type, self.cmp_param = "-", []

    def set_md(self, md: str):
        parts = md.split("x")
        self.dtype = parts[-1]
        self.shape = [int(p) for p in parts[:-1] if p != ""]

    def set_fill(self, fill: str):
        s = fill.split(":")
        self.fill_type, self.fill_param = s[0], s[1:]

    def set_cmp(self, cmp: str):
        s = cmp.split(":")
        self.cmp_type, self.cmp_param = s[0], s[1:]

    def describe(self) -> str:
        return (f"arg{self.index} shape: {self.shape} dtype: {self.dtype} fill_type: {self.fill_type} "
                f"fill_param: {self.fill_param} cmp_type: {self.cmp_type} cmp_param: {self.cmp_param}")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="benchmark tool for graph compiler (B200 backend)")
    p.add_argument("--mode", choices=["C", "P"], default="C")
    p.add_argument("--driver", choices=["linalg", "tensor", "mlir", "pattern"])
    p.add_argument("--case", type=str)
    p.add_argument("--md", type=str, default=[], action="append")
    p.add_argument("--fill", type=str, default=[], action="append")
    p.add_argument("--cmp", type=str, default=[], action="append")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--verbose", type=int, default=NO_VERBOSE, choices=range(0, 7))
    p.add_argument("--entry", type=str, default="entry")
    p.add_argument("--ir_printing", action="store_true")
    p.add_argument("--cpu_cache_sizes", type=str)        # accepted and ignored: CPU target description
    p.add_argument("--max_vector_width", type=int)       # accepted and ignored
    p.add_argument("--cast", choices=["cast_signed", "cast_unsigned"], default="cast_signed")
    p.add_argument("--bench_kind", choices=["py", "wrapper"], default="py")
    p.add_argument("--warm_up", type=int, default=100)
    p.add_argument("--repeat", type=int, default=100)
    # --driver pattern --case mlp (test/benchgc/src/benchgc/pattern/mlp.py:33-49)
    p.add_argument("--batch_size", type=int, default=1)
    p.add_argument("--hidden_size_list", type=str, default="")
    p.add_argument("--has_bias", type=str)
    p.add_argument("--act_type", choices=["noop", "relu", "sigmoid"], default="noop")
    p.add_argument("--dtype", choices=["f32", "bf16"], default="f32")
    return p


def _module_text(flags) -> str:
    if flags.driver == "mlir":
        with open(flags.case, "r") as f:
            return f.read()
    if flags.driver == "pattern":
        if flags.case != "mlp":
            raise mlir_text.Unimplemented(f"pattern {flags.case}")
        hidden = [int(x) for x in flags.hidden_size_list.split("x") if x]
        layers = len(hidden) - 1
        if flags.batch_size <= 0 or layers < 1:
            raise ValueError("batch size should be greater than 0 and hidden_size_list should have at least 2 elements")
        has_bias = [False] * layers if flags.has_bias is None else [bool(int(x)) for x in flags.has_bias.split("x")]
        if len(has_bias) != layers:
            raise ValueError("has_bias should have the same length as hidden_size_list")
        return mlir_text.mlp_module(flags.batch_size, hidden, has_bias, flags.act_type, flags.dtype, flags.entry)
    if flags.driver == "linalg":
        args = [Arg(i) for i in range(len(flags.md))]
        for md in flags.md:
            idx, rest = md.split(":", 1)
            args[int(idx)].set_md(rest)
        if len(args) != 3:
            raise ValueError("a matmul case takes three --md descriptions")
        ty = [mlir_text.TensorType(tuple(a.shape), mlir_text._MLIR_DTYPES.get(a.dtype, a.dtype)) for a in args]
        return mlir_text.matmul_module(flags.case, ty[0], ty[1], ty[2], flags.entry)
    raise mlir_text.Unimplemented(f"driver {flags.driver}")


def _matmul_driver_fill(shape, dtype: str, name: str, src_dt: str, wei_dt: str, dst_dt: str, amp: int, seed: int) -> torch.Tensor:
    """The integer-valued fill of the matmul driver: products and sums stay exactly representable
    (test/benchgc/src/benchgc/arg/matmul.py:97-147)."""
    rng = [{"f32": (-64, 64), "bf16": (-4, 4), "f16": (-4, 4)}, {"f32": (-128, 128), "bf16": (-8, 8), "f16": (-2, 2)}]
    digits = {"f32": 24, "f64": 53, "s8": 7, "u8": 8, "f16": 11, "bf16": 8}
    s_lo, s_hi = rng[0][src_dt]
    w_lo, w_hi = rng[1][wei_dt]
    max_value = max(abs(s_lo), abs(s_hi)) * max(abs(w_lo), abs(w_hi))
    safe_n_acc = (1 << min(digits["f32"], digits[dst_dt])) // max_value
    if name == "src":
        lo, hi, density = s_lo, s_hi, 1.0
    else:
        lo, hi, density = w_lo, w_hi, min(safe_n_acc / int(amp), 1.0)
    compat.seed_all(seed + (0 if name == "src" else 1))
    value = torch.bernoulli(torch.full(list(shape), density)) * torch.randint(lo, hi, list(shape))
    while value.flatten()[0] <= 0:
        value.flatten()[0] = torch.randint(lo, hi + 1, size=[1])[0].item()
    return value.to(compat.get_dtype(dtype))


def _defaults(flags, args: List[Arg], n_in: int):
    """Default fill and compare per argument (arg/__init__.py:41-92, arg/matmul.py:47-95,149-173, pattern/mlp.py:152-173)."""
    for i, a in enumerate(args):
        is_ret = i >= n_in
        if a.fill_type == "-":
            if is_ret:
                a.fill_type, a.fill_param = "Z", []
            elif flags.driver == "linalg" and i <= 1:
                amp = a.shape[-1] if (flags.case == "matmul_transpose_b" or (flags.case == "matmul" and i == 0)) else a.shape[-2]
                a.fill_type = "D"
                a.fill_param = ["matmul", "src" if i == 0 else "wei", args[0].dtype, args[1].dtype, args[2].dtype, str(amp)]
            elif flags.driver == "pattern":
                a.fill_type, a.fill_param = "U", ["0", "1"]
            else:
                a.fill_type, a.fill_param = "N", ["0", "1"]
        if a.cmp_type == "-":
            fp = a.dtype in ("f32", "bf16", "f16")
            if is_ret and flags.driver == "linalg":
                eps = 1e-6 if a.dtype == "f32" else torch.finfo(compat.get_dtype(a.dtype)).eps
                a.cmp_type, a.cmp_param = "P", [str(eps), "90.0"]
            elif is_ret and flags.driver == "pattern":
                a.cmp_type, a.cmp_param = "P", [str(1e-5 if a.dtype == "f32" else 5e-2), "100.0"]
            else:
                a.cmp_type, a.cmp_param = "P", [str(1e-5) if fp else "0", "70.0" if is_ret else "100.0"]


def _fill(flags, a: Arg) -> torch.Tensor:
    if a.fill_type == "D":
        if not a.fill_param or a.fill_param[0] != "matmul":
            raise mlir_text.Unimplemented(f"driver fill {a.fill_param[:1]}")
        _, name, sdt, wdt, ddt, amp = a.fill_param
        return _matmul_driver_fill(a.shape, a.dtype, name, sdt, wdt, ddt, int(amp), flags.seed)
    if a.fill_type == "F":
        t = torch.load(a.fill_param[0])
        if tuple(t.shape) != tuple(a.shape) or t.dtype != compat.get_dtype(a.dtype):
            raise ValueError(f"tensor object from file {a.fill_param[0]} does not match shape or dtype")
        return t
    return compat.fill_tensor(a.shape, a.dtype, a.fill_type, a.fill_param, a.index, flags.seed)


def ref_run(fn: mlir_text.Func, tensors: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
    """Host interpretation of the parsed module, op by op in each tensor's own dtype — what the reference's
    harness computes with torch as its ground truth (test/benchgc/src/benchgc/linalg/matmul.py `ref_matmul*`,
    binary.py, eltwise.py)."""
    env = dict(tensors)

    def val(name: str) -> torch.Tensor:
        if name in env:
            return env[name]
        v = fn.values[name]
        dt = compat.get_dtype(v.type.dtype)
        if v.kind in ("const", "zero_fill"):
            return torch.full(v.type.shape, v.const or 0.0, dtype=dt)
        if v.kind == "bcast":
            src = val(v.src)
            shape = [1 if i in v.bdims else d for i, d in enumerate(v.type.shape)]
            return src.reshape(shape).expand(v.type.shape)
        raise mlir_text.ParseError(f"{name} has no value")

    for op in fn.ops:
        x = [val(n) for n in op.ins]
        if op.name == "matmul":
            a = x[0].transpose(-1, -2) if op.attrs["transpose_a"] else x[0]
            b = x[1].transpose(-1, -2) if op.attrs["transpose_b"] else x[1]
            env[op.out] = torch.matmul(a, b)
        elif op.name == "add":
            env[op.out] = torch.add(x[0], x[1])
        elif op.name == "sub":
            env[op.out] = torch.sub(x[0], x[1])
        elif op.name == "mul":
            env[op.out] = torch.mul(x[0], x[1])
        elif op.name == "div":
            env[op.out] = torch.div(x[0], x[1])
        elif op.name == "relu":
            env[op.out] = torch.max(x[0], torch.zeros_like(x[0]))
        elif op.name == "sigmoid":
            env[op.out] = torch.sigmoid(x[0])
        elif op.name == "neg":
            env[op.out] = torch.neg(x[0])
        elif op.name == "exp":
            env[op.out] = torch.exp(x[0])
        elif op.name == "cast":
            env[op.out] = x[0].to(compat.get_dtype(fn.values[op.out].type.dtype))
        elif op.name == "reshape":
            env[op.out] = x[0].reshape(fn.values[op.out].type.shape)
        elif op.name == "pow":
            env[op.out] = torch.pow(x[0], op.attrs["beta"])
        elif op.name == "reduce_sum":
            env[op.out] = torch.sum(x[0], dim=list(op.attrs["axes"]))
        elif op.name == "qmatmul":
            # exact in f64: |sum| < 2^53
            env[op.out] = torch.matmul(x[0].double() - float(op.attrs["src_zp"]), x[1].double()).to(torch.int32)
        elif op.name == "softmax":
            env[op.out] = torch.softmax(x[0], op.attrs["dimension"])
        elif op.name == "batch_matmul":
            a = x[0].transpose(-1, -2) if op.attrs["transpose_a"] else x[0]
            b = x[1].transpose(-1, -2) if op.attrs["transpose_b"] else x[1]
            env[op.out] = torch.matmul(a, b)
        else:
            raise mlir_text.Unimplemented(op.name)
    return [env[r] for r in fn.results]


def main(argv=None) -> int:
    flags = build_parser().parse_args(argv)
    if flags.driver is None or flags.case is None:
        print("--driver and --case are required", file=sys.stderr)
        return 2
    try:
        text = _module_text(flags)
        fn = mlir_text.parse_module(text, flags.entry)
        graph_json, arg_ids, out_ids, consts = mlir_text.to_partition(fn)
    except mlir_text.Unimplemented as e:
        print(f"unimplemented: {e}", file=sys.stderr)
        return 3
    if flags.verbose >= MODULE_VERBOSE:
        print(text)

    args: List[Arg] = []
    for i, v in enumerate(fn.args):
        a = Arg(i)
        a.dtype, a.shape = v.type.dtype, list(v.type.shape)
        args.append(a)
    for j, t in enumerate(fn.result_types):
        a = Arg(len(fn.args) + j)
        a.dtype, a.shape = t.dtype, list(t.shape)
        args.append(a)
    for f in flags.fill:
        idx, rest = f.split(":", 1)
        args[int(idx)].set_fill(rest)
    for c in flags.cmp:
        idx, rest = c.split(":", 1)
        args[int(idx)].set_cmp(rest)
    _defaults(flags, args, len(fn.args))
    if flags.verbose >= ARG_VERBOSE:
        for a in args:
            print(a.describe())

    from .api import GraphCompiler   # needs the CUDA library; fails loudly without it

    tensors = {v.name: _fill(flags, args[i]) for i, v in enumerate(fn.args)}
    outs = [torch.zeros(t.shape, dtype=compat.get_dtype(t.dtype)) for t in fn.result_types]
    gc = GraphCompiler()
    t0 = timeit.default_timer()
    exe = gc.compile(graph_json)
    compile_cost = (timeit.default_timer() - t0) * 1000
    used = set(json.loads(graph_json)["input_ports"])
    ins = {arg_ids[i]: tensors[v.name] for i, v in enumerate(fn.args) if arg_ids[i] in used}
    # splat constants the module uses as operands travel as one-element inputs
    ins.update({cid: torch.full((1,), val, dtype=compat.get_dtype(dt)) for cid, (val, dt) in consts.items() if cid in used})
    outs_b = dict(zip(out_ids, outs))

    if flags.mode == "C":
        exe.execute(ins, outs_b)
        ref = ref_run(fn, {k: t.clone() for k, t in tensors.items()})
        fail, mistrust = False, False
        for j, (r, o) in enumerate(zip(ref, outs)):
            a = args[len(fn.args) + j]
            if a.cmp_type == "N":
                ok, mis = compat.norm(float(a.cmp_param[0]), r, o)
            elif a.cmp_type == "P":
                if flags.verbose >= COMPARE_VERBOSE:
                    print(f"p2p check: threshold: {float(a.cmp_param[0]):.7f}")
                ok, mis = compat.p2p(float(a.cmp_param[0]), float(a.cmp_param[1]), r, o)
            else:
                raise mlir_text.Unimplemented(f"compare type {a.cmp_type}")
            fail |= not ok
            mistrust |= bool(mis)
        name = f"{flags.driver}.{flags.case}"
        if fail:
            print(f"FAIL: {name}")
            return 1
        print(f"MISTRUST: {name}" if mistrust else f"PASSED: {name}")
        return 0

    # performance mode: the reference times the call with its arguments already in the memory the
    # device computes from (host memory for a CPU, test/benchgc/src/benchgc/bench.py:33-60); the same
    # here: arguments are placed in device memory once, every timed call is the synchronous C API call
    dev_ins = {k: t.cuda() for k, t in ins.items()}
    dev_outs = {k: t.cuda() for k, t in outs_b.items()}
    bound = exe.bind(dev_ins, dev_outs)
    run = bound.run
    timeit.timeit(run, number=flags.warm_up)
    total = timeit.timeit(run, number=flags.repeat)
    print("===========bench result===========")
    print(json.dumps({"args": vars(flags), "compile_cost(ms)": compile_cost, "execute_cost(ms)": total * 1000 / flags.repeat}, indent=4))
    return 0


if __name__ == "__main__":
    sys.exit(main())
