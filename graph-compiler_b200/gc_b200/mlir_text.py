"""Structural reader for the linalg-on-tensor MLIR that benchgc produces for the matmul / MLP path.

benchgc hands the reference one `func.func` whose body is a straight line of
`tensor.empty`, `arith.constant`, `linalg.fill`, `linalg.matmul[_transpose_a|_transpose_b]`,
`linalg.broadcast`, `linalg.add|sub|mul|div`, `linalg.max` (against a zero splat: ReLU),
`linalgx.sigmoid` and `return` (test/benchgc/src/benchgc/pattern/mlp.py:68-150,
test/benchgc/src/benchgc/linalg/matmul.py).  No MLIR library is needed to read
that subset: this module parses the text line by line into a list of ops over
named SSA values, checks the shapes, and lowers the list to the oneDNN-graph
JSON partition the C API compiles (the inverse of
lib/gc/Transforms/OneDNNGraphToLinalg.cpp:345-499).  Anything outside the subset
raises ``Unimplemented`` — the same class of answer the reference gives for an
unsupported op kind.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class Unimplemented(Exception):
    """The text uses an op, type or form outside the supported subset."""


class ParseError(Exception):
    """The text is not well-formed for the subset (bad type, unknown value, shape mismatch)."""


_MLIR_DTYPES = {"f32": "f32", "bf16": "bf16", "f16": "f16", "i8": "s8", "si8": "s8", "ui8": "u8", "i32": "s32", "si32": "s32"}


@dataclass
class TensorType:
    shape: Tuple[int, ...]
    dtype: str            # oneDNN-graph spelling (f32, bf16, s8, ...)

    @property
    def rank(self):
        return len(self.shape)


def parse_type(text: str) -> TensorType:
    """`tensor<128x512xbf16>` -> TensorType; a bare element type is a rank-0 scalar."""
    text = text.strip()
    m = re.fullmatch(r"tensor<(.*)>", text)
    if not m:
        if text in _MLIR_DTYPES:
            return TensorType((), _MLIR_DTYPES[text])
        raise Unimplemented(f"type {text!r}")
    parts = m.group(1).split("x")
    et = parts[-1].strip()
    if et not in _MLIR_DTYPES:
        raise Unimplemented(f"element type {et!r}")
    dims = []
    for p in parts[:-1]:
        if not p.isdigit():
            raise Unimplemented(f"dynamic or malformed dimension in {text!r}")
        dims.append(int(p))
    return TensorType(tuple(dims), _MLIR_DTYPES[et])


@dataclass
class Value:
    name: str
    type: TensorType
    kind: str                       # arg | empty | const | zero_fill | bcast | op
    const: Optional[float] = None   # splat value for kind == const
    src: Optional[str] = None       # broadcast source
    bdims: Tuple[int, ...] = ()     # dimensions added by the broadcast


@dataclass
class Op:
    name: str                       # matmul | add | sub | mul | div | relu | sigmoid
    ins: List[str]
    out: str
    attrs: Dict[str, object] = field(default_factory=dict)


@dataclass
class Func:
    entry: str
    args: List[Value]
    results: List[str]
    result_types: List[TensorType]
    values: Dict[str, Value]
    ops: List[Op]


_FUNC_RE = re.compile(r"func\.func\s+@(\w+)\s*\((.*?)\)\s*->\s*(.+?)\s*(?:attributes\s*\{.*?\}\s*)?\{\s*$")
_RES_RE = re.compile(r"^\s*(%[\w#.]+)\s*=\s*(.*)$")


def _split_top(text: str, sep: str = ",") -> List[str]:
    """Split at `sep` outside <>, (), [] and {}."""
    out, depth, cur = [], 0, []
    for ch in text:
        if ch in "<([{":
            depth += 1
        elif ch in ">)]}":
            depth -= 1
        if ch == sep and depth == 0:
            out.append("".join(cur))
            cur = []
        else:
            cur.append(ch)
    if "".join(cur).strip():
        out.append("".join(cur))
    return [o.strip() for o in out]


def _operands(clause: str) -> Tuple[List[str], List[TensorType]]:
    """`%a, %b : tensor<..>, tensor<..>` -> names, types."""
    if ":" not in clause:
        raise ParseError(f"operand clause without types: {clause!r}")
    names, types = clause.split(":", 1)
    ns = [n.strip() for n in names.split(",") if n.strip()]
    ts = [parse_type(t) for t in _split_top(types)]
    if len(ns) != len(ts):
        raise ParseError(f"{len(ns)} operands but {len(ts)} types in {clause!r}")
    return ns, ts


def _clause(body: str, key: str) -> Optional[str]:
    """Text inside `key( ... )` with balanced parentheses, or None."""
    i = body.find(key + "(")
    if i < 0:
        return None
    j = i + len(key) + 1
    depth, k = 1, j
    while k < len(body) and depth:
        depth += body[k] == "("
        depth -= body[k] == ")"
        k += 1
    return body[j:k - 1]


_BINARY = {"linalg.add": "add", "linalg.sub": "sub", "linalg.mul": "mul", "linalg.div": "div"}
_MATMUL = {"linalg.matmul": (False, False), "linalg.matmul_transpose_a": (True, False), "linalg.matmul_transpose_b": (False, True)}


def parse_module(text: str, entry: str = "entry") -> Func:
    """Parse the entry function of a module printed by MLIR's generic-free (pretty) printer."""
    lines = [ln.rstrip() for ln in text.splitlines()]
    fn = None
    body: List[str] = []
    depth_in = False
    for ln in lines:
        s = ln.strip()
        if not depth_in:
            m = _FUNC_RE.search(s)
            if m and m.group(1) == entry:
                fn = m
                depth_in = True
            continue
        if s == "}":
            break
        if s:
            body.append(s)
    if fn is None:
        raise ParseError(f"no func.func @{entry} found")

    values: Dict[str, Value] = {}
    args: List[Value] = []
    for a in _split_top(fn.group(2)):
        if not a:
            continue
        name, ty = a.split(":", 1)
        v = Value(name.strip(), parse_type(ty), "arg")
        values[v.name] = v
        args.append(v)
    res_text = fn.group(3).strip()
    if res_text.startswith("("):
        res_text = res_text[1:res_text.rindex(")")]
    result_types = [parse_type(t) for t in _split_top(res_text)]

    def get(name: str) -> Value:
        if name not in values:
            raise ParseError(f"use of undefined value {name}")
        return values[name]

    ops: List[Op] = []
    results: List[str] = []
    for s in body:
        if s.startswith("return") or s.startswith("func.return"):
            rest = s.split("return", 1)[1].strip()
            if rest:
                names = rest.split(":", 1)[0]
                results = [n.strip() for n in names.split(",") if n.strip()]
            continue
        m = _RES_RE.match(s)
        if not m:
            raise Unimplemented(f"statement {s!r}")
        res, rhs = m.group(1), m.group(2)
        opname = rhs.split()[0].split("(")[0]
        if opname == "tensor.empty":
            values[res] = Value(res, parse_type(rhs.rsplit(":", 1)[1]), "empty")
        elif opname == "arith.constant":
            ty = parse_type(rhs.rsplit(":", 1)[1])
            lit = rhs[len("arith.constant"):].rsplit(":", 1)[0].strip()
            d = re.fullmatch(r"dense<(.+)>", lit)
            if d:
                lit = d.group(1)
            try:
                c = float(lit)
            except ValueError:
                raise Unimplemented(f"non-splat constant {lit!r}")
            values[res] = Value(res, ty, "const", const=c)
        elif opname == "linalg.fill":
            ins, _ = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            c = get(ins[0])
            if c.kind != "const":
                raise Unimplemented("linalg.fill with a non-constant scalar")
            get(outs[0])
            if c.const == 0.0:
                values[res] = Value(res, ot[0], "zero_fill")
            else:
                values[res] = Value(res, ot[0], "const", const=c.const)
        elif opname in _MATMUL:
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            for n, t in zip(ins + outs, it + ot):
                if get(n).type.shape != t.shape or get(n).type.dtype != t.dtype:
                    raise ParseError(f"type of {n} does not match its definition")
            init = get(outs[0])
            if init.kind not in ("zero_fill",):
                # accumulating into live data is outside the partition forms the C API takes
                raise Unimplemented("linalg.matmul whose init operand is not a zero fill")
            ta, tb = _MATMUL[opname]
            a, b = it
            if a.rank != 2 or b.rank != 2:
                raise Unimplemented("matmul operands must be rank 2")
            m_, k_ = (a.shape[1], a.shape[0]) if ta else a.shape
            k2, n_ = (b.shape[1], b.shape[0]) if tb else b.shape
            if k_ != k2 or ot[0].shape != (m_, n_):
                raise ParseError(f"matmul shapes do not agree: {a.shape} x {b.shape} -> {ot[0].shape}")
            values[res] = Value(res, ot[0], "op")
            ops.append(Op("matmul", ins, res, {"transpose_a": ta, "transpose_b": tb}))
        elif opname == "linalg.broadcast":
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            d = re.search(r"dimensions\s*=\s*\[([\d,\s]*)\]", rhs)
            if not d:
                raise ParseError("linalg.broadcast without dimensions")
            bd = tuple(int(x) for x in d.group(1).split(",") if x.strip())
            kept = tuple(x for i, x in enumerate(ot[0].shape) if i not in bd)
            if kept != it[0].shape:
                raise ParseError(f"broadcast of {it[0].shape} along {bd} does not give {ot[0].shape}")
            get(ins[0])
            values[res] = Value(res, ot[0], "bcast", src=ins[0], bdims=bd)
        elif opname in _BINARY or opname == "linalg.max":
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            for n in ins + outs:
                get(n)
            if it[0].shape != ot[0].shape or it[1].shape != ot[0].shape:
                raise ParseError(f"{opname}: operand shapes differ from the result shape")
            if opname == "linalg.max":
                zeros = [n for n in ins if values[n].kind in ("const", "zero_fill") and (values[n].const or 0.0) == 0.0]
                if len(zeros) != 1:
                    raise Unimplemented("linalg.max is only taken as ReLU (one operand a zero splat)")
                x = ins[1] if zeros[0] == ins[0] else ins[0]
                ops.append(Op("relu", [x], res))
            else:
                ops.append(Op(_BINARY[opname], ins, res))
            values[res] = Value(res, ot[0], "op")
        elif opname == "linalgx.sigmoid":
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            get(ins[0])
            ops.append(Op("sigmoid", ins, res))
            values[res] = Value(res, ot[0], "op")
        else:
            raise Unimplemented(f"op {opname}")

    if not results:
        raise ParseError("function does not return a value")
    for r, t in zip(results, result_types):
        if get(r).type.shape != t.shape:
            raise ParseError(f"returned value {r} does not have the declared result type")
    return Func(entry, args, results, result_types, values, ops)


# ------------------------------------------------------------------------------------- lowering
_KIND = {"add": "Add", "sub": "Subtract", "mul": "Multiply", "div": "Divide", "relu": "ReLU", "sigmoid": "Sigmoid"}


def to_partition(fn: Func) -> Tuple[str, List[int], List[int]]:
    """The oneDNN-graph JSON of `fn`.  Returns (json text, input tensor ids in argument order, output ids).

    A broadcast along the leading dimensions becomes numpy auto-broadcast of its source
    (lib/gc/Transforms/OneDNNGraphToLinalg.cpp:484-494 goes the other way).
    """
    ids: Dict[str, int] = {a.name: i for i, a in enumerate(fn.args)}
    nxt = len(fn.args)

    def tensor(name: str) -> dict:
        v = fn.values[name]
        if v.kind == "bcast":
            lead = tuple(range(len(v.bdims)))
            if v.bdims != lead:
                raise Unimplemented("broadcast along a non-leading dimension")
            return tensor(v.src)
        if v.kind in ("const", "zero_fill", "empty"):
            raise Unimplemented(f"{name}: a constant or uninitialised tensor as a graph input")
        if name not in ids:
            raise ParseError(f"{name} is used before it is produced")
        return {"id": ids[name], "dtype": v.type.dtype, "shape": list(v.type.shape)}

    graph = []
    for k, op in enumerate(fn.ops):
        ins = [tensor(n) for n in op.ins]
        ids[op.out] = nxt
        nxt += 1
        node = {"id": k, "name": f"{op.name}_{k}", "kind": "MatMul" if op.name == "matmul" else _KIND[op.name], "attrs": {},
                "inputs": ins, "outputs": [tensor(op.out)]}
        if op.name == "matmul":
            for a in ("transpose_a", "transpose_b"):
                if op.attrs[a]:
                    node["attrs"][a] = {"type": "bool", "value": 1}
        elif op.name in ("add", "sub", "mul", "div"):
            node["attrs"]["auto_broadcast"] = {"type": "string", "value": "numpy"}
        graph.append(node)
    used = {t["id"] for n in graph for t in n["inputs"]}
    in_ids = [ids[a.name] for a in fn.args if ids[a.name] in used]
    out_ids = [ids[r] for r in fn.results]
    js = {"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "strict", "input_ports": in_ids, "output_ports": out_ids,
          "graph": graph}
    return json.dumps(js), [ids[a.name] for a in fn.args], out_ids


# ------------------------------------------------------------------------------------- printers
def _ty(shape, dtype: str) -> str:
    mlir = {"f32": "f32", "bf16": "bf16", "f16": "f16", "s8": "i8", "u8": "ui8", "s32": "i32"}[dtype]
    return "tensor<" + "".join(f"{d}x" for d in shape) + mlir + ">"


def mlp_module(batch: int, hidden: List[int], has_bias: List[bool], act: str, dtype: str, entry: str = "entry") -> str:
    """Text of the module benchgc's `--driver pattern --case mlp` builds (pattern/mlp.py:68-150)."""
    et = {"f32": "f32", "bf16": "bf16"}[dtype]
    layers = len(hidden) - 1
    sig = [f"%arg0: {_ty([batch, hidden[0]], dtype)}"]
    for i in range(layers):
        sig.append(f"%arg{i + 1}: {_ty([hidden[i], hidden[i + 1]], dtype)}")
    b_idx = layers + 1
    bias_arg = {}
    for i in range(layers):
        if has_bias[i]:
            bias_arg[i] = f"%arg{b_idx}"
            sig.append(f"%arg{b_idx}: {_ty([hidden[i + 1]], dtype)}")
            b_idx += 1
    out_t = _ty([batch, hidden[-1]], dtype)
    L = ["module {", f"  func.func @{entry}({', '.join(sig)}) -> {out_t} attributes {{llvm.emit_c_interface}} {{",
         f"    %cst = arith.constant 0.000000e+00 : {et}"]
    n = 0

    def new():
        nonlocal n
        n += 1
        return f"%{n - 1}"

    data, data_t = "%arg0", _ty([batch, hidden[0]], dtype)
    for i in range(layers):
        t = _ty([batch, hidden[i + 1]], dtype)
        wt = _ty([hidden[i], hidden[i + 1]], dtype)
        e = new()
        L.append(f"    {e} = tensor.empty() : {t}")
        f = new()
        L.append(f"    {f} = linalg.fill ins(%cst : {et}) outs({e} : {t}) -> {t}")
        mm = new()
        L.append(f"    {mm} = linalg.matmul ins({data}, %arg{i + 1} : {data_t}, {wt}) outs({f} : {t}) -> {t}")
        data, data_t = mm, t
        if has_bias[i]:
            e = new()
            L.append(f"    {e} = tensor.empty() : {t}")
            bc = f"%broadcasted_{i}"
            L.append(f"    {bc} = linalg.broadcast ins({bias_arg[i]} : {_ty([hidden[i + 1]], dtype)}) outs({e} : {t}) dimensions = [0]")
            e = new()
            L.append(f"    {e} = tensor.empty() : {t}")
            ad = new()
            L.append(f"    {ad} = linalg.add ins({data}, {bc} : {t}, {t}) outs({e} : {t}) -> {t}")
            data = ad
        if act == "relu":
            c = f"%cst_{i}"
            L.append(f"    {c} = arith.constant dense<0.000000e+00> : {t}")
            e = new()
            L.append(f"    {e} = tensor.empty() : {t}")
            mx = new()
            L.append(f"    {mx} = linalg.max ins({data}, {c} : {t}, {t}) outs({e} : {t}) -> {t}")
            data = mx
        elif act == "sigmoid":
            e = new()
            L.append(f"    {e} = tensor.empty() : {t}")
            sg = new()
            L.append(f"    {sg} = linalgx.sigmoid ins({data} : {t}) outs({e} : {t}) -> {t}")
            data = sg
    L += [f"    return {data} : {out_t}", "  }", "}"]
    return "\n".join(L) + "\n"


def matmul_module(case: str, a: TensorType, b: TensorType, c: TensorType, entry: str = "entry") -> str:
    """Text of the single-op module benchgc's `--driver linalg --case matmul*` builds
    (test/benchgc/src/benchgc/linalg/matmul.py, mlir/module.py)."""
    if "linalg." + case not in _MATMUL:
        raise Unimplemented(f"linalg case {case}")
    ta, tb, tc = _ty(a.shape, a.dtype), _ty(b.shape, b.dtype), _ty(c.shape, c.dtype)
    et = {"f32": "f32", "bf16": "bf16", "f16": "f16"}[c.dtype]
    return "\n".join([
        "module {",
        f"  func.func @{entry}(%arg0: {ta}, %arg1: {tb}) -> {tc} attributes {{llvm.emit_c_interface}} {{",
        f"    %cst = arith.constant 0.000000e+00 : {et}",
        f"    %0 = tensor.empty() : {tc}",
        f"    %1 = linalg.fill ins(%cst : {et}) outs(%0 : {tc}) -> {tc}",
        f"    %2 = linalg.{case} {{cast = #linalg.type_fn<cast_signed>}} ins(%arg0, %arg1 : {ta}, {tb}) outs(%1 : {tc}) -> {tc}",
        f"    return %2 : {tc}", "  }", "}"]) + "\n"
