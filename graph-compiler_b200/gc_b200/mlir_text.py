"""Structural reader for the linalg-on-tensor MLIR that benchgc produces for the matmul / MLP path.

benchgc hands the reference one `func.func` whose body is a straight line of
`tensor.empty`, `arith.constant`, `linalg.fill`, `linalg.matmul[_transpose_a|_transpose_b]`,
`linalg.broadcast`, `linalg.add|sub|mul|div`, `linalg.max` (against a zero splat: ReLU),
`linalgx.sigmoid` and `return` (test/benchgc/src/benchgc/pattern/mlp.py:68-150,
test/benchgc/src/benchgc/linalg/matmul.py); the reference's llama2 decoder case
(test/benchgc/cases/llama2.mlir) adds `tensor.collapse_shape` / `tensor.expand_shape`,
`linalg.copy` (a cast), `linalg.powf` by a splat, `linalg.reduce` with an add body,
`linalg.negf`, `linalg.exp` and splat constants as operands; attention arrives as
`linalg.batch_matmul_transpose_b` -> `linalg.mul` by a splat -> `linalg.softmax` ->
`linalg.batch_matmul`, which is recognised as one fused partition.  No MLIR library is needed to read
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
_INT_DTYPES = ("s8", "u8", "s32")


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
_UNARY = {"linalgx.sigmoid": "sigmoid", "linalg.negf": "neg", "linalg.exp": "exp", "linalg.copy": "cast"}
_BATCH_MATMUL = {"linalg.batch_matmul": (False, False), "linalg.batch_matmul_transpose_a": (True, False),
                 "linalg.batch_matmul_transpose_b": (False, True)}
_MATMUL = {"linalg.matmul": (False, False), "linalg.matmul_transpose_a": (True, False), "linalg.matmul_transpose_b": (False, True)}


def parse_module(text: str, entry: str = "entry") -> Func:
    """Parse the entry function of a module printed by MLIR's generic-free (pretty) printer."""
    lines = [ln.rstrip() for ln in text.splitlines()]
    fn = None
    body: List[str] = []
    depth_in = False
    nest = 0   # regions opened inside the function body (linalg.reduce carries one)
    for ln in lines:
        s = ln.strip()
        if not depth_in:
            m = _FUNC_RE.search(s)
            if m and m.group(1) == entry:
                fn = m
                depth_in = True
            continue
        if s == "}" and nest == 0:
            break
        if s.endswith("{"):
            nest += 1
        elif s.startswith("}"):
            nest -= 1
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
    pos = 0
    while pos < len(body):
        s = body[pos]
        pos += 1
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
        elif opname in _UNARY:
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            get(ins[0])
            if it[0].shape != ot[0].shape:
                raise ParseError(f"{opname}: operand shape differs from the result shape")
            ops.append(Op(_UNARY[opname], ins, res))
            values[res] = Value(res, ot[0], "op")
        elif opname in ("tensor.collapse_shape", "tensor.expand_shape"):
            m2 = re.match(r"tensor\.\w+\s+(%[\w#.]+)\s*\[(.*?)\]\s*(?:output_shape\s*\[[^\]]*\]\s*)?:\s*(tensor<.*?>)\s+into\s+(tensor<.*?>)\s*$", rhs)
            if not m2:
                raise ParseError(f"malformed reshape: {rhs!r}")
            src, t_in, t_out = m2.group(1), parse_type(m2.group(3)), parse_type(m2.group(4))
            if get(src).type.shape != t_in.shape:
                raise ParseError(f"type of {src} does not match its definition")
            n_in = n_out = 1
            for d in t_in.shape:
                n_in *= d
            for d in t_out.shape:
                n_out *= d
            if n_in != n_out or t_in.dtype != t_out.dtype:
                raise ParseError(f"{opname} changes the element count or type: {rhs!r}")
            ops.append(Op("reshape", [src], res))
            values[res] = Value(res, t_out, "op")
        elif opname == "linalg.powf":
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            e = get(ins[1])
            if e.kind != "const":
                raise Unimplemented("linalg.powf whose exponent is not a splat constant")
            get(ins[0])
            ops.append(Op("pow", [ins[0]], res, {"beta": e.const}))
            values[res] = Value(res, ot[0], "op")
        elif opname == "linalg.reduce":
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            d = re.search(r"dimensions\s*=\s*\[([\d,\s]*)\]", rhs)
            if not d:
                raise ParseError("linalg.reduce without dimensions")
            axes = [int(x) for x in d.group(1).split(",") if x.strip()]
            # the combiner region follows on its own lines: only a sum (arith.addf of the two block arguments) is taken
            region = []
            while pos < len(body):
                ln2 = body[pos]
                pos += 1
                region.append(ln2)
                if ln2.startswith("}"):
                    break
            if not any("arith.addf" in r for r in region) or sum("arith." in r for r in region) != 1:
                raise Unimplemented("linalg.reduce with a combiner other than addition")
            init = get(outs[0])
            if init.kind != "zero_fill":
                raise Unimplemented("linalg.reduce whose init operand is not a zero fill")
            kept = tuple(x for i, x in enumerate(it[0].shape) if i not in axes)
            if kept != ot[0].shape:
                raise ParseError(f"reduce of {it[0].shape} over {axes} does not give {ot[0].shape}")
            get(ins[0])
            ops.append(Op("reduce_sum", [ins[0]], res, {"axes": axes}))
            values[res] = Value(res, ot[0], "op")
        elif opname == "linalg.softmax":
            d = re.search(r"dimension\((\d+)\)", rhs)
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            if not d:
                raise ParseError("linalg.softmax without dimension")
            get(ins[0])
            ops.append(Op("softmax", ins, res, {"dimension": int(d.group(1))}))
            values[res] = Value(res, ot[0], "op")
        elif opname == "linalg.quantized_matmul":
            # C[m,n] (+)= sum_k (A[m,k] - a_zp) * (B[k,n] - b_zp) in i32; here A is ui8 (u8 activations with their zero
            # point), B is i8 with a zero zero-point (symmetric weights): BASELINE's int8 configuration
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            if len(ins) != 4:
                raise ParseError("linalg.quantized_matmul takes A, B and the two zero points")
            for n in ins:
                get(n)
            azp, bzp = get(ins[2]), get(ins[3])
            if azp.kind != "const" or bzp.kind != "const":
                raise Unimplemented("quantized_matmul with zero points that are not constants")
            if int(bzp.const) != 0 or it[0].dtype != "u8" or it[1].dtype != "s8" or ot[0].dtype != "s32":
                raise Unimplemented("quantized_matmul is taken as ui8 x i8 -> i32 with a zero weight zero-point")
            if get(outs[0]).kind != "zero_fill":
                raise Unimplemented("linalg.quantized_matmul whose init operand is not a zero fill")
            a, b = it[0], it[1]
            if a.rank != 2 or b.rank != 2 or a.shape[1] != b.shape[0] or ot[0].shape != (a.shape[0], b.shape[1]):
                raise ParseError(f"quantized_matmul shapes do not agree: {a.shape} x {b.shape} -> {ot[0].shape}")
            ops.append(Op("qmatmul", ins[:2], res, {"src_zp": int(azp.const)}))
            values[res] = Value(res, ot[0], "op")
        elif opname in _BATCH_MATMUL:
            ins, it = _operands(_clause(rhs, "ins"))
            outs, ot = _operands(_clause(rhs, "outs"))
            for n in ins:
                get(n)
            if get(outs[0]).kind != "zero_fill":
                raise Unimplemented("linalg.batch_matmul whose init operand is not a zero fill")
            ta, tb = _BATCH_MATMUL[opname]
            a, b = it
            if a.rank != 3 or b.rank != 3 or a.shape[0] != b.shape[0]:
                raise ParseError("batch_matmul operands must be rank 3 with one batch size")
            m_, k_ = (a.shape[2], a.shape[1]) if ta else a.shape[1:]
            k2, n_ = (b.shape[2], b.shape[1]) if tb else b.shape[1:]
            if k_ != k2 or ot[0].shape != (a.shape[0], m_, n_):
                raise ParseError(f"batch_matmul shapes do not agree: {a.shape} x {b.shape} -> {ot[0].shape}")
            ops.append(Op("batch_matmul", ins, res, {"transpose_a": ta, "transpose_b": tb}))
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
_KIND = {"add": "Add", "sub": "Subtract", "mul": "Multiply", "div": "Divide", "relu": "ReLU", "sigmoid": "Sigmoid",
         "neg": "Negate", "exp": "Exp", "cast": "Typecast", "reshape": "StaticReshape", "pow": "Pow", "reduce_sum": "ReduceSum"}


def _fuse_attention(fn: Func, ops: List[Op]) -> List[Op]:
    """batch_matmul_transpose_b(Q, K) [-> mul by a splat scale] -> softmax over the last dimension -> batch_matmul(., V),
    every intermediate used once: one fused attention op (softmax as DecomposeAggregatedOps.cpp:24-38 defines it)."""
    uses: Dict[str, int] = {}
    for op in ops:
        for n in op.ins:
            uses[n] = uses.get(n, 0) + 1
    for r in fn.results:
        uses[r] = uses.get(r, 0) + 1
    by_out = {op.out: op for op in ops}
    out: List[Op] = []
    dead = set()
    for op in ops:
        if op.name != "batch_matmul" or op.attrs["transpose_a"] or op.attrs["transpose_b"]:
            continue
        sm = by_out.get(op.ins[0])
        if not sm or sm.name != "softmax" or uses.get(sm.out, 0) != 1:
            continue
        if sm.attrs["dimension"] != fn.values[sm.out].type.rank - 1:
            continue
        scale, cur = 1.0, by_out.get(sm.ins[0])
        if cur and cur.name == "mul" and uses.get(cur.out, 0) == 1:
            consts = [n for n in cur.ins if fn.values[n].kind == "const"]
            if len(consts) == 1:
                scale = float(fn.values[consts[0]].const)
                other = cur.ins[1] if cur.ins[0] == consts[0] else cur.ins[0]
                dead.add(cur.out)
                cur = by_out.get(other)
        if not cur or cur.name != "batch_matmul" or cur.attrs["transpose_a"] or not cur.attrs["transpose_b"] or uses.get(cur.out, 0) != 1:
            dead.discard(by_out[sm.ins[0]].out if sm.ins[0] in by_out else "")
            continue
        q, k, v = cur.ins[0], cur.ins[1], op.ins[1]
        if not (fn.values[q].type.shape == fn.values[k].type.shape == fn.values[v].type.shape):
            raise Unimplemented("attention with different Q, K and V shapes")
        dead.update({cur.out, sm.out})
        op.name, op.ins, op.attrs = "sdpa", [q, k, v], {"scale": scale}
    for op in ops:
        if op.out not in dead:
            out.append(op)
    for op in out:
        if op.name in ("softmax", "batch_matmul"):
            raise Unimplemented(f"{op.name} outside the fused attention pattern")
    return out


def _fuse_dequant(fn: Func, ops: List[Op]) -> List[Op]:
    """qmatmul -> copy to f32 -> mul by a broadcast [N] scale argument [-> add a broadcast [N] bias argument], each
    intermediate used once: one QuantizedMatMul with per-channel dequantisation (the epilogue of the int8 kernel)."""
    uses: Dict[str, int] = {}
    for op in ops:
        for n in op.ins:
            uses[n] = uses.get(n, 0) + 1
    for r in fn.results:
        uses[r] = uses.get(r, 0) + 1
    consumer = {}
    for op in ops:
        for n in op.ins:
            consumer.setdefault(n, op)

    def channel_vector(name: str, n: int) -> Optional[str]:
        v = fn.values[name]
        if v.kind == "bcast" and fn.values[v.src].kind == "arg" and fn.values[v.src].type.shape == (n,) and v.bdims == (0,):
            return v.src
        return None

    dead = set()
    for op in ops:
        if op.name != "qmatmul" or uses.get(op.out, 0) != 1:
            continue
        n = fn.values[op.out].type.shape[1]
        cast = consumer.get(op.out)
        if not cast or cast.name != "cast" or fn.values[cast.out].type.dtype != "f32" or uses.get(cast.out, 0) != 1:
            continue
        mul = consumer.get(cast.out)
        if not mul or mul.name != "mul":
            continue
        other = mul.ins[1] if mul.ins[0] == cast.out else mul.ins[0]
        scale = channel_vector(other, n)
        if scale is None:
            continue
        final, bias = mul, None
        add = consumer.get(mul.out) if uses.get(mul.out, 0) == 1 else None
        if add and add.name == "add":
            o2 = add.ins[1] if add.ins[0] == mul.out else add.ins[0]
            b = channel_vector(o2, n)
            if b is not None:
                final, bias = add, b
                dead.add(mul.out)
        dead.update({op.out, cast.out})
        final.name, final.ins, final.attrs = "qmatmul_dequant", op.ins + [scale] + ([bias] if bias else []), dict(op.attrs)
    return [op for op in ops if op.out not in dead]


def to_partition(fn: Func):
    """The oneDNN-graph JSON of `fn`.  Returns (json text, input tensor ids in argument order, output ids, constants),
    where ``constants`` maps the id of every extra one-element input to its (value, dtype): splat constants that the
    module uses as operands become partition inputs that the caller fills.

    A broadcast becomes numpy auto-broadcast of its source, reshaped first when the new dimensions are not the
    leading ones (lib/gc/Transforms/OneDNNGraphToLinalg.cpp:484-494 goes the other way).
    """
    ids: Dict[str, int] = {a.name: i for i, a in enumerate(fn.args)}
    nxt = len(fn.args)
    consts: Dict[int, Tuple[float, str]] = {}
    const_ids: Dict[Tuple[float, str], int] = {}
    graph: List[dict] = []
    reshaped: Dict[Tuple[str, Tuple[int, ...]], dict] = {}

    def fresh() -> int:
        nonlocal nxt
        nxt += 1
        return nxt - 1

    def node(kind: str, ins: List[dict], outs: List[dict], attrs: Optional[dict] = None):
        graph.append({"id": len(graph), "name": f"{kind.lower()}_{len(graph)}", "kind": kind, "attrs": attrs or {}, "inputs": ins,
                      "outputs": outs})

    def tensor(name: str) -> dict:
        v = fn.values[name]
        if v.kind == "bcast":
            src = tensor(v.src)
            lead = tuple(range(len(v.bdims)))
            if v.bdims == lead:
                return src
            # new dimensions in the middle or at the end: give the source size-1 dimensions there, then auto-broadcast
            shape = tuple(1 if i in v.bdims else d for i, d in enumerate(v.type.shape))
            key = (v.src, shape)
            if key not in reshaped:
                out = {"id": fresh(), "dtype": src["dtype"], "shape": list(shape)}
                node("StaticReshape", [src], [out])
                reshaped[key] = out
            return reshaped[key]
        if v.kind == "const" or v.kind == "zero_fill":
            key = (float(v.const or 0.0), v.type.dtype)
            if key not in const_ids:
                const_ids[key] = fresh()
                consts[const_ids[key]] = key
            return {"id": const_ids[key], "dtype": v.type.dtype, "shape": [1], "property_type": "constant"}
        if v.kind == "empty":
            raise Unimplemented(f"{name}: an uninitialised tensor as an operand")
        if name not in ids:
            raise ParseError(f"{name} is used before it is produced")
        return {"id": ids[name], "dtype": v.type.dtype, "shape": list(v.type.shape)}

    # the fusion passes rewrite ops: work on copies, the parsed function stays as the text said
    work = [Op(o.name, list(o.ins), o.out, dict(o.attrs)) for o in fn.ops]
    for op in _fuse_dequant(fn, _fuse_attention(fn, work)):
        ins = [tensor(n) for n in op.ins]
        ids[op.out] = fresh()
        out = tensor(op.out)
        if op.name == "matmul":
            attrs = {a: {"type": "bool", "value": 1} for a in ("transpose_a", "transpose_b") if op.attrs[a]}
            node("MatMul", ins, [out], attrs)
        elif op.name in ("qmatmul", "qmatmul_dequant"):
            node("QuantizedMatMul", ins, [out], {"src_zp": {"type": "s64", "value": int(op.attrs["src_zp"])}})
        elif op.name == "sdpa":
            node("SDPA", ins, [out], {"scale": {"type": "f32", "value": op.attrs["scale"]}, "causal": {"type": "bool", "value": 0}})
        elif op.name in ("add", "sub", "mul", "div"):
            node(_KIND[op.name], ins, [out], {"auto_broadcast": {"type": "string", "value": "numpy"}})
        elif op.name == "pow":
            node("Pow", ins, [out], {"beta": {"type": "f32", "value": float(op.attrs["beta"])}})
        elif op.name == "reduce_sum":
            node("ReduceSum", ins, [out], {"axes": {"type": "s64[]", "value": list(op.attrs["axes"])}, "keep_dims": {"type": "bool", "value": 0}})
        elif op.name in _KIND:
            node(_KIND[op.name], ins, [out])
        else:
            raise Unimplemented(op.name)
    used = {t["id"] for n in graph for t in n["inputs"]}
    in_ids = [ids[a.name] for a in fn.args if ids[a.name] in used] + [c for c in consts if c in used]
    out_ids = [ids[r] for r in fn.results]
    js = {"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "strict", "input_ports": in_ids, "output_ports": out_ids,
          "graph": graph}
    return json.dumps(js), [ids[a.name] for a in fn.args], out_ids, consts


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


def llama2_mlp_module(batch: int = 1, seq: int = 32, hidden: int = 4096, inter: int = 11008, entry: str = "entry") -> str:
    """Text of a llama2 decoder block's second half in linalg form, the module the reference keeps as its
    ``--driver mlir`` case (test/benchgc/cases/llama2.mlir): attention output projection + residual, RMSNorm,
    gate / up projections with SiLU spelled as negf, exp, add 1, div, the down projection + residual, RMSNorm.
    Arguments: x [B,S,H], w_o [H,H], residual [B,S,H], eps1 [1] f32 (unused), g1 [H], w_gate [I,H], w_up [I,H],
    w_down [H,I], eps2 [1] f32, g2 [H]; results: the normalised output and the second residual sum."""
    B, S, H, I, T = batch, seq, hidden, inter, batch * seq
    bf = lambda *d: _ty(d, "bf16")
    f = lambda *d: _ty(d, "f32")
    L: List[str] = []
    n = 0

    def emit(rhs: str, name: Optional[str] = None) -> str:
        nonlocal n
        if name is None:
            name = f"%{n}"
            n += 1
        L.append(f"    {name} = {rhs}")
        return name

    def empty(t: str) -> str:
        return emit(f"tensor.empty() : {t}")

    def zero(t: str, et: str) -> str:
        c = emit(f"arith.constant 0.000000e+00 : {et}", f"%z{len(L)}")
        return emit(f"linalg.fill ins({c} : {et}) outs({empty(t)} : {t}) -> {t}")

    def binary(op: str, a: str, b: str, t: str) -> str:
        return emit(f"linalg.{op} ins({a}, {b} : {t}, {t}) outs({empty(t)} : {t}) -> {t}")

    def splat(v: float, t: str) -> str:
        return emit(f"arith.constant dense<{v:e}> : {t}", f"%c{len(L)}")

    def proj(x2: str, w: str, rows: int, k: int, nn: int) -> str:
        return emit(f"linalg.matmul_transpose_b ins({x2}, {w} : {bf(rows, k)}, {bf(nn, k)}) outs({zero(bf(rows, nn), 'bf16')} : "
                    f"{bf(rows, nn)}) -> {bf(rows, nn)}")

    def rmsnorm(x: str, eps: str, gamma: str) -> str:
        xf = emit(f"linalg.copy ins({x} : {bf(B, S, H)}) outs({empty(f(B, S, H))} : {f(B, S, H)}) -> {f(B, S, H)}")
        sq = emit(f"linalg.powf ins({xf}, {splat(2.0, f(B, S, H))} : {f(B, S, H)}, {f(B, S, H)}) outs({empty(f(B, S, H))} : {f(B, S, H)}) -> {f(B, S, H)}")
        init = zero(f(B, S), "f32")
        red = emit(f"linalg.reduce ins({sq} : {f(B, S, H)}) outs({init} : {f(B, S)}) dimensions = [2]", f"%reduced{len(L)}")
        L.extend(["      (%in: f32, %init: f32) {", "        %sum = arith.addf %in, %init : f32", "        linalg.yield %sum : f32", "      }"])
        mean = binary("div", red, splat(float(H), f(B, S)), f(B, S))
        m3 = emit(f"tensor.expand_shape {mean} [[0], [1, 2]] output_shape [{B}, {S}, 1] : {f(B, S)} into {f(B, S, 1)}", f"%expanded{len(L)}")
        eb = emit(f"linalg.broadcast ins({eps} : {f(1)}) outs({empty(f(B, S, 1))} : {f(B, S, 1)}) dimensions = [0, 1]", f"%broadcasted{len(L)}")
        ve = binary("add", m3, eb, f(B, S, 1))
        rs = emit(f"linalg.powf ins({ve}, {splat(-0.5, f(B, S, 1))} : {f(B, S, 1)}, {f(B, S, 1)}) outs({empty(f(B, S, 1))} : {f(B, S, 1)}) -> {f(B, S, 1)}")
        r2 = emit(f"tensor.collapse_shape {rs} [[0], [1, 2]] : {f(B, S, 1)} into {f(B, S)}", f"%collapsed{len(L)}")
        rb = emit(f"linalg.broadcast ins({r2} : {f(B, S)}) outs({empty(f(B, S, H))} : {f(B, S, H)}) dimensions = [2]", f"%broadcasted{len(L)}")
        y = binary("mul", xf, rb, f(B, S, H))
        yb = emit(f"linalg.copy ins({y} : {f(B, S, H)}) outs({empty(bf(B, S, H))} : {bf(B, S, H)}) -> {bf(B, S, H)}")
        gb = emit(f"linalg.broadcast ins({gamma} : {bf(H)}) outs({empty(bf(B, S, H))} : {bf(B, S, H)}) dimensions = [0, 1]", f"%broadcasted{len(L)}")
        return binary("mul", gb, yb, bf(B, S, H))

    sig = (f"%arg0: {bf(B, S, H)}, %arg1: {bf(H, H)}, %arg2: {bf(B, S, H)}, %arg3: {f(1)}, %arg4: {bf(H)}, %arg5: {bf(I, H)}, "
           f"%arg6: {bf(I, H)}, %arg7: {bf(H, I)}, %arg8: {f(1)}, %arg9: {bf(H)}")
    head = ["module {", f"  func.func @{entry}({sig}) -> ({bf(B, S, H)}, {bf(B, S, H)}) attributes {{llvm.emit_c_interface}} {{"]
    x2 = emit(f"tensor.collapse_shape %arg0 [[0, 1], [2]] : {bf(B, S, H)} into {bf(T, H)}", "%collapsed")
    o = proj(x2, "%arg1", T, H, H)
    o3 = emit(f"tensor.expand_shape {o} [[0, 1], [2]] output_shape [{B}, {S}, {H}] : {bf(T, H)} into {bf(B, S, H)}", "%expanded")
    r1 = binary("add", "%arg2", o3, bf(B, S, H))
    h = rmsnorm(r1, "%arg8", "%arg4")
    h2 = emit(f"tensor.collapse_shape {h} [[0, 1], [2]] : {bf(B, S, H)} into {bf(T, H)}", f"%collapsed{len(L)}")
    gate = proj(h2, "%arg5", T, H, I)
    g3 = emit(f"tensor.expand_shape {gate} [[0, 1], [2]] output_shape [{B}, {S}, {I}] : {bf(T, I)} into {bf(B, S, I)}", f"%expanded{len(L)}")
    one = splat(1.0, bf(B, S, I))
    ng = emit(f"linalg.negf ins({g3} : {bf(B, S, I)}) outs({empty(bf(B, S, I))} : {bf(B, S, I)}) -> {bf(B, S, I)}")
    ex = emit(f"linalg.exp ins({ng} : {bf(B, S, I)}) outs({empty(bf(B, S, I))} : {bf(B, S, I)}) -> {bf(B, S, I)}")
    den = binary("add", one, ex, bf(B, S, I))
    sg = binary("div", one, den, bf(B, S, I))
    silu = binary("mul", sg, g3, bf(B, S, I))
    h2b = emit(f"tensor.collapse_shape {h} [[0, 1], [2]] : {bf(B, S, H)} into {bf(T, H)}", f"%collapsed{len(L)}")
    up = proj(h2b, "%arg6", T, H, I)
    u3 = emit(f"tensor.expand_shape {up} [[0, 1], [2]] output_shape [{B}, {S}, {I}] : {bf(T, I)} into {bf(B, S, I)}", f"%expanded{len(L)}")
    act = binary("mul", silu, u3, bf(B, S, I))
    a2 = emit(f"tensor.collapse_shape {act} [[0, 1], [2]] : {bf(B, S, I)} into {bf(T, I)}", f"%collapsed{len(L)}")
    down = proj(a2, "%arg7", T, I, H)
    d3 = emit(f"tensor.expand_shape {down} [[0, 1], [2]] output_shape [{B}, {S}, {H}] : {bf(T, H)} into {bf(B, S, H)}", f"%expanded{len(L)}")
    r2 = binary("add", r1, d3, bf(B, S, H))
    out = rmsnorm(r2, "%arg8", "%arg9")
    return "\n".join(head + L + [f"    return {out}, {r2} : {bf(B, S, H)}, {bf(B, S, H)}", "  }", "}"]) + "\n"


def attention_module(batch_heads: int, seq: int, dim: int, scale: float, entry: str = "entry") -> str:
    """Attention spelled with the ops the reference's drivers emit one by one (linalg/matmul.py batch_matmul*,
    linalg/softmax.py): scores = Q K^T, scaled, softmax over the keys, times V."""
    t, ts = _ty((batch_heads, seq, dim), "bf16"), _ty((batch_heads, seq, seq), "bf16")
    return "\n".join([
        "module {",
        f"  func.func @{entry}(%arg0: {t}, %arg1: {t}, %arg2: {t}) -> {t} attributes {{llvm.emit_c_interface}} {{",
        "    %cst = arith.constant 0.000000e+00 : bf16",
        f"    %0 = tensor.empty() : {ts}",
        f"    %1 = linalg.fill ins(%cst : bf16) outs(%0 : {ts}) -> {ts}",
        f"    %2 = linalg.batch_matmul_transpose_b ins(%arg0, %arg1 : {t}, {t}) outs(%1 : {ts}) -> {ts}",
        f"    %cst_0 = arith.constant dense<{scale:e}> : {ts}",
        f"    %3 = tensor.empty() : {ts}",
        f"    %4 = linalg.mul ins(%2, %cst_0 : {ts}, {ts}) outs(%3 : {ts}) -> {ts}",
        f"    %5 = tensor.empty() : {ts}",
        f"    %6 = linalg.softmax dimension(2) ins(%4 : {ts}) outs(%5 : {ts}) -> {ts}",
        f"    %7 = tensor.empty() : {t}",
        f"    %8 = linalg.fill ins(%cst : bf16) outs(%7 : {t}) -> {t}",
        f"    %9 = linalg.batch_matmul ins(%6, %arg2 : {ts}, {t}) outs(%8 : {t}) -> {t}",
        f"    return %9 : {t}", "  }", "}"]) + "\n"


def quantized_matmul_module(M: int, N: int, K: int, src_zp: int = 128, dequant: bool = True, bias: bool = True, entry: str = "entry") -> str:
    """BASELINE's int8 configuration in linalg form: ui8 activations (zero point ``src_zp``) times i8 weights with
    linalg.quantized_matmul into i32, then (``dequant``) a cast to f32, per-output-channel scales and a bias."""
    ta, tb, tc, tf, tv = _ty((M, K), "u8"), _ty((K, N), "s8"), _ty((M, N), "s32"), _ty((M, N), "f32"), _ty((N,), "f32")
    sig = f"%arg0: {ta}, %arg1: {tb}" + (f", %arg2: {tv}" if dequant else "") + (f", %arg3: {tv}" if dequant and bias else "")
    L = ["module {", f"  func.func @{entry}({sig}) -> {tf if dequant else tc} attributes {{llvm.emit_c_interface}} {{",
         "    %c0_i32 = arith.constant 0 : i32", f"    %c{src_zp}_i32 = arith.constant {src_zp} : i32" if src_zp else "",
         f"    %0 = tensor.empty() : {tc}", f"    %1 = linalg.fill ins(%c0_i32 : i32) outs(%0 : {tc}) -> {tc}",
         f"    %2 = linalg.quantized_matmul ins(%arg0, %arg1, %c{src_zp}_i32, %c0_i32 : {ta}, {tb}, i32, i32) outs(%1 : {tc}) -> {tc}"]
    res = "%2"
    if dequant:
        L += [f"    %3 = tensor.empty() : {tf}", f"    %4 = linalg.copy ins(%2 : {tc}) outs(%3 : {tf}) -> {tf}",
              f"    %5 = tensor.empty() : {tf}", f"    %broadcasted = linalg.broadcast ins(%arg2 : {tv}) outs(%5 : {tf}) dimensions = [0]",
              f"    %6 = tensor.empty() : {tf}", f"    %7 = linalg.mul ins(%4, %broadcasted : {tf}, {tf}) outs(%6 : {tf}) -> {tf}"]
        res = "%7"
        if bias:
            L += [f"    %8 = tensor.empty() : {tf}", f"    %broadcasted_0 = linalg.broadcast ins(%arg3 : {tv}) outs(%8 : {tf}) dimensions = [0]",
                  f"    %9 = tensor.empty() : {tf}", f"    %10 = linalg.add ins(%7, %broadcasted_0 : {tf}, {tf}) outs(%9 : {tf}) -> {tf}"]
            res = "%10"
    L += [f"    return {res} : {tf if dequant else tc}", "  }", "}"]
    return "\n".join(x for x in L if x) + "\n"
