"""Builders for the oneDNN-graph JSON partitions this backend runs.

The envelope and tensor-object schema are the reference's
(test/dnnl/resources/*.json; reader src/dnnl/JsonParser.cpp:34-320).  ``mlp``
produces the graph benchgc's mlp pattern describes
(test/benchgc/src/benchgc/pattern/mlp.py:113-150): per layer MatMul(+bias) and an
optional ReLU, arguments ordered src, weights..., biases....  ``quantized_matmul``
and ``sdpa`` use the two extension kinds.
"""
from __future__ import annotations

import json
from typing import Sequence


def _t(tid, dtype, shape, constant=False):
    d = {"id": tid, "dtype": dtype, "shape": list(shape)}
    if constant:
        d["property_type"] = "constant"
    return d


def _envelope(graph, inputs, outputs):
    return json.dumps({"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "any", "input_ports": list(inputs),
                       "output_ports": list(outputs), "graph": graph})


def mlp(batch: int, hidden: Sequence[int], dtype: str = "bf16", has_bias: Sequence[bool] | None = None,
        act: str = "relu", constant_weights: bool = False, separate_add: bool = False):
    """Returns (json, input ids in benchgc argument order, output id).

    ids: src = 0, weight i = 1 + i, bias j = 1 + layers + j; intermediates follow.
    ``separate_add`` spells the bias as MatMul -> Add like the second layer of
    test/dnnl/resources/mpl.json.
    """
    layers = len(hidden) - 1
    has_bias = [True] * layers if has_bias is None else list(has_bias)
    w_ids = [1 + i for i in range(layers)]
    b_ids, nxt = [], 1 + layers
    for i in range(layers):
        b_ids.append(nxt if has_bias[i] else None)
        nxt += 1 if has_bias[i] else 0
    graph, cur, cur_shape = [], 0, [batch, hidden[0]]
    for i in range(layers):
        out_shape = [batch, hidden[i + 1]]
        ins = [_t(cur, dtype, cur_shape), _t(w_ids[i], dtype, [hidden[i], hidden[i + 1]], constant_weights)]
        if has_bias[i] and not separate_add:
            ins.append(_t(b_ids[i], dtype, [hidden[i + 1]], constant_weights))
        mm_out = nxt
        nxt += 1
        graph.append({"kind": "MatMul", "inputs": ins, "outputs": [_t(mm_out, dtype, out_shape)]})
        cur = mm_out
        if has_bias[i] and separate_add:
            graph.append({"kind": "Add", "inputs": [_t(cur, dtype, out_shape), _t(b_ids[i], dtype, [hidden[i + 1]], constant_weights)],
                          "outputs": [_t(nxt, dtype, out_shape)]})
            cur = nxt
            nxt += 1
        if act == "relu":
            graph.append({"kind": "ReLU", "inputs": [_t(cur, dtype, out_shape)], "outputs": [_t(nxt, dtype, out_shape)]})
            cur = nxt
            nxt += 1
        cur_shape = out_shape
    inputs = [0] + w_ids + [b for b in b_ids if b is not None]
    return _envelope(graph, inputs, [cur]), inputs, cur


def matmul(M: int, N: int, K: int, dtype: str = "bf16", transpose_a=False, transpose_b=False, bias=False, relu=False):
    """Single MatMul partition: ids A=0, B=1, bias=2; returns (json, inputs, output id)."""
    a_shape = [K, M] if transpose_a else [M, K]
    b_shape = [N, K] if transpose_b else [K, N]
    ins = [_t(0, dtype, a_shape), _t(1, dtype, b_shape)]
    if bias:
        ins.append(_t(2, dtype, [N]))
    op = {"kind": "MatMul", "attrs": {"transpose_a": {"type": "bool", "value": int(transpose_a)},
                                      "transpose_b": {"type": "bool", "value": int(transpose_b)}},
          "inputs": ins, "outputs": [_t(3, dtype, [M, N])]}
    graph, out = [op], 3
    if relu:
        graph.append({"kind": "ReLU", "inputs": [_t(3, dtype, [M, N])], "outputs": [_t(4, dtype, [M, N])]})
        out = 4
    return _envelope(graph, [0, 1] + ([2] if bias else []), [out]), [0, 1] + ([2] if bias else []), out


def quantized_matmul(M: int, N: int, K: int, src_zp: int = 128, bias: bool = True, want_acc: bool = False,
                     constant_weights: bool = False):
    """Extension kind: u8 [M,K] x s8 [K,N] -> f32 with per-channel scales; ids 0..3, out 4 (acc 5)."""
    ins = [_t(0, "u8", [M, K]), _t(1, "s8", [K, N], constant_weights), _t(2, "f32", [N], constant_weights)]
    if bias:
        ins.append(_t(3, "f32", [N], constant_weights))
    outs = [_t(4, "f32", [M, N])] + ([_t(5, "s32", [M, N])] if want_acc else [])
    op = {"kind": "QuantizedMatMul", "attrs": {"src_zp": {"type": "s64", "value": src_zp}}, "inputs": ins, "outputs": outs}
    inputs = [0, 1, 2] + ([3] if bias else [])
    return _envelope([op], inputs, [4] + ([5] if want_acc else [])), inputs, 4


def sdpa(batch: int, heads: int, seq: int, dim: int, scale: float, causal: bool):
    """Extension kind: fused attention on bf16 [B,H,S,D]; ids Q=0, K=1, V=2, O=3."""
    sh = [batch, heads, seq, dim]
    op = {"kind": "SDPA", "attrs": {"scale": {"type": "f32", "value": scale}, "causal": {"type": "bool", "value": int(causal)}},
          "inputs": [_t(0, "bf16", sh), _t(1, "bf16", sh), _t(2, "bf16", sh)], "outputs": [_t(3, "bf16", sh)]}
    return _envelope([op], [0, 1, 2], [3]), [0, 1, 2], 3


def llama2_mlp(batch: int = 1, seq: int = 32, hidden: int = 4096, inter: int = 11008, constant_weights: bool = False):
    """The llama2 decoder MLP block of the reference's tests
    (test/mlir/test/gc/Dialect/OneDNNGraph/onednn-graph-llama2.mlir:5-45; linalg form
    test/benchgc/cases/llama2.mlir): attention-output projection + residual, RMSNorm, SiLU-gated MLP with
    three transpose_b MatMuls, residual, second RMSNorm.  Only the reference's own op kinds are used.

    Returns (json, {name: id} of the ten arguments in the reference's order, [id of the normed output, id of the residual output]).
    Arguments: x [B,S,H], wo [H,H], resid [B,S,H], eps1 [1] f32 (unused by the graph, kept for the signature),
    g1 [H], w_gate [I,H], w_up [I,H], w_down [H,I], eps [1] f32, g2 [H]."""
    B, S, H, I = batch, seq, hidden, inter
    bf, f32 = "bf16", "f32"
    act, act32, row = [B, S, H], [B, S, H], [B, S, 1]
    ids = {"x": 0, "wo": 1, "resid": 2, "eps1": 3, "g1": 4, "w_gate": 5, "w_up": 6, "w_down": 7, "eps": 8, "g2": 9}
    nxt = [10]

    def new():
        nxt[0] += 1
        return nxt[0] - 1

    g = []
    cw = constant_weights

    def op(kind, ins, out, attrs=None):
        d = {"kind": kind, "inputs": ins, "outputs": [out]}
        if attrs:
            d["attrs"] = attrs
        g.append(d)
        return out["id"]

    tb = {"transpose_b": {"type": "bool", "value": 1}}
    t5 = op("MatMul", [_t(ids["x"], bf, act), _t(ids["wo"], bf, [H, H], cw)], _t(new(), bf, act), tb)
    t7 = op("Add", [_t(ids["resid"], bf, act), _t(t5, bf, act)], _t(new(), bf, act))

    def rmsnorm(src, gamma):
        c = op("Typecast", [_t(src, bf, act)], _t(new(), f32, act32))
        sq = op("Pow", [_t(c, f32, act32)], _t(new(), f32, act32), {"beta": {"type": "f32", "value": 2.0}})
        mean = op("ReduceMean", [_t(sq, f32, act32)], _t(new(), f32, row),
                  {"axes": {"type": "s64[]", "value": [-1]}, "keep_dims": {"type": "bool", "value": 1}})
        pe = op("Add", [_t(mean, f32, row), _t(ids["eps"], f32, [1])], _t(new(), f32, row))
        rs = op("Pow", [_t(pe, f32, row)], _t(new(), f32, row), {"beta": {"type": "f32", "value": -0.5}})
        sc = op("Multiply", [_t(c, f32, act32), _t(rs, f32, row)], _t(new(), f32, act32))
        back = op("Typecast", [_t(sc, f32, act32)], _t(new(), bf, act))
        return op("Multiply", [_t(gamma, bf, [H], cw), _t(back, bf, act)], _t(new(), bf, act))

    t27 = rmsnorm(t7, ids["g1"])
    wide = [B, S, I]
    t30 = op("MatMul", [_t(t27, bf, act), _t(ids["w_gate"], bf, [I, H], cw)], _t(new(), bf, wide), tb)
    t31 = op("Sigmoid", [_t(t30, bf, wide)], _t(new(), bf, wide))
    t32 = op("Multiply", [_t(t31, bf, wide), _t(t30, bf, wide)], _t(new(), bf, wide))
    t35 = op("MatMul", [_t(t27, bf, act), _t(ids["w_up"], bf, [I, H], cw)], _t(new(), bf, wide), tb)
    t36 = op("Multiply", [_t(t32, bf, wide), _t(t35, bf, wide)], _t(new(), bf, wide))
    t39 = op("MatMul", [_t(t36, bf, wide), _t(ids["w_down"], bf, [H, I], cw)], _t(new(), bf, act), tb)
    t41 = op("Add", [_t(t7, bf, act), _t(t39, bf, act)], _t(new(), bf, act))
    t61 = rmsnorm(t41, ids["g2"])
    used = [ids[k] for k in ("x", "wo", "resid", "g1", "w_gate", "w_up", "w_down", "eps", "g2")]
    return _envelope(g, used, [t61, t41]), ids, [t61, t41]
