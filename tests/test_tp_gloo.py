"""Host logic of the tensor-parallel MLP under gloo, world_size 2 and 4, on CPU.

The compute calls are replaced by the CPU oracle (test infrastructure), so what is tested is the
sharding, the order of collective and epilogue, and the numerics rule "f32 partial sums, reduce,
then cast / bias / ReLU": the result must equal the oracle's single-device chain within the
partial-sum reordering (bit-identical where sums are exact)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from gc_b200.tensor_parallel import TensorParallelMLP, shard_range, shard_weights


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _from_bits(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


class OracleOps:
    def linear(self, x, w, b, relu):
        return _from_bits(oracle.linear_bf16(_bits(x), _bits(w), None if b is None else _bits(b), relu=relu))

    def linear_partial(self, x, w):
        _, acc = oracle.linear_bf16(_bits(x), _bits(w), return_acc=True)
        return torch.from_numpy(acc)

    def epilogue(self, planes, b, relu):
        return _from_bits(oracle.reduce_epilogue_bf16(planes.numpy(), None if b is None else _bits(b), relu=relu))


def _make(exact: bool):
    g = torch.Generator().manual_seed(0)
    hidden = (64, 256, 96, 128, 32)
    if exact:   # small integers: every partial sum is exact, so any reduction order gives the same bits
        X = torch.randint(-2, 3, (24, hidden[0]), generator=g).bfloat16()
        Ws = [torch.randint(-1, 2, (hidden[i], hidden[i + 1]), generator=g).bfloat16() for i in range(4)]
        Bs = [torch.randint(-2, 3, (hidden[i + 1],), generator=g).bfloat16() for i in range(4)]
    else:
        X = torch.randn(24, hidden[0], generator=g).bfloat16()
        Ws = [(torch.randn(hidden[i], hidden[i + 1], generator=g) * 0.1).bfloat16() for i in range(4)]
        Bs = [(torch.randn(hidden[i + 1], generator=g) * 0.1).bfloat16() for i in range(4)]
    return X, Ws, Bs


def _worker(rank, world, port, exact, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        X, Ws, Bs = _make(exact)
        ws, bs = shard_weights(Ws, Bs, world, rank)
        tp = TensorParallelMLP(ws, bs, relu=True, ops=OracleOps())
        y = tp.step(X)
        q.put((rank, _bits(y).copy()))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("exact", [True, False])
def test_tensor_parallel_mlp_matches_single_device_chain(world, exact):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, exact, q)) for r in range(world)]
    for p in procs:
        p.start()
    outs = dict(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    X, Ws, Bs = _make(exact)
    want = oracle.mlp_bf16(_bits(X), [_bits(w) for w in Ws], [_bits(b) for b in Bs], relu=True)
    for r in range(world):
        assert np.array_equal(outs[r], outs[0])          # every rank holds the full result
    if exact:
        assert np.array_equal(outs[0], want)
    else:
        g = (outs[0].astype(np.uint32) << 16).view(np.float32)
        w = (want.astype(np.uint32) << 16).view(np.float32)
        assert np.all(np.abs(g - w) <= 2e-2 * np.maximum(np.abs(w), np.sqrt(np.mean(w ** 2))))
        assert (outs[0] == want).mean() > 0.9


def test_shard_helpers():
    assert shard_range(16384, 8, 3) == (6144, 8192)
    with pytest.raises(ValueError):
        shard_range(10, 4, 0)
    W = [torch.zeros(8, 12), torch.zeros(12, 8)]
    ws, bs = shard_weights(W, [torch.zeros(12), torch.zeros(8)], 4, 1)
    assert ws[0].shape == (8, 3) and ws[1].shape == (3, 8) and bs[0].shape == (3,) and bs[1].shape == (8,)
    with pytest.raises(ValueError):
        TensorParallelMLP([W[0]], [None])


# ------------------------------------------------------------------------------ the other sharded paths
class _HostOps:
    """CPU stand-ins for the kernels (exact integer-valued data, so results are bit-comparable)."""

    def linear(self, x, w, b, relu):
        return (x.float() @ w.float()).bfloat16()

    def quant_linear(self, A, W, scale, bias, zp):
        acc = A.to(torch.int32) @ W.to(torch.int32)
        comp = zp * W.to(torch.int32).sum(0)
        return (acc - comp).float() * scale + bias

    def attention(self, q, k, v, scale, causal):
        s = (q.float() @ k.float().transpose(-1, -2)) * scale
        if causal:
            S = s.shape[-1]
            s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        return (torch.softmax(s, -1) @ v.float()).bfloat16()


def _worker_sharded(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gc_b200.tensor_parallel import ShardedAttention, ShardedGemm, ShardedQuantGemm

        g = torch.Generator().manual_seed(1)
        A = torch.randint(-3, 4, (16, 64), generator=g).bfloat16()
        B = torch.randint(-2, 3, (64, 96), generator=g).bfloat16()
        lo, hi = shard_range(96, world, rank)
        c = ShardedGemm(B[:, lo:hi].contiguous(), world, rank, ops=_HostOps()).step(A)
        Aq = torch.randint(0, 256, (8, 32), generator=g, dtype=torch.uint8)
        Wq = torch.randint(-127, 128, (32, 48), generator=g, dtype=torch.int8)
        sc, bi = torch.rand(48, generator=g), torch.randn(48, generator=g)
        lo, hi = shard_range(48, world, rank)
        cq = ShardedQuantGemm(Wq[:, lo:hi].contiguous(), sc[lo:hi], bi[lo:hi], 128, world, rank, ops=_HostOps()).step(Aq)
        Q, K, V = (torch.randn(2, 4, 16, 8, generator=g).bfloat16() for _ in range(3))
        o = ShardedAttention(world, rank, ops=_HostOps()).step(Q, K, V, 8 ** -0.5, True, gather=True)
        q.put((rank, c.float().numpy(), cq.numpy(), o.float().numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_sharded_gemms_and_head_sharded_attention(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker_sharded, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict((r, rest) for r, *rest in (q.get(timeout=120) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    g = torch.Generator().manual_seed(1)
    A = torch.randint(-3, 4, (16, 64), generator=g).bfloat16()
    B = torch.randint(-2, 3, (64, 96), generator=g).bfloat16()
    Aq = torch.randint(0, 256, (8, 32), generator=g, dtype=torch.uint8)
    Wq = torch.randint(-127, 128, (32, 48), generator=g, dtype=torch.int8)
    sc, bi = torch.rand(48, generator=g), torch.randn(48, generator=g)
    Q, K, V = (torch.randn(2, 4, 16, 8, generator=g).bfloat16() for _ in range(3))
    ops = _HostOps()
    want = (ops.linear(A, B, None, False).float().numpy(), ops.quant_linear(Aq, Wq, sc, bi, 128).numpy(),
            ops.attention(Q.reshape(8, 1, 16, 8), K.reshape(8, 1, 16, 8), V.reshape(8, 1, 16, 8), 8 ** -0.5, True).reshape(2, 4, 16, 8).float().numpy())
    for r in range(world):
        for got, w in zip(res[r], want):
            assert np.array_equal(got, w), r      # every rank holds the full result, identical to one device


def test_fused_plan_counters_agree_across_ranks():
    """The tensor-parallel plan behind the C ABI (gcb200_tp_mlp_create / _describe; host only): what every owner's
    reduction waits for per step equals what all ranks' row-parallel GEMMs add to its counter, what the next layer
    waits for equals what all owners' reductions add, for 2, 4 and 8 ranks of BASELINE configs[2]; bad shapes are
    refused with a clear message."""
    import re

    from gc_b200 import lib

    hidden = [4096, 16384, 4096, 16384, 4096]
    for world in (2, 4, 8):
        fake = lambda base: [base + 0x100000 * i for i in range(world)]
        texts = []
        for rank in range(world):
            plan = lib.TpMlpPlan(world, rank, 512, hidden, [0x1000, 0x2000, 0x3000, 0x4000], [0x5000, 0x5100, 0x5200, 0x5300], True,
                                 [fake(0x10000000), fake(0x20000000)], [fake(0x30000000), fake(0x40000000)], fake(0x50000000), fake(0x60000000))
            texts.append(plan.describe(148))
            plan.destroy()
        for x in range(2):
            adds = [int(re.search(rf"part_landed\[{x}\] \+= (\d+) per rank", t).group(1)) for t in texts]
            waits = [int(re.search(rf"waits part_landed\[{x}\] \+= (\d+) per step", t).group(1)) for t in texts]
            assert len(set(adds)) == 1 and all(w == sum(adds) for w in waits)
            ctas = [int(re.search(rf"reduce {x}: .*?, (\d+) CTAs", t).group(1)) for t in texts]
            assert len(set(ctas)) == 1
            if x == 0:
                nxt = [int(re.search(r"waits rows_landed\[0\] \+= (\d+) per step", t).group(1)) for t in texts]
                assert all(n == sum(ctas) for n in nxt)
        rows = [re.search(r"rows (\d+)\.\.(\d+)", t).groups() for t in texts]
        assert [int(a) for a, _ in rows] == [r * 512 // world for r in range(world)]          # every row has exactly one owner
    with pytest.raises(lib.GcB200Error) as ei:
        lib.TpMlpPlan(8, 0, 384, hidden, [1] * 4, [0] * 4, True, [[16] * 8, [16] * 8], [[16] * 8, [16] * 8], [16] * 8)
    assert "multiple of 128" in str(ei.value)
    with pytest.raises(lib.GcB200Error):
        lib.TpMlpPlan(3, 0, 384, [4096, 16384, 4096], [1] * 2, [0] * 2, True, [[16] * 3, [16] * 3], [[16] * 3, [16] * 3], [16] * 3)   # 4096 % 24
    # time stamps exist only for a plan that has taken a step with GC_B200_TP_TRACE=1: asking earlier is an argument error
    # (answered on the host, no device needed)
    plan = lib.TpMlpPlan(2, 0, 512, hidden, [0x1000] * 4, [0] * 4, True, [[16] * 2, [16] * 2], [[16] * 2, [16] * 2], [16] * 2)
    with pytest.raises(lib.GcB200Error) as ei:
        plan.trace()
    assert "GC_B200_TP_TRACE" in str(ei.value)

