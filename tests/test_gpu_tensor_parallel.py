"""Tensor-parallel MLP on real GPUs (needs >= 2 devices; skipped otherwise): the two fused
GEMM-epilogue peer-store exchanges (all-to-all and reduce-scatter + all-gather) and the NCCL
all-reduce baseline against the oracle's single-device chain.  Ranks are child processes, one per GPU; NVLS is switched off and the
kernels use plain peer stores, so a rank that fails cannot fault its peers' GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle
from _util import assert_bf16_close

pytestmark = pytest.mark.gpu

HIDDEN = (512, 2048, 512, 2048, 256)
BATCH = 256


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _make():
    g = torch.Generator().manual_seed(0)
    X = torch.randn(BATCH, HIDDEN[0], generator=g).bfloat16()
    Ws = [(torch.randn(HIDDEN[i], HIDDEN[i + 1], generator=g) * 0.05).bfloat16() for i in range(4)]
    Bs = [(torch.randn(HIDDEN[i + 1], generator=g) * 0.1).bfloat16() for i in range(4)]
    return X, Ws, Bs


def _worker(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from gc_b200 import lib
    from gc_b200.tensor_parallel import (AllReduceExchange, CudaOps, PeerPushExchange, PeerReduceScatterExchange,
                                         TensorParallelMLP, shard_weights)

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        X, Ws, Bs = _make()
        ws, bs = shard_weights([w.to(dev) for w in Ws], [b.to(dev) for b in Bs], world, rank)
        fused = {"peer_push": PeerPushExchange, "peer_reduce_scatter": PeerReduceScatterExchange}.get(mode)
        ex = fused(BATCH, HIDDEN[2], dev) if fused else AllReduceExchange(CudaOps())
        # the two row-parallel layers have different widths: one exchange object per width
        ex2 = fused(BATCH, HIDDEN[4], dev) if fused else ex
        tp1 = TensorParallelMLP(ws[:2], bs[:2], relu=True, exchange=ex)
        tp2 = TensorParallelMLP(ws[2:], bs[2:], relu=True, exchange=ex2)
        outs = []
        for _ in range(3):                     # repeated steps exercise the alternating receive buffers
            y = tp2.step(tp1.step(X.to(dev)))
            torch.cuda.synchronize()
            outs.append(_bits(y).copy())          # copied out at once: the exchange's result buffers alternate
        assert lib.device_error() == 0
        q.put((rank, outs))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode", ["all_reduce", "peer_push", "peer_reduce_scatter"])
def test_tensor_parallel_mlp_on_gpus(mode):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    if world == 3:
        world = 2
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    X, Ws, Bs = _make()
    want = oracle.mlp_bf16(_bits(X), [_bits(w) for w in Ws], [_bits(b) for b in Bs], relu=True)
    for r in range(world):
        for step in range(3):
            assert np.array_equal(res[r][step], res[0][0]), (r, step)   # every rank, every step: identical bits
    # last layer: bf16(bf16(acc) + bias) rounds twice; |acc| <= |result| + |bias| bounds the pre-bias value
    from _util import bf16_f32
    pre = np.abs(bf16_f32(want)) + np.abs(bf16_f32(_bits(Bs[3])))[None, :]
    mx, same = assert_bf16_close(res[0][0], want, max(HIDDEN), what=f"tp {mode}", floor_div=1.0, pre=pre)
    print(f"tp{world} {mode}: max_abs={mx:.4g} bit-identical={same:.5f}")
