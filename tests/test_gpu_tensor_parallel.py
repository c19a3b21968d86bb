"""Multi-GPU paths on real GPUs (need >= 2 devices; skipped otherwise).  The tensor-parallel MLP with its exchanges
fused into the GEMM epilogue (peer stores to every rank, reduce-scatter + all-gather, one multimem store per chunk through
the NVSwitch multicast mapping) and with the NCCL all-reduce baseline, against the oracle's single-device chain; the
column-sharded bf16 / int8 GEMMs whose all-gather is done by the epilogue, and head-sharded attention.  Ranks are child
processes, one per GPU, NCCL's own NVLS off.  No rank is made to fail here: failure handling is tested on the host
(tests/test_capi_host.py), so no rank leaves while its memory is bound to a multicast object."""
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
        if mode == "peer_push_multicast":
            fused = lambda m, n, d: PeerPushExchange(m, n, d, multicast=True)
        else:
            fused = {"peer_push": PeerPushExchange, "peer_reduce_scatter": PeerReduceScatterExchange}.get(mode)
        ex = fused(BATCH, HIDDEN[2], dev) if fused else AllReduceExchange(CudaOps())
        # the two row-parallel layers have different widths: one exchange object per width
        ex2 = fused(BATCH, HIDDEN[4], dev) if fused else ex
        if mode == "peer_push_multicast" and not (ex.multicast and ex2.multicast):
            q.put((rank, None))              # symmetric memory without a multicast mapping on this machine
            return
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


def _fused_worker(rank, world, port, full, q):
    """The tensor-parallel step behind the C ABI (gcb200_tp_mlp_*): device-resident steps (eager, captured, replayed)
    and the host-buffer form, on the small chain or on BASELINE configs[2] at full size."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from gc_b200 import lib
    from gc_b200.tensor_parallel import FusedTensorParallelMLP, shard_weights

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        X, Ws, Bs, batch, hidden = _make_full() if full else (*_make(), BATCH, HIDDEN)
        ws, bs = shard_weights([w.to(dev) for w in Ws], [b.to(dev) for b in Bs], world, rank)
        tp = FusedTensorParallelMLP(ws, bs, batch, hidden, dev, relu=True)
        Xd = X.to(dev)
        outs = []
        for _ in range(4):                     # eager, captured, replayed, replayed: counters and buffers carry over
            y = tp.step(Xd)
            torch.cuda.synchronize()
            outs.append(_bits(y).copy())
        assert lib.device_error() == 0
        xh, yh = X.pin_memory(), torch.empty(batch, hidden[-1], dtype=torch.bfloat16).pin_memory()
        for _ in range(3):                     # the synchronous host-buffer form, every rank reading the result
            yh.zero_()
            tp.execute(xh, yh)
            outs.append(_bits(yh).copy())
        assert lib.device_error() == 0
        dist.barrier()
        tp.close()
        rows = slice(None) if not full else FULL_ROWS
        q.put((rank, [o[rows] for o in outs]))
    finally:
        dist.destroy_process_group()


FULL_ROWS = [0, 1, 63, 64, 127, 128, 129, 255, 256, 300, 383, 384, 447, 448, 510, 511]


def _make_full():
    from gc_b200 import benchgc_compat as bc

    hidden = (4096, 16384, 4096, 16384, 4096)
    X = bc.fill_tensor((512, hidden[0]), "bf16", "N", (0, 1), 0)
    Ws = [bc.fill_tensor((hidden[i], hidden[i + 1]), "bf16", "N", (0, 0.02), 1 + i) for i in range(4)]
    Bs = [torch.zeros(hidden[i + 1], dtype=torch.bfloat16) for i in range(4)]
    return X, Ws, Bs, 512, hidden


@pytest.mark.parametrize("full", [False, True])
def test_fused_tensor_parallel_step_behind_the_c_abi(full):
    """Every hand-off between the GPUs is a device counter of this library's own kernels.  Small chain: the whole
    result against the oracle; BASELINE configs[2] at full size (512 x 4096-16384-4096-16384-4096): 16 rows against
    the oracle.  Every rank, every step (device-resident and host-buffer form): identical bits."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    if world == 3:
        world = 2
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_fused_worker, args=(r, world, port, full, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for r in range(world):
        for step in range(len(res[r])):
            assert np.array_equal(res[r][step], res[0][0]), (r, step)
    if full:
        X, Ws, Bs, _, hidden = _make_full()
        h = _bits(X)[FULL_ROWS]
        for W, b in zip(Ws, Bs):
            h = oracle.linear_bf16(h, _bits(W), _bits(b), relu=True)
        mx, same = assert_bf16_close(res[0][0], h, 16384, what="fused tp, configs[2] full size", floor_div=1.0)
    else:
        X, Ws, Bs = _make()
        want = oracle.mlp_bf16(_bits(X), [_bits(w) for w in Ws], [_bits(b) for b in Bs], relu=True)
        from _util import bf16_f32
        pre = np.abs(bf16_f32(want)) + np.abs(bf16_f32(_bits(Bs[3])))[None, :]
        mx, same = assert_bf16_close(res[0][0], want, max(HIDDEN), what="fused tp", floor_div=1.0, pre=pre)
    print(f"tp{world} fused counters full={full}: max_abs={mx:.4g} bit-identical={same:.5f}")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode", ["all_reduce", "peer_push", "peer_reduce_scatter", "peer_push_multicast"])
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
    if any(v is None for v in res.values()):
        pytest.skip("no NVLink multicast mapping for symmetric memory here")
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


def _gather_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from gc_b200 import lib
    from gc_b200.tensor_parallel import PeerGatherGemm, ShardedAttention, shard_range

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        A, B, bias, Aq, Wq, sc, bi, Q, K, V = _gather_inputs()
        M, N = A.shape[0], B.shape[1]
        lo, hi = shard_range(N, world, rank)
        gg = PeerGatherGemm(B[:, lo:hi].contiguous().to(dev), M, N, dev, bias_shard=bias[lo:hi].contiguous().to(dev), relu=True)
        gq = PeerGatherGemm(Wq[:, lo:hi].contiguous().to(dev), M, N, dev, bias_shard=bi[lo:hi].contiguous().to(dev),
                            quant=(sc[lo:hi].contiguous().to(dev), 128))
        gd = PeerGatherGemm(B[:, lo:hi].contiguous().to(dev), 16, N, dev, bias_shard=bias[lo:hi].contiguous().to(dev), relu=True)
        dec = gd.step(A[:16].contiguous().to(dev))       # decode-shaped batch: the weight-stationary kernel stores to the peers
        torch.cuda.synchronize()
        dec = _bits(dec).copy()
        outs = []
        for _ in range(3):                     # repeated steps exercise the alternating result buffers
            c = gg.step(A.to(dev))
            cq = gq.step(Aq.to(dev))
            torch.cuda.synchronize()
            outs.append((_bits(c).copy(), cq.cpu().numpy().copy()))
        # the same two GEMMs with one multimem store per chunk (NVSwitch multicast), where symmetric memory offers it
        mg = PeerGatherGemm(B[:, lo:hi].contiguous().to(dev), M, N, dev, bias_shard=bias[lo:hi].contiguous().to(dev), relu=True,
                            multicast=True)
        mq = PeerGatherGemm(Wq[:, lo:hi].contiguous().to(dev), M, N, dev, bias_shard=bi[lo:hi].contiguous().to(dev),
                            quant=(sc[lo:hi].contiguous().to(dev), 128), multicast=True)
        if mg.multicast and mq.multicast:
            for _ in range(2):
                c = mg.step(A.to(dev))
                cq = mq.step(Aq.to(dev))
                torch.cuda.synchronize()
                assert np.array_equal(_bits(c), outs[0][0]), "multicast gather differs from the peer-store gather"
                assert np.array_equal(cq.cpu().numpy(), outs[0][1])
        o = ShardedAttention(world, rank).step(Q.to(dev), K.to(dev), V.to(dev), 128 ** -0.5, True, gather=True)
        torch.cuda.synchronize()
        assert lib.device_error() == 0
        q.put((rank, outs, _bits(o).copy(), dec))
    finally:
        dist.destroy_process_group()


def _gather_inputs():
    g = torch.Generator().manual_seed(3)
    M, N, K = 256, 2048, 1024
    A = (torch.rand(M, K, generator=g) * 2 - 1).bfloat16()
    B = (torch.rand(K, N, generator=g) * 2 - 1).bfloat16()
    bias = (torch.rand(N, generator=g) * 2 - 1).bfloat16()
    Aq = torch.randint(0, 256, (M, K), generator=g, dtype=torch.uint8)
    Wq = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    sc, bi = torch.rand(N, generator=g) * 0.009 + 0.001, torch.rand(N, generator=g) * 2 - 1
    Q, Kt, V = (torch.randn(2, 4, 256, 128, generator=g).bfloat16() for _ in range(3))
    return A, B, bias, Aq, Wq, sc, bi, Q, Kt, V


def test_column_sharded_gemms_gathered_by_the_epilogue_and_head_sharded_attention():
    """BASELINE's N-sharded GEMM sweep and int8 GEMM with the all-gather of C done by peer stores from the GEMM
    epilogue, and attention sharded by (batch, head): every rank must end with the single-device result."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    if world == 3:
        world = 2
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = {r: (outs, att, dec) for r, outs, att, dec in got}
    A, B, bias, Aq, Wq, sc, bi, Q, K, V = _gather_inputs()
    want, acc = oracle.linear_bf16(_bits(A), _bits(B), _bits(bias), relu=True, return_acc=True)
    _, wantq = oracle.linear_u8s8(Aq.numpy(), Wq.numpy(), sc.numpy(), bi.numpy(), zp_a=128)
    for r in range(world):
        for step in range(3):
            assert np.array_equal(res[r][0][step][0], res[0][0][0][0]), (r, step)
            assert np.array_equal(res[r][0][step][1], wantq), (r, step)       # int8: exact sums, same two f32 operations
        assert np.array_equal(res[r][1], res[0][1])
        assert np.array_equal(res[r][2], res[0][2])
    mx, same = assert_bf16_close(res[0][0][0][0], want, A.shape[1], what="gathered gemm", pre=acc)
    assert_bf16_close(res[0][2], want[:16], A.shape[1], what="gathered decode-shaped gemm", pre=acc[:16])
    from gc_b200 import lib
    dev = torch.device("cuda", 0)
    single = lib.attention_bf16(Q.to(dev), K.to(dev), V.to(dev), 128 ** -0.5, True)
    assert np.array_equal(res[0][1], _bits(single))     # heads are independent: sharding changes no bit
    print(f"gathered gemm on {world} GPUs: max_abs={mx:.4g} bit-identical={same:.5f}")
