"""Column/row tensor-parallel execution of a chained-MLP partition across GPUs.

The reference splits one matmul over CPU threads along M, N and K
(``MThreads x NThreads x KThreads``, lib/gc/Transforms/DeepTileContractionOp.cpp:562-601);
a K split produces f32 partial sums that are reduced and only then cast
(:446-471, :988-996).  Across GPUs the same two rules apply per layer pair:

  * odd layers (1st, 3rd, ...) are split along N: rank r owns ``W[:, r-th block]`` and the matching
    bias block; bias add and ReLU stay local (the NThreads rule);
  * even layers are split along K: rank r owns ``W[r-th block, :]``, produces f32 partial sums
    for the whole [M, N] result, the partial sums are all-reduced (sum, f32) and only then
    cast / biased / activated on every rank (the KThreads rule).

One process per GPU; the only collective is that all-reduce.  The compute calls
are injected (``ops``) so that the sharding logic can run under gloo on CPU with a
stand-in for the kernels.
"""
from __future__ import annotations

from typing import List, Optional, Sequence


def shard_range(n: int, world: int, rank: int):
    """Contiguous block of ``n`` owned by ``rank`` (n must divide evenly)."""
    if n % world:
        raise ValueError(f"dimension {n} is not divisible by world size {world}")
    step = n // world
    return rank * step, (rank + 1) * step


def shard_weights(weights: Sequence, biases: Sequence, world: int, rank: int):
    """Slice full [K,N] weights / [N] biases for ``rank``.  Layer i (0-based) is column-parallel
    when i is even, row-parallel when odd.  Returns (weight shards, bias shards) where the bias
    of a row-parallel layer is kept whole (applied after the reduction)."""
    ws, bs = [], []
    for i, (W, b) in enumerate(zip(weights, biases)):
        if i % 2 == 0:
            lo, hi = shard_range(W.shape[1], world, rank)
            ws.append(W[:, lo:hi].contiguous())
            bs.append(None if b is None else b[lo:hi].contiguous())
        else:
            lo, hi = shard_range(W.shape[0], world, rank)
            ws.append(W[lo:hi, :].contiguous())
            bs.append(b)
    return ws, bs


class CudaOps:
    """The launchers a step needs, bound to the C ABI."""

    def __init__(self):
        from . import lib

        self._lib = lib

    def linear(self, x, w, b, relu):
        return self._lib.matmul_bf16(x, w, b, relu=relu)

    def linear_partial(self, x, w):
        return self._lib.matmul_bf16_f32out(x, w)

    def epilogue(self, planes, b, relu):
        """planes: f32 [nparts, M, N] — summed in plane order, then cast, bias, ReLU."""
        return self._lib.reduce_bias_act_bf16(planes, b, relu=relu)


def _multicast_ptr(handle) -> int:
    """The NVLink multicast address of a symmetric-memory allocation, or 0 when the allocation has none."""
    try:
        return int(getattr(handle, "multicast_ptr", 0) or 0)
    except Exception:
        return 0


class AllReduceExchange:
    """Baseline exchange: local f32 partial sums, one NCCL/gloo all-reduce, then the epilogue on every rank."""

    name = "all_reduce"
    launches_per_pair = 3

    def __init__(self, ops, group=None):
        self.ops, self.group = ops, group

    def row_parallel(self, x, w, bias, relu):
        import torch.distributed as dist

        part = self.ops.linear_partial(x, w)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
        return self.ops.epilogue(part.unsqueeze(0), bias, relu)


class PeerPushExchange:
    """Fused exchange, all-to-all form: the GEMM epilogue stores this rank's partial sums into plane `rank` of
    every rank's receive buffer (peer-mapped symmetric memory, plain NVLink stores), one cross-rank barrier,
    then every rank reduces its g planes locally in rank order.  Every partial sum crosses NVLink g - 1 times:
    fine for two ranks, wasteful beyond (see PeerReduceScatterExchange).  Two receive buffers alternate so that
    a buffer is only overwritten after the barrier of the following exchange."""

    name = "peer_push"
    launches_per_pair = 3

    def __init__(self, M: int, N: int, device, group=None, multicast: bool = False):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import lib

        self._lib = lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.bufs, self.hdls, self.ptrs, self.mc = [], [], [], []
        for _ in range(2):
            t = symm.empty((self.world, M, N), dtype=torch.float32, device=device)
            h = symm.rendezvous(t, self.group)
            self.bufs.append(t)
            self.hdls.append(h)
            self.ptrs.append([int(p) for p in h.buffer_ptrs])
            self.mc.append(_multicast_ptr(h) if multicast else 0)
        # one multimem store per chunk through the NVSwitch instead of one store per peer (needs multicast-capable
        # symmetric memory and the row-major kernel, M > 64)
        self.multicast = bool(multicast and all(self.mc) and M > 64)
        if self.multicast:
            self.name = "peer_push_multicast"
        self.turn = 0

    def row_parallel(self, x, w, bias, relu):
        i = self.turn
        self.turn ^= 1
        if self.multicast:
            self._lib.matmul_bf16_f32out_push_mc(x, w, self.mc[i], self.rank)
        else:
            self._lib.matmul_bf16_f32out_push(x, w, self.ptrs[i], self.rank)
        self.hdls[i].barrier(channel=0)   # every rank's stores have landed and are visible
        return self._lib.reduce_bias_act_bf16(self.bufs[i], bias, relu=relu)


class PeerReduceScatterExchange:
    """Fused exchange with an all-reduce's traffic.  The GEMM epilogue stores row block d of this rank's f32
    partial sums into peer d's receive buffer only (reduce-scatter by rows, overlapped with the tiles still
    being computed); barrier; rank d sums the g planes of its rows in rank order, applies bias / ReLU, casts
    once and stores the bf16 rows into EVERY rank's result buffer (all-gather by peer stores); barrier.  Per
    GPU (g - 1)/g of the f32 partial sums and (g - 1)/g of the bf16 result cross NVLink, instead of g - 1
    copies of the partial sums.  Every rank ends with identical bits: each row is reduced exactly once.
    Result buffers alternate so that a step's output survives the next exchange."""

    name = "peer_reduce_scatter"
    launches_per_pair = 3

    def __init__(self, M: int, N: int, device, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import lib

        self._lib = lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if M % self.world:
            raise ValueError(f"{M} rows are not divisible by {self.world} ranks")
        self.rows = M // self.world
        self.recv = symm.empty((self.world, self.rows, N), dtype=torch.float32, device=device)
        self.recv_h = symm.rendezvous(self.recv, self.group)
        self.recv_ptrs = [int(p) for p in self.recv_h.buffer_ptrs]
        self.outs, self.out_ptrs = [], []
        for _ in range(2):
            t = symm.empty((M, N), dtype=torch.bfloat16, device=device)
            h = symm.rendezvous(t, self.group)
            self.outs.append(t)
            self.out_ptrs.append([int(p) for p in h.buffer_ptrs])
        self.turn = 0

    def row_parallel(self, x, w, bias, relu):
        i = self.turn
        self.turn ^= 1
        self._lib.matmul_bf16_f32out_scatter(x, w, self.recv_ptrs, self.rank)
        self.recv_h.barrier(channel=0)   # my rows of every rank's partial sums have landed
        self._lib.reduce_slice_broadcast_bf16(self.recv, bias, relu, self.out_ptrs[i], self.rank * self.rows)
        self.recv_h.barrier(channel=1)   # every rank's rows of the result have landed here; recv is free again
        return self.outs[i]


class FusedTensorParallelMLP:
    """The tensor-parallel MLP step behind the C ABI (``gcb200_tp_mlp_*``, csrc/tp.cu): this class only allocates
    the memory every rank can address (torch symmetric memory: plumbing) and hands the address tables to the
    library, whose own kernels do the GEMMs, the exchange and every hand-off between GPUs (device counters, no
    barrier kernels of another library, no host round trip between layers).

    ``weight_shards`` / ``bias_shards`` as returned by ``shard_weights``; ``hidden`` the full layer widths."""

    name = "fused_counters"

    def __init__(self, weight_shards, bias_shards, batch: int, hidden, device, relu: bool = True, group=None, with_input: bool = True):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import lib

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.batch, self.hidden = batch, list(hidden)
        self.w, self.b = list(weight_shards), list(bias_shards)
        nmax = max(self.hidden[2::2])
        self._bufs = []

        def shared(shape, dtype):
            t = symm.empty(shape, dtype=dtype, device=device)
            h = symm.rendezvous(t, self.group)
            self._bufs.append((t, h))
            return t, [int(p) for p in h.buffer_ptrs]

        self.recv, self.act, recv_p, act_p = [], [], [], []
        for _ in range(2):
            t, p = shared((2 * self.world, batch // self.world, nmax), torch.float32)   # one plane per rank and K split
            self.recv.append(t); recv_p.append(p)
            t, p = shared((batch, nmax), torch.bfloat16)
            self.act.append(t); act_p.append(p)
        self.signals, sig_p = shared((16,), torch.int32)
        self.signals.zero_()
        x_p = None
        if with_input:
            self.x_in, x_p = shared((batch, self.hidden[0]), torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier(self.group)          # every rank's counters are zero before anyone adds to them
        self.plan = lib.TpMlpPlan(self.world, self.rank, batch, self.hidden, [w.data_ptr() for w in self.w],
                                  [0 if b is None else b.data_ptr() for b in self.b], relu, recv_p, act_p, sig_p, x_p,
                                  recv_planes=2 * self.world)
        self.launches_per_step = 3 * (len(self.w) // 2) + 1
        self.collectives_per_step = 0
        self._slot = (len(self.w) // 2 - 1) & 1
        self._n_out = self.hidden[-1]

    def _result(self):
        t = self.act[self._slot]
        return t if t.shape[1] == self._n_out else t.view(-1)[: self.batch * self._n_out].view(self.batch, self._n_out)

    def step(self, x):
        """x: bf16 [batch, hidden[0]] on this rank's device (the same values on every rank)."""
        self.plan.step(x.data_ptr())
        return self._result()

    def execute(self, x_host, y_host=None):
        """Synchronous host-buffer form (pinned tensors): every rank passes the same full input."""
        self.plan.execute(x_host.data_ptr(), 0 if y_host is None else y_host.data_ptr())
        return self._result()

    def close(self):
        import torch

        torch.cuda.synchronize()
        self.plan.destroy()
        self._bufs.clear()


class TensorParallelMLP:
    """An even number of bias+ReLU layers, sharded as described in the module docstring."""

    def __init__(self, weight_shards: List, bias_shards: List, relu: bool = True, ops=None, group=None, exchange=None):
        if len(weight_shards) % 2:
            raise ValueError("tensor-parallel MLP needs an even number of layers (column then row)")
        self.w, self.b, self.relu = list(weight_shards), list(bias_shards), relu
        self.ops = ops if ops is not None else CudaOps()
        self.group = group
        self.exchange = exchange if exchange is not None else AllReduceExchange(self.ops, group)
        self.launches_per_step = self.exchange.launches_per_pair * (len(self.w) // 2)
        self.collectives_per_step = len(self.w) // 2

    def step(self, x):
        h = x
        for i in range(0, len(self.w), 2):
            h = self.ops.linear(h, self.w[i], self.b[i], self.relu)                       # column-parallel, local post-ops
            h = self.exchange.row_parallel(h, self.w[i + 1], self.b[i + 1], self.relu)   # row-parallel: partial sums, exchange, epilogue
        return h


# ------------------------------------------------------------------------------------------------
# The other paths that shard: independent output columns (bf16 GEMM sweep, int8 GEMM) and independent
# (batch, head) units (attention).  No exchange is needed to compute; the only collective is the optional
# all-gather that reassembles the full result on every rank.
class ShardedGemm:
    """C = A . B with B (and C) split along N: rank r owns ``B[:, r-th block]`` and computes
    ``C[:, r-th block]``; A is replicated.  ``gather=True`` all-gathers the column blocks."""

    def __init__(self, B_shard, world: int, rank: int, ops=None, group=None):
        self.B, self.world, self.rank, self.group = B_shard, world, rank, group
        self.ops = ops if ops is not None else CudaOps()

    def step(self, A, gather: bool = True):
        import torch
        import torch.distributed as dist

        c = self.ops.linear(A, self.B, None, False)            # [M, N / world]
        if not gather or self.world == 1:
            return c
        parts = [torch.empty_like(c) for _ in range(self.world)]
        dist.all_gather(parts, c.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)


class PeerGatherGemm:
    """Column-sharded GEMM with the all-gather fused into the GEMM: the epilogue stores every finished chunk of
    this rank's column block into the same place of EVERY rank's full [M, N] result (peer-mapped symmetric
    memory, plain NVLink stores that overlap the tiles still being computed); one cross-rank barrier and every
    rank holds the whole C.  ``quant`` selects the u8 x s8 form (f32 result; scales, bias and zero-point
    compensation split with the columns).  Two result buffers alternate, so a result stays valid until the
    step after the next one.  Batches of at most 64 rows run the weight-stationary kernel, which stores its
    elements to the peers one by one (the result is small)."""

    def __init__(self, W_shard, M: int, N_total: int, device, bias_shard=None, relu: bool = False, quant=None, group=None,
                 multicast: bool = False):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import lib

        self._lib = lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.W, self.bias, self.relu, self.quant = W_shard, bias_shard, relu, quant
        self.N = N_total
        n_shard = W_shard.shape[1]
        if n_shard * self.world != N_total:
            raise ValueError(f"{self.world} column blocks of {n_shard} do not make {N_total} columns")
        dtype = torch.float32 if quant is not None else torch.bfloat16
        esz = 4 if quant is not None else 2
        if quant is not None:
            scale, zp = quant
            self.scale = scale
            self.comp = lib.colsum_s8(W_shard, zp)    # zp * sum_k W[k, n]: per column, so it splits with N
        self.bufs, self.hdls, self.ptrs, self.mc = [], [], [], []
        for _ in range(2):
            t = symm.empty((M, N_total), dtype=dtype, device=device)
            h = symm.rendezvous(t, self.group)
            self.bufs.append(t)
            self.hdls.append(h)
            self.ptrs.append([int(p) + self.rank * n_shard * esz for p in h.buffer_ptrs])
            mc = _multicast_ptr(h) if multicast else 0
            self.mc.append(mc + self.rank * n_shard * esz if mc else 0)
        # multicast: each chunk leaves this GPU once and the NVSwitch writes it into every rank's result
        self.multicast = bool(multicast and all(self.mc) and M > 64)
        self.turn = 0

    def step(self, A):
        i = self.turn
        self.turn ^= 1
        if self.multicast and self.quant is not None:
            self._lib.matmul_u8s8_allgather_mc(A, self.W, self.scale, self.bias, self.comp, self.mc[i], self.N)
        elif self.multicast:
            self._lib.matmul_bf16_allgather_mc(A, self.W, self.bias, self.relu, self.mc[i], self.N)
        elif self.quant is not None:
            self._lib.matmul_u8s8_allgather(A, self.W, self.scale, self.bias, self.comp, self.ptrs[i], self.N)
        else:
            self._lib.matmul_bf16_allgather(A, self.W, self.bias, self.relu, self.ptrs[i], self.N)
        self.hdls[i].barrier(channel=0)   # every rank's column block has landed here and is visible
        return self.bufs[i]


class ShardedQuantGemm:
    """u8 x s8 GEMM split along N: weights, scales, bias (and the zero-point compensation, which is a
    per-column sum over K) all split with the columns, so every rank's block is complete by itself."""

    def __init__(self, W_shard, scale_shard, bias_shard, zp: int, world: int, rank: int, ops=None, group=None):
        self.W, self.scale, self.bias, self.zp = W_shard, scale_shard, bias_shard, zp
        self.world, self.rank, self.group, self.ops = world, rank, group, ops

    def step(self, A, gather: bool = True):
        import torch
        import torch.distributed as dist

        if self.ops is not None:
            c = self.ops.quant_linear(A, self.W, self.scale, self.bias, self.zp)
        else:
            from . import lib

            comp = lib.colsum_s8(self.W, self.zp)          # zp * sum_k W[k, n]: per column, so it splits with N
            c, _ = lib.matmul_u8s8(A, self.W, self.scale, self.bias, comp)
        if not gather or self.world == 1:
            return c
        parts = [torch.empty_like(c) for _ in range(self.world)]
        dist.all_gather(parts, c.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)


def shard_heads(t, world: int, rank: int):
    """[B, H, S, D] -> this rank's contiguous block of the B*H independent (batch, head) units, as [units, 1, S, D]."""
    B, H, S, D = t.shape
    lo, hi = shard_range(B * H, world, rank)
    return t.reshape(B * H, 1, S, D)[lo:hi].contiguous()


class ShardedAttention:
    """Attention over (batch, head) units split across ranks; no collective on the data path."""

    def __init__(self, world: int, rank: int, ops=None, group=None):
        self.world, self.rank, self.ops, self.group = world, rank, ops, group

    def step(self, Q, K, V, scale: float, causal: bool, gather: bool = False):
        import torch
        import torch.distributed as dist

        q, k, v = (shard_heads(t, self.world, self.rank) for t in (Q, K, V))
        if self.ops is not None:
            o = self.ops.attention(q, k, v, scale, causal)
        else:
            from . import lib

            o = lib.attention_bf16(q, k, v, scale, causal)
        if not gather or self.world == 1:
            return o
        parts = [torch.empty_like(o) for _ in range(self.world)]
        dist.all_gather(parts, o.contiguous(), group=self.group)
        return torch.cat(parts, dim=0).reshape(Q.shape)
