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
    """The three launchers a step needs, bound to the C ABI."""

    def __init__(self):
        from . import lib

        self._lib = lib

    def linear(self, x, w, b, relu):
        return self._lib.matmul_bf16(x, w, b, relu=relu)

    def linear_partial(self, x, w):
        return self._lib.matmul_bf16_f32out(x, w)

    def epilogue(self, partial, b, relu):
        return self._lib.reduce_bias_act_bf16(partial.unsqueeze(0), b, relu=relu)


class TensorParallelMLP:
    """An even number of bias+ReLU layers, sharded as described in the module docstring."""

    def __init__(self, weight_shards: List, bias_shards: List, relu: bool = True, ops=None, group=None):
        if len(weight_shards) % 2:
            raise ValueError("tensor-parallel MLP needs an even number of layers (column then row)")
        self.w, self.b, self.relu = list(weight_shards), list(bias_shards), relu
        self.ops = ops if ops is not None else CudaOps()
        self.group = group
        self.launches_per_step = 3 * (len(self.w) // 2)
        self.collectives_per_step = len(self.w) // 2

    def step(self, x):
        import torch.distributed as dist

        h = x
        for i in range(0, len(self.w), 2):
            h = self.ops.linear(h, self.w[i], self.b[i], self.relu)          # column-parallel, local post-ops
            part = self.ops.linear_partial(h, self.w[i + 1])                 # row-parallel, f32 partial sums
            if dist.is_initialized() and dist.get_world_size(self.group) > 1:
                dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
            h = self.ops.epilogue(part, self.b[i + 1], self.relu)            # cast, bias, ReLU after the reduce
        return h
