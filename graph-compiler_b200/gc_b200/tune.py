"""Find the fastest matmul configuration of a shape by timing candidates on the device, and record it.

The tile selector (``select_matmul_config``) is a time model fitted to a few shapes.  ``tune_matmul``
times the model's choice and its neighbours (tile width, K split, K blocks per stage) with CUDA events
and records the winner in the library's measured-configuration cache, which every later launch of that
exact shape consults first; ``lib.tune_cache_save`` / the ``GC_B200_TUNE_CACHE`` environment variable
persist it across processes.  The reference chooses per op with hand-set cost functions and lets a user
override the choice through op attributes (lib/gc/Analysis/MatmulConfigAnalysis.cpp:368-401, :435-552).

    python -m gc_b200.tune --shapes 512x16384x4096,512x4096x16384 --out matmul.tune
    GC_B200_TUNE_CACHE=matmul.tune python bench.py
"""
from __future__ import annotations

import argparse
import itertools
from typing import Iterable, List, Optional, Tuple

from . import lib


def candidates(M: int, N: int, K: int, dtype_bytes: int = 2, out_bytes: int = 2, sms: int = 148) -> List[lib.MatmulConfig]:
    """The model's configuration first, then its neighbours: tile widths, K splits and K blocks per stage
    that the kernels accept for this shape.  Pure host logic."""
    base = lib.model_matmul_config(M, N, K, dtype_bytes, out_bytes, sms)
    k_blocks = -(-K // (128 // dtype_bytes))
    out: List[lib.MatmulConfig] = [base]
    seen = {(base.bn, base.splits, base.kpb)}
    if base.swapped:
        grid = list(itertools.product([base.bn], [1, 2, 3, 4, 6, 8], [1, 2]))
    else:
        gran = 64 if out_bytes == 2 else 32
        widths = [w for w in (256, 192, 128, 64) if w % gran == 0 and (w <= max(gran, -(-N // gran) * gran) or w == base.bn)]
        grid = list(itertools.product(widths, [1, 2, 3, 4, 6, 8], [1, 2]))
    tiles_m = -(-M // 128)
    for bn, splits, kpb in grid:
        if (bn, splits, kpb) in seen:
            continue
        if kpb == 2 and (bn > 128 and not base.swapped or k_blocks < 4):
            continue                                     # three stages of two K blocks must fit in shared memory
        if splits > 1 and (k_blocks < 16 * splits or -(-k_blocks // splits) % kpb):
            continue                                     # a stage must not straddle two splits
        tiles = -(-N // 128) if base.swapped else tiles_m * -(-N // bn)
        if splits > 1 and tiles >= sms:
            continue
        c = lib.MatmulConfig(base.swapped, bn, splits, 8 if kpb == 1 else 3, base.group_m, min(tiles * splits, sms), 0, kpb)
        out.append(c)
        seen.add((bn, splits, kpb))
    if not base.swapped and dtype_bytes == 2 and M >= 256:
        # the CTA-pair kernel (256 x bn tiles on two SMs) with and without a K split, whichever the model chose
        have = {(c.bn, c.splits, max(c.kpb, 1), c.pair) for c in out}
        for pair in (0, 1):
            for splits in sorted({1, 2, base.splits}):
                if splits > 1 and (k_blocks < 16 * splits or tiles_m * -(-N // 256) >= sms):
                    continue
                if (256, splits, 1, pair) not in have:
                    out.append(lib.MatmulConfig(0, 256, splits, 8, base.group_m, min(tiles_m * -(-N // 256) * splits, sms), pair, 1))
                    have.add((256, splits, 1, pair))
    return out


def _time(fn, iters: int, flush) -> float:
    import torch

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        fn()
        en.record()
        torch.cuda.synchronize()
        tot += st.elapsed_time(en)
    return tot / iters * 1e3


def tune_matmul(M: int, N: int, K: int, int8: bool = False, iters: int = 10, record: bool = True,
                configs: Optional[Iterable[lib.MatmulConfig]] = None) -> Tuple[lib.MatmulConfig, float, List[Tuple[str, float]]]:
    """Times every candidate for a bf16 (or u8 x s8, dequantised f32) matmul of this shape on the current device.
    Returns (best configuration, its microseconds, [(repr, microseconds or nan)] for all candidates); records the
    best one in the measured-configuration cache unless ``record`` is False.  Inputs smaller than 256 MB are timed
    with a write of a 256 MiB buffer between launches so that operands come from HBM."""
    import torch

    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)
    eb, ob = (1, 4) if int8 else (2, 2)
    if int8:
        A = torch.randint(0, 256, (M, K), generator=g, device=dev, dtype=torch.uint8)
        W = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)
        sc = torch.rand(N, generator=g, device=dev) * 0.009 + 0.001
        comp = lib.colsum_s8(W, 128)
        run = lambda: lib.matmul_u8s8(A, W, sc, None, comp)
    else:
        A = (torch.rand((M, K), generator=g, device=dev) * 2 - 1).bfloat16()
        W = (torch.rand((K, N), generator=g, device=dev) * 2 - 1).bfloat16()
        Y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        run = lambda: lib.matmul_bf16(A, W, None, out=Y)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if (M * K + K * N) * eb + M * N * ob < 256e6 else None
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    cands = list(configs) if configs is not None else candidates(M, N, K, eb, ob, sms)
    results, best, best_us = [], None, float("inf")
    saved = lib.tune_cache_get(M, N, K, eb, ob)
    try:
        for c in cands:
            try:
                lib.tune_cache_put(M, N, K, c, eb, ob)     # the launchers pick the recorded configuration up
                us = _time(run, iters, flush)
            except RuntimeError:                           # a candidate the kernels reject (shared memory, alignment)
                us = float("nan")
            results.append((repr(c), us))
            if us == us and us < best_us:
                best, best_us = c, us
        if lib.device_error() != 0:
            raise RuntimeError("a kernel reported a wait time-out while tuning")
    finally:
        if saved is not None:                              # leave the cache as it was unless a winner is recorded below
            lib.tune_cache_put(M, N, K, saved, eb, ob)
        else:
            lib.tune_cache_erase(M, N, K, eb, ob)
    if best is not None and record:
        lib.tune_cache_put(M, N, K, best, eb, ob)
    return best, best_us, results


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shapes", required=True, help="comma-separated MxNxK list")
    ap.add_argument("--int8", action="store_true", help="u8 x s8 with dequantised f32 output instead of bf16")
    ap.add_argument("--out", default=None, help="write the cache here (entries already in the file are kept)")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    import os

    if a.out and os.path.exists(a.out):
        lib.tune_cache_load(a.out)
    for spec in a.shapes.split(","):
        M, N, K = (int(v) for v in spec.lower().split("x"))
        best, us, results = tune_matmul(M, N, K, int8=a.int8, iters=a.iters)
        base_us = results[0][1]
        print(f"{M}x{N}x{K}: model {base_us:.1f} us -> best {us:.1f} us  {best}")
    if a.out:
        print(f"wrote {lib.tune_cache_save(a.out)} entries to {a.out}")


if __name__ == "__main__":
    main()
