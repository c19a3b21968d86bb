"""benchgc-compatible input fills and comparison rule.

The reference's benchmark/correctness harness (test/benchgc) fills argument
``i`` after seeding torch with ``seed + i`` and compares results point-to-point
with a relative/absolute switch.  The partitions run here take the same flags,
so inputs and verdicts are identical to a benchgc run on the same command line.

  fill_tensor : test/benchgc/src/benchgc/arg/__init__.py:94-153, util.py:163-171
  p2p         : test/benchgc/src/benchgc/arg/compare.py:60-137
"""
from __future__ import annotations

import random
from typing import Sequence, Tuple

import numpy
import torch

_DTYPES = {
    "f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "f64": torch.float64,
    "s32": torch.int32, "s8": torch.int8, "u8": torch.uint8, "s64": torch.int64, "boolean": torch.bool,
}


def get_dtype(name: str) -> torch.dtype:
    if name not in _DTYPES:
        raise ValueError(f"data type not support: {name}")
    return _DTYPES[name]


def seed_all(seed: int) -> None:
    torch.manual_seed(seed)
    numpy.random.seed(seed)
    random.seed(seed)


def fill_tensor(shape: Sequence[int], dtype: str, fill_type: str, fill_param: Sequence, idx: int,
                seed: int = 0) -> torch.Tensor:
    """Argument ``idx`` of a partition, filled the way ``--fill idx:TYPE:params`` does.

    TYPE: N mean std | U a b | I a b (inclusive) | P lambda | B n p | Z.
    """
    seed_all(seed + idx)
    shape = list(shape)
    p = [str(x) for x in fill_param]
    if fill_type == "N" and len(p) == 2:
        t = torch.normal(mean=float(p[0]), std=float(p[1]), size=shape)
    elif fill_type == "P" and len(p) == 1:
        t = torch.poisson(torch.full(shape, float(p[0])))
    elif fill_type == "B" and len(p) == 2:
        t = torch.distributions.binomial.Binomial(total_count=int(p[0]), probs=float(p[1])).sample(torch.Size(shape))
    elif fill_type == "U" and len(p) == 2:
        t = torch.distributions.uniform.Uniform(float(p[0]), float(p[1])).sample(torch.Size(shape))
    elif fill_type == "I" and len(p) == 2:
        t = torch.randint(int(p[0]), int(p[1]) + 1, torch.Size(shape))
    elif fill_type == "Z":
        t = torch.zeros(size=shape)
    else:
        raise ValueError("invalid fill type or fill parameter")
    return t.to(get_dtype(dtype))


def p2p(threshold: float, zero_percent: float, ref: torch.Tensor, res: torch.Tensor) -> Tuple[bool, bool | None]:
    """Point-to-point check: relative error where |ref| > 1e-5, else absolute.

    Returns (passed, mistrust); ``mistrust`` flags an output with too many zeros.
    """
    f32_ref, f32_res = ref.to(torch.float32), res.to(torch.float32)
    check = f32_ref.isnan() & f32_res.isnan()
    check |= f32_ref.isneginf() & f32_res.isneginf()
    check |= f32_ref.isposinf() & f32_res.isposinf()
    abs_diff = (f32_ref - f32_res).abs()
    tiny = float(numpy.finfo(numpy.float32).smallest_subnormal)
    rel_diff = abs_diff / torch.where(f32_ref.abs() > tiny, f32_ref.abs(), torch.ones_like(f32_ref))
    diff = torch.where(f32_ref.abs() > 1e-5, rel_diff, abs_diff)
    check |= diff <= threshold
    if bool(check.all()):
        zero = res.nelement() - int(res.count_nonzero())
        mistrust = False if res.nelement() < 10 else zero * 100.0 / res.nelement() > zero_percent
        return True, mistrust
    return False, None


def norm(threshold: float, ref: torch.Tensor, res: torch.Tensor) -> Tuple[bool, bool | None]:
    """Norm check, the harness's other comparison (test/benchgc/src/benchgc/arg/compare.py:42-57, ``--cmp i:N:threshold``):
    sqrt(sum (ref - res)^2 / sum ref^2) < threshold, evaluated in f32."""
    r, s = ref.to(torch.float32), res.to(torch.float32)
    if r.nelement() == 0:
        return True, None
    l2 = torch.sqrt(torch.square(r - s).sum() / torch.square(r).sum()).item()
    return l2 < threshold, None


def max_errors(ref: torch.Tensor, res: torch.Tensor) -> Tuple[float, float]:
    """(max abs error, max rel error over |ref| > 1e-5) — reported per config."""
    r, s = ref.to(torch.float32), res.to(torch.float32)
    ad = (r - s).abs()
    mask = r.abs() > 1e-5
    rel = (ad[mask] / r.abs()[mask]).max().item() if bool(mask.any()) else 0.0
    return ad.max().item(), rel
