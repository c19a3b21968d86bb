"""Shared helpers for the parity tests."""
import numpy as np
import torch


def tbits(t: torch.Tensor) -> np.ndarray:
    """bf16 torch tensor -> uint16 bit patterns (numpy, on host)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(a: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(device)


def bf16_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def assert_bf16_close(got_bits: np.ndarray, want_bits: np.ndarray, K: int, rtol: float = 1e-2, what: str = "",
                      pre: np.ndarray | None = None, floor_div: float = 16.0):
    """BASELINE tolerance for bf16 paths: relative 1e-2 per element (benchgc's point-to-point rule,
    test/benchgc/src/benchgc/arg/compare.py:84-93), with the two places where a *correct* result may
    exceed a purely relative bound stated explicitly:

      * an element far below the tensor's own scale (|want| < rms/floor_div) is held to
        rtol * rms/floor_div — f32 summation order alone moves such near-cancelled sums by more than
        1e-2 of themselves.  floor_div = 16 for one layer; chained layers pass 1 (tolerance relative
        to max(|want|, rms)): 1-ulp flips of one layer's bf16 activations are noise of the next layer's
        sums, which grows with depth relative to the small elements of the final tensor;
      * when a bias is added after the first rounding (``pre`` = the oracle's f32 accumulators), one
        bf16 ulp of the pre-bias value plus one of the result (<= 2^-7 (|pre| + |want|)) is allowed:
        bf16(bf16(acc)+bias) rounds twice, so a 1-ulp flip of bf16(acc) — which any change of f32
        summation order can cause — reaches the output as up to two ulps, and as an absolute
        difference that can be large relative to a small (cancelled) sum.

    Returns (max_abs, bit_identical_fraction)."""
    g, w = bf16_f32(got_bits).astype(np.float64), bf16_f32(want_bits).astype(np.float64)
    assert g.shape == w.shape, (g.shape, w.shape)
    nan_ok = np.isnan(g) & np.isnan(w)
    diff = np.abs(g - w)
    nz = np.abs(w[np.isfinite(w) & (w != 0)])
    floor = float(np.sqrt(np.mean(nz ** 2))) / floor_div if nz.size else 0.0
    tol = rtol * np.maximum(np.abs(w), floor)
    if pre is not None:
        tol = np.maximum(tol, 2.0 ** -7 * (np.abs(pre.astype(np.float64)) + np.abs(w)))
    ok = nan_ok | (diff <= tol)
    if not ok.all():
        bad = np.argwhere(~ok)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} of {ok.size} elements outside rtol={rtol}; first {i}: got {g[i]} want {w[i]}")
    return float(np.nanmax(diff)) if diff.size else 0.0, float((got_bits == want_bits).mean())
