"""Generate the golden fixtures in this directory from the reference's own Python code.

Run once, in a container that has the reference tree:

    python tests/golden/make_golden.py --ref /path/to/graph-compiler

It imports benchgc from ``<ref>/test/benchgc/src`` (the MLIR python bindings it
pulls in are absent here and are replaced by inert stub modules — only benchgc's
torch code is executed: ``fill_tensor``, the matmul driver's ``fill``, the
``ref_*`` op evaluators and ``compare.p2p``) and writes ``benchgc_golden.npz`` and
``benchgc_golden.json``.  The fixtures are small (inputs are stored as a SHA-256
plus a leading slice; reference outputs in full for the small cases) and are
what the test-suite reads; nothing at test time touches the reference tree.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.abc
import importlib.machinery
import json
import os
import sys
import types
from unittest import mock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


class _Stub(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return mock.MagicMock()


class _StubFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path, target=None):
        if name == "gc_mlir" or name.startswith("gc_mlir."):
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        m = _Stub(spec.name)
        m.__path__ = []
        return m

    def exec_module(self, module):
        pass


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(bits(t).tobytes()).hexdigest()


class _Cache:
    def __init__(self, opr):
        self.opr = opr


def main():
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--ref", default=os.environ.get("GC_REFERENCE_DIR") or
                    os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference"),
                    help="checkout of the reference (default: $GC_REFERENCE_DIR, else ../reference beside this repository)")
    a = ap.parse_args()
    sys.path.insert(0, os.path.join(a.ref, "test", "benchgc", "src"))
    sys.meta_path.insert(0, _StubFinder())
    import benchgc.arg as barg
    import benchgc.arg.compare as bcmp
    import benchgc.arg.matmul as bmatmul
    import benchgc.linalg.binary as lbin
    import benchgc.linalg.matmul as lmm
    import benchgc.linalg.softmax  # noqa: F401  (import check only)
    import benchgc.util as butil
    from benchgc.arg.arg import Arg

    flags = argparse.Namespace(verbose=0)
    arrays: dict[str, np.ndarray] = {}
    meta: dict = {"torch": torch.__version__, "fills": [], "cases": [], "p2p": []}

    def fill(idx, dtype, shape, ftype, params, seed=0):
        butil.set_seed(seed)
        arg = Arg(idx)
        arg.dtype, arg.shape, arg.fill_type, arg.fill_param = dtype, list(shape), ftype, [str(p) for p in params]
        return barg.fill_tensor(flags, arg, idx)

    # --- 1. fill semantics: (seed + arg index) then the torch call -------------------------
    for idx, dtype, shape, ftype, params, seed in [
        (0, "bf16", (128, 512), "U", (-1, 1), 0),
        (1, "bf16", (512, 256), "U", (-1, 1), 0),
        (2, "bf16", (256,), "U", (-1, 1), 0),
        (0, "bf16", (64, 96), "N", (0, 1), 0),
        (1, "bf16", (96, 32), "N", (0, 0.02), 0),
        (3, "f32", (33, 7), "N", (0, 1), 5),
        (0, "u8", (64, 128), "I", (0, 255), 0),
        (1, "s8", (128, 64), "I", (-127, 127), 0),
        (2, "f32", (64,), "U", (0.001, 0.01), 0),
        (4, "f32", (17,), "Z", (), 0),
        (1, "f32", (32, 16), "U", (0, 1), 3),
    ]:
        t = fill(idx, dtype, shape, ftype, params, seed)
        key = f"fill{len(meta['fills'])}"
        arrays[key + "_head"] = bits(t).reshape(-1)[:64].copy()
        meta["fills"].append(dict(key=key, idx=idx, dtype=dtype, shape=list(shape), fill_type=ftype,
                                  fill_param=[str(p) for p in params], seed=seed, sha256=sha(t)))

    # --- 2. reference results of the partitions, evaluated by benchgc's own ref_* ----------
    def run_mlp(name, batch, hidden, dtype, has_bias, act, fills, seed=0):
        """Mirror of benchgc pattern mlp (pattern/mlp.py:31-173): args are
        src, weights..., biases...; each layer = matmul, [broadcast+add], [max(x,0)]."""
        nl = len(hidden) - 1
        src = fill(0, dtype, (batch, hidden[0]), *fills["src"], seed=seed)
        ws = [fill(1 + i, dtype, (hidden[i], hidden[i + 1]), *fills["w"], seed=seed) for i in range(nl)]
        bs, j = [], 0
        for i in range(nl):
            if has_bias[i]:
                bs.append(fill(1 + nl + j, dtype, (hidden[i + 1],), *fills["b"], seed=seed))
                j += 1
            else:
                bs.append(None)
        var = {"h": src}
        for i in range(nl):
            var["w"] = ws[i]
            (h,) = lmm.ref_matmul(_Cache(["h", "w"]), None, var)
            if bs[i] is not None:
                var["m"], var["b"] = h, bs[i].reshape(1, -1).broadcast_to(h.shape).contiguous()
                (h,) = lbin.ref_add(_Cache(["m", "b"]), None, var)
            if act == "relu":
                var["x"], var["z"] = h, torch.zeros_like(h)
                (h,) = lbin.ref_max(_Cache(["x", "z"]), None, var)
            var["h"] = h
        arrays[name + "_out"] = bits(var["h"])
        meta["cases"].append(dict(name=name, kind="mlp", batch=batch, hidden=list(hidden), dtype=dtype,
                                  has_bias=list(has_bias), act=act, seed=seed,
                                  fills={k: [v[0], [str(p) for p in v[1]]] for k, v in fills.items()},
                                  in_sha=[sha(src)] + [sha(w) for w in ws] + [sha(b) for b in bs if b is not None]))

    U11 = dict(src=("U", (-1, 1)), w=("U", (-1, 1)), b=("U", (-1, 1)))
    U01 = dict(src=("U", (0, 1)), w=("U", (0, 1)), b=("U", (0, 1)))
    # BASELINE configs[0]: single-layer bf16 MLP 128x512 -> 256, bias, relu
    run_mlp("cfg1_mlp_bf16", 128, (512, 256), "bf16", (1,), "relu", U11)
    # scripts/correctness.sh:115 — f32 32 -> 16 -> 64 with bias, no activation, default fill U(0,1)
    run_mlp("mlp_f32_32x16x64", 32, (32, 16, 64), "f32", (1, 1), "noop", U01)
    # the two-layer graph of test/dnnl/resources/mpl.json in bf16 (128x512 -> 64 -> 256)
    run_mlp("mpl_json_bf16", 128, (512, 64, 256), "bf16", (1, 1), "relu", U11)
    # ragged, not a multiple of any tile
    run_mlp("mlp_bf16_ragged", 50, (72, 40), "bf16", (1,), "relu", U11)

    # scripts/correctness.sh:9 — bf16 matmul 32x128x64 with the matmul driver's sparse-integer fill
    for name, (M, K, N), dt in [("matmul_bf16_32x128x64", (32, 128, 64), "bf16"),
                                ("matmul_f32_64x96x48", (64, 96, 48), "f32")]:
        butil.set_seed(0)
        tdt = butil.get_dtype(dt)
        A = bmatmul.fill([M, K], tdt, ["src", dt, dt, dt, str(K)])
        B = bmatmul.fill([K, N], tdt, ["wei", dt, dt, dt, str(K)])
        (Cm,) = lmm.ref_matmul(_Cache(["a", "b"]), None, {"a": A, "b": B})
        arrays[name + "_a"], arrays[name + "_b"], arrays[name + "_out"] = bits(A), bits(B), bits(Cm)
        meta["cases"].append(dict(name=name, kind="matmul", M=M, K=K, N=N, dtype=dt))

    # --- 3. compare rule: verdicts of the reference's p2p on hand-made pairs -----------------
    refv = torch.tensor([1.0, 1.0, 1e-6, 1e-6, 0.0, float("nan"), float("inf"), -2.0, 100.0, 3e-5])
    resv = torch.tensor([1.009, 1.011, 2e-6, 0.02, 0.009, float("nan"), float("inf"), -2.03, 100.9, 3.1e-5])
    for thr in (1e-2, 5e-2, 1e-6):
        verdicts = []
        for i in range(refv.numel()):
            ok, _ = bcmp.p2p(thr, 100.0, refv[i : i + 1], resv[i : i + 1], 0)
            verdicts.append(bool(ok))
        meta["p2p"].append(dict(threshold=thr, verdicts=verdicts))
    arrays["p2p_ref"], arrays["p2p_res"] = refv.numpy(), resv.numpy()

    np.savez_compressed(os.path.join(HERE, "benchgc_golden.npz"), **arrays)
    with open(os.path.join(HERE, "benchgc_golden.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print("wrote", len(arrays), "arrays;", os.path.getsize(os.path.join(HERE, "benchgc_golden.npz")), "bytes")


if __name__ == "__main__":
    main()
