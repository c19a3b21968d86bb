"""Pin the CPU oracle: against the reference's own naive brgemm (oracle/_ref),
the closed-form tiles of the reference's brgemm lit tests, its C-API matmul test
and golden vectors produced by benchgc's torch evaluators."""
import numpy as np
import pytest
import torch

import oracle
from gc_b200 import benchgc_compat as bc

needs_ref = pytest.mark.skipif(not oracle.have_ref(), reason="oracle/_ref not built")


def tbits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def rnd_bf16(rng, shape, lo=-1.0, hi=1.0):
    return oracle.f32_to_bf16(rng.uniform(lo, hi, size=shape).astype(np.float32))


# ----------------------------------------------------------------------------- conversions
def test_bf16_rounding_matches_torch_rne():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(100000).astype(np.float32) * 10,
        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, np.inf, -np.inf, 1e-40], np.float32),
        # exact ties: bit 15 set, lower bits clear -> round to even
        np.array([0x3F808000, 0x3F818000, 0xBF808000], np.uint32).view(np.float32),
    ])
    got = oracle.f32_to_bf16(x)
    want = tbits(torch.from_numpy(x).to(torch.bfloat16))
    assert np.array_equal(got, want)
    # NaN maps to the canonical quiet NaN (BrgemmInterface.h:84-85)
    assert oracle.f32_to_bf16(np.array([np.nan], np.float32))[0] == 0x7FC0
    assert np.array_equal(oracle.bf16_to_f32(got), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


# ----------------------------------------------------------------------------- brgemm vs reference
DT = {"f32": oracle.DT_F32, "bf16": oracle.DT_BF16, "s8": oracle.DT_S8, "u8": oracle.DT_U8}


def _brgemm_inputs(rng, dta, dtb, M, N, K, bs):
    if dta == "f32":
        A = rng.uniform(-1, 1, (bs, M, K)).astype(np.float32)
        B = rng.uniform(-1, 1, (bs, K, N)).astype(np.float32)
        Bp, ldb, sb = B, N, K * N
        C0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    elif dta == "bf16":
        A = rnd_bf16(rng, (bs, M, K))
        B = rnd_bf16(rng, (bs, K, N))
        Bp = np.stack([oracle.pack_vnni(B[b], 2) for b in range(bs)])
        ldb, sb = N, Bp[0].size
        C0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    else:
        A = rng.integers(0, 256, (bs, M, K)).astype(np.uint8) if dta == "u8" else rng.integers(-128, 128, (bs, M, K)).astype(np.int8)
        B = rng.integers(0, 256, (bs, K, N)).astype(np.uint8) if dtb == "u8" else rng.integers(-128, 128, (bs, K, N)).astype(np.int8)
        Bp = np.stack([oracle.pack_vnni(B[b], 4) for b in range(bs)])
        ldb, sb = N, Bp[0].size
        C0 = rng.integers(-1000, 1000, (M, N)).astype(np.int32)
    return A, B, Bp, ldb, sb, C0


@needs_ref
@pytest.mark.parametrize("dta,dtb", [("f32", "f32"), ("bf16", "bf16"), ("u8", "s8"), ("s8", "s8"), ("s8", "u8"), ("u8", "u8")])
@pytest.mark.parametrize("beta", [0.0, 1.0])
@pytest.mark.parametrize("shape", [(32, 32, 32, 4), (8, 24, 14, 3), (5, 7, 9, 2)])
def test_brgemm_port_equals_reference_naive(dta, dtb, beta, shape):
    """The shapes/dtypes of test/mlir/unittests/ExecutionEngine/BrgemmRuntime.cpp:146-206 plus
    K tails; the restatement must equal the reference's naive kernel bit for bit."""
    M, N, K, bs = shape
    rng = np.random.default_rng(hash((dta, dtb, beta, shape)) % (2**32))
    A, B, Bp, ldb, sb, C0 = _brgemm_inputs(rng, dta, dtb, M, N, K, bs)
    c_port, c_ref = C0.copy(), C0.copy()
    args = (M, N, K, K, ldb, N, M * K, sb, beta, DT[dta], DT[dtb])
    assert oracle.brgemm(*args, A, 0, Bp, 0, c_port, 0, bs, backend="port") == 0
    oracle.brgemm(*args, A, 0, Bp, 0, c_ref, 0, bs, backend="ref")
    assert np.array_equal(c_port.view(np.uint32), c_ref.view(np.uint32))
    # and both equal a plain-layout contraction
    if dta in ("u8", "s8"):
        want = np.einsum("bmk,bkn->mn", A.astype(np.int64), B.astype(np.int64)) + (C0 if beta else 0)
        assert np.array_equal(c_port.astype(np.int64), want)


@pytest.mark.parametrize("backend", ["port", pytest.param("ref", marks=needs_ref)])
def test_known_answer_brgemm_parallel_f32(backend):
    """test/mlir/test/gc/cpu-runner/brgemm-parallel.mlir: A=1, B=2, batch 16 of 32x32x32,
    C0 = -64*i*j, beta=1, +3, ReLU  =>  every element of block (i,j) is max(0, 1027-64*i*j)."""
    A = np.ones((4, 16, 32, 32), np.float32)
    B = np.full((8, 16, 32, 32), 2.0, np.float32)
    for i in range(4):
        for j in range(8):
            Cb = np.full((32, 32), -64.0 * i * j, np.float32)
            oracle.brgemm(32, 32, 32, 32, 32, 32, 1024, 1024, 1.0, oracle.DT_F32, oracle.DT_F32,
                          A, i * 16 * 1024, B, j * 16 * 1024, Cb, 0, 16, backend=backend)
            out = np.maximum(Cb + 3.0, 0.0)
            assert np.all(out == max(0.0, 1027.0 - 64.0 * i * j)), (i, j)


@pytest.mark.parametrize("backend", ["port", pytest.param("ref", marks=needs_ref)])
def test_known_answer_brgemm_multilevel_bf16(backend):
    """test/mlir/test/gc/cpu-runner/brgemm-multilevel-for.mlir: bf16 A=1, VNNI B=2; after the
    4x8 sweep a second batch-2 brgemm accumulates onto block (i,0): 1027 + 2*32*1*2 = 1155."""
    one, two = oracle.f32_to_bf16(np.float32(1))[()], oracle.f32_to_bf16(np.float32(2))[()]
    A = np.full((4, 16, 32, 32), one, np.uint16)
    B = np.full((8, 16, 16, 32, 2), two, np.uint16)
    out = np.zeros((4, 8, 32, 32), np.float32)
    for i in range(4):
        for j in range(8):
            Cb = np.full((32, 32), -64.0 * i * j, np.float32)
            oracle.brgemm(32, 32, 32, 32, 32, 32, 1024, 1024, 1.0, oracle.DT_BF16, oracle.DT_BF16,
                          A, i * 16 * 1024, B, j * 16 * 1024, Cb, 0, 16, backend=backend)
            out[i, j] = np.maximum(Cb + 3.0, 0.0)
        Cb = out[i, 0].copy()
        oracle.brgemm(32, 32, 32, 32, 32, 32, 1024, 1024, 1.0, oracle.DT_BF16, oracle.DT_BF16,
                      A, i * 16 * 1024, B, i * 16 * 1024, Cb, 0, 2, backend=backend)
        out[i, 0] = Cb
    for i in range(4):
        assert np.all(out[i, 0] == 1155.0)
        for j in range(1, 8):
            assert np.all(out[i, j] == max(0.0, 1027.0 - 64.0 * i * j))


# ----------------------------------------------------------------------------- layers
@pytest.mark.parametrize("backend", ["port", pytest.param("ref", marks=needs_ref)])
@pytest.mark.parametrize("M,K,N", [(128, 512, 256), (64, 96, 160), (50, 72, 40)])
def test_linear_bf16_equals_brgemm_nest(backend, M, K, N):
    """The vectorisable (m,k,n) restatement and the block-by-block brgemm nest (driven through
    the reference's own microkernel when backend == 'ref') agree bit for bit, accumulators included."""
    rng = np.random.default_rng(M * 7 + N)
    A, W, b = rnd_bf16(rng, (M, K)), rnd_bf16(rng, (K, N)), rnd_bf16(rng, (N,))
    y1, acc1 = oracle.linear_bf16(A, W, b, relu=True, return_acc=True)
    y2, acc2 = oracle.linear_bf16_brgemm_nest(A, W, b, relu=True, backend=backend, return_acc=True)
    assert np.array_equal(acc1.view(np.uint32), acc2.view(np.uint32))
    assert np.array_equal(y1, y2)


def test_linear_bf16_transposes():
    rng = np.random.default_rng(3)
    A, W = rnd_bf16(rng, (40, 24)), rnd_bf16(rng, (24, 56))
    y = oracle.linear_bf16(A, W)
    assert np.array_equal(y, oracle.linear_bf16(np.ascontiguousarray(A.T), W, transA=True))
    assert np.array_equal(y, oracle.linear_bf16(A, np.ascontiguousarray(W.T), transB=True))


def test_matmul_f32_capi_case():
    """test/dnnl/TestApiOps.cpp:69-119: out = A^T.B + bias with A[i][j]=i+j, B[i][j]=i-j, bias[j]=j;
    all partial sums are integers below 2^24, so the f32 result is exact."""
    A = (np.arange(128)[:, None] + np.arange(512)[None, :]).astype(np.float32)
    B = (np.arange(128)[:, None] - np.arange(64)[None, :]).astype(np.float32)
    bias = np.arange(64, dtype=np.float32)
    got = oracle.matmul_f32(A, B, bias, transA=True)
    want = (A.astype(np.int64).T @ B.astype(np.int64) + bias.astype(np.int64)).astype(np.float32)
    assert got.shape == (512, 64) and np.array_equal(got, want)


@pytest.mark.parametrize("backend", ["port", pytest.param("ref", marks=needs_ref)])
def test_linear_u8s8_accumulators_exact(backend):
    rng = np.random.default_rng(11)
    M, K, N = 64, 256, 96
    A = rng.integers(0, 256, (M, K)).astype(np.uint8)
    W = rng.integers(-127, 128, (K, N)).astype(np.int8)
    scale = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    acc, out = oracle.linear_u8s8(A, W, scale, bias, zp_a=128)
    want = A.astype(np.int64) @ W.astype(np.int64)
    assert np.array_equal(acc.astype(np.int64), want)
    assert np.array_equal(acc, oracle.linear_u8s8_brgemm_nest(A, W, backend=backend))
    comp = 128 * W.astype(np.int64).sum(0)
    want_out = (want - comp).astype(np.float32) * scale + bias  # numpy: one fmul then one fadd in f32
    assert np.array_equal(out, want_out)


def test_reduce_epilogue_matches_single_pass_when_one_part():
    rng = np.random.default_rng(5)
    A, W, b = rnd_bf16(rng, (32, 64)), rnd_bf16(rng, (64, 48)), rnd_bf16(rng, (48,))
    y, acc = oracle.linear_bf16(A, W, b, relu=True, return_acc=True)
    assert np.array_equal(y, oracle.reduce_epilogue_bf16(acc[None], b, relu=True))


def test_softmax_and_attention_against_torch_f32():
    rng = np.random.default_rng(2)
    X = rng.standard_normal((17, 300)).astype(np.float32) * 3
    np.testing.assert_allclose(oracle.softmax_f32(X), torch.softmax(torch.from_numpy(X), -1).numpy(), rtol=2e-6, atol=1e-8)
    B, H, S, D = 2, 3, 70, 32
    q, k, v = (torch.randn(B, H, S, D, generator=torch.Generator().manual_seed(i)).bfloat16() for i in range(3))
    for causal in (False, True):
        o = oracle.attention_bf16(tbits(q), tbits(k), tbits(v), 1.0 / np.sqrt(D), causal)
        s = (q.float() @ k.float().transpose(-1, -2)) / np.sqrt(D)
        if causal:
            s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
        want = (torch.softmax(s, -1) @ v.float()).bfloat16()
        diff = (torch.from_numpy(oracle.bf16_to_f32(o)) - want.float()).abs().max().item()
        assert diff <= 2 ** -7  # at most one bf16 ulp of |O| <~ 2 from f32 summation order


# ----------------------------------------------------------------------------- golden vectors
def test_fill_matches_benchgc_golden(golden):
    meta, arrays = golden
    import hashlib

    for f in meta["fills"]:
        t = bc.fill_tensor(f["shape"], f["dtype"], f["fill_type"], f["fill_param"], f["idx"], seed=f["seed"])
        raw = tbits(t) if t.dtype == torch.bfloat16 else t.contiguous().numpy()
        assert np.array_equal(raw.reshape(-1)[:64], arrays[f["key"] + "_head"]), f
        assert hashlib.sha256(raw.tobytes()).hexdigest() == f["sha256"], f


def test_p2p_matches_benchgc_golden(golden):
    meta, arrays = golden
    ref, res = torch.from_numpy(arrays["p2p_ref"]), torch.from_numpy(arrays["p2p_res"])
    for case in meta["p2p"]:
        got = [bc.p2p(case["threshold"], 100.0, ref[i : i + 1], res[i : i + 1])[0] for i in range(ref.numel())]
        assert got == case["verdicts"], case


def _mlp_inputs(case):
    nl = len(case["hidden"]) - 1
    f = case["fills"]
    src = bc.fill_tensor((case["batch"], case["hidden"][0]), case["dtype"], f["src"][0], f["src"][1], 0, case["seed"])
    ws = [bc.fill_tensor((case["hidden"][i], case["hidden"][i + 1]), case["dtype"], f["w"][0], f["w"][1], 1 + i, case["seed"]) for i in range(nl)]
    bs, j = [], 0
    for i in range(nl):
        if case["has_bias"][i]:
            bs.append(bc.fill_tensor((case["hidden"][i + 1],), case["dtype"], f["b"][0], f["b"][1], 1 + nl + j, case["seed"]))
            j += 1
        else:
            bs.append(None)
    return src, ws, bs


def test_oracle_mlp_against_benchgc_reference_outputs(golden):
    """benchgc's torch evaluators (torch.mm -> add -> max, each rounding to bf16) on the same seeded
    inputs: the oracle must agree within the reference's own mlp thresholds (pattern/mlp.py:161-173)
    and within BASELINE's 1e-2 for the bf16 cases; differences come from f32 summation order only."""
    meta, arrays = golden
    for case in [c for c in meta["cases"] if c["kind"] == "mlp"]:
        src, ws, bs = _mlp_inputs(case)
        want = arrays[case["name"] + "_out"]
        relu = case["act"] == "relu"
        if case["dtype"] == "bf16":
            h = tbits(src)
            for W, b in zip(ws, bs):
                h = oracle.linear_bf16(h, tbits(W), None if b is None else tbits(b), relu=relu)
            got = torch.from_numpy(oracle.bf16_to_f32(h))
            ref = torch.from_numpy(oracle.bf16_to_f32(want))
            ok, _ = bc.p2p(1e-2, 100.0, ref, got)
            # elements whose accumulator sits next to zero may differ by summation-order noise only
            near0 = ((ref - got).abs() <= 1e-5 * np.sqrt(max(case["hidden"])) * 8)
            rel_ok = ((ref - got).abs() <= 1e-2 * ref.abs()) | near0
            assert bool(rel_ok.all()), case["name"]
            assert (got != ref).float().mean().item() < 0.02, case["name"]  # >98 % bit-identical
        else:
            h = src.numpy()
            for W, b in zip(ws, bs):
                h = oracle.matmul_f32(h, W.numpy(), None if b is None else b.numpy(), relu=relu)
            ok, _ = bc.p2p(1e-5, 100.0, torch.from_numpy(want), torch.from_numpy(h))
            assert ok, case["name"]


def test_oracle_matmul_against_benchgc_integer_fill(golden):
    """scripts/correctness.sh:9 form: the matmul driver fills sparse small integers so that every
    partial sum is exact — the oracle must be bit-identical to benchgc's torch.mm."""
    meta, arrays = golden
    for case in [c for c in meta["cases"] if c["kind"] == "matmul"]:
        A, B, want = (arrays[case["name"] + s] for s in ("_a", "_b", "_out"))
        if case["dtype"] == "bf16":
            assert np.array_equal(oracle.linear_bf16(A, B), want)
        else:
            assert np.array_equal(oracle.matmul_f32(A, B), want)
