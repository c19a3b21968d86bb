"""Parity of the CUDA matmul kernels with the CPU oracle, through the C ABI.
bf16: within rtol 1e-2 (max abs error printed per case); int8: s32 accumulators bit-exact."""
import numpy as np
import pytest
import torch

import oracle
from _util import assert_bf16_close, from_bits, tbits
from gc_b200 import benchgc_compat as bc
from gc_b200 import lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand_bf16(shape, seed, lo=-1.0, hi=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(shape, generator=g) * (hi - lo) + lo).bfloat16()


def _no_device_error():
    assert lib.device_error() == 0


@pytest.mark.parametrize("M,N,K,ta,tb,bias,relu", [
    (128, 256, 512, 0, 0, 1, 1),     # BASELINE configs[0]
    (128, 256, 64, 0, 0, 0, 0),      # one tile, one K block
    (256, 512, 192, 0, 1, 1, 0),     # transpose_b: K-major weights
    (192, 320, 256, 1, 0, 1, 1),     # transpose_a: MN-major activations
    (200, 328, 136, 0, 0, 1, 1),     # ragged in M, N and K
    (50, 72, 40, 0, 0, 1, 1),        # smaller than one tile (swapped orientation)
    (16, 512, 1024, 0, 0, 1, 1),     # decode-shaped: swapped + split-K
    (48, 1024, 512, 0, 1, 0, 1),
    (1024, 1024, 1024, 0, 0, 1, 1),  # several waves of tiles
    (130, 36, 100, 0, 0, 1, 0),      # rows not 16-byte aligned: exact-order SIMT path
    (1, 8, 8, 0, 0, 0, 0),
])
def test_matmul_bf16_matches_oracle(M, N, K, ta, tb, bias, relu):
    A, B, b = _rand_bf16((M, K), 1), _rand_bf16((K, N), 2), _rand_bf16((N,), 3)
    Ad = (A.t().contiguous() if ta else A).to(DEV)
    Bd = (B.t().contiguous() if tb else B).to(DEV)
    Y = lib.matmul_bf16(Ad, Bd, b.to(DEV) if bias else None, bool(relu), bool(ta), bool(tb))
    torch.cuda.synchronize()
    _no_device_error()
    want, acc = oracle.linear_bf16(tbits(A), tbits(B), tbits(b) if bias else None, relu=bool(relu), return_acc=True)
    mx, same = assert_bf16_close(tbits(Y), want, K, what=f"{M}x{N}x{K}", pre=acc if bias else None)
    print(f"matmul_bf16 {M}x{N}x{K} ta={ta} tb={tb}: max_abs={mx:.4g} bit-identical={same:.5f}")
    assert same > 0.99


def test_cfg1_against_benchgc_golden_output(golden):
    """BASELINE configs[0] on benchgc's own seeded inputs, against the output of benchgc's torch
    evaluators (committed fixture) and against the oracle."""
    meta, arrays = golden
    case = next(c for c in meta["cases"] if c["name"] == "cfg1_mlp_bf16")
    f = case["fills"]
    A = bc.fill_tensor((128, 512), "bf16", f["src"][0], f["src"][1], 0)
    W = bc.fill_tensor((512, 256), "bf16", f["w"][0], f["w"][1], 1)
    b = bc.fill_tensor((256,), "bf16", f["b"][0], f["b"][1], 2)
    Y = lib.matmul_bf16(A.to(DEV), W.to(DEV), b.to(DEV), relu=True)
    torch.cuda.synchronize()
    want, acc = oracle.linear_bf16(tbits(A), tbits(W), tbits(b), relu=True, return_acc=True)
    mx, same = assert_bf16_close(tbits(Y), want, 512, what="cfg1 vs oracle", pre=acc)
    mx2, same2 = assert_bf16_close(tbits(Y), arrays["cfg1_mlp_bf16_out"], 512, what="cfg1 vs benchgc torch reference", pre=acc)
    ok, _ = bc.p2p(5e-2, 100.0, from_bits(arrays["cfg1_mlp_bf16_out"]), Y.cpu())  # the reference's own mlp threshold
    assert ok
    print(f"cfg1: vs oracle max_abs={mx:.4g} identical={same:.5f}; vs benchgc max_abs={mx2:.4g} identical={same2:.5f}")


def test_forced_tile_configurations_agree():
    """Every tile shape / split / pipeline depth computes the same layer."""
    M, N, K = 384, 512, 1024
    A, B, b = _rand_bf16((M, K), 4), _rand_bf16((K, N), 5), _rand_bf16((N,), 6)
    want, acc = oracle.linear_bf16(tbits(A), tbits(B), tbits(b), relu=True, return_acc=True)
    Ad, Bd, bd = A.to(DEV), B.to(DEV), b.to(DEV)
    for swapped, bn, splits, stages, gm in [(0, 256, 1, 4, 8), (0, 128, 1, 6, 1), (0, 64, 1, 8, 3), (0, 256, 4, 2, 8),
                                            (0, 128, 16, 3, 2), (0, 192, 1, 3, 8),
                                            # widths that are not a whole number of 64-column slabs: the last 16, 32 or
                                            # 48 columns of every tile take the register-store tail of the epilogue
                                            (0, 224, 1, 4, 8), (0, 240, 2, 3, 8), (0, 112, 1, 4, 2), (0, 80, 1, 4, 8),
                                            (0, 208, 4, 3, 1), (0, 176, 1, 4, 8)]:
        cfg = lib.MatmulConfig(swapped, bn, splits, stages, gm, 0)
        Y = lib.matmul_bf16(Ad, Bd, bd, relu=True, cfg=cfg)
        torch.cuda.synchronize()
        _no_device_error()
        assert_bf16_close(tbits(Y), want, K, what=repr(cfg), pre=acc)
        if bn % 128 == 0:
            # the same tile on a CTA pair (256 x bn over two SMs): same MMAs in the same order per output element
            cfg2 = lib.MatmulConfig(swapped, bn, splits, stages, gm, 0, 1, 0)
            Y2 = lib.matmul_bf16(Ad, Bd, bd, relu=True, cfg=cfg2)
            torch.cuda.synchronize()
            _no_device_error()
            assert torch.equal(Y2, Y), repr(cfg2)
        # K-major weights ([N, K]) walk the same tiles through the other operand layout
        Yt = lib.matmul_bf16(Ad, Bd.t().contiguous(), bd, relu=True, transpose_b=True, cfg=cfg)
        torch.cuda.synchronize()
        _no_device_error()
        assert torch.equal(Yt, Y), repr(cfg)


def test_f32out_and_reduce_epilogue_match_k_split_rule():
    """Row-parallel form: two K halves -> f32 partial sums -> reduce -> cast -> bias -> ReLU."""
    M, N, K = 256, 384, 1024
    A, B, b = _rand_bf16((M, K), 7), _rand_bf16((K, N), 8), _rand_bf16((N,), 9)
    Ad, Bd = A.to(DEV), B.to(DEV)
    parts = torch.stack([lib.matmul_bf16_f32out(Ad[:, :512].contiguous(), Bd[:512].contiguous()),
                         lib.matmul_bf16_f32out(Ad[:, 512:].contiguous(), Bd[512:].contiguous())])
    Y = lib.reduce_bias_act_bf16(parts, b.to(DEV), relu=True)
    torch.cuda.synchronize()
    _, acc0 = oracle.linear_bf16(tbits(A[:, :512].contiguous()), tbits(B[:512].contiguous()), return_acc=True)
    _, acc1 = oracle.linear_bf16(tbits(A[:, 512:].contiguous()), tbits(B[512:].contiguous()), return_acc=True)
    np.testing.assert_allclose(parts[0].cpu().numpy(), acc0, rtol=1e-5, atol=1e-5)
    want = oracle.reduce_epilogue_bf16(np.stack([acc0, acc1]), tbits(b), relu=True)
    assert_bf16_close(tbits(Y), want, K, what="k-split", pre=acc0 + acc1)
    # the reduction + epilogue itself is deterministic: feed it the oracle's partial sums
    Y2 = lib.reduce_bias_act_bf16(torch.from_numpy(np.stack([acc0, acc1])).to(DEV), b.to(DEV), relu=True)
    assert np.array_equal(tbits(Y2), want)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 384), (100, 208, 80), (16, 512, 1024), (1024, 4096, 4096)])
def test_matmul_u8s8_bit_exact(M, N, K):
    """s32 accumulators bit-exact; the dequantised output equals the oracle's bit for bit too
    (separate fmul and fadd on both sides).  The last case is BASELINE configs[1] at full size."""
    g = torch.Generator().manual_seed(M + N)
    A = torch.randint(0, 256, (M, K), generator=g, dtype=torch.uint8)
    W = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    scale = torch.rand(N, generator=g) * 0.009 + 0.001
    bias = torch.rand(N, generator=g) * 2 - 1
    Wd = W.to(DEV)
    comp = lib.colsum_s8(Wd, 128)
    out, acc = lib.matmul_u8s8(A.to(DEV), Wd, scale.to(DEV), bias.to(DEV), comp, want_acc=True)
    torch.cuda.synchronize()
    _no_device_error()
    wacc, wout = oracle.linear_u8s8(A.numpy(), W.numpy(), scale.numpy(), bias.numpy(), zp_a=128)
    assert np.array_equal(acc.cpu().numpy(), wacc)
    assert np.array_equal(out.cpu().numpy(), wout)
    _, acc_only = lib.matmul_u8s8(A.to(DEV), Wd)
    assert np.array_equal(acc_only.cpu().numpy(), wacc)


def test_matmul_u8s8_on_cta_pairs_bit_exact():
    """The CTA-pair kernel on u8 x s8 (the selector's choice for several waves of tiles, forced here on a small shape
    through the measured-configuration cache): s32 accumulators and dequantised output bit-identical to the oracle."""
    M, N, K = 512, 1024, 2048
    g = torch.Generator().manual_seed(77)
    A = torch.randint(0, 256, (M, K), generator=g, dtype=torch.uint8)
    W = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    scale = torch.rand(N, generator=g) * 0.009 + 0.001
    bias = torch.rand(N, generator=g) * 2 - 1
    Wd = W.to(DEV)
    comp = lib.colsum_s8(Wd, 128)
    saved = lib.tune_cache_get(M, N, K, 1, 4)
    try:
        lib.tune_cache_put(M, N, K, lib.MatmulConfig(0, 256, 1, 8, 8, 0, 1, 1), 1, 4)
        out, acc = lib.matmul_u8s8(A.to(DEV), Wd, scale.to(DEV), bias.to(DEV), comp, want_acc=True)
        out_tma, _ = lib.matmul_u8s8(A.to(DEV), Wd, scale.to(DEV), bias.to(DEV), comp)   # copy-engine epilogue
        torch.cuda.synchronize()
        _no_device_error()
    finally:
        if saved is not None:
            lib.tune_cache_put(M, N, K, saved, 1, 4)
        else:
            lib.tune_cache_erase(M, N, K, 1, 4)
    wacc, wout = oracle.linear_u8s8(A.numpy(), W.numpy(), scale.numpy(), bias.numpy(), zp_a=128)
    assert np.array_equal(acc.cpu().numpy(), wacc)
    assert np.array_equal(out.cpu().numpy(), wout)
    assert np.array_equal(out_tma.cpu().numpy(), wout)


def test_matmul_f32_capi_case():
    """test/dnnl/TestApiOps.cpp:69-119 values."""
    A = (torch.arange(128)[:, None] + torch.arange(512)[None, :]).float()
    B = (torch.arange(128)[:, None] - torch.arange(64)[None, :]).float()
    bias = torch.arange(64).float()
    Y = lib.matmul_f32(A.to(DEV), B.to(DEV), bias.to(DEV), transpose_a=True)
    want = oracle.matmul_f32(A.numpy(), B.numpy(), bias.numpy(), transA=True)
    assert np.array_equal(Y.cpu().numpy(), want)
    # general data: same accumulation order as the oracle -> bit-identical
    g = torch.Generator().manual_seed(0)
    A, B = torch.randn(70, 90, generator=g), torch.randn(90, 50, generator=g)
    Y = lib.matmul_f32(A.to(DEV), B.to(DEV), relu=True)
    assert np.array_equal(Y.cpu().numpy(), oracle.matmul_f32(A.numpy(), B.numpy(), relu=True))


def test_full_size_gemm_rows_against_oracle():
    """BASELINE configs[4] at 8192^3: a random subset of output rows is recomputed by the oracle
    (rows of a matmul are independent), plus linearity C(A1+A2) == C(A1)+C(A2) on exact data."""
    N = 8192
    A, B = _rand_bf16((N, N), 10).to(DEV), _rand_bf16((N, N), 11).to(DEV)
    Y = lib.matmul_bf16(A, B)
    torch.cuda.synchronize()
    _no_device_error()
    rows = torch.randperm(N, generator=torch.Generator().manual_seed(0))[:64].sort().values
    want = oracle.linear_bf16(tbits(A[rows]), tbits(B))
    mx, same = assert_bf16_close(tbits(Y[rows]), want, N, what="8192^3 row subset")
    print(f"gemm 8192^3 rows: max_abs={mx:.4g} bit-identical={same:.5f}")
    # exact-arithmetic property: small integers -> every partial sum exact -> bit-identical to any order
    Ai = torch.randint(-2, 3, (512, 4096), generator=torch.Generator().manual_seed(1)).bfloat16().to(DEV)
    Bi = torch.randint(-2, 3, (4096, 2048), generator=torch.Generator().manual_seed(2)).bfloat16().to(DEV)
    Yi = lib.matmul_bf16(Ai, Bi)
    assert torch.equal(Yi.float(), (Ai.float() @ Bi.float()).bfloat16().float())


@pytest.mark.parametrize("n,rows", [(2048, 64), (4096, 48), (16384, 24)])
def test_gemm_sweep_sizes_rows_against_oracle(n, rows):
    """BASELINE configs[4] at 2048^3, 4096^3 and 16384^3 (with 1024^3 and 8192^3 above, the whole square sweep):
    a random subset of output rows recomputed by the oracle, spread so that the first and the last tile row,
    the last wave and (at 16384^3: 2^28 outputs, 512 MiB per operand) the largest offsets are all hit."""
    A, B = _rand_bf16((n, n), 20 + n % 7).to(DEV), _rand_bf16((n, n), 21 + n % 5).to(DEV)
    Y = lib.matmul_bf16(A, B)
    torch.cuda.synchronize()
    _no_device_error()
    pick = torch.randperm(n, generator=torch.Generator().manual_seed(n))[: rows - 2]
    idx = torch.cat([torch.tensor([0, n - 1]), pick]).unique().sort().values
    want = oracle.linear_bf16(tbits(A[idx]), tbits(B))
    mx, same = assert_bf16_close(tbits(Y[idx]), want, n, what=f"{n}^3 row subset")
    print(f"gemm {n}^3, {len(idx)} rows: max_abs={mx:.4g} bit-identical={same:.5f}")
    assert same > 0.99
    # every output was written (no tile skipped): the finite, non-zero check costs one pass on the device
    assert bool(torch.isfinite(Y.float()).all()) and int((Y == 0).sum()) < n


def test_decode_shape_against_oracle():
    """BASELINE configs[4] decode shape M=16, K=8192, N=28672 (weights streamed once)."""
    M, K, N = 16, 8192, 28672
    A, B = _rand_bf16((M, K), 12), _rand_bf16((K, N), 13)
    Y = lib.matmul_bf16(A.to(DEV), B.to(DEV))
    torch.cuda.synchronize()
    _no_device_error()
    want = oracle.linear_bf16(tbits(A), tbits(B))
    mx, same = assert_bf16_close(tbits(Y), want, K, what="decode")
    print(f"decode 16x28672x8192: max_abs={mx:.4g} bit-identical={same:.5f}")


# ----------------------------------------------------------------------------- brgemm runtime ABI
DT = {"f32": 3, "bf16": 2, "s8": 5, "u8": 6}


@pytest.mark.parametrize("dta,dtb", [("f32", "f32"), ("bf16", "bf16"), ("u8", "s8"), ("s8", "s8"), ("s8", "u8"), ("u8", "u8")])
@pytest.mark.parametrize("beta", [0.0, 1.0])
def test_brgemm_abi_matches_reference_naive(dta, dtb, beta):
    """The pattern of test/mlir/unittests/ExecutionEngine/BrgemmRuntime.cpp:58-144 with the device
    implementation of dnnl_brgemm_* on one side and the reference's naive kernel (or its restatement
    when oracle/_ref is absent) on the other: f32/bf16 within rtol 1e-4 + atol 1e-6 (in fact
    bit-identical: same accumulation chain), int8 exactly equal."""
    M = N = K = 32
    bs = 4
    rng = np.random.default_rng(7)
    if dta == "f32":
        A = rng.uniform(-1, 1, (bs, M, K)).astype(np.float32)
        Bp = rng.uniform(-1, 1, (bs, K, N)).astype(np.float32)
        C0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    elif dta == "bf16":
        A = oracle.f32_to_bf16(rng.uniform(-1, 1, (bs, M, K)).astype(np.float32))
        Bp = np.stack([oracle.pack_vnni(oracle.f32_to_bf16(rng.uniform(-1, 1, (K, N)).astype(np.float32)), 2) for _ in range(bs)])
        C0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    else:
        A = (rng.integers(0, 256, (bs, M, K)).astype(np.uint8) if dta == "u8" else rng.integers(-128, 128, (bs, M, K)).astype(np.int8))
        Bq = (rng.integers(0, 256, (bs, K, N)).astype(np.uint8) if dtb == "u8" else rng.integers(-128, 128, (bs, K, N)).astype(np.int8))
        Bp = np.stack([oracle.pack_vnni(Bq[b], 4) for b in range(bs)])
        C0 = rng.integers(-1000, 1000, (M, N)).astype(np.int32)
    args = (M, N, K, K, N, N, M * K, Bp[0].size, beta, DT[dta], DT[dtb])
    want = C0.copy()
    oracle.brgemm(*args, A, 0, Bp, 0, want, 0, bs, backend="ref" if oracle.have_ref() else "port")
    l = lib.load()
    h = l.dnnl_brgemm_dispatch(*args)
    Ad, Bd, Cd = (torch.from_numpy(x.view(np.int16) if x.dtype == np.uint16 else x).to(DEV) for x in (A, Bp, C0))
    l.dnnl_brgemm_tileconfig(h)
    l.dnnl_brgemm_execute(h, Ad.data_ptr(), 0, Bd.data_ptr(), 0, Cd.data_ptr(), 0, bs)
    l.dnnl_brgemm_tilerelease()
    torch.cuda.synchronize()
    got = Cd.cpu().numpy()
    if dta in ("f32", "bf16"):
        np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-6)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    else:
        assert np.array_equal(got, want)


def test_brgemm_abi_known_answer_tiles():
    """test/mlir/test/gc/cpu-runner/brgemm-parallel.mlir: every element of block (i,j) = max(0, 1027-64ij)."""
    l = lib.load()
    A = torch.ones(4, 16, 32, 32, device=DEV)
    B = torch.full((8, 16, 32, 32), 2.0, device=DEV)
    h = l.dnnl_brgemm_dispatch(32, 32, 32, 32, 32, 32, 1024, 1024, 1.0, 3, 3)
    for i in range(4):
        for j in range(8):
            Cb = torch.full((32, 32), -64.0 * i * j, device=DEV)
            l.dnnl_brgemm_execute(h, A.data_ptr(), i * 16 * 1024, B.data_ptr(), j * 16 * 1024, Cb.data_ptr(), 0, 16)
            torch.cuda.synchronize()
            assert bool((torch.relu(Cb + 3.0) == max(0.0, 1027.0 - 64.0 * i * j)).all())
