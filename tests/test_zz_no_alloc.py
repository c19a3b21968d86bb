"""The allocation-free split-K matmul entry point, called through the C ABI.

Collected last on purpose: it is an add-on for hosts that cannot allocate device memory at run
time (a server whose own pool owns all of HBM, a thread that must not take the driver's allocation
lock), and a failure here should not hide the parity tests.  Works alone in a fresh process (its
first call does its own set-up) and after the other tests (which have created the library's
ordinary per-device state)."""
import ctypes as C

import pytest
import torch

import oracle
from _util import assert_bf16_close, tbits
from gc_b200 import lib

pytestmark = pytest.mark.gpu


def _static(A, B, bias, relu, splits):
    M, K = A.shape
    N = B.shape[1]
    Y = torch.empty(M, N, dtype=torch.bfloat16, device=A.device)
    st = lib.load().gcb200_matmul_bf16_splitk_static(A.data_ptr(), B.data_ptr(), None if bias is None else bias.data_ptr(),
                                                     Y.data_ptr(), M, N, K, splits, int(relu),
                                                     C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return st, Y


def test_static_scratch_matmul_matches_existing_entry_point_twice():
    g = torch.Generator().manual_seed(0)
    cases = [(16, 4096, 2048, 4), (128, 512, 1024, 2), (48, 1024, 4096, 0)]
    for call in range(2):                         # two calls in a row share the same static planes
        for M, N, K, splits in cases:
            A = (torch.rand(M, K, generator=g) * 2 - 1).bfloat16().cuda()
            B = (torch.rand(K, N, generator=g) * 2 - 1).bfloat16().cuda()
            bias = (torch.rand(N, generator=g) * 2 - 1).bfloat16().cuda()
            st, Y = _static(A, B, bias, True, splits)
            assert st == 0, lib.load().gcb200_last_error()
            torch.cuda.synchronize()
            code = C.c_int(-1)
            assert lib.load().gcb200_static_error(None, C.byref(code)) == 0 and code.value == 0
            want = lib.matmul_bf16(A, B, bias, relu=True)      # the existing entry point
            torch.cuda.synchronize()
            # same arithmetic, possibly a different split count: the tolerance of the parity tests
            acc = A.float() @ B.float()
            mx, same = assert_bf16_close(tbits(Y), tbits(want), K, what=f"static {M}x{N}x{K} call {call}", pre=acc.cpu().numpy())
            assert same > 0.99
            # and against the CPU oracle of the reference's arithmetic, like every other parity test
            want_o, acc_o = oracle.linear_bf16(tbits(A), tbits(B), tbits(bias), relu=True, return_acc=True)
            mx_o, same_o = assert_bf16_close(tbits(Y), want_o, K, what=f"static {M}x{N}x{K} call {call} vs oracle", pre=acc_o)
            assert same_o > 0.99
            if splits > 0:
                # with the same split count the two paths add the same planes in the same order
                cfg = lib.select_matmul_config(M, N, K, 2, 4, lib.sm_count())
                cfg.splits = splits
                ref = lib.matmul_bf16(A, B, bias, relu=True, cfg=cfg)
                torch.cuda.synchronize()
                assert torch.equal(Y, ref)


def test_static_scratch_rejects_oversized_requests():
    A = torch.zeros(2048, 64, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(64, 4096, dtype=torch.bfloat16, device="cuda")
    st, _ = _static(A, B, None, False, 1)        # 2048 * 4096 * 4 = 32 MiB > 16 MiB
    assert st == 1
    msg = lib.load().gcb200_last_error().decode()
    assert "exceeds the static scratch" in msg and "16777216" in msg
    # sizes whose byte count would wrap 64 bits are refused as well, not truncated (no memory is touched: the
    # check comes before any launch)
    st = lib.load().gcb200_matmul_bf16_splitk_static(A.data_ptr(), B.data_ptr(), None, A.data_ptr(), 1 << 40, 1 << 24, 64, 1, 0,
                                                     C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 1
