"""Failure paths on the GPU, exercised without faulting, trapping or hanging it: a bounded wait that nothing
satisfies runs out and reports through the device error word (the path every wait in the kernels takes when a
copy or a peer never answers), and a guard band of the workspace arena that lost its canary is detected after
the call.  The reference maps every run-time failure of an executable to dnnl_runtime_error
(src/dnnl/dnnl_graph_compiler.cpp:217-225)."""
import numpy as np
import pytest
import torch

import oracle
from _util import assert_bf16_close, tbits
from gc_b200 import api, lib, partitions
from gc_b200 import benchgc_compat as bc

pytestmark = pytest.mark.gpu


def _cfg1():
    A = bc.fill_tensor((128, 512), "bf16", "U", (-1, 1), 0)
    W = bc.fill_tensor((512, 256), "bf16", "U", (-1, 1), 1)
    b = bc.fill_tensor((256,), "bf16", "U", (-1, 1), 2)
    js, ins, out_id = partitions.mlp(128, (512, 256), "bf16", [True], "relu")
    want, acc = oracle.linear_bf16(tbits(A), tbits(W), tbits(b), relu=True, return_acc=True)
    return js, {0: A, 1: W, 2: b}, out_id, want, acc


def test_a_wait_that_runs_out_sets_the_error_word_and_the_next_execute_reports_it_once():
    assert lib.device_error() == 0
    js, ins, out_id, want, acc = _cfg1()
    exe = api.GraphCompiler().compile(js)
    out = torch.empty(128, 256, dtype=torch.bfloat16)
    exe.execute(ins, {out_id: out})                                  # healthy
    lib.wait_selftest(1_000_000)                                     # ~0.5 ms: waits on a counter nobody adds to, gives up
    torch.cuda.synchronize()
    with pytest.raises(api.DnnlError) as ei:                         # the word is read behind the results of the next call
        exe.execute(ins, {out_id: out})
    assert ei.value.status == api.RUNTIME_ERROR and "code 7" in str(ei.value)
    out.zero_()
    exe.execute(ins, {out_id: out})                                  # cleared: the context is intact and results are right
    assert_bf16_close(tbits(out), want, 512, what="after a reported time-out", pre=acc)
    assert lib.device_error() == 0
    # the direct launchers see the same word through gcb200_device_error
    lib.wait_selftest(200_000)
    assert lib.device_error() == 7 and lib.device_error() == 0
    with pytest.raises(lib.GcB200Error):
        lib.wait_selftest(10 ** 12)                                  # longer than the library's own limit: refused


def test_guard_bands_catch_a_damaged_canary(monkeypatch):
    monkeypatch.setenv("GC_B200_GUARD", "256")
    js, in_ids, out_id = partitions.mlp(256, (512, 1024, 256), "bf16", [True, True], "relu")
    exe = api.GraphCompiler().compile(js)
    monkeypatch.delenv("GC_B200_GUARD")
    assert "guard_bytes: 256" in exe.plan()
    g = torch.Generator().manual_seed(0)
    X = (torch.rand(256, 512, generator=g) * 2 - 1).bfloat16()
    Ws = [(torch.rand(512, 1024, generator=g) - 0.5).bfloat16(), (torch.rand(1024, 256, generator=g) - 0.5).bfloat16()]
    Bs = [(torch.rand(1024, generator=g) - 0.5).bfloat16(), (torch.rand(256, generator=g) - 0.5).bfloat16()]
    out = torch.empty(256, 256, dtype=torch.bfloat16)
    ins = dict(zip(in_ids, [X] + Ws + Bs))
    exe.execute(ins, {out_id: out})                                  # the kernels stay inside their slices
    assert exe.guard_check() == 0
    want = oracle.mlp_bf16(tbits(X), [tbits(w) for w in Ws], [tbits(b) for b in Bs], relu=True)
    assert_bf16_close(tbits(out), want, 1024, what="guarded arena", floor_div=1.0,
                      pre=np.abs(oracle.bf16_to_f32(want)) + np.abs(oracle.bf16_to_f32(tbits(Bs[1])))[None, :])
    exe.guard_selftest()                                             # one byte of a band loses its canary (host memset)
    assert exe.guard_check() == 1
    with pytest.raises(api.DnnlError) as ei:
        exe.execute(ins, {out_id: out})
    assert ei.value.status == api.RUNTIME_ERROR and "guard band" in str(ei.value) and "tensor" in str(ei.value)
    exe.execute(ins, {out_id: out})                                  # re-armed
    assert exe.guard_check() == 0
