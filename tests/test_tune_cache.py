"""Measured-configuration cache of the matmul tile selector: host logic (no device needed) and, on a GPU, the
tuner that fills it."""
import os
import subprocess
import sys

import numpy as np
import pytest

from gc_b200 import lib, tune


@pytest.fixture(autouse=True)
def _clean_cache():
    lib.tune_cache_clear()
    yield
    lib.tune_cache_clear()


def _cfg(c):
    return (c.swapped, c.bn, c.splits, c.stages, c.group_m, c.grid, c.pair, c.kpb)


def test_a_recorded_configuration_beats_the_model_for_exactly_that_shape():
    model = lib.select_matmul_config(512, 4096, 16384)
    assert _cfg(model) == _cfg(lib.model_matmul_config(512, 4096, 16384))
    mine = lib.MatmulConfig(0, 128, 4, 3, 8, 148, 0, 2)
    lib.tune_cache_put(512, 4096, 16384, mine)
    assert _cfg(lib.select_matmul_config(512, 4096, 16384)) == _cfg(mine)
    assert _cfg(lib.model_matmul_config(512, 4096, 16384)) == _cfg(model)          # the model itself is untouched
    assert _cfg(lib.select_matmul_config(512, 4096, 8192)) == _cfg(lib.model_matmul_config(512, 4096, 8192))
    assert _cfg(lib.select_matmul_config(512, 4096, 16384, 1, 4)) == _cfg(lib.model_matmul_config(512, 4096, 16384, 1, 4))
    lib.tune_cache_erase(512, 4096, 16384)
    assert lib.tune_cache_get(512, 4096, 16384) is None
    assert _cfg(lib.select_matmul_config(512, 4096, 16384)) == _cfg(model)


def test_grid_is_fitted_to_the_device_that_asks():
    lib.tune_cache_put(8192, 8192, 8192, lib.MatmulConfig(0, 256, 1, 4, 8, 148, 0, 1))
    assert lib.select_matmul_config(8192, 8192, 8192, sms=132).grid == 132


def test_configurations_no_kernel_can_run_are_rejected():
    for bad in (lib.MatmulConfig(0, 100, 1, 4, 8, 148, 0, 1),    # tile width not a multiple of 32
                lib.MatmulConfig(0, 512, 1, 4, 8, 148, 0, 1),    # wider than one MMA
                lib.MatmulConfig(0, 256, 0, 4, 8, 148, 0, 1),    # no K split factor
                lib.MatmulConfig(0, 256, 1, 1, 8, 148, 0, 1),    # a one-stage ring
                lib.MatmulConfig(1, 128, 1, 4, 8, 148, 0, 1)):   # weight-stationary form holds at most 64 batch rows
        with pytest.raises(RuntimeError):
            lib.tune_cache_put(1024, 1024, 1024, bad)
    with pytest.raises(RuntimeError):
        lib.tune_cache_put(0, 1024, 1024, lib.MatmulConfig(0, 256, 1, 4, 8, 148, 0, 1))
    # a weight-stationary entry is ignored for a batch it cannot hold
    lib.tune_cache_put(512, 1024, 1024, lib.MatmulConfig(1, 64, 1, 4, 8, 8, 0, 2))
    assert lib.select_matmul_config(512, 1024, 1024).swapped == 0


def test_save_and_load_round_trip(tmp_path):
    a, b = lib.MatmulConfig(0, 128, 4, 3, 8, 148, 0, 2), lib.MatmulConfig(1, 16, 2, 8, 8, 148, 0, 2)
    lib.tune_cache_put(512, 4096, 16384, a)
    lib.tune_cache_put(16, 28672, 8192, b)
    lib.tune_cache_put(1024, 4096, 4096, a, 1, 4)
    path = str(tmp_path / "matmul.tune")
    assert lib.tune_cache_save(path) == 3
    lib.tune_cache_clear()
    assert lib.tune_cache_get(512, 4096, 16384) is None
    assert lib.tune_cache_load(path) == 3
    assert _cfg(lib.tune_cache_get(512, 4096, 16384)) == _cfg(a)
    assert _cfg(lib.tune_cache_get(16, 28672, 8192)) == _cfg(b)
    assert _cfg(lib.tune_cache_get(1024, 4096, 4096, 1, 4)) == _cfg(a)
    assert lib.tune_cache_get(1024, 4096, 4096) is None                  # dtype and output width are part of the key


def test_malformed_files_are_reported_with_their_line(tmp_path):
    path = tmp_path / "bad.tune"
    path.write_text("# comment\n\n512 4096 16384 2 2 : 0 128 4 3 8 148 0 2   # fine\n512 4096 : 0 128\n")
    with pytest.raises(RuntimeError, match="line 4"):
        lib.tune_cache_load(str(path))
    with pytest.raises(RuntimeError, match="cannot open"):
        lib.tune_cache_load(str(tmp_path / "missing.tune"))


def test_the_environment_variable_names_the_file_read_at_first_use(tmp_path):
    path = tmp_path / "env.tune"
    path.write_text("256 512 1024 2 2 : 0 64 2 3 8 16 0 2\n")
    code = ("import sys; sys.path.insert(0, %r); from gc_b200 import lib; c = lib.select_matmul_config(256, 512, 1024); "
            "print(c.bn, c.splits, c.kpb)" % os.path.join(os.path.dirname(__file__), "..", "graph-compiler_b200"))
    env = dict(os.environ, GC_B200_TUNE_CACHE=str(path))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, check=True).stdout.split()
    assert out == ["64", "2", "2"]
    env["GC_B200_TUNE_CACHE"] = str(tmp_path / "not-there-yet.tune")       # a missing file is an empty cache
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, check=True).stdout.split()
    m = lib.model_matmul_config(256, 512, 1024)
    assert out == [str(m.bn), str(m.splits), str(m.kpb)]


def test_candidates_start_with_the_model_and_respect_the_kernels_limits():
    for shape in ((512, 4096, 16384, 2, 2), (16, 28672, 8192, 2, 2), (1024, 4096, 4096, 1, 4), (128, 256, 512, 2, 2)):
        cands = tune.candidates(*shape)
        M, N, K, eb, ob = shape
        assert _cfg(cands[0]) == _cfg(lib.model_matmul_config(*shape))
        assert len({(c.bn, c.splits, c.kpb, c.pair) for c in cands}) == len(cands)
        k_blocks = -(-K // (128 // eb))
        for c in cands[1:]:
            assert c.swapped == cands[0].swapped and 1 <= c.grid <= 148
            assert c.splits == 1 or (k_blocks >= 16 * c.splits and -(-k_blocks // c.splits) % max(1, c.kpb) == 0)
            assert c.kpb == 1 or c.swapped or c.bn <= 128
            lib.tune_cache_put(M, N, K, c, eb, ob)         # every candidate passes the cache's own validation


@pytest.mark.gpu
def test_tuner_records_a_configuration_that_still_matches_the_oracle():
    import torch

    import oracle
    from _util import assert_bf16_close, tbits

    M, N, K = 256, 1024, 4096
    best, us, results = tune.tune_matmul(M, N, K, iters=3)
    assert best is not None and us > 0 and len(results) >= 4
    assert all(t != t or t > 0 for _, t in results)
    assert _cfg(lib.tune_cache_get(M, N, K)) == _cfg(best) == _cfg(lib.select_matmul_config(M, N, K))
    g = torch.Generator().manual_seed(11)
    A = (torch.rand(M, K, generator=g) * 2 - 1).bfloat16()
    B = (torch.rand(K, N, generator=g) * 2 - 1).bfloat16()
    want, acc = oracle.linear_bf16(tbits(A), tbits(B), None, relu=False, return_acc=True)
    Y = lib.matmul_bf16(A.cuda(), B.cuda())
    torch.cuda.synchronize()
    assert lib.device_error() == 0
    assert_bf16_close(tbits(Y), want, K, what="tuned configuration", pre=acc)
    # every timed candidate also computes the same thing
    for c in tune.candidates(M, N, K)[:6]:
        Yc = lib.matmul_bf16(A.cuda(), B.cuda(), cfg=c)
        torch.cuda.synchronize()
        assert_bf16_close(tbits(Yc), want, K, what=f"candidate {c}", pre=acc)
    assert lib.device_error() == 0
