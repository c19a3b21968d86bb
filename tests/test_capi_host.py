"""Host-side tests of the C ABI: the library loads and exports what the headers
declare, the JSON reader accepts/rejects what the reference's reader does
(status classes of src/dnnl/dnnl_graph_compiler.cpp:193-206), the launch plan
fuses post-ops, the arena planner never overlaps live buffers.  No GPU needed —
compile is host-only, like the reference's."""
import ctypes as C
import json
import os
import re

import pytest

from gc_b200 import api, lib, partitions

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout: GC_REFERENCE_DIR, else a directory named "reference" beside this repository; the test
# that reads it is skipped where neither exists
REF_JSON = os.path.join(os.environ.get("GC_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference"),
                        "test", "dnnl", "resources")


def test_library_exports_every_declared_symbol():
    l = lib.load()
    declared = set()
    for h in ("gc_b200.h", "dnnl_graph_compiler.h"):
        src = open(os.path.join(ROOT, "include", h)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        declared |= set(re.findall(r"\b((?:gcb200|dnnl_graph_compiler|dnnl_brgemm)_\w+)\s*\(", src))
    assert len(declared) >= 20
    for name in sorted(declared):
        assert hasattr(l, name), f"{name} is declared but not exported"


def test_version():
    apiv, gcv = api.get_version()
    assert apiv[:3] == (0, 1, 0)
    assert all(x != 255 for x in gcv[:3])  # test/dnnl/TestApiBasic.cpp:69-72


def test_create_accepts_null_context_and_compile_is_host_only():
    gc = api.GraphCompiler()          # ctx == NULL, as test/dnnl/TestApiOps.cpp:45
    gc4 = api.GraphCompiler(num_threads=4)
    js, ins, out = partitions.mlp(128, (512, 256))
    exe = gc.compile(js)
    assert "MatMul+ReLU" in exe.plan()
    exe.destroy(); gc.destroy(); gc4.destroy()


def _status(js):
    gc = api.GraphCompiler()
    try:
        gc.compile(js).destroy()
        return api.SUCCESS
    except api.DnnlError as e:
        return e.status
    finally:
        gc.destroy()


def _base():
    return json.loads(partitions.mlp(8, (16, 8))[0])


def test_error_classes_follow_the_reference_reader():
    assert _status(json.dumps(_base())) == api.SUCCESS
    g = _base(); g["bogus"] = 1
    assert _status(json.dumps(g)) == api.INVALID_GRAPH            # unrecognised key (JsonParser.cpp:70)
    g = _base(); g["graph"][0]["kind"] = "Convolution"
    assert _status(json.dumps(g)) == api.UNIMPLEMENTED            # unsupported op (JsonParser.cpp:155)
    g = _base(); g["engine_kind"] = "fpga"
    assert _status(json.dumps(g)) == api.UNIMPLEMENTED            # :49
    g = _base(); g["fpmath_mode"] = "bf16"
    assert _status(json.dumps(g)) == api.UNIMPLEMENTED            # :54-57
    g = _base(); g["graph"][0]["inputs"][0]["dtype"] = "f128"
    assert _status(json.dumps(g)) == api.UNIMPLEMENTED            # :281
    g = _base(); g["graph"][0]["inputs"][0]["layout_type"] = "opaque"
    assert _status(json.dumps(g)) == api.UNIMPLEMENTED            # :293
    g = _base(); g["graph"][0]["inputs"][0]["colour"] = "red"
    assert _status(json.dumps(g)) == api.INVALID_GRAPH            # :301
    g = _base(); del g["graph"][0]["kind"]
    assert _status(json.dumps(g)) == api.INVALID_GRAPH            # :211
    g = _base(); g["input_ports"] = g["input_ports"][:-1]
    assert _status(json.dumps(g)) == api.INVALID_GRAPH            # :76-80
    g = _base(); g["output_ports"] = [777]
    assert _status(json.dumps(g)) == api.INVALID_GRAPH            # :100-104
    g = _base(); g["graph"][0]["attrs"] = {"transpose_a": {"value": 1, "type": "bool"}}
    assert _status(json.dumps(g)) == api.INVALID_GRAPH            # attr keys are ordered: type, value (:228-233)
    g = _base(); g["graph"][0]["attrs"] = {"transpose_a": {"type": "complex", "value": 1}}
    assert _status(json.dumps(g)) == api.UNIMPLEMENTED            # :256
    g = _base(); g["graph"][1]["inputs"][0]["shape"] = [3, 3]
    assert _status(json.dumps(g)) == api.INVALID_GRAPH            # type mismatch for a produced value (:196-199)
    assert _status("{ not json") == api.INVALID_GRAPH
    assert _status("[]") == api.INVALID_GRAPH


def test_malformed_post_ops_and_unwritable_outputs_are_refused_at_compile_time():
    """A MatMul followed by an input-less ReLU or an output-less Add is a malformed graph, not a crash; an output
    with non-dense strides, or an output that is one of the partition's own inputs, is refused (unimplemented)
    instead of being returned unwritten."""
    t = lambda i, s: {"id": i, "dtype": "bf16", "shape": s}
    mm = {"kind": "MatMul", "inputs": [t(0, [32, 64]), t(1, [64, 48])], "outputs": [t(2, [32, 48])]}
    env = lambda graph, **kw: json.dumps({"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "strict", "graph": graph, **kw})
    assert _status(env([mm, {"kind": "ReLU", "inputs": [], "outputs": [t(3, [32, 48])]}])) == api.INVALID_GRAPH
    assert _status(env([mm, {"kind": "Add", "inputs": [t(2, [32, 48]), t(4, [48])], "outputs": []}])) == api.INVALID_GRAPH
    relu = {"kind": "ReLU", "inputs": [t(2, [32, 48])], "outputs": [dict(t(3, [32, 48]), layout_type="strided", stride=[96, 2])]}
    assert _status(env([mm, relu])) == api.UNIMPLEMENTED
    relu["outputs"][0]["stride"] = [48, 1]                          # dense strides spelled out: fine
    assert _status(env([mm, relu])) == api.SUCCESS
    assert _status(env([mm], input_ports=[0, 1], output_ports=[2, 0])) == api.UNIMPLEMENTED   # output 0 is an input


def test_column_sum_scratch_is_not_shared_with_other_temporaries():
    """The zero-point column sums of a QuantizedMatMul are kept from one call to the next (constant weights), so
    the planner must not hand their region to a later temporary of the same partition."""
    t = lambda i, d, s, c=False: dict({"id": i, "dtype": d, "shape": s}, **({"property_type": "constant"} if c else {}))
    M, N, K = 64, 128, 64
    graph = [
        {"kind": "QuantizedMatMul", "attrs": {"src_zp": {"type": "s64", "value": 128}},
         "inputs": [t(0, "u8", [M, K]), t(1, "s8", [K, N], True), t(2, "f32", [N], True)], "outputs": [t(3, "f32", [M, N])]},
        {"kind": "Sigmoid", "inputs": [t(3, "f32", [M, N])], "outputs": [t(4, "f32", [M, N])]},
        {"kind": "Multiply", "inputs": [t(3, "f32", [M, N]), t(4, "f32", [M, N])], "outputs": [t(5, "f32", [M, N])]},
        {"kind": "ReLU", "inputs": [t(5, "f32", [M, N])], "outputs": [t(6, "f32", [M, N])]},
    ]
    js = json.dumps({"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "strict", "graph": graph})
    plan = api.GraphCompiler().compile(js).plan()
    # three f32 [M,N] temporaries (all live in the Multiply step) + the column sums (N * 4 bytes in a 1 KiB slot of
    # their own): without the whole-partition lifetime the planner would put temporary 5 on top of the sums
    assert "arena_bytes: %d" % (3 * M * N * 4 + 1024) in plan, plan
    offs = sorted(int(m) for m in re.findall(r"@arena\+(\d+)", plan))
    assert M * N * 4 not in offs and set(offs) == {0, M * N * 4 + 1024, 2 * M * N * 4 + 1024}, plan


def test_debug_log_filter_and_verbose_plan_follow_the_reference_switches():
    """GC_DEBUG is an extended regex over source paths (include/gc/Utils/Log.h:43-66): matching files print
    "[DEBUG] [file:line] ..." lines on stdout; GC_B200_VERBOSE prints the launch plan with the chosen tiles at compile.
    Both are read once per process, so each setting runs in a child process."""
    import subprocess
    import sys

    prog = ("import sys; sys.path[:0] = [%r, %r]\n"
            "from gc_b200 import api, partitions\n"
            "exe = api.GraphCompiler().compile(partitions.mlp(512, (4096, 16384, 4096))[0])\n"
            "print('LAUNCHES', exe.launches().count('gemm_kernel'))\n") % (ROOT, os.path.join(ROOT, "graph-compiler_b200"))

    def run(**env):
        e = dict(os.environ)
        for k in ("GC_DEBUG", "GC_B200_VERBOSE"):
            e.pop(k, None)
        e.update(env)
        r = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=e, timeout=120)
        assert r.returncode == 0, r.stderr
        return r.stdout

    quiet = run()
    assert "[DEBUG]" not in quiet and "launch plan" not in quiet and "LAUNCHES 2" in quiet
    dbg = run(GC_DEBUG=".*")
    assert re.search(r"\[DEBUG\] \[.*executable\.cu:\d+\] compiled a partition of 4 ops into 2 steps", dbg), dbg
    assert "[DEBUG]" in run(GC_DEBUG="execut(able|or)") and "[DEBUG]" not in run(GC_DEBUG="/NoSuchDir/")
    verbose = run(GC_B200_VERBOSE="1")
    assert "[gc_b200] launch plan" in verbose
    assert re.search(r"step 0 MatMul\+ReLU: gemm_kernel<bf16> 512x16384x4096 tile 128x\d+ splits 1 stages \d+ K blocks/stage \d+ grid 148", verbose), verbose
    assert re.search(r"step 1 MatMul\+ReLU: gemm_kernel<bf16> 512x4096x16384 tile 128x\d+ splits 2 .* \+ reduce_planes", verbose), verbose


def test_guard_bands_are_planned_around_every_arena_slice(monkeypatch):
    """GC_B200_GUARD=<bytes> at compile time: each temporary gets a canary band before and after it (the debug
    memory pool of the reference keeps one per allocation, MemoryPool.cpp:55-60); offsets move, sizes grow, the
    slices still never overlap."""
    js = partitions.mlp(128, (512, 64, 256), has_bias=[True, True])[0]
    plain = api.GraphCompiler().compile(js).plan()
    assert "guard_bytes" not in plain and "arena_bytes: 16384" in plain and "@arena+0" in plain
    monkeypatch.setenv("GC_B200_GUARD", "100")                      # rounded up to 256
    guarded = api.GraphCompiler().compile(js).plan()
    assert "guard_bytes: 256 (2 bands)" in guarded
    assert "arena_bytes: %d" % (16384 + 2 * 256 + 512) in guarded   # slice sizes are 1 KiB aligned: 16896 -> 17408
    assert "@arena+256" in guarded
    monkeypatch.delenv("GC_B200_GUARD")
    assert api.GraphCompiler().compile(js).plan() == plain


def test_mpl_graph_structure():
    """The 2-layer MLP of test/dnnl/resources/mpl.json (TestJsonParser.cpp:138-225): arguments
    0,1,2,5,7 in first-use order, result 9; both spellings of bias (+ReLU) fuse into the matmuls."""
    t = lambda i, s: {"id": i, "dtype": "bf16", "shape": s}
    graph = [
        {"kind": "MatMul", "inputs": [t(0, [128, 512]), t(1, [512, 64]), t(2, [64])], "outputs": [t(3, [128, 64])]},
        {"kind": "ReLU", "inputs": [t(3, [128, 64])], "outputs": [t(4, [128, 64])]},
        {"kind": "MatMul", "inputs": [t(4, [128, 64]), t(5, [64, 256])], "outputs": [t(6, [128, 256])]},
        {"kind": "Add", "inputs": [t(6, [128, 256]), t(7, [256])], "outputs": [t(8, [128, 256])]},
        {"kind": "ReLU", "inputs": [t(8, [128, 256])], "outputs": [t(9, [128, 256])]},
    ]
    js = json.dumps({"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "any", "input_ports": [0, 1, 2, 5, 7],
                     "output_ports": [9], "graph": graph})
    gc = api.GraphCompiler()
    plan = gc.compile(js).plan()
    assert "inputs: 0 1 2 5 7" in plan and "outputs: 9" in plan
    steps = [l for l in plan.splitlines() if l.startswith("step")]
    assert len(steps) == 2
    assert "MatMul+ReLU" in steps[0] and "bias=1 relu=1" in steps[0] and "4@arena+0" in steps[0]
    assert "MatMul+Add+ReLU" in steps[1] and "bias=1 relu=1" in steps[1] and "9@out0" in steps[1]
    assert "arena_bytes: 16384" in plan  # one 128x64 bf16 temporary


@pytest.mark.skipif(not os.path.isdir(REF_JSON), reason="reference fixtures not present")
def test_reference_json_fixtures_compile():
    """Every partition file the reference's C-API tests use compiles (test/dnnl/resources/*.json)."""
    gc = api.GraphCompiler()
    names = sorted(f for f in os.listdir(REF_JSON) if f.endswith(".json"))
    assert len(names) == 13
    for n in names:
        exe = gc.compile(open(os.path.join(REF_JSON, n)).read())
        assert exe.plan().count("step") >= 1, n


def test_fusion_is_blocked_by_a_second_consumer_or_an_output():
    t = lambda i, s: {"id": i, "dtype": "bf16", "shape": s}
    graph = [
        {"kind": "MatMul", "inputs": [t(0, [32, 64]), t(1, [64, 48])], "outputs": [t(2, [32, 48])]},
        {"kind": "ReLU", "inputs": [t(2, [32, 48])], "outputs": [t(3, [32, 48])]},
    ]
    env = {"version": "3.5.0", "engine_kind": "cpu", "fpmath_mode": "strict", "graph": graph}
    gc = api.GraphCompiler()
    assert gc.compile(json.dumps(env)).plan().count("step") == 1
    env["output_ports"] = [2, 3]            # the un-activated value is also a result
    assert gc.compile(json.dumps(env)).plan().count("step") == 2
    del env["output_ports"]
    graph.append({"kind": "Add", "inputs": [t(2, [32, 48]), t(3, [32, 48])], "outputs": [t(4, [32, 48])]})
    assert gc.compile(json.dumps(env)).plan().count("step") == 3


def test_mlp_chain_ping_pongs_in_the_arena():
    js, ins, out = partitions.mlp(512, (4096, 16384, 4096, 16384, 4096), has_bias=[True] * 4)
    plan = api.GraphCompiler().compile(js).plan()
    steps = [l for l in plan.splitlines() if l.startswith("step")]
    assert len(steps) == 4 and all("MatMul+ReLU" in s for s in steps)
    # live at once: one 512x16384 and one 512x4096 bf16 activation
    assert "arena_bytes: %d" % (512 * 16384 * 2 + 512 * 4096 * 2) in plan


def test_arena_planner_never_overlaps_live_buffers():
    import random

    rng = random.Random(0)
    for trial in range(50):
        n = rng.randint(1, 24)
        sizes = [rng.choice([0, 1, 64, 100, 160, 4096, 5000]) for _ in range(n)]
        first = [rng.randint(0, 20) for _ in range(n)]
        last = [f + rng.randint(0, 6) for f in first]
        off, total = api.plan_arena(sizes, first, last, align=64)
        for i in range(n):
            assert off[i] % 64 == 0 and off[i] + sizes[i] <= total
            for j in range(i):
                if first[i] <= last[j] and first[j] <= last[i] and sizes[i] and sizes[j]:
                    assert off[i] + sizes[i] <= off[j] or off[j] + sizes[j] <= off[i], (trial, i, j)
        peak = max(sum(s for s, f, l in zip(sizes, first, last) if f <= t <= l) for t in range(30))
        assert total >= peak
    # disjoint lifetimes share memory
    off, total = api.plan_arena([1000, 1000, 1000], [0, 1, 2], [0, 1, 2], align=64)
    assert total == 1024 and off == [0, 0, 0]


def test_tile_selection_for_the_benchmark_shapes():
    sel = lambda M, N, K, db=2, ob=2: lib.select_matmul_config(M, N, K, db, ob, 148)
    c = sel(8192, 8192, 8192)
    assert (c.swapped, c.bn, c.splits) == (0, 256, 1) and c.grid == 148
    c = sel(16, 28672, 8192)            # decode shape: weights on the MMA M side, two K blocks per stage
    assert c.swapped == 1 and c.bn == 16 and c.splits == 1 and c.kpb == 2
    c = sel(16, 512, 8192)              # few weight tiles: split K to fill the SMs
    assert c.swapped == 1 and c.splits > 1 and (8192 // 64 // c.splits) % c.kpb == 0
    c = sel(512, 4096, 16384)           # 64 tiles of 128 x 256: K split in two fills 128 SMs
    assert (c.bn, c.kpb, c.splits) == (256, 1, 2)
    c = sel(512, 4096, 4096)            # one wave of 128-wide tiles, two K blocks per stage
    assert (c.bn, c.kpb, c.splits) == (128, 2, 1)
    c = sel(128, 256, 512)              # BASELINE configs[0]
    assert c.swapped == 0 and c.bn in (64, 128, 256)
    c = sel(1024, 4096, 4096, 1, 4)     # int8, less than a wave of 256-wide tiles: 128-wide, two K blocks per stage
    assert c.swapped == 0 and (c.bn, c.kpb, c.splits, c.grid) == (128, 2, 1, 148)
    c = sel(8192, 8192, 8192, 1, 4)     # int8, many waves: 256-wide tiles
    assert (c.bn, c.kpb, c.splits) == (256, 1, 1)
    for M, N, K in [(1, 1, 1), (5, 7, 9), (200, 328, 136), (64, 128, 64), (65, 100000, 64)]:
        c = sel(M, N, K)
        assert 16 <= c.bn <= 256 and c.bn % 16 == 0 and 2 <= c.stages <= 8 and c.splits >= 1 and c.grid >= 1


def test_launchers_fail_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    n = C.c_int(0)
    assert lib.load().gcb200_sm_count(C.byref(n)) == 3  # GCB200_NO_DEVICE: no CPU fallback
    assert b"CUDA" in lib.load().gcb200_last_error() or b"device" in lib.load().gcb200_last_error()
    import numpy as np

    js, ins, out = partitions.mlp(8, (16, 8), dtype="f32")
    exe = api.GraphCompiler().compile(js)
    with pytest.raises(api.DnnlError) as ei:
        exe.execute({0: np.zeros((8, 16), np.float32), 1: np.zeros((16, 8), np.float32), 2: np.zeros(8, np.float32)},
                    {out: np.zeros((8, 8), np.float32)})
    assert ei.value.status == api.RUNTIME_ERROR
