"""The benchgc-compatible command line, run as a user would run the reference's harness (correctness mode, mode C):
the single-layer MLP of BASELINE configs[0], the bf16 matmul line of the reference's own correctness script
(scripts/correctness.sh:9), the llama2 decoder block in linalg form (the module the reference keeps as
test/benchgc/cases/llama2.mlir, printed here by mlir_text.llama2_mlp_module) and attention spelled with
batch_matmul / softmax.  Each must end with the harness's "PASSED" verdict."""
import os
import subprocess
import sys

import pytest

from gc_b200 import mlir_text

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _benchgc(*argv):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, os.path.join(ROOT, "graph-compiler_b200")]))
    r = subprocess.run([sys.executable, "-m", "gc_b200.benchgc", *argv], capture_output=True, text=True, env=env, timeout=600)
    return r.returncode, r.stdout + r.stderr


def test_cfg1_mlp_pattern_passes():
    rc, out = _benchgc("--driver", "pattern", "--case", "mlp", "--batch_size", "128", "--hidden_size_list", "512x256", "--has_bias", "1",
                       "--act_type", "relu", "--dtype", "bf16", "--fill", "0:U:-1:1", "--fill", "1:U:-1:1", "--fill", "2:U:-1:1")
    assert rc == 0 and "PASSED: pattern.mlp" in out, out


def test_bf16_matmul_line_of_the_reference_correctness_script_passes():
    rc, out = _benchgc("--verbose", "0", "--driver", "linalg", "--case", "matmul", "--md", "0:32x128xbf16", "--md", "1:128x64xbf16",
                       "--md", "2:32x64xbf16", "--cast", "cast_signed")
    assert rc == 0 and "PASSED: linalg.matmul" in out, out


def test_llama2_decoder_block_module_passes(tmp_path):
    path = tmp_path / "llama2.mlir"
    path.write_text(mlir_text.llama2_mlp_module(1, 32, 4096, 11008))
    # weights N(0, 0.02) as in a trained block; both results held to the harness's norm check (bf16: 2^-8 per op)
    fills = []
    for i in (1, 5, 6, 7):
        fills += ["--fill", f"{i}:N:0:0.02"]
    rc, out = _benchgc("--driver", "mlir", "--case", str(path), *fills, "--fill", "8:U:0.00001:0.00002", "--cmp", "10:N:0.02", "--cmp", "11:N:0.02")
    assert rc == 0 and "PASSED: mlir." in out, out


def test_attention_module_passes(tmp_path):
    path = tmp_path / "attention.mlir"
    path.write_text(mlir_text.attention_module(8, 512, 128, 128 ** -0.5))
    rc, out = _benchgc("--driver", "mlir", "--case", str(path), "--cmp", "3:N:0.02")
    assert rc == 0 and "PASSED: mlir." in out, out


def test_int8_module_passes_bit_exactly(tmp_path):
    """BASELINE configs[1] in small, as a linalg module: exact s32 accumulators (threshold 0) and the dequantised f32
    result (same f32 operations on both sides: threshold 0 as well)."""
    acc = tmp_path / "int8_acc.mlir"
    acc.write_text(mlir_text.quantized_matmul_module(256, 512, 1024, src_zp=128, dequant=False))
    rc, out = _benchgc("--driver", "mlir", "--case", str(acc), "--fill", "0:I:0:255", "--fill", "1:I:-127:127", "--cmp", "2:P:0:100")
    assert rc == 0 and "PASSED: mlir." in out, out
    deq = tmp_path / "int8.mlir"
    deq.write_text(mlir_text.quantized_matmul_module(256, 512, 1024, src_zp=128))
    rc, out = _benchgc("--driver", "mlir", "--case", str(deq), "--fill", "0:I:0:255", "--fill", "1:I:-127:127", "--fill", "2:U:0.001:0.01",
                       "--fill", "3:U:-1:1", "--cmp", "4:P:0.000001:100")
    assert rc == 0 and "PASSED: mlir." in out, out
