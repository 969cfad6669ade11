"""Without a CUDA device nothing of the model runs: the entry points say so instead of falling back."""
import os
import subprocess
import sys

import pytest
import torch

import helpers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
no_cuda = pytest.mark.skipif(torch.cuda.is_available(), reason="this box has a CUDA device")


@no_cuda
def test_engine_and_replay_refuse_to_run_without_cuda(tmp_path):
    from pulsar_b200.engine.engine import Engine
    from pulsar_b200.replay import Replay
    folder = helpers.make_folder(str(tmp_path / "m"), helpers.TINY_A, 0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine(folder, dict(dtype="float32", num_pages=8))
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine(folder, dict(dtype="float32", num_pages=8, device="cpu"))
    with pytest.raises(RuntimeError, match="no CPU path"):
        Replay(folder, "float32", 64)


@no_cuda
def test_kernel_wrappers_refuse_cpu_tensors():
    from pulsar_b200 import ops
    a = torch.zeros(4, 8)
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.gemm_simt(a, torch.zeros(3, 8), torch.zeros(4, 3))
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.embed(torch.zeros(10, 8), torch.zeros(4, dtype=torch.int32), torch.zeros(4, 8))


@no_cuda
def test_trace_run_and_the_command_line_fail_loudly(tmp_path):
    folder = helpers.make_folder(str(tmp_path / "m"), helpers.TINY_A, 0)
    step = '{"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]}], "end": []}\n'
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out",
                           str(tmp_path / "out"), "--max-tokens", "64"], input=step, capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0 and "no CPU path" in proc.stderr and "done 0" not in proc.stdout
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "pulsar-generate"), "--model", folder, "--prompt_ids", "1,2,3",
                           "--gen_tokens", "2", "--dtype", "float32"], capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0 and "no CPU path" in (proc.stderr + proc.stdout)
