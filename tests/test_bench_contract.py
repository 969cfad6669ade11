"""What bench.py answers without touching a GPU: more than one GPU is refused with one line and exit code 2, and
the reference arm says in one JSON line why it is unavailable (not built, or built but no GPU here)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused():
    proc = _run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert proc.returncode == 2
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_is_unavailable_in_one_json_line():
    proc = _run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert proc.returncode == 0
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_shapes_name_every_size_of_their_configuration():
    sys.path.insert(0, ROOT)
    import bench
    for name, shape in bench.SHAPES.items():
        assert shape["num_attention_heads"] % shape["num_key_value_heads"] == 0
        assert shape["max_window_layers"] == shape["num_hidden_layers"]
        for key in ("vocab_size", "hidden_size", "intermediate_size", "head_dim", "rope_theta", "rms_norm_eps"):
            assert key in shape, (name, key)
    assert bench.SHAPES["8b"]["num_hidden_layers"] == 36 and bench.SHAPES["8b"]["hidden_size"] == 4096
