"""What `bench.py` promises before it touches a GPU: more than one GPU is refused with one line and exit code 2, the
reference arm says in one JSON line why it cannot run and exits 0, and the flat `config` of every named configuration
stays within what a record keeps."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_the_reference_arm_says_why_it_is_unavailable():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_the_named_configurations_have_a_workload_and_sizes():
    sys.path.insert(0, ROOT)
    import bench
    for name, spec in bench.CONFIGS.items():
        assert {"name", "seed", "layers", "sizes", "workload"} <= set(spec), name
        assert spec["workload"]["batch"] >= 1 and spec["workload"]["steps"] >= 1
        sizes = spec["sizes"]
        assert sizes["hidden_size"] % 8 == 0 and sizes["num_attention_heads"] % sizes["num_key_value_heads"] == 0, name
