"""bench.py's contract on the host: more than one GPU is answered with one line and exit code 2; the byte and flop
counts behind its roofline figures; the reference arm says `unavailable` (and exits 0) where the reference is not
built."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_more_than_one_gpu_is_refused_with_one_line():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True,
                       cwd=ROOT, timeout=300)
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_bytes_and_flops_of_the_headline_shape():
    sys.path.insert(0, ROOT)
    import bench
    cfg = bench.SHAPES["8b"]
    per_layer = bench.layer_params(cfg)
    # q|k|v + output + gate|up + down matrices, two norm gains, two per-head gains
    assert per_layer == (32 + 16) * 128 * 4096 + 4096 * 4096 + 3 * 4096 * 12288 + 2 * 4096 + 2 * 128
    weights = 2 * (36 * per_layer + 151936 * 4096 + 4096)
    cache = 8 * 2048 * 36 * 2 * 8 * 128 * 2
    assert bench.decode_bytes(cfg, 8, 2048) == weights + 2 * 8 * 4096 + cache
    T = 2048
    assert bench.prefill_flops(cfg, T) == 2.0 * T * 36 * per_layer + 2.0 * 151936 * 4096 + 36 * 4.0 * 32 * 128 * T * (T + 1) / 2
    # the record's configuration stays flat and short
    assert len(bench.SHAPES) == 3 and all(v["head_dim"] == 128 for v in bench.SHAPES.values())


def test_reference_arm_without_a_built_reference(tmp_path):
    """With no built reference and no sources to build it from, the arm prints its reason and exits 0."""
    env = dict(os.environ, LLME_REFERENCE=str(tmp_path / "nowhere"))
    built = os.path.join(ROOT, "baseline", "_ref", "reference_bench")
    if os.path.exists(built):
        import pytest
        pytest.skip("the reference is built here: the arm would try to run it")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], capture_output=True, text=True,
                       cwd=ROOT, env=env, timeout=600)
    assert p.returncode == 0
    rec = json.loads([l for l in p.stdout.splitlines() if l.strip()][-1])
    assert rec["impl"] == "reference" and "unavailable" in rec
