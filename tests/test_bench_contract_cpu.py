"""The command-line contracts that need no GPU: the reference arm of bench.py prints its one-line reason, the collective sweep refuses a single
rank with a JSON line, the CPU DDP benchmark prints its metric with both equivalence checks true."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _last_json(cmd, timeout=600):
    r = subprocess.run([sys.executable] + cmd, capture_output=True, text=True, timeout=timeout, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_reference_arm_reports_unavailable():
    d = _last_json(["bench.py", "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and len(d["unavailable"]) > 10


def test_collective_sweep_needs_two_ranks():
    d = _last_json(["bench_collectives.py"])
    assert d["bench"] == "collectives" and "unavailable" in d


def test_cpu_ddp_benchmark_line():
    d = _last_json(["bench_cpu_ddp.py", "--steps", "20"])
    assert d["metric"] == "cpu_ddp_tcp_ms_per_step" and d["value"] > 0 and d["world"] == 2 and d["higher_is_better"] is False
    assert d["ranks_bit_identical"] is True and d["matches_single_process_1e-5"] is True
