"""CPU: the parts of bench.py's output contract that need no GPU.

The roofline's `traffic` is read from the committed profiler summary of the kernel that is
timed; the reference arm runs the CPU oracle on rank 0 and prints one JSON line with the agreed
keys; the list of profiler workloads names only cases `run_case` knows."""
import json
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_traffic_comes_from_the_committed_summary_of_the_timed_kernel():
    import bench
    t = bench.measured_traffic()
    assert t is not None, "profiles/kq_mv_q4k_K2560_N10240.md is missing or has no DRAM lines"
    # DRAM traffic of a launch equals its algorithmic bytes to within a percent: no re-reads
    assert abs(t - bench.Q4K_BYTES) / bench.Q4K_BYTES < 0.01
    src = open(os.path.join(ROOT, "bench.py")).read()
    assert "kq_mv_kernel<12,false>" in src  # the kernel the summary is about is the one named


def test_reference_arm_prints_one_json_line_with_the_agreed_keys():
    env = dict(os.environ, OMP_NUM_THREADS="1")  # what torch.distributed.run exports
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True,
                       env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "quant matvec HBM GB/s" and d["unit"] == "GB/s"
    assert d["higher_is_better"] is True and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] == d["value"]
    # the arm asks for the host's cores itself, whatever OMP_NUM_THREADS says
    assert d["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}


def test_non_zero_ranks_of_the_reference_arm_exit_without_work():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--gpus", "2", "--steps", "1", "--warmup", "0"], capture_output=True,
                       text=True, env=env, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_every_listed_profiler_case_exists():
    import bench
    src = open(os.path.join(ROOT, "bench.py")).read()
    listed = set()
    for m in re.finditer(r"^  ([a-z0-9_]+(?: / [a-z0-9_]+)*)\s{2,}", bench.CASES, re.M):
        listed.update(x.strip() for x in m.group(1).split("/"))
    handled = set(re.findall(r'"([a-z0-9_]+)"', src[src.index("def run_case"):src.index("def main")]))
    assert listed, "the case list was not found"
    assert listed <= handled, listed - handled
    for f in os.listdir(os.path.join(ROOT, "profiles")):
        txt = open(os.path.join(ROOT, "profiles", f)).read()
        for case in re.findall(r"bench\.py --case (\w+)", txt):
            assert case in handled or case == "gemma", (f, case)  # "gemma$b" in a shell loop
