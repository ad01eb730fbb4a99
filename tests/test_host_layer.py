"""The C++ mirror of the reference's host layer (Graph / Tensor / ops / reverse /
optimizers): builds tests/host/host_scenarios.cpp against libmp_host.so and the
oracle, and runs it on the GPU.  The scenarios replay the reference's example
programs and the README feed-forward block."""
import json
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "metaphor_b200" / "lib"


def build_scenarios(tmp_path, orc) -> Path:
    exe = tmp_path / "host_scenarios"
    subprocess.run(["g++", "-O2", "-std=c++17", "-Wall", "-o", str(exe), str(ROOT / "tests" / "host" / "host_scenarios.cpp"),
                    f"-L{LIB}", "-lmp_host", "-lmp_kernels", f"-L{ROOT / 'oracle'}", "-loracle",
                    f"-Wl,-rpath,{LIB}", f"-Wl,-rpath,{ROOT / 'oracle'}"], check=True, capture_output=True)
    return exe


def test_host_layer_and_scenarios_compile(mp, orc, tmp_path):
    assert (LIB / "libmp_host.so").exists()
    assert build_scenarios(tmp_path, orc).exists()


def test_rank_n_contraction_plans_on_the_cpu(mp, orc, tmp_path):
    """Every plan of the rank-N contraction planner, carried out with plain loops, equals the contraction summed
    from its expression (forward and both gradient expressions); no device call."""
    exe = tmp_path / "contraction_plans"
    subprocess.run(["g++", "-O2", "-std=c++17", "-Wall", "-o", str(exe), str(ROOT / "tests" / "host" / "contraction_plans.cpp"),
                    f"-L{LIB}", "-lmp_host", "-lmp_kernels", f"-Wl,-rpath,{LIB}"], check=True, capture_output=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "ALL PLANS PASSED" in res.stdout


@pytest.mark.gpu
def test_reference_examples_and_feed_forward_block(mp, orc, tmp_path):
    exe = build_scenarios(tmp_path, orc)
    res = subprocess.run([str(exe), "200", str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "ALL SCENARIOS PASSED" in res.stdout
    m = re.search(r"FEED_FORWARD_TIMING (\{.*\})", res.stdout)
    assert m, res.stdout
    timing = json.loads(m.group(1))
    print("feed-forward block timing:", timing)
    assert timing["forward_us"] > 0
