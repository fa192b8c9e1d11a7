"""Host-side pieces of ``bench.py`` that need no GPU: what a line says about its workload, how many repeats a timing
takes, which plan config 4 runs, the stale-capture rule for ``roofline.traffic``."""

import importlib.util
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_workload_text_names_the_configuration():
    bench = _bench()
    from tensorfold_b200 import synthetic

    c2 = bench.workload_config(synthetic.C2, 64, 1)
    assert "config 2" in c2["workload"] and "64-token" in c2["workload"] and c2["parallelism"] == "single"
    c4 = bench.workload_config(synthetic.C4, 32, 8, "c4")
    assert "256 tokens over the ranks" in c4["workload"] and c4["parallelism"] == "ep8"
    c5 = bench.workload_config(synthetic.C5, 0, 8, "c5")
    assert "batches of 1, 8, 32, 128, 512 tokens" in c5["workload"] and "0 tokens" not in c5["workload"]
    assert "model" not in c2 and "model" not in c5


def test_repeats_cover_three_hundred_steps():
    bench = _bench()
    assert bench.repeats_for(20) * 20 >= 300 and bench.repeats_for(100) == 3 and bench.repeats_for(1) == 25
    assert bench.repeats_for(10 ** 6) == 3


def test_config_4_runs_the_split_plan_unless_told_otherwise():
    bench = _bench()
    assert bench.hot_pairs_for("c4", -1) == bench.C4_HOT_PAIRS > 0
    assert bench.hot_pairs_for("c2", -1) == 0
    assert bench.hot_pairs_for("c4", 0) == 0 and bench.hot_pairs_for("c2", 48) == 48


def test_traffic_is_quoted_only_for_the_captured_kernel_sources():
    bench = _bench()
    text = (ROOT / "profiles" / "decode_kernel_c2_64tokens.md").read_text()
    recorded = re.search(r"kernel_source_sha:\s*([0-9a-f]+)", text).group(1)
    nbytes, why = bench.captured_traffic()
    if recorded == bench.kernel_source_sha():
        assert nbytes == int(re.search(r"traffic_bytes_per_launch:\s*(\d+)", text).group(1)) and "same kernel sources" in why
        # the capture must be plausible: between the algorithmic bytes of the launch and 1.2 times them
        assert 224985088 <= nbytes <= 1.2 * 224985088
    else:
        assert nbytes is None and "stale" in why


def test_reference_arm_prints_its_line_without_a_gpu():
    """`bench.py --impl reference` (the reference's CPU path restated, on the host cores) needs no GPU and prints the
    contract's line: the same metric, unit and config as the GPU arm, its own `cpu_baseline` and a zero-copy `e2e`."""

    import json
    import subprocess
    import sys

    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == "moe_layer_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["value"] > 0
    assert "config 2" in line["config"]["workload"]
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] and base["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
