"""The benchmark script end to end on a small shard: the JSON line carries every key of the contract and
its numbers are self-consistent."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _bench(*args):
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_default_workload_line_on_a_small_shard():
    d = _bench("--tokens", "4096", "--steps", "3", "--warmup", "3", "--cpu-tokens", "256")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "clocks", "gpu_launches"):
        assert key in d, key
    assert d["unit"] == "GB/s" and d["n_gpus"] == 1 and d["steps"] == 3 and d["dtype"] == "bf16" and d["vs_baseline"] is None
    assert d["gpu_launches"] == 8 * 3                      # eight kernels per step, all from this library
    assert d["roofline"]["bound"] == "hbm" and 0.2 < d["roofline"]["frac"] < 1.3
    assert d["e2e"]["h2d_bytes_per_step"] > 1e9 and d["e2e"]["d2h_bytes_per_step"] == 4 and 0 < d["e2e"]["value"] < d["value"]
    assert d["cpu_baseline"]["kind"] == "port" and 0 < d["cpu_baseline"]["value"] < d["e2e"]["value"]
    per_op = d["per_op"]
    assert abs(sum(v["ms"] for v in per_op.values()) - d["ms_per_step"]) < 0.15 * d["ms_per_step"]
    for op in ("norm", "rope", "swiglu"):
        assert abs(per_op[op]["fwd_ms"] + per_op[op]["bwd_ms"] - per_op[op]["ms"]) < 1e-6


def test_small_config_is_flushed_and_replayed_from_a_graph():
    d = _bench("--config", "c1", "--steps", "3", "--no-e2e", "--no-cpu-baseline", "--no-extras")
    assert "flush" in json.dumps(d["config"]).lower()
    for op, v in d["per_op"].items():
        assert all(us > 0 for us in v["graph_replay_us"].values()), op
    # launch-free, L2-resident replays are faster than cold, individually launched kernels
    assert d["per_op"]["norm"]["graph_replay_us"]["fwd"] < d["per_op"]["norm"]["fwd_ms"] * 1e3
