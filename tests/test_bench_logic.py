"""Host-side logic of bench.py: the algorithmic-byte formulas (the figures the roofline fractions are
computed from) and the CPU reference arm."""
import json
import subprocess
import sys
from pathlib import Path

import bench

ROOT = Path(__file__).resolve().parent.parent


def test_algorithmic_bytes_match_the_documented_worked_examples():
    c1, c2, c3 = bench.CONFIGS["c1"], bench.CONFIGS["c2"], bench.CONFIGS["c3"]
    b2 = bench.algorithmic_bytes(c2, 32768, 0.0)
    assert abs(b2["norm"] / 1e9 - 2.147) < 0.01            # add+RMSNorm 8*M*N*s
    assert abs(b2["swiglu"] / 1e9 - 7.516) < 0.01          # 8*M*N*s
    assert abs(b2["cross_entropy"] / 1e9 - 16.81) < 0.01   # M*V*s*2
    assert abs(b2["rope"] / 1e9 - 1.342) < 0.01            # 4*T*(QH+KH)*D*s (+cos/sin)
    b3 = bench.algorithmic_bytes(c3, 32768, 0.10)
    assert abs(b3["swiglu"] / 1e9 - 9.93) < 0.01
    assert abs(b3["norm"] / 1e9 - 5 * 32768 * 3584 * 2 / 1e9) < 1e-6      # plain RMSNorm: 5*M*N*s
    assert abs(b3["cross_entropy"] - (32768 * 152064 * 2 * 1.9 + 16 * 32768)) < 1
    b1 = bench.algorithmic_bytes(c1, 4096, 0.05)
    assert abs(b1["norm"] / 1e6 - 36.7) < 0.1
    assert abs(b1["cross_entropy"] / 1e9 - 2.43) < 0.01


def test_l2_flush_is_requested_only_for_configs_that_fit_l2():
    assert bench.needs_l2_flush(bench.CONFIGS["c1"])
    assert not bench.needs_l2_flush(bench.CONFIGS["c2"])
    assert not bench.needs_l2_flush(bench.CONFIGS["c3"])


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                        "--cpu-tokens", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]
    assert d["metric"] == "fused_opset_fwd_bwd_algorithmic_hbm_throughput"


def test_phases_cover_every_operator_once_per_direction():
    """A step is seven launch groups: forward and backward of three operators plus the one-pass loss; each
    names an OpSet method, and every operator of the byte table is covered."""
    ops = [op for op, _, _ in bench.PHASES]
    assert set(ops) == set(bench.OPS) and ops == sorted(ops, key=bench.OPS.index)
    for op in ("norm", "rope", "swiglu"):
        assert [d for o, d, _ in bench.PHASES if o == op] == ["fwd", "bwd"]
    assert [d for o, d, _ in bench.PHASES if o == "cross_entropy"] == ["fwd+bwd"]
    for _, _, method in bench.PHASES:
        assert callable(getattr(bench.OpSet, method))
