"""The benchmark's reference arm runs on CPU (it times the oracle port), so its JSON line can be checked here:
one line, the keys the harness reads, the metric and unit of the headline workload."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "attn_decode_hbm_gbs" and d["unit"] == "GB/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 1
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["vs_baseline"] is None
    assert d["config"]["workload"] == "gqa_decode_b32"
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


def test_both_arms_describe_the_workload_with_the_same_config():
    """The GPU arm and the CPU arm print the same `config` object (it is built without a device)."""
    sys.path.insert(0, ROOT)
    import bench
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    d = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][0])
    assert d["config"] == bench.GqaDecodeB32.describe(bench.decode_lens(0))
    assert d["config"]["workload"] == "gqa_decode_b32" and d["config"]["sum_context"] == int(bench.decode_lens(0).sum())
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    # the strong-scaled split of the same batch covers every sequence exactly once
    from inferno_b200.sharding import shard_sequences
    for world in (2, 4, 8):
        covered = sorted(i for r in range(world) for i in range(*shard_sequences(32, world, r)))
        assert covered == list(range(32))
