"""bench.py --impl reference must finish and print its JSON line when a launcher starts it, at world size > 1 too.

Under torch.distributed.run every rank inherits the launcher's variables (TORCHELASTIC_USE_AGENT_STORE among
them); the gloo ranks the CPU baseline starts must not pick them up, or they all wait for a store nobody hosts.
"""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _json_line(out: str) -> dict:
    lines = [l for l in out.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out[-2000:]
    return json.loads(lines[0])


def test_reference_arm_under_launcher_two_ranks():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29733", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--impl", "reference", "--steps", "4", "--warmup", "1"]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    line = _json_line(r.stdout)
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    assert line["steps"] >= 1 and line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["e2e"]["value"] == line["value"] and line["gpu_launches"] == 0


def test_cpu_baseline_port_and_reference_agree_on_shape_of_result():
    """Both kinds run the same layer; the port is the fallback when the reference's install is absent."""
    from oracle import cpu_baseline
    small = dict(hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, intermediate=512)
    kinds = ["port"] + (["reference"] if cpu_baseline.reference_available() else [])
    for kind in kinds:
        r = cpu_baseline.time_decoder_layer(small, 8, 2, 1, 3, max_seconds=5.0, kind=kind)
        assert r["kind"] == kind and r["steps"] == 3 and r["seconds_per_layer"] > 0
