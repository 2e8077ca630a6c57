"""CPU: the byte and flop tables every roofline figure of bench.py is computed from. One table, pinned here, so that a
change to it is a deliberate one (the kernel table of the design document quotes the same numbers)."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_stage_bytes_of_the_gated_delta_step():
    t = bench.stage_table("gated_delta")
    got = {k: v[0] for k, v in t.items()}
    assert got == {"wy_fwd": 1286, "delta_fwd_h": 1540, "chunk_fwd_o": 1540, "dv_local": 1028, "delta_bwd_dhu": 2052,
                   "dqkwg": 3336, "wy_bwd": 2066, "cumsum": 8}
    assert sum(got.values()) - got["cumsum"] == 12848          # seven stage kernels
    assert sum(v[2] for v in t.values()) == 8                    # launches per step


def test_stage_bytes_of_the_plain_delta_and_simple_gla_steps():
    d = {k: v[0] for k, v in bench.stage_table("delta").items()}
    assert d == {"wy_fwd": 1154, "delta_fwd_h": 1536, "chunk_fwd_o": 1536, "dv_local": 1024, "delta_bwd_dhu": 2048,
                 "dqkwg": 3328, "wy_bwd": 1926}
    s = bench.stage_table("simple_gla")
    assert sum(v[2] for v in s.values()) == 7 and s["cumsum"][2] == 2


def test_whole_step_compulsory_bytes_and_flops():
    # inputs read once, outputs and gradients written once; fla's operation counts with dense 64 x 64 tiles
    assert bench.whole_op("gated_delta", 128, 128, torch.bfloat16) == (2828, 606208)
    assert bench.whole_op("delta", 128, 128, torch.bfloat16)[0] == 2820
    assert bench.whole_op("decode", 128, 128, torch.bfloat16)[0] == 132104
    for name in bench.NCU_BYTES_PER_TOKENHEAD:  # every profiled stage is a stage of the table, and moves no more than its bytes + 3 %
        assert bench.NCU_BYTES_PER_TOKENHEAD[name] <= 1.03 * bench.stage_table("gated_delta")[name][0]


def test_reference_arm_line_is_well_formed_on_cpu():
    """`--impl reference` needs no GPU: one JSON line with the contract's keys and an honest record of what it timed."""
    env = dict(os.environ, OMP_NUM_THREADS="4")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "gla_fp32", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["gpu_launches"] == 0 and line["higher_is_better"] is True
    assert line["steps"] == line["cpu_baseline"]["passes"] and line["warmup"] == line["cpu_baseline"]["warmup_passes"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"] > 0
    assert "reference_sample" in line["config"]
