#!/usr/bin/env python
"""Benchmark of the chunked linear-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward + backward pass of the op over one synthetic batch.  The default
workload is the configuration the headline metric is quoted on: chunk_gated_delta_rule, bf16,
B=8 T=4096 H=16 K=V=128, initial state given, final state requested.  With N > 1 (torchrun, one
rank per GPU) every rank runs the same per-GPU batch (sequences and heads are independent, so the
path shards with no data-path collective): weak scaling, value = tokens of all ranks / max time.

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM; `e2e` = the same
step with host (pinned) input buffers copied in and every result copied back inside the timed
region; `roofline` = the dominant kernel timed on its own with CUDA events; `cpu_baseline` = the
CPU oracle (a port of the reference's naive recurrence) on a bounded sample.
`--impl reference` times that CPU path only (it is the reference's own CPU implementation of the
path, restated; the reference checkout does not travel to the GPU box).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "flash-linear-attention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

METRIC = "chunk fwd+bwd tokens/s (GDN H=16 D=128 T=4K bf16)"  # the headline metric: default workload only
UNIT = "tokens/s"
# side workloads name themselves, so that a line can never be mistaken for the headline number
SIDE_METRICS = {
    "delta": "chunk_delta_rule fwd+bwd tokens/s (H=16 D=128 T=4K bf16)",
    "retention": "chunk_simple_gla / retention fwd+bwd tokens/s (H=16 D=128 T=4K bf16)",
    "gla_fp32": "chunk_gla fwd+bwd tokens/s (fp32 B=2 T=512 H=4 D=64)",
    "gla": "chunk_gla fwd+bwd tokens/s (H=16 D=128 T=4K bf16)",
    "varlen": "chunk_gated_delta_rule fwd+bwd tokens/s (64 packed sequences, H=32 D=128 bf16)",
    "decode": "fused_recurrent_gated_delta_rule decode tokens/s (256 sequences, H=16 D=128)",
    "long": "chunk_gated_delta_rule fwd+bwd tokens/s (ONE sequence of 262144 tokens, H=16 D=128 bf16)",
    "l2norm": "l2_norm fwd+bwd tokens/s (q and k of B=8 T=4096 H=16 D=128 bf16)",
    "norm_gate": "FusedRMSNormSwishGate fwd+bwd tokens/s (o and gate of B=8 T=4096 H=16 D=128 bf16)",
    "short_conv": "ShortConvolution fwd+bwd tokens/s (B=8 T=4096 D=2048 W=4 silu bf16)",
}

# DRAM bytes per token-head of each stage's kernel, from the ncu capture summarised in
# profiles/gdn_kernels_ncu_full_T2048.md (dram__bytes_read.sum + dram__bytes_write.sum at T=2048, 262 144
# token-heads; the traffic of these kernels is proportional to the number of tokens)
NCU_BYTES_PER_TOKENHEAD = {"wy_fwd": 1074, "delta_fwd_h": 1415, "chunk_fwd_o": 1499, "dv_local": 941,
                           "delta_bwd_dhu": 1953, "dqkwg": 3240, "wy_bwd": 1966}

WORKLOADS = {
    # name: (op, B, T, H, K, V)
    "gdn": ("gated_delta", 8, 4096, 16, 128, 128),
    "delta": ("delta", 8, 4096, 16, 128, 128),
    "retention": ("simple_gla", 8, 4096, 16, 128, 128),
    "gla_fp32": ("gla", 2, 512, 4, 64, 64),
    "gla": ("gla", 8, 4096, 16, 128, 128),  # not a listed configuration: the GLA kernels at the shape of the others
    # 64 sequences of 256..8192 tokens (seeded), packed into one row with cu_seqlens, H=32
    "varlen": ("gated_delta_varlen", 1, 0, 32, 128, 128),
    # one decode step of 256 sequences: fused_recurrent_gated_delta_rule, T = 1, fp32 state carried
    "decode": ("decode", 256, 1, 16, 128, 128),
    # one long sequence (a quarter of the 2^20-token configuration, so that the host-side input generation stays short):
    # 16 (sequence, head) chains only, the scans run split into slabs of T
    "long": ("gated_delta", 1, 262144, 16, 128, 128),
    # the step before the op in the reference's layers: l2_norm of q and of k, forward and backward (4 launches)
    "l2norm": ("l2norm", 8, 4096, 16, 128, 128),
    # the step after the op: RMS norm with weight times swish gate on the op's output, forward and backward (2 launches)
    "norm_gate": ("norm_gate", 8, 4096, 16, 128, 128),
    # the convolution in front of q (or k, v): [B, T, H * D] channels-last, filter of 4, SiLU, forward and backward
    "short_conv": ("short_conv", 8, 4096, 16, 128, 128),
}


def varlen_lengths():
    g0 = torch.Generator().manual_seed(0)
    return torch.randint(256, 8193, (64,), generator=g0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def make_inputs(op, B, T, H, K, V, seed, dtype):
    """Seeded synthetic inputs (CPU generator, so every implementation sees identical bits)."""
    g0 = torch.Generator().manual_seed(seed)
    q, k = torch.randn(B, T, H, K, generator=g0), torch.randn(B, T, H, K, generator=g0)
    v = torch.randn(B, T, H, V, generator=g0)
    d = {}
    if op in ("gated_delta_varlen", "decode"):
        q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
        d["beta"] = torch.randn(B, T, H, generator=g0).sigmoid().to(dtype)
        d["g"] = F.logsigmoid(torch.randn(B, T, H, generator=g0))
        n_seq = 64 if op == "gated_delta_varlen" else B
        d["h0"] = torch.randn(n_seq, H, K, V, generator=g0) * 0.1
        if op == "gated_delta_varlen":
            d["offsets"] = torch.cat([torch.zeros(1, dtype=torch.long), varlen_lengths().cumsum(0)]).int()
    if op in ("gated_delta", "delta"):
        q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
        d["beta"] = torch.randn(B, T, H, generator=g0).sigmoid().to(dtype)
        d["h0"] = torch.randn(B, H, K, V, generator=g0) * 0.1
    if op == "gated_delta":
        d["g"] = F.logsigmoid(torch.randn(B, T, H, generator=g0))
    if op == "simple_gla":
        # per-head decay log(1 - 2^(-5 - h*7/16)), constant along T
        s = (1 - torch.tensor(2.).pow(-5. - torch.arange(H, dtype=torch.float) * 7 / 16)).log()
        d["g"] = s[None, None, :].expand(B, T, H).contiguous()
    if op == "gla":
        d["g"] = F.logsigmoid(torch.randn(B, T, H, K, generator=g0)) / 16
        d["h0"] = torch.zeros(B, H, K, V)
    d.update(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype))
    d["do"] = torch.randn(B, T, H, V, generator=g0).to(dtype)
    if "h0" in d:
        d["dht"] = torch.randn(d["h0"].shape, generator=g0)
    return d


GRAD_NAMES = {"gated_delta_varlen": ["q", "k", "v", "g", "beta", "h0"], "decode": [], "l2norm": ["q", "k"], "norm_gate": ["q", "k"], "short_conv": ["q"],
              "gated_delta": ["q", "k", "v", "g", "beta", "h0"], "delta": ["q", "k", "v", "beta", "h0"],
              "simple_gla": ["q", "k", "v", "g"], "gla": ["q", "k", "v", "g", "h0"]}


def call_op(op, i, mod):
    """mod = fla_b200.ops (CUDA) or the oracle (CPU)."""
    st = "h0" in i
    if mod == "oracle":
        import oracle
        if op == "gated_delta":
            return oracle.gated_delta_rule(i["q"], i["k"], i["v"], i["beta"], g=i["g"], initial_state=i["h0"], output_final_state=True, head_first=False)
        if op == "delta":
            return oracle.delta_rule(i["q"], i["k"], i["v"], i["beta"], initial_state=i["h0"], output_final_state=True, head_first=False)
        if op == "simple_gla":
            return oracle.simple_gla(i["q"], i["k"], i["v"], i["g"], head_first=False)
        return oracle.gla(i["q"], i["k"], i["v"], gk=i["g"], initial_state=i["h0"], output_final_state=True, head_first=False)
    import fla_b200.ops as o
    if op == "gated_delta_varlen":
        return o.chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"], output_final_state=True,
                                        cu_seqlens=i["offsets"], head_first=False)
    if op == "decode":
        return o.fused_recurrent_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"],
                                                  output_final_state=True, head_first=False)
    if op == "gated_delta":
        return o.chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"], output_final_state=st, head_first=False)
    if op == "delta":
        return o.chunk_delta_rule(i["q"], i["k"], i["v"], i["beta"], initial_state=i["h0"], output_final_state=st, head_first=False)
    if op == "simple_gla":
        return o.chunk_simple_gla(i["q"], i["k"], i["v"], i["g"], head_first=False)
    return o.chunk_gla(i["q"], i["k"], i["v"], i["g"], initial_state=i["h0"], output_final_state=st, head_first=False)


def fwd_bwd(op, i, mod="ours"):
    if op == "l2norm":
        from fla_b200.modules import l2_norm
        i["q"].grad = i["k"].grad = None
        yq, yk = l2_norm(i["q"]), l2_norm(i["k"])
        torch.autograd.backward([yq, yk], [i["do"], i["do"]])
        return yq, yk
    if op == "short_conv":
        i["q"].grad = None
        i["conv"].weight.grad = None
        y, _ = i["conv"](i["q"].view(i["q"].shape[0], i["q"].shape[1], -1))
        torch.autograd.backward([y], [i["do"].view(y.shape)])
        return y, None
    if op == "norm_gate":  # x = "q", gate = "k" (same shape as the op's output at K = V)
        from fla_b200.modules import rms_norm_swish_gate_fn
        i["q"].grad = i["k"].grad = i["w"].grad = None
        y = rms_norm_swish_gate_fn(i["q"], i["k"], i["w"], eps=1e-5)
        torch.autograd.backward([y], [i["do"]])
        return y, None
    if op == "decode":  # forward only; the new state replaces the old one
        o, ht = call_op(op, i, mod)
        i["h0"] = ht
        return o, ht
    for n in GRAD_NAMES[op]:
        i[n].grad = None
    o, ht = call_op(op, i, mod)
    outs, gouts = [o], [i["do"]]
    if ht is not None:
        outs.append(ht)
        gouts.append(i["dht"])
    torch.autograd.backward(outs, gouts)
    return o, ht


# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.stop_flag, self.thread = index, [], False, None

    def _run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop_flag = True
        self.thread.join(timeout=6)

    def summary(self):
        mhz = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, val in zip(names, s[2:6]) if val.lower().startswith("active")})
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def time_stage(fn, reps=10, warm=3):
    """Average device time of fn() in ms (CUDA events on the current stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    # one event pair per call and the median over calls: a call that makes the caching allocator go to the driver
    # (a device-wide stall that is not the kernel's) does not leak into the stage's figure
    evs = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    return statistics.median(x.elapsed_time(y) for x, y in evs)


def stage_breakdown(op, i):
    """Times every stage of the op's forward+backward on its own; returns
    {stage: dict(ms, launches_per_step, bytes, flops)} (algorithmic bytes / dense-tile flops per launch)."""
    from fla_b200.ops import common as C
    from fla_b200.utils import Geometry
    if op not in ("gated_delta", "delta", "simple_gla"):
        return {}
    q, k, v, do = (i[n].detach() for n in ("q", "k", "v", "do"))
    geo = Geometry(k, v, None, False)
    B, T, H, K, V = geo.B, geo.T, geo.H, geo.K, geo.V
    TH = B * T * H
    scale = K ** -0.5
    e = 2  # bytes per bf16 element
    st = K * V * e / 64  # chunk-state bytes per token*head
    table = {}
    if op == "simple_gla":
        g = i["g"].detach()
        gc = C.chunk_local_cumsum(g, head_first=False)
        h, _ = C.chunk_fwd_h(geo, k, v, g=gc)
        dh, _ = C.chunk_bwd_dh(geo, q, do, scale, g=gc)
        table = {
            "cumsum": (lambda: C.chunk_local_cumsum(g, head_first=False), 2, 8, 0),
            "chunk_fwd_h": (lambda: C.chunk_fwd_h(geo, k, v, g=gc), 1, (K + V) * e + 4 + st, 2 * K * V),
            "chunk_fwd_o": (lambda: C.chunk_fwd_o(geo, q, k, v, h, g=gc, scale=scale), 1, (2 * K + 2 * V) * e + 4 + st, 2 * K * V + 2 * 64 * K + 2 * 64 * V),
            "chunk_bwd_dh": (lambda: C.chunk_bwd_dh(geo, q, do, scale, g=gc), 1, (K + V) * e + 4 + st, 2 * K * V),
            "dqkwg": (lambda: C.chunk_bwd_dqkwg(geo, q, k, v, h, dh, do, scale, g=gc), 1, (4 * K + 2 * V) * e + 8 + 2 * st, 4 * K * V + 2 * 64 * V + 6 * 64 * K),
            "chunk_bwd_dv": (lambda: C.chunk_bwd_dv(geo, q, k, gc, do, dh, scale), 1, (2 * K + 2 * V) * e + 4 + st, 2 * K * V + 2 * 64 * K + 2 * 64 * V),
        }
    else:
        beta, h0, dht = (i[n].detach() for n in ("beta", "h0", "dht"))
        gated = op == "gated_delta"
        gc = C.chunk_local_cumsum(i["g"].detach(), head_first=False) if gated else None
        aw, au, w, u = C.fwd_prepare_wy_repr(geo, k, v, beta, g=gc)
        h, v_new, _ = C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, g=gc, h0=h0, output_final_state=True)
        dv = C.chunk_bwd_dv_local(geo, q, k, gc, do, scale)
        dh, dh0, dv2 = C.chunk_gated_delta_rule_bwd_dhu(geo, q, k, w, do, dv, scale, g=gc, dht=dht, want_dh0=True)
        dq, dk, dw, dg = C.chunk_bwd_dqkwg(geo, q, k, v_new, h, dh, do, scale, g=gc, w=w, dv=dv2)
        na = 2 if gated else 1
        table = {
            "wy_fwd": (lambda: C.fwd_prepare_wy_repr(geo, k, v, beta, g=gc), 1, (2 * K + 2 * V) * e + na * 64 * e + 6, 2 * 64 * K + 2 * 64 * (K + V) + 2 * 64 * 64),
            "delta_fwd_h": (lambda: C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, g=gc, h0=h0, output_final_state=True), 1, (2 * K + 2 * V) * e + 4 + st, 4 * K * V),
            "chunk_fwd_o": (lambda: C.chunk_fwd_o(geo, q, k, v_new, h, g=gc, scale=scale), 1, (2 * K + 2 * V) * e + 4 + st, 2 * K * V + 2 * 64 * K + 2 * 64 * V),
            "dv_local": (lambda: C.chunk_bwd_dv_local(geo, q, k, gc, do, scale), 1, (2 * K + 2 * V) * e + 4, 2 * 64 * K + 2 * 64 * V),
            "delta_bwd_dhu": (lambda: C.chunk_gated_delta_rule_bwd_dhu(geo, q, k, w, do, dv, scale, g=gc, dht=dht, want_dh0=True), 1, (3 * K + 3 * V) * e + 4 + st, 6 * K * V),
            "dqkwg": (lambda: C.chunk_bwd_dqkwg(geo, q, k, v_new, h, dh, do, scale, g=gc, w=w, dv=dv2), 1, (6 * K + 3 * V) * e + 8 + 2 * st, 6 * K * V + 2 * 64 * V + 6 * 64 * K),
            "wy_bwd": (lambda: C.bwd_prepare_wy_repr(geo, k, v, beta, aw, dw, dv2, g=gc, au=au), 1, (4 * K + 4 * V) * e + na * 64 * e + 14, 8 * 64 * K + 4 * 64 * V + 8 * 64 * 64),
        }
        if gated:
            g = i["g"].detach()
            table["cumsum"] = (lambda: C.chunk_local_cumsum(g, head_first=False), 2, 8, 0)
    out = {}
    for name, (fn, launches, bytes_th, flops_th) in table.items():
        ms = time_stage(fn)
        out[name] = dict(ms=ms, launches_per_step=launches, bytes=bytes_th * TH, flops=flops_th * TH)
    return out


def cpu_sample(op, B, T, H, K, V, dtype, steps=1, warmup=0):
    """Oracle (CPU port of the reference's naive recurrence) forward+backward on a T-truncated sample."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Ts = min(T, 128 if op != "gla" else T)
    i = make_inputs(op, B, Ts, H, K, V, 0, dtype)
    i = {n: x.float() for n, x in i.items()}
    for n in GRAD_NAMES[op]:
        i[n].requires_grad_(True)
    times = []
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        fwd_bwd(op, i, "oracle")
        if s >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return dict(value=B * Ts / sec, unit=UNIT, cores=cores, kind="port",
                sample=f"{op} fwd+bwd via the oracle, fp32, B={B} T={Ts} (of {T}) H={H} K={K} V={V}, {len(times)} pass(es) of {sec:.2f} s"), sec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gdn", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip e2e / roofline / cpu_baseline legs")
    ap.add_argument("--seq-len", type=int, default=0, help="override T (small cases for profiler captures)")
    args = ap.parse_args()
    op, B, T, H, K, V = WORKLOADS[args.workload]
    T = args.seq_len or T
    if op == "gated_delta_varlen":
        T = int(varlen_lengths().sum())
    dtype = torch.float32 if args.workload == "gla_fp32" else torch.bfloat16
    if op in ("gated_delta_varlen", "decode", "l2norm", "norm_gate", "short_conv") or args.workload == "long":
        args.no_extras = True  # side workloads: device-resident timing (and the decode roofline) only
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    config = {"workload": f"{'fused_recurrent_gated_delta_rule decode step' if op == 'decode' else 'chunk_' + op + ' fwd+bwd'} {str(dtype).split('.')[-1]} B={B} T={T} H={H} K={K} V={V} seq-first, "
              f"initial_state given, output_final_state=True, per GPU", "timing": "inputs (>600 MB) larger than the 126 MB L2",
              "parallelism": f"{world} independent per-GPU batches (sequence x head shards, no collective)"}

    if args.impl == "reference":
        if rank != 0:
            return
        base, sec = cpu_sample(op, B, T, H, K, V, dtype, steps=max(1, min(args.steps, 3)), warmup=min(args.warmup, 1))
        line = {"impl": "reference", "metric": SIDE_METRICS.get(args.workload, METRIC), "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": base, "gpu_launches": 0,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from fla_b200 import _lib

    host = make_inputs(op, B, T, H, K, V, 1000 + rank, dtype)
    pinned = {n: x.pin_memory() for n, x in host.items()}
    i = {n: x.to(dev) for n, x in host.items()}
    for n in GRAD_NAMES[op]:
        i[n].requires_grad_(True)
    if op == "norm_gate":
        i["w"] = torch.ones(K, device=dev, requires_grad=True)
    if op == "short_conv":
        from fla_b200.modules import ShortConvolution
        i["conv"] = ShortConvolution(H * K, 4, activation="silu").to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # L2 hygiene: a step whose tensors exceed the 126 MB L2 evicts its own inputs; a small one gets an explicit
    # flush (a 256 MB write) between timed iterations, outside the events that are summed.
    in_bytes = sum(x.numel() * x.element_size() for x in i.values() if isinstance(x, torch.Tensor))
    flush = None
    if in_bytes < 256 * 2 ** 20:
        flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)
    config["timing"] = (f"inputs {in_bytes / 2 ** 20:.0f} MB > 126 MB L2, no flush needed" if flush is None
                        else f"inputs {in_bytes / 2 ** 20:.1f} MB: L2 flushed (256 MB write) between timed iterations")
    for _ in range(max(args.warmup, 3)):
        fwd_bwd(op, i)
    barrier()
    launches0 = _lib.LAUNCHES
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        barrier()
        if flush is None:
            a.record()
            for _ in range(args.steps):
                fwd_bwd(op, i)
            b.record()
            barrier()
            ms_total = a.elapsed_time(b)
        else:
            evs = []
            for _ in range(args.steps):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fwd_bwd(op, i)
                e1.record()
                evs.append((e0, e1))
            barrier()
            ms_total = sum(x.elapsed_time(y) for x, y in evs)
    launches = (_lib.LAUNCHES - launches0) // args.steps
    if world > 1:
        tmax = torch.tensor([ms_total], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms_total = tmax.item()
    ms_step = ms_total / args.steps
    tokens = B * T * world
    value = tokens / (ms_step * 1e-3)

    line = {"metric": SIDE_METRICS.get(args.workload, METRIC) if not args.seq_len else f"{SIDE_METRICS.get(args.workload, METRIC)} at T={T}", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "data": "synthetic", "config": config,
            "clocks": clk.summary(), "gpu_launches": launches}

    if op == "l2norm" and rank == 0:
        # pure streaming: forward reads x and writes y, backward reads x and dy and writes dx. The step above also pays
        # the autograd and launch overhead of four small calls, so the kernels are timed on their own as well.
        from fla_b200.modules.l2norm import l2norm_bwd, l2norm_fwd
        pk = peaks()
        xq, dyq = i["q"].detach(), i["do"]
        ms_f = time_stage(lambda: l2norm_fwd(xq), reps=30, warm=5)
        ms_b = time_stage(lambda: l2norm_bwd(xq, dyq), reps=30, warm=5)
        tensor_bytes = B * T * H * K * 2
        ach_f, ach_b = 2 * tensor_bytes / (ms_f * 1e-3) / 1e9, 3 * tensor_bytes / (ms_b * 1e-3) / 1e9
        line["roofline"] = {"kernel": "l2norm_bwd_vec_kernel", "bound": "hbm", "achieved": ach_b, "peak": pk["hbm_gbs"], "unit": "GB/s",
                            "frac": ach_b / pk["hbm_gbs"], "traffic": 371e6 if (B, T, H, K) == (8, 4096, 16, 128) else None,
                            "traffic_source": "ncu, same workload (profiles/streaming_modules_ncu_dram.md)", "peak_source": pk["source"],
                            "ms_per_launch": ms_b}
        line["kernels"] = {"l2norm_fwd_vec_kernel": {"ms": ms_f, "GB/s": ach_f, "frac": ach_f / pk["hbm_gbs"]},
                           "l2norm_bwd_vec_kernel": {"ms": ms_b, "GB/s": ach_b, "frac": ach_b / pk["hbm_gbs"]}}
    if op in ("short_conv", "norm_gate") and rank == 0:
        # streaming kernels of 0.05 - 0.2 ms: through the modules the Python side of a call costs as much as the kernel, so the
        # kernels are also timed through the C entry points on preallocated buffers (pointers taken once)
        pk = peaks()
        lib = _lib.load()
        st = torch.cuda.current_stream().cuda_stream
        tb = B * T * H * K * 2  # bytes of one [B, T, H * K] bf16 tensor
        x, dyv = i["q"].detach(), i["do"]
        y, dx = torch.empty_like(x), torch.empty_like(x)
        if op == "short_conv":
            w32 = i["conv"].weight.detach().float().reshape(H * K, 4).contiguous()
            dw = torch.zeros_like(w32)
            P = [t_.data_ptr() for t_ in (x, w32, y, dyv, dx, dw)]
            ms_f = time_stage(lambda: lib.flab_short_conv_fwd(P[0], P[1], None, P[2], B, T, H * K, 4, 1, 0, st), reps=30, warm=5)
            ms_b = time_stage(lambda: lib.flab_short_conv_bwd(P[0], P[1], None, P[3], P[4], P[5], None, B, T, H * K, 4, 1, 0, st), reps=30, warm=5)
            nf, nb, names = 2, 3, ("short_conv_fwd_kernel", "short_conv_bwd_kernel")
        else:
            g, w32 = i["k"].detach(), i["w"].detach()
            rows = B * T * H
            rstd, dg = torch.empty(rows, device=dev), torch.empty_like(x)
            parts = lib.flab_rms_norm_swish_gate_partials(rows, K, 0)
            dwp = torch.empty(parts, K, device=dev)
            P = [t_.data_ptr() for t_ in (x, g, w32, y, rstd, dyv, dx, dg, dwp)]
            ms_f = time_stage(lambda: lib.flab_rms_norm_swish_gate_fwd(P[0], P[1], P[2], P[3], P[4], rows, K, 0, 1e-5, st), reps=30, warm=5)
            ms_b = time_stage(lambda: lib.flab_rms_norm_swish_gate_bwd(P[0], P[1], P[2], P[5], P[4], P[6], P[7], P[8], rows, K, 0, st), reps=30, warm=5)
            nf, nb, names = 3, 5, ("norm_gate_fwd_vec_kernel", "norm_gate_bwd_vec_kernel")
        ach_f, ach_b = nf * tb / (ms_f * 1e-3) / 1e9, nb * tb / (ms_b * 1e-3) / 1e9
        # DRAM read + write per launch of the backward kernel at this shape (profiles/streaming_modules_ncu_dram.md)
        traffic = {"short_conv": 379e6, "norm_gate": 635e6}[op] if (B, T, H, K) == (8, 4096, 16, 128) else None
        line["roofline"] = {"kernel": names[1], "bound": "hbm", "achieved": ach_b, "peak": pk["hbm_gbs"], "unit": "GB/s",
                            "frac": ach_b / pk["hbm_gbs"], "traffic": traffic, "traffic_source": "ncu, same workload",
                            "peak_source": pk["source"], "ms_per_launch": ms_b}
        line["kernels"] = {names[0]: {"ms": ms_f, "GB/s": ach_f, "frac": ach_f / pk["hbm_gbs"]},
                           names[1]: {"ms": ms_b, "GB/s": ach_b, "frac": ach_b / pk["hbm_gbs"]}}
    if op == "decode" and rank == 0:
        # the decode kernel alone (the public-API step above also pays Python / launch overhead per call)
        from fla_b200.ops.recurrent import recurrent_delta_fwd
        from fla_b200.utils import Geometry
        geo = Geometry(i["k"], i["v"], None, False)
        h0 = i["h0"].float().contiguous()
        ms_k = time_stage(lambda: recurrent_delta_fwd(geo, i["q"], i["k"], i["v"], i["beta"], i["g"], K ** -0.5, h0, True, False),
                          reps=50, warm=5)
        pk = peaks()
        nbytes = B * H * (2 * K * V * 4 + (2 * K + 2 * V) * 2 + 8)
        ach = nbytes / (ms_k * 1e-3) / 1e9
        line["roofline"] = {"kernel": "recurrent_stream_kernel (decode)", "bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"],
                            "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "traffic": 485e6,
                            "traffic_source": "ncu, same workload (profiles/decode_stream_kernel_ncu_full.md)", "peak_source": pk["source"],
                            "ms_per_launch": ms_k}
        # the same step replayed from a CUDA graph (fla_b200.decode): fixed buffers, state updated in place
        from fla_b200.decode import GatedDeltaRuleDecoder
        dec = GatedDeltaRuleDecoder(B, H, K, V, dtype=dtype, initial_state=h0)
        for n_ in ("q", "k", "v", "g", "beta"):
            getattr(dec, n_).copy_(i[n_].view_as(getattr(dec, n_)))
        ms_g = time_stage(dec.replay, reps=50, warm=5)
        line["graph_replay"] = {"ms_per_step": ms_g, "value": B / (ms_g * 1e-3), "unit": UNIT}

    # ---- end to end: host buffers in, every result back to the host, inside the timed region
    if not args.no_extras:
        grads_host = {n: torch.empty_like(host[n], dtype=(torch.float32 if n in ("g", "h0") else host[n].dtype)).pin_memory()
                      for n in GRAD_NAMES[op]}
        o_host = torch.empty_like(host["do"]).pin_memory()
        ht_host = torch.empty(B, H, K, V).pin_memory() if "h0" in host else None

        # Three streams (copy in, compute, copy out) and two device input sets: the host->device copy of step i+1
        # and the device->host copy of step i-1 run while step i computes; every step still moves all of its
        # inputs in and all of its results out inside the timed region.
        s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dev_in = [{n: torch.empty_like(x, device=dev) for n, x in pinned.items()} for _ in range(2)]
        for ds in dev_in:
            for n in GRAD_NAMES[op]:
                ds[n].requires_grad_(True)
        ev_free = [None, None]

        def e2e_step(step):
            ds = dev_in[step & 1]
            with torch.cuda.stream(s_in):
                if ev_free[step & 1] is not None:
                    s_in.wait_event(ev_free[step & 1])  # step - 2 has finished with this input set
                with torch.no_grad():
                    for n, x in pinned.items():
                        ds[n].copy_(x, non_blocking=True)
                e_in = torch.cuda.Event()
                e_in.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(e_in)
                for n in GRAD_NAMES[op]:
                    ds[n].grad = None
                o, ht = fwd_bwd(op, ds)
                e_c = torch.cuda.Event()
                e_c.record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(e_c)
                outs = [o.detach()] + ([ht.detach()] if ht is not None else []) + [ds[n].grad for n in GRAD_NAMES[op]]
                o_host.copy_(outs[0], non_blocking=True)
                if ht is not None:
                    ht_host.copy_(outs[1], non_blocking=True)
                for n in GRAD_NAMES[op]:
                    grads_host[n].copy_(ds[n].grad, non_blocking=True)
                for x in outs:
                    x.record_stream(s_out)
                e_o = torch.cuda.Event()
                e_o.record(s_out)
            ev_free[step & 1] = e_o
        for w_ in range(3):
            e2e_step(w_)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(s_in)
        for st_ in range(args.steps):
            e2e_step(3 + st_)
        b.record(s_out)
        barrier()
        e_ms = a.elapsed_time(b)
        if world > 1:
            tmax = torch.tensor([e_ms], device=dev)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            e_ms = tmax.item()
        h2d = sum(x.numel() * x.element_size() for x in pinned.values())
        d2h = o_host.numel() * o_host.element_size() + (ht_host.numel() * 4 if ht_host is not None else 0) + \
            sum(x.numel() * x.element_size() for x in grads_host.values())
        line["e2e"] = {"value": tokens / (e_ms / args.steps * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": d2h}

    if rank == 0 and not args.no_extras:
        pk = peaks()
        stages = stage_breakdown(op, i)
        if stages:
            top = max(stages, key=lambda s: stages[s]["ms"] * stages[s]["launches_per_step"])
            s = stages[top]
            t_hbm = s["bytes"] / (pk["hbm_gbs"] * 1e9)
            t_tc = s["flops"] / (pk["bf16_tflops"] * 1e12)
            if t_hbm >= t_tc:
                ach, peak, unit, bound = s["bytes"] / (s["ms"] * 1e-3) / 1e9, pk["hbm_gbs"], "GB/s", "hbm"
            else:
                ach, peak, unit, bound = s["flops"] / (s["ms"] * 1e-3) / 1e12, pk["bf16_tflops"], "TFLOP/s", "tensor"
            line["roofline"] = {"kernel": top, "bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                                "traffic": (NCU_BYTES_PER_TOKENHEAD[top] * B * T * H if op == "gated_delta" and top in NCU_BYTES_PER_TOKENHEAD else None),
                                "traffic_source": "ncu at T=2048 scaled by tokens (profiles/gdn_kernels_ncu_full_T2048.md)",
                                "peak_source": pk["source"], "ms_per_launch": s["ms"],
                                "tensor_frac": s["flops"] / (s["ms"] * 1e-3) / 1e12 / pk["bf16_tflops"]}
            line["stages_ms"] = {k_: round(v_["ms"] * v_["launches_per_step"], 4) for k_, v_ in stages.items()}
        line["cpu_baseline"], _ = cpu_sample(op, B, T, H, K, V, dtype)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
