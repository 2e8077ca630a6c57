#!/usr/bin/env python
"""Benchmark of the chunked linear-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward + backward pass of the op over one synthetic batch.  The default
workload is the configuration the headline metric is quoted on: chunk_gated_delta_rule, bf16,
B=8 T=4096 H=16 K=V=128, initial state given, final state requested.  With N > 1 (torchrun, one
rank per GPU) every rank runs the same per-GPU batch (sequences and heads are independent, so the
path shards with no data-path collective): weak scaling, value = tokens of all ranks / max time.

Prints ONE JSON line (rank 0):
  value            tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e              the same step with pinned host inputs copied in and every result copied back inside the timed region
  roofline         the stage kernel with the largest share of the step, timed alone (bytes / flops from STAGE_TABLE)
  roofline_step    the whole step against its compulsory bytes and algorithmic flops (WHOLE_OP)
  cpu_baseline     the CPU oracle (a port of the reference's naive recurrence) on a bounded sample
  triton_reference the reference's own Triton kernels (from baseline/_ref or $FLA_REFERENCE), same inputs, same GPU,
                   same process, with the relative L2 distance between its results and ours   (1 GPU only)
  configs          every benchmark configuration: ours, its roofline fractions, the reference's Triton time (1 GPU only)
  sp, varlen_shard the sequence-parallel long sequence and the token-balanced packed batch over the N ranks (N > 1 only)
`--impl reference` times the CPU oracle only: the reference's CPU implementation of the headline op lives in its
test suite (tests/ops/test_gated_delta.py:30), which is not part of its installed package, so the restated port is what
runs (`kind: "port"`); its Triton path needs a GPU and is reported by the default arm as `triton_reference`.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import types

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

# ------------------------------------------------------------------------------------------------
# THE byte / flop table (per token-head, 16-bit elements, K = V = 128, chunk of 64 tokens).  X = one [B,T,H,128] tensor
# = 256 B per token-head; a pass over the chunk states h or dh is K*V*2/64 = 512 B = 2X; A = one [B,T,H,64] tensor = 128 B.
# bytes = what the stage must read and write once (its inputs and outputs, nothing re-read); flops = dense-tile count,
# 1 MAC = 2 flops.  The design document quotes this table; nothing else in the repository defines these numbers.
# ------------------------------------------------------------------------------------------------
X, ST, A64 = 256, 512, 128
KV, CK, CV, CC = 128 * 128, 64 * 128, 64 * 128, 64 * 64


def stage_table(op):
    """{stage: (bytes per token-head, flops per token-head, launches per step)}"""
    if op == "simple_gla":
        return {
            "cumsum": (8, 0, 2),                                            # g in, b out (fp32); forward and reverse
            "chunk_fwd_h": (2 * X + 4 + ST, 2 * KV, 1),                     # k, v, b -> h
            "chunk_fwd_o": (3 * X + 4 + ST + X, 2 * KV + 2 * CK + 2 * CV, 1),   # q, k, v, b, h -> o
            "chunk_bwd_dh": (2 * X + 4 + ST, 2 * KV, 1),                    # q, do, b -> dh
            "dqkwg": (4 * X + 4 + 2 * ST + 2 * X + 4, 4 * KV + 2 * CV + 6 * CK, 1),   # q, k, v, do, b, h, dh -> dq, dk, dg
            "chunk_bwd_dv": (3 * X + 4 + ST + X, 2 * KV + 2 * CK + 2 * CV, 1),  # q, k, do, b, dh -> dv
        }
    gated = op == "gated_delta"
    na = 2 if gated else 1           # inverse factors stored: Aw (and Au with gates)
    gb = 4 if gated else 0           # the cumsummed gate, fp32
    t = {
        "wy_fwd": (2 * X + 2 + gb + 2 * X + na * A64, 2 * CK + 2 * 64 * (128 + 128) + 2 * CC, 1),   # k, v, beta, b -> w, u, Aw, Au
        "delta_fwd_h": (3 * X + gb + ST + X, 4 * KV, 1),                    # k, w, u, b -> h, v_new
        "chunk_fwd_o": (3 * X + gb + ST + X, 2 * KV + 2 * CK + 2 * CV, 1),  # q, k, v_new, b, h -> o
        "dv_local": (3 * X + gb + X, 2 * CK + 2 * CV, 1),                   # q, k, do, b -> dv
        "delta_bwd_dhu": (5 * X + gb + ST + X, 6 * KV, 1),                  # q, k, w, do, dv, b -> dh, dv2
        "dqkwg": (6 * X + gb + 2 * ST + 3 * X + gb, 6 * KV + 2 * CV + 6 * CK, 1),   # q, k, w, v_new, do, dv2, b, h, dh -> dq, dk, dw, dg
        "wy_bwd": (5 * X + na * A64 + 2 + 2 * gb + 2 * X + 4 + gb, 8 * CK + 4 * CV + 8 * CC, 1),  # k, v, dw, dv2, dk, Aw, Au, beta, b, dg(dqkwg) -> dk, dv, dbeta, dg
    }
    if gated:
        t["cumsum"] = (8, 0, 1)  # forward only: the reverse cumsum of dg is done by the last backward kernel
    return t


# compulsory bytes (inputs read once, outputs and gradients written once) and algorithmic flops per token-head of the
# WHOLE forward + backward: fla's published operation counts restated (dense 64 x 64 tiles counted in full)
WHOLE_OP = {
    "simple_gla": (22 * 128 + 8, 12 * KV + 8 * CK + 6 * CV),
    "retention": (22 * 128, 12 * KV + 8 * CK + 6 * CV),
    "delta": (22 * 128 + 4, 18 * KV + 20 * CK + 12 * CV + 4 * CC),
    "gated_delta": (22 * 128 + 12, 18 * KV + 22 * CK + 12 * CV + 8 * CC),
    "gated_delta_varlen": (22 * 128 + 12, 18 * KV + 22 * CK + 12 * CV + 8 * CC),
}


def whole_op(op, K, V, dtype):
    if op == "gla":  # the 22 D of the scalar-gate ops plus the per-channel gate in and its gradient out, in the element size
        e = 4 if dtype == torch.float32 else 2
        return (e * 24 * (K + V) // 2, 12 * K * V + 6 * 64 * K + 6 * 64 * V)
    if op == "decode":  # per (sequence, head): the fp32 state in and out, q k v o, g and beta
        return (2 * K * V * 4 + (2 * K + 2 * V) * 2 + 8, 6 * K * V)
    return WHOLE_OP[op]


def varlen_lengths():
    g0 = torch.Generator().manual_seed(0)
    return torch.randint(256, 8193, (64,), generator=g0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def make_inputs(op, B, T, H, K, V, seed, dtype, device="cpu", offsets=None):
    """Seeded synthetic inputs.  On the CPU generator every implementation sees identical bits; the large side workloads
    are generated on the device (`device="cuda"`) with the same distributions."""
    g0 = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g0, device=device)  # noqa: E731
    q, k = rn(B, T, H, K), rn(B, T, H, K)
    v = rn(B, T, H, V)
    d = {}
    if op in ("gated_delta_varlen", "decode"):
        q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
        d["beta"] = rn(B, T, H).sigmoid().to(dtype)
        d["g"] = F.logsigmoid(rn(B, T, H))
        if op == "gated_delta_varlen":
            off = offsets if offsets is not None else torch.cat([torch.zeros(1, dtype=torch.long), varlen_lengths().cumsum(0)])
            d["offsets"] = off.int().to(device)
            n_seq = off.numel() - 1
        else:
            n_seq = B
        d["h0"] = rn(n_seq, H, K, V) * 0.1
    if op in ("gated_delta", "delta"):
        q, k = F.normalize(q, p=2, dim=-1), F.normalize(k, p=2, dim=-1)
        d["beta"] = rn(B, T, H).sigmoid().to(dtype)
        d["h0"] = rn(B, H, K, V) * 0.1
    if op == "gated_delta":
        d["g"] = F.logsigmoid(rn(B, T, H))
    if op in ("simple_gla", "retention"):
        # simple_gla: per-head decay log(1 - 2^(-5 - h*7/16)), constant along T; retention uses its native decay
        s = (1 - torch.tensor(2.).pow(-5. - torch.arange(H, dtype=torch.float) * 7 / 16)).log().to(device)
        d["g"] = s[None, None, :].expand(B, T, H).contiguous()
    if op == "gla":
        d["g"] = F.logsigmoid(rn(B, T, H, K)) / 16
        d["h0"] = torch.zeros(B, H, K, V, device=device)
    d.update(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype))
    d["do"] = rn(B, T, H, V).to(dtype)
    if "h0" in d:
        d["dht"] = rn(*d["h0"].shape)
    return d


GRAD_NAMES = {"gated_delta_varlen": ["q", "k", "v", "g", "beta", "h0"], "decode": [], "l2norm": ["q", "k"], "norm_gate": ["q", "k"], "short_conv": ["q"],
              "gated_delta": ["q", "k", "v", "g", "beta", "h0"], "delta": ["q", "k", "v", "beta", "h0"],
              "simple_gla": ["q", "k", "v", "g"], "retention": ["q", "k", "v"], "gla": ["q", "k", "v", "g", "h0"]}


def call_op(op, i, mod):
    """mod = our package ("ours"), the CPU oracle ("oracle") or a dict of the reference's Triton functions."""
    st = "h0" in i
    if mod == "oracle":
        import oracle
        if op == "gated_delta":
            return oracle.gated_delta_rule(i["q"], i["k"], i["v"], i["beta"], g=i["g"], initial_state=i["h0"], output_final_state=True, head_first=False)
        if op == "delta":
            return oracle.delta_rule(i["q"], i["k"], i["v"], i["beta"], initial_state=i["h0"], output_final_state=True, head_first=False)
        if op in ("simple_gla", "retention"):
            return oracle.simple_gla(i["q"], i["k"], i["v"], i["g"], head_first=False)
        return oracle.gla(i["q"], i["k"], i["v"], gk=i["g"], initial_state=i["h0"], output_final_state=True, head_first=False)
    if isinstance(mod, dict):
        o = types.SimpleNamespace(**mod)
        off = {"offsets": i["offsets"].long()} if "offsets" in i else {}
    else:
        import fla_b200.ops as o
        off = {"cu_seqlens": i["offsets"]} if "offsets" in i else {}
    if op == "gated_delta_varlen":
        return o.chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"], output_final_state=True,
                                        head_first=False, **off)
    if op == "decode":
        return o.fused_recurrent_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"],
                                                  output_final_state=True, head_first=False)
    if op == "gated_delta":
        return o.chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"], output_final_state=st, head_first=False)
    if op == "delta":
        return o.chunk_delta_rule(i["q"], i["k"], i["v"], i["beta"], initial_state=i["h0"], output_final_state=st, head_first=False)
    if op == "simple_gla":
        return o.chunk_simple_gla(i["q"], i["k"], i["v"], i["g"], head_first=False)
    if op == "retention":
        return o.chunk_retention(i["q"], i["k"], i["v"], head_first=False)
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
    """Samples SM clocks and throttle reasons while the measurements run: through NVML in a thread (a few hundred samples
    per second, read-only queries), or by polling nvidia-smi when NVML is not importable.  `mark()` / `window()` let
    the caller ask how many samples fell inside one timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, period=0.002):
        self.index, self.period, self.samples, self.stop_flag, self.thread = index, period, [], False, None
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            # CUDA_VISIBLE_DEVICES may renumber the devices: find the NVML handle by the PCI bus id of the CUDA device
            h = None
            if torch.cuda.is_available():
                bus = torch.cuda.get_device_properties(index).pci_bus_id if hasattr(torch.cuda.get_device_properties(index), "pci_bus_id") else None
                if bus is not None:
                    for j in range(pynvml.nvmlDeviceGetCount()):
                        hj = pynvml.nvmlDeviceGetHandleByIndex(j)
                        if pynvml.nvmlDeviceGetPciInfo(hj).bus == bus:
                            h = hj
                            break
            self.handle = h if h is not None else pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _sample_nvml(self):
        n = self.nvml
        mhz = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        r = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        names = []
        for name, bit in (("hw_slowdown", n.nvmlClocksEventReasonHwSlowdown), ("hw_thermal_slowdown", n.nvmlClocksEventReasonHwThermalSlowdown),
                          ("sw_thermal_slowdown", n.nvmlClocksEventReasonSwThermalSlowdown), ("sw_power_cap", n.nvmlClocksEventReasonSwPowerCap)):
            if r & bit:
                names.append(name)
        return (time.perf_counter(), float(mhz), float(mx), names)

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        s = [x.strip() for x in out.split(",")]
        names = [n for n, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], s[2:6])
                 if val.lower().startswith("active")]
        return (time.perf_counter(), float(s[0]), float(s[1]), names)

    def _run(self):
        while not self.stop_flag:
            try:
                self.samples.append(self._sample_nvml() if self.nvml is not None else self._sample_smi())
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop_flag = True
        self.thread.join(timeout=6)

    @staticmethod
    def mark():
        return time.perf_counter()

    def summary(self, t0=None, t1=None):
        sel = [s for s in self.samples if (t0 is None or s[0] >= t0) and (t1 is None or s[0] <= t1)]
        mhz = [s[1] for s in sel]
        mx = [s[2] for s in sel]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_min_mhz": min(mhz) if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted({n for s in sel for n in s[3]}), "samples": len(sel),
                "source": "nvml" if self.nvml is not None else "nvidia-smi"}


def time_stage(fn, reps=10, warm=3, flush=None):
    """Median device time of fn() in ms (one CUDA event pair per call on the current stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    # one event pair per call and the median over calls: a call that makes the caching allocator go to the driver
    # (a device-wide stall that is not the kernel's) does not leak into the stage's figure
    evs = []
    for _ in range(reps):
        if flush is not None:
            flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    return statistics.median(x.elapsed_time(y) for x, y in evs)


def stage_breakdown(op, i):
    """Times every stage of the op's forward+backward on its own; returns
    {stage: dict(ms, launches_per_step, bytes, flops)} (bytes / flops per launch from `stage_table`)."""
    from fla_b200.ops import common as C
    from fla_b200.utils import Geometry
    if op not in ("gated_delta", "delta", "simple_gla"):
        return {}
    q, k, v, do = (i[n].detach() for n in ("q", "k", "v", "do"))
    geo = Geometry(k, v, None, False)
    TH = geo.B * geo.T * geo.H
    scale = geo.K ** -0.5
    if op == "simple_gla":
        g = i["g"].detach()
        gc = C.chunk_local_cumsum(g, head_first=False)
        h, _ = C.chunk_fwd_h(geo, k, v, g=gc)
        dh, _ = C.chunk_bwd_dh(geo, q, do, scale, g=gc)
        fns = {
            "cumsum": lambda: C.chunk_local_cumsum(g, head_first=False),
            "chunk_fwd_h": lambda: C.chunk_fwd_h(geo, k, v, g=gc),
            "chunk_fwd_o": lambda: C.chunk_fwd_o(geo, q, k, v, h, g=gc, scale=scale),
            "chunk_bwd_dh": lambda: C.chunk_bwd_dh(geo, q, do, scale, g=gc),
            "dqkwg": lambda: C.chunk_bwd_dqkwg(geo, q, k, v, h, dh, do, scale, g=gc),
            "chunk_bwd_dv": lambda: C.chunk_bwd_dv(geo, q, k, gc, do, dh, scale),
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
        fns = {
            "wy_fwd": lambda: C.fwd_prepare_wy_repr(geo, k, v, beta, g=gc),
            "delta_fwd_h": lambda: C.chunk_gated_delta_rule_fwd_h(geo, k, w, u, g=gc, h0=h0, output_final_state=True),
            "chunk_fwd_o": lambda: C.chunk_fwd_o(geo, q, k, v_new, h, g=gc, scale=scale),
            "dv_local": lambda: C.chunk_bwd_dv_local(geo, q, k, gc, do, scale),
            "delta_bwd_dhu": lambda: C.chunk_gated_delta_rule_bwd_dhu(geo, q, k, w, do, dv, scale, g=gc, dht=dht, want_dh0=True),
            "dqkwg": lambda: C.chunk_bwd_dqkwg(geo, q, k, v_new, h, dh, do, scale, g=gc, w=w, dv=dv2),
            "wy_bwd": lambda: C.bwd_prepare_wy_repr(geo, k, v, beta, aw, dw, dv2, g=gc, au=au, dk_in=dk, dg_in=dg if gated else None),
        }
        if gated:
            g = i["g"].detach()
            fns["cumsum"] = lambda: C.chunk_local_cumsum(g, head_first=False)
    table = stage_table(op)
    out = {}
    for name, fn in fns.items():
        bytes_th, flops_th, launches = table[name]
        out[name] = dict(ms=time_stage(fn), launches_per_step=launches, bytes=bytes_th * TH, flops=flops_th * TH)
    return out


CPU_SAMPLE_T = 128  # tokens per sequence of the CPU sample (autograd through the recurrence keeps one state per token)


def cpu_sample(op, B, T, H, K, V, dtype, steps=3, warmup=1, budget_s=60.0):
    """Oracle (CPU port of the reference's naive recurrence) forward+backward on a T-truncated sample.
    Runs `warmup` untimed and up to `steps` timed passes, stopping early once `budget_s` is spent; returns the record
    (which states what really ran) and the mean seconds per pass."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Ts = min(T, CPU_SAMPLE_T if op != "gla" else T)
    i = make_inputs(op, B, Ts, H, K, V, 0, dtype)
    i = {n: x.float() for n, x in i.items()}
    for n in GRAD_NAMES[op]:
        i[n].requires_grad_(True)
    times, t_start, warm_done = [], time.perf_counter(), 0
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        fwd_bwd(op, i, "oracle")
        if s >= warmup:
            times.append(time.perf_counter() - t0)
        else:
            warm_done += 1
        if time.perf_counter() - t_start > budget_s and times:
            break
    sec = sum(times) / len(times)
    return dict(value=B * Ts / sec, unit=UNIT, cores=cores, kind="port", passes=len(times), warmup_passes=warm_done, sample_T=Ts,
                sample=f"{op} fwd+bwd via the CPU oracle (port of the reference's naive recurrence), fp32, the first {Ts} tokens of every "
                       f"sequence: B={B} T={Ts} (of {T}) H={H} K={K} V={V}; {warm_done} warm-up + {len(times)} timed pass(es), mean {sec:.3f} s"), sec


# ------------------------------------------------------------------------------------------------
# the reference's Triton kernels, from its own installed package
# ------------------------------------------------------------------------------------------------
def reference_ops():
    """The reference's public functions, imported from $FLA_REFERENCE or baseline/_ref through a stub parent package
    (its top-level __init__ imports model code that does not load under this image's transformers)."""
    ref = os.environ.get("FLA_REFERENCE") or os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "fla", "ops")):
        raise RuntimeError(f"no reference install at {ref}")
    if "fla" not in sys.modules:
        stub = types.ModuleType("fla")
        stub.__path__ = [os.path.join(ref, "fla")]
        sys.modules["fla"] = stub
    from fla.ops.delta_rule import chunk_delta_rule
    from fla.ops.gated_delta_rule import chunk_gated_delta_rule, fused_recurrent_gated_delta_rule
    from fla.ops.gla import chunk_gla
    from fla.ops.retention import chunk_retention
    from fla.ops.simple_gla import chunk_simple_gla
    return dict(chunk_delta_rule=chunk_delta_rule, chunk_gated_delta_rule=chunk_gated_delta_rule,
                fused_recurrent_gated_delta_rule=fused_recurrent_gated_delta_rule, chunk_gla=chunk_gla,
                chunk_retention=chunk_retention, chunk_simple_gla=chunk_simple_gla)


def rel_l2(ref, out):
    ref, out = ref.detach().double(), out.detach().double()
    return ((ref - out).square().mean().sqrt() / (ref.square().mean().sqrt() + 1e-30)).item()


def triton_vs_ours(op, i, tri, warm=10, reps=20, flush=None, parity=True):
    """Times the reference's Triton path on the inputs `i` (>= 10 warm-up steps let its autotuner finish) and, with
    `parity`, reports the relative L2 distance between its outputs / gradients and ours on the same bits."""
    rec = {}
    try:
        rec["ms"] = time_stage(lambda: fwd_bwd(op, i, tri), reps=reps, warm=warm, flush=flush)
        if parity and op != "decode":
            o_t, ht_t = fwd_bwd(op, i, tri)
            g_t = {n: i[n].grad.detach().clone() for n in GRAD_NAMES[op]}
            o_t, ht_t = o_t.detach().clone(), (None if ht_t is None else ht_t.detach().clone())
            o_o, ht_o = fwd_bwd(op, i, "ours")
            d = {"o": rel_l2(o_t, o_o)}
            if ht_t is not None:
                d["ht"] = rel_l2(ht_t, ht_o)
            for n in GRAD_NAMES[op]:
                d["d" + n] = rel_l2(g_t[n], i[n].grad)
            rec["ours_vs_triton_rel_l2"] = {n: float(f"{e:.3e}") for n, e in d.items()}
    except Exception as e:  # a kernel that does not compile or run on this GPU: record why
        rec["error"] = repr(e)[:400]
    return rec


def long_sequence_triton(i, tri, slab=65536, warm=2, reps=3):
    """The reference cannot take the 2^20-token sequence in one call (its kernels index chunk states with 32-bit
    offsets: NT*H*K*V = 2^32 here), so it is called slab by slab, chaining initial_state / final state through autograd."""
    def step():
        for n in GRAD_NAMES["gated_delta"]:
            i[n].grad = None
        S, outs = i["h0"], []
        T = i["q"].shape[1]
        for lo in range(0, T, slab):
            sl = slice(lo, min(lo + slab, T))
            o, S = tri["chunk_gated_delta_rule"](i["q"][:, sl], i["k"][:, sl], i["v"][:, sl], i["g"][:, sl], i["beta"][:, sl],
                                                 initial_state=S, output_final_state=True, head_first=False)
            outs.append(o)
        torch.autograd.backward([torch.cat(outs, 1), S], [i["do"], i["dht"]])
    try:
        return {"ms": time_stage(step, reps=reps, warm=warm), "how": f"{slab}-token slabs chained through initial_state"}
    except Exception as e:
        return {"error": repr(e)[:400]}


def configs_record(dev, tri, deadline):
    """Every benchmark configuration at one GPU: our time, tokens/s, fractions of the HBM and tensor roofs for the whole
    op (compulsory bytes / algorithmic flops of WHOLE_OP), and the reference's Triton time on the same inputs."""
    pk = peaks()
    out = {}
    cases = [
        ("c1_gla_fp32", "gla", 2, 512, 4, 64, 64, torch.float32),
        ("c2_retention", "retention", 8, 4096, 16, 128, 128, torch.bfloat16),
        ("c2_simple_gla", "simple_gla", 8, 4096, 16, 128, 128, torch.bfloat16),
        ("c3_delta", "delta", 8, 4096, 16, 128, 128, torch.bfloat16),
        ("c4_varlen", "gated_delta_varlen", 1, int(varlen_lengths().sum()), 32, 128, 128, torch.bfloat16),
        ("c5a_long", "gated_delta", 1, 1 << 20, 16, 128, 128, torch.bfloat16),
        ("c5b_decode", "decode", 256, 1, 16, 128, 128, torch.bfloat16),
    ]
    for name, op, B, T, H, K, V, dtype in cases:
        rec = {"shape": f"B={B} T={T} H={H} K={K} V={V} {str(dtype).split('.')[-1]}"}
        try:
            i = make_inputs(op, B, T, H, K, V, 7, dtype, device=dev)
            for n in GRAD_NAMES[op]:
                i[n].requires_grad_(True)
            nbytes = sum(x.numel() * x.element_size() for x in i.values())
            flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev) if nbytes < 256 * 2 ** 20 else None
            big = name == "c5a_long"
            ms = time_stage(lambda: fwd_bwd(op, i), reps=5 if big else 20, warm=3 if big else 5, flush=flush)
            tokens = B * T
            units = B * H if op == "decode" else B * T * H
            b_alg, f_alg = whole_op(op, K, V, dtype)
            rec.update(ms=ms, tokens_per_s=tokens / (ms * 1e-3), hbm_frac=b_alg * units / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                       tensor_frac=f_alg * units / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], bound="hbm",
                       l2=("flushed between iterations" if flush is not None else "inputs larger than L2"))
            if tri is None:
                rec["triton"] = {"error": "reference not importable"}
            elif time.perf_counter() > deadline:
                rec["triton"] = {"skipped": "time budget of the benchmark run spent"}
            elif big:
                rec["triton"] = long_sequence_triton(i, tri)
            else:
                rec["triton"] = triton_vs_ours(op, i, tri, flush=flush, parity=(op != "decode"))
            if "ms" in rec.get("triton", {}):
                rec["vs_triton"] = rec["triton"]["ms"] / ms
        except Exception as e:
            rec["error"] = repr(e)[:400]
        out[name] = rec
        del i
        torch.cuda.empty_cache()
    out["layer_path"] = layer_path_record(dev)
    torch.cuda.empty_cache()
    return out


def layer_path_record(dev):
    """The data path of the reference's Gated DeltaNet layer around the op (fla/layers/gated_deltanet.py:205-282), forward
    + backward at the headline shape: short convolution + SiLU on q, k, v -> L2 norm of q, k -> gate / beta prologue ->
    chunk_gated_delta_rule -> RMS norm x swish gate.  Timed twice: with the prologue as the reference writes it (five
    elementwise PyTorch kernels, the op's own cumsum launch) and with this library's fused prologue kernel."""
    from fla_b200.modules import ShortConvolution, gdn_gate_beta, l2_norm, rms_norm_swish_gate_fn
    from fla_b200.ops import chunk_gated_delta_rule
    B, T, H, D = 8, 4096, 16, 128
    g0 = torch.Generator(device=dev).manual_seed(11)
    rn = lambda *s: torch.randn(*s, generator=g0, device=dev)  # noqa: E731
    xs = {n: rn(B, T, H * D).bfloat16().requires_grad_(True) for n in ("q", "k", "v")}
    a, b = rn(B, T, H).bfloat16().requires_grad_(True), rn(B, T, H).bfloat16().requires_grad_(True)
    gate = rn(B, T, H, D).bfloat16().requires_grad_(True)
    A_log, dt_bias = torch.zeros(H, device=dev, requires_grad=True), torch.zeros(H, device=dev, requires_grad=True)
    w_norm = torch.ones(D, device=dev, requires_grad=True)
    convs = {n: ShortConvolution(H * D, 4, activation="silu").to(dev).bfloat16() for n in xs}
    do = rn(B, T, H, D).bfloat16()
    leaves = list(xs.values()) + [a, b, gate, A_log, dt_bias, w_norm] + [c.weight for c in convs.values()]

    def step(fused):
        for t_ in leaves:
            t_.grad = None
        q, k, v = (convs[n](xs[n])[0].view(B, T, H, D) for n in ("q", "k", "v"))
        q, k = l2_norm(q), l2_norm(k)
        if fused:
            g, beta = gdn_gate_beta(a, b, A_log, dt_bias)
        else:
            beta = b.sigmoid()
            g = -A_log.float().exp() * F.softplus(a.float() + dt_bias)
        o, _ = chunk_gated_delta_rule(q, k, v, g, beta, head_first=False)
        y = rms_norm_swish_gate_fn(o, gate, w_norm, eps=1e-5)
        torch.autograd.backward([y], [do])
    rec = {"shape": f"B={B} T={T} H={H} D={D} bf16, conv W=4"}
    try:
        rec["ms_reference_style_prologue"] = time_stage(lambda: step(False), reps=10, warm=3)
        rec["ms_fused_prologue"] = time_stage(lambda: step(True), reps=10, warm=3)
        rec["tokens_per_s"] = B * T / (rec["ms_fused_prologue"] * 1e-3)
    except Exception as e:
        rec["error"] = repr(e)[:400]
    return rec


# ------------------------------------------------------------------------------------------------
# the sharded configurations over N ranks
# ------------------------------------------------------------------------------------------------
def _max_over_ranks(x, dev):
    import torch.distributed as dist
    t = torch.tensor([float(x)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def sp_record(dev, rank, world, steps=5, warm=3):
    """ONE sequence of 2^20 tokens (H=16, K=V=128, bf16) cut into `world` contiguous slabs, forward + backward through
    `sp_chunk_gated_delta_rule`: per-rank scans, the [H,K,V] fp32 boundary states passed rank to rank (NCCL send/recv),
    a local correction pass.  Times: the whole step, and inside it the two hand-off chains and the two state-only passes."""
    import torch.distributed as dist
    from fla_b200 import parallel as P
    T, H, K, V = 1 << 20, 16, 128, 128
    Tr = T // world
    i = make_inputs("gated_delta", 1, Tr, H, K, V, 2000 + rank, torch.bfloat16, device=dev)
    names = ["q", "k", "v", "g", "beta"]
    for n in names + ["h0"]:
        i[n].requires_grad_(True)

    def step():
        for n in names + ["h0"]:
            i[n].grad = None
        o, ht = P.sp_chunk_gated_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], initial_state=i["h0"], output_final_state=True)
        torch.autograd.backward([o, ht], [i["do"], i["dht"]])
    for _ in range(warm):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    P.STAGE_EVENTS = {}
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = _max_over_ranks(a.elapsed_time(b) / steps, dev)
    stages = P.stage_times_ms()
    P.STAGE_EVENTS = None
    rec = {"workload": f"chunk_gated_delta_rule fwd+bwd, ONE sequence T={T} H={H} K=V={K} bf16, {world} slabs of {Tr} tokens",
           "ms_per_step": ms, "value": T / (ms * 1e-3), "unit": UNIT, "steps": steps, "warmup": warm,
           "handoff_bytes_per_hop": H * K * V * 4}
    for n in ("handoff_fwd", "handoff_bwd", "state_pass_fwd", "state_pass_bwd"):
        rec[n + "_ms"] = _max_over_ranks(stages.get(n, 0.0) / steps, dev)
    rec["handoff_share"] = (rec["handoff_fwd_ms"] + rec["handoff_bwd_ms"]) / ms
    return rec


def varlen_shard_record(dev, rank, world, steps=5, warm=3):
    """The packed variable-length configuration (64 seeded sequences of 256..8192 tokens, H=32) sharded over the ranks by
    the token-balanced partition of whole sequences (`shard_sequences`), every rank with its own re-based offsets."""
    import torch.distributed as dist
    from fla_b200.parallel import rebased_offsets, shard_sequences
    lens = [int(x) for x in varlen_lengths()]
    ids = shard_sequences(lens, world)[rank]
    off = rebased_offsets(lens, ids)
    Tr, H, K, V = int(off[-1]), 32, 128, 128
    i = make_inputs("gated_delta_varlen", 1, Tr, H, K, V, 3000 + rank, torch.bfloat16, device=dev, offsets=off)
    for n in GRAD_NAMES["gated_delta_varlen"]:
        i[n].requires_grad_(True)
    for _ in range(warm):
        fwd_bwd("gated_delta_varlen", i)
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fwd_bwd("gated_delta_varlen", i)
    b.record()
    dist.barrier()
    torch.cuda.synchronize()
    mine = a.elapsed_time(b) / steps
    ms = _max_over_ranks(mine, dev)
    toks = torch.zeros(world, device=dev)
    toks[rank] = Tr
    dist.all_reduce(toks)
    per_rank = [int(x) for x in toks.tolist()]
    return {"workload": f"chunk_gated_delta_rule fwd+bwd, 64 packed sequences ({sum(lens)} tokens) H={H} K=V={K} bf16, whole sequences "
                        f"partitioned over {world} ranks (longest first, least loaded rank)",
            "ms_per_step": ms, "value": sum(lens) / (ms * 1e-3), "unit": UNIT, "tokens_per_rank": per_rank,
            "imbalance": max(per_rank) / (sum(per_rank) / world), "steps": steps, "warmup": warm}


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gdn", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip e2e / roofline / cpu_baseline / triton / configs legs")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration and multi-rank records")
    ap.add_argument("--seq-len", type=int, default=0, help="override T (small cases for profiler captures)")
    args = ap.parse_args()
    t_begin = time.perf_counter()
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
        base, sec = cpu_sample(op, B, T, H, K, V, dtype, steps=max(1, args.steps), warmup=max(0, args.warmup), budget_s=90.0)
        config["reference_sample"] = (f"each timed pass covers the first {base['sample_T']} tokens of every sequence of the workload above "
                                      f"(B={B} T={base['sample_T']} of {T}); tokens/s of that sample")
        line = {"impl": "reference", "metric": SIDE_METRICS.get(args.workload, METRIC), "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": base["passes"], "warmup": base["warmup_passes"], "steps_requested": args.steps, "warmup_requested": args.warmup,
                "ms_per_step": sec * 1e3, "higher_is_better": True,
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
        from datetime import timedelta
        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=300))  # a failed rank ends the others' collectives soon
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
    clk = ClockSampler(local_rank)
    clk.__enter__()
    for _ in range(max(args.warmup, 3)):
        fwd_bwd(op, i)
    barrier()
    launches0 = _lib.LAUNCHES
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_region0 = clk.mark()
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
    t_region1 = clk.mark()
    launches = (_lib.LAUNCHES - launches0) // args.steps
    if world > 1:
        ms_total = _max_over_ranks(ms_total, dev)
    ms_step = ms_total / args.steps
    tokens = B * T * world
    value = tokens / (ms_step * 1e-3)

    line = {"metric": SIDE_METRICS.get(args.workload, METRIC) if not args.seq_len else f"{SIDE_METRICS.get(args.workload, METRIC)} at T={T}", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "data": "synthetic", "config": config,
            "gpu_launches": launches}
    pk = peaks()
    if op in WHOLE_OP or op in ("gla", "decode"):
        b_alg, f_alg = whole_op(op, K, V, dtype)
        units = (B * H if op == "decode" else B * T * H)  # per rank
        t_s = ms_step * 1e-3
        line["roofline_step"] = {
            "bytes_per_token_head": b_alg, "flops_per_token_head": f_alg,
            "hbm": {"achieved": b_alg * units / t_s / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": b_alg * units / t_s / 1e9 / pk["hbm_gbs"]},
            "tensor": {"achieved": f_alg * units / t_s / 1e12, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                       "frac": f_alg * units / t_s / 1e12 / pk["bf16_tflops"]},
            "bound": "hbm", "peak_source": pk["source"],
            "note": "whole forward+backward step against its compulsory bytes (inputs read once, outputs and gradients written once) "
                    "and algorithmic flops; 'tensor.frac' is the '% of tensor peak' of the metric"}

    if op == "l2norm" and rank == 0:
        # pure streaming: forward reads x and writes y, backward reads x and dy and writes dx. The step above also pays
        # the autograd and launch overhead of four small calls, so the kernels are timed on their own as well.
        from fla_b200.modules.l2norm import l2norm_bwd, l2norm_fwd
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
        nbytes = B * H * (2 * K * V * 4 + (2 * K + 2 * V) * 2 + 8)
        ach = nbytes / (ms_k * 1e-3) / 1e9
        line["roofline"] = {"kernel": "recurrent_stream_kernel (decode)", "bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"],
                            "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "traffic": 484e6,
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
            e_ms = _max_over_ranks(e_ms, dev)
        h2d = sum(x.numel() * x.element_size() for x in pinned.values())
        d2h = o_host.numel() * o_host.element_size() + (ht_host.numel() * 4 if ht_host is not None else 0) + \
            sum(x.numel() * x.element_size() for x in grads_host.values())
        e_step_s = e_ms / args.steps * 1e-3
        line["e2e"] = {"value": tokens / e_step_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "gbs_per_direction_per_gpu": max(h2d, d2h) / e_step_s / 1e9,
                       "note": "bound by the host link: all inputs in and o, ht and every gradient out each step; the ranks of one box share "
                               "the host's memory and PCIe root complexes"}
        del dev_in, grads_host, o_host

    if rank == 0 and not args.no_extras:
        stages = stage_breakdown(op, i)
        if stages:
            # the stage with the largest share of the step; shares within 2 % of the largest count as tied, ties go to the
            # name that sorts first, so that run-to-run jitter cannot flip the choice
            share = {s: stages[s]["ms"] * stages[s]["launches_per_step"] for s in stages}
            top_ms = max(share.values())
            top = sorted(s for s in share if share[s] >= 0.98 * top_ms)[0]
            s = stages[top]
            t_hbm = s["bytes"] / (pk["hbm_gbs"] * 1e9)
            t_tc = s["flops"] / (pk["bf16_tflops"] * 1e12)
            if t_hbm >= t_tc:
                ach, peak, unit, bound = s["bytes"] / (s["ms"] * 1e-3) / 1e9, pk["hbm_gbs"], "GB/s", "hbm"
            else:
                ach, peak, unit, bound = s["flops"] / (s["ms"] * 1e-3) / 1e12, pk["bf16_tflops"], "TFLOP/s", "tensor"
            ncu = NCU_BYTES_PER_TOKENHEAD.get(top) if op == "gated_delta" else None
            line["roofline"] = {"kernel": top, "bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                                "bytes_per_launch": s["bytes"], "traffic": (ncu * B * T * H if ncu else None),
                                "traffic_source": "ncu at T=2048 scaled by tokens (profiles/gdn_kernels_ncu_full_T2048.md)",
                                "peak_source": pk["source"], "ms_per_launch": s["ms"],
                                "tensor_frac": s["flops"] / (s["ms"] * 1e-3) / 1e12 / pk["bf16_tflops"]}
            line["stages_ms"] = {k_: round(share[k_], 4) for k_ in stages}
            line["stages_hbm_frac"] = {k_: round(v_["bytes"] / (v_["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3) for k_, v_ in stages.items()}
    clk.__exit__()
    line["clocks"] = clk.summary()
    line["clocks"]["samples_in_timed_region"] = clk.summary(t_region0, t_region1)["samples"]
    line["clocks"]["window"] = "warm-up, the timed steps, the end-to-end steps and the per-stage timings of this process"

    tri = None
    if rank == 0 and world == 1 and not args.no_extras:
        try:
            tri = reference_ops()
        except Exception as e:
            line["triton_reference"] = {"unavailable": repr(e)[:300]}
        if tri is not None:
            with ClockSampler(local_rank) as clk_t:
                rec = triton_vs_ours(op, i, tri)
            rec["clocks"] = clk_t.summary()
            rec["how"] = ("the reference's public chunk function from its installed package, same device tensors as `value`, 10 warm-up "
                          "(autotune) + 20 timed steps, one CUDA event pair per step, median")
            if "ms" in rec:
                rec["value"] = B * T / (rec["ms"] * 1e-3)
                rec["unit"] = UNIT
                line["vs_triton"] = rec["ms"] / ms_step
            line["triton_reference"] = rec
        line["cpu_baseline"], _ = cpu_sample(op, B, T, H, K, V, dtype, steps=3, warmup=1)
    del i
    torch.cuda.empty_cache()
    if not args.no_extras and not args.no_configs and args.workload == "gdn" and not args.seq_len:
        if world == 1:
            line["configs"] = configs_record(dev, tri, deadline=t_begin + 420.0)
        else:
            sp = sp_record(dev, rank, world)
            vs = varlen_shard_record(dev, rank, world)
            if rank == 0:
                line["sp"], line["varlen_shard"] = sp, vs
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes per token-head of each stage's kernel, from the ncu capture summarised in
# profiles/gdn_kernels_ncu_full_T2048.md (dram__bytes_read.sum + dram__bytes_write.sum at T=2048, 262 144
# token-heads; the traffic of these kernels is proportional to the number of tokens)
NCU_BYTES_PER_TOKENHEAD = {"wy_fwd": 1076, "delta_fwd_h": 1412, "chunk_fwd_o": 1476, "dv_local": 925,
                           "delta_bwd_dhu": 1960, "dqkwg": 3241, "wy_bwd": 1970}


if __name__ == "__main__":
    main()
