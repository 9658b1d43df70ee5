"""Benchmark of the fused attention block on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one call of the whole block (RMSNorm statistics -> QKV projection -> attention
[-> per-key statistics]) on one batch of synthetic input.  The default workload is the PreNorm Llama3-8B
bf16 configuration: X[8,2048,4096], RMSNorm eps 1e-5 with gamma, Wq 4096x4096, Wk/Wv 4096x1024, causal
GQA attention with 32 query / 8 KV heads of 128.  Work per step is counted algorithmically:
2*T*N*(Hq+2Hkv)*D for the projection plus 4*B*Hq*D*S(S+1)/2 for causal attention (recomputation, masked
tile waste, exp and norm work are not counted).

Under torchrun (one rank per GPU) every rank runs the same workload on its own data — the block has no
exchange step — so `value` is the aggregate over ranks from the slowest rank's device time ("weak").

`--impl reference` times the reference's CPU path for the same block (the fp32 PyTorch restatement of
ref_rms.py in oracle/, all host threads) on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: variant, B, S, N, Hq, Hkv, D, project, topk
    "prenorm_llama": dict(variant="prenorm", B=8, S=2048, N=4096, Hq=32, Hkv=8, D=128, project=True, topk=0),
    # one batch item of the above: the size used for ncu captures (inputs still exceed the L2)
    "prenorm_llama_b1": dict(variant="prenorm", B=1, S=2048, N=4096, Hq=32, Hkv=8, D=128, project=True, topk=0),
    "vanilla_llama": dict(variant="vanilla", B=1, S=512, N=4096, Hq=32, Hkv=8, D=128, project=True, topk=0),
    "qknorm_falcon": dict(variant="qknorm", B=4, S=2048, N=4544, Hq=71, Hkv=1, D=64, project=True, topk=0),
    "keyformer_llama": dict(variant="keyformer", B=4, S=4096, N=0, Hq=32, Hkv=8, D=128, project=False, topk=1024),
    "roco_falcon": dict(variant="roco", B=2, S=8192, N=0, Hq=71, Hkv=1, D=64, project=False, topk=2048),
    # one batch item of the KeyFormer workload: the size used for ncu captures of its two passes
    "keyformer_llama_b1": dict(variant="keyformer", B=1, S=4096, N=0, Hq=32, Hkv=8, D=128, project=False, topk=1024),
    # standalone RMSNorm (HBM-bound): rows x cols, bf16, eps 1e-5, gamma
    "rmsnorm_llama": dict(variant="rmsnorm", rows=16384, cols=4096),
    "rmsnorm_falcon": dict(variant="rmsnorm", rows=8192, cols=4544),
}
# The reference's own benchmark shapes (M = 16 new tokens, P = 1024 cached keys, fp16; vanilla_llama_benchmark.py
# and its siblings), run the way its harness runs them: IR program -> convert_ir_to_triton -> forward(*tensors),
# 10 warm-up calls, CUDA-graph capture, 100 replays.  `--impl reference` runs the Triton module the reference's own
# generator emitted for the same program (oracle/_ref/, produced by oracle/make_reference_kernels.py) through the
# same procedure on the same GPU.
NATIVE_PROGRAMS = ("vanilla", "prenorm", "prenorm_fused", "qknorm", "keyformer", "roco", "rmsnorm")
for _prog in NATIVE_PROGRAMS:
    for _model in ("llama", "falcon"):
        WORKLOADS[f"native_{_prog}_{_model}"] = dict(variant="native", program=_prog, model=_model)
# ... and the neighbouring LoRA operator on the configurations of lora_benchmark.py:545-548
for _cfg in ("base", "large"):
    WORKLOADS[f"native_lora_{_cfg}"] = dict(variant="native", program="lora", model=_cfg)
METRIC = "fused attn-block TFLOP/s"


def algorithmic_flops(w) -> tuple:
    T = w["B"] * w["S"]
    proj = 2 * T * w["N"] * (w["Hq"] + 2 * w["Hkv"]) * w["D"] if w["project"] else 0
    attn = 4 * w["B"] * w["Hq"] * w["D"] * (w["S"] * (w["S"] + 1) // 2)
    return proj, attn


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(tflops=d["bf16_tflops"], sustained=d.get("bf16_tflops_sustained"), hbm=d["hbm_gbs"], kind="measured")
    return dict(tflops=1590.0, sustained=1400.0, hbm=6650.0, kind="fallback")


# ------------------------------------------------------------------------------------------------
# clocks during the timed region (NVML polling thread; read-only)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------------------------------------
# CPU reference arm / baseline: the oracle on a bounded sample of the workload
# ------------------------------------------------------------------------------------------------
def cpu_sample(w, dt_name="bf16"):
    """One batch item and `heads` query heads (with their KV heads) of the workload, fp32 on the host."""
    import torch
    from oracle import attn_block_ref as O
    torch.manual_seed(0)
    grp = w["Hq"] // w["Hkv"]
    hq = min(w["Hq"], 8 if grp <= 8 else grp)
    hkv = max(1, hq // grp)
    S, D, N = w["S"], w["D"], w["N"]
    if w["project"]:
        X = torch.randn(S, N)
        Wq, Wk, Wv = torch.randn(N, hq * D) / N ** 0.5, torch.randn(N, hkv * D) / N ** 0.5, torch.randn(N, hkv * D) / N ** 0.5
        gamma = 1 + 0.1 * torch.randn(N) if w["variant"] == "prenorm" else None
        gq = 1 + 0.1 * torch.randn(D) if w["variant"] == "qknorm" else None
        fn = lambda: O.attn_block(w["variant"], X=X, Wq=Wq, Wk=Wk, Wv=Wv, B=1, M=S, P=0, Hq=hq, Hkv=hkv, D=D, causal=True,
                                  scale=D ** -0.5, pre_eps=1e-5, pre_gamma=gamma, qk_eps=1e-5, gamma_q=gq, gamma_k=gq)
        proj = 2 * S * N * (hq + 2 * hkv) * D
    else:
        hq = min(hq, 2 * grp) if w["S"] >= 8192 else hq
        hkv = max(1, hq // grp)
        Q, K, V = torch.randn(1, hq, S, D), torch.randn(1, hkv, S, D), torch.randn(1, hkv, S, D)
        noise = O.gumbel_noise(0, 1, hq, S, S) if w["variant"] == "keyformer" else None
        fn = lambda: O.attn_block(w["variant"], Q=Q, K=K, V=V, B=1, M=S, P=0, Hq=hq, Hkv=hkv, D=D, causal=True,
                                  scale=D ** -0.5, tau=1.0, noise=noise)
        proj = 0
    flops = proj + 4 * hq * D * (S * (S + 1) // 2)
    desc = f"1 of {w['B']} batch items x {hq} of {w['Hq']} query heads ({hkv} kv), fp32 torch on host cores"
    return fn, flops, desc


def time_cpu(fn, steps, warmup):
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    with torch.no_grad():
        for _ in range(warmup):
            fn()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        return (time.perf_counter() - t0) / steps


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    fn, flops, desc = cpu_sample(w)
    # bounded: at most ~120 s of CPU work whatever K is
    t1 = time_cpu(fn, 1, 1)
    steps = max(1, min(args.steps, int(120 / max(t1, 1e-3))))
    warm = min(args.warmup, 2)
    sec = time_cpu(fn, steps, warm)
    value = flops / sec / 1e12
    full = sum(algorithmic_flops(w))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": sec * 1e3 * full / flops, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, **{k: w[k] for k in ("variant", "B", "S", "N", "Hq", "Hkv", "D")},
                       "note": "ms_per_step is the sample's time scaled to the whole workload by algorithmic flops"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args, w):
    import torch
    import torch.distributed as dist
    from triton_b200 import _lib as L
    from triton_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    dt = torch.bfloat16
    B, S, N, Hq, Hkv, D = (w[k] for k in ("B", "S", "N", "Hq", "Hkv", "D"))
    variant = w["variant"]
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)

    q = torch.empty(B, S, Hq, D, device=dev, dtype=dt)
    kc = torch.empty(B, Hkv, S, D, device=dev, dtype=dt)
    vc = torch.empty(B, Hkv, S, D, device=dev, dtype=dt)
    o = torch.empty(B, S, Hq, D, device=dev, dtype=dt)
    kw = {}
    x = None
    if w["project"]:
        x = rnd(B * S, N).to(dt)
        kw = dict(x=x, wq=(rnd(N, Hq * D) / N ** 0.5).to(dt), wk=(rnd(N, Hkv * D) / N ** 0.5).to(dt),
                  wv=(rnd(N, Hkv * D) / N ** 0.5).to(dt), pre_eps=1e-5, qk_eps=1e-5)
        if variant == "prenorm":
            kw["pre_gamma"] = (1 + 0.1 * rnd(N)).to(dt)
        if variant == "qknorm":
            kw["gamma_q"], kw["gamma_k"] = (1 + 0.1 * rnd(D)).to(dt), (1 + 0.1 * rnd(D)).to(dt)
    else:
        q.copy_(rnd(B, S, Hq, D)); kc.copy_(rnd(B, Hkv, S, D)); vc.copy_(rnd(B, Hkv, S, D))
    sp = torch.empty(B, Hq, S, device=dev) if variant in ("keyformer", "roco") else None
    sp2 = torch.empty(B, Hq, S, device=dev) if variant == "roco" else None
    idx = torch.empty(B, Hq, w["topk"], device=dev, dtype=torch.int32) if w["topk"] else None
    plan = ops.BlockPlan(variant, B=B, M=S, P=0, Hq=Hq, Hkv=Hkv, D=D, q=ops.as_bshd(q, "bshd"),
                         k_cache=ops.as_bshd(kc, "bhsd"), v_cache=ops.as_bshd(vc, "bhsd"), o=ops.as_bshd(o, "bshd"),
                         causal=True, scale=D ** -0.5, noise_mode=L.TRN_NOISE_GUMBEL if variant == "keyformer" else 0,
                         tau=1.0, seed=0, sum_p=sp, sum_p2=sp2, **kw)

    def step():
        plan.run()
        if idx is not None:
            ops.topk_keys(sp, w["topk"], out=idx)

    launches_per_step = {"vanilla": 2, "prenorm": 3, "qknorm": 2, "keyformer": 3, "roco": 2}[variant]
    if not w["project"]:
        launches_per_step -= 1
    if idx is not None:
        launches_per_step += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if L.kernel_status() != 0:
        raise RuntimeError(f"kernel status {L.kernel_status()} after warm-up")

    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)

    # ---- per-kernel device times over the same data (events around each launch, same stream)
    kern_us = {}
    if rank == 0:
        sc = D ** -0.5
        qv, kv_, vv, ov = ops.as_bshd(q, "bshd"), ops.as_bshd(kc, "bhsd"), ops.as_bshd(vc, "bhsd"), ops.as_bshd(o, "bshd")
        stages = []
        if w["project"]:
            xn = torch.empty_like(x) if variant == "prenorm" else None
            if variant == "prenorm":
                stages.append(("rmsnorm", lambda: ops.rmsnorm(x, kw["pre_gamma"], 1e-5, out=xn)))
            xin = xn if variant == "prenorm" else x
            stages.append(("qkv_gemm", lambda: ops.qkv_project(
                xin, kw["wq"], kw["wk"], kw["wv"], q=qv, k_cache=kv_, v_cache=vv, B=B, M=S, P=0, Hq=Hq, Hkv=Hkv, D=D,
                qk_norm=variant == "qknorm", qk_eps=1e-5, gamma_q=kw.get("gamma_q"), gamma_k=kw.get("gamma_k"))))
        lse = torch.empty(B, Hq, S, device=dev)
        if variant == "keyformer":
            # one pass: attention output, lse and the perturbed scores' lse (as the block runs it)
            lse_p = torch.empty_like(lse)
            stages.append(("attention+perturbed_lse", lambda: ops.attention(
                qv, kv_, vv, ov, P=0, causal=True, scale=sc, lse=lse, lse_pert=lse_p, noise_mode=L.TRN_NOISE_GUMBEL,
                tau=1.0, seed=0)))
            stages.append(("colstats", lambda: ops.attn_colstats(qv, kv_, lse_p, sp, None, P=0, causal=True, scale=sc,
                                                                 noise_mode=L.TRN_NOISE_GUMBEL, tau=1.0, seed=0)))
        else:
            stages.append(("attention", lambda: ops.attention(qv, kv_, vv, ov, P=0, causal=True, scale=sc, lse=lse)))
        if variant == "roco":
            stages.append(("colstats", lambda: ops.attn_colstats(qv, kv_, lse, sp, sp2, P=0, causal=True, scale=sc)))
        if idx is not None:
            stages.append(("topk", lambda: ops.topk_keys(sp, w["topk"], out=idx)))
        n_rep = min(args.steps, 20)
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)] for _ in range(n_rep)]
        for ev in evs:
            ev[0].record(stream)
            for i, (_, fn) in enumerate(stages):
                fn()
                ev[i + 1].record(stream)
        torch.cuda.synchronize()
        for i, (name, _) in enumerate(stages):
            kern_us[name] = sum(ev[i].elapsed_time(ev[i + 1]) for ev in evs) / len(evs) * 1e3

    # ---- end to end through the C ABI with host buffers (H2D of X, D2H of O inside the timed region)
    e2e = None
    if w["project"]:
        xh = torch.empty(B * S, N, dtype=dt).pin_memory()
        xh.copy_(x.cpu())
        oh = torch.empty(B, S, Hq, D, dtype=dt).pin_memory()
        ha = L.TrnBlockHostArgs()
        C.memmove(C.byref(ha.dev), C.byref(plan.args), C.sizeof(L.TrnBlockArgs))
        ha.x_host, ha.o_host = xh.data_ptr(), oh.data_ptr()
        ha.x_bytes, ha.o_bytes = xh.numel() * 2, oh.numel() * 2
        lib = L.load()
        sraw = stream.cuda_stream
        for _ in range(2):
            L.check(lib.trinity_attn_block_host(C.byref(ha), sraw))
        barrier()
        n_e2e = max(3, min(args.steps, 20))
        t0 = time.perf_counter()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(n_e2e):
            L.check(lib.trinity_attn_block_host(C.byref(ha), sraw))
        f1.record(stream)
        barrier()
        e2e_ms = f0.elapsed_time(f1) / n_e2e
        e2e = (e2e_ms, ha.x_bytes, ha.o_bytes, float(oh.float().abs().mean()))
    clocks = sampler.stop()

    ms_step = ms_total / args.steps
    if world > 1:
        t = torch.tensor([ms_step, e2e[0] if e2e else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t[0])
        if e2e:
            e2e = (float(t[1]),) + e2e[1:]
    status = L.kernel_status()
    if status != 0:
        raise RuntimeError(f"kernel status {status}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    proj_f, attn_f = algorithmic_flops(w)
    flops = proj_f + attn_f
    peaks = measured_peaks()
    value = world * flops / (ms_step * 1e-3) / 1e12
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "variant": variant, "B": B, "S": S, "N": N, "Hq": Hq, "Hkv": Hkv, "D": D,
                       "causal": True, "parallelism": f"replicas x{world} (no data-path collective)",
                       "l2": "per-step working set (X, W, Q, K/V, O ~ 0.57 GB) is larger than the 126 MB L2",
                       "flops_per_step": flops},
            "us_per_call": ms_step * 1e3,
            "frac_of_bf16_peak": value / world / peaks["tflops"], "peak_kind": peaks["kind"],
            "clocks": clocks, "gpu_launches": launches_per_step * args.steps}
    if e2e:
        line["e2e"] = {"value": world * flops / (e2e[0] * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e[0],
                       "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2],
                       "api": "trinity_attn_block_host (pinned host X in, O out; weights resident)"}
    else:
        line["e2e"] = None
    if kern_us:
        line["kernels_us"] = kern_us
        algo = {"qkv_gemm": proj_f, "attention": attn_f, "attention+perturbed_lse": attn_f}
        top = max((k for k in kern_us if k in algo and algo[k] > 0), key=lambda k: kern_us[k])
        ach = algo[top] / (kern_us[top] * 1e-6) / 1e12
        line["roofline"] = {"kernel": {"qkv_gemm": "qkv_gemm_kernel", "attention": "attn_fwd_kernel",
                                       "attention+perturbed_lse": "attn_fwd_kernel"}[top],
                            "bound": "tensor", "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s",
                            "frac": ach / peaks["tflops"], "peak_source": peaks["kind"] + " burst",
                            "traffic": TRAFFIC_BYTES.get((args.workload, top))}
        for k in algo:
            if k in kern_us and algo[k] > 0:
                line[k + "_tflops"] = algo[k] / (kern_us[k] * 1e-6) / 1e12
    if world == 1 and not args.no_cpu:
        fn, cflops, desc = cpu_sample(w)
        sec = time_cpu(fn, 2, 1)
        line["cpu_baseline"] = {"value": cflops / sec / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                                "sample": desc}
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the named kernel at the workload's full
# size, from the ncu captures summarised under profiles/ (None where no capture was taken)
TRAFFIC_BYTES = {
    ("prenorm_llama", "qkv_gemm"): 409042944 + 178885120,
    ("prenorm_llama", "attention"): 308813824 + 99281152,
    "rmsnorm_llama": 134235648 + 79863808,
}


def run_rmsnorm(args, w):
    """Standalone RMSNorm: algorithmic bytes = 2 * rows * cols * 2 (read x, write y) + gamma."""
    import torch
    from triton_b200 import _lib as L
    from triton_b200 import ops
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if int(os.environ.get("RANK", "0")) != 0 or world != 1:
        if int(os.environ.get("RANK", "0")) != 0:
            return
    torch.cuda.set_device(local)
    rows, cols = w["rows"], w["cols"]
    dt = torch.bfloat16
    x = torch.randn(rows, cols, device="cuda").to(dt)
    g = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dt)
    y = torch.empty_like(x)
    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        ops.rmsnorm(x, g, 1e-5, out=y)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        ops.rmsnorm(x, g, 1e-5, out=y)
    e1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    nbytes = 2 * rows * cols * 2 + cols * 2
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    if L.kernel_status() != 0:
        raise RuntimeError("kernel status")
    line = {"metric": "rmsnorm GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "us_per_call": ms * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "rows": rows, "cols": cols, "eps": 1e-5, "gamma": True,
                       "l2": "x and y (2 x %.0f MB) are larger than the 126 MB L2" % (rows * cols * 2 / 1e6)},
            "clocks": clocks, "gpu_launches": args.steps, "e2e": None,
            "roofline": {"kernel": "rmsnorm_cta_kernel", "bound": "hbm", "achieved": gbs, "peak": peaks["hbm"],
                         "unit": "GB/s", "frac": gbs / peaks["hbm"], "peak_source": peaks["kind"],
                         "traffic": TRAFFIC_BYTES.get(args.workload)}}
    print(json.dumps(line))


def run_native(args, w):
    """One of the reference's own shapes through the reference's own harness procedure; ours or the reference's
    generated Triton kernels."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import importlib.util
    import torch
    from triton_b200 import _lib as L
    from triton_b200.convert_module import convert_ir_to_triton
    from triton_b200.harness import AttnBlockBenchmark, tables_for
    prog, model = w["program"], w["model"]
    SHAPE_DICT, consts = tables_for(prog, model)
    M, N, P = (consts[k] for k in ("M", "N", "P"))
    D, H = consts.get("D"), consts.get("H")
    ref_path = os.path.join(ROOT, "oracle", "_ref", f"{prog}_{model}.py")
    base = {"metric": METRIC, "unit": "TFLOP/s", "n_gpus": 1, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "program": prog, "model": model, **consts,
                       "procedure": "10 warm-up calls, CUDA-graph capture, 100 replays (the reference harness)"}}
    if args.impl == "reference" and not os.path.isfile(ref_path):
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref is not generated on this machine "
                          "(python oracle/make_reference_kernels.py needs the reference checkout)"}))
        return
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    bench = AttnBlockBenchmark(consts, seed=42, shape_dict=SHAPE_DICT)
    if args.impl == "reference":
        spec = importlib.util.spec_from_file_location(f"refgen_{prog}_{model}", ref_path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
    else:
        ir = open(os.path.join(ROOT, "triton_b200", "ir_programs", f"{prog}.txt")).read()
        mod = bench.compile_and_load_kernel(convert_ir_to_triton(ir, SHAPE_DICT, consts), 0)
    bench.create_test_tensors(mod.TENSOR_PARAMS)
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    try:
        ms = bench.benchmark_kernel(mod, warmup_runs=10, benchmark_runs=100)
        err = None
    except Exception as e:                       # the reference's QKNorm kernels overflow fp16 at these inputs
        ms, err = float("nan"), str(e)
    # the harness's event pairs around one replay resolve about 2 us; a second figure with 20 calls per captured
    # graph and one event pair around 50 replays separates operators that take a few microseconds
    us_batched = None
    if err is None:
        tensors = [bench.tensors[name] for name in mod.TENSOR_PARAMS]
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    mod.forward(*tensors)
            side.synchronize()
            for _ in range(3):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(50):
                graph.replay()
            e1.record(side)
        side.synchronize()
        us_batched = e0.elapsed_time(e1) / (50 * 20) * 1e3
    clocks = sampler.stop()
    if prog == "rmsnorm":
        flops = 3 * M * N
    elif prog == "lora":
        R = consts["R"]
        flops = 2 * M * N * P + 2 * M * N * R + 2 * M * R * P
    else:
        flops = 2 * M * N * 3 * H * D + 4 * H * D * M * (P + M)
    line = dict(base, value=None if err else flops / (ms * 1e-3) / 1e12, steps=100, warmup=10,
                ms_per_step=None if err else ms, us_per_call=None if err else ms * 1e3,
                us_per_call_20_per_graph=us_batched, clocks=clocks,
                gpu_launches=100, e2e=None)
    if err:
        line["error"] = err
    if args.impl == "reference":
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                "sample": "the Triton module the reference generator emits for this program, on this GPU"}
    elif L.kernel_status() != 0:
        raise RuntimeError("kernel status")
    print(json.dumps(line))
    bench.cleanup()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="prenorm_llama")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if w["variant"] == "native":
        run_native(args, w)
    elif w["variant"] == "rmsnorm":
        run_rmsnorm(args, w)
    elif args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
