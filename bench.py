"""Benchmark of the fused attention block on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|flashinfer|cublas] [--workload NAME]
                    [--replicas]

One "step" is one call of the whole block (RMSNorm statistics -> QKV projection -> attention
[-> per-key statistics -> top-k]) on one batch of synthetic input.  The default workload is the PreNorm
Llama3-8B bf16 configuration: X[8,2048,4096], RMSNorm eps 1e-5 with gamma, Wq 4096x4096, Wk/Wv 4096x1024, causal
GQA attention with 32 query / 8 KV heads of 128.  Work per step is counted algorithmically:
2*T*N*(Hq+2Hkv)*D for the projection plus 4*B*Hq*D*S(S+1)/2 for causal attention (recomputation, masked
tile waste, exp and norm work are not counted).

Under torchrun (one rank per GPU) the ONE workload is sharded: its (batch, kv-head group) units — (batch, query
head) units when all heads share one KV head — are dealt out to the ranks (triton_b200/shard.py); a rank binds only
the X rows, the WQ / WK / WV column slices and the cache heads of its units.  There is no exchange step, so no
collective on the data path; `value` = the whole workload's algorithmic flops / the slowest rank's device time
("strong").  After the timed region every rank's output checksum is gathered (NCCL all_gather) and compared with
single-GPU runs of sample units on rank 0 ("shard_check").  `--replicas` runs the whole workload on every rank
instead ("weak").

`--impl reference` times the reference's CPU path for the same block (the fp32 PyTorch restatement of ref_rms.py in
oracle/, all host threads) on the FULL configuration.  `--impl flashinfer` times the attention core of the workload
with FlashInfer's kernels beside this library's on the same q / k / v, same GPU, same run.  `--impl cublas` runs
cuBLAS (torch.matmul) beside the projection GEMM for about 2.5 s each with the SM clock sampled, to compare per clock.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
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
# ... and the gated MLP of gmlp_benchmark.py:53-74 (SiLU gate)
for _cfg in ("base", "large"):
    WORKLOADS[f"native_gmlp_{_cfg}"] = dict(variant="native", program="gmlp", model=_cfg)
METRIC = "fused attn-block TFLOP/s"
SEED = 1234


def algorithmic_flops(w) -> tuple:
    T = w["B"] * w["S"]
    proj = 2 * T * w["N"] * (w["Hq"] + 2 * w["Hkv"]) * w["D"] if w["project"] else 0
    attn = 4 * w["B"] * w["Hq"] * w["D"] * (w["S"] * (w["S"] + 1) // 2)
    return proj, attn


def workload_config(name, w) -> dict:
    """The `config` object of the JSON line: identical for every arm of one workload."""
    return {"workload": name, "variant": w["variant"], "B": w["B"], "S": w["S"], "N": w["N"], "Hq": w["Hq"],
            "Hkv": w["Hkv"], "D": w["D"], "causal": True, "topk": w["topk"], "flops_per_step": sum(algorithmic_flops(w)),
            "l2": "per-step working set (X, W, Q, K/V, O) is larger than the 126 MB L2"}


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

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self.period_s = period_s
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
            time.sleep(self.period_s)

    def mark(self) -> int:
        return len(self.samples)

    def median(self, lo: int = 0, hi=None):
        s = sorted(self.samples[lo:hi])
        return s[len(s) // 2] if s else None

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        return {"sm_mhz": self.median(), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# CPU reference arm / baseline: the oracle on the FULL configuration, batch item by batch item
# ------------------------------------------------------------------------------------------------
def cpu_full(w):
    """The whole workload in fp32 on the host through oracle/ (= the reference's PyTorch path, ref_rms.py:29-280,
    with the configuration's flags): one call of the returned function is one step.  Batch items are evaluated one
    after the other and, for the long-context configurations, a few query heads at a time, so that the
    [heads, S, S] fp32 scores fit host memory."""
    import torch
    from oracle import attn_block_ref as O
    torch.manual_seed(0)
    B, S, D, N, Hq, Hkv = (w[k] for k in ("B", "S", "D", "N", "Hq", "Hkv"))
    variant = w["variant"]
    if w["project"]:
        X = torch.randn(B, S, N)
        Wq, Wk, Wv = (torch.randn(N, h * D) / N ** 0.5 for h in (Hq, Hkv, Hkv))
        gamma = 1 + 0.1 * torch.randn(N) if variant == "prenorm" else None
        gq = 1 + 0.1 * torch.randn(D) if variant == "qknorm" else None
        gk = 1 + 0.1 * torch.randn(D) if variant == "qknorm" else None

        def fn():
            for b in range(B):
                O.attn_block(variant, X=X[b], Wq=Wq, Wk=Wk, Wv=Wv, B=1, M=S, P=0, Hq=Hq, Hkv=Hkv, D=D, causal=True,
                             scale=D ** -0.5, pre_eps=1e-5, pre_gamma=gamma, qk_eps=1e-5, gamma_q=gq, gamma_k=gk)
        chunk = Hq
    else:
        Q, K, V = torch.randn(B, Hq, S, D), torch.randn(B, Hkv, S, D), torch.randn(B, Hkv, S, D)
        grp = Hq // Hkv
        chunk = max(grp if Hkv > 1 else 1, min(Hq, (1 << 27) // (S * S)))        # <= 512 MiB of fp32 scores per chunk
        if Hkv > 1:
            chunk -= chunk % grp
        noise_chunk = None
        if variant == "keyformer":
            # the reference takes the noise as an input tensor (ref_rms.py:147-172): drawing it is not part of the
            # forward.  One Gumbel(0,1) chunk is drawn here and reused for every chunk of heads.
            u = torch.rand(1, chunk, S, S).clamp_(1e-7, 1 - 1e-7)
            noise_chunk = -torch.log(-torch.log(u))
            del u

        def fn():
            r = O.attn_block_chunked(variant, head_chunk=chunk, Q=Q, K=K, V=V, P=0, causal=True, scale=D ** -0.5, tau=1.0,
                                     noise_fn=(lambda b, h0, h1: noise_chunk[:, :h1 - h0]) if noise_chunk is not None else None)
            if w["topk"]:
                O.topk_keys(r["sum_p"], w["topk"])
    desc = (f"the full configuration: {B} batch items x {Hq} query heads ({Hkv} kv), {chunk} heads at a time, "
            "fp32 torch (oracle/) on all host cores")
    return fn, sum(algorithmic_flops(w)), desc


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
    import torch
    fn, flops, desc = cpu_full(w)
    # bounded: K and W are honoured as long as the whole run stays within about 150 s of CPU work
    t1 = time_cpu(fn, 1, 1)
    budget = 150.0 - 2 * t1
    warm = max(0, min(args.warmup - 1, int(0.25 * budget / max(t1, 1e-3))))     # one warm-up call is done already
    steps = max(1, min(args.steps, int((budget - warm * t1) / max(t1, 1e-3))))
    sec = time_cpu(fn, steps, warm)
    value = flops / sec / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm + 1, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.workload, w),
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": os.cpu_count(), "threads": torch.get_num_threads(),
                             "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# our arm: per-rank launches of the (sharded) workload
# ------------------------------------------------------------------------------------------------
class LaunchData:
    """Device tensors and the bound plan of one shard.Launch.  Data are a function of the GLOBAL problem (seed,
    batch item, head), so a unit has the same numbers whichever rank, and however many ranks, compute it."""

    def __init__(self, w, la, dev, seed, topk=True):
        import torch
        from triton_b200 import _lib as L
        from triton_b200 import ops
        dt = torch.bfloat16
        B, S, N, Hq, Hkv, D = (w[k] for k in ("B", "S", "N", "Hq", "Hkv", "D"))
        variant = w["variant"]
        nb, nh, nkv = la.nb, la.h1 - la.h0, la.kv1 - la.kv0
        self.la, self.w = la, w

        def gen(tag, idx):
            return torch.Generator(device=dev).manual_seed(seed + 1000003 * tag + idx)

        self.q = torch.empty(nb, S, nh, D, device=dev, dtype=dt)
        self.kc = torch.empty(nb, nkv, S, D, device=dev, dtype=dt)
        self.vc = torch.empty(nb, nkv, S, D, device=dev, dtype=dt)
        self.o = torch.empty(nb, S, nh, D, device=dev, dtype=dt)
        kw = {}
        self.x = None
        if w["project"]:
            # weights: the full matrices are drawn (same seed on every rank), the rank keeps its column slices
            def wslice(tag, heads, lo, hi):
                full = torch.randn(N, heads * D, device=dev, generator=gen(tag, 0)) / N ** 0.5
                return full[:, lo * D:hi * D].to(dt).contiguous()
            self.x = torch.cat([torch.randn(S, N, device=dev, generator=gen(1, la.b0 + i)).to(dt) for i in range(nb)])
            kw = dict(x=self.x, wq=wslice(2, Hq, la.h0, la.h1), wk=wslice(3, Hkv, la.kv0, la.kv1),
                      wv=wslice(4, Hkv, la.kv0, la.kv1), pre_eps=1e-5, qk_eps=1e-5)
            if variant == "prenorm":
                kw["pre_gamma"] = (1 + 0.1 * torch.randn(N, device=dev, generator=gen(5, 0))).to(dt)
            if variant == "qknorm":
                kw["gamma_q"] = (1 + 0.1 * torch.randn(D, device=dev, generator=gen(6, 0))).to(dt)
                kw["gamma_k"] = (1 + 0.1 * torch.randn(D, device=dev, generator=gen(7, 0))).to(dt)
        else:
            for i in range(nb):
                b = la.b0 + i
                self.q[i].copy_(torch.randn(S, Hq, D, device=dev, generator=gen(8, b))[:, la.h0:la.h1])
                self.kc[i].copy_(torch.randn(Hkv, S, D, device=dev, generator=gen(9, b))[la.kv0:la.kv1])
                self.vc[i].copy_(torch.randn(Hkv, S, D, device=dev, generator=gen(10, b))[la.kv0:la.kv1])
        stats = variant in ("keyformer", "roco")
        self.sp = torch.empty(nb, nh, S, device=dev) if stats else None
        self.sp2 = torch.empty(nb, nh, S, device=dev) if variant == "roco" else None
        self.idx = torch.empty(nb, nh, w["topk"], device=dev, dtype=torch.int32) if (w["topk"] and topk) else None
        self.kw = kw
        self.plan = ops.BlockPlan(variant, B=nb, M=S, P=0, Hq=nh, Hkv=nkv, D=D, q=ops.as_bshd(self.q, "bshd"),
                                  k_cache=ops.as_bshd(self.kc, "bhsd"), v_cache=ops.as_bshd(self.vc, "bhsd"),
                                  o=ops.as_bshd(self.o, "bshd"), causal=True, scale=D ** -0.5,
                                  noise_mode=L.TRN_NOISE_GUMBEL if variant == "keyformer" else 0, tau=1.0, seed=0,
                                  sum_p=self.sp, sum_p2=self.sp2,
                                  # a slice of the whole problem sees the whole problem's generated noise
                                  noise_heads=Hq, noise_bh0=la.b0 * Hq + la.h0, **kw)
        self.flops = sum(algorithmic_flops(dict(w, B=nb, Hq=nh, Hkv=nkv)))

    def step(self):
        from triton_b200 import ops
        self.plan.run()
        if self.idx is not None:
            ops.topk_keys(self.sp, self.w["topk"], out=self.idx)

    def launches_per_step(self) -> int:
        n = {"vanilla": 2, "prenorm": 3, "qknorm": 2, "keyformer": 3, "roco": 3}[self.w["variant"]]
        if not self.w["project"]:
            n -= 1
        return n + (1 if self.idx is not None else 0)

    def checksum(self, n_heads):
        """float64 sum and sum of magnitudes of the output of the first batch item's first n_heads heads."""
        o = self.o[0, :, :n_heads].double()
        c = [float(o.sum()), float(o.abs().sum())]
        if self.sp is not None:                       # per-key statistics of the same heads (KeyFormer: noise included)
            c[0] += float(self.sp[0, :n_heads].double().sum())
            c[1] += float(self.sp[0, :n_heads].double().abs().sum())
        return c


def run_ours(args, w):
    import torch
    import torch.distributed as dist
    from triton_b200 import _lib as L
    from triton_b200 import ops, shard

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
    sharded = world > 1 and not args.replicas
    if sharded:
        launches = shard.rank_launches(B, Hq, Hkv, rank, world)
        seed = SEED
    else:
        launches = [shard.Launch(0, B, 0, Hq, 0, Hkv)]
        seed = SEED + rank                       # replicas: every rank its own data
    data = [LaunchData(w, la, dev, seed) for la in launches]
    my_flops = sum(d.flops for d in data)
    n_launch = sum(d.launches_per_step() for d in data)

    def step():
        for d in data:
            d.step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    if L.kernel_status() != 0:
        raise RuntimeError(f"kernel status {L.kernel_status()} after warm-up")

    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    m0 = sampler.mark()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    m1 = sampler.mark()
    ms_total = e0.elapsed_time(e1)
    ms_step = ms_total / args.steps

    # ---- a second, longer timed region (>= 1 s of back-to-back steps): the figure under the sustained power cap,
    #      with the SM clock sampled during it
    n_long = max(args.steps, min(20000, int(1100.0 / max(ms_step, 1e-3)) + 1)) if not args.no_sustained else 0
    sustained = None
    if n_long:
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        m2 = sampler.mark()
        g0.record(stream)
        for _ in range(n_long):
            step()
        g1.record(stream)
        barrier()
        m3 = sampler.mark()
        sustained = (g0.elapsed_time(g1) / n_long, n_long, sampler.median(m2, m3))

    # ---- per-kernel device times over the same tensors (events around each launch, same stream), rank 0's shard
    kern_us, kern_flops = {}, {}
    if rank == 0:
        d0 = data[0]
        nb, nh, nkv = d0.la.nb, d0.la.h1 - d0.la.h0, d0.la.kv1 - d0.la.kv0
        pf, af = algorithmic_flops(dict(w, B=nb, Hq=nh, Hkv=nkv))
        sc = D ** -0.5
        qv, kv_, vv, ov = (ops.as_bshd(d0.q, "bshd"), ops.as_bshd(d0.kc, "bhsd"), ops.as_bshd(d0.vc, "bhsd"),
                           ops.as_bshd(d0.o, "bshd"))
        stages = []
        kw = d0.kw
        if w["project"]:
            xin = d0.x
            if variant == "prenorm":
                xn = d0.plan._x_norm                     # the block's own X_norm buffer
                stages.append(("rmsnorm", lambda: ops.rmsnorm(d0.x, kw["pre_gamma"], 1e-5, out=xn)))
                xin = xn
            stages.append(("qkv_gemm", lambda: ops.qkv_project(
                xin, kw["wq"], kw["wk"], kw["wv"], q=qv, k_cache=kv_, v_cache=vv, B=nb, M=S, P=0, Hq=nh, Hkv=nkv, D=D,
                qk_norm=variant == "qknorm", qk_eps=1e-5, gamma_q=kw.get("gamma_q"), gamma_k=kw.get("gamma_k"))))
            kern_flops["qkv_gemm"] = pf
        lse = torch.empty(nb, nh, S, device=dev)
        if variant == "keyformer":
            # one pass: attention output, lse and the perturbed scores' lse (as the block runs it)
            lse_p = torch.empty_like(lse)
            stages.append(("attention+perturbed_lse", lambda: ops.attention(
                qv, kv_, vv, ov, P=0, causal=True, scale=sc, lse=lse, lse_pert=lse_p, noise_mode=L.TRN_NOISE_GUMBEL,
                tau=1.0, seed=0)))
            stages.append(("colstats", lambda: ops.attn_colstats(qv, kv_, lse_p, d0.sp, None, P=0, causal=True, scale=sc,
                                                                 noise_mode=L.TRN_NOISE_GUMBEL, tau=1.0, seed=0)))
            kern_flops["attention+perturbed_lse"] = af
        else:
            stages.append(("attention", lambda: ops.attention(qv, kv_, vv, ov, P=0, causal=True, scale=sc, lse=lse)))
            kern_flops["attention"] = af
        if variant == "roco":
            stages.append(("colstats", lambda: ops.attn_colstats(qv, kv_, lse, d0.sp, d0.sp2, P=0, causal=True, scale=sc)))
        if d0.idx is not None:
            stages.append(("topk", lambda: ops.topk_keys(d0.sp, w["topk"], out=d0.idx)))
        n_rep = max(5, min(args.steps, 50))
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)] for _ in range(n_rep)]
        for _ in range(2):
            for _, fn in stages:
                fn()
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
        hosts = []
        for d in data:
            xh = torch.empty(d.x.shape, dtype=dt).pin_memory()
            xh.copy_(d.x.cpu())
            oh = torch.empty(d.o.shape, dtype=dt).pin_memory()
            hosts.append((d, xh, oh))

        def e2e_step():
            for d, xh, oh in hosts:
                d.plan.run_host(xh, oh)
        for _ in range(2):
            e2e_step()
        barrier()
        n_e2e = max(3, min(args.steps, 100))
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(n_e2e):
            e2e_step()
        f1.record(stream)
        barrier()
        e2e = [f0.elapsed_time(f1) / n_e2e, float(sum(xh.numel() * 2 for _, xh, _ in hosts)),
               float(sum(oh.numel() * 2 for _, _, oh in hosts))]
    clocks = sampler.stop()
    mhz_timed = sampler.median(m0, m1)

    # ---- reductions over ranks (device time: max; bytes: sum), then the shard check
    shard_check = None
    if world > 1:
        t = torch.tensor([ms_step, e2e[0] if e2e else 0.0, sustained[0] if sustained else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t[0])
        if e2e:
            e2e[0] = float(t[1])
        if sustained:
            sustained = (float(t[2]),) + sustained[1:]
        tot = torch.tensor([e2e[1] if e2e else 0.0, e2e[2] if e2e else 0.0, float(n_launch), float(my_flops)],
                           device=dev, dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        if e2e:
            e2e[1], e2e[2] = float(tot[0]), float(tot[1])
        n_launch_total, flops_total = int(tot[2]), float(tot[3])
        if sharded:
            # validation, outside every timed region: each rank's checksum of its first unit's output (after one
            # plain device step) is gathered with NCCL and compared with a single-GPU run of that unit alone on rank 0
            grp = Hq // Hkv
            nchk = 1 if Hkv == 1 else grp
            step()
            torch.cuda.synchronize()
            la0 = launches[0]
            mine = torch.tensor([la0.b0, la0.h0, la0.kv0] + data[0].checksum(nchk), device=dev, dtype=torch.float64)
            allv = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(allv, mine)
            if rank == 0:
                worst = 0.0
                for v in allv:
                    b, h0, kv0 = int(v[0]), int(v[1]), int(v[2])
                    one = LaunchData(w, shard.Launch(b, 1, h0, h0 + nchk, kv0, kv0 + 1), dev, seed, topk=False)
                    one.plan.run()
                    torch.cuda.synchronize()
                    ref = one.checksum(nchk)
                    worst = max(worst, abs(ref[0] - float(v[3])) / max(ref[1], 1e-30), abs(ref[1] - float(v[4])) / max(ref[1], 1e-30))
                    del one
                shard_check = {"result": "ok" if worst <= 1e-5 else "MISMATCH", "units_checked": world,
                               "max_rel_checksum_diff": worst,
                               "how": "NCCL all_gather of per-rank output checksums vs single-GPU runs of the same units on rank 0"}
    else:
        n_launch_total, flops_total = n_launch, float(my_flops)
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
    # sharded: the ONE workload's algorithmic flops (work a rank repeats for its slice, such as the shared KV head's
    # projection under MQA, is not counted twice); replicas: one workload per rank
    flops_total = float(flops) if sharded or world == 1 else float(world * flops)
    peaks = measured_peaks()
    value = flops_total / (ms_step * 1e-3) / 1e12
    if sharded:
        par = (f"one workload sharded over {world} ranks by "
               + ("(batch, query head)" if Hkv == 1 and Hq > 1 else "(batch, kv-head group)")
               + " units, no data-path collective; rank 0 runs " + ", ".join(
                   f"batch [{l.b0},{l.b0 + l.nb}) heads [{l.h0},{l.h1})" for l in launches))
    else:
        par = f"replicas x{world} (no data-path collective)" if world > 1 else "1 GPU"
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if (sharded or world == 1) else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, w), "parallelism": par,
            "us_per_call": ms_step * 1e3,
            "frac_of_bf16_peak": value / world / peaks["tflops"], "peak_kind": peaks["kind"],
            "clocks": clocks, "gpu_launches": n_launch_total * args.steps,
            # clock-normalised: device time x the SM clock sampled during it (rank 0) = SM kilocycles per step
            "clock_normalised": {"sm_mhz_timed_region": mhz_timed,
                                 "kcycles_per_step": None if mhz_timed is None else ms_step * mhz_timed}}
    if sustained:
        line["sustained"] = {"value": flops_total / (sustained[0] * 1e-3) / 1e12, "unit": "TFLOP/s",
                             "ms_per_step": sustained[0], "steps": sustained[1], "sm_mhz_median": sustained[2],
                             "kcycles_per_step": None if sustained[2] is None else sustained[0] * sustained[2],
                             "frac_of_sustained_peak": (flops_total / (sustained[0] * 1e-3) / 1e12 / world / peaks["sustained"])
                             if peaks.get("sustained") else None}
    if shard_check:
        line["shard_check"] = shard_check
    if e2e:
        line["e2e"] = {"value": flops_total / (e2e[0] * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e[0],
                       "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2],
                       "api": "trinity_attn_block_host (pinned host X in, O out; weights resident); bytes summed over ranks"}
    else:
        line["e2e"] = None
    if kern_us:
        line["kernels_us"] = kern_us
        top = max(kern_flops, key=lambda k: kern_us[k])
        ach = kern_flops[top] / (kern_us[top] * 1e-6) / 1e12
        traffic = TRAFFIC_BYTES.get((args.workload, top)) if world == 1 else None
        line["roofline"] = {"kernel": {"qkv_gemm": "qkv_gemm2_kernel (CTA pairs; qkv_gemm_kernel below one wave of 256 x 256 tiles)", "attention": "attn_fwd_kernel",
                                       "attention+perturbed_lse": "attn_fwd_kernel"}[top],
                            "bound": "tensor", "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s",
                            "frac": ach / peaks["tflops"], "peak_source": peaks["kind"] + " burst",
                            "traffic": traffic,
                            "traffic_source": None if traffic is None else
                            "dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch, ncu capture of this "
                            "kernel (profiles/prenorm_llama_full_size_kernels.md), not re-measured in this run"}
        for k in kern_flops:
            line[k + "_tflops"] = kern_flops[k] / (kern_us[k] * 1e-6) / 1e12
    if world == 1 and not args.no_cpu:
        fn, cflops, desc = cpu_full(w)
        sec = time_cpu(fn, 2, 1)
        line["cpu_baseline"] = {"value": cflops / sec / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                                "sample": desc + "; 1 warm-up + 2 timed calls", "ms_per_step": sec * 1e3}
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the named kernel at the workload's full
# size, from ncu captures (None where no capture was taken)
TRAFFIC_BYTES = {
    ("prenorm_llama", "qkv_gemm"): 517946880 + 183176704,
    ("prenorm_llama", "attention"): 297662720 + 102904832,
    "rmsnorm_llama": 134235392 + 81776128,
}


# ------------------------------------------------------------------------------------------------
# FlashInfer beside this library on the attention core (same q / k / v, same GPU, same run)
# ------------------------------------------------------------------------------------------------
def run_flashinfer(args, w):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from triton_b200 import _lib as L
    from triton_b200 import ops
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if w["variant"] == "native":
        from triton_b200.harness import tables_for
        _, c = tables_for(w["program"], w["model"])
        B, M, P, Hq, Hkv, D, causal, scale, dt = 1, c["M"], c["P"], c["H"], c["H"], c["D"], False, 1.0, torch.float16
        torch.manual_seed(42)
        q = (torch.randn(B, M, Hq, D, device=dev) * D ** -0.25).to(dt)
        kc = (torch.randn(B, Hkv, P + M, D, device=dev) * D ** -0.25).to(dt)
        vc = torch.randn(B, Hkv, P + M, D, device=dev).to(dt)
    else:
        from triton_b200 import shard
        d = LaunchData(w, shard.Launch(0, w["B"], 0, w["Hq"], 0, w["Hkv"]), dev, SEED, topk=False)
        d.plan.run()                                   # q / k / v as the block stores them
        torch.cuda.synchronize()
        B, M, P, Hq, Hkv, D, causal, scale, dt = w["B"], w["S"], 0, w["Hq"], w["Hkv"], w["D"], True, w["D"] ** -0.5, torch.bfloat16
        q, kc, vc = d.q, d.kc, d.vc
    L_ = P + M
    o = torch.empty(B, M, Hq, D, device=dev, dtype=dt)
    ws_bytes = ops.attention_workspace_bytes(B, M, P, Hq, Hkv, D)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev) if ws_bytes else None
    flops = 4 * B * Hq * D * ((M * (M + 1) // 2 + M * P) if causal else M * L_)
    stream = torch.cuda.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if w["variant"] == "native" else None

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        tot = 0.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(reps):
            if flush is not None:
                flush.zero_()                          # inputs smaller than the L2: flush it between calls
            e0.record(stream)
            fn()
            e1.record(stream)
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / reps * 1e3

    reps = max(5, min(args.steps, 50))
    ours = lambda: ops.attention(ops.as_bshd(q, "bshd"), ops.as_bshd(kc, "bhsd"), ops.as_bshd(vc, "bhsd"),
                                 ops.as_bshd(o, "bshd"), P=P, causal=causal, scale=scale, workspace=ws)
    res = {"ours": {"us": timed(ours, reps)}}
    o_ours = o.clone()
    try:
        import flashinfer
        res["flashinfer_version"] = flashinfer.__version__
    except Exception as e:                             # noqa: BLE001
        print(json.dumps({"impl": "flashinfer", "unavailable": f"import flashinfer failed: {e}"}))
        return
    for backend in [b for b in args.fi_backends.split(",") if b]:
        try:
            if backend == "cutlass":
                # FlashInfer's sm_100a CUTLASS FMHA (variable-length entry point; NHD tensors)
                import flashinfer.prefill as FP
                qn = q.reshape(B * M, Hq, D)
                kn = kc.permute(0, 2, 1, 3).reshape(B * L_, Hkv, D).contiguous()
                vn = vc.permute(0, 2, 1, 3).reshape(B * L_, Hkv, D).contiguous()
                qo = torch.arange(0, (B + 1) * M, M, device=dev, dtype=torch.int32)
                kvo = torch.arange(0, (B + 1) * L_, L_, device=dev, dtype=torch.int32)
                out = torch.empty_like(qn)
                fn = lambda: FP.fmha_varlen(qn, kn, vn, qo, kvo, max_qo_len=M, out=out, causal=causal, sm_scale=scale)
                fn()
                got = out.view(B, M, Hq, D)
            else:
                outs = [None] * B
                def fn():
                    for b in range(B):
                        outs[b] = flashinfer.single_prefill_with_kv_cache(
                            q[b], kc[b], vc[b], causal=causal, kv_layout="HND", pos_encoding_mode="NONE", sm_scale=scale,
                            backend=backend)
                fn()
                got = torch.stack(outs)
            torch.cuda.synchronize()
            diff = (got.float() - o_ours.float()).abs().max().item()
            res[backend] = {"us": timed(fn, reps), "max_abs_diff_vs_ours": diff}
        except Exception as e:                         # noqa: BLE001
            res[backend] = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
    for r in res.values():
        if isinstance(r, dict) and "us" in r:
            r["tflops"] = flops / (r["us"] * 1e-6) / 1e12
    line = {"impl": "flashinfer", "metric": "attention core us/call (this library beside FlashInfer)", "unit": "us",
            "n_gpus": 1, "config": {"workload": args.workload, "B": B, "M": M, "P": P, "Hq": Hq, "Hkv": Hkv, "D": D,
                                    "causal": causal, "dtype": str(dt).replace("torch.", "")},
            "results": res, "reps": reps,
            "note": "ref_rms.py:1223-1229 calls flashinfer.single_prefill_with_kv_cache(q, k, v, kv_layout='HND', "
                    "pos_encoding_mode='NONE') once per problem; here once per batch item; 'cutlass' is FlashInfer's "
                    "sm_100a FMHA over the whole batch in one launch"}
    if L.kernel_status() != 0:
        raise RuntimeError("kernel status")
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# cuBLAS beside this library's projection GEMM: sustained TFLOP/s and the same per sampled SM clock
# ------------------------------------------------------------------------------------------------
def run_cublas(args, w):
    """torch.matmul (cuBLAS) at 8192^3 and at the workload's projection shape, this library's projection and its
    attention core, each back to back for about 2.5 s in ONE process with the SM clock sampled through NVML every
    ~0.5 ms: TFLOP/s / median MHz -> multiply-accumulates per clock per SM."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from triton_b200 import _lib as L
    from triton_b200 import ops
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    B, S, N, Hq, Hkv, D = (w[k] for k in ("B", "S", "N", "Hq", "Hkv", "D"))
    dt = torch.bfloat16
    out = {}

    def run(name, fn, flops, seconds=2.5):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        n = max(10, int(seconds * 1e3 / (e0.elapsed_time(e1) / 10)))
        smp = ClockSampler(dev.index, period_s=0.0005)
        smp.start()
        time.sleep(0.05)
        m0 = smp.mark()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        m1 = smp.mark()
        c = smp.stop()
        ms, mhz = e0.elapsed_time(e1) / n, smp.median(m0, m1)
        tf = flops / (ms * 1e-3) / 1e12
        out[name] = {"ms": ms, "calls": n, "tflops": tf, "sm_mhz_median": mhz, "clock_samples": m1 - m0,
                     "mac_per_clk_per_sm": tf * 1e12 / 2 / sms / (mhz * 1e6) if mhz else None, "reasons": c["reasons"]}

    a = torch.randn(8192, 8192, device=dev, dtype=dt)
    b = torch.randn(8192, 8192, device=dev, dtype=dt)
    c = torch.empty(8192, 8192, device=dev, dtype=dt)
    run("cublas_8192", lambda: torch.matmul(a, b, out=c), 2 * 8192 ** 3)
    x = torch.randn(B * S, N, device=dev).to(dt)
    wq, wk, wv = ((torch.randn(N, h * D, device=dev) / N ** 0.5).to(dt) for h in (Hq, Hkv, Hkv))
    q = torch.empty(B, S, Hq, D, device=dev, dtype=dt)
    kc = torch.empty(B, Hkv, S, D, device=dev, dtype=dt)
    vc = torch.empty(B, Hkv, S, D, device=dev, dtype=dt)
    qv, kv, vv = ops.as_bshd(q, "bshd"), ops.as_bshd(kc, "bhsd"), ops.as_bshd(vc, "bhsd")
    pf = 2 * B * S * N * (Hq + 2 * Hkv) * D
    run("ours_qkv_gemm", lambda: ops.qkv_project(x, wq, wk, wv, q=qv, k_cache=kv, v_cache=vv, B=B, M=S, P=0, Hq=Hq, Hkv=Hkv, D=D), pf)
    wcat = torch.cat([wq, wk, wv], dim=1).contiguous()
    oc = torch.empty(B * S, wcat.shape[1], device=dev, dtype=dt)
    run("cublas_projection_shape", lambda: torch.matmul(x, wcat, out=oc), pf)
    o = torch.empty_like(q)
    run("ours_attention", lambda: ops.attention(qv, kv, vv, ops.as_bshd(o, "bshd"), P=0, causal=True, scale=D ** -0.5),
        4 * B * Hq * D * (S * (S + 1) // 2))
    if L.kernel_status() != 0:
        raise RuntimeError("kernel status")
    print(json.dumps({"impl": "cublas", "metric": "sustained TFLOP/s and MAC per sampled SM clock per SM", "n_gpus": 1,
                      "sms": sms, "config": {"workload": args.workload, "B": B, "S": S, "N": N, "Hq": Hq, "Hkv": Hkv, "D": D},
                      "results": out}))


def run_rmsnorm(args, w):
    """Standalone RMSNorm: algorithmic bytes = 2 * rows * cols * 2 (read x, write y) + gamma."""
    import torch
    from triton_b200 import _lib as L
    from triton_b200 import ops
    local = int(os.environ.get("LOCAL_RANK", "0"))
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
                         "traffic": TRAFFIC_BYTES.get(args.workload),
                         "traffic_source": None if TRAFFIC_BYTES.get(args.workload) is None else
                         "ncu capture of this kernel inside the PreNorm block (profiles/prenorm_llama_full_size_kernels.md), "
                         "not re-measured in this run"}}
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
    M, N, P = consts["M"], consts["N"], consts.get("P", 0)
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
    elif prog == "gmlp":
        flops = 4 * M * consts["K"] * N
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference", "flashinfer", "cublas"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="prenorm_llama")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sustained", action="store_true", help="skip the second (>= 1 s) timed region")
    ap.add_argument("--replicas", action="store_true",
                    help="N > 1: every rank runs the whole workload on its own data (weak) instead of a shard of it")
    ap.add_argument("--fi-backends", default="fa2,cutlass", help="--impl flashinfer: FlashInfer kernels to time")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "cublas":
        if w["variant"] in ("rmsnorm", "native") or not w["project"]:
            raise SystemExit("--impl cublas needs a workload with a projection")
        run_cublas(args, w)
    elif args.impl == "flashinfer":
        if w["variant"] == "rmsnorm":
            raise SystemExit("--impl flashinfer times an attention core")
        run_flashinfer(args, w)
    elif w["variant"] == "native":
        run_native(args, w)
    elif w["variant"] == "rmsnorm":
        run_rmsnorm(args, w)
    elif args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
