"""One parameterised benchmark harness in place of the reference's ten per-variant scripts
({vanilla,prenorm,qknorm,keyformer,roco}_{llama,falcon}_benchmark.py, which differ only in shape tables,
device index and file paths).

Same procedure and on-disk formats:
  * IR file: one candidate per line, ``<id>: (<expr>)``; lines containing ``dummydata`` are skipped
    (vanilla_llama_benchmark.py:141-161); a file holding a single bare program is accepted as id 0;
  * tensor configs: JSON list of {M, N, D, H, P} (vanilla_llama_benchmark.py:743-744);
  * per candidate: generate the module with convert_ir_to_triton, import it from a temp file, call
    forward once, 10 warm-ups on a side stream, capture forward in a CUDA graph, time 100 replays with
    CUDA events, NaN-check the output (vanilla_llama_benchmark.py:223-301);
  * results: JSON list of {ir_id, ir_expression, execution_time_ms, tensor_config, error}, rewritten
    after every tensor config (vanilla_llama_benchmark.py:390-398, 517-547);
  * flags --ir --output --start --num --end --topk --all (vanilla_llama_benchmark.py:746-753) plus
    --variant / --model / --tensors to pick what the ten scripts hard-code.

    python -m triton_b200.harness --variant vanilla --model llama
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import sys
import tempfile
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from .convert_module import convert_ir_to_triton

IR_DIR = Path(__file__).resolve().parent / "ir_programs"
VARIANTS = ("vanilla", "prenorm", "qknorm", "keyformer", "roco", "rmsnorm")

# the reference's native shapes (convert_eval_rms.py:33-60)
MODEL_CONFIGS = {
    "llama": {"M": 16, "N": 4096, "D": 128, "H": 32, "P": 1024},
    "falcon": {"M": 16, "N": 4544, "D": 64, "H": 71, "P": 1024},
}

# symbolic shape table of the operator's tensor vocabulary (convert_eval_rms.py:62-108)
SHAPE_DICT: Dict[str, Tuple[str, ...]] = {
    "X": ("M", "N"), "X2": ("M",), "X_norm": ("M", "N"),
    "WQ": ("N", "N"), "WK": ("N", "N"), "WV": ("N", "N"),
    "Q": ("H", "M", "D"), "K": ("H", "M", "D"), "V": ("H", "M", "D"),
    "Q1": ("M", "N"), "K1": ("M", "N"), "V1": ("M", "N"),
    "Q2": ("M", "H", "D"), "K2": ("M", "H", "D"), "V2": ("M", "H", "D"),
    "K_cache": ("H", "P+M", "D"), "V_cache": ("H", "P+M", "D"),
    "O": ("H", "M", "D"), "O1": ("M", "H", "D"), "O2": ("M", "N"),
    "C": ("H", "M", "P"), "C_exp": ("H", "M", "P+M"), "C_div": ("H", "M", "P+M"), "C_sum": ("H", "M"),
    "noise": ("H", "M", "P+M"), "C_perturb": ("H", "M", "P+M"), "C_exp_perturb": ("H", "M", "P+M"),
    "C_sum_perturb": ("H", "M"), "C_div_perturb": ("H", "M", "P+M"), "C_out": ("H", "P+M"),
    "C_out1": ("H", "P+M"), "C_out2": ("H", "P+M"),
    "Q_norm": ("H", "M", "D"), "K_norm": ("H", "M", "D"),
}
# inputs get random values, everything else starts at zero (vanilla_llama_benchmark.py:131-139)
INPUT_TENSORS = ("X", "WQ", "WK", "WV", "K_cache", "V_cache", "noise", "W", "A", "B", "W1", "W2")

# the LoRA harness has a tensor table of its own (lora_benchmark.py:41-64; configurations :545-548)
LORA_SHAPE_DICT: Dict[str, Tuple[str, ...]] = {
    "X": ("M", "N"), "W": ("N", "P"), "A": ("N", "R"), "B": ("R", "P"), "O": ("M", "P"),
    "C": ("M", "P"), "D": ("M", "R"), "E": ("M", "P"),
}
LORA_CONFIGS = {
    "base": {"M": 16, "N": 1024, "P": 512, "R": 64},
    "large": {"M": 16, "N": 2048, "P": 1024, "R": 128},
}


# ... and so has the gated-MLP harness (gmlp_benchmark.py:53-74; constants M, N, K, :46-48; its tensor-config file is
# not part of the reference: two configurations in the spirit of the LoRA ones stand in)
GMLP_SHAPE_DICT: Dict[str, Tuple[str, ...]] = {
    "X": ("M", "K"), "W1": ("K", "N"), "W2": ("K", "N"), "O": ("M", "N"),
    "C1": ("M", "N"), "C2": ("M", "N"), "C1_exp": ("M", "N"),
}
GMLP_CONFIGS = {
    "base": {"M": 16, "N": 4096, "K": 1024},
    "large": {"M": 16, "N": 8192, "K": 2048},
}


def configs_of(program: str) -> Dict[str, Dict[str, int]]:
    """The named configurations a packaged program is run on."""
    if program == "lora":
        return LORA_CONFIGS
    if program.startswith("gmlp"):
        return GMLP_CONFIGS
    return MODEL_CONFIGS


def tables_for(program: str, model: str):
    """(shape table, constants) a packaged program is run with: the attention programs on a model's shape, the LoRA
    program on one of its own configurations."""
    if program == "lora":
        return LORA_SHAPE_DICT, LORA_CONFIGS[model]
    if program.startswith("gmlp"):
        return GMLP_SHAPE_DICT, GMLP_CONFIGS[model]
    return SHAPE_DICT, MODEL_CONFIGS[model]


@dataclass
class BenchmarkResult:
    ir_id: int
    ir_expression: str
    execution_time: float
    tensor_config: Dict[str, int]
    error: Optional[str] = None


def parse_ir_file(path: str) -> List[Tuple[int, str]]:
    text = Path(path).read_text()
    out: List[Tuple[int, str]] = []
    for line in text.splitlines():
        line = line.strip()
        head, sep, rest = line.partition(":")
        if sep and head.strip().lstrip("-").isdigit():
            if "dummydata" not in rest:
                out.append((int(head), rest.strip()))
    if not out and "(" in text:
        out.append((0, text))          # a single multi-line program
    return out


def resolve_dim(sym, consts: Dict[str, int]) -> int:
    if isinstance(sym, int):
        return sym
    return sum(consts[t] if t in consts else int(t) for t in sym.split("+"))


class AttnBlockBenchmark:
    def __init__(self, tensor_config: Dict[str, int], device: Optional[torch.device] = None,
                 dtype: torch.dtype = torch.float16, seed: Optional[int] = None,
                 shape_dict: Optional[Dict[str, Tuple[str, ...]]] = None):
        self.tensor_config = dict(tensor_config)
        self.const_dict = dict(tensor_config)
        self.shape_dict = dict(SHAPE_DICT if shape_dict is None else shape_dict)
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA device not available: the sm_100a kernels have no CPU path")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        self.seed = seed
        self.tensors: Dict[str, torch.Tensor] = {}
        self._temp_files: List[str] = []

    def create_test_tensors(self, names) -> None:
        """Inputs ~ randn.clamp(-1,1)*0.01 ("to avoid numerical overflow", convert_eval_rms.py:174-183;
        noise ~ randn, :201); outputs and intermediates zero.  Only the named tensors are allocated."""
        if self.seed is not None:
            torch.manual_seed(self.seed)
        for name in names:
            shape = tuple(resolve_dim(s, self.const_dict) for s in self.shape_dict[name])
            if name == "noise" or (name in INPUT_TENSORS and "W1" in self.shape_dict):
                # noise, and every input of the gated-MLP harness, are plain randn (gmlp_benchmark.py:98-99)
                t = torch.randn(shape, dtype=self.dtype, device=self.device)
            elif name in INPUT_TENSORS:
                t = torch.randn(shape, dtype=self.dtype, device=self.device).clamp(-1, 1) * 0.01
            else:
                t = torch.zeros(shape, dtype=self.dtype, device=self.device)
            self.tensors[name] = t

    def compile_and_load_kernel(self, code: str, kernel_id: int):
        with tempfile.NamedTemporaryFile(mode="w", suffix=".py", delete=False) as f:
            f.write(code)
            path = f.name
        self._temp_files.append(path)
        name = f"trinity_b200_kernel_{kernel_id}"
        spec = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[name] = module
        spec.loader.exec_module(module)
        if not hasattr(module, "forward"):
            raise RuntimeError("generated module has no forward()")
        return module

    def benchmark_kernel(self, module, warmup_runs: int = 10, benchmark_runs: int = 100) -> float:
        params = list(module.TENSOR_PARAMS)
        missing = [p for p in params if p not in self.tensors]
        self.create_test_tensors(missing)
        for name, t in self.tensors.items():
            if name not in INPUT_TENSORS:
                t.zero_()
        args = [self.tensors[p] for p in params]
        fn = module.forward
        fn(*args)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(self.device)
        with torch.cuda.stream(stream):
            for _ in range(warmup_runs):
                fn(*args)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                fn(*args)
        stream.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            start.record()
            for _ in range(benchmark_runs):
                graph.replay()
            end.record()
        stream.synchronize()
        for out_name in ("O2", "O1", "O", "X_norm"):
            if out_name not in self.tensors:
                continue
            if out_name in params and torch.isnan(self.tensors[out_name]).any():
                raise RuntimeError(f"NaN in {out_name}")
        return start.elapsed_time(end) / benchmark_runs

    def run_single_benchmark(self, ir_id: int, ir_expr: str) -> BenchmarkResult:
        try:
            code = convert_ir_to_triton(ir_expr, self.shape_dict, self.const_dict)
            module = self.compile_and_load_kernel(code, ir_id)
            ms = self.benchmark_kernel(module)
            return BenchmarkResult(ir_id, ir_expr, ms, self.tensor_config)
        except Exception as e:  # recorded, not raised: the sweep goes on (vanilla_llama_benchmark.py:329-332)
            return BenchmarkResult(ir_id, ir_expr, float("inf"), self.tensor_config, str(e))

    def run_all_benchmarks(self, ir_file: str, start: Optional[int] = None,
                           num: Optional[int] = None) -> List[BenchmarkResult]:
        """Candidates with id >= start, at most `num` of them (None: all) — vanilla_llama_benchmark.py:334-348."""
        exprs = parse_ir_file(ir_file)
        if start is not None:
            exprs = [e for e in exprs if e[0] >= start]
            if num:
                exprs = exprs[:num]
        return [self.run_single_benchmark(i, e) for i, e in exprs]

    def cleanup(self) -> None:
        for p in self._temp_files:
            try:
                os.unlink(p)
            except OSError:
                pass
        self._temp_files.clear()
        self.tensors.clear()


def results_to_json(results: List[BenchmarkResult]) -> List[Dict]:
    """The reference's record (vanilla_llama_benchmark.py:390-398, 536-542); a failed candidate keeps
    execution_time_ms = inf, which json writes as Infinity exactly as the reference's files have it."""
    return [{"ir_id": r.ir_id, "ir_expression": r.ir_expression, "execution_time_ms": r.execution_time,
             "tensor_config": r.tensor_config, "error": r.error} for r in results]


def save_incremental_results(results: List[BenchmarkResult], output_file: str) -> None:
    """Appends one configuration's records to the output file (vanilla_llama_benchmark.py:517-547)."""
    try:
        existing = json.loads(Path(output_file).read_text())
    except (OSError, ValueError):
        existing = []
    Path(output_file).write_text(json.dumps(existing + results_to_json(results), indent=2))


def find_best_kernels(results: List[BenchmarkResult], top_k: int = 10) -> List[BenchmarkResult]:
    ok = [r for r in results if r.error is None and math.isfinite(r.execution_time)]
    return sorted(ok, key=lambda r: r.execution_time)[:top_k]


def write_evaluation_tree(root: str) -> List[str]:
    """Writes the input files the reference's own *_benchmark.py scripts read, so that they run unmodified against
    this package's convert_module: ./evaluation/<variant>/<variant>_<model>_cost6_kern2.txt (one `id: (expr)` line per
    candidate, vanilla_llama_benchmark.py:141-161, 729) and ./evaluation/<model>_configs.json (:731, 743-744).  The
    reference ships neither (both are git-ignored there); the candidates are this package's IR programs."""
    written = []
    ev = Path(root) / "evaluation"
    for variant in VARIANTS:
        text = (IR_DIR / f"{variant}.txt").read_text()
        one_line = " ".join(line.split(";", 1)[0].strip() for line in text.splitlines()).strip()
        one_line = " ".join(one_line.split())
        for model in MODEL_CONFIGS:
            d = ev / variant
            d.mkdir(parents=True, exist_ok=True)
            f = d / f"{variant}_{model}_cost6_kern2.txt"
            f.write_text(f"0: {one_line}\n")
            written.append(str(f))
    for model, cfg in MODEL_CONFIGS.items():
        f = ev / f"{model}_configs.json"
        f.write_text(json.dumps([cfg], indent=2))
        written.append(str(f))
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Benchmark IR candidates of one attention-block variant (or the LoRA layer)")
    ap.add_argument("--variant", choices=VARIANTS + ("prenorm_fused", "lora", "gmlp", "gmlp_glu"), default="vanilla")
    ap.add_argument("--model", choices=sorted(set(MODEL_CONFIGS) | set(LORA_CONFIGS) | set(GMLP_CONFIGS)), default=None,
                    help="llama / falcon for the attention programs (default llama); base / large for lora (default base)")
    ap.add_argument("--ir", type=str, default=None, help="IR candidates file (default: the packaged program)")
    ap.add_argument("--tensors", type=str, default=None, help="JSON list of {M,N,D,H,P} (default: the model's)")
    ap.add_argument("--output", type=str, default=None)
    ap.add_argument("--write-evaluation", type=str, default=None, metavar="DIR",
                    help="write DIR/evaluation/... (IR candidate files and tensor-config JSONs) for the reference's own "
                         "*_benchmark.py scripts and exit")
    # the reference's flags (vanilla_llama_benchmark.py:746-753)
    ap.add_argument("--start", type=int, default=0, help="start from candidate id")
    ap.add_argument("--num", type=int, default=10, help="number of candidates to benchmark")
    ap.add_argument("--end", action="store_true", help="run from the start id to the last candidate")
    ap.add_argument("--topk", type=int, default=5, help="number of best kernels to report")
    ap.add_argument("--all", action="store_true", help="run every candidate of the file")
    args = ap.parse_args(argv)
    if args.write_evaluation:
        for f in write_evaluation_tree(args.write_evaluation):
            print(f)
        return 0
    if args.end and args.num != 10:
        print("Error: Cannot use --end and --num together. Use either --num or --end, not both.")
        return 1

    ir_file = args.ir or str(IR_DIR / f"{args.variant}.txt")
    model = args.model or ("base" if args.variant in ("lora", "gmlp", "gmlp_glu") else "llama")
    shapes, default_cfg = tables_for(args.variant, model)
    configs = json.loads(Path(args.tensors).read_text()) if args.tensors else [default_cfg]
    output = args.output or f"{args.variant}_{model}.json"
    num = None if (args.all or args.end) else args.num
    for cfg in configs:
        bench = AttnBlockBenchmark(cfg, shape_dict=shapes)
        res = bench.run_all_benchmarks(ir_file, args.start, num)
        bench.cleanup()
        save_incremental_results(res, output)
        for r in find_best_kernels(res, args.topk):
            print(f"config {cfg}  IR {r.ir_id}: {r.execution_time * 1e3:9.1f} us")
        for r in res:
            if r.error is not None:
                print(f"config {cfg}  IR {r.ir_id}: error: {r.error}")
    print(f"All results saved to: {output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
