"""Test infrastructure, not product code: runs the reference's OWN generator over the packaged IR programs and
stores the Triton modules it emits, so that on a GPU the reference's real kernels can be executed beside this
library's (parity check in tests/test_gpu_reference_kernels.py, timing through `bench.py --impl reference` on
the native_* workloads).

    python oracle/make_reference_kernels.py [/path/to/reference]

Writes oracle/_ref/<program>_<model>.py for model in {llama, falcon} (the LoRA and gated-MLP programs: their configurations {base, large}) (git-ignored: derived from the reference,
regenerated wherever the reference checkout is present, never committed).  The IR text is this repository's
(`triton_b200/ir_programs/`; the reference ships no IR files) with one substitution: the head tile of the
parallel loops, written symbolically there (`(ploop 0 N D n`), is given as the number the model uses
(`(ploop 0 N 128 n`).  With a symbolic tile the reference generator autotunes BLOCK_N over {32, 64, 128}
although its own stores assume BLOCK_N = D (TritonGen.py:388-391, 2974); a numeric tile fixes BLOCK_N, and only
BLOCK_K / BLOCK_P are autotuned, every choice of which is valid.  Nothing else is touched: the emitted text is
the reference's unmodified output for that program (IrParser.py:21-25 -> TritonGen.py:348).
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)

from triton_b200.harness import configs_of, tables_for  # noqa: E402


def generate(ref_dir: str, out_dir: str) -> int:
    sys.path.insert(0, ref_dir)
    from IrParser import IRParser          # the reference's
    from TritonGen import TritonCodeGen    # the reference's
    os.makedirs(out_dir, exist_ok=True)
    ir_dir = os.path.join(ROOT, "triton_b200", "ir_programs")
    n = 0
    for fn in sorted(os.listdir(ir_dir)):
        if not fn.endswith(".txt"):
            continue
        program = fn[:-4]
        for model in configs_of(program):
            shapes, consts = tables_for(program, model)
            text = open(os.path.join(ir_dir, fn)).read()
            if "D" in consts:
                text = text.replace("(ploop 0 N D n", f"(ploop 0 N {consts['D']} n")
            code = TritonCodeGen().generate(IRParser().parse(text), dict(shapes), dict(consts))
            compile(code, fn, "exec")      # the emitted module must at least be valid Python
            with open(os.path.join(out_dir, f"{program}_{model}.py"), "w") as f:
                f.write(code)
            n += 1
    return n


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRINITY_REFERENCE_DIR")
    if not ref:
        sys.exit("usage: python " + sys.argv[0] + " <reference checkout>   (or set TRINITY_REFERENCE_DIR)")
    print(generate(ref, os.path.join(HERE, "_ref")), "modules written to oracle/_ref/")
