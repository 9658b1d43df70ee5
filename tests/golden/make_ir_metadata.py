"""Runs the reference front end and generator over the packaged IR programs and records what they
produce, so that the tests can check this repository's parser and recogniser against the reference
without the reference checkout:

    python tests/golden/make_ir_metadata.py [/path/to/reference]

Writes ir_metadata.json: per program the reference's AST (IrParser.py:21-25) as nested lists, and the
TENSOR_PARAMS / BLOCK_PARAMS / forward signature its TritonCodeGen emits (TritonGen.py:563-584).
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from triton_b200.harness import configs_of, tables_for  # noqa: E402


def tree(node):
    return [node.node_type.value, node.value, [tree(c) for c in node.children]]


def main():
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRINITY_REFERENCE_DIR")
    if not ref_dir:
        sys.exit("usage: python " + sys.argv[0] + " <reference checkout>   (or set TRINITY_REFERENCE_DIR)")
    sys.path.insert(0, ref_dir)
    from IrParser import IRParser          # the reference's
    from TritonGen import TritonCodeGen    # the reference's
    out = {}
    ir_dir = os.path.join(ROOT, "triton_b200", "ir_programs")
    for fn in sorted(os.listdir(ir_dir)):
        if not fn.endswith(".txt"):
            continue
        name = fn[:-4]
        text = open(os.path.join(ir_dir, fn)).read()
        ast = IRParser().parse(text)
        shapes, consts = tables_for(name, sorted(configs_of(name))[0] if "llama" not in configs_of(name) else "llama")
        code = TritonCodeGen().generate(ast, dict(shapes), dict(consts))
        out[name] = {
            "ast": tree(ast),
            "tensor_params": eval(re.search(r"TENSOR_PARAMS = (.*)", code).group(1)),
            "block_params": eval(re.search(r"BLOCK_PARAMS = (.*)", code).group(1)),
            "forward": re.search(r"def forward\((.*)\):", code).group(1),
            "n_kernels": len(re.findall(r"@triton.jit", code)),
        }
        print(name, out[name]["tensor_params"], out[name]["block_params"], out[name]["n_kernels"])
    with open(os.path.join(HERE, "ir_metadata.json"), "w") as f:
        json.dump(out, f)


if __name__ == "__main__":
    main()
