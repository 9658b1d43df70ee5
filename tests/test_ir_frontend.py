"""Front end and drop-in boundary on CPU: the parser builds the same tree as the reference's
IrParser.py, the recogniser reports the same TENSOR_PARAMS / BLOCK_PARAMS as the reference's
TritonCodeGen (fixture tests/golden/ir_metadata.json), and convert_ir_to_triton returns module source
with the contract the harness relies on (vanilla_llama_benchmark.py:180-256)."""
import ast as pyast
import json
import os

import pytest

from triton_b200.convert_module import convert_ir_to_triton
from triton_b200.harness import MODEL_CONFIGS, SHAPE_DICT, configs_of, parse_ir_file, resolve_dim, tables_for
from triton_b200.ir import ASTNode, IRParser, NodeType
from triton_b200.recognise import recognise

HERE = os.path.dirname(os.path.abspath(__file__))
IR_DIR = os.path.join(os.path.dirname(HERE), "triton_b200", "ir_programs")
META = json.load(open(os.path.join(HERE, "golden", "ir_metadata.json")))
PROGRAMS = sorted(META)


def tree(node):
    return [node.node_type.value, node.value, [tree(c) for c in node.children]]


def first_model(name):
    return "llama" if "llama" in configs_of(name) else sorted(configs_of(name))[0]


def read(name):
    return open(os.path.join(IR_DIR, name + ".txt")).read()


@pytest.mark.parametrize("name", PROGRAMS)
def test_parser_builds_reference_tree(name):
    assert tree(IRParser().parse(read(name))) == META[name]["ast"]


@pytest.mark.parametrize("name", PROGRAMS)
def test_recogniser_matches_reference_metadata(name):
    prog = recognise(IRParser().parse(read(name)), tables_for(name, first_model(name))[0])
    assert prog.variant == name.split("_")[0]          # prenorm_fused / gmlp_glu are second candidates of an operator
    assert prog.tensor_params == META[name]["tensor_params"]
    assert prog.block_params == META[name]["block_params"]
    assert prog.n_kernels == META[name]["n_kernels"]


@pytest.mark.parametrize("name", PROGRAMS)
def test_generated_module_contract(name):
    src = convert_ir_to_triton(read(name), *tables_for(name, first_model(name)))
    mod = pyast.parse(src)
    assigned = {t.id for n in mod.body if isinstance(n, pyast.Assign) for t in n.targets}
    assert {"TENSOR_PARAMS", "BLOCK_PARAMS"} <= assigned
    fwd = next(n for n in mod.body if isinstance(n, pyast.FunctionDef) and n.name == "forward")
    args = [a.arg for a in fwd.args.args]
    assert ", ".join(args[:len(META[name]["tensor_params"])]) == ", ".join(META[name]["tensor_params"])
    # same signature text as the reference's generated forward(): tensors then block_*=16
    sig = ", ".join(META[name]["tensor_params"] + [f"{b}=16" for b in META[name]["block_params"]])
    assert sig == META[name]["forward"]
    assert f"def forward({sig}):" in src
    # executes on a machine without a GPU (binding happens at the first forward call)
    ns = {}
    exec(compile(src, f"<{name}>", "exec"), ns)
    assert ns["TENSOR_PARAMS"] == META[name]["tensor_params"] and callable(ns["forward"])


def test_parser_details():
    p = IRParser()
    assert p.tokenize("(a b) ; comment (x\n c,d") == ["(", "a", "b", ")", "c", ",", "d"]
    n = p.parse("(index fulltile (tile n) (elem k) (const_tile P M) -3 dummy)")
    assert [c.node_type for c in n.children] == [NodeType.FULLTILE, NodeType.TILE, NodeType.ELEM,
                                                 NodeType.CONST_TILE, NodeType.NUM, NodeType.DUMMY]
    assert n.children[4].value == -3
    multi = p.parse("(load (input Q1,K1, V1) (index fulltile))")
    assert [c.value for c in multi.children[0].children] == ["Q1", "K1", "V1"]
    assert p.parse("(tensor P+M)").children[0].value == "P+M"
    with pytest.raises(ValueError, match="Unknown operation"):
        p.parse("(frobnicate 1 2)")
    with pytest.raises(ValueError):
        p.parse("(seq (load (input X) (index fulltile))")
    with pytest.raises(ValueError):
        p.parse("")
    assert isinstance(n, ASTNode) and repr(p.parse("7")) == "num(7)"


def test_recogniser_rejects_foreign_programs():
    linear = "(store (output O) (* (load (input X) (index fulltile fulltile)) (load (input W) (index fulltile fulltile))) (index fulltile fulltile))"
    with pytest.raises(ValueError):
        recognise(IRParser().parse(linear), None)           # a plain linear layer is none of the operators
    with pytest.raises(ValueError, match="missing from the shape table"):
        recognise(IRParser().parse(linear), SHAPE_DICT)
    # an attention program whose result lands in a tensor the operator surface does not know as an output
    broken = read("vanilla").replace("(output O2)", "(output C)")
    with pytest.raises(ValueError, match="no output"):
        recognise(IRParser().parse(broken), SHAPE_DICT)
    # KeyFormer without its per-key score
    with pytest.raises(ValueError, match="C_out"):
        recognise(IRParser().parse(read("keyformer").replace("(output C_out)", "(output C)")), SHAPE_DICT)


def test_ir_file_format(tmp_path):
    f = tmp_path / "cands.txt"
    one_line = " ".join(l.split(";")[0] for l in read("vanilla").splitlines())
    f.write_text(f"3: {one_line}\n4: (dummydata)\nnot a candidate\n7: {one_line}\n")
    got = parse_ir_file(str(f))
    assert [i for i, _ in got] == [3, 7]
    assert tree(IRParser().parse(got[0][1])) == META["vanilla"]["ast"]
    assert parse_ir_file(os.path.join(IR_DIR, "roco.txt"))[0][0] == 0
    assert resolve_dim("P+M", MODEL_CONFIGS["llama"]) == 1040 and resolve_dim(5, {}) == 5


def test_schedule_follows_the_candidates_fusion_structure():
    """The launch-plan choices the recogniser derives from a candidate's loop / fusion structure."""
    from triton_b200.ir import IRParser
    from triton_b200.recognise import recognise
    ir_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "triton_b200", "ir_programs")
    progs = {n: recognise(IRParser().parse(open(os.path.join(ir_dir, n + ".txt")).read()))
             for n in ("vanilla", "prenorm", "prenorm_fused", "keyformer", "roco", "rmsnorm")}
    assert progs["prenorm"].variant == progs["prenorm_fused"].variant == "prenorm"
    assert progs["prenorm"].schedule["x_norm_in_memory"] is True          # a kernel of its own stores X_norm
    assert progs["prenorm_fused"].schedule["x_norm_in_memory"] is False   # normalised inside the projection loop
    assert progs["prenorm"].schedule["kernels"] == 4 and progs["prenorm_fused"].schedule["kernels"] == 3
    assert progs["vanilla"].schedule == {"kernels": 2, "in_memory": [], "x_norm_in_memory": False,
                                         "scores_in_memory": []}
    # candidates that keep a [H, M, P+M] score tensor in memory: accepted, the kernels never materialise it
    assert progs["keyformer"].schedule["scores_in_memory"] == ["C_exp_perturb"]
    assert progs["roco"].schedule["scores_in_memory"] == ["C_exp"]
    assert progs["rmsnorm"].schedule["in_memory"] == ["X2"]


_V_DIV = ("(store (tensor O) (/ (load (tensor O) (index (elem n) fulltile fulltile)) (bcast (load (tensor C_sum) "
          "(index (elem n) fulltile)) 2)) (index (elem n) fulltile fulltile))\n")


@pytest.mark.parametrize("what,edit,msg", (
    ("no softmax division", lambda s: s.replace(_V_DIV, ""), "without the division"),
    ("scores scaled inside exp", lambda s: s.replace("(exp (* (load (input Q)", "(exp (x 2 (* (load (input Q)")
     .replace("0 2 1)))", "0 2 1))))", 1), "multiplied by 2"),
    ("K and V swapped", lambda s: s.replace("(load (input V_cache) (index (elem n) (tile p) fulltile))",
                                            "(load (input K_cache) (index (elem n) (tile p) fulltile))"), "instead of V_cache"),
    ("cache overwritten, not appended", lambda s: s.replace("(index (elem n) (const_tile P M) fulltile))))",
                                                            "(index (elem n) fulltile fulltile))))"), "const_tile"),
    ("k projected with the wrong weight", lambda s: s.replace("(load (input WK)", "(load (input WQ)"), "WK"),
))
def test_candidates_whose_arithmetic_differs_are_refused(what, edit, msg):
    """A candidate that is not the canonical operator must raise (the harness records the error per candidate,
    vanilla_llama_benchmark.py:329-332) instead of silently getting the canonical operator's result."""
    bad = edit(read("vanilla"))
    assert bad != read("vanilla"), what
    with pytest.raises(ValueError, match=msg):
        recognise(IRParser().parse(bad), SHAPE_DICT)


def test_norms_and_statistics_are_checked_where_they_apply():
    # QKNorm whose q is stored without the per-head norm
    q = read("qknorm")
    i = q.index("(store (tensor Q1) (/ (load (tensor Q1)")
    j = q.index("(store (output Q_norm)")
    with pytest.raises(ValueError, match="Q_norm is not the per-head RMS norm"):
        recognise(IRParser().parse(q[:i] + q[j:]), SHAPE_DICT)
    # PreNorm that divides by sqrt(X2 / D) instead of sqrt(X2 / N)
    with pytest.raises(ValueError, match="normalised X"):
        recognise(IRParser().parse(read("prenorm_fused").replace("(index fulltile)) N))", "(index fulltile)) D))")), SHAPE_DICT)
    # RoCo whose second statistic is not squared
    with pytest.raises(ValueError, match="C_out2"):
        recognise(IRParser().parse(read("roco").replace("(rsum (sqr (/ (load (tensor C_exp)", "(rsum (x 1 (/ (load (tensor C_exp)")),
                  SHAPE_DICT)


def test_keyformer_temperature_comes_from_the_candidate():
    kf = read("keyformer")
    prog = recognise(IRParser().parse(kf), SHAPE_DICT)
    assert prog.schedule["tau"] == pytest.approx(1.5)              # (x 2 ..) / 3
    assert recognise(IRParser().parse(kf), SHAPE_DICT, {"TAU_E3": 1500}).schedule["tau"] == pytest.approx(1.5)
    with pytest.raises(ValueError, match="tau"):
        recognise(IRParser().parse(kf), SHAPE_DICT, {"TAU_E3": 1000})
    # tau = 1: the perturbed scores enter exp unscaled
    one = kf.replace("(exp (/ (x 2 (+ (*", "(exp (+ (*").replace("(index (elem n) fulltile (tile p))))) 3))", "(index (elem n) fulltile (tile p)))))")
    assert recognise(IRParser().parse(one), SHAPE_DICT).schedule["tau"] == pytest.approx(1.0)


def test_gated_mlp_gate_comes_from_the_candidate():
    from triton_b200.harness import GMLP_SHAPE_DICT
    silu = recognise(IRParser().parse(read("gmlp")), GMLP_SHAPE_DICT)
    glu = recognise(IRParser().parse(read("gmlp_glu")), GMLP_SHAPE_DICT)
    assert silu.variant == glu.variant == "gmlp" and silu.schedule["gate"] == 0 and glu.schedule["gate"] == 1
    # sigmoid spelled through exp: e / (1 + e)
    via_exp = read("gmlp_glu").replace("(sigmoid (load (tensor C1) (index fulltile (tile n))))",
                                       "(/ (exp (load (tensor C1) (index fulltile (tile n)))) (+ 1 (exp (load (tensor C1) (index fulltile (tile n))))))")
    assert recognise(IRParser().parse(via_exp), GMLP_SHAPE_DICT).schedule["gate"] == 1
    # the gate applied to the wrong product, and no gate at all
    with pytest.raises(ValueError, match="neither"):
        recognise(IRParser().parse(read("gmlp").replace("(sigmoid (load (tensor C1)", "(sigmoid (load (tensor C2)")), GMLP_SHAPE_DICT)
    with pytest.raises(ValueError, match="neither"):
        recognise(IRParser().parse(read("gmlp_glu").replace("(sigmoid (load (tensor C1) (index fulltile (tile n))))",
                                                              "(load (tensor C1) (index fulltile (tile n)))")), GMLP_SHAPE_DICT)
