"""Maps a parsed IR program onto the operator the CUDA backend runs for it.

The reference lowers the AST statement by statement into Triton source (TritonGen.py:348-539).  Here
the AST is only *recognised*: which of the operators it spells (by the tensor vocabulary of
convert_eval_rms.py:62-108 and the operations applied to it), which tensors the caller must pass
(TENSOR_PARAMS, TritonGen.py:563-570) and which block-size keywords the loops imply (BLOCK_PARAMS,
TritonGen.py:548-556, 571).  Everything the kernels need beyond that comes from the shape and constant
dictionaries the harness supplies.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Tuple

from .ir import ASTNode, NodeType
from .skeleton import check_skeleton

_TENSOR_NODES = (NodeType.INPUT, NodeType.OUTPUT, NodeType.TENSOR)
_LOOPS = (NodeType.PLOOP, NodeType.SLOOP)


@dataclass
class Access:
    name: str
    kind: NodeType              # INPUT / OUTPUT / TENSOR
    is_store: bool
    kernel: int                 # index of the top-level seq child
    sloop: Optional[int]        # id of the innermost enclosing sloop (None outside any)
    tiled_by_sloop: bool        # the index expression tiles a dim with an sloop variable


@dataclass
class Program:
    variant: str                        # vanilla | prenorm | qknorm | keyformer | roco | rmsnorm | lora | gmlp
    tensor_params: List[str]
    block_params: List[str]
    tensors: Set[str] = field(default_factory=set)
    n_kernels: int = 1
    # What the candidate's loop / fusion structure selects in the CUDA backend's launch plan:
    #   kernels            top-level statements = kernels the reference would launch (TritonGen.py:590)
    #   in_memory          `tensor` temporaries the candidate keeps in memory between kernels or sloops
    #   x_norm_in_memory   PreNorm: X_norm is stored by one kernel and loaded by another -> the backend runs
    #                      normalise-then-project and fills the caller's X_norm; otherwise the row scale is
    #                      folded into the projection's epilogue and X_norm never exists
    #   scores_in_memory   the candidate materialises [H, M, P+M] score tensors (C, C_exp, ...): the backend
    #                      never does (online softmax); those tensors are accepted and left untouched
    schedule: Dict[str, object] = field(default_factory=dict)


def _names(node: ASTNode) -> List[str]:
    return [c.value for c in node.children if c.node_type == NodeType.VAR]


def _flatten_seq(node: ASTNode) -> List[ASTNode]:
    """Top-level `seq` children, nested seqs flattened, dummy-only statements dropped
    (TritonGen.py:441-455)."""
    if node.node_type != NodeType.SEQ:
        return [node]
    out: List[ASTNode] = []
    for c in node.children:
        if c.node_type == NodeType.SEQ:
            out.extend(_flatten_seq(c))
        elif c.node_type != NodeType.DUMMY:
            out.append(c)
    return out


def _collect(node: ASTNode, kernel: int, sloop_vars: Dict[str, int], cur_sloop: Optional[int], out: List[Access],
             blocks: Set[str], counter: List[int]) -> None:
    t = node.node_type
    if t in _LOOPS:
        # (ploop|sloop start end tile var body)
        if len(node.children) < 5:
            raise ValueError(f"{t.value} needs (start end tile var body)")
        tile, var = node.children[2], node.children[3]
        if tile.node_type == NodeType.VAR and var.node_type == NodeType.VAR:
            blocks.add(f"block_{var.value}")
        inner_vars = dict(sloop_vars)
        inner_sloop = cur_sloop
        if t == NodeType.SLOOP:
            counter[0] += 1
            inner_sloop = counter[0]
            inner_vars[var.value] = inner_sloop
        for body in node.children[4:]:
            _collect(body, kernel, inner_vars, inner_sloop, out, blocks, counter)
        return
    if t in (NodeType.LOAD, NodeType.STORE):
        target = node.children[0]
        if target.node_type in _TENSOR_NODES:
            index = node.children[-1]
            tiled = any(n.node_type == NodeType.TILE and n.children and n.children[0].value in sloop_vars
                        for n in index.walk())
            for name in _names(target):
                out.append(Access(name, target.node_type, t == NodeType.STORE, kernel, cur_sloop, tiled))
        for c in node.children[1:]:
            _collect(c, kernel, sloop_vars, cur_sloop, out, blocks, counter)
        return
    for c in node.children:
        _collect(c, kernel, sloop_vars, cur_sloop, out, blocks, counter)


def _memory_resident(accesses: Sequence[Access]) -> Set[str]:
    """Tensors the caller has to pass: every input / output, plus `tensor` temporaries that cannot
    stay in registers — used by more than one kernel, or tiled by an sloop variable and touched in
    more than one sloop (the reference's cross-kernel / cross-sloop-memory classes,
    TritonGen.py:1007-1042, 1573-1744)."""
    resident: Set[str] = set()
    by_name: Dict[str, List[Access]] = {}
    for a in accesses:
        by_name.setdefault(a.name, []).append(a)
    for name, acc in by_name.items():
        if any(a.kind in (NodeType.INPUT, NodeType.OUTPUT) for a in acc):
            resident.add(name)
            continue
        if len({a.kernel for a in acc}) > 1:
            resident.add(name)
            continue
        loops = {a.sloop for a in acc if a.tiled_by_sloop}
        if len(loops) > 1:
            resident.add(name)
    return resident


def _has_op(root: ASTNode, op: NodeType) -> bool:
    return any(n.node_type == op for n in root.walk())


def recognise(ast: ASTNode, shape_dict: Optional[Dict[str, Tuple]] = None,
              const_dict: Optional[Dict[str, int]] = None) -> Program:
    """Names the operator, then checks that the candidate's arithmetic IS that operator (skeleton.py): a candidate
    that differs from it (no softmax division, another score scale, a norm applied elsewhere, K and V swapped ...)
    raises ValueError instead of being given the canonical operator's result."""
    kernels = _flatten_seq(ast)
    accesses: List[Access] = []
    blocks: Set[str] = set()
    counter = [0]
    for ki, k in enumerate(kernels):
        _collect(k, ki, {}, None, accesses, blocks, counter)
    if not accesses:
        raise ValueError("IR program touches no tensor")
    names = {a.name for a in accesses}
    if shape_dict is not None:
        unknown = sorted(n for n in names if n not in shape_dict)
        if unknown:
            raise ValueError(f"IR uses tensors missing from the shape table: {unknown}")
    # tensors the program delivers: stores through an (output ...) node
    stored = {a.name for a in accesses if a.is_store and a.kind == NodeType.OUTPUT}

    has_attention = _has_op(ast, NodeType.EXP) and _has_op(ast, NodeType.MATMUL)
    if {"X", "W", "A", "B"} <= names and "O" in stored and "K_cache" not in names:
        # LoRA linear layer (lora_benchmark.py:41-64): O = X @ W + (X @ A) @ B
        tensor_params = sorted(_memory_resident(accesses))
        schedule = {"kernels": len(kernels), "in_memory": sorted(n for n in tensor_params if n in ("C", "D", "E")),
                    "x_norm_in_memory": False, "scores_in_memory": []}
        check_skeleton(ast, "lora", const_dict)
        return Program("lora", tensor_params, sorted(blocks), names, len(kernels), schedule)
    if {"X", "W1", "W2"} <= names and "O" in stored and "K_cache" not in names:
        # gated MLP (gmlp_benchmark.py:53-74): O = gate(X @ W1) x (X @ W2); the gate is what the candidate spells
        derived = check_skeleton(ast, "gmlp", const_dict)
        tensor_params = sorted(_memory_resident(accesses))
        schedule = {"kernels": len(kernels), "in_memory": sorted(n for n in tensor_params if n in ("C1", "C1_exp", "C2")),
                    "x_norm_in_memory": False, "scores_in_memory": [], "gate": int(derived["gate"])}
        return Program("gmlp", tensor_params, sorted(blocks), names, len(kernels), schedule)
    if "noise" in names:
        variant = "keyformer"
    elif {"C_out1", "C_out2"} & names:
        variant = "roco"
    elif {"Q_norm", "K_norm"} & names:
        variant = "qknorm"
    elif ({"X_norm", "X2"} & names) and has_attention:
        # X2 (row sums of squares of X) marks the candidates that normalise inside the projection loop and
        # never name X_norm
        variant = "prenorm"
    elif has_attention:
        variant = "vanilla"
    elif "X_norm" in stored:
        variant = "rmsnorm"
    else:
        raise ValueError("IR program is not one of: vanilla, prenorm, qknorm, keyformer, roco, rmsnorm")

    if variant != "rmsnorm":
        need = {"X", "WQ", "WK", "WV", "K_cache", "V_cache"}
        missing = sorted(need - names)
        if missing:
            raise ValueError(f"attention block IR lacks tensors {missing}")
        if not ({"O2", "O1", "O"} & stored):
            raise ValueError("attention block IR stores no output tensor (O2, O1 or O)")
        if variant == "keyformer" and "C_out" not in stored:
            raise ValueError("KeyFormer IR must store C_out")
        if variant == "roco" and not {"C_out1", "C_out2"} <= stored:
            raise ValueError("RoCo IR must store C_out1 and C_out2")
    derived = check_skeleton(ast, variant, const_dict)
    tensor_params = sorted(_memory_resident(accesses))
    declared_io = {a.name for a in accesses if a.kind in (NodeType.INPUT, NodeType.OUTPUT)}
    in_memory = sorted(n for n in tensor_params if n not in declared_io)
    score_like = {"C", "C_exp", "C_div", "C_sum", "C_perturb", "C_exp_perturb", "C_sum_perturb", "C_div_perturb"}
    schedule = {
        "kernels": len(kernels),
        "in_memory": in_memory,
        "x_norm_in_memory": variant == "prenorm" and "X_norm" in tensor_params,
        "scores_in_memory": sorted(score_like & set(tensor_params)),
    }
    if "tau" in derived:
        schedule["tau"] = round(derived["tau"], 9)      # KeyFormer's temperature as the candidate spells it
    return Program(variant, tensor_params, sorted(blocks), names, len(kernels), schedule)
