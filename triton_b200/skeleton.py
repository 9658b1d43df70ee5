"""Checks that an IR candidate spells the arithmetic of the operator the CUDA backend will run for it.

The reference lowers every statement of a candidate (TritonGen.py:2177-3209), so a candidate whose arithmetic
differs from the canonical operator computes something different there.  This backend runs one fixed,
hand-written operator per variant; before binding it, the candidate's data flow is resolved symbolically and
compared with that operator's skeleton:

  projection   q, k, v = acc(x' * WQ|WK|WV)                      ref_rms.py:47-49
               x' = X (or X / sqrt(rsum(sqr X) / N) for PreNorm, ref_rms.py:102-103)
  per-head norm (QKNorm) of q and the appended k: t / sqrt(rsum(sqr t) / D)       ref_rms.py:217-220
  cache append: K_cache / V_cache stored through (const_tile P M)                  ref_rms.py:72-73
  scores       s = q * K_cache (unscaled), e = exp(s)                              ref_rms.py:77-78
  output       acc(e * V_cache) / acc(rsum e)   (or the division applied to e first)   ref_rms.py:78-80
  KeyFormer    e' = exp((s + noise) / tau), C_out = rsum_q(e' / acc(rsum e'))      ref_rms.py:172-174
  RoCo         C_out1 = rsum_q(p), C_out2 = rsum_q(sqr p), p = e / acc(rsum e)     ref_rms.py:274-275

Layout-only nodes (permute3, squeeze, unsqueeze, bcast), `(x 1 t)` and index expressions are ignored; loads of
`tensor` temporaries are replaced by what was last stored there; `(store T (+ (x 1 (load T)) u))` is the
accumulation idiom (TritonGen.py:2871-2892) and becomes acc(u).  Anything that does not match raises ValueError,
which the harness records for that candidate (vanilla_llama_benchmark.py:329-332) instead of timing an operator
the candidate does not describe.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

from .ir import ASTNode, NodeType

Sym = Tuple  # ('leaf', name) | ('const', value) | ('acc', e) | (op, e...) with op a NodeType value

_LAYOUT = (NodeType.PERMUTE3, NodeType.SQUEEZE, NodeType.UNSQUEEZE, NodeType.BCAST)
_TENSOR_NODES = (NodeType.INPUT, NodeType.OUTPUT, NodeType.TENSOR)
_ARITH = (NodeType.ADD, NodeType.SUB, NodeType.MUL, NodeType.DIV, NodeType.MATMUL, NodeType.EXP, NodeType.SQR,
          NodeType.SQRT, NodeType.SIGMOID, NodeType.RSUM, NodeType.CONCAT)


class Flow:
    """Symbolic values of every tensor after the program has run, statement by statement."""

    def __init__(self) -> None:
        self.temps: Dict[str, Sym] = {}            # `tensor` temporaries: last stored value
        self.outputs: Dict[str, Sym] = {}          # (output ...) tensors: last stored value
        self.append_index: Dict[str, bool] = {}    # output name -> stored through a const_tile index

    def _names(self, node: ASTNode) -> List[str]:
        return [c.value for c in node.children if c.node_type == NodeType.VAR]

    def sym(self, n: ASTNode) -> Sym:
        t = n.node_type
        if t == NodeType.NUM:
            return ("const", n.value)
        if t == NodeType.VAR:
            return ("const", n.value)
        if t in _LAYOUT:
            return self.sym(n.children[0])
        if t == NodeType.LOAD:
            target = n.children[0]
            names = self._names(target)
            if target.node_type not in _TENSOR_NODES or len(names) != 1:
                raise ValueError("load needs one (input|output|tensor name)")
            name = names[0]
            if target.node_type == NodeType.TENSOR and name in self.temps:
                return self.temps[name]
            return ("leaf", name)
        if t == NodeType.MUL:
            a, b = self.sym(n.children[0]), self.sym(n.children[1])
            if a == ("const", 1):
                return b
            if b == ("const", 1):
                return a
            return ("x", a, b)
        if t in _ARITH:
            kids = n.children
            if t == NodeType.RSUM:          # the axis is layout
                kids = kids[:1]
            return (t.value,) + tuple(self.sym(c) for c in kids)
        raise ValueError(f"unexpected {t.value} inside an expression")

    def _is_self_load(self, n: ASTNode, name: str) -> bool:
        while n.node_type in _LAYOUT or (n.node_type == NodeType.MUL and n.children[0].node_type == NodeType.NUM
                                         and n.children[0].value == 1):
            n = n.children[1] if n.node_type == NodeType.MUL else n.children[0]
        return n.node_type == NodeType.LOAD and self._names(n.children[0]) == [name]

    def store(self, n: ASTNode) -> None:
        target, value, index = n.children[0], n.children[1], n.children[-1]
        names = self._names(target)
        appended = any(c.node_type == NodeType.CONST_TILE for c in index.walk())
        for name in names:
            if value.node_type == NodeType.ADD and self._is_self_load(value.children[0], name):
                v: Sym = ("acc", self.sym(value.children[1]))
            elif value.node_type == NodeType.ADD and self._is_self_load(value.children[1], name):
                v = ("acc", self.sym(value.children[0]))
            else:
                v = self.sym(value)
            if target.node_type == NodeType.OUTPUT:
                self.outputs[name] = v
                self.append_index[name] = appended
            else:
                self.temps[name] = v

    def run(self, n: ASTNode) -> None:
        t = n.node_type
        if t == NodeType.SEQ:
            for c in n.children:
                self.run(c)
        elif t in (NodeType.PLOOP, NodeType.SLOOP):
            for c in n.children[4:]:
                self.run(c)
        elif t == NodeType.STORE:
            self.store(n)
        elif t == NodeType.DUMMY:
            return
        else:
            raise ValueError(f"statement expected, found {t.value}")


def _unacc(e: Sym) -> Sym:
    return e[1] if e[0] == "acc" else e


def _leaf(e: Sym, name: str) -> bool:
    return e == ("leaf", name)


def _rms_div(e: Sym, dim: str) -> Optional[Sym]:
    """e = t / sqrt(rsum(sqr t') / dim) -> (t, t'), else None."""
    if e[0] != "/" or e[2][0] != "sqrt":
        return None
    mean = e[2][1]
    if mean[0] != "/" or mean[2] != ("const", dim):
        return None
    ss = _unacc(mean[1])
    if ss[0] != "rsum" or ss[1][0] != "sqr":
        return None
    return (e[1], ss[1][1])


def _fail(what: str) -> None:
    raise ValueError(f"IR candidate does not spell the operator this backend runs: {what}")


def _scale_to(e: Sym, stop) -> Tuple[float, Sym]:
    """Strips constant multipliers / divisors above `stop(e)`; returns (factor, inner)."""
    f = 1.0
    while not stop(e):
        if e[0] == "x" and e[1][0] == "const" and isinstance(e[1][1], int):
            f, e = f * e[1][1], e[2]
        elif e[0] == "x" and e[2][0] == "const" and isinstance(e[2][1], int):
            f, e = f * e[2][1], e[1]
        elif e[0] == "/" and e[2][0] == "const" and isinstance(e[2][1], int) and e[2][1] != 0:
            f, e = f / e[2][1], e[1]
        else:
            break
    return f, e


class _Checker:
    def __init__(self, flow: Flow, variant: str, consts: Optional[Dict[str, int]]):
        self.f, self.variant, self.c = flow, variant, dict(consts or {})
        self.derived: Dict[str, float] = {}      # operator parameters the IR itself spells (tau)

    # ---- x as the projection reads it
    def x_ok(self, e: Sym) -> bool:
        if self.variant == "prenorm":
            if _leaf(e, "X_norm"):
                d = self.f.outputs.get("X_norm")
                r = _rms_div(d, "N") if d is not None else None
                return r is not None and _leaf(r[0], "X") and _leaf(r[1], "X")
            r = _rms_div(e, "N")
            return r is not None and _leaf(r[0], "X") and _leaf(r[1], "X")
        return _leaf(e, "X")

    def proj_ok(self, e: Sym, w: str) -> bool:
        e0 = _unacc(e)
        if e0[0] == "*" and _leaf(e0[2], w) and self.x_ok(e0[1]):
            return True
        if self.variant == "prenorm":           # row scale applied after the contraction: the same product
            r = _rms_div(e, "N")
            if r is not None and _leaf(r[1], "X"):
                inner = _unacc(r[0])
                return inner[0] == "*" and _leaf(inner[1], "X") and _leaf(inner[2], w)
        return False

    def headnorm_ok(self, e: Sym, w: str) -> bool:
        r = _rms_div(e, "D")
        return r is not None and r[0] == r[1] and self.proj_ok(r[0], w)

    def projection(self) -> str:
        out = self.f.outputs
        norm = self.variant == "qknorm"
        q_name = "Q_norm" if (norm and "Q_norm" in out) else "Q"
        if q_name in out:
            ok = self.headnorm_ok(out[q_name], "WQ") if norm else self.proj_ok(out[q_name], "WQ")
            if not ok:
                _fail(f"{q_name} is not {'the per-head RMS norm of ' if norm else ''}X @ WQ"
                      + (" on the normalised X" if self.variant == "prenorm" else ""))
        for name, w, normed in (("K_cache", "WK", norm), ("V_cache", "WV", False)):
            if name not in out:
                _fail(f"{name} rows [P, P+M) are never stored")
            if not self.f.append_index.get(name, False):
                _fail(f"{name} is not stored through (const_tile P M): the cache append")
            ok = self.headnorm_ok(out[name], w) if normed else self.proj_ok(out[name], w)
            if not ok:
                _fail(f"{name} does not receive {'the per-head RMS norm of ' if normed else ''}X @ {w}")
        return q_name

    # ---- attention core
    def score_ok(self, s: Sym, q_name: str) -> bool:
        if s[0] != "*" or not _leaf(s[2], "K_cache"):
            return False
        q = s[1]
        if _leaf(q, q_name):
            return q_name in self.f.outputs
        return self.headnorm_ok(q, "WQ") if self.variant == "qknorm" else self.proj_ok(q, "WQ")

    def plain_exp(self, e: Sym, q_name: str) -> bool:
        if e[0] != "exp":
            return False
        f, s = _scale_to(e[1], lambda t: t[0] == "*")
        if not self.score_ok(s, q_name):
            return False
        if abs(f - 1.0) > 1e-9:
            _fail(f"the scores are multiplied by {f:g} inside exp; the score scale of this backend comes from the "
                  "SCALE_RSQRT_D constant, the IR must leave q k^T unscaled")
        return True

    def pert_exp(self, e: Sym, q_name: str) -> bool:
        if e[0] != "exp":
            return False
        f, s = _scale_to(e[1], lambda t: t[0] == "+")
        if s[0] != "+":
            return False
        a, b = s[1], s[2]
        if _leaf(a, "noise"):
            a, b = b, a
        if not (_leaf(b, "noise") and self.score_ok(a, q_name)):
            return False
        if not f > 0:
            _fail("the perturbed scores are scaled by a non-positive constant")
        if "TAU_E3" in self.c:
            tau = self.c["TAU_E3"] * 1e-3
            if abs(f * tau - 1.0) > 1e-6:
                _fail(f"the perturbed scores are scaled by {f:g}, but tau = {tau:g} (TAU_E3) means 1 / tau = {1 / tau:g}")
        self.derived["tau"] = 1.0 / f          # the temperature is what the candidate spells, e.g. (x 2 ..) / 3 = 1 / 1.5
        return True

    def softmax_of(self, p: Sym, exp_ok) -> bool:
        """p = e / acc(rsum e) with e accepted by exp_ok."""
        if p[0] != "/":
            return False
        den = _unacc(p[2])
        return exp_ok(p[1]) and den[0] == "rsum" and den[1] == p[1]

    def attention(self, q_name: str) -> None:
        out = self.f.outputs
        o_name = next((n for n in ("O2", "O1", "O") if n in out), None)
        if o_name is None:
            _fail("no output tensor (O2, O1 or O) is stored")
        o = out[o_name]
        plain = lambda e: self.plain_exp(e, q_name)
        ok = False
        if o[0] == "/":                                   # acc(e * V) / acc(rsum e)
            num, den = _unacc(o[1]), _unacc(o[2])
            ok = (num[0] == "*" and plain(num[1]) and _leaf(num[2], "V_cache") and den[0] == "rsum" and den[1] == num[1])
            if not ok and num[0] == "*" and plain(num[1]) and _leaf(num[2], "K_cache"):
                _fail("the probabilities multiply K_cache instead of V_cache")
        else:                                             # acc((e / acc(rsum e)) * V)
            num = _unacc(o)
            ok = num[0] == "*" and self.softmax_of(num[1], plain) and _leaf(num[2], "V_cache")
            if not ok and num[0] == "*" and num[1][0] == "exp":
                _fail(f"{o_name} is exp(q k^T) @ V_cache without the division by the row sums (no softmax)")
        if not ok:
            _fail(f"{o_name} is not softmax(q k^T) @ V_cache")
        if self.variant == "keyformer":
            co = out.get("C_out")
            pert = lambda e: self.pert_exp(e, q_name)
            if co is None or co[0] != "rsum" or not self.softmax_of(co[1], pert):
                _fail("C_out is not the sum over queries of softmax((q k^T + noise) / tau)")
        if self.variant == "roco":
            c1, c2 = out.get("C_out1"), out.get("C_out2")
            if c1 is None or c1[0] != "rsum" or not self.softmax_of(c1[1], plain):
                _fail("C_out1 is not the sum over queries of the attention probabilities")
            if c2 is None or c2[0] != "rsum" or c2[1][0] != "sqr" or not self.softmax_of(c2[1][1], plain):
                _fail("C_out2 is not the sum over queries of the squared attention probabilities")


def _check_gmlp(ast: ASTNode) -> Dict[str, float]:
    """Gated MLP (gmlp_benchmark.py:53-74): O = gate(C1) x C2 with C1 = acc(X * W1), C2 = acc(X * W2) and
    gate(c) = c x sigmoid(c) (SiLU) or sigmoid(c).  sigmoid may be spelled (sigmoid c) or e / (1 + e) with e = exp(c).
    Returns {"gate": 0 | 1} (TRN_GATE_SILU | TRN_GATE_SIGMOID)."""
    flow = Flow()
    flow.run(ast)
    o = flow.outputs.get("O")
    if o is None:
        _fail("the gated MLP stores no output O")

    def prod(e, w):
        e = _unacc(e)
        return e[0] == "*" and _leaf(e[1], "X") and _leaf(e[2], w)

    def sigm(e):
        if e[0] == "sigmoid" and prod(e[1], "W1"):
            return True
        if e[0] == "/" and e[1][0] == "exp" and prod(e[1][1], "W1") and e[2][0] == "+":
            a, b = e[2][1], e[2][2]
            return (a == ("const", 1) and b == e[1]) or (b == ("const", 1) and a == e[1])
        return False

    def factors(e):
        return factors(e[1]) + factors(e[2]) if e[0] == "x" else [e]

    fs = factors(o)
    n_c2 = sum(1 for f in fs if prod(f, "W2"))
    n_sig = sum(1 for f in fs if sigm(f))
    n_c1 = sum(1 for f in fs if prod(f, "W1"))
    if n_c2 == 1 and n_sig == 1 and n_c1 == 1 and len(fs) == 3:
        return {"gate": 0}
    if n_c2 == 1 and n_sig == 1 and len(fs) == 2:
        return {"gate": 1}
    _fail("O is neither (C1 x sigmoid(C1)) x C2 nor sigmoid(C1) x C2 with C1 = X @ W1, C2 = X @ W2")
    return {}


def check_skeleton(ast: ASTNode, variant: str, consts: Optional[Dict[str, int]] = None) -> Dict[str, float]:
    """Raises ValueError unless the candidate's arithmetic is the operator `variant` of this backend.  Returns the
    operator parameters the candidate spells itself (KeyFormer: {"tau": ...})."""
    if variant == "lora":
        return {}       # recognised by its tensor table only (lora_benchmark.py:41-64)
    if variant == "gmlp":
        return _check_gmlp(ast)
    flow = Flow()
    flow.run(ast)
    ck = _Checker(flow, variant, consts)
    if variant == "rmsnorm":
        d = flow.outputs.get("X_norm")
        r = _rms_div(d, "N") if d is not None else None
        if r is None or not (_leaf(r[0], "X") and _leaf(r[1], "X")):
            _fail("X_norm is not X / sqrt(rsum(sqr X) / N)")
        return {}
    q_name = ck.projection()
    ck.attention(q_name)
    return ck.derived
