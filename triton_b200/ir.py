"""Front end for Trinity's tile-level IR: s-expression text -> ASTNode tree.

Same language and same node vocabulary as the reference front end (IrParser.py:6-134, NodeType.py:3-33,
AstNode.py:5-9), so that IR files written for the reference parse to the same tree here:
  * `;` starts a comment; tokens are `(`, `)`, `,` or runs of other non-space characters;
  * integers (optionally negative) become NUM nodes, bare `fulltile` / `dummy` become their node types,
    every other atom is a VAR;
  * `tensor` / `input` / `output` take one name or a comma-separated list of names (fan-out);
  * an unknown operator raises ValueError.
This module is what the package ships (the reference checkout is not needed at run time).
"""
from __future__ import annotations

import enum
import re
from dataclasses import dataclass, field
from typing import Any, Iterator, List, Optional


class NodeType(enum.Enum):
    PLOOP = "ploop"
    SLOOP = "sloop"
    INPUT = "input"
    OUTPUT = "output"
    TILE = "tile"
    FULLTILE = "fulltile"
    DUMMY = "dummy"
    INDEX = "index"
    LOAD = "load"
    STORE = "store"
    SEQ = "seq"
    ADD = "+"
    SUB = "-"
    MUL = "x"
    DIV = "/"
    MATMUL = "*"
    EXP = "exp"
    SQR = "sqr"
    SQRT = "sqrt"
    SIGMOID = "sigmoid"
    RSUM = "rsum"
    CONCAT = "concat"
    BCAST = "bcast"
    NUM = "num"
    VAR = "var"
    ELEM = "elem"
    PERMUTE3 = "permute3"
    SQUEEZE = "squeeze"
    UNSQUEEZE = "unsqueeze"
    CONST_TILE = "const_tile"
    TENSOR = "tensor"


# operators that may open a list; NUM and VAR are atoms only
_OPERATORS = {t.value: t for t in NodeType if t not in (NodeType.NUM, NodeType.VAR)}
_NAME_LIST_OPS = ("tensor", "input", "output")
_TOKEN = re.compile(r"[(),]|[^\s(),]+")
_INT = re.compile(r"-?\d+\Z")


@dataclass
class ASTNode:
    node_type: NodeType
    children: List["ASTNode"] = field(default_factory=list)
    value: Any = None

    def __repr__(self) -> str:
        if self.value is not None:
            return f"{self.node_type.value}({self.value})"
        return f"{self.node_type.value}({self.children})"

    def walk(self) -> Iterator["ASTNode"]:
        """Pre-order traversal."""
        stack = [self]
        while stack:
            n = stack.pop()
            yield n
            stack.extend(reversed(n.children))


class IRParser:
    """Recursive-descent parser over the token list."""

    def __init__(self) -> None:
        self.tokens: List[str] = []
        self.pos = 0

    def tokenize(self, code: str) -> List[str]:
        lines = (line.split(";", 1)[0] for line in code.splitlines())
        return _TOKEN.findall("\n".join(lines))

    def parse(self, code: str) -> ASTNode:
        self.tokens = self.tokenize(code)
        self.pos = 0
        return self._expr()

    # -- helpers
    def _peek(self) -> Optional[str]:
        return self.tokens[self.pos] if self.pos < len(self.tokens) else None

    def _take(self) -> str:
        if self.pos >= len(self.tokens):
            raise ValueError("Unexpected end of input")
        tok = self.tokens[self.pos]
        self.pos += 1
        return tok

    def _atom(self, tok: str) -> ASTNode:
        if _INT.match(tok):
            return ASTNode(NodeType.NUM, [], int(tok))
        if tok == "fulltile":
            return ASTNode(NodeType.FULLTILE, [])
        if tok == "dummy":
            return ASTNode(NodeType.DUMMY, [])
        return ASTNode(NodeType.VAR, [], tok)

    def _expr(self) -> ASTNode:
        tok = self._take()
        if tok != "(":
            return self._atom(tok)
        op = self._take()
        if op in _NAME_LIST_OPS:
            children = self._name_list()
        else:
            children = []
            while self._peek() not in (")", None):
                children.append(self._expr())
        if self._peek() is None:
            raise ValueError("Missing closing parenthesis")
        self._take()  # ')'
        if op not in _OPERATORS:
            raise ValueError(f"Unknown operation: {op}")
        return ASTNode(_OPERATORS[op], children)

    def _name_list(self) -> List[ASTNode]:
        """`a` or `a, b, c` -> one child per name (a lone name may also be any expression)."""
        first = self._expr()
        names = [first]
        while self._peek() == ",":
            self._take()
            names.append(self._atom(self._take()))
        return names


def parse(code: str) -> ASTNode:
    return IRParser().parse(code)
