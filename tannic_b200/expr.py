"""Lazy elementwise expressions that evaluate as ONE fused kernel.

The reference builds an expression template per operator (`Binary<Op, L, R>`, `Unary`, `Function`:
include/tannic/operations.hpp:168-313, include/tannic/functions.hpp:52-160) and evaluates it node by node:
every `forward()` allocates a full-size temporary and launches one kernel (include/tannic/tensor.hpp:351-371).
This module keeps the same surface — operators and functions on tensors, `forward()` to get the result — but
hands the whole tree to `tn_eltwise_program`, so that an expression like `log(X) + Y * Y - exp(X)` reads X and
Y once and writes Z once.

    from tannic_b200.expr import lazy, log, exp
    X, Y = lazy(x), lazy(y)
    z = (log(X) + Y * Y - exp(X)).forward()

A tree is fused when it fits the program format (one dtype, at most TN_PROGRAM_MAX_INPUTS distinct tensors and
TN_PROGRAM_MAX_NODES nodes after common subexpressions are merged); otherwise it is evaluated node by node
through the single-operator entry points, exactly like the reference (mixed dtypes promote there).
Results are identical either way: the fused kernel rounds every node to the storage dtype.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import _abi as A
from . import ops

MAX_INPUTS = 4
MAX_NODES = 16

_BINARY = {"add": A.OP_ADD, "sub": A.OP_SUB, "mul": A.OP_MUL, "pow": A.OP_POW}
_UNARY = {"neg": A.OP_NEG, "log": A.OP_LOG, "exp": A.OP_EXP, "sqrt": A.OP_SQRT, "rsqrt": A.OP_RSQRT, "abs": A.OP_ABS,
          "sin": A.OP_SIN, "cos": A.OP_COS, "tan": A.OP_TAN, "sinh": A.OP_SINH, "cosh": A.OP_COSH, "tanh": A.OP_TANH}


class Expr:
    """A node of the tree: a tensor leaf, a unary / binary operator, or a multiplication by a scalar."""

    __slots__ = ("op", "args", "imm", "tensor")

    def __init__(self, op: str, args: Sequence["Expr"] = (), imm: float = 0.0, tensor: torch.Tensor | None = None):
        self.op, self.args, self.imm, self.tensor = op, tuple(args), float(imm), tensor

    # ---- operators (include/tannic/operations.hpp:252-313) ----
    def __add__(self, other): return Expr("add", (self, lazy(other)))
    def __radd__(self, other): return Expr("add", (lazy(other), self))
    def __sub__(self, other): return Expr("sub", (self, lazy(other)))
    def __rsub__(self, other): return Expr("sub", (lazy(other), self))
    def __neg__(self): return Expr("neg", (self,))
    def __pow__(self, other): return Expr("pow", (self, lazy(other)))

    def __mul__(self, other):
        if isinstance(other, (int, float)):
            return Expr("scale", (self,), imm=other)  # Scalar(value, tensor.dtype()): operations.hpp:295-313
        return Expr("mul", (self, lazy(other)))

    def __rmul__(self, other):
        if isinstance(other, (int, float)):
            return Expr("scale", (self,), imm=other)
        return Expr("mul", (lazy(other), self))

    # ---- structure ----
    def key(self):
        if self.op == "leaf":
            t = self.tensor
            return ("leaf", t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype, str(t.device))
        return (self.op, self.imm) + tuple(a.key() for a in self.args)

    def compile(self, require_device: bool = True):
        """(inputs, nodes) for `tn_eltwise_program`, or None when the tree does not fit its format."""
        inputs, input_ids, value_of, nodes = [], {}, {}, []

        def visit(e: "Expr"):
            k = e.key()
            if k in value_of:
                return value_of[k]
            if e.op == "leaf":
                if k not in input_ids:
                    if len(inputs) == MAX_INPUTS:
                        raise _TooBig
                    input_ids[k] = len(inputs)
                    inputs.append(e.tensor)
                vid = input_ids[k]
            else:
                operands = [visit(a) for a in e.args]
                if len(nodes) == MAX_NODES:
                    raise _TooBig
                if e.op == "scale":
                    nodes.append((A.OP_SCALE, operands[0], operands[0], e.imm))
                elif e.op in _UNARY:
                    nodes.append((_UNARY[e.op], operands[0], operands[0], e.imm))
                else:
                    nodes.append((_BINARY[e.op], operands[0], operands[1], 0.0))
                vid = MAX_INPUTS + len(nodes) - 1
            value_of[k] = vid
            return vid

        try:
            visit(self)
        except _TooBig:
            return None
        if not nodes:
            return None
        dtypes = {t.dtype for t in inputs}
        if len(dtypes) != 1 or next(iter(dtypes)) not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
            return None
        if require_device and (any(not t.is_cuda for t in inputs) or len({t.device for t in inputs}) != 1):
            return None
        return inputs, nodes

    def forward(self) -> torch.Tensor:
        if self.op == "leaf":
            return self.tensor
        plan = self.compile()
        if plan is not None:
            inputs, nodes = plan
            return ops.program(inputs, nodes)
        return self._eval({})

    def _eval(self, memo) -> torch.Tensor:
        k = self.key()
        if k in memo:
            return memo[k]
        if self.op == "leaf":
            out = self.tensor
        elif self.op == "scale":
            out = ops.scale(self.args[0]._eval(memo), self.imm)
        elif self.op == "rsqrt":
            out = ops.rsqrt(self.args[0]._eval(memo), self.imm)
        elif self.op in _UNARY:
            out = getattr(ops, self.op)(self.args[0]._eval(memo))
        else:
            out = getattr(ops, self.op)(self.args[0]._eval(memo), self.args[1]._eval(memo))
        memo[k] = out
        return out


class _TooBig(Exception):
    pass


def lazy(x) -> Expr:
    """Wraps a tensor as a leaf (an Expr is returned as it is)."""
    if isinstance(x, Expr):
        return x
    if not isinstance(x, torch.Tensor):
        raise TypeError("operands are tensors or expressions; a scalar only multiplies")
    return Expr("leaf", tensor=x)


def _function(name):
    def fn(x):
        return Expr(name, (lazy(x),))
    fn.__name__ = name
    fn.__doc__ = f"include/tannic/functions.hpp: {name}(tensor) as a lazy node."
    return fn


log, exp, sqrt, abs_, sin, cos, tan, sinh, cosh, tanh = (_function(n) for n in ("log", "exp", "sqrt", "abs", "sin", "cos", "tan", "sinh", "cosh", "tanh"))


def rsqrt(x, epsilon: float = 0.0) -> Expr:
    """include/tannic/functions.hpp: rsqrt(tensor, epsilon) = 1 / sqrt(x + epsilon)."""
    return Expr("rsqrt", (lazy(x),), imm=epsilon)
