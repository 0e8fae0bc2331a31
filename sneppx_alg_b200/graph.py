"""Expression graph with an op-fusion planner (the reference's ``kernel/tensor/tensor_expr.c``:
``SNEPPX_expr_plan_fusions`` — unary chains and matmul epilogues, toposort, memory estimate; Python
``graph_compiler.py`` / ``graph_optimizer.py``).

The planner maps  matmul -> (+ bias) -> (activation)  onto ONE tensor-core GEMM launch with a fused epilogue
(``ops.gemm(bias=, act=)``) and collapses chains of unary element-wise ops into one composed callable."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch
import torch.nn.functional as F

from .ops.gemm import gemm

UNARY: Dict[str, Callable] = {"relu": torch.relu, "gelu": F.gelu, "silu": F.silu, "tanh": torch.tanh,
                              "sigmoid": torch.sigmoid, "neg": torch.neg, "exp": torch.exp, "sqrt": torch.sqrt}
EPILOGUE_ACTS = ("relu", "gelu", "silu")


@dataclass
class ExprNode:
    op: str                       # input | const | matmul | add | mul | <unary>
    inputs: List[int] = field(default_factory=list)
    value: Optional[torch.Tensor] = None
    name: str = ""


class ExprGraph:
    def __init__(self):
        self.nodes: List[ExprNode] = []

    def _add(self, op, inputs=(), value=None, name=""):
        self.nodes.append(ExprNode(op, list(inputs), value, name))
        return len(self.nodes) - 1

    def input(self, name):
        return self._add("input", name=name)

    def const(self, value):
        return self._add("const", value=value)

    def matmul(self, a, w):
        """a @ w^T with w stored [out, in] (the linear-layer convention)."""
        return self._add("matmul", (a, w))

    def add(self, a, b):
        return self._add("add", (a, b))

    def mul(self, a, b):
        return self._add("mul", (a, b))

    def unary(self, op, a):
        assert op in UNARY
        return self._add(op, (a,))

    # ---- analysis
    def toposort(self, outputs):
        seen, order = set(), []

        def visit(i):
            if i in seen:
                return
            seen.add(i)
            for j in self.nodes[i].inputs:
                visit(j)
            order.append(i)
        for o in outputs:
            visit(o)
        return order

    def users(self):
        u = {i: [] for i in range(len(self.nodes))}
        for i, n in enumerate(self.nodes):
            for j in n.inputs:
                u[j].append(i)
        return u

    def plan_fusions(self, outputs):
        """Returns a list of fused groups [{'kind': 'gemm_epilogue'|'unary_chain', 'nodes': [...]}]."""
        users, groups, taken = self.users(), [], set()
        for i in self.toposort(outputs):
            n = self.nodes[i]
            if n.op == "matmul" and i not in taken:
                grp, cur = [i], i
                if len(users[cur]) == 1 and self.nodes[users[cur][0]].op == "add":
                    add = users[cur][0]
                    other = [j for j in self.nodes[add].inputs if j != cur]
                    if other and self.nodes[other[0]].op == "const" and self.nodes[other[0]].value.dim() == 1:
                        grp.append(add)
                        cur = add
                if len(users[cur]) == 1 and self.nodes[users[cur][0]].op in EPILOGUE_ACTS:
                    grp.append(users[cur][0])
                if len(grp) > 1:
                    groups.append({"kind": "gemm_epilogue", "nodes": grp})
                    taken.update(grp)
            elif n.op in UNARY and i not in taken:
                grp, cur = [i], i
                while len(users[cur]) == 1 and self.nodes[users[cur][0]].op in UNARY and users[cur][0] not in taken:
                    cur = users[cur][0]
                    grp.append(cur)
                if len(grp) > 1:
                    groups.append({"kind": "unary_chain", "nodes": grp})
                    taken.update(grp)
        return groups

    def memory_estimate(self, outputs, shapes: Dict[int, tuple], elem_bytes=2, fused=True):
        """Bytes of intermediate tensors materialised; fused groups materialise only their last node."""
        hidden = set()
        if fused:
            for g in self.plan_fusions(outputs):
                hidden.update(g["nodes"][:-1])
        total = 0
        for i in self.toposort(outputs):
            if self.nodes[i].op not in ("input", "const") and i not in hidden and i in shapes:
                n = 1
                for d in shapes[i]:
                    n *= d
                total += n * elem_bytes
        return total

    # ---- execution
    def run(self, outputs, feeds: Dict[str, torch.Tensor], fuse=True):
        vals: Dict[int, torch.Tensor] = {}
        plan = {g["nodes"][0]: g for g in self.plan_fusions(outputs)} if fuse else {}
        skip = {j for g in plan.values() for j in g["nodes"][1:]}
        self.launches = 0
        for i in self.toposort(outputs):
            n = self.nodes[i]
            if i in skip:
                continue
            if n.op == "input":
                vals[i] = feeds[n.name]
            elif n.op == "const":
                vals[i] = n.value
            elif i in plan and plan[i]["kind"] == "gemm_epilogue":
                g = plan[i]["nodes"]
                a, w = vals[n.inputs[0]], vals[n.inputs[1]]
                bias, act = None, None
                for j in g[1:]:
                    nj = self.nodes[j]
                    if nj.op == "add":
                        bias = self.nodes[[k for k in nj.inputs if self.nodes[k].op == "const"][0]].value
                    else:
                        act = nj.op
                a2 = a.reshape(-1, a.shape[-1])
                vals[g[-1]] = gemm(a2, w, bias=bias, act=act).view(*a.shape[:-1], w.shape[0])
                self.launches += 1
            elif i in plan:
                g = plan[i]["nodes"]
                x = vals[n.inputs[0]]
                for j in g:
                    x = UNARY[self.nodes[j].op](x)
                vals[g[-1]] = x
                self.launches += 1
            elif n.op == "matmul":
                a = vals[n.inputs[0]]
                vals[i] = gemm(a.reshape(-1, a.shape[-1]), vals[n.inputs[1]]).view(*a.shape[:-1], -1)
                self.launches += 1
            elif n.op == "add":
                vals[i] = vals[n.inputs[0]] + vals[n.inputs[1]]
                self.launches += 1
            elif n.op == "mul":
                vals[i] = vals[n.inputs[0]] * vals[n.inputs[1]]
                self.launches += 1
            else:
                vals[i] = UNARY[n.op](vals[n.inputs[0]])
                self.launches += 1
        return [vals[o] for o in outputs]
