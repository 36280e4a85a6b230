"""torch.nn.Module -> linalg-on-tensors MLIR text.

The reference does this step with torch-mlir (python/torch/torch2linalg/convert.py:12-38:
`export_and_import(..., output_type=LINALG_ON_TENSORS)`).  torch-mlir is not a dependency here: the model is
traced with `torch.export` and the ATen graph is written out directly as `linalg.generic` / `linalg.fill` /
`linalg.matmul` on tensors, one op per ATen node, for the operator subset of the fused-group path:

    add sub mul div maximum minimum (tensor-tensor with numpy broadcasting, tensor-scalar), relu, leaky_relu, neg, abs,
    clamp / clamp_min / clamp_max with number bounds,
    unsqueeze / squeeze of unit dimensions and t / transpose / permute (views, no op emitted: a permuted operand of
    an elementwise op becomes a permuted indexing map), sum over the last dimension,
    mm / matmul of 2-D operands, addmm with a row-broadcast bias.

Dynamic dimensions become `?` and are read back with `tensor.dim`.  Anything else raises UnsupportedTorchOp
naming the node, so an unsupported model fails at conversion time and never silently computes something else.
Fusing the per-node generics into one group is the job of afir-opt, as in the reference.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch

ELEM_TYPES = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}
Size = Union[int, str]  # static extent, or the name of a dynamic-size symbol


class UnsupportedTorchOp(NotImplementedError):
    pass


@dataclass
class _Tensor:
    """A value of the traced graph: a materialised tensor (`ssa`, `base` extents) seen through a view: every base
    dimension appears once in `view` (in any order: a permutation), entries None are inserted unit dimensions."""
    ssa: str
    elem: str
    base: List[Size]
    view: List[Optional[int]] = field(default_factory=list)

    def __post_init__(self):
        if not self.view:
            self.view = list(range(len(self.base)))

    @property
    def shape(self) -> List[Size]:
        return [1 if v is None else self.base[v] for v in self.view]

    @property
    def type(self) -> str:
        return _tensor_type(self.base, self.elem)


def _tensor_type(sizes: Sequence[Size], elem: str) -> str:
    return "tensor<" + "".join(("?" if isinstance(s, str) else str(s)) + "x" for s in sizes) + elem + ">"


def _float_literal(v: float) -> str:
    return f"{float(v):.6e}"


class _Emitter:
    def __init__(self, func_name: str):
        self.func_name = func_name
        self.lines: List[str] = []
        self.maps: Dict[str, str] = {}      # map text -> alias
        self.dim_ssa: Dict[str, str] = {}   # symbol -> index SSA value
        self.index_consts: Dict[int, str] = {}
        self.float_consts: Dict[Tuple[str, str], str] = {}
        self.counter = 0

    # ---- small helpers ----
    def fresh(self, stem: str) -> str:
        self.counter += 1
        return f"%{stem}{self.counter}"

    def emit(self, line: str):
        self.lines.append("    " + line)

    def index_const(self, v: int) -> str:
        if v not in self.index_consts:
            name = f"%c{v}"
            self.index_consts[v] = name
            self.emit(f"{name} = arith.constant {v} : index")
        return self.index_consts[v]

    def float_const(self, v: float, elem: str) -> str:
        key = (_float_literal(v), elem)
        if key not in self.float_consts:
            name = self.fresh("cst")
            self.float_consts[key] = name
            self.emit(f"{name} = arith.constant {key[0]} : {elem}")
        return self.float_consts[key]

    def map_alias(self, rank: int, results: Sequence[Union[int, None]]) -> str:
        dims = ", ".join(f"d{i}" for i in range(rank))
        res = ", ".join("0" if r is None else f"d{r}" for r in results)
        text = f"affine_map<({dims}) -> ({res})>"
        if text not in self.maps:
            self.maps[text] = f"#map{len(self.maps)}"
        return self.maps[text]

    def bind_dims(self, t: _Tensor):
        """Read the dynamic extents of a function argument once, the first time a symbol is seen."""
        for axis, s in enumerate(t.base):
            if isinstance(s, str) and s not in self.dim_ssa:
                name = f"%dim_{s}"
                self.emit(f"{name} = tensor.dim {t.ssa}, {self.index_const(axis)} : {t.type}")
                self.dim_ssa[s] = name

    def empty(self, sizes: Sequence[Size], elem: str) -> str:
        name = self.fresh("e")
        dyn = ", ".join(self.dim_ssa[s] for s in sizes if isinstance(s, str))
        self.emit(f"{name} = tensor.empty({dyn}) : {_tensor_type(sizes, elem)}")
        return name

    # ---- structured ops ----
    def elementwise(self, operands: Sequence[_Tensor], body) -> _Tensor:
        """One all-parallel generic over the broadcast of the operands' shapes; `body(args) -> (lines, result)`."""
        elem = operands[0].elem
        if any(o.elem != elem for o in operands):
            raise UnsupportedTorchOp("mixed element types in one elementwise op: " + ", ".join(o.elem for o in operands))
        rank = max(len(o.view) for o in operands)
        out: List[Size] = [1] * rank
        for o in operands:
            off = rank - len(o.view)
            for p, s in enumerate(o.shape):
                if s != 1:
                    if out[off + p] not in (1, s):
                        raise UnsupportedTorchOp(f"cannot broadcast extents {out[off + p]} and {s}")
                    out[off + p] = s
        maps = []
        for o in operands:
            off = rank - len(o.view)
            res: List[Optional[int]] = []
            for axis in range(len(o.base)):
                p = o.view.index(axis)
                res.append(None if (o.base[axis] == 1 and out[off + p] != 1) else off + p)
            maps.append(self.map_alias(rank, res))
        maps.append(self.map_alias(rank, list(range(rank))))
        dest = self.empty(out, elem)
        result = self.fresh("v")
        args = [f"%in{i}" for i in range(len(operands))]
        lines, yielded = body(args)
        iters = ", ".join('"parallel"' for _ in range(rank))
        out_type = _tensor_type(out, elem)
        self.emit(f"{result} = linalg.generic {{indexing_maps = [{', '.join(maps)}], iterator_types = [{iters}]}}")
        self.emit(f"    ins({', '.join(o.ssa for o in operands)} : {', '.join(o.type for o in operands)}) outs({dest} : {out_type}) {{")
        self.emit("^bb0(" + ", ".join(f"{a}: {elem}" for a in args) + f", %out: {elem}):")
        for l in lines:
            self.emit("  " + l)
        self.emit(f"  linalg.yield {yielded} : {elem}")
        self.emit(f"}} -> {out_type}")
        return _Tensor(result, elem, out)

    def binary(self, arith: str, a: Any, b: Any) -> _Tensor:
        tensors = [x for x in (a, b) if isinstance(x, _Tensor)]
        if not tensors:
            raise UnsupportedTorchOp(f"{arith} of two scalars")
        elem = tensors[0].elem

        def body(args):
            it = iter(args)
            lhs = next(it) if isinstance(a, _Tensor) else self.float_const(a, elem)
            rhs = next(it) if isinstance(b, _Tensor) else self.float_const(b, elem)
            return [f"%r = arith.{arith} {lhs}, {rhs} : {elem}"], "%r"

        # constants are function-level values: create them before the generic that uses them
        for x in (a, b):
            if not isinstance(x, _Tensor):
                self.float_const(x, elem)
        return self.elementwise(tensors, body)

    def leaky_relu(self, x: _Tensor, slope: float) -> _Tensor:
        alpha = self.float_const(slope, x.elem)
        return self.elementwise([x], lambda args: ([f"%s = arith.mulf {args[0]}, {alpha} : {x.elem}",
                                                    f"%r = arith.maximumf {args[0]}, %s : {x.elem}"], "%r"))

    def row_sum(self, x: _Tensor) -> _Tensor:
        """Sum over the last dimension of a rank-2 value, accumulating from zero."""
        x = self.materialise(x)
        if len(x.base) != 2:
            raise UnsupportedTorchOp(f"sum over the last dimension needs a rank-2 operand, got rank {len(x.base)}")
        zero = self.float_const(0.0, x.elem)
        out_sizes = [x.base[0]]
        dest = self.empty(out_sizes, x.elem)
        out_type = _tensor_type(out_sizes, x.elem)
        init = self.fresh("init")
        self.emit(f"{init} = linalg.fill ins({zero} : {x.elem}) outs({dest} : {out_type}) -> {out_type}")
        result = self.fresh("sum")
        self.emit(f"{result} = linalg.generic {{indexing_maps = [{self.map_alias(2, [0, 1])}, {self.map_alias(2, [0])}], "
                  f'iterator_types = ["parallel", "reduction"]}}')
        self.emit(f"    ins({x.ssa} : {x.type}) outs({init} : {out_type}) {{")
        self.emit(f"^bb0(%in0: {x.elem}, %acc: {x.elem}):")
        self.emit(f"  %r = arith.addf %acc, %in0 : {x.elem}")
        self.emit(f"  linalg.yield %r : {x.elem}")
        self.emit(f"}} -> {out_type}")
        return _Tensor(result, x.elem, out_sizes)

    def matmul(self, a: _Tensor, b: _Tensor, bias: Optional[_Tensor] = None) -> _Tensor:
        """A . B accumulated in f32, optional bias[n] added in f32, rounded once to the operands' type."""
        # B read through a transpose (x @ w.t(), torch.nn.Linear) stays where it is: linalg.matmul_transpose_b takes
        # it as [N, K], and the kernel loads K-major tiles of it
        trans_b = len(b.base) == 2 and b.view == [1, 0]
        a = self.materialise(a)
        if not trans_b:
            b = self.materialise(b)
        if len(a.base) != 2 or len(b.base) != 2 or a.elem != b.elem:
            raise UnsupportedTorchOp("matmul needs two rank-2 operands of one element type")
        k_of_b, n_of_b = (b.base[1], b.base[0]) if trans_b else (b.base[0], b.base[1])
        if a.base[1] != k_of_b:
            raise UnsupportedTorchOp(f"matmul inner extents differ: {a.base[1]} and {k_of_b}")
        sizes = [a.base[0], n_of_b]
        b_type = _tensor_type(b.base, b.elem)
        acc_type = _tensor_type(sizes, "f32")
        zero = self.float_const(0.0, "f32")
        acc0 = self.empty(sizes, "f32")
        init = self.fresh("init")
        self.emit(f"{init} = linalg.fill ins({zero} : f32) outs({acc0} : {acc_type}) -> {acc_type}")
        prod = self.fresh("mm")
        op = "linalg.matmul_transpose_b" if trans_b else "linalg.matmul"
        self.emit(f"{prod} = {op} ins({a.ssa}, {b.ssa} : {a.type}, {b_type}) outs({init} : {acc_type}) -> {acc_type}")
        if a.elem == "f32" and bias is None:
            return _Tensor(prod, "f32", sizes)
        # epilogue generic: (+ bias) in f32, then the result type
        elem = a.elem
        out_type = _tensor_type(sizes, elem)
        dest = self.empty(sizes, elem)
        result = self.fresh("v")
        ins, types, maps, args = [prod], [acc_type], [self.map_alias(2, [0, 1])], ["%in0: f32"]
        lines, cur = [], "%in0"
        if bias is not None:
            bias = self.materialise(bias)
            if len(bias.base) != 1 or bias.base[0] != sizes[1]:
                raise UnsupportedTorchOp("addmm bias must be a vector of the output's column count")
            ins.append(bias.ssa)
            types.append(bias.type)
            maps.append(self.map_alias(2, [1]))
            args.append(f"%in1: {bias.elem}")
            bias_val = "%in1"
            if bias.elem != "f32":
                lines.append(f"%bf = arith.extf %in1 : {bias.elem} to f32")
                bias_val = "%bf"
            lines.append(f"%x = arith.addf {cur}, {bias_val} : f32")
            cur = "%x"
        if elem != "f32":
            lines.append(f"%t = arith.truncf {cur} : f32 to {elem}")
            cur = "%t"
        maps.append(self.map_alias(2, [0, 1]))
        self.emit(f"{result} = linalg.generic {{indexing_maps = [{', '.join(maps)}], iterator_types = [\"parallel\", \"parallel\"]}}")
        self.emit(f"    ins({', '.join(ins)} : {', '.join(types)}) outs({dest} : {out_type}) {{")
        self.emit("^bb0(" + ", ".join(args) + f", %out: {elem}):")
        for l in lines:
            self.emit("  " + l)
        self.emit(f"  linalg.yield {cur} : {elem}")
        self.emit(f"}} -> {out_type}")
        return _Tensor(result, elem, sizes)

    def materialise(self, t: _Tensor) -> _Tensor:
        """Structured ops other than elementwise ones need the value itself, not a view of it."""
        if t.view == list(range(len(t.base))):
            return t
        if any(v is None for v in t.view):
            raise UnsupportedTorchOp("a view with inserted unit dimensions feeds an op that needs a materialised tensor")
        # a permutation: one copy generic that reads the value through the permuted map (a bare permutation group)
        return self.elementwise([t], lambda args: ([], args[0]))


# ---------------------------------------------------------------------------------------------------------
# ATen graph walk
# ---------------------------------------------------------------------------------------------------------

_BINARY = {"add": "addf", "sub": "subf", "mul": "mulf", "div": "divf", "maximum": "maximumf", "minimum": "minimumf"}


def _size_of(s: Any) -> Size:
    if isinstance(s, int):
        return s
    text = str(s)
    if not text.isidentifier():
        raise UnsupportedTorchOp(f"derived dynamic extent '{text}' (only plain symbols are supported)")
    return text


def _scalar(x: Any) -> float:
    if isinstance(x, (int, float)) and not isinstance(x, bool):
        return float(x)
    raise UnsupportedTorchOp(f"operand {x!r} is neither a tensor nor a number")


def _lower_node(em: _Emitter, node, env: Dict[str, _Tensor]) -> _Tensor:
    aten = torch.ops.aten
    target = node.target
    name = getattr(target, "__name__", str(target))
    stem = name.split(".")[0]

    def arg(i, default=None):
        if i < len(node.args):
            a = node.args[i]
        else:
            return default
        return env[a.name] if isinstance(a, torch.fx.Node) else a

    def operand(i):
        a = arg(i)
        return a if isinstance(a, _Tensor) else _scalar(a)

    if stem in _BINARY and target in (aten.add.Tensor, aten.sub.Tensor, aten.mul.Tensor, aten.div.Tensor,
                                      aten.maximum.default, aten.minimum.default, aten.add.Scalar, aten.sub.Scalar,
                                      aten.mul.Scalar, aten.div.Scalar):
        a, b = operand(0), operand(1)
        alpha = node.kwargs.get("alpha", 1)
        if alpha != 1:
            raise UnsupportedTorchOp(f"{name} with alpha={alpha}")
        if target in (aten.div.Tensor, aten.div.Scalar) and node.kwargs.get("rounding_mode") is not None:
            raise UnsupportedTorchOp("div with a rounding mode")
        return em.binary(_BINARY[stem], a, b)
    if target == aten.relu.default:
        return em.binary("maximumf", operand(0), 0.0)
    if target == aten.neg.default:
        return em.binary("subf", 0.0, operand(0))
    if target == aten.abs.default:
        x = operand(0)
        return em.binary("maximumf", x, em.binary("subf", 0.0, x))
    if target in (aten.clamp_min.default, aten.clamp_max.default, aten.clamp.default):
        x = operand(0)
        lo = arg(1) if target != aten.clamp_max.default else None
        hi = arg(1) if target == aten.clamp_max.default else (arg(2) if target == aten.clamp.default else None)
        if isinstance(lo, _Tensor) or isinstance(hi, _Tensor):
            raise UnsupportedTorchOp("clamp with tensor bounds")
        if lo is not None:
            x = em.binary("maximumf", x, _scalar(lo))
        if hi is not None:
            x = em.binary("minimumf", x, _scalar(hi))
        return x
    if target in (aten.t.default, aten.transpose.int, aten.permute.default):
        x = arg(0)
        rank = len(x.view)
        if target == aten.t.default:
            perm = [1, 0] if rank == 2 else list(range(rank))
        elif target == aten.transpose.int:
            d0, d1 = (int(arg(1)) % rank, int(arg(2)) % rank)
            perm = list(range(rank))
            perm[d0], perm[d1] = perm[d1], perm[d0]
        else:
            perm = [int(d) % rank for d in arg(1)]
        if sorted(perm) != list(range(rank)):
            raise UnsupportedTorchOp(f"{name} with dims {perm}")
        return _Tensor(x.ssa, x.elem, x.base, [x.view[d] for d in perm])
    if target in (aten.contiguous.default, aten.clone.default):
        x = arg(0)
        return x if x.view == list(range(len(x.base))) else em.materialise(x)
    if target == aten.leaky_relu.default:
        return em.leaky_relu(arg(0), float(arg(1, 0.01)))
    if target == aten.unsqueeze.default:
        x, dim = arg(0), int(arg(1))
        rank = len(x.view) + 1
        dim = dim + rank if dim < 0 else dim
        view = list(x.view)
        view.insert(dim, None)
        return _Tensor(x.ssa, x.elem, x.base, view)
    if target in (aten.squeeze.dim, aten.squeeze.dims):
        x, dims = arg(0), arg(1)
        dims = [dims] if isinstance(dims, int) else list(dims)
        dims = sorted(d + len(x.view) if d < 0 else d for d in dims)
        view = [v for p, v in enumerate(x.view) if not (p in dims and v is None)]
        if len(view) != len(x.view) - len(dims):
            raise UnsupportedTorchOp("squeeze of a dimension that is not a view-only unit dimension")
        return _Tensor(x.ssa, x.elem, x.base, view)
    if target == aten.sum.dim_IntList:
        x, dims = arg(0), list(arg(1))
        if arg(2, False) or node.kwargs.get("dtype") is not None:
            raise UnsupportedTorchOp("sum with keepdim or an explicit dtype")
        rank = len(x.view)
        if [d + rank if d < 0 else d for d in dims] != [rank - 1]:
            raise UnsupportedTorchOp(f"sum over dims {dims} (only the last dimension is supported)")
        return em.row_sum(x)
    if target in (aten.mm.default, aten.matmul.default):
        return em.matmul(arg(0), arg(1))
    if target == aten.linear.default:  # x @ w.t() + b with w kept as [N, K]
        w = arg(1)
        if len(w.view) != 2:
            raise UnsupportedTorchOp("linear needs a rank-2 weight")
        wt = _Tensor(w.ssa, w.elem, w.base, [w.view[1], w.view[0]])
        return em.matmul(arg(0), wt, bias=arg(2) if len(node.args) > 2 and node.args[2] is not None else None)
    if target == aten.addmm.default:
        if node.kwargs.get("beta", 1) != 1 or node.kwargs.get("alpha", 1) != 1:
            raise UnsupportedTorchOp("addmm with beta/alpha other than 1")
        return em.matmul(arg(1), arg(2), bias=arg(0))
    raise UnsupportedTorchOp(f"ATen op {name} (node '{node.name}') is outside the supported subset")


def torch_to_linalg(model: torch.nn.Module, inputs: Sequence[torch.Tensor], dynamic_shapes=None,
                    func_name: str = "forward") -> str:
    """MLIR text (linalg on tensors) of `model(*inputs)`; `dynamic_shapes` as torch.export takes it.

    Same call shape as the reference's torch_to_linalg (python/torch/torch2linalg/convert.py:12-38).  Models
    with parameters or buffers are refused by this entry point (pass them as inputs, or use
    torch_to_linalg_with_state, which appends them to the function's arguments).
    """
    text, state = torch_to_linalg_with_state(model, inputs, dynamic_shapes, func_name)
    if state:
        raise UnsupportedTorchOp(f"model state '{state[0][0]}' (parameters and buffers must be passed as inputs)")
    return text


def torch_to_linalg_with_state(model: torch.nn.Module, inputs: Sequence[torch.Tensor], dynamic_shapes=None,
                               func_name: str = "forward"):
    """(MLIR text, [(name, tensor), ...]): parameters and buffers of the model become function arguments AFTER the
    user inputs, in the order of the list; a caller passes `inputs + [t for _, t in state]`."""
    exported = torch.export.export(model.eval(), tuple(inputs), dynamic_shapes=dynamic_shapes)
    graph = exported.graph
    sig = exported.graph_signature
    user_inputs = {s.arg.name for s in sig.input_specs if s.kind.name == "USER_INPUT"}
    state_of = {}
    for spec in sig.input_specs:
        if spec.kind.name in ("PARAMETER", "BUFFER") and spec.target in exported.state_dict:
            state_of[spec.arg.name] = (spec.target, exported.state_dict[spec.target])
        elif spec.kind.name in ("BUFFER", "CONSTANT_TENSOR") and spec.target in exported.constants:
            state_of[spec.arg.name] = (spec.target, exported.constants[spec.target])
    em = _Emitter(func_name)
    env: Dict[str, _Tensor] = {}
    args: List[_Tensor] = []
    state: List = []
    result: Optional[_Tensor] = None
    body_nodes = []
    placeholders = [n for n in graph.nodes if n.op == "placeholder"]
    body_nodes = [n for n in graph.nodes if n.op != "placeholder"]
    for node in [n for n in placeholders if n.name in user_inputs] + [n for n in placeholders if n.name not in user_inputs]:
        if node.name not in user_inputs:
            if node.name not in state_of:
                raise UnsupportedTorchOp(f"graph input '{node.name}' is neither a user input nor a parameter, buffer or constant tensor")
            state.append((state_of[node.name][0], state_of[node.name][1].detach()))
        val = node.meta["val"]
        if val.dtype not in ELEM_TYPES:
            raise UnsupportedTorchOp(f"input '{node.name}' has unsupported dtype {val.dtype}")
        t = _Tensor(f"%arg{len(args)}", ELEM_TYPES[val.dtype], [_size_of(s) for s in val.shape])
        env[node.name] = t
        args.append(t)
    for t in args:
        em.bind_dims(t)
    for node in body_nodes:
        if node.op == "call_function":
            env[node.name] = _lower_node(em, node, env)
        elif node.op == "output":
            outs = node.args[0]
            outs = outs if isinstance(outs, (tuple, list)) else (outs,)
            if len(outs) != 1 or not isinstance(outs[0], torch.fx.Node):
                raise UnsupportedTorchOp("models must return exactly one tensor")
            result = env[outs[0].name]
        else:
            raise UnsupportedTorchOp(f"graph node kind '{node.op}'")
    if result is None:
        raise UnsupportedTorchOp("model has no output")
    if result.view != list(range(len(result.base))):
        result = em.materialise(result)  # a permuted output is written out by a copy group; unit-dim views are refused there
    sig_text = ", ".join(f"{t.ssa}: {t.type}" for t in args)
    head = [f"{alias} = {text}" for text, alias in em.maps.items()]
    text = "\n".join(head + ["module {", f"  func.func @{func_name}({sig_text}) -> {result.type} {{"] + em.lines +
                     [f"    return {result.ssa} : {result.type}", "  }", "}"]) + "\n"
    return text, state
