"""TEST INFRASTRUCTURE ONLY -- CPU oracle for the native provider path.

A restatement, in this project's own words, of how the reference evaluates a plan equation on
the CPU with PyTorch (youngchan2/Trinity-BE, src/emit/wrapper/reference.py:9-79):

* every elementwise operator computes in FP32 (operands are widened with ``.float()``),
* a matrix product is taken in float64 and narrowed to FP32 once (reference.py:37-39),
* rounding to a storage type happens only where a value is *stored*: each step of a ``stores``
  sequence writes its FP32 result into a buffer of the declared dtype, unless the value lives
  in a register, in which case it stays FP32 (reference.py:11-23),
* constants stay Python scalars until an operator needs a tensor.

Nothing outside ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
reference legs may import this module; the product path never does.

Pinned by ``tests/golden/*.pt``: outputs of the reference's own evaluator (imported from the
mounted reference tree by ``tests/golden/make_golden.py``) on seeded inputs.
"""
import torch

DTYPES = {"fp16": torch.float16, "float16": torch.float16, "bf16": torch.bfloat16,
          "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32}


def _tensor(x):
    return torch.as_tensor(x, dtype=torch.float32)


def _strided(base, view, extra_offset=0):
    return base.as_strided(view["shape"], view["strides"], extra_offset + view["offset"])


def evaluate(node, env):
    """Evaluates one equation node against ``env`` (value id -> tensor)."""
    kind = node["op"]
    if kind == "stores":                                     # reference.py:11-23
        scope = dict(env)
        last = None
        for step in node["steps"]:
            last = evaluate(step["expression"], scope)
            kept = torch.float32 if step["register"] else DTYPES[step["dtype"]]
            buffer = torch.empty(step["shape"], dtype=kept, device=last.device)
            _strided(buffer, step["output"]).copy_(last)
            scope[step["output"]["value"]] = buffer
        return last.reshape(node["shape"])
    if kind == "view":                                       # reference.py:24-28
        base = env[node["view"]["value"]]
        return _strided(base, node["view"], base.storage_offset()).float()
    if kind == "load":                                       # reference.py:29-33
        value = env[node["value"]]
        if node.get("view_shape") is not None:
            value = value.view(node["view_shape"])
        return value.float()
    if kind == "constant":                                   # reference.py:34-35
        return node["value"]
    args = [evaluate(child, env) for child in node["args"]]
    if kind == "matmul":                                     # reference.py:37-39
        return (args[0].double() @ args[1].double()).float()
    if kind == "concat":
        return torch.cat(args, dim=node["axis"])
    if kind == "add":
        return args[0] + args[1]
    if kind == "sub":
        return args[0] - args[1]
    if kind == "mul":
        return args[0] * args[1]
    if kind == "div":
        return args[0] / args[1]
    if kind == "sqr":
        return args[0] * args[0]
    if kind == "sqrt":
        return torch.sqrt(_tensor(args[0]))
    if kind == "sigmoid":
        return torch.sigmoid(_tensor(args[0]))
    if kind == "relu":
        return torch.clamp_min(_tensor(args[0]), 0)
    if kind == "sum":
        return args[0].sum(dim=node["axis"])
    if kind == "unsqueeze":
        return args[0].unsqueeze(node["axis"])
    if kind == "squeeze":
        return args[0].squeeze(node["axis"])
    if kind == "max_reduce":
        return args[0].amax(dim=node["axis"])
    if kind == "min_reduce":
        return args[0].amin(dim=node["axis"])
    if kind in ("exp", "erf", "abs"):
        return getattr(torch, kind)(args[0])
    if kind in ("maximum", "minimum"):
        left = torch.as_tensor(args[0])
        return getattr(torch, kind)(left, torch.as_tensor(args[1], device=left.device))
    if kind == "cast":
        return args[0].to(DTYPES[node["dtype"].lstrip("?")]).float()
    raise ValueError(f"unknown equation operator: {kind}")


# ---------------------------------------------------------------- equation builders
def load(value):
    return {"op": "load", "value": value}


def const(value):
    return {"op": "constant", "value": value}


def op(kind, *args, **attrs):
    return {"op": kind, "args": list(args), **attrs}


def store_root(expression, shape, dtype, value="out"):
    """A single-step ``stores`` node: evaluate in FP32, round once to the storage dtype."""
    strides = []
    pitch = 1
    for extent in reversed(shape):
        strides.insert(0, pitch)
        pitch *= extent
    return {"op": "stores", "shape": list(shape), "steps": [{
        "expression": expression, "register": False, "dtype": dtype, "shape": list(shape),
        "output": {"value": value, "shape": list(shape), "strides": strides, "offset": 0}}]}


def run(equation, env, shape, dtype):
    """Evaluates ``equation`` and returns the stored (rounded) result tensor."""
    root = store_root(equation, shape, dtype)
    scope = dict(env)
    result = evaluate(root, scope)
    return result.to(DTYPES[dtype])
