"""TEST INFRASTRUCTURE ONLY -- oracle equations of the benchmark workloads.

The equations are written in the vocabulary of ``oracle.evaluator`` and therefore carry the
reference's precision rules (FP32 elementwise math, float64 matrix products, one rounding at
the store).  The seeded input generators live in ``trinity_lowering.synthetic`` (the product
and the benchmark draw from there without touching this package); they are re-exported here so
a parity test names inputs and expected results through one module.
"""
import torch

from trinity_lowering.synthetic import (_gen, _normal, dyadic_gemm_inputs, ffn_block_inputs, ffn_ir_inputs,  # noqa: F401
                                        gemm_inputs, mla_inputs, mlp_inputs, rownorm_inputs)

from . import evaluator as ev


# ---------------------------------------------------------------- GEMM + epilogue
def gemm_equation(activation=None, bias="col"):
    """act(A @ W + bcast(bias)) over value ids 'A', 'W', 'bias'."""
    e = ev.op("matmul", ev.load("A"), ev.load("W"))
    if bias == "col":
        e = ev.op("add", e, ev.op("unsqueeze", ev.load("bias"), axis=0))
    elif bias == "row":
        e = ev.op("add", e, ev.op("unsqueeze", ev.load("bias"), axis=1))
    elif bias == "matrix":
        e = ev.op("add", e, ev.load("bias"))
    if activation == "relu":
        e = ev.op("relu", e)
    elif activation == "silu":
        e = ev.op("mul", e, ev.op("sigmoid", e))
    return e


def gemm_oracle(a, w, bias, activation=None, bias_mode="col", out_dtype="bf16", rows=None):
    """Oracle result for all rows, or only for the row indices in ``rows``."""
    env = {"A": a if rows is None else a[rows], "W": w, "bias": bias}
    if bias is not None and bias_mode in ("row", "matrix") and rows is not None:
        env["bias"] = bias[rows]
    shape = [env["A"].shape[0], w.shape[1]]
    return ev.run(gemm_equation(activation, bias_mode if bias is not None else None), env, shape,
                  out_dtype)


def gated_equation():
    """(A @ Wu) * ((A @ Wg) * sigmoid(A @ Wg)): the reference FFN's SwiGLU form."""
    up = ev.op("matmul", ev.load("A"), ev.load("Wu"))
    gate = ev.op("matmul", ev.load("A"), ev.load("Wg"))
    return ev.op("mul", up, ev.op("mul", gate, ev.op("sigmoid", gate)))


def gated_oracle(a, w_up, w_gate, rows=None):
    env = {"A": a if rows is None else a[rows], "Wu": w_up, "Wg": w_gate}
    return ev.run(gated_equation(), env, [env["A"].shape[0], w_up.shape[1]], "bf16")


# ---------------------------------------------------------------- row kernels
def rmsnorm_equation(cols, eps, gain=True):
    x = ev.load("X")
    mean = ev.op("div", ev.op("sum", ev.op("sqr", x), axis=1), ev.const(float(cols)))
    if eps != 0.0:
        mean = ev.op("add", mean, ev.const(float(eps)))
    e = ev.op("div", x, ev.op("unsqueeze", ev.op("sqrt", mean), axis=1))
    if gain:
        e = ev.op("mul", e, ev.op("unsqueeze", ev.load("g"), axis=0))
    return e


def rmsnorm_oracle(x, gain, eps):
    env = {"X": x, "g": gain}
    return ev.run(rmsnorm_equation(x.shape[1], eps, gain is not None), env, list(x.shape), "bf16")


def softmax_equation():
    x = ev.load("X")
    shifted = ev.op("sub", x, ev.op("unsqueeze", ev.op("max_reduce", x, axis=1), axis=1))
    e = ev.op("exp", shifted)
    return ev.op("div", e, ev.op("unsqueeze", ev.op("sum", e, axis=1), axis=1))


def softmax_oracle(x):
    return ev.run(softmax_equation(), {"X": x}, list(x.shape), "bf16")


# ---------------------------------------------------------------- MLA decode
def mla_oracle(q, cache, scale, d_v, batches=None):
    """softmax_s(scale * q.cache^T) @ cache[..., :d_v] per batch, with the evaluator's rules:
    float64 matrix products narrowed to FP32, FP32 softmax, one BF16 rounding of the output.
    Scores follow the reference fixture's E = exp(S) / sum form
    (tests/fixtures/batched_mla/batched_mla_postprocessed_stage14.txt:62-68) with the scale and
    maximum subtraction the decode configuration adds."""
    outs = []
    for b in (range(q.shape[0]) if batches is None else batches):
        env = {"Q": q[b], "Kt": cache[b].t().contiguous(), "V": cache[b][:, :d_v].contiguous()}
        s = ev.op("mul", ev.op("matmul", ev.load("Q"), ev.load("Kt")), ev.const(float(scale)))
        shifted = ev.op("sub", s, ev.op("unsqueeze", ev.op("max_reduce", s, axis=1), axis=1))
        e = ev.op("exp", shifted)
        p = ev.op("div", e, ev.op("unsqueeze", ev.op("sum", e, axis=1), axis=1))
        o = ev.op("matmul", p, ev.load("V"))
        outs.append(ev.run(o, env, [q.shape[1], d_v], "bf16"))
    return torch.stack(outs)


# ---------------------------------------------------------------- TP MLP
def mlp_oracle(x, w_gate, w_up, w_down, rows=None):
    """Y = (silu(X@Wg) * (X@Wu)) @ Wd with the hidden activation stored once in BF16."""
    xs = x if rows is None else x[rows]
    hidden = gated_oracle(xs, w_up, w_gate)
    env = {"H": hidden, "Wd": w_down}
    return ev.run(ev.op("matmul", ev.load("H"), ev.load("Wd")), env,
                  [xs.shape[0], w_down.shape[1]], "bf16")


def ffn_block_oracle(t, eps):
    """X1 = attn@Wo + R; Xn = rmsnorm(X1)*g; H = (Xn@Wu)*silu(Xn@Wg); Y = H@Wd + X1, every
    intermediate stored in BF16 as the plan declares (the block of the reference's
    tests/fixtures/ir/IR.v3.txt, whose own interpreter is not part of that repository)."""
    x1 = gemm_oracle(t["attn"], t["Wo"], t["R"], None, "matrix")
    xn = rmsnorm_oracle(x1, t["g"], eps)
    hidden = gated_oracle(xn, t["Wu"], t["Wg"])
    return gemm_oracle(hidden, t["Wd"], x1, None, "matrix")


def ffn_ir_oracle(t):
    """The feed-forward block in the spelling of the reference's loop-IR fixture
    (tests/fixtures/ir/IR.v3.txt:1-131 there): every named tensor is stored in BF16, the row sums
    of squares in FP32, the normalisation has neither eps nor gain, SwiGLU is four separate
    steps.  FP32 elementwise math, float64 products narrowed once, as the reference evaluator."""
    d_model = t["attn"].shape[1]
    bf = torch.bfloat16
    p = gemm_oracle(t["attn"], t["Wo"], None)
    q = (p.float() + t["X"].float()).to(bf)
    s = q.float().square().sum(dim=1, keepdim=True)
    n = (q.float() / torch.sqrt(s / float(d_model))).to(bf)
    a = gemm_oracle(n, t["Wa"], None)
    b = gemm_oracle(n, t["Wb"], None)
    sw = (b.float() * torch.sigmoid(b.float())).to(bf)
    h = (a.float() * sw.float()).to(bf)
    return gemm_oracle(h, t["Wd"], None)
