"""TEST INFRASTRUCTURE ONLY -- seeded inputs and oracle equations of the benchmark workloads.

Each workload is a synthetic, seeded stand-in with the shapes and value distributions the
benchmark configurations state; inputs are drawn in FP32 from a torch CPU generator and cast to
BF16.  The equations are written in the vocabulary of ``oracle.evaluator`` and therefore carry
the reference's precision rules (FP32 elementwise math, float64 matrix products, one rounding
at the store).
"""
import math

import torch

from . import evaluator as ev


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def _normal(shape, std, g, mean=0.0):
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std + mean).bfloat16()


def _uniform(shape, g):
    return (torch.rand(shape, generator=g, dtype=torch.float32) * 2 - 1).bfloat16()


# ---------------------------------------------------------------- GEMM + epilogue
def gemm_inputs(m, n, k, seed, distribution="normal"):
    """A[m,k], W[k,n], bias[n].  'uniform': all U(-1,1) (streamed example shape class);
    'normal': A~N(0,1), W~N(0,1/k), bias~N(0,0.1) (graph-replay configuration)."""
    g = _gen(seed)
    if distribution == "uniform":
        return _uniform((m, k), g), _uniform((k, n), g), _uniform((n,), g)
    return (_normal((m, k), 1.0, g), _normal((k, n), 1.0 / math.sqrt(k), g),
            _normal((n,), 0.1, g))


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


def dyadic_gemm_inputs(m, n, k):
    """The exactly-representable operand pattern of the reference's GEMM harness
    (src/emit/provider/cute/operator/gemm/tests/reference.cu:17-19): every product and FP32
    partial sum is exact, so any correct kernel must match bit for bit."""
    i = torch.arange(m * k, dtype=torch.int64)
    a = (((i * 13 + (i // k) * 7) % 17 - 8).float() / 8.0).reshape(m, k).bfloat16()
    j = torch.arange(k * n, dtype=torch.int64)
    b = (((j * 11 + (j // n) * 3) % 19 - 9).float() / 8.0).reshape(k, n).bfloat16()
    return a, b


# ---------------------------------------------------------------- row kernels
def rownorm_inputs(rows, cols, seed):
    g = _gen(seed)
    return _normal((rows, cols), 1.0, g), _normal((cols,), 0.02, g, mean=1.0)


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
def mla_inputs(batch, heads, seq, d_qk, seed):
    g = _gen(seed)
    return _normal((batch, heads, d_qk), 1.0, g), _normal((batch, seq, d_qk), 1.0, g)


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
def mlp_inputs(m, d_model, d_ff, seed):
    g = _gen(seed)
    return (_normal((m, d_model), 1.0, g), _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
            _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
            _normal((d_ff, d_model), 1.0 / math.sqrt(d_ff), g))


def mlp_oracle(x, w_gate, w_up, w_down, rows=None):
    """Y = (silu(X@Wg) * (X@Wu)) @ Wd with the hidden activation stored once in BF16."""
    xs = x if rows is None else x[rows]
    hidden = gated_oracle(xs, w_up, w_gate)
    env = {"H": hidden, "Wd": w_down}
    return ev.run(ev.op("matmul", ev.load("H"), ev.load("Wd")), env,
                  [xs.shape[0], w_down.shape[1]], "bf16")


def ffn_block_inputs(m, d_model, d_ff, seed):
    """attn, Wo, residual, gain, Wg, Wu, Wd for the decode-time feed-forward block."""
    g = _gen(seed)
    return {
        "attn": _normal((m, d_model), 1.0, g),
        "Wo": _normal((d_model, d_model), 1.0 / math.sqrt(d_model), g),
        "R": _normal((m, d_model), 1.0, g),
        "g": _normal((d_model,), 0.02, g, mean=1.0),
        "Wg": _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
        "Wu": _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
        "Wd": _normal((d_ff, d_model), 1.0 / math.sqrt(d_ff), g),
    }


def ffn_block_oracle(t, eps):
    """X1 = attn@Wo + R; Xn = rmsnorm(X1)*g; H = (Xn@Wu)*silu(Xn@Wg); Y = H@Wd + X1, every
    intermediate stored in BF16 as the plan declares (the block of the reference's
    tests/fixtures/ir/IR.v3.txt, whose own interpreter is not part of that repository)."""
    x1 = gemm_oracle(t["attn"], t["Wo"], t["R"], None, "matrix")
    xn = rmsnorm_oracle(x1, t["g"], eps)
    hidden = gated_oracle(xn, t["Wu"], t["Wg"])
    return gemm_oracle(hidden, t["Wd"], x1, None, "matrix")


def ffn_ir_inputs(m, d_model, d_ff, seed):
    g = _gen(seed)
    return {
        "attn": _normal((m, d_model), 1.0, g),
        "Wo": _normal((d_model, d_model), 1.0 / math.sqrt(d_model), g),
        "X": _normal((m, d_model), 1.0, g),
        "Wa": _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
        "Wb": _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
        "Wd": _normal((d_ff, d_model), 1.0 / math.sqrt(d_ff), g),
    }


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
