"""Seeded synthetic inputs of the benchmark configurations.

Each generator is a stand-in with the shapes and value distributions the configurations state:
values are drawn in FP32 from a torch CPU generator and cast to BF16, so a seed names the same
tensors on every machine.  The benchmark, the smoke run and the parity tests all draw their
inputs from here; nothing in this module computes a result.
"""
import math

import torch


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def _normal(shape, std, g, mean=0.0):
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std + mean).bfloat16()


def _uniform(shape, g):
    return (torch.rand(shape, generator=g, dtype=torch.float32) * 2 - 1).bfloat16()


def gemm_inputs(m, n, k, seed, distribution="normal"):
    """A[m,k], W[k,n], bias[n].  'uniform': all U(-1,1) (streamed example shape class);
    'normal': A~N(0,1), W~N(0,1/k), bias~N(0,0.1) (graph-replay configuration)."""
    g = _gen(seed)
    if distribution == "uniform":
        return _uniform((m, k), g), _uniform((k, n), g), _uniform((n,), g)
    return (_normal((m, k), 1.0, g), _normal((k, n), 1.0 / math.sqrt(k), g),
            _normal((n,), 0.1, g))


def dyadic_gemm_inputs(m, n, k):
    """The exactly-representable operand pattern of the reference's GEMM harness
    (src/emit/provider/cute/operator/gemm/tests/reference.cu:17-19): every product and FP32
    partial sum is exact, so any correct kernel must match bit for bit."""
    i = torch.arange(m * k, dtype=torch.int64)
    a = (((i * 13 + (i // k) * 7) % 17 - 8).float() / 8.0).reshape(m, k).bfloat16()
    j = torch.arange(k * n, dtype=torch.int64)
    b = (((j * 11 + (j // n) * 3) % 19 - 9).float() / 8.0).reshape(k, n).bfloat16()
    return a, b


def rownorm_inputs(rows, cols, seed):
    """X[rows, cols] ~ N(0,1) and a gain[cols] ~ N(1, 0.02)."""
    g = _gen(seed)
    return _normal((rows, cols), 1.0, g), _normal((cols,), 0.02, g, mean=1.0)


def mla_inputs(batch, heads, seq, d_qk, seed):
    """q[batch, heads, d_qk] and the compressed cache[batch, seq, d_qk], both ~ N(0,1)."""
    g = _gen(seed)
    return _normal((batch, heads, d_qk), 1.0, g), _normal((batch, seq, d_qk), 1.0, g)


def mlp_inputs(m, d_model, d_ff, seed):
    """X ~ N(0,1), W_gate and W_up ~ N(0, 1/d_model), W_down ~ N(0, 1/d_ff)."""
    g = _gen(seed)
    return (_normal((m, d_model), 1.0, g), _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
            _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
            _normal((d_ff, d_model), 1.0 / math.sqrt(d_ff), g))


def mlp_shard_on_device(rank, d_model, shard, d_ff, device, seed=1238):
    """Rank `rank`'s weight shards of the tensor-parallel MLP, drawn on `device` (the full
    weights of the benchmark configuration are 1.4 GB, so every rank draws only its own part).
    The same (seed, rank, device type) yields the same shards in every process."""
    g = torch.Generator(device=device)
    g.manual_seed(seed + rank)

    def normal(shape, std):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).bfloat16()

    return (normal((d_model, shard), 1.0 / math.sqrt(d_model)),
            normal((d_model, shard), 1.0 / math.sqrt(d_model)),
            normal((shard, d_model), 1.0 / math.sqrt(d_ff)))


def mlp_activations_on_device(m, d_model, device, seed=1238):
    """The replicated X[m, d_model] ~ N(0,1) of the tensor-parallel MLP, drawn on `device`."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn((m, d_model), generator=g, device=device).bfloat16()


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


def ffn_ir_inputs(m, d_model, d_ff, seed):
    """Inputs of the feed-forward block in the loop-IR fixture's spelling."""
    g = _gen(seed)
    return {
        "attn": _normal((m, d_model), 1.0, g),
        "Wo": _normal((d_model, d_model), 1.0 / math.sqrt(d_model), g),
        "X": _normal((m, d_model), 1.0, g),
        "Wa": _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
        "Wb": _normal((d_model, d_ff), 1.0 / math.sqrt(d_model), g),
        "Wd": _normal((d_ff, d_model), 1.0 / math.sqrt(d_ff), g),
    }
