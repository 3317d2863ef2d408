"""The public path on a B200: plan -> emit -> compile -> load -> prepare -> run / Graph, on
PyTorch tensors and streams, checked against the CPU oracle.  Scenarios follow the reference's
GPU tests (python/tests/test_gpu.py, test_tensor_ops.py, test_cuda_runtime.py)."""
import math
import threading

import pytest
import torch

import trinity_lowering as tl
from oracle import workloads as wl
from parity import assert_close_bf16
from trinity_lowering import plans

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build(plan):
    artifact = tl.compile(tl.emit(plan))
    module = tl.load(artifact, DEV)
    artifact.close()   # the loader owns a private copy of the library
    return module


@torch.inference_mode()
def test_streamed_gemm_bias_on_side_streams_with_allocator_pressure():
    m = n = k = 1024
    module = build(plans.gemm_bias(m, n, k))
    a, w, bias = wl.gemm_inputs(m, n, k, 1234, "uniform")
    producer, runner, consumer = [torch.cuda.Stream(device=module.device) for _ in range(3)]
    with torch.cuda.stream(producer):
        ad, wd, bd = a.to(DEV, non_blocking=True), w.to(DEV, non_blocking=True), bias.to(DEV, non_blocking=True)
        produced = producer.record_event()
    execution = module.prepare({"A": ad, "W": wd, "bias": bd})
    with pytest.raises(tl.ResourceBusy):
        module.close()
    with torch.cuda.stream(runner):
        execution.run(wait_for=[produced])
        first = execution.output.clone()
        for _ in range(16):
            execution.run()
        done = runner.record_event()
    with torch.cuda.stream(consumer):
        consumer.wait_event(done)
        copy = first.clone()
        _pressure = [torch.empty(m, n, device=DEV, dtype=torch.bfloat16) for _ in range(64)]
    execution.wait(timeout=30)
    consumer.synchronize()
    expected = wl.gemm_oracle(a, w, bias)
    assert_close_bf16(copy.cpu(), expected, max_ulp=1)
    torch.testing.assert_close(copy.cpu().float(), expected.float(), atol=0.125, rtol=0.02)
    execution.run(stream=consumer)
    execution.wait(timeout=30)
    execution.close()
    module.close()


@torch.inference_mode()
def test_graph_capture_and_replay_of_gemm_bias_relu():
    m = n = k = 2048
    module = build(plans.gemm_bias(m, n, k, "relu"))
    io = module.allocate_io()
    a, w, bias = wl.gemm_inputs(m, n, k, 1235, "normal")
    io.inputs["A"].copy_(a)
    io.inputs["W"].copy_(w)
    io.inputs["bias"].copy_(bias)
    execution = module.prepare(io.inputs, out=io.output)
    stream = torch.cuda.Stream(device=module.device)
    stream.wait_stream(torch.cuda.current_stream(module.device))
    graph = tl.Graph.capture(execution.run, executions=[execution], stream=stream)
    with pytest.raises(tl.ResourceBusy):
        execution.close()
    with pytest.raises(tl.ResourceBusy):
        execution.run(stream=stream)
    with torch.cuda.stream(stream):
        for _ in range(10):
            graph.replay()
        snapshot = graph.output.clone()
    graph.wait(timeout=30)
    rows = torch.arange(0, m, 29)
    assert_close_bf16(snapshot.cpu()[rows], wl.gemm_oracle(a, w, bias, "relu", rows=rows), max_ulp=1, max_abs=2e-2)
    # inputs change, replay sees the new values (static addresses)
    io.inputs["bias"].zero_()
    with torch.cuda.stream(stream):
        graph.replay()
    graph.wait(timeout=30)
    assert_close_bf16(graph.output.cpu()[rows], wl.gemm_oracle(a, w, torch.zeros_like(bias), "relu", rows=rows),
                      max_ulp=1, max_abs=2e-2)
    # dropping a Graph from another thread keeps pending native state alive
    with torch.cuda.stream(stream):
        graph.replay()
    holder = [graph]
    del graph
    thread = threading.Thread(target=holder.clear)
    thread.start()
    thread.join()
    stream.synchronize()
    tl.runtime.native().collect_local()
    execution.close()
    module.close()


@torch.inference_mode()
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 128, 320), (256, 256, 192)])
def test_reference_example_plan_three_statements(m, n, k):
    """GEMM into a BF16 global, [M,N] bias add, ReLU: three launches; tolerance and reference
    expression of python/tests/test_gpu.py:27,55,88-91."""
    module = build(plans.reference_gemm(m, n, k, relu=True))
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(k, n, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    execution = module.prepare({"X": x, "W": w, "bias": bias})
    out = execution.run()
    execution.wait(30)
    reference = torch.relu((x.float() @ w.float()).bfloat16() + bias)
    torch.testing.assert_close(out, reference, atol=0.125, rtol=0.02)
    execution.close()
    module.close()


@torch.inference_mode()
def test_storage_replacement_is_detected():
    module = build(plans.softmax(8, 256))
    x = torch.randn(8, 256, device=DEV, dtype=torch.bfloat16)
    execution = module.prepare({"X": x})
    execution.run()
    execution.wait(30)
    x.set_(torch.randn(8, 256, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="storage"):
        execution.run()
    execution.close()
    module.close()


@torch.inference_mode()
def test_binding_validation():
    module = build(plans.softmax(8, 256))
    good = torch.zeros(8, 256, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="expected exactly input names"):
        module.prepare({})
    with pytest.raises(ValueError, match="mismatch"):
        module.prepare({"X": good.float()})
    with pytest.raises(ValueError, match="mismatch"):
        module.prepare({"X": torch.zeros(8, 512, device=DEV, dtype=torch.bfloat16)[:, ::2]})
    with pytest.raises(TypeError):
        module.prepare({"X": 3})
    with pytest.raises(ValueError, match="overlap"):
        module.prepare({"X": good}, out=good)
    module.close()


@torch.inference_mode()
def test_fused_row_regions_and_mla_through_plans():
    x, g = wl.rownorm_inputs(64, 4096, 5)
    for eps, gain in ((1e-6, True), (0.0, False)):
        module = build(plans.rmsnorm(64, 4096, eps, gain))
        inputs = {"X": x.to(DEV)}
        if gain:
            inputs["g"] = g.to(DEV)
        execution = module.prepare(inputs)
        out = execution.run().clone()
        execution.wait(30)
        assert_close_bf16(out.cpu(), wl.rmsnorm_oracle(x, g if gain else None, eps), max_ulp=1)
        execution.close()
        module.close()
    module = build(plans.softmax(64, 4096))
    execution = module.prepare({"X": x.to(DEV)})
    out = execution.run().clone()
    execution.wait(30)
    assert_close_bf16(out.cpu(), wl.softmax_oracle(x), max_ulp=1)
    execution.close()
    module.close()
    q, cache = wl.mla_inputs(2, 128, 512, 576, 6)
    scale = 1.0 / math.sqrt(192.0)
    module = build(plans.mla_decode(2, 128, 512, scale=scale))
    execution = module.prepare({"q": q.to(DEV), "cache": cache.to(DEV)})
    out = execution.run().clone()
    execution.wait(30)
    assert_close_bf16(out.cpu(), wl.mla_oracle(q, cache, scale, 512), max_ulp=None, max_abs=2e-2)
    execution.close()
    module.close()


@torch.inference_mode()
def test_gated_gemm_plan():
    a, wg, wu, _ = wl.mlp_inputs(256, 512, 384, 11)
    module = build(plans.gated_gemm(256, 384, 512))
    execution = module.prepare({"A": a.to(DEV), "Wg": wg.to(DEV), "Wu": wu.to(DEV)})
    out = execution.run().clone()
    execution.wait(30)
    assert_close_bf16(out.cpu(), wl.gated_oracle(a, wu, wg), max_ulp=1)
    execution.close()
    module.close()


@torch.inference_mode()
@pytest.mark.parametrize("m,d_model,d_ff", [(16, 512, 1024), (200, 1024, 2816)])
def test_ffn_block_plan(m, d_model, d_ff):
    """Output projection + residual, RMSNorm, SwiGLU, down projection + residual as one plan of
    four launches with BF16 intermediates (decode-time M = 16: one partly filled row tile).
    Each stage is within one ulp of its own oracle, but a one-ulp difference in an
    intermediate is amplified by the next product, so the chain is held to the path's
    rel-L2 / max-abs bar."""
    tensors = wl.ffn_block_inputs(m, d_model, d_ff, 31)
    module = build(plans.ffn_block(m, d_model, d_ff, 1e-6))
    execution = module.prepare({name: t.to(DEV) for name, t in tensors.items()})
    out = execution.run().clone()
    execution.wait(30)
    expected = wl.ffn_block_oracle(tensors, 1e-6)
    # outputs reach |y| ~ 7, where a BF16 ulp is 2^-5: allow two ulps of the largest output
    top = expected.float().abs().max().item()
    assert_close_bf16(out.cpu(), expected, max_ulp=None, max_abs=2.0 ** (math.floor(math.log2(top)) - 6))
    execution.close()
    module.close()


@torch.inference_mode()
def test_ffn_block_from_loop_ir_text():
    """The same block read from loop-IR text in the reference fixture's spelling (rows taken
    whole, symbolic tile widths, two projections under one tile loop, normalisation through a
    broadcast expression): lower_ir -> nine launches -> oracle."""
    m, d_model, d_ff = 16, 512, 1024
    text, symbols, dtypes = plans.ffn_ir(m, d_model, d_ff)
    (plan,) = tl.lower_ir(text, symbols, dtypes)
    module = build(plan)
    tensors = wl.ffn_ir_inputs(m, d_model, d_ff, 47)
    execution = module.prepare({name: t.to(DEV) for name, t in tensors.items()})
    out = execution.run().clone()
    execution.wait(30)
    expected = wl.ffn_ir_oracle(tensors)
    top = expected.float().abs().max().item()
    assert_close_bf16(out.cpu(), expected, max_ulp=None, max_abs=2.0 ** (math.floor(math.log2(top)) - 6))
    execution.close()
    module.close()


# ---------------------------------------------------------------- primitive plans (reference fixtures)
def _pointwise_plan(name, shape, dtypes, scalar=None):
    import struct
    b = tl.PhysicalPlanBuilder()
    inputs = []
    for i, dt in enumerate(dtypes[:-1]):
        v = b.add_value(dt, list(shape), "external")
        b.bind_input(f"X{i}", v)
        inputs.append(v)
    out = b.add_value(dtypes[-1], list(shape), "external")
    parts = ["(clipped_tile col 128)"] if len(shape) == 1 else ["(tile row 1)", "(clipped_tile col 128)"]
    access = plans.index(*parts)
    args = [plans.load(v, shape, access) for v in inputs]
    if scalar is not None:
        args.append(f"(float_bits {struct.unpack('I', struct.pack('f', scalar))[0]})")
    operator = {"add": "+", "mul": "*", "div": "/", "scalar_div": "/", "square": "sqr"}.get(name, name)
    body = plans.store(out, shape, f"({operator} {' '.join(args)})", access)
    node = b.add_operation(inputs, [out], expression=body)
    node = b.add_loop("parallel", "col", 0, ((shape[-1] + 127) // 128) * 128, 128, [node])
    if len(shape) == 2:
        node = b.add_loop("parallel", "row", 0, shape[0], 1, [node])
    return b.build([node], "Y", out)


def _assert_result(actual, reference):
    # python/tests/test_tensor_ops.py:105-119: NaN / inf masks equal, <= 1 BF16 ulp, FP32 1e-5
    torch.testing.assert_close(torch.isnan(actual), torch.isnan(reference))
    torch.testing.assert_close(torch.isposinf(actual), torch.isposinf(reference))
    finite = torch.isfinite(reference)
    if actual.dtype == torch.bfloat16:
        from parity import ulp_distance
        assert (ulp_distance(actual.cpu(), reference.cpu())[finite.cpu()] <= 1).all()
    else:
        torch.testing.assert_close(actual, reference, rtol=1e-5, atol=1e-6, equal_nan=True)


@torch.inference_mode()
@pytest.mark.parametrize("shape", [(1,), (127,), (129,), (3, 257), (16, 4096)])
def test_primitive_pointwise_plans(shape):
    for name in ("add", "mul", "div", "scalar_div", "square", "sqrt", "sigmoid", "relu"):
        binary = name in ("add", "mul", "div")
        dtypes = ["bf16", "fp32", "bf16"] if binary else ["bf16", "fp32"]
        module = build(_pointwise_plan(name, shape, dtypes, 4096.0 if name == "scalar_div" else None))
        x0 = torch.randn(shape, device=DEV).bfloat16()
        if name == "sqrt":
            x0 = x0.abs()
        inputs = {"X0": x0}
        if binary:
            inputs["X1"] = torch.randn(shape, device=DEV) + 2.0
        execution = module.prepare(inputs)
        out = execution.run()
        execution.wait(30)
        a = x0.float()
        ref = {"add": lambda: a + inputs["X1"], "mul": lambda: a * inputs["X1"], "div": lambda: a / inputs["X1"],
               "scalar_div": lambda: a / 4096.0, "square": lambda: a * a, "sqrt": lambda: a.sqrt(),
               "sigmoid": lambda: 1.0 / (1.0 + torch.exp(-a)), "relu": lambda: torch.relu(a)}[name]()
        _assert_result(out, ref.to(out.dtype))
        execution.close()
        module.close()


@torch.inference_mode()
def test_relu_special_values_bit_exact():
    # python/tests/test_tensor_ops.py:161-186
    values = torch.tensor([-float("inf"), -2.0, -1e-8, -0.0, 0.0, 1e-8, 2.0, float("inf"), float("nan")], device=DEV)
    x = values.repeat(15)[:129].bfloat16()
    module = build(_pointwise_plan("relu", (129,), ["bf16", "fp32"]))
    execution = module.prepare({"X0": x})
    out = execution.run()
    execution.wait(30)
    reference = torch.relu(x.float())
    torch.testing.assert_close(out, reference, rtol=0, atol=0, equal_nan=True)
    zeros = reference == 0
    # -0.0 stays -0.0 under `x < 0 ? 0 : x`, as in the reference's kernel
    assert torch.equal(torch.signbit(out[zeros] ) | (x.float()[zeros] < 0), torch.signbit(x.float()[zeros]) | (x.float()[zeros] < 0))
    execution.close()
    module.close()


@torch.inference_mode()
def test_unfused_normalization_chain_keeps_zero_over_zero_nan():
    """square -> row sum -> scalar_div -> sqrt -> broadcast -> div as six statements
    (python/tests/tensor_ops.py:115-123), eps-free: an all-zero row gives NaN."""
    rows, cols = 16, 4096
    b = tl.PhysicalPlanBuilder()
    x = b.add_value("bf16", [rows, cols], "external")
    b.bind_input("X", x)
    full = plans.index("(tile row 1)", "(clipped_tile col 128)")
    vec = plans.index("(clipped_tile col 128)")
    statements = []

    def pointwise(out_dtype, shape, rhs, inflows, storage="global"):
        out = b.add_value(out_dtype, shape, storage)
        access = full if len(shape) == 2 else vec
        node = b.add_operation(inflows, [out], expression=plans.store(out, shape, rhs, access))
        node = b.add_loop("parallel", "col", 0, ((shape[-1] + 127) // 128) * 128, 128, [node])
        if len(shape) == 2:
            node = b.add_loop("parallel", "row", 0, shape[0], 1, [node])
        statements.append(node)
        return out

    square = pointwise("fp32", [rows, cols], f"(sqr {plans.load(x, [rows, cols], full)})", [x])
    total = b.add_value("fp32", [rows], "global")
    red = plans.index("(tile row 1)")
    chunk = plans.index("(tile row 1)", "(clipped_tile k 128)")
    rhs = f"(+ {plans.load(total, [rows], red)} (rsum {plans.load(square, [rows, cols], chunk)} 1))"
    node = b.add_operation([square], [total], expression=plans.store(total, [rows], rhs, red))
    node = b.add_loop("sequential", "k", 0, cols, 128, [node])
    statements.append(b.add_loop("parallel", "row", 0, rows, 1, [node]))
    mean = pointwise("fp32", [rows], f"(/ {plans.load(total, [rows], vec)} {plans.float_bits(float(cols))})", [total])
    root = pointwise("fp32", [rows], f"(sqrt {plans.load(mean, [rows], vec)})", [mean])
    wide = pointwise("fp32", [rows, cols], f"(bcast {plans.load(root, [rows], plans.index('(tile row 1)'))} 1)", [root])
    y = pointwise("bf16", [rows, cols], f"(/ {plans.load(x, [rows, cols], full)} {plans.load(wide, [rows, cols], full)})",
                  [x, wide], "external")
    plan = b.build(statements, "Y", y)
    source = tl.emit(plan)
    assert source.launch_count == 6
    vectors = [buf for buf in source.requirements.buffers if buf.shape == (rows,)]
    assert len(vectors) == 3 and all(v.dtype == "fp32" and v.bytes == 64 and v.strides == (1,) for v in vectors)
    module = build(plan)
    xs = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    xs[0].zero_()
    execution = module.prepare({"X": xs})
    for _ in range(3):
        out = execution.run()
    execution.wait(30)
    v = xs.float()
    _assert_result(out, (v / torch.sqrt(v.square().sum(1, keepdim=True) / cols)).bfloat16())
    assert torch.isnan(out[0].float()).all()
    execution.close()
    module.close()
