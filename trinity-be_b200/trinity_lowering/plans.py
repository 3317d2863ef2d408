"""Explicit loop programs for the benchmark configurations, in the reference's builder notation.

The plans keep the reference's tile vocabulary (``tile m 128``, ``tile k 64``, ``tile row 1``,
``clipped_tile col 128``) so the same builder calls are accepted by the reference's planner; the
sm_100a provider treats the loops as the logical iteration space and picks its own tiling.
"""
import math
import struct

from .compiler import PhysicalPlanBuilder


# ---------------------------------------------------------------- notation helpers
def view(value, shape):
    axes = " ".join(f"(axis a{i} {n})" for i, n in enumerate(shape))
    return f"(view (tensor v{value}) (layout {axes}))"


def index(*parts):
    return "(keyed_index " + " ".join(f"(slot a{i} {p})" for i, p in enumerate(parts)) + ")"


def load(value, shape, access):
    return f"(load {view(value, shape)} {access})"


def store(value, shape, rhs, access):
    return f"(store {view(value, shape)} {rhs} {access})"


def float_bits(x):
    return f"(float_bits {struct.unpack('I', struct.pack('f', x))[0]})"


def all_reduce(source, source_shape, source_index, destination, destination_shape, destination_index):
    return (f"(all_reduce {view(source, source_shape)} {source_index} "
            f"{view(destination, destination_shape)} {destination_index})")


def all_gather(source, source_shape, source_index, destination, destination_shape, destination_index, axis):
    return (f"(all_gather {view(source, source_shape)} {source_index} "
            f"{view(destination, destination_shape)} {destination_index} {axis})")


def gather(axis=0, world_size=2, rows=128, cols=128, target="sm100"):
    """Rank-major all-gather of a BF16 [rows, cols] shard along `axis` with a source tile loop, in
    the form of the reference's example (python/examples/plans.py:61-73 there)."""
    shapes = [[rows, cols], [rows, cols]]
    shapes[1][axis] *= world_size
    b = PhysicalPlanBuilder(world_size, target)
    x, y = [b.add_value("bf16", shape, "external") for shape in shapes]
    b.bind_input("X", x)
    access = index("(tile row 64)", "(tile col 64)")
    body = all_gather(x, shapes[0], access, y, shapes[1], access, axis)
    op = b.add_operation([x], [y], expression=body)
    col = b.add_loop("parallel", "col", 0, cols, 64, [op])
    row = b.add_loop("parallel", "row", 0, rows, 64, [col])
    return b.build([row], "Y", y)


def row_parallel_gemm(m, n, k_shard, world_size, target="sm100"):
    """Y (on every GPU) = sum over GPUs of A_r[m, k_shard] @ B_r[k_shard, n]: every rank multiplies
    its own K shard into an FP32 register accumulator and the partial products are summed across
    the GPUs (`all_reduce` of the accumulator into Y), which the provider does inside the GEMM's
    epilogue.  The down projection of a tensor-parallel MLP has this form."""
    b = PhysicalPlanBuilder(world_size, target)
    a = b.add_value("bf16", [m, k_shard], "external")
    w = b.add_value("bf16", [k_shard, n], "external")
    acc = b.add_value("fp32", [m, n], "register")
    y = b.add_value("bf16", [m, n], "external")
    b.bind_input("A", a)
    b.bind_input("W", w)
    tile_m, tile_n, tile_k = ("clipped_tile m 128", "clipped_tile n 128", "clipped_tile k 64")
    ai, bi, ci = index(f"({tile_m})", f"({tile_k})"), index(f"({tile_k})", f"({tile_n})"), index(f"({tile_m})", f"({tile_n})")
    rhs = f"(+ {load(acc, [m, n], ci)} (@ {load(a, [m, k_shard], ai)} {load(w, [k_shard, n], bi)}))"
    mma = b.add_operation([a, w], [acc], expression=store(acc, [m, n], rhs, ci))
    reduction = b.add_loop("sequential", "k", 0, _ceil(k_shard, 64), 64, [mma])
    total = b.add_operation([acc], [y], expression=all_reduce(acc, [m, n], ci, y, [m, n], ci))
    cols = b.add_loop("parallel", "n", 0, _ceil(n, 128), 128, [reduction, total])
    rows = b.add_loop("parallel", "m", 0, _ceil(m, 128), 128, [cols])
    return b.build([rows], "Y", y)


# ---------------------------------------------------------------- GEMM + epilogue
def gemm_bias(m, n, k, activation=None, bias="col", out_dtype="bf16", world_size=1, target="sm100"):
    """out = act(A[m,k] @ W[k,n] + bias): FP32 register accumulator, one rounding at the store.

    bias: "col" = bias[n] (``bcast ... 0``), "row" = bias[m], "matrix" = bias[m,n], None.
    activation: None | "relu" | "silu"."""
    b = PhysicalPlanBuilder(world_size, target)
    a = b.add_value("bf16", [m, k], "external")
    w = b.add_value("bf16", [k, n], "external")
    acc = b.add_value("fp32", [m, n], "register")
    b.bind_input("A", a)
    b.bind_input("W", w)
    tile_m, tile_n, tile_k = ("clipped_tile m 128", "clipped_tile n 128", "clipped_tile k 64")
    ai, bi, ci = index(f"({tile_m})", f"({tile_k})"), index(f"({tile_k})", f"({tile_n})"), index(f"({tile_m})", f"({tile_n})")
    rhs = f"(+ {load(acc, [m, n], ci)} (@ {load(a, [m, k], ai)} {load(w, [k, n], bi)}))"
    mma = b.add_operation([a, w], [acc], expression=store(acc, [m, n], rhs, ci))
    reduction = b.add_loop("sequential", "k", 0, _ceil(k, 64), 64, [mma])
    value = load(acc, [m, n], ci)
    inflows = [acc]
    if bias is not None:
        shape = {"col": [n], "row": [m], "matrix": [m, n]}[bias]
        bias_v = b.add_value("bf16", shape, "external")
        b.bind_input("bias", bias_v)
        inflows.append(bias_v)
        if bias == "col":
            side = f"(bcast {load(bias_v, shape, index(f'({tile_n})'))} 0)"
        elif bias == "row":
            side = f"(bcast {load(bias_v, shape, index(f'({tile_m})'))} 1)"
        else:
            side = load(bias_v, shape, ci)
        value = f"(+ {value} {side})"
    if activation == "relu":
        value = f"(relu {value})"
    elif activation == "silu":
        value = f"(* {value} (sigmoid {value}))"
    out = b.add_value(out_dtype, [m, n], "external")
    epilogue = b.add_operation(inflows, [out], expression=store(out, [m, n], value, ci))
    cols = b.add_loop("parallel", "n", 0, _ceil(n, 128), 128, [reduction, epilogue])
    rows = b.add_loop("parallel", "m", 0, _ceil(m, 128), 128, [cols])
    return b.build([rows], "Y", out)


def gated_gemm(m, n, k, world_size=1, target="sm100"):
    """H = (A @ Wu) * ((A @ Wg) * sigmoid(A @ Wg)): the reference FFN's SwiGLU spelling, two
    register accumulators under one tile nest."""
    b = PhysicalPlanBuilder(world_size, target)
    a = b.add_value("bf16", [m, k], "external")
    wg = b.add_value("bf16", [k, n], "external")
    wu = b.add_value("bf16", [k, n], "external")
    b.bind_input("A", a)
    b.bind_input("Wg", wg)
    b.bind_input("Wu", wu)
    up = b.add_value("fp32", [m, n], "register")
    gate = b.add_value("fp32", [m, n], "register")
    out = b.add_value("bf16", [m, n], "external")
    tm, tn, tk = "(clipped_tile m 128)", "(clipped_tile n 128)", "(clipped_tile k 64)"
    ai, ci = index(tm, tk), index(tm, tn)
    loops = []
    for acc, weight, var in ((up, wu, "ku"), (gate, wg, "kg")):
        kt = f"(clipped_tile {var} 64)"
        rhs = (f"(+ {load(acc, [m, n], ci)} (@ {load(a, [m, k], index(tm, kt))} "
               f"{load(weight, [k, n], index(kt, tn))}))")
        op = b.add_operation([a, weight], [acc], expression=store(acc, [m, n], rhs, ci))
        loops.append(b.add_loop("sequential", var, 0, _ceil(k, 64), 64, [op]))
    del ai
    g = load(gate, [m, n], ci)
    value = f"(* {load(up, [m, n], ci)} (* {g} (sigmoid {g})))"
    epilogue = b.add_operation([up, gate], [out], expression=store(out, [m, n], value, ci))
    cols = b.add_loop("parallel", "n", 0, _ceil(n, 128), 128, [*loops, epilogue])
    rows = b.add_loop("parallel", "m", 0, _ceil(m, 128), 128, [cols])
    return b.build([rows], "H", out)


def reference_gemm(m=128, n=128, k=64, relu=False, world_size=1, target="sm100"):
    """The reference's shipped example shape (python/examples/plans.py:27-58 there): BF16 GEMM
    into a global product, a [M,N] bias addition and optionally ReLU, each its own statement."""
    b = PhysicalPlanBuilder(world_size, target)
    shapes = [[m, k], [k, n], [m, n]]
    x = b.add_value("bf16", shapes[0], "external")
    weight = b.add_value("bf16", shapes[1], "external")
    product = b.add_value("bf16", shapes[2], "global")
    bias = b.add_value("bf16", shapes[2], "external")
    linear = b.add_value("bf16", shapes[2], "global" if relu else "external")
    b.bind_input("X", x)
    b.bind_input("W", weight)
    b.bind_input("bias", bias)
    ai, bi, ci = index("(tile m 128)", "(tile k 64)"), index("(tile k 64)", "(tile n 128)"), index("(tile m 128)", "(tile n 128)")
    rhs = f"(+ {load(product, shapes[2], ci)} (@ {load(x, shapes[0], ai)} {load(weight, shapes[1], bi)}))"
    op = b.add_operation([x, weight], [product], expression=store(product, shapes[2], rhs, ci))
    reduction = b.add_loop("sequential", "k", 0, k, 64, [op])
    columns = b.add_loop("parallel", "n", 0, n, 128, [reduction])
    rows = b.add_loop("parallel", "m", 0, m, 128, [columns])
    access = index("(tile row 1)", "(clipped_tile col 128)")
    rhs = f"(+ {load(product, shapes[2], access)} {load(bias, shapes[2], access)})"
    op = b.add_operation([product, bias], [linear], expression=store(linear, shapes[2], rhs, access))
    col = b.add_loop("parallel", "col", 0, _ceil(n, 128), 128, [op])
    row = b.add_loop("parallel", "row", 0, m, 1, [col])
    statements = [rows, row]
    output = linear
    if relu:
        output = b.add_value("bf16", shapes[2], "external")
        body = store(output, shapes[2], f"(relu {load(linear, shapes[2], access)})", access)
        op = b.add_operation([linear], [output], expression=body)
        col = b.add_loop("parallel", "col", 0, _ceil(n, 128), 128, [op])
        statements.append(b.add_loop("parallel", "row", 0, m, 1, [col]))
    return b.build(statements, "Y", output)


# ---------------------------------------------------------------- row kernels
def rmsnorm(rows, cols, eps=1e-6, gain=True, target="sm100"):
    """y = x / bcast(sqrt(rsum(sqr x) / cols + eps), 1) * bcast(g, 0), FP32 math, BF16 I/O."""
    b = PhysicalPlanBuilder(1, target)
    x = b.add_value("bf16", [rows, cols], "external")
    b.bind_input("X", x)
    ss = b.add_value("fp32", [rows], "register")
    y = b.add_value("bf16", [rows, cols], "external")
    row = "(tile row 1)"
    red = index(row)
    chunk = index(row, "(clipped_tile k 128)")
    rhs = f"(+ {load(ss, [rows], red)} (rsum (sqr {load(x, [rows, cols], chunk)}) 1))"
    reduce = b.add_operation([x], [ss], expression=store(ss, [rows], rhs, red))
    kloop = b.add_loop("sequential", "k", 0, _ceil(cols, 128), 128, [reduce])
    tile = index(row, "(clipped_tile col 128)")
    mean = f"(/ {load(ss, [rows], red)} {float_bits(float(cols))})"
    if eps:
        mean = f"(+ {mean} {float_bits(eps)})"
    value = f"(/ {load(x, [rows, cols], tile)} (bcast (sqrt {mean}) 1))"
    inflows = [x, ss]
    if gain:
        g = b.add_value("bf16", [cols], "external")
        b.bind_input("g", g)
        inflows.append(g)
        value = f"(* {value} (bcast {load(g, [cols], index('(clipped_tile col 128)'))} 0))"
    norm = b.add_operation(inflows, [y], expression=store(y, [rows, cols], value, tile))
    cloop = b.add_loop("parallel", "col", 0, _ceil(cols, 128), 128, [norm])
    rloop = b.add_loop("parallel", "row", 0, rows, 1, [kloop, cloop])
    return b.build([rloop], "Y", y)


def softmax(rows, cols, target="sm100"):
    """Stable row softmax: m = rmax x; e = exp(x - bcast m); s = rsum e; y = e / bcast s."""
    b = PhysicalPlanBuilder(1, target)
    x = b.add_value("bf16", [rows, cols], "external")
    b.bind_input("X", x)
    m = b.add_value("fp32", [rows], "register")
    e = b.add_value("fp32", [rows, cols], "register")
    s = b.add_value("fp32", [rows], "register")
    y = b.add_value("bf16", [rows, cols], "external")
    r1, r2 = index("(tile row 1)"), index("(tile row 1)", "fulltile")
    ops = [
        b.add_operation([x], [m], expression=store(m, [rows], f"(rmax {load(x, [rows, cols], r2)} 1)", r1)),
        b.add_operation([x, m], [e], expression=store(
            e, [rows, cols], f"(exp (- {load(x, [rows, cols], r2)} (bcast {load(m, [rows], r1)} 1)))", r2)),
        b.add_operation([e], [s], expression=store(s, [rows], f"(rsum {load(e, [rows, cols], r2)} 1)", r1)),
        b.add_operation([e, s], [y], expression=store(
            y, [rows, cols], f"(/ {load(e, [rows, cols], r2)} (bcast {load(s, [rows], r1)} 1))", r2)),
    ]
    loop = b.add_loop("parallel", "row", 0, rows, 1, ops)
    return b.build([loop], "Y", y)


# ---------------------------------------------------------------- whole FFN block
def ffn_block(m, d_model, d_ff, eps=1e-6, target="sm100"):
    """The decode-time feed-forward block of the reference's FFN fixture (tests/fixtures/ir/IR.v3.txt
    there: output projection, residual add, RMSNorm, SwiGLU, down projection, residual add) as one
    plan of four statements with BF16 intermediates in global memory:

        X1 = attn @ Wo + R                      (GEMM, residual as a matrix side operand)
        Xn = X1 / sqrt(mean(X1^2) + eps) * g    (RMSNorm)
        H  = (Xn @ Wu) * silu(Xn @ Wg)          (gated GEMM)
        Y  = H @ Wd + X1                        (GEMM, second residual)"""
    b = PhysicalPlanBuilder(1, target)

    def gemm(a, a_shape, weights, n, side, out, tag):
        """out[m,n] = f(sum_k a @ weights[i]) with f given by `side`; returns the statement."""
        k = a_shape[1]
        tm, tn = f"(clipped_tile m{tag} 128)", f"(clipped_tile n{tag} 128)"
        ci = index(tm, tn)
        loops, accs = [], []
        for i, weight in enumerate(weights):
            acc = b.add_value("fp32", [m, n], "register")
            var = f"k{tag}{i}"
            kt = f"(clipped_tile {var} 64)"
            rhs = (f"(+ {load(acc, [m, n], ci)} (@ {load(a, a_shape, index(tm, kt))} "
                   f"{load(weight, [k, n], index(kt, tn))}))")
            op = b.add_operation([a, weight], [acc], expression=store(acc, [m, n], rhs, ci))
            loops.append(b.add_loop("sequential", var, 0, _ceil(k, 64), 64, [op]))
            accs.append(acc)
        inflows, value = side(accs, ci)
        epilogue = b.add_operation(inflows, [out], expression=store(out, [m, n], value, ci))
        cols = b.add_loop("parallel", f"n{tag}", 0, _ceil(n, 128), 128, [*loops, epilogue])
        return b.add_loop("parallel", f"m{tag}", 0, _ceil(m, 128), 128, [cols])

    attn = b.add_value("bf16", [m, d_model], "external")
    wo = b.add_value("bf16", [d_model, d_model], "external")
    residual = b.add_value("bf16", [m, d_model], "external")
    gain = b.add_value("bf16", [d_model], "external")
    wg = b.add_value("bf16", [d_model, d_ff], "external")
    wu = b.add_value("bf16", [d_model, d_ff], "external")
    wd = b.add_value("bf16", [d_ff, d_model], "external")
    for name, v in (("attn", attn), ("Wo", wo), ("R", residual), ("g", gain), ("Wg", wg), ("Wu", wu), ("Wd", wd)):
        b.bind_input(name, v)
    x1 = b.add_value("bf16", [m, d_model], "global")
    xn = b.add_value("bf16", [m, d_model], "global")
    h = b.add_value("bf16", [m, d_ff], "global")
    y = b.add_value("bf16", [m, d_model], "external")

    def plus(matrix):
        def side(accs, ci):
            return [accs[0], matrix], f"(+ {load(accs[0], [m, d_model], ci)} {load(matrix, [m, d_model], ci)})"
        return side

    def swiglu(accs, ci):
        g = load(accs[1], [m, d_ff], ci)
        return [accs[0], accs[1]], f"(* {load(accs[0], [m, d_ff], ci)} (* {g} (sigmoid {g})))"

    first = gemm(attn, [m, d_model], [wo], d_model, plus(residual), x1, "a")
    # RMSNorm of X1 (the row kernels' plan form, see rmsnorm above)
    ss = b.add_value("fp32", [m], "register")
    row = "(tile row 1)"
    red, chunk, tile = index(row), index(row, "(clipped_tile k 128)"), index(row, "(clipped_tile col 128)")
    rhs = f"(+ {load(ss, [m], red)} (rsum (sqr {load(x1, [m, d_model], chunk)}) 1))"
    reduce = b.add_operation([x1], [ss], expression=store(ss, [m], rhs, red))
    kloop = b.add_loop("sequential", "k", 0, _ceil(d_model, 128), 128, [reduce])
    mean = f"(+ (/ {load(ss, [m], red)} {float_bits(float(d_model))}) {float_bits(eps)})"
    value = (f"(* (/ {load(x1, [m, d_model], tile)} (bcast (sqrt {mean}) 1)) "
             f"(bcast {load(gain, [d_model], index('(clipped_tile col 128)'))} 0))")
    norm = b.add_operation([x1, ss, gain], [xn], expression=store(xn, [m, d_model], value, tile))
    cloop = b.add_loop("parallel", "col", 0, _ceil(d_model, 128), 128, [norm])
    second = b.add_loop("parallel", "row", 0, m, 1, [kloop, cloop])
    third = gemm(xn, [m, d_model], [wu, wg], d_ff, swiglu, h, "b")
    fourth = gemm(h, [m, d_ff], [wd], d_model, plus(x1), y, "c")
    return b.build([first, second, third, fourth], "Y", y)


def ffn_ir(m, d_model, d_ff, tile_n=128, tile_k=64, tile_p=128):
    """The same block in the loop-IR *text* notation that ``lower_ir`` reads, spelled the way the
    reference's feed-forward fixture spells it (tests/fixtures/ir/IR.v3.txt there): no row loop
    (rows are ``fulltile``), symbolic tile widths, BF16 tensors between all steps, RMSNorm without
    eps or gain, SwiGLU as two projections followed by separate pointwise steps:

        P = attn @ Wo; Q = P + X; s = rsum(Q^2); N = Q / sqrt(s / d_model)
        A = N @ Wa; B = N @ Wb; S = B * sigmoid(B); H = A * S; Y = H @ Wd

    Returns (text, symbols, dtypes) for ``lower_ir``; nine launches on the sm_100a provider."""
    def view(kind, name, *extents):
        axes = " ".join(f"(axis a_{i} {n})" for i, n in enumerate(extents))
        return f"(view ({kind} {name}) (layout {axes}))"

    def at(*slots):
        return "(keyed_index " + " ".join(f"(slot a_{i} {s})" for i, s in enumerate(slots)) + ")"

    def tile(var):
        return f"(tile {var} tile_{var})"

    def matmul(dst_kind, dst, lhs_kind, lhs, weight, rows, inner, cols, out_var, k_var):
        c = view(dst_kind, dst, rows, cols)
        ci = at("fulltile", tile(out_var))
        a = f"(load {view(lhs_kind, lhs, rows, inner)} {at('fulltile', tile(k_var))})"
        b = f"(load {view('input', weight, inner, cols)} {at(tile(k_var), tile(out_var))})"
        return f"(sloop 0 {inner} tile_{k_var} {k_var} (store {c} (+ (load {c} {ci}) (@ {a} {b})) {ci}))"

    def pointwise(dst, cols, var, rhs):
        return f"(ploop 0 {cols} tile_{var} {var} (store {view('tensor', dst, m, cols)} {rhs} {at('fulltile', tile(var))}))"

    def elem(kind, name, cols, var):
        return f"(load {view(kind, name, m, cols)} {at('fulltile', tile(var))})"

    vec = view("tensor", "s", m)
    steps = [
        f"(ploop 0 {d_model} tile_n n {matmul('tensor', 'P', 'input', 'attn', 'Wo', m, d_model, d_model, 'n', 'k')})",
        pointwise("Q", d_model, "n", f"(+ {elem('tensor', 'P', d_model, 'n')} {elem('input', 'X', d_model, 'n')})"),
        (f"(sloop 0 {d_model} tile_k k (store {vec} (+ (load {vec} {at('fulltile')}) "
         f"(rsum (sqr {elem('tensor', 'Q', d_model, 'k')}) 1)) {at('fulltile')}))"),
        pointwise("N", d_model, "k",
                  f"(/ {elem('tensor', 'Q', d_model, 'k')} (bcast (sqrt (/ (load {vec} {at('fulltile')}) {d_model})) 1))"),
        (f"(ploop 0 {d_ff} tile_p p (seq {matmul('tensor', 'A', 'tensor', 'N', 'Wa', m, d_model, d_ff, 'p', 'k')} "
         f"{matmul('tensor', 'B', 'tensor', 'N', 'Wb', m, d_model, d_ff, 'p', 'k')}))"),
        pointwise("S", d_ff, "p", f"(* {elem('tensor', 'B', d_ff, 'p')} (sigmoid {elem('tensor', 'B', d_ff, 'p')}))"),
        pointwise("H", d_ff, "p", f"(* {elem('tensor', 'A', d_ff, 'p')} {elem('tensor', 'S', d_ff, 'p')})"),
        f"(ploop 0 {d_model} tile_n n {matmul('output', 'Y', 'tensor', 'H', 'Wd', m, d_ff, d_model, 'n', 'p')})",
    ]
    text = steps[-1]
    for step in reversed(steps[:-1]):
        text = f"(seq {step} {text})"
    dtypes = {name: "bf16" for name in ("attn", "Wo", "X", "Wa", "Wb", "Wd", "P", "Q", "N", "A", "B", "S", "H", "Y")}
    dtypes["s"] = "fp32"
    return text, {"tile_n": tile_n, "tile_k": tile_k, "tile_p": tile_p}, dtypes


# ---------------------------------------------------------------- MLA decode
def mla_decode(batch, heads, seq, d_qk=576, d_v=512, scale=None, target="sm100"):
    """out[b] = softmax(scale * q[b] @ cache[b]^T) @ cache[b][:, :d_v] for every batch entry."""
    scale = 1.0 / math.sqrt(192.0) if scale is None else scale
    b = PhysicalPlanBuilder(1, target)
    q = b.add_value("bf16", [batch, heads, d_qk], "external")
    cache = b.add_value("bf16", [batch, seq, d_qk], "external")
    b.bind_input("q", q)
    b.bind_input("cache", cache)
    S = b.add_value("fp32", [batch, heads, seq], "register")
    m = b.add_value("fp32", [batch, heads], "register")
    E = b.add_value("fp32", [batch, heads, seq], "register")
    l = b.add_value("fp32", [batch, heads], "register")
    P = b.add_value("fp32", [batch, heads, seq], "register")
    out = b.add_value("bf16", [batch, heads, d_v], "external")
    e3 = index("(elem b)", "fulltile", "fulltile")
    e2 = index("(elem b)", "fulltile")
    qs, cs, ss, os_, ms = [batch, heads, d_qk], [batch, seq, d_qk], [batch, heads, seq], [batch, heads, d_v], [batch, heads]
    ops = [
        b.add_operation([q, cache], [S], expression=store(
            S, ss, f"(* (@ {load(q, qs, e3)} (transpose {load(cache, cs, e3)})) {float_bits(scale)})", e3)),
        b.add_operation([S], [m], expression=store(m, ms, f"(rmax {load(S, ss, e3)} 2)", e2)),
        b.add_operation([S, m], [E], expression=store(
            E, ss, f"(exp (- {load(S, ss, e3)} (bcast {load(m, ms, e2)} 2)))", e3)),
        b.add_operation([E], [l], expression=store(l, ms, f"(rsum {load(E, ss, e3)} 2)", e2)),
        b.add_operation([E, l], [P], expression=store(
            P, ss, f"(/ {load(E, ss, e3)} (bcast {load(l, ms, e2)} 2))", e3)),
    ]
    values = index("(elem b)", "fulltile", f"(tile v {d_v})")
    pv = b.add_operation([P, cache], [out], expression=store(
        out, os_, f"(+ {load(out, os_, e3)} (@ {load(P, ss, e3)} {load(cache, cs, values)}))", e3))
    vloop = b.add_loop("sequential", "v", 0, d_v, d_v, [pv])
    loop = b.add_loop("parallel", "b", 0, batch, 1, [*ops, vloop])
    return b.build([loop], "out", out)


def _ceil(extent, tile):
    return ((extent + tile - 1) // tile) * tile
