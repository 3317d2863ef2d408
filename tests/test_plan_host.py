"""Planner / emitter / artifact builder on the CPU (no GPU): the C++ host library through its
C ABI, checked against the behaviour the reference's tests pin."""
import json
import subprocess

import pytest

import trinity_lowering as tl
from trinity_lowering import plans


def copy_builder():
    b = tl.PhysicalPlanBuilder()
    x = b.add_value("fp32", [64], "external", name="X")
    y = b.add_value("fp32", [64], "external", name="Y")
    b.bind_input("X", x)
    return b, x, y


def expression(access):
    return ("(store (view (output Y) (layout (axis a 64))) (sqrt (load (view (input X) (layout (axis a 64))) "
            f"(keyed_index (slot a {access})))) (keyed_index (slot a {access})))")


def test_operation_metadata_and_no_inferred_loop():
    # python/tests/test_explicit_plan.py:40-60 of the reference
    b, x, y = copy_builder()
    with pytest.raises(TypeError, match="expression"):
        b.add_operation([x], [y])
    node = b.add_operation(inflows=[x], outflows=[y], expression=expression("fulltile"))
    metadata = json.loads(b.build([node], "Y", y).metadata_json())
    assert metadata["statements"] == [{"operations": [0]}]
    assert metadata["operations"] == [{"id": 0, "inflows": [metadata["inputs"][0]["value"]],
                                       "outflows": [metadata["output"]["value"]]}]


def test_serial_domain_is_preserved_and_matches_text_ir():
    # python/tests/test_explicit_plan.py:58-73
    b, x, y = copy_builder()
    body = expression("(tile i 16)")
    op = b.add_operation([x], [y], expression=body)
    loop = b.add_loop("sequential", "i", 16, 64, 16, [op])
    plan = json.loads(b.build([loop], "Y", y).metadata_json())
    assert plan["statements"][0]["loop"]["domain"] == {
        "variable": "lv0", "start": {"Constant": 16}, "stop": {"Constant": 64}, "step": {"Constant": 16}}
    assert plan["statements"][0]["loop"]["body"] == [{"operations": [0]}]
    (ir,) = tl.lower_ir(f"(sloop 16 64 16 i {body})", {}, {"X": "fp32", "Y": "fp32"})
    assert json.loads(ir.metadata_json()) == plan


def test_nested_bounds_are_renamed_and_duplicate_membership_is_rejected():
    # python/tests/test_explicit_plan.py:76-95
    b, x, y = copy_builder()
    op = b.add_operation([x], [y], expression=expression("fulltile"))
    inner = b.add_loop("sequential", "j", "i", "(+ i 1)", 1, [op])
    outer = b.add_loop("parallel", "i", 0, 2, 1, [inner])
    plan = json.loads(b.build([outer], "Y", y).metadata_json())
    inner = plan["statements"][0]["loop"]["body"][0]["loop"]
    assert inner["domain"]["start"] == {"Variable": "lv0"}
    assert inner["domain"]["stop"] == {"Add": [{"Variable": "lv0"}, {"Constant": 1}]}
    b, x, y = copy_builder()
    op = b.add_operation([x], [y], expression=expression("fulltile"))
    loop = b.add_loop("parallel", "i", 0, 1, 1, [op])
    with pytest.raises(ValueError, match="multiple statements"):
        b.build([op, loop], "Y", y)


def test_inputs_sorted_by_name_and_ids_in_first_use_order():
    # tests/physical_plan.rs:82-88, src/tests.rs:147-158
    def build(order):
        b = tl.PhysicalPlanBuilder()
        ids = {}
        for name in order:
            ids[name] = b.add_value("bf16", [128, 128], "external")
        for name in order:
            if name != "Y":
                b.bind_input(name, ids[name])
        acc = index = "(keyed_index (slot a0 (tile r 1)) (slot a1 (clipped_tile c 128)))"
        def v(i):
            return f"(view (tensor v{i}) (layout (axis a0 128) (axis a1 128)))"
        body = f"(store {v(ids['Y'])} (+ (load {v(ids['B'])} {index}) (load {v(ids['A'])} {index})) {acc})"
        op = b.add_operation([ids["A"], ids["B"]], [ids["Y"]], expression=body)
        col = b.add_loop("parallel", "c", 0, 128, 128, [op])
        row = b.add_loop("parallel", "r", 0, 128, 1, [col])
        return b.build([row], "Y", ids["Y"])
    first, second = build(["A", "B", "Y"]), build(["Y", "B", "A"])
    assert first == second and hash(first) == hash(second)
    data = json.loads(first.metadata_json())
    assert [i["name"] for i in data["inputs"]] == ["A", "B"]
    assert data["operations"][0]["inflows"] == [data["inputs"][1]["value"], data["inputs"][0]["value"]]


def test_zero_started_accumulation_is_not_an_inflow():
    # src/tests.rs:252-300: inside a single-operation sequential loop the destination load is the
    # implicit zero; outside such a loop the same spelling needs a producer
    data = json.loads(plans.gemm_bias(256, 256, 128, bias=None).metadata_json())
    acc = data["operations"][0]["outflows"][0]
    assert acc not in data["operations"][0]["inflows"]
    b = tl.PhysicalPlanBuilder()
    x = b.add_value("fp32", [64], "external", name="X")
    y = b.add_value("fp32", [64], "external", name="Y")
    b.bind_input("X", x)
    body = ("(store (view (output Y) (layout (axis a 64))) (+ (load (view (output Y) (layout (axis a 64))) "
            "(keyed_index (slot a fulltile))) (load (view (input X) (layout (axis a 64))) (keyed_index (slot a fulltile)))) "
            "(keyed_index (slot a fulltile)))")
    op = b.add_operation([x, y], [y], expression=body)
    with pytest.raises(ValueError, match="MissingProducer"):
        b.build([op], "Y", y)


def test_error_taxonomy():
    b, x, y = copy_builder()
    b.bind_input("X", y)
    op = b.add_operation([x], [y], expression=expression("fulltile"))
    with pytest.raises(ValueError, match="DuplicateInputTensor"):
        b.build([op], "Y", y)
    b, x, y = copy_builder()
    with pytest.raises(ValueError, match="unknown value"):
        b.add_operation([999], [y], expression="(store invalid)")
    b, x, y = copy_builder()
    op = b.add_operation([x], [y], expression=expression("(tile i 16)"))
    with pytest.raises(ValueError, match="unbound index"):
        b.build([op], "Y", y)
    b, x, y = copy_builder()
    with pytest.raises(ValueError, match="declared inflows"):
        op = b.add_operation([], [y], expression=expression("fulltile"))
        b.build([op], "Y", y)
    b, x, y = copy_builder()
    t = b.add_value("fp32", [64], "global", name="T")
    with pytest.raises(ValueError, match="declared outflow"):
        op = b.add_operation([x], [t], expression=expression("fulltile"))
        b.build([op], "Y", y)
    with pytest.raises(ValueError, match="unexpected trailing input"):
        tl.lower_ir("(seq dummy dummy) x", {}, {})
    with pytest.raises(ValueError, match="unclosed expression"):
        tl.lower_ir("(seq dummy", {}, {})


def test_register_values_cannot_cross_statements():
    b = tl.PhysicalPlanBuilder()
    x = b.add_value("fp32", [64], "external", name="X")
    t = b.add_value("fp32", [64], "register", name="T")
    y = b.add_value("fp32", [64], "external", name="Y")
    b.bind_input("X", x)
    def unary(dst, src, role_dst, role_src):
        return (f"(store (view ({role_dst} {dst}) (layout (axis a 64))) (sqrt (load (view ({role_src} {src}) "
                "(layout (axis a 64))) (keyed_index (slot a fulltile)))) (keyed_index (slot a fulltile)))")
    a = b.add_operation([x], [t], expression=unary("T", "X", "tensor", "input"))
    c = b.add_operation([t], [y], expression=unary("Y", "T", "output", "tensor"))
    with pytest.raises(ValueError, match="CrossStatementStorage"):
        b.build([a, c], "Y", y)


def test_bind_symbols_binds_tile_widths_and_bounds_together():
    # tests/plan_access.rs:53-99
    b, x, y = copy_builder()
    op = b.add_operation([x], [y], expression=expression("(tile i T)"))
    loop = b.add_loop("parallel", "i", 0, 64, "T", [op])
    plan = b.build([loop], "Y", y)
    assert plan.symbols == ["T"]
    with pytest.raises(ValueError, match="bind_symbols"):
        tl.emit(plan)
    with pytest.raises(ValueError):
        plan.bind_symbols({})
    with pytest.raises(ValueError):
        plan.bind_symbols({"T": 0})
    bound = plan.bind_symbols({"T": 16})
    assert bound.symbols == []
    b, x, y = copy_builder()
    op = b.add_operation([x], [y], expression=expression("(tile i 16)"))
    loop = b.add_loop("parallel", "i", 0, 64, 16, [op])
    assert bound == b.build([loop], "Y", y)


def test_identity_plan_emits_without_a_launch():
    # python/tests/test_explicit_plan.py:16-23
    b = tl.PhysicalPlanBuilder()
    x = b.add_value("fp32", [4], "external")
    b.bind_input("X", x)
    source = tl.emit(b.build([], "Y", x))
    assert source.launch_count == 0 and "trinity_sm100_gemm_bf16(&" not in source.code
    assert source.requirements.buffers[0].alignment == 4
    assert source.requirements.buffers[0].input_names == ("X",) and source.requirements.buffers[0].output_name == "Y"


def test_emit_is_deterministic_and_counts_launches():
    # tests/streamed.rs:117-173
    p = plans.gemm_bias(1024, 1024, 1024)
    assert tl.emit(p).code == tl.emit(plans.gemm_bias(1024, 1024, 1024)).code
    assert tl.emit(p).launch_count == 1                       # K loop + bias fused into one launch
    ref = plans.reference_gemm(256, 256, 192, relu=True)      # three statements, three launches
    source = tl.emit(ref)
    assert source.launch_count == 3
    assert sum(not b.external for b in source.requirements.buffers) == 2
    assert all(b.dtype == "bf16" for b in source.requirements.buffers)
    data = json.loads(ref.metadata_json())
    assert {b["name"] for b in data["inputs"]} == {"X", "W", "bias"}
    assert len(data["operations"]) == len(data["statements"]) == 3
    # only External / Global values get buffer slots
    fused = tl.emit(plans.rmsnorm(64, 4096))
    assert [b.shape for b in fused.requirements.buffers] == [(64, 4096), (4096,), (64, 4096)]


def test_ffn_block_plan_emits_four_launches():
    """GEMM + residual, RMSNorm, gated GEMM, GEMM + residual: one launch per statement, the
    intermediates are global values the runtime allocates."""
    plan = plans.ffn_block(16, 512, 1024)
    source = tl.emit(plan)
    assert source.launch_count == 4
    kernels = [line.split("rc = ")[1].split("(")[0] for line in source.code.splitlines()
               if "rc = trinity_sm100_" in line and "_bf16" in line]
    assert kernels == ["trinity_sm100_gemm_bf16", "trinity_sm100_rmsnorm_bf16",
                       "trinity_sm100_gemm_bf16", "trinity_sm100_gemm_bf16"]
    metadata = json.loads(plan.metadata_json())
    assert [v["storage"] for v in metadata["values"]].count("global") == 3
    assert [i["name"] for i in metadata["inputs"]] == sorted(["attn", "Wo", "R", "g", "Wg", "Wu", "Wd"])


def test_ffn_loop_ir_text_lowers_and_emits_nine_launches():
    """Loop-IR text in the spelling of the reference's feed-forward fixture: rows are `fulltile`
    (no row loop), tile widths are symbols bound at lowering, the two SwiGLU projections sit
    under one tile loop, the normalisation broadcasts an expression over the row sums."""
    text, symbols, dtypes = plans.ffn_ir(16, 512, 1024)
    (plan,) = tl.lower_ir(text, symbols, dtypes)
    metadata = json.loads(plan.metadata_json())
    assert [i["name"] for i in metadata["inputs"]] == ["Wa", "Wb", "Wd", "Wo", "X", "attn"]
    assert len(metadata["operations"]) == 9 and len(metadata["statements"]) == 8
    source = tl.emit(plan)
    kernels = [line.split("rc = ")[1].split("(")[0] for line in source.code.splitlines()
               if "rc = trinity_sm100_" in line and "stream)" in line and "synchronize" not in line]
    assert kernels == ["trinity_sm100_gemm_bf16", "trinity_sm100_pointwise", "trinity_sm100_row_reduce_sum",
                       "trinity_sm100_pointwise", "trinity_sm100_gemm_bf16", "trinity_sm100_gemm_bf16",
                       "trinity_sm100_pointwise", "trinity_sm100_pointwise", "trinity_sm100_gemm_bf16"]
    # a tile width that does not divide the extent is refused, as for any `tile` access
    with pytest.raises(ValueError, match="exactly divide"):
        tl.emit(tl.lower_ir(text, {**symbols, "tile_n": 96}, dtypes)[0])


def test_world_size_other_than_one_is_refused_like_the_reference():
    # tests/streamed.rs:202-209, python/tests/test_tensor_ops.py:25-28
    with pytest.raises(NotImplementedError, match="Persistent"):
        tl.emit(plans.gemm_bias(256, 256, 128, world_size=2))


def test_all_gather_plans_become_persistent_artifacts():
    """A multi-GPU plan whose statements are rank-major all-gathers (python/examples/plans.py:61-73
    there) is emitted as a persistent artifact: mode 2 in the descriptor, PersistentLaunch in
    trinity_launch, the shard a symmetric buffer, a workspace that starts with the peer table."""
    for axis in (0, 1):
        source = tl.emit(plans.gather(axis=axis, world_size=4))
        assert source.launch_count == 1 and "trinity_sm100_allgather_bf16(workspace, 0, bindings[1], 128, 128, "\
            f"{axis}, 4, stream)" in source.code
        assert "PersistentLaunch const* launch_args" in source.code and "describe(2," in source.code
        needs = json.loads(source._native.requirements_json())
        assert needs["world_size"] == 4 and needs["workspace_bytes"] == 1024 and needs["workspace_symmetric"]
        assert [b["symmetric"] for b in needs["buffers"]] == [True, False]
        assert needs["buffers"][1]["shape"] == ([512, 128] if axis == 0 else [128, 512])
    artifact = tl.compile(tl.emit(plans.gather(axis=1, world_size=2)))
    try:
        manifest = json.loads((artifact.directory / "manifest.json").read_text())
        assert manifest["execution"] == "persistent" and manifest["requirements"]["nvshmem"] is True
        exported = subprocess.run(["nm", "-D", "--defined-only", str(artifact.directory / "program.so")],
                                  capture_output=True, text=True, check=True).stdout.split()
        assert sorted(n for n in exported if n.startswith("trinity_")) == [
            "trinity_abi", "trinity_launch", "trinity_prepare", "trinity_release", "trinity_status"]
    finally:
        artifact.close()
    # the down projection of a tensor-parallel MLP: one launch, the sum across GPUs in the GEMM's epilogue
    fused = tl.emit(plans.row_parallel_gemm(512, 1024, 1024, 2))
    assert fused.launch_count == 1 and "trinity_sm100_gemm_allreduce_workspace_bf16(&g, workspace, " in fused.code
    needs = json.loads(fused._native.requirements_json())
    assert [b["symmetric"] for b in needs["buffers"]] == [False, False, True]      # A, W local; Y symmetric
    assert needs["workspace_bytes"] == 1024 + 4 * (64 + 16 * 2 + 16)                 # peer table + flag pad
    found = tl.kernel_candidates(plans.row_parallel_gemm(512, 1024, 1024, 2))
    assert all([c["provider"] for c in entry["candidates"]] == ["sm100.gemm_all_reduce"] for entry in found.values())
    # a shard whose rows are not multiples of 16 bytes, or a destination of the wrong extent, is declined
    with pytest.raises(NotImplementedError, match="all_gather"):
        tl.emit(plans.gather(axis=0, world_size=2, rows=64, cols=68))


def test_hazards_are_errors():
    # tests/plan_access.rs:213-249: overlapping tiles and partial coverage
    def tiled(step, stop):
        b, x, y = copy_builder()
        op = b.add_operation([x], [y], expression=expression("(clipped_tile i 16)"))
        loop = b.add_loop("parallel", "i", 0, stop, step, [op])
        return b.build([loop], "Y", y)
    with pytest.raises(ValueError, match="overlap between CTAs"):
        tl.emit(tiled(8, 64))
    with pytest.raises(ValueError, match="output region is not fully produced"):
        tl.emit(tiled(16, 32))
    assert tl.emit(tiled(16, 64)).launch_count == 1


def test_kernel_candidates_list_per_operation_offers_and_rejections():
    """Candidate discovery (src/emit/candidate.rs:107-207 there): nothing is selected; each
    operation carries the launches that would cover it and, per recogniser that declined, the
    reason.  An operation nothing covers keeps an empty candidate list with its diagnostics."""
    found = tl.kernel_candidates(plans.gemm_bias(256, 256, 128, "relu"))
    assert sorted(found) == ["0", "1"]                      # the K-loop product and its epilogue
    for entry in found.values():
        assert entry["scope"] == {"statement": 0}
        assert entry["candidates"] == [{"provider": "sm100.gemm", "kind": "native",
                                        "kernel": "trinity_sm100_gemm_bf16", "operations": [0, 1]}]
        declined = {r["provider"]: r["reason"] for r in entry["rejections"]}
        assert declined["sm100.pointwise"] == "no applicable implementations"
        assert "not part of" in declined["triton"] and "not part of" in declined["quack"]
    norm = tl.kernel_candidates(plans.rmsnorm(64, 4096))
    assert {c["provider"] for c in norm["0"]["candidates"]} == {"sm100.rmsnorm"}
    assert {"provider": "sm100.gemm", "reason": "sm100.gemm: not load(acc) + matmul"} in norm["0"]["rejections"]

    def overlapping():
        b, x, y = copy_builder()
        op = b.add_operation([x], [y], expression=expression("(clipped_tile i 16)"))
        return b.build([b.add_loop("parallel", "i", 0, 64, 8, [op])], "Y", y)
    bad = tl.kernel_candidates(overlapping())
    assert bad["0"]["candidates"] == []
    reasons = {r["provider"]: r["reason"] for r in bad["0"]["rejections"]}
    assert "overlap between CTAs" in reasons["sm100.pointwise"]
    # single-GPU kernels are not offered to multi-GPU plans, whose collective has its own recogniser
    multi = tl.kernel_candidates(plans.gemm_bias(256, 256, 128, world_size=2))
    assert multi["0"]["candidates"] == [] and any("Persistent" in r["reason"] for r in multi["0"]["rejections"])
    gathered = tl.kernel_candidates(plans.gather(axis=0, world_size=2))
    assert [c["provider"] for c in gathered["0"]["candidates"]] == ["sm100.all_gather"]
    # plan-level refusals stay plan-level, as the reference's prepare step fails the whole call
    b = tl.PhysicalPlanBuilder()
    x = b.add_value("fp16", [64], "external", name="X")
    b.bind_input("X", x)
    assert "fp16" in tl.kernel_candidates(b.build([], "Y", x))["error"]


def test_unsupported_operations_report_no_provider():
    b = tl.PhysicalPlanBuilder()
    x = b.add_value("fp16", [64], "external", name="X")
    b.bind_input("X", x)
    with pytest.raises(NotImplementedError):
        tl.emit(b.build([], "Y", x))


def test_artifact_exports_exactly_five_symbols_and_cleans_up():
    # src/compile/cuda/tests.rs:243-266, python/tests/test_compiler.py:22-73
    source = tl.emit(plans.gemm_bias(256, 256, 128, "relu"))
    first, second = tl.compile(source), tl.compile(source)
    assert first.directory != second.directory
    names = subprocess.run(["nm", "-D", "--defined-only", str(first.artifact_path)], capture_output=True,
                           text=True, check=True).stdout.split()
    exported = sorted(n for n in names if n.startswith("trinity_"))
    assert exported == ["trinity_abi", "trinity_launch", "trinity_prepare", "trinity_release", "trinity_status"]
    assert {p.name for p in first.directory.iterdir()} == {
        "source.cu", "exports.map", "program.so", "manifest.json", "diagnostics.json"}
    on_disk = json.loads((first.directory / "manifest.json").read_text())
    assert on_disk["requirements"] == json.loads(source._native.requirements_json())
    assert on_disk["execution"] == "streamed" and on_disk["library"] == "program.so"
    assert first.diagnostics["exit_code"] == 0
    directory = first.directory
    first.close()
    assert not directory.exists()
    kept = second.persist()
    second.close()
    assert (kept / "program.so").exists()
    import shutil
    shutil.rmtree(kept)


def test_compile_failure_carries_diagnostics():
    source = tl.emit(plans.softmax(8, 256))
    with pytest.raises(tl.CompileError) as info:
        tl.compile(source, tl.CompileConfig(host_compiler="/nonexistent/bin/g++"))
    assert "MissingCompiler" in str(info.value)
    assert info.value.diagnostics["exit_code"] != 0
    with pytest.raises(tl.CompileError) as info:   # a "compiler" that runs but produces nothing
        tl.compile(source, tl.CompileConfig(host_compiler="/bin/true"))
    assert "MissingArtifact" in str(info.value)


def test_requirements_validation_rejects_corruption():
    # python/tests/test_tensor_ops.py:88-102
    from trinity_lowering.metadata import requirements
    data = json.loads(tl.emit(plans.softmax(8, 256))._native.requirements_json())
    assert requirements(data).buffers[-1].bytes == 8 * 256 * 2
    for update in ({"bytes": 258}, {"strides": [2, 1]}, {"shape": [1, 1, 1, 8], "strides": [8, 8, 8, 1]},
                   {"dtype": "fp64"}, {"alignment": 3}):
        corrupted = json.loads(json.dumps(data))
        corrupted["buffers"][-1].update(update)
        with pytest.raises(ValueError):
            requirements(corrupted)


def test_implementation_enumeration():
    # python/tests/test_tensor_ops.py:66-86
    def definition(name):
        return next(d for d in tl.pointwise_implementations() if d.id == f"cuda.{name}")
    assert [d.id for d in tl.gemm_implementations()][0] == "blackwell.tcgen05.bf16"
    with pytest.raises(ValueError):
        definition("add").enumerate(["fp32"] * 3, [[16], [17], [16]])
    with pytest.raises(ValueError):
        definition("square").enumerate(["fp32"] * 3, [[16]] * 3)
    with pytest.raises(ValueError):
        definition("scalar_div").enumerate(["fp32"] * 2, [[16]] * 2)
    with pytest.raises(ValueError):
        definition("sqrt").enumerate(["fp32"] * 2, [[16]] * 2, scalar=2.0)
    with pytest.raises(ValueError):
        tl.reduce_sum_implementations()[0].enumerate(["fp32"] * 2, [[16, 32], [33]])
    with pytest.raises(ValueError):
        tl.broadcast_implementations()[0].enumerate(["fp32", "bf16"], [[16], [16, 32]])
    assert tl.reduce_sum_implementations()[0].enumerate(["bf16"] * 2, [[16, 32], [16]]) == []
    assert tl.reduce_sum_implementations()[0].enumerate(["fp32"] * 2, [[16, 32], [32]], axis=0) == []


def test_c_abi_libraries_export_every_declared_symbol():
    import ctypes
    import re
    from pathlib import Path
    from trinity_lowering import _host, kernels
    root = Path(__file__).resolve().parents[1]
    for header, lib, prefix in (("trinity_sm100.h", kernels.library_path(), "trinity_sm100_"),
                                ("trinity_host.h", _host._LIB_PATH, "th_")):
        declared = set(re.findall(r"\b(" + prefix + r"\w+)\s*\(", (root / "include" / header).read_text()))
        declared -= {"trinity_sm100_mla", "trinity_sm100_gemm"}
        handle = ctypes.CDLL(str(lib))
        missing = [name for name in sorted(declared) if not hasattr(handle, name)]
        assert not missing, missing
        assert len(declared) >= 15


def test_mla_schedule_queries_need_no_device():
    """The schedule the MLA entry point will pick is a host computation (148 SMs are assumed when
    no device is current): scratch sizing and slot counts can be asked for ahead of time."""
    import ctypes
    from trinity_lowering import kernels
    lib = ctypes.CDLL(str(kernels.library_path()))
    lib.trinity_sm100_mla_default_splits.argtypes = [ctypes.c_int32] * 2
    lib.trinity_sm100_mla_balanced_slots.argtypes = [ctypes.c_int32] * 2
    lib.trinity_sm100_mla_scratch_bytes.argtypes = [ctypes.c_int32] * 4
    lib.trinity_sm100_mla_scratch_bytes.restype = ctypes.c_size_t
    # one cluster per sequence fills 64 of 74 SM pairs: sequences are not cut
    assert lib.trinity_sm100_mla_default_splits(64, 4096) == 1
    assert lib.trinity_sm100_mla_scratch_bytes(64, 128, 512, 1) == 0
    # few long sequences: equal splits, about one cluster per SM pair
    splits = lib.trinity_sm100_mla_default_splits(8, 16384)
    assert 8 <= splits <= 9
    # a sequence of 64 chunks over runs of 4096 / 74 = 55 chunks touches two or three clusters
    assert lib.trinity_sm100_mla_balanced_slots(64, 4096) in (2, 3)
    # more sequences than SM pairs, poorly filled second wave: balanced runs
    assert lib.trinity_sm100_mla_default_splits(100, 4096) == lib.trinity_sm100_mla_balanced_slots(100, 4096) == 2
    # never finer than eight chunks per cluster on average
    assert lib.trinity_sm100_mla_default_splits(1, 512) == 1
    assert lib.trinity_sm100_mla_balanced_slots(1, 65536) == 74
    slots = lib.trinity_sm100_mla_balanced_slots(5, 1000)
    need = lib.trinity_sm100_mla_scratch_bytes(5, 128, 512, slots)
    assert need >= 5 * slots * 128 * (512 + 2) * 4 and need % 256 == 0
    assert lib.trinity_sm100_mla_default_splits(0, 4096) == 1


def test_package_keeps_the_reference_names():
    """python/src/trinity_lowering/__init__.py:29-58 of the reference; the Triton entry points
    import but refuse."""
    reference_names = [
        "CompileConfig", "CompileError", "CudaArtifact", "CudaSource", "Implementation", "PhysicalPlan",
        "PhysicalPlanBuilder", "TritonProgram", "all_gather_implementations", "pointwise_implementations",
        "reduce_sum_implementations", "broadcast_implementations", "compile", "emit", "emit_python",
        "emit_triton", "lower_triton", "gemm_implementations", "lower_ir", "DistributedFailure",
        "ResourceBusy", "RuntimeFailure", "Graph", "IOBuffers", "LoadedModule", "PreparedExecution",
        "load", "World"]
    for name in reference_names:
        assert hasattr(tl, name) and name in tl.__all__, name
    for refused in (tl.emit_python, tl.emit_triton, tl.lower_triton, tl.TritonProgram):
        with pytest.raises(NotImplementedError):
            refused(None)


def test_text_reader_grammar_and_located_errors():
    """Comments to end of line, located errors with a byte offset, arity of `seq`, the nesting
    limit, ranks 1-3 only, unknown operators; loop variables are renamed, so spelling them
    differently gives the same plan (the reader rules of src/analysis/ir/syntax.rs:82-143 and
    src/analysis/plan/ir.rs:447,503 in the reference)."""
    base = ("(ploop 0 256 128 c (store (view (output Y) (layout (axis a 256))) (relu (load (view (input X) "
            "(layout (axis a 256))) (keyed_index (slot a (tile c 128))))) (keyed_index (slot a (tile c 128)))))")
    dtypes = {"X": "bf16", "Y": "bf16"}
    (plan,) = tl.lower_ir("; a comment line\n" + base + " ; trailing comment", {}, dtypes)
    renamed = base.replace("128 c (store", "128 col (store").replace("tile c 128", "tile col 128")
    assert plan.same_body(tl.lower_ir(renamed, {}, dtypes)[0])
    assert not plan.same_body(tl.lower_ir(base.replace("relu", "sqrt"), {}, dtypes)[0])
    domain = json.loads(plan.metadata_json())["statements"][0]["loop"]["domain"]
    assert domain == {"variable": "lv0", "start": {"Constant": 0}, "stop": {"Constant": 256}, "step": {"Constant": 128}}
    rank4 = ("(ploop 0 4 1 c (store (view (output Y) (layout (axis a 4) (axis b 2) (axis c 2) (axis d 2))) (load "
             "(view (input X) (layout (axis a 4) (axis b 2) (axis c 2) (axis d 2))) (keyed_index (slot a (elem c)) "
             "(slot b fulltile) (slot c fulltile) (slot d fulltile))) (keyed_index (slot a (elem c)) (slot b fulltile) "
             "(slot c fulltile) (slot d fulltile))))")
    for text, fragment in ((base + " (extra)", "unexpected trailing input"),
                           (base[:-1], "unclosed expression"),
                           ("(" * 300 + ")" * 300, "nesting exceeds 256"),
                           (f"(seq {base} {base} {base})", "'seq' expects 2 arguments"),
                           (base.replace("relu", "tanh"), "unsupported operation tanh"),
                           (rank4, "supported tensor ranks are 1, 2, 3")):
        with pytest.raises(ValueError, match=fragment + ".* at byte"):
            tl.lower_ir(text, {}, dtypes)
    with pytest.raises(ValueError, match="missing dtype"):
        tl.lower_ir(base, {}, {"X": "bf16"})


def test_split_loops_and_view_operators_of_the_attention_fixtures():
    """`mloop` is normalised to a parallel loop over the split around a sequential loop over the
    split's share (src/analysis/plan/ir.rs:527-599 there); `permute`, `bcast`, `unsqueeze` and
    `elem` accesses are read in the spelling of the reference's batched-MLA fixtures
    (tests/fixtures/batched_mla/batched_mla_postprocessed_stage14.txt:27-56 there)."""
    def view(kind, name):
        return f"(view ({kind} {name}) (layout (axis a 256)))"
    tile = "(keyed_index (slot a (tile c 64)))"
    body = f"(store {view('output', 'Y')} (relu (load {view('input', 'X')} {tile})) {tile})"
    dtypes = {"X": "bf16", "Y": "bf16"}
    (split,) = tl.lower_ir(f"(mloop 0 256 64 c s 2 {body})", {}, dtypes)
    (nest,) = tl.lower_ir(f"(ploop 0 2 1 s (sloop (+ 0 (* s 128)) (+ (+ 0 (* s 128)) 128) 64 c {body}))", {}, dtypes)
    assert split.same_body(nest)
    loops = json.loads(split.metadata_json())["statements"][0]["loop"]
    assert loops["kind"] == "parallel" and loops["domain"]["stop"] == {"Constant": 2}
    assert loops["body"][0]["loop"]["kind"] == "sequential"
    for text, fragment in ((f"(mloop 0 256 64 c s 3 {body})", "mloop split must exactly divide"),
                           (f"(mloop 0 256 96 c s 2 {body})", "mloop split must exactly divide"),
                           (f"(ploop 0 4 1 s (mloop 0 256 64 c s 2 {body}))", "split variable shadows an active loop"),
                           (f"(sloop 0 4 1 k (mloop 0 256 64 c s 2 {body}))", "parallel work inside")):
        with pytest.raises(ValueError, match=fragment):
            tl.lower_ir(text, {}, dtypes)

    def projection(axes):
        q = "(view (input Q) (layout (axis b 4) (axis h 16) (axis k 128)))"
        w = "(view (input W) (layout (axis k 128) (axis m 512)))"
        t = "(view (output T) (layout (axis b 4) (axis h 16) (axis m 512)))"
        at = "(keyed_index (slot b (tile b 2)) (slot h (elem n)) (slot m (tile m 128)))"
        return (f"(ploop 0 4 2 b (ploop 0 16 1 n (ploop 0 512 128 m (store {t} (@ (load {q} (keyed_index (slot b (tile b 2)) "
                f"(slot h (elem n)) (slot k fulltile))) (permute (bcast (load {w} (keyed_index (slot k fulltile) "
                f"(slot m (tile m 128)))) 0) {axes})) {at}))))")
    dtypes = {"Q": "bf16", "W": "bf16", "T": "bf16"}
    (plan,) = tl.lower_ir(projection("0 2 1"), {}, dtypes)
    assert not plan.same_body(tl.lower_ir(projection("0 1 2"), {}, dtypes)[0])
    with pytest.raises(ValueError, match="permute axes must be a permutation"):
        tl.lower_ir(projection("0 2 2"), {}, dtypes)
    found = tl.kernel_candidates(plan)["0"]       # no kernel region has this form yet: recorded, not hidden
    assert found["candidates"] == [] and found["rejections"]


def test_text_reader_rejects_hazards_where_the_reference_does():
    """Reader-level rejections with the reference's message fragments (tests/streamed.rs:183-190,
    tests/ir.rs:52-63, src/analysis/storage/mod.rs:303-312, :352-363 there): parallel work inside
    a sequential loop, a write that a parallel loop does not index, a read beyond what earlier
    kernels wrote.  A write of a loop-invariant value to an un-indexed location is allowed."""
    def view(kind, name):
        return f"(view ({kind} {name}) (layout (axis a 256)))"
    tile, half, full = ("(keyed_index (slot a (tile c 128)))", "(keyed_index (slot a (tile c 64)))",
                        "(keyed_index (slot a fulltile))")
    dtypes = {"X": "bf16", "Y": "bf16", "T": "fp32"}

    def produce(index, stop=256, start=0):
        return (f"(ploop {start} {stop} 128 c (store {view('tensor', 'T')} "
                f"(sqr (load {view('input', 'X')} {index})) {index}))")
    consume = f"(ploop 0 256 128 c (store {view('output', 'Y')} (relu (load {view('tensor', 'T')} {tile})) {tile}))"
    (plan,) = tl.lower_ir(f"(seq {produce(tile)} {consume})", {}, dtypes)
    assert [v["storage"] for v in json.loads(plan.metadata_json())["values"]] == ["external", "global", "external"]
    for text, fragment in (
            (f"(seq {produce(tile, stop=128)} {consume})", "not covered"),
            (f"(seq {produce(half)} {consume})", "not covered"),          # 64-wide tiles every 128: gaps
            (f"(ploop 0 256 128 c (store {view('output', 'Y')} (relu (load {view('input', 'X')} {tile})) {full}))",
             "not proven disjoint"),
            (f"(sloop 0 256 128 k {consume.replace('tensor', 'input').replace(' T)', ' X)')})", "parallel work inside")):
        with pytest.raises(ValueError, match=fragment + ".* at byte [1-9]"):
            tl.lower_ir(text, {}, dtypes)
    # two kernels that write one half each cover a later read of the whole tensor
    halves = f"(seq (seq {produce(tile, stop=128)} {produce(tile, start=128)}) {consume})"
    assert len(tl.lower_ir(halves, {}, dtypes)) == 1
    invariant = f"(ploop 0 256 128 c (store {view('output', 'Y')} (relu (load {view('input', 'X')} {full})) {full}))"
    assert len(tl.lower_ir(invariant, {}, dtypes)) == 1
