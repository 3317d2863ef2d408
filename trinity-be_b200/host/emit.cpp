// sm_100a provider: recognises whole regions of a plan and maps each onto one call of the
// kernel library.
//
// The plan keeps the reference's tile vocabulary (tile m 128, tile k 64, tile row 1,
// clipped_tile col 128, ...).  Those loops are treated as the *logical* iteration space: for a
// rectangular tiling (start 0, step == tile width) coverage of [0, extent) and disjointness of
// the tiles follow in closed form, without visiting blocks as the reference's validator does
// (src/emit/native/cuda/validation.rs:328-395); the kernels then choose their own physical
// tiling.  Messages for the hazards keep the reference's wording ("overlap between CTAs",
// "output region is not fully produced").
//
// Region grammar for GEMM + epilogue follows the reference's provider-neutral recogniser
// (src/emit/provider/quack/recognition.rs:209-348): a chain of parallel loops, a sequential K
// loop whose single operation is `acc = load(acc) + A @ B`, then plain operations writing the
// same coordinates built from pointwise nodes over the accumulator and side operands.
#include "emit.hpp"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <functional>
#include <sstream>

namespace trinity::host {

std::string g_include_dir;  // set through the C API; holds trinity_abi.h and trinity_sm100.h

namespace {

[[noreturn]] void unsupported(const std::string& what) { throw PlanError(ErrorKind::NotImplemented, what); }
[[noreturn]] void invalid_execution(const std::string& what) {
  throw PlanError(ErrorKind::Value, "InvalidExecution: " + what);
}

struct LoopInfo {
  std::string variable;
  int64_t start, stop, step;
  LoopKind kind;
};

bool constant_loop(const Statement& s, LoopInfo& out) {
  if (!s.is_loop || !s.domain.start.is_constant() || !s.domain.stop.is_constant() ||
      !s.domain.step.is_constant())
    return false;
  out = {s.domain.variable, s.domain.start.value, s.domain.stop.value, s.domain.step.value, s.kind};
  return true;
}

// Strips a chain of single-child parallel loops; returns the innermost body.
const std::vector<Statement>* strip_parallel(const Statement& s, std::vector<LoopInfo>& loops) {
  const Statement* cur = &s;
  const std::vector<Statement>* body = nullptr;
  while (cur->is_loop && cur->kind == LoopKind::Parallel) {
    LoopInfo info;
    if (!constant_loop(*cur, info)) unsupported("NoProvider: parallel loop bounds must be constants; bind_symbols first");
    loops.push_back(info);
    body = &cur->body;
    if (cur->body.size() != 1) break;
    cur = &cur->body[0];
  }
  return body;
}

const LoopInfo* find_loop(const std::vector<LoopInfo>& loops, const std::string& v) {
  for (auto& l : loops)
    if (l.variable == v) return &l;
  return nullptr;
}

// Closed-form proof that a tiled axis written under a parallel loop covers [0, extent) without
// overlap between CTAs.
void check_parallel_axis(const AccessIndex& index, const LoopInfo& loop, int64_t extent, const char* what) {
  const int64_t width = index.kind == AccessIndex::Elem ? 1 : index.width.constant;
  if (loop.step <= 0 || loop.start != 0) unsupported(std::string("NoProvider: ") + what + " loop must start at 0 with a positive step");
  if (loop.step < width) invalid_execution(std::string(what) + ": overlap between CTAs (loop step smaller than tile width)");
  if (loop.step > width || loop.stop < extent)
    invalid_execution(std::string(what) + ": output region is not fully produced");
  if (index.kind == AccessIndex::Tile && (loop.stop != extent || extent % width != 0))
    invalid_execution(std::string(what) + ": tile width must exactly divide the extent (use clipped_tile)");
}

bool same_access(const TensorAccess& a, const TensorAccess& b) { return a == b; }

const char* dt_enum(DType d) { return d == DType::Fp32 ? "TRINITY_SM100_FP32" : "TRINITY_SM100_BF16"; }

std::string slot_ptr(int slot) { return "bindings[" + std::to_string(slot) + "]"; }

struct Emitter {
  const PhysicalPlan& plan;
  std::vector<int> slots;  // value -> buffer slot or -1
  std::vector<BufferRequirement> buffers;
  std::vector<Launch> launches;
  std::vector<std::string> rejections;  // per-statement reasons when nothing matched

  explicit Emitter(const PhysicalPlan& p) : plan(p) {}

  const Value& value(int id) const { return plan.values[id]; }
  int slot(int v) const {
    if (slots[v] < 0) throw PlanError(ErrorKind::Value, "Combination: value " + std::to_string(v) + " has no buffer slot");
    return slots[v];
  }
  void need_alignment(int v, int bytes) {
    auto& b = buffers[slot(v)];
    if (b.alignment < bytes) b.alignment = bytes;
  }

  void build_buffers() {
    slots.assign(plan.values.size(), -1);
    for (size_t id = 0; id < plan.values.size(); ++id) {
      const Value& v = plan.values[id];
      if (v.storage == Storage::Register) continue;
      BufferRequirement b;
      b.slot = int(buffers.size());
      for (auto& in : plan.inputs)
        if (in.value == int(id)) b.input_names.push_back(in.tensor);
      if (!plan.outputs.empty() && plan.outputs[0].value == int(id)) {
        b.is_output = true;
        b.output_name = plan.outputs[0].tensor;
      }
      b.shape = v.shape;
      b.strides.assign(v.shape.size(), 1);
      int64_t elements = 1;
      for (int axis = int(v.shape.size()) - 1; axis >= 0; --axis) {
        b.strides[axis] = elements;
        elements *= v.shape[axis];
      }
      b.dtype = v.dtype;
      b.bytes = elements * dtype_bytes(v.dtype);
      b.alignment = dtype_bytes(v.dtype);
      b.external = v.storage == Storage::External;
      slots[id] = b.slot;
      buffers.push_back(std::move(b));
    }
  }

  // ------------------------------------------------------------------ GEMM region
  struct Accumulator {
    int op = -1, acc = -1, a = -1, b = -1;
    TensorAccess acc_access;
    int64_t m = 0, n = 0, k = 0;
  };

  bool match_accumulate(const Statement& loop, const std::vector<LoopInfo>& parallel, Accumulator& out,
                        std::string& why) {
    LoopInfo k;
    if (!loop.is_loop || loop.kind != LoopKind::Sequential || loop.body.size() != 1 || loop.body[0].is_loop ||
        !constant_loop(loop, k)) {
      why = "not a single-operation sequential loop with constant bounds";
      return false;
    }
    const Operation& op = plan.operations[loop.body[0].operation];
    const Expression& e = *op.expression;
    if (e.kind != Expression::Store || e.args[0]->kind != Expression::Add) { why = "not an accumulation"; return false; }
    const Expression& sum = *e.args[0];
    if (sum.args[0]->kind != Expression::Load || !same_access(sum.args[0]->access, e.access) ||
        sum.args[1]->kind != Expression::Matmul) { why = "not load(acc) + matmul"; return false; }
    const Expression& mm = *sum.args[1];
    if (mm.args[0]->kind != Expression::Load || mm.args[1]->kind != Expression::Load) { why = "matmul operands must be loads"; return false; }
    const TensorAccess& A = mm.args[0]->access;
    const TensorAccess& B = mm.args[1]->access;
    const TensorAccess& C = e.access;
    if (!A.view_shape.empty() || !B.view_shape.empty() || !C.view_shape.empty() || A.indices.size() != 2 ||
        B.indices.size() != 2 || C.indices.size() != 2) { why = "operands must be rank-2 base views"; return false; }
    auto tiled = [](const AccessIndex& i) {
      return (i.kind == AccessIndex::Tile || i.kind == AccessIndex::ClippedTile) && !i.width.symbolic;
    };
    // The row axis may be taken whole (`fulltile`: a decode-time GEMM with a handful of rows and
    // no row loop, as the reference's feed-forward IR writes it); every other axis is tiled.
    const bool full_rows = A.indices[0].kind == AccessIndex::FullTile && C.indices[0].kind == AccessIndex::FullTile;
    for (auto* acc : {&A, &B, &C})
      for (size_t axis = 0; axis < 2; ++axis)
        if (!tiled(acc->indices[axis]) && !(full_rows && axis == 0 && acc != &B)) {
          why = "accesses must be constant-width tiles (rows may be fulltile)";
          return false;
        }
    const std::string &mv = C.indices[0].variable, &nv = C.indices[1].variable, &kv = k.variable;
    if ((!full_rows && A.indices[0].variable != mv) || A.indices[1].variable != kv || B.indices[0].variable != kv ||
        B.indices[1].variable != nv) { why = "tile variables do not form C[m,n] += A[m,k] B[k,n]"; return false; }
    const Value &va = value(A.value), &vb = value(B.value), &vc = value(C.value);
    if (va.dtype != DType::Bf16 || vb.dtype != DType::Bf16) { why = "operands must be bf16"; return false; }
    if (vc.dtype == DType::Fp16) { why = "fp16 accumulators are not supported"; return false; }
    const int64_t M = va.shape[0], K = va.shape[1], N = vb.shape[1];
    if (vb.shape[0] != K || vc.shape[0] != M || vc.shape[1] != N) { why = "shape mismatch"; return false; }
    if (K % 8 || N % 8) { why = "K and N must be multiples of 8"; return false; }
    const LoopInfo* ml = full_rows ? nullptr : find_loop(parallel, mv);
    const LoopInfo* nl = find_loop(parallel, nv);
    if ((!full_rows && !ml) || !nl) { why = "output tiles must be indexed by the enclosing parallel loops"; return false; }
    if (parallel.size() != (full_rows ? 1u : 2u))
      invalid_execution("gemm: overlap between CTAs (a parallel loop does not index the output)");
    if (!full_rows) check_parallel_axis(C.indices[0], *ml, M, "gemm rows");
    check_parallel_axis(C.indices[1], *nl, N, "gemm columns");
    if ((!full_rows && A.indices[0].width.constant != C.indices[0].width.constant) ||
        B.indices[1].width.constant != C.indices[1].width.constant)
      invalid_execution("gemm: operand tiles differ from the output tile");
    const int64_t wk = A.indices[1].width.constant;
    if (B.indices[0].width.constant != wk) invalid_execution("gemm: A and B disagree on the K tile width");
    if (k.start != 0 || k.step != wk || k.stop < K || (A.indices[1].kind == AccessIndex::Tile && (k.stop != K || K % wk)))
      invalid_execution("gemm: the K loop must cover [0, K) in steps of the K tile width (exactly divide, or use clipped_tile)");
    out.op = loop.body[0].operation;
    out.acc = C.value;
    out.a = A.value;
    out.b = B.value;
    out.acc_access = C;
    out.m = M; out.n = N; out.k = K;
    return true;
  }

  // Symbolic form of an epilogue value: which accumulator(s), side operand, activation.
  struct Form {
    int acc = -1;        // accumulator index (0/1), -1 none
    int gate_acc = -1;   // gated: acc * silu(gate_acc)
    int bias = -1, bias_mode = 0;
    int act = 0;         // 0 none, 1 relu, 2 silu
    bool valid = false;
    bool plain() const { return valid && gate_acc < 0 && bias < 0 && act == 0; }
    bool operator==(const Form& o) const {
      return acc == o.acc && gate_acc == o.gate_acc && bias == o.bias && bias_mode == o.bias_mode && act == o.act && valid == o.valid;
    }
  };

  void emit_plain_gemm(const Accumulator& a) {
    const Value& vo = value(a.acc);
    std::ostringstream c;
    c << "  {\n    trinity_sm100_gemm g = {};\n";
    c << "    g.a = " << slot_ptr(slot(a.a)) << ";\n    g.b = " << slot_ptr(slot(a.b)) << ";\n";
    c << "    g.out = " << slot_ptr(slot(a.acc)) << ";\n";
    need_alignment(a.a, 16);
    need_alignment(a.b, 16);
    need_alignment(a.acc, 16);
    c << "    g.m = " << a.m << "; g.n = " << a.n << "; g.k = " << a.k << ";\n";
    c << "    g.lda = " << a.k << "; g.ldb = " << a.n << "; g.ldo = " << a.n << ";\n";
    c << "    g.activation = 0;\n    g.out_dtype = " << dt_enum(vo.dtype) << ";\n";
    c << "    rc = trinity_sm100_gemm_bf16(&g, stream);\n  }\n";
    Launch l;
    l.kernel = "trinity_sm100_gemm_bf16";
    l.code = c.str();
    l.operations = {a.op};
    l.shared_memory_bytes = 230656;
    l.block_threads = 192;
    launches.push_back(std::move(l));
  }

  bool try_gemm(const Statement& top) {
    std::vector<LoopInfo> parallel;
    const std::vector<Statement>* body = strip_parallel(top, parallel);
    if (!body || parallel.empty()) return false;
    std::vector<Accumulator> accs;
    size_t next = 0;
    std::string why;
    while (next < body->size() && (*body)[next].is_loop) {
      Accumulator a;
      if (!match_accumulate((*body)[next], parallel, a, why)) {
        if (accs.empty()) { rejections.push_back("sm100.gemm: " + why); return false; }
        unsupported("NoProvider: sm100.gemm: " + why);
      }
      accs.push_back(a);
      ++next;
    }
    if (accs.empty()) return false;
    // Several accumulations under one tile nest, each into its own global value and none consumed
    // by an epilogue (the reference's feed-forward IR computes the two SwiGLU projections so):
    // independent GEMMs, one launch each.
    if (next == body->size() && accs.size() >= 2) {
      for (auto& a : accs)
        if (value(a.acc).storage == Storage::Register)
          unsupported("NoProvider: sm100.gemm: a register accumulator without an epilogue is never stored");
      for (auto& a : accs) emit_plain_gemm(a);
      return true;
    }
    if (accs.size() > 2) return false;
    if (accs.size() == 2 && (accs[0].a != accs[1].a || accs[0].m != accs[1].m || accs[0].n != accs[1].n ||
                             !same_access(accs[0].acc_access.indices == accs[1].acc_access.indices ? accs[0].acc_access : accs[0].acc_access, accs[0].acc_access)))
      unsupported("NoProvider: sm100.gemm: two accumulators must share the left operand and shape");
    // epilogue: symbolic evaluation of the following plain operations
    std::map<int, Form> forms;
    for (size_t i = 0; i < accs.size(); ++i) {
      Form f;
      f.valid = true;
      f.acc = int(i);
      forms[accs[i].acc] = f;
    }
    const auto& tile = accs[0].acc_access.indices;
    std::vector<int> ops;
    for (auto& a : accs) ops.push_back(a.op);
    int out_value = accs.size() == 1 ? accs[0].acc : -1;
    Form out_form = forms[accs[0].acc];
    std::function<Form(const Expression&)> eval = [&](const Expression& e) -> Form {
      Form bad;
      switch (e.kind) {
        case Expression::Load: {
          auto it = forms.find(e.access.value);
          if (it != forms.end() && e.access.indices == tile) return it->second;
          return bad;
        }
        case Expression::Add: {
          for (int side = 0; side < 2; ++side) {
            Form x = eval(*e.args[side]);
            if (!x.plain()) continue;
            const Expression& s = *e.args[1 - side];
            Form r = x;
            if (s.kind == Expression::Load && s.access.indices == tile && !forms.count(s.access.value)) {
              r.bias = s.access.value; r.bias_mode = 3; return r;
            }
            if (s.kind == Expression::Broadcast && s.args[0]->kind == Expression::Load) {
              const TensorAccess& b = s.args[0]->access;
              if (b.indices.size() == 1 && s.axis == 0 && b.indices[0] == tile[1]) { r.bias = b.value; r.bias_mode = 1; return r; }
              if (b.indices.size() == 1 && s.axis == 1 && b.indices[0] == tile[0]) { r.bias = b.value; r.bias_mode = 2; return r; }
            }
          }
          return bad;
        }
        case Expression::Relu: {
          Form x = eval(*e.args[0]);
          if (x.valid && x.act == 0 && x.gate_acc < 0) { x.act = 1; return x; }
          return bad;
        }
        case Expression::Max: {
          for (int side = 0; side < 2; ++side) {
            const Expression& z = *e.args[1 - side];
            const bool zero = (z.kind == Expression::ConstInt && z.integer == 0) || (z.kind == Expression::ConstF32 && (z.f32_bits << 1) == 0);
            Form x = eval(*e.args[side]);
            if (zero && x.valid && x.act == 0 && x.gate_acc < 0) { x.act = 1; return x; }
          }
          return bad;
        }
        case Expression::Mul: {
          for (int side = 0; side < 2; ++side) {
            const Expression& l = *e.args[side];
            const Expression& r = *e.args[1 - side];
            Form x = eval(l);
            if (!x.valid) continue;
            // x * sigmoid(x) -> silu
            if (r.kind == Expression::Sigmoid) {
              Form y = eval(*r.args[0]);
              if (y.valid && y == x && x.act == 0 && x.gate_acc < 0) { x.act = 2; return x; }
            }
            // up * silu(gate)
            Form g = eval(r);
            if (x.plain() && g.valid && g.act == 2 && g.bias < 0 && g.gate_acc < 0 && g.acc != x.acc) {
              Form out = x;
              out.gate_acc = g.acc;
              return out;
            }
          }
          return bad;
        }
        default:
          return bad;
      }
    };
    for (; next < body->size(); ++next) {
      const Statement& s = (*body)[next];
      if (s.is_loop) unsupported("NoProvider: sm100.gemm: loops after the K loop are not part of an epilogue");
      const Operation& op = plan.operations[s.operation];
      const Expression& e = *op.expression;
      if (e.kind != Expression::Store || !(e.access.indices == tile) || !e.access.view_shape.empty())
        unsupported("NoProvider: sm100.gemm: epilogue operations must write the accumulator's coordinates");
      Form f = eval(*e.args[0]);
      if (!f.valid) unsupported("NoProvider: sm100.gemm: epilogue expression is not bias / relu / silu / gate over the accumulator");
      forms[e.access.value] = f;
      ops.push_back(s.operation);
      out_value = e.access.value;
      out_form = f;
    }
    if (out_value < 0 || value(out_value).storage == Storage::Register)
      unsupported("NoProvider: sm100.gemm: the region must end in a store to a global or external value");
    if (accs.size() == 2 && out_form.gate_acc < 0)
      unsupported("NoProvider: sm100.gemm: two accumulators need the gated form up * (gate * sigmoid(gate))");
    for (auto& a : accs)
      if (a.acc != out_value && value(a.acc).storage != Storage::Register)
        unsupported("NoProvider: sm100.gemm: an accumulator consumed by an epilogue must be a register value");
    const Value& vo = value(out_value);
    if (vo.dtype == DType::Fp16) unsupported("NoProvider: fp16 output");
    const Accumulator& up = accs[out_form.acc];
    std::ostringstream c;
    c << "  {\n    trinity_sm100_gemm g = {};\n";
    c << "    g.a = " << slot_ptr(slot(up.a)) << ";\n    g.b = " << slot_ptr(slot(up.b)) << ";\n";
    need_alignment(up.a, 16);
    need_alignment(up.b, 16);
    int activation = out_form.act;  // 0,1,2 match the library enum
    if (out_form.gate_acc >= 0) {
      const Accumulator& gate = accs[out_form.gate_acc];
      c << "    g.b2 = " << slot_ptr(slot(gate.b)) << ";\n";
      need_alignment(gate.b, 16);
      activation = 3;
    }
    if (out_form.bias >= 0) {
      c << "    g.bias = " << slot_ptr(slot(out_form.bias)) << ";\n    g.bias_mode = " << out_form.bias_mode << ";\n";
      if (out_form.bias_mode == 3) c << "    g.ld_bias = " << up.n << ";\n";
      if (value(out_form.bias).dtype != DType::Bf16) unsupported("NoProvider: sm100.gemm: bias must be bf16");
      need_alignment(out_form.bias, 16);
    }
    c << "    g.out = " << slot_ptr(slot(out_value)) << ";\n";
    need_alignment(out_value, 16);
    c << "    g.m = " << up.m << "; g.n = " << up.n << "; g.k = " << up.k << ";\n";
    c << "    g.lda = " << up.k << "; g.ldb = " << up.n << "; g.ldo = " << up.n << ";\n";
    c << "    g.activation = " << activation << ";\n    g.out_dtype = " << dt_enum(vo.dtype) << ";\n";
    c << "    rc = trinity_sm100_gemm_bf16(&g, stream);\n  }\n";
    Launch l;
    l.kernel = "trinity_sm100_gemm_bf16";
    l.code = c.str();
    l.operations = ops;
    l.shared_memory_bytes = 230656;
    l.block_threads = 192;
    launches.push_back(std::move(l));
    return true;
  }

  // ------------------------------------------------------------------ pointwise statement
  struct PwBuild {
    std::vector<std::pair<int, int>> operands;  // (value, broadcast)
    std::vector<uint32_t> program;
  };
  int pw_operand(PwBuild& b, int value_id, int broadcast) {
    for (size_t i = 0; i < b.operands.size(); ++i)
      if (b.operands[i] == std::make_pair(value_id, broadcast)) return int(i);
    b.operands.emplace_back(value_id, broadcast);
    return int(b.operands.size()) - 1;
  }
  // The operand of a broadcast: a vector along the output's rows (axis 1) or columns (axis 0), or
  // a pointwise expression over such vectors and constants (`bcast (sqrt (/ v 4096)) 1`).  The
  // interpreter evaluates it per output element, which repeats a little arithmetic per row.
  bool pw_compile_vector(const Expression& e, const TensorAccess& dst, int axis, PwBuild& b, std::string& why) {
    switch (e.kind) {
      case Expression::ConstInt: {
        const float f = float(e.integer);
        uint32_t bits;
        memcpy(&bits, &f, 4);
        b.program.push_back(2);
        b.program.push_back(bits);
        return true;
      }
      case Expression::ConstF32: b.program.push_back(2); b.program.push_back(e.f32_bits); return true;
      case Expression::Load: {
        const TensorAccess& s = e.access;
        if (s.indices.size() != 1 || !s.view_shape.empty()) { why = "broadcast of a non-vector"; return false; }
        const int along = axis == 1 ? 0 : 1;   // the output axis the vector follows
        if (s.indices[0] == dst.indices[along] && value(s.value).shape[0] == value(dst.value).shape[along]) {
          b.program.push_back(1u | (uint32_t(pw_operand(b, s.value, axis == 1 ? 1 : 2)) << 8));
          return true;
        }
        why = "broadcast operand does not follow the output rows or columns";
        return false;
      }
      case Expression::Add: case Expression::Sub: case Expression::Mul: case Expression::Div: case Expression::Max: {
        if (!pw_compile_vector(*e.args[0], dst, axis, b, why) || !pw_compile_vector(*e.args[1], dst, axis, b, why)) return false;
        b.program.push_back(e.kind == Expression::Add ? 16 : e.kind == Expression::Sub ? 17 : e.kind == Expression::Mul ? 18 : e.kind == Expression::Div ? 19 : 20);
        return true;
      }
      case Expression::Sqr: case Expression::Sqrt: case Expression::Sigmoid: case Expression::Relu: case Expression::Exp: {
        if (!pw_compile_vector(*e.args[0], dst, axis, b, why)) return false;
        b.program.push_back(e.kind == Expression::Sqr ? 32 : e.kind == Expression::Sqrt ? 33 : e.kind == Expression::Sigmoid ? 34 : e.kind == Expression::Relu ? 35 : 36);
        return true;
      }
      default:
        why = "broadcast of an expression that is not pointwise over vectors";
        return false;
    }
  }

  bool pw_compile(const Expression& e, const TensorAccess& dst, PwBuild& b, std::string& why) {
    auto constant = [&](float f) {
      uint32_t bits;
      memcpy(&bits, &f, 4);
      b.program.push_back(2);
      b.program.push_back(bits);
    };
    switch (e.kind) {
      case Expression::ConstInt: constant(float(e.integer)); return true;
      case Expression::ConstF32: b.program.push_back(2); b.program.push_back(e.f32_bits); return true;
      case Expression::Load:
        if (!(e.access.indices == dst.indices) || e.access.view_shape != dst.view_shape ||
            value(e.access.value).shape != value(dst.value).shape) { why = "operand access differs from the output access"; return false; }
        b.program.push_back(1u | (uint32_t(pw_operand(b, e.access.value, 0)) << 8));
        return true;
      case Expression::Broadcast: {
        if (dst.indices.size() != 2 || (e.axis != 0 && e.axis != 1)) { why = "broadcast of a non-vector"; return false; }
        return pw_compile_vector(*e.args[0], dst, e.axis, b, why);
      }
      case Expression::Add: case Expression::Sub: case Expression::Mul: case Expression::Div: case Expression::Max: {
        if (!pw_compile(*e.args[0], dst, b, why) || !pw_compile(*e.args[1], dst, b, why)) return false;
        b.program.push_back(e.kind == Expression::Add ? 16 : e.kind == Expression::Sub ? 17 : e.kind == Expression::Mul ? 18 : e.kind == Expression::Div ? 19 : 20);
        return true;
      }
      case Expression::Sqr: case Expression::Sqrt: case Expression::Sigmoid: case Expression::Relu: case Expression::Exp: {
        if (!pw_compile(*e.args[0], dst, b, why)) return false;
        b.program.push_back(e.kind == Expression::Sqr ? 32 : e.kind == Expression::Sqrt ? 33 : e.kind == Expression::Sigmoid ? 34 : e.kind == Expression::Relu ? 35 : 36);
        return true;
      }
      default:
        why = "operator is not pointwise";
        return false;
    }
  }

  // Checks that `access` tiles its value rectangularly under `loops`; FullTile axes need no loop.
  bool check_tiled_output(const TensorAccess& access, const std::vector<LoopInfo>& loops, std::string& why) {
    const auto& shape = access.view_shape.empty() ? value(access.value).shape : access.view_shape;
    std::set<std::string> used;
    for (size_t axis = 0; axis < access.indices.size(); ++axis) {
      const AccessIndex& i = access.indices[axis];
      if (i.kind == AccessIndex::FullTile) continue;
      if (i.kind != AccessIndex::Elem && i.width.symbolic) { why = "symbolic tile width; bind_symbols first"; return false; }
      const LoopInfo* l = find_loop(loops, i.variable);
      if (!l) { why = "index variable is not an enclosing parallel loop"; return false; }
      check_parallel_axis(i, *l, shape[axis], "pointwise axis");
      used.insert(i.variable);
    }
    for (auto& l : loops)
      if (!used.count(l.variable)) invalid_execution("overlap between CTAs: parallel loop " + l.variable + " does not index the output");
    return true;
  }

  bool try_pointwise(const Statement& top) {
    std::vector<LoopInfo> loops;
    const Statement* leaf = &top;
    if (top.is_loop) {
      const std::vector<Statement>* body = strip_parallel(top, loops);
      if (!body || body->size() != 1 || (*body)[0].is_loop) return false;
      leaf = &(*body)[0];
    }
    const Operation& op = plan.operations[leaf->operation];
    const Expression& e = *op.expression;
    if (e.kind != Expression::Store) return false;
    const Value& out = value(e.access.value);
    if (out.storage == Storage::Register || out.shape.size() > 2 || !e.access.view_shape.empty()) return false;
    std::string why;
    if (!check_tiled_output(e.access, loops, why)) { rejections.push_back("sm100.pointwise: " + why); return false; }
    PwBuild b;
    if (!pw_compile(*e.args[0], e.access, b, why)) { rejections.push_back("sm100.pointwise: " + why); return false; }
    if (b.operands.size() > 4 || b.program.size() > 32) { rejections.push_back("sm100.pointwise: expression too large"); return false; }
    if (out.dtype == DType::Fp16) return false;
    std::ostringstream c;
    c << "  {\n    trinity_sm100_pointwise_args p = {};\n";
    for (size_t i = 0; i < b.operands.size(); ++i) {
      const Value& v = value(b.operands[i].first);
      if (v.dtype == DType::Fp16) return false;
      c << "    p.operands[" << i << "].data = " << slot_ptr(slot(b.operands[i].first)) << "; p.operands[" << i
        << "].dtype = " << dt_enum(v.dtype) << "; p.operands[" << i << "].broadcast = " << b.operands[i].second << ";\n";
    }
    c << "    p.operand_count = " << b.operands.size() << ";\n    p.out = " << slot_ptr(slot(e.access.value))
      << "; p.out_dtype = " << dt_enum(out.dtype) << ";\n";
    const int64_t rows = out.shape.size() == 2 ? out.shape[0] : 1, cols = out.shape.back();
    c << "    p.rows = " << rows << "; p.cols = " << cols << ";\n    p.program_length = " << b.program.size() << ";\n";
    c << "    static const uint32_t program[] = {";
    for (size_t i = 0; i < b.program.size(); ++i) c << (i ? ", " : "") << b.program[i] << "u";
    c << "};\n    for (int i = 0; i < " << b.program.size() << "; ++i) p.program[i] = program[i];\n";
    c << "    rc = trinity_sm100_pointwise(&p, stream);\n  }\n";
    Launch l;
    l.kernel = "trinity_sm100_pointwise";
    l.code = c.str();
    l.operations = {leaf->operation};
    l.block_threads = 256;
    launches.push_back(std::move(l));
    return true;
  }

  // ------------------------------------------------------------------ row reduce-sum statement
  bool try_row_reduce(const Statement& top) {
    std::vector<LoopInfo> loops;
    // Either one parallel row loop around the reduction loop, or the reduction loop alone with
    // all rows taken at once (`fulltile`, as the reference's feed-forward IR writes it).
    const bool whole = top.is_loop && top.kind == LoopKind::Sequential;
    const std::vector<Statement>* body = whole ? nullptr : strip_parallel(top, loops);
    if (!whole && (!body || loops.size() != 1 || body->size() != 1)) return false;
    const Statement& k = whole ? top : (*body)[0];
    LoopInfo kl;
    if (!k.is_loop || k.kind != LoopKind::Sequential || k.body.size() != 1 || k.body[0].is_loop || !constant_loop(k, kl))
      return false;
    const Operation& op = plan.operations[k.body[0].operation];
    const Expression& e = *op.expression;
    if (e.kind != Expression::Store || e.args[0]->kind != Expression::Add) return false;
    const Expression& sum = *e.args[0];
    if (sum.args[0]->kind != Expression::Load || !same_access(sum.args[0]->access, e.access) ||
        sum.args[1]->kind != Expression::ReduceSum || sum.args[1]->axis != 1)
      return false;
    const Expression* inner = sum.args[1]->args[0].get();
    bool square = false;
    if (inner->kind == Expression::Sqr) { square = true; inner = inner->args[0].get(); }
    if (inner->kind != Expression::Load) return false;
    const TensorAccess& X = inner->access;
    const TensorAccess& Y = e.access;
    const Value &vx = value(X.value), &vy = value(Y.value);
    if (vx.shape.size() != 2 || vy.shape.size() != 1 || vy.shape[0] != vx.shape[0] || vy.dtype != DType::Fp32 ||
        vy.storage == Storage::Register || vx.dtype == DType::Fp16)
      return false;
    if ((Y.indices[0].kind == AccessIndex::FullTile) != whole || X.indices[0] != Y.indices[0] ||
        X.indices[1].kind == AccessIndex::FullTile || X.indices[1].variable != kl.variable || X.indices[1].width.symbolic)
      return false;
    if (!whole) check_parallel_axis(Y.indices[0], loops[0], vy.shape[0], "reduce rows");
    const int64_t wk = X.indices[1].width.constant;
    if (kl.start != 0 || kl.step != wk || kl.stop < vx.shape[1])
      invalid_execution("reduce_sum: the reduction loop must cover the row in steps of its tile width");
    std::ostringstream c;
    c << "  rc = trinity_sm100_row_reduce_sum(" << slot_ptr(slot(X.value)) << ", " << dt_enum(vx.dtype) << ", "
      << slot_ptr(slot(Y.value)) << ", " << vx.shape[0] << ", " << vx.shape[1] << ", " << (square ? 1 : 0) << ", stream);\n";
    Launch l;
    l.kernel = "trinity_sm100_row_reduce_sum";
    l.code = c.str();
    l.operations = {k.body[0].operation};
    l.block_threads = 256;
    launches.push_back(std::move(l));
    return true;
  }

  // ------------------------------------------------------------------ fused row regions
  // Both regions are spelled one way only; the recogniser rebuilds the canonical text of every
  // operation from the values it found and compares.
  static std::string acc1(int v, const std::string& row) { return "(access v" + std::to_string(v) + " (tile " + row + " 1))"; }
  static std::string acc2(int v, const std::string& row, const std::string& col) {
    return "(access v" + std::to_string(v) + " (tile " + row + " 1) " + col + ")";
  }

  bool try_rmsnorm(const Statement& top) {
    LoopInfo row;
    if (!top.is_loop || top.kind != LoopKind::Parallel || !constant_loop(top, row) || top.body.size() != 2) return false;
    const Statement &k = top.body[0], &c = top.body[1];
    LoopInfo kl, cl;
    if (!k.is_loop || k.kind != LoopKind::Sequential || k.body.size() != 1 || k.body[0].is_loop || !constant_loop(k, kl)) return false;
    if (!c.is_loop || c.kind != LoopKind::Parallel || c.body.size() != 1 || c.body[0].is_loop || !constant_loop(c, cl)) return false;
    const Operation& reduce = plan.operations[k.body[0].operation];
    const Operation& norm = plan.operations[c.body[0].operation];
    if (reduce.expression->kind != Expression::Store || norm.expression->kind != Expression::Store) return false;
    const int ss = reduce.expression->access.value, y = norm.expression->access.value;
    if (reduce.inflows.size() != 1) return false;
    const int x = reduce.inflows[0];
    const Value &vx = value(x), &vss = value(ss), &vy = value(y);
    if (vx.shape.size() != 2 || vx.dtype != DType::Bf16 || vy.dtype != DType::Bf16 || vy.shape != vx.shape ||
        vss.storage != Storage::Register || vss.dtype != DType::Fp32 || vy.storage == Storage::Register)
      return false;
    const int64_t rows = vx.shape[0], cols = vx.shape[1];
    const std::string r = row.variable;
    const std::string ktile = "(clipped_tile " + kl.variable + " " + std::to_string(kl.step) + ")";
    const std::string ctile = "(clipped_tile " + cl.variable + " " + std::to_string(cl.step) + ")";
    const std::string expect_reduce = "(store " + acc1(ss, r) + " (+ (load " + acc1(ss, r) + ") (rsum (sqr (load " +
                                      acc2(x, r, ktile) + ")) 1)))";
    if (reduce.expression->text() != expect_reduce) return false;
    // y = x / bcast(sqrt(ss / cols [+ eps]), 1) [* bcast(g, 0)]
    int gain = -1;
    for (int v : norm.inflows)
      if (v != x && v != ss) gain = v;
    float eps = 0.0f;
    bool matched = false;
    uint32_t colbits;
    const float colsf = float(cols);
    memcpy(&colbits, &colsf, 4);
    // the divisor may be written as an integer, or as float_bits of the same value
    const std::string divisors[2] = {std::to_string(cols), "(float_bits " + std::to_string(colbits) + ")"};
    std::vector<const Expression*> consts;
    std::function<void(const Expression&)> find_consts = [&](const Expression& e) {
      if (e.kind == Expression::ConstF32) consts.push_back(&e);
      for (auto& a : e.args) find_consts(*a);
    };
    find_consts(*norm.expression);
    for (const std::string& div : divisors) {
      for (int with_eps = 0; with_eps < 2 && !matched; ++with_eps) {
        std::string mean = "(/ (load " + acc1(ss, r) + ") " + div + ")";
        if (with_eps) {
          // eps is whichever FP32 constant is present that is not the divisor
          const Expression* e = nullptr;
          for (auto* k2 : consts)
            if ("(float_bits " + std::to_string(k2->f32_bits) + ")" != div) e = k2;
          if (!e) continue;
          mean = "(+ " + mean + " (float_bits " + std::to_string(e->f32_bits) + "))";
          memcpy(&eps, &e->f32_bits, 4);
        } else {
          eps = 0.0f;
        }
        std::string body = "(/ (load " + acc2(x, r, ctile) + ") (bcast (sqrt " + mean + ") 1))";
        if (gain >= 0) body = "(* " + body + " (bcast (load (access v" + std::to_string(gain) + " " + ctile + ")) 0))";
        matched = norm.expression->text() == "(store " + acc2(y, r, ctile) + " " + body + ")";
      }
      if (matched) break;
    }
    if (!matched) return false;
    if (gain >= 0 && (value(gain).dtype != DType::Bf16 || value(gain).shape != std::vector<int64_t>{cols})) return false;
    if (row.start != 0 || row.step != 1 || row.stop != rows) invalid_execution("rmsnorm: output region is not fully produced");
    if (kl.start != 0 || kl.stop < cols || cl.start != 0 || cl.stop < cols) invalid_execution("rmsnorm: output region is not fully produced");
    if (cols % 8 || cols > 8192) unsupported("NoProvider: sm100.rmsnorm needs cols % 8 == 0 and cols <= 8192");
    need_alignment(x, 16);
    need_alignment(y, 16);
    if (gain >= 0) need_alignment(gain, 16);
    uint32_t eps_bits;
    memcpy(&eps_bits, &eps, 4);
    std::ostringstream code;
    code << "  {\n    const uint32_t eps_bits = " << eps_bits << "u; float eps; std::memcpy(&eps, &eps_bits, 4);\n"
         << "    rc = trinity_sm100_rmsnorm_bf16(" << slot_ptr(slot(x)) << ", " << (gain >= 0 ? slot_ptr(slot(gain)) : std::string("nullptr"))
         << ", " << slot_ptr(slot(y)) << ", " << rows << ", " << cols << ", eps, stream);\n  }\n";
    Launch l;
    l.kernel = "trinity_sm100_rmsnorm_bf16";
    l.code = code.str();
    l.operations = {k.body[0].operation, c.body[0].operation};
    l.block_threads = 256;
    launches.push_back(std::move(l));
    return true;
  }

  bool try_softmax(const Statement& top) {
    LoopInfo row;
    if (!top.is_loop || top.kind != LoopKind::Parallel || !constant_loop(top, row) || top.body.size() != 4) return false;
    for (auto& s : top.body)
      if (s.is_loop) return false;
    const Operation* ops[4];
    for (int i = 0; i < 4; ++i) ops[i] = &plan.operations[top.body[i].operation];
    for (auto* o : ops)
      if (o->expression->kind != Expression::Store) return false;
    if (ops[0]->inflows.size() != 1) return false;
    const int x = ops[0]->inflows[0];
    const int m = ops[0]->expression->access.value, e = ops[1]->expression->access.value,
              s = ops[2]->expression->access.value, y = ops[3]->expression->access.value;
    const Value &vx = value(x), &vy = value(y);
    if (vx.shape.size() != 2 || vx.dtype != DType::Bf16 || vy.dtype != DType::Bf16 || vy.shape != vx.shape) return false;
    for (int v : {m, e, s})
      if (value(v).storage != Storage::Register || value(v).dtype != DType::Fp32) return false;
    const std::string r = row.variable, full = "fulltile";
    const std::string t0 = "(store " + acc1(m, r) + " (rmax (load " + acc2(x, r, full) + ") 1))";
    const std::string t1 = "(store " + acc2(e, r, full) + " (exp (- (load " + acc2(x, r, full) + ") (bcast (load " + acc1(m, r) + ") 1))))";
    const std::string t2 = "(store " + acc1(s, r) + " (rsum (load " + acc2(e, r, full) + ") 1))";
    const std::string t3 = "(store " + acc2(y, r, full) + " (/ (load " + acc2(e, r, full) + ") (bcast (load " + acc1(s, r) + ") 1)))";
    if (ops[0]->expression->text() != t0 || ops[1]->expression->text() != t1 || ops[2]->expression->text() != t2 ||
        ops[3]->expression->text() != t3)
      return false;
    const int64_t rows = vx.shape[0], cols = vx.shape[1];
    if (row.start != 0 || row.step != 1 || row.stop != rows) invalid_execution("softmax: output region is not fully produced");
    if (cols % 8 || cols > 8192) unsupported("NoProvider: sm100.softmax needs cols % 8 == 0 and cols <= 8192");
    need_alignment(x, 16);
    need_alignment(y, 16);
    std::ostringstream code;
    code << "  rc = trinity_sm100_softmax_bf16(" << slot_ptr(slot(x)) << ", " << slot_ptr(slot(y)) << ", " << rows << ", " << cols
         << ", stream);\n";
    Launch l;
    l.kernel = "trinity_sm100_softmax_bf16";
    l.code = code.str();
    for (auto& st : top.body) l.operations.push_back(st.operation);
    l.block_threads = 256;
    launches.push_back(std::move(l));
    return true;
  }

  // ------------------------------------------------------------------ MLA decode region
  // ploop b { S = (q[b] @ transpose(cache[b])) * scale ; m = rmax S ; E = exp(S - bcast m) ;
  //           l = rsum E ; P = E / bcast l ; sloop v(0,512,512) { O[b] = O[b] + P @ cache[b][:, v-tile] } }
  bool try_mla(const Statement& top) {
    LoopInfo batch;
    if (!top.is_loop || top.kind != LoopKind::Parallel || !constant_loop(top, batch) || top.body.size() != 6) return false;
    for (int i = 0; i < 5; ++i)
      if (top.body[i].is_loop) return false;
    const Statement& vloop = top.body[5];
    LoopInfo vl;
    if (!vloop.is_loop || vloop.kind != LoopKind::Sequential || vloop.body.size() != 1 || vloop.body[0].is_loop || !constant_loop(vloop, vl))
      return false;
    const Operation* ops[6];
    for (int i = 0; i < 5; ++i) ops[i] = &plan.operations[top.body[i].operation];
    ops[5] = &plan.operations[vloop.body[0].operation];
    for (auto* o : ops)
      if (o->expression->kind != Expression::Store) return false;
    if (ops[0]->inflows.size() != 2) return false;
    const int q = ops[0]->inflows[0], cache = ops[0]->inflows[1];
    const int S = ops[0]->expression->access.value, m = ops[1]->expression->access.value,
              E = ops[2]->expression->access.value, l = ops[3]->expression->access.value,
              P = ops[4]->expression->access.value, O = ops[5]->expression->access.value;
    const Value &vq = value(q), &vc = value(cache), &vo = value(O);
    if (vq.shape.size() != 3 || vc.shape.size() != 3 || vo.shape.size() != 3) return false;
    if (vq.dtype != DType::Bf16 || vc.dtype != DType::Bf16 || vo.dtype != DType::Bf16) return false;
    const int64_t B = vq.shape[0], H = vq.shape[1], D = vq.shape[2], Sq = vc.shape[1], Dv = vo.shape[2];
    if (vc.shape[0] != B || vc.shape[2] != D || vo.shape[0] != B || vo.shape[1] != H) return false;
    const std::string b = batch.variable, v = vl.variable;
    auto a3 = [&](int val, const std::string& last) {
      return "(access v" + std::to_string(val) + " (elem " + b + ") fulltile " + last + ")";
    };
    auto a2 = [&](int val) { return "(access v" + std::to_string(val) + " (elem " + b + ") fulltile)"; };
    const Expression& scale_mul = *ops[0]->expression->args[0];
    if (scale_mul.kind != Expression::Mul || scale_mul.args[1]->kind != Expression::ConstF32) return false;
    const uint32_t scale_bits = scale_mul.args[1]->f32_bits;
    const std::string t0 = "(store " + a3(S, "fulltile") + " (* (@ (load " + a3(q, "fulltile") + ") (transpose (load " +
                           a3(cache, "fulltile") + "))) (float_bits " + std::to_string(scale_bits) + ")))";
    const std::string t1 = "(store " + a2(m) + " (rmax (load " + a3(S, "fulltile") + ") 2))";
    const std::string t2 = "(store " + a3(E, "fulltile") + " (exp (- (load " + a3(S, "fulltile") + ") (bcast (load " + a2(m) + ") 2))))";
    const std::string t3 = "(store " + a2(l) + " (rsum (load " + a3(E, "fulltile") + ") 2))";
    const std::string t4 = "(store " + a3(P, "fulltile") + " (/ (load " + a3(E, "fulltile") + ") (bcast (load " + a2(l) + ") 2)))";
    const std::string vt = "(tile " + v + " " + std::to_string(Dv) + ")";
    const std::string t5 = "(store " + a3(O, "fulltile") + " (+ (load " + a3(O, "fulltile") + ") (@ (load " + a3(P, "fulltile") +
                           ") (load " + a3(cache, vt) + "))))";
    const std::string got[6] = {ops[0]->expression->text(), ops[1]->expression->text(), ops[2]->expression->text(),
                                ops[3]->expression->text(), ops[4]->expression->text(), ops[5]->expression->text()};
    const std::string want[6] = {t0, t1, t2, t3, t4, t5};
    for (int i = 0; i < 6; ++i)
      if (got[i] != want[i]) return false;
    for (int r : {S, m, E, l, P})
      if (value(r).storage != Storage::Register) return false;
    if (batch.start != 0 || batch.step != 1 || batch.stop != B || vl.start != 0 || vl.stop != Dv || vl.step != Dv)
      invalid_execution("mla: output region is not fully produced");
    if (D != 576 || Dv != 512 || H > 128) unsupported("NoProvider: sm100.mla_decode is built for d_qk 576, d_v 512, up to 128 heads");
    need_alignment(q, 16);
    need_alignment(cache, 16);
    need_alignment(O, 16);
    std::ostringstream code;
    code << "  {\n    trinity_sm100_mla a = {};\n    a.q = " << slot_ptr(slot(q)) << "; a.cache = " << slot_ptr(slot(cache))
         << "; a.out = " << slot_ptr(slot(O)) << ";\n    a.batch = " << B << "; a.heads = " << H << "; a.seq = " << Sq
         << "; a.d_qk = " << D << "; a.d_v = " << Dv << ";\n    a.kv_splits = 0;\n"
         << "    const uint32_t scale_bits = " << scale_bits << "u; std::memcpy(&a.scale, &scale_bits, 4);\n"
         << "    rc = trinity_sm100_mla_decode_bf16_noalloc(&a, stream);\n  }\n";
    Launch launch;
    launch.kernel = "trinity_sm100_mla_decode_bf16_noalloc";
    launch.code = code.str();
    for (int i = 0; i < 5; ++i) launch.operations.push_back(top.body[i].operation);
    launch.operations.push_back(vloop.body[0].operation);
    launch.shared_memory_bytes = 216576;   // four cache stages, four exchange tiles, barriers
    launch.block_threads = 480;            // producer, two MMA issuers, twelve softmax warps
    launches.push_back(std::move(launch));
    return true;
  }

  // ------------------------------------------------------------------ all-gather (multi-GPU plans)
  // ploop row { ploop col { (all_gather X[tile row, tile col] Y[tile row, tile col] axis) } } with
  // X [R, C] on every rank and Y [R * world, C] (axis 0) or [R, C * world] (axis 1): one launch
  // of the peer-memory all-gather.  X becomes a symmetric buffer (every rank's copy mapped
  // everywhere) and the artifact a persistent one whose workspace holds the peer table.
  bool try_all_gather(const Statement& top) {
    std::vector<LoopInfo> loops;
    const Statement* leaf = &top;
    if (top.is_loop) {
      const std::vector<Statement>* body = strip_parallel(top, loops);
      if (!body || body->size() != 1 || (*body)[0].is_loop) return false;
      leaf = &(*body)[0];
    }
    const Operation& op = plan.operations[leaf->operation];
    const Expression& e = *op.expression;
    if (e.kind != Expression::AllGather) return false;
    const Value &x = value(e.source.value), &y = value(e.access.value);
    auto decline = [&](const std::string& why) { rejections.push_back("sm100.all_gather: " + why); return false; };
    if (x.dtype != DType::Bf16 || y.dtype != DType::Bf16) return decline("shards must be bf16");
    if (x.shape.size() != 2 || y.shape.size() != 2 || (e.axis != 0 && e.axis != 1)) return decline("rank-2 shards along axis 0 or 1");
    const int64_t rows = x.shape[0], cols = x.shape[1];
    if (y.shape[e.axis] != x.shape[e.axis] * plan.world_size || y.shape[1 - e.axis] != x.shape[1 - e.axis])
      return decline("destination must be the shard extent times the world size along the axis");
    if (cols % 8) return decline("shard rows must be multiples of 16 bytes");
    if (x.storage != Storage::External) return decline("the shard must be an external (bound) value");
    if (!e.source.view_shape.empty() || !e.access.view_shape.empty()) return decline("views are not gathered");
    // the tile loops must walk the whole shard exactly once
    for (int axis = 0; axis < 2; ++axis) {
      const AccessIndex& index = e.source.indices[axis];
      if (index != e.access.indices[axis]) return decline("source and destination must be indexed alike");
      if (index.kind == AccessIndex::FullTile) continue;
      const LoopInfo* loop = find_loop(loops, index.variable);
      if (!loop) return decline("index variable " + index.variable + " is not a parallel loop of the region");
      check_parallel_axis(index, *loop, x.shape[axis], "all_gather");
    }
    buffers[slot(e.source.value)].symmetric = true;
    need_alignment(e.source.value, 16);
    need_alignment(e.access.value, 16);
    int symmetric_index = 0;
    for (int b = 0; b < slot(e.source.value); ++b)
      if (buffers[b].symmetric) ++symmetric_index;
    Launch launch;
    launch.kernel = "trinity_sm100_allgather_bf16";
    std::ostringstream c;
    c << "  rc = trinity_sm100_allgather_bf16(workspace, " << symmetric_index << ", " << slot_ptr(slot(e.access.value)) << ", "
      << rows << ", " << cols << ", " << e.axis << ", " << plan.world_size << ", stream);\n";
    launch.code = c.str();
    launch.operations.push_back(leaf->operation);
    launch.block_threads = 512;
    launches.push_back(std::move(launch));
    return true;
  }

  // ------------------------------------------------------------------ row-parallel GEMM + all-reduce
  // ploop m { ploop n { sloop k { acc += A[m,k] @ B[k,n] } ; (all_reduce acc[m,n] Y[m,n]) } } with
  // a register accumulator: every rank multiplies its own K shard and the partial products are
  // summed across the GPUs inside the GEMM's epilogue.  Y becomes a symmetric buffer, the flag pad
  // of the reduction lives in the workspace behind the peer table.
  size_t workspace_bytes = 0;
  bool try_gemm_all_reduce(const Statement& top) {
    std::vector<LoopInfo> parallel;
    const std::vector<Statement>* body = strip_parallel(top, parallel);
    if (!body || parallel.empty() || body->size() != 2 || !(*body)[0].is_loop || (*body)[1].is_loop) return false;
    const Operation& reduce = plan.operations[(*body)[1].operation];
    if (reduce.expression->kind != Expression::AllReduce) return false;
    auto decline = [&](const std::string& why) { rejections.push_back("sm100.gemm_all_reduce: " + why); return false; };
    Accumulator a;
    std::string why;
    if (!match_accumulate((*body)[0], parallel, a, why)) return decline(why);
    const Expression& e = *reduce.expression;
    if (!(e.source == a.acc_access)) return decline("the reduced value must be the accumulator at its own coordinates");
    if (!(e.access.indices == a.acc_access.indices) || !e.access.view_shape.empty())
      return decline("the destination must be written at the accumulator's coordinates");
    const Value &vacc = value(a.acc), &vy = value(e.access.value);
    if (vacc.storage != Storage::Register) return decline("the accumulator must be a register value");
    if (vy.dtype != DType::Bf16 || vy.shape != vacc.shape) return decline("the destination must be a bf16 matrix of the accumulator's shape");
    if (vy.storage != Storage::External) return decline("the destination must be an external (bound) value");
    buffers[slot(e.access.value)].symmetric = true;
    need_alignment(a.a, 16);
    need_alignment(a.b, 16);
    need_alignment(e.access.value, 16);
    int symmetric_index = 0;
    for (int b = 0; b < slot(e.access.value); ++b)
      if (buffers[b].symmetric) ++symmetric_index;
    // trinity_sm100_gemm_allreduce_workspace_bytes(m, n, world): table + flag pad
    const size_t tiles = (size_t((a.m + 127) / 128) + 1) / 2 * 2 * size_t((a.n + 255) / 256);
    workspace_bytes = std::max(workspace_bytes, size_t(1024) + 4 * (64 + tiles * size_t(plan.world_size) + 16));
    std::ostringstream c;
    c << "  {\n    trinity_sm100_gemm g = {};\n";
    c << "    g.a = " << slot_ptr(slot(a.a)) << ";\n    g.b = " << slot_ptr(slot(a.b)) << ";\n";
    c << "    g.out = " << slot_ptr(slot(e.access.value)) << ";\n";
    c << "    g.m = " << a.m << "; g.n = " << a.n << "; g.k = " << a.k << ";\n";
    c << "    g.lda = " << a.k << "; g.ldb = " << a.n << "; g.ldo = " << a.n << ";\n";
    c << "    g.activation = 0;\n    g.out_dtype = TRINITY_SM100_BF16;\n";
    c << "    rc = trinity_sm100_gemm_allreduce_workspace_bf16(&g, workspace, launch_args->workspace_bytes, " << symmetric_index
      << ", stream);\n  }\n";
    Launch l;
    l.kernel = "trinity_sm100_gemm_allreduce_workspace_bf16";
    l.code = c.str();
    l.operations = {a.op, (*body)[1].operation};
    l.shared_memory_bytes = 230656;
    l.block_threads = 352;   // producer, issuer, four epilogue, four reducer warps, one signalling warp
    launches.push_back(std::move(l));
    return true;
  }

  void run() {
    check_plan();
    build_buffers();
    if (plan.world_size != 1) {
      // A multi-GPU plan becomes a persistent artifact; what it may contain today is the
      // rank-major all-gather (the reference's own emitter refuses every multi-GPU plan,
      // src/emit/native/mod.rs:161-165).
      for (auto& s : plan.statements) {
        rejections.clear();
        if (try_all_gather(s) || try_gemm_all_reduce(s)) continue;
        std::string reasons;
        for (auto& r : rejections) reasons += (reasons.empty() ? "" : "; ") + r;
        unsupported("UnsupportedExecution: Persistent emission covers all_gather and GEMM + all_reduce plans only" +
                    (reasons.empty() ? std::string() : " (" + reasons + ")"));
      }
      return;
    }
    for (auto& s : plan.statements) {
      rejections.clear();
      if (try_gemm(s) || try_rmsnorm(s) || try_softmax(s) || try_mla(s) || try_row_reduce(s) || try_pointwise(s)) continue;
      std::vector<int> ops;
      s.operations(ops);
      std::string reasons;
      for (auto& r : rejections) reasons += (reasons.empty() ? "" : "; ") + r;
      unsupported("NoProvider: no sm100 kernel for operation " + std::to_string(ops.empty() ? -1 : ops[0]) +
                  (reasons.empty() ? "" : " (" + reasons + ")"));
    }
  }

  // Candidate discovery (src/emit/candidate.rs:107-207): every recogniser is offered every
  // top-level statement, nothing is selected.  An operation gets, per recogniser, either the
  // launch that would cover it or the recogniser's reason for declining.
  struct Offer {
    std::string provider;
    bool matched = false;
    std::vector<Launch> launches;   // when matched
    std::string reason;             // when not
  };
  void check_plan() {
    if (plan.world_size < 1 || plan.world_size > 8)
      unsupported("UnsupportedExecution: Persistent emission serves worlds of up to 8 GPUs in one NVLink domain");
    if (!plan.symbols().empty())
      throw PlanError(ErrorKind::Value, "InvalidExecution: plan has unbound symbols; call bind_symbols first");
    for (auto& v : plan.values)
      if (v.dtype == DType::Fp16) unsupported("UnsupportedExecution: fp16 values are not supported by the native provider");
    if (plan.outputs.size() != 1) unsupported("UnsupportedExecution: native CUDA ABI requires one output");
  }
  std::vector<Offer> offers(const Statement& s) {
    using Recogniser = bool (Emitter::*)(const Statement&);
    const std::pair<const char*, Recogniser> recognisers[] = {
        {"sm100.gemm", &Emitter::try_gemm},         {"sm100.rmsnorm", &Emitter::try_rmsnorm},
        {"sm100.softmax", &Emitter::try_softmax},   {"sm100.mla_decode", &Emitter::try_mla},
        {"sm100.row_reduce", &Emitter::try_row_reduce}, {"sm100.pointwise", &Emitter::try_pointwise},
        {"sm100.all_gather", &Emitter::try_all_gather}, {"sm100.gemm_all_reduce", &Emitter::try_gemm_all_reduce}};
    std::vector<Offer> result;
    for (auto& [name, recogniser] : recognisers) {
      Offer offer;
      offer.provider = name;
      const size_t before = launches.size();
      rejections.clear();
      const bool collective = recogniser == &Emitter::try_all_gather || recogniser == &Emitter::try_gemm_all_reduce;
      if (collective != (plan.world_size != 1)) {
        // single-GPU kernels serve streamed plans, the collectives serve multi-GPU plans
        offer.reason = collective ? "collectives need a multi-GPU plan"
                                  : "UnsupportedExecution: Persistent emission covers all_gather and GEMM + all_reduce plans only";
        result.push_back(std::move(offer));
        continue;
      }
      try {
        offer.matched = (this->*recogniser)(s);
      } catch (const PlanError& declined) {
        offer.matched = false;
        offer.reason = declined.what();
      }
      if (offer.matched) {
        offer.launches.assign(launches.begin() + before, launches.end());
      } else if (offer.reason.empty()) {
        for (auto& r : rejections) offer.reason += (offer.reason.empty() ? "" : "; ") + r;
        if (offer.reason.empty()) offer.reason = "no applicable implementations";
      }
      launches.resize(before);
      result.push_back(std::move(offer));
    }
    return result;
  }
};

std::string read_file(const std::string& path) {
  std::ifstream in(path);
  if (!in) throw PlanError(ErrorKind::Runtime, "cannot read " + path);
  std::ostringstream s;
  s << in.rdbuf();
  return s.str();
}

std::string requirements_json(const PhysicalPlan& plan, const std::vector<BufferRequirement>& buffers,
                              const std::vector<Launch>& launches, size_t workspace_bytes = 0) {
  std::ostringstream out;
  out << "{\"target\":\"" << target_name(Target::Sm100) << "\",\"world_size\":" << plan.world_size << ",\"buffers\":[";
  for (size_t i = 0; i < buffers.size(); ++i) {
    const auto& b = buffers[i];
    if (i) out << ",";
    out << "{\"value\":" << b.slot << ",\"input_names\":[";
    for (size_t k = 0; k < b.input_names.size(); ++k) out << (k ? "," : "") << "\"" << json_escape(b.input_names[k]) << "\"";
    out << "],\"output_name\":";
    if (b.is_output) out << "\"" << json_escape(b.output_name) << "\"";
    else out << "null";
    out << ",\"shape\":[";
    for (size_t k = 0; k < b.shape.size(); ++k) out << (k ? "," : "") << b.shape[k];
    out << "],\"dtype\":\"" << dtype_name(b.dtype) << "\",\"strides\":[";
    for (size_t k = 0; k < b.strides.size(); ++k) out << (k ? "," : "") << b.strides[k];
    out << "],\"bytes\":" << b.bytes << ",\"alignment\":" << b.alignment << ",\"external\":" << (b.external ? "true" : "false")
        << ",\"symmetric\":" << (b.symmetric ? "true" : "false") << "}";
  }
  int smem = 0, threads = 128;
  for (auto& l : launches) {
    smem = std::max(smem, l.shared_memory_bytes);
    threads = std::max(threads, l.block_threads);
  }
  // A multi-GPU artifact is persistent: its workspace (symmetric memory) starts with the peer
  // table the kernels read.  The manifest keeps the reference's field names: `nvshmem` says that
  // the artifact needs a World (here: peer-mapped symmetric memory, not NVSHMEM) and
  // `cooperative_launch` that the ranks' grids must be running at the same time.
  const bool multi = plan.world_size > 1;
  out << "],\"workspace_bytes\":" << (multi ? std::max<size_t>(1024, workspace_bytes) : 0) << ",\"workspace_alignment\":" << (multi ? 256 : 1)
      << ",\"workspace_symmetric\":" << (multi ? "true" : "false") << ",\"cooperative_launch\":" << (multi ? "true" : "false")
      << ",\"shared_memory_bytes\":" << smem << ",\"block_threads\":" << threads << ",\"nvshmem\":"
      << (multi ? "true" : "false") << ",\"nvls\":false}";
  return out.str();
}

std::string render(const std::string& requirements, const std::vector<BufferRequirement>& buffers,
                   const std::vector<Launch>& launches, bool persistent) {
  std::ostringstream c;
  c << "// Generated by the sm_100a provider: host shim over libtrinity_sm100.so (no device code here).\n"
    << "#include <cstdint>\n#include <cstring>\n\n";
  c << read_file(g_include_dir + "/trinity_abi.h") << "\n" << read_file(g_include_dir + "/trinity_sm100.h") << "\n";
  c << "namespace {\nusing namespace trinity::abi;\nconst char kRequirements[] = R\"trinity(" << requirements << ")trinity\";\n";
  c << "constexpr std::size_t kBindingCount = " << buffers.size() << ";\nconst unsigned kAlignment[kBindingCount + 1] = {";
  for (auto& b : buffers) c << b.alignment << ", ";
  c << "1};\nint prepared_device = -1;\n}  // namespace\n\n";
  c << "#define TRINITY_EXPORT extern \"C\" __attribute__((visibility(\"default\")))\n\n";
  c << "TRINITY_EXPORT Descriptor const* trinity_abi() {\n  static const Descriptor d = describe(" << (persistent ? 2 : 1)
    << ", kRequirements, sizeof(kRequirements) - 1);\n  return &d;\n}\n\n";
  c << "TRINITY_EXPORT int trinity_prepare(unsigned* maximum_workers, ErrorInfo* error) {\n"
    << "  if (!maximum_workers) return report(error, generated, -1, validate);\n"
    << "  std::int32_t device = -1;\n  const int rc = trinity_sm100_prepare_device(&device);\n"
    << "  if (rc) return report(error, runtime, rc, prepare);\n"
    << "  prepared_device = device;\n  *maximum_workers = 1;\n  return report(error, none, 0, prepare);\n}\n\n";
  c << "TRINITY_EXPORT int trinity_launch(" << (persistent ? "PersistentLaunch" : "StreamedLaunch")
    << " const* launch_args, ErrorInfo* error) {\n"
    << "  if (!launch_args || prepared_device < 0) return report(error, generated, -1, validate);\n"
    << "  std::int32_t device = -1;\n"
    << "  if (trinity_sm100_current_device(&device) || device != prepared_device) return report(error, generated, -2, validate);\n"
    << "  if (launch_args->binding_count != kBindingCount) return report(error, generated, -3, validate);\n"
    << "  void* const* bindings = launch_args->bindings;\n"
    << "  for (std::size_t i = 0; i < kBindingCount; ++i)\n"
    << "    if (!bindings[i] || reinterpret_cast<std::uintptr_t>(bindings[i]) % kAlignment[i]) return report(error, generated, -4, validate);\n"
    << "  void* stream = launch_args->stream;\n  int rc = 0;\n  (void)stream; (void)bindings;\n";
  if (persistent)
    c << "  // the workspace starts with the peer table the kernels read on the device\n"
      << "  void* workspace = launch_args->workspace;\n"
      << "  if (!workspace || launch_args->workspace_bytes < TRINITY_SM100_PEER_TABLE_BYTES ||\n"
      << "      reinterpret_cast<std::uintptr_t>(workspace) % 256 || launch_args->worker_count != 1)\n"
      << "    return report(error, generated, -4, validate);\n";
  for (size_t i = 0; i < launches.size(); ++i) {
    c << "  // launch " << i << ": " << launches[i].kernel << "\n" << launches[i].code
      << "  if (rc) return report(error, runtime, rc, launch, " << (i > 0 ? "true" : "false") << ");\n";
  }
  c << "  return report(error, none, 0, launch, " << (launches.empty() ? "false" : "true") << ");\n}\n\n";
  c << "TRINITY_EXPORT int trinity_status(" << (persistent ? "void const* workspace, " : "") << "void* stream, ErrorInfo* error) {\n"
    << (persistent ? "  (void)workspace;\n" : "")
    << "  int rc = trinity_sm100_stream_synchronize(stream);\n  if (rc) return report(error, runtime, rc, completion, true);\n"
    << "  std::uint32_t status = 0;\n  rc = trinity_sm100_device_status(&status, 0);\n"
    << "  if (rc) return report(error, runtime, rc, completion, true);\n"
    << "  if (status) return report(error, generated, TRINITY_SM100_E_TIMEOUT, completion, true);\n"
    << "  return report(error, none, 0, completion);\n}\n\n";
  c << "TRINITY_EXPORT int trinity_release(ErrorInfo* error) {\n  prepared_device = -1;\n  return report(error, none, 0, release);\n}\n";
  return c.str();
}

}  // namespace

CudaSource emit(const PhysicalPlan& plan) {
  Emitter e(plan);
  e.run();
  CudaSource source;
  source.persistent = plan.world_size > 1;
  source.requirements_json = requirements_json(plan, e.buffers, e.launches, e.workspace_bytes);
  source.code = render(source.requirements_json, e.buffers, e.launches, source.persistent);
  source.launches = std::move(e.launches);
  source.buffers = std::move(e.buffers);
  return source;
}

std::string kernel_candidates_json(const PhysicalPlan& plan) {
  std::ostringstream out;
  out << "{";
  try {
    Emitter e(plan);
    e.check_plan();
    e.build_buffers();
    bool first = true;
    for (size_t index = 0; index < plan.statements.size(); ++index) {
      const Statement& statement = plan.statements[index];
      std::vector<int> ops;
      statement.operations(ops);
      const std::vector<Emitter::Offer> offers = e.offers(statement);
      for (int op : ops) {
        out << (first ? "" : ",") << "\"" << op << "\":{\"scope\":{\"statement\":" << index << "},\"candidates\":[";
        first = false;
        bool first_candidate = true;
        for (auto& offer : offers) {
          if (!offer.matched) continue;
          for (auto& launch : offer.launches) {
            if (std::find(launch.operations.begin(), launch.operations.end(), op) == launch.operations.end()) continue;
            out << (first_candidate ? "" : ",") << "{\"provider\":\"" << offer.provider
                << "\",\"kind\":\"native\",\"kernel\":\"" << json_escape(launch.kernel) << "\",\"operations\":[";
            for (size_t i = 0; i < launch.operations.size(); ++i) out << (i ? "," : "") << launch.operations[i];
            out << "]}";
            first_candidate = false;
          }
        }
        out << "],\"rejections\":[";
        bool first_rejection = true;
        for (auto& offer : offers) {
          if (offer.matched) continue;
          out << (first_rejection ? "" : ",") << "{\"provider\":\"" << offer.provider << "\",\"reason\":\""
              << json_escape(offer.reason) << "\"}";
          first_rejection = false;
        }
        // the reference's other providers produce opaque Python candidates; they are not part of
        // this library, which is recorded the way a provider records an unsupported operation
        for (const char* absent : {"triton", "quack"})
          out << (first_rejection ? "" : ",") << "{\"provider\":\"" << absent
              << "\",\"reason\":\"provider is not part of the sm_100a library\"}", first_rejection = false;
        out << "]}";
      }
    }
  } catch (const PlanError& err) {
    out << "\"error\":\"" << json_escape(err.what()) << "\"";
  }
  out << "}";
  return out.str();
}

}  // namespace trinity::host
