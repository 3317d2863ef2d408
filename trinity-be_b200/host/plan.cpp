// Plan construction, normalisation and canonicalisation.
//
// Rules restated from the reference planner:
//  * values named in first-use order, inputs sorted by tensor name, value and operation ids
//    renumbered in first-use order, loop variables renamed lv0, lv1, ... in pre-order skipping
//    configuration symbols (src/analysis/plan/normalize.rs:9-52, :136-251)
//  * inflows are recomputed from the expression; in a sequential loop with a single operation
//    a `store(dst, load(dst) + rhs)` whose destination does not use the loop variable starts
//    from zero and `dst` is not an inflow (normalize.rs:59-133, expression.rs:366-391)
//  * boundary storage, storage scope, producer and membership checks
//    (src/analysis/plan/builder.rs:95-330)
#include "plan.hpp"

#include <algorithm>
#include <cstring>
#include <functional>
#include <sstream>

namespace trinity::host {

// ------------------------------------------------------------------ names
const char* dtype_name(DType d) { return d == DType::Fp16 ? "fp16" : d == DType::Bf16 ? "bf16" : "fp32"; }
const char* storage_name(Storage s) {
  return s == Storage::External ? "external" : s == Storage::Global ? "global" : "register";
}
const char* target_name(Target t) {
  switch (t) {
    case Target::Hopper: return "hopper";
    case Target::Sm89: return "sm89";
    case Target::Sm120: return "sm120";
    default: return "sm100";
  }
}
DType parse_dtype(const std::string& s) {
  if (s == "fp16" || s == "float16") return DType::Fp16;
  if (s == "bf16" || s == "bfloat16") return DType::Bf16;
  if (s == "fp32" || s == "float32") return DType::Fp32;
  invalid("unknown dtype " + s);
}
Storage parse_storage(const std::string& s) {
  if (s == "external") return Storage::External;
  if (s == "global") return Storage::Global;
  if (s == "register") return Storage::Register;
  invalid("unknown storage " + s);
}
Target parse_target(const std::string& s) {
  if (s == "hopper" || s == "sm90" || s == "sm_90a" || s == "sm90a") return Target::Hopper;
  if (s == "sm89" || s == "sm_89" || s == "ada") return Target::Sm89;
  if (s == "sm120" || s == "sm_120" || s == "blackwell_rtx") return Target::Sm120;
  if (s == "sm100" || s == "sm_100a" || s == "sm100a" || s == "b200" || s == "blackwell")
    return Target::Sm100;
  invalid("unknown target " + s);
}

std::string json_escape(const std::string& s) {
  std::string out;
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\t': out += "\\t"; break;
      case '\r': out += "\\r"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else {
          out += char(c);
        }
    }
  }
  return out;
}

static bool is_symbol_name(const std::string& raw) {
  std::string name = (!raw.empty() && raw[0] == '?') ? raw.substr(1) : raw;
  if (name.empty() || !(isalpha((unsigned char)name[0]) || name[0] == '_')) return false;
  for (unsigned char c : name)
    if (!(isalnum(c) || c == '_')) return false;
  return true;
}
static bool parse_int(const std::string& s, int64_t& out) {
  if (s.empty()) return false;
  char* end = nullptr;
  errno = 0;
  long long v = strtoll(s.c_str(), &end, 10);
  if (errno || *end) return false;
  out = v;
  return true;
}

// ------------------------------------------------------------------ IndexExpr
bool IndexExpr::operator==(const IndexExpr& o) const {
  return kind == o.kind && value == o.value && name == o.name && operands == o.operands;
}
void IndexExpr::rename(const std::map<std::string, std::string>& names) {
  if (kind == Variable) {
    auto it = names.find(name);
    if (it != names.end()) name = it->second;
  }
  for (auto& e : operands) e.rename(names);
}
void IndexExpr::collect_variables(std::set<std::string>& out) const {
  if (kind == Variable) out.insert(name);
  for (auto& e : operands) e.collect_variables(out);
}
IndexExpr IndexExpr::bind(const std::map<std::string, int64_t>& symbols) const {
  if (kind == Constant) return *this;
  if (kind == Variable) {
    auto it = symbols.find(name);
    return it == symbols.end() ? *this : constant(it->second);
  }
  IndexExpr l = operands[0].bind(symbols), r = operands[1].bind(symbols);
  if (l.is_constant() && r.is_constant()) {
    switch (kind) {
      case Add: return constant(l.value + r.value);
      case Sub: return constant(l.value - r.value);
      case Mul: return constant(l.value * r.value);
      case Div:
        if (r.value == 0) invalid("division by zero in index expression");
        return constant(l.value / r.value);
      default: break;
    }
  }
  IndexExpr e;
  e.kind = kind;
  e.operands = {l, r};
  return e;
}
std::string IndexExpr::json() const {
  switch (kind) {
    case Constant: return "{\"Constant\":" + std::to_string(value) + "}";
    case Variable: return "{\"Variable\":\"" + json_escape(name) + "\"}";
    default: {
      const char* tag = kind == Add ? "Add" : kind == Sub ? "Sub" : kind == Mul ? "Mul" : "Div";
      return std::string("{\"") + tag + "\":[" + operands[0].json() + "," + operands[1].json() + "]}";
    }
  }
}
static IndexExpr index_from_node(const Node& node) {
  if (node.is_atom) {
    int64_t v;
    if (parse_int(node.text, v)) return IndexExpr::constant(v);
    return IndexExpr::variable(node.text);
  }
  const auto& a = node.args(2);
  IndexExpr e;
  if (node.op() == "+") e.kind = IndexExpr::Add;
  else if (node.op() == "-") e.kind = IndexExpr::Sub;
  else if (node.op() == "*") e.kind = IndexExpr::Mul;
  else if (node.op() == "/") e.kind = IndexExpr::Div;
  else throw SyntaxError(node.offset, "unsupported index expression");
  e.operands = {index_from_node(a[0]), index_from_node(a[1])};
  return e;
}
IndexExpr parse_index(const std::string& text) {
  try {
    return index_from_node(parse_sexpr(text));
  } catch (const SyntaxError& e) {
    invalid(e.what());
  }
}

// ------------------------------------------------------------------ Expression
static const char* op_token(Expression::Kind k) {
  switch (k) {
    case Expression::Add: return "+";
    case Expression::Sub: return "-";
    case Expression::Mul: return "*";
    case Expression::Div: return "/";
    case Expression::Matmul: return "@";
    case Expression::Max: return "max";
    case Expression::Sqr: return "sqr";
    case Expression::Sqrt: return "sqrt";
    case Expression::Sigmoid: return "sigmoid";
    case Expression::Relu: return "relu";
    case Expression::Exp: return "exp";
    case Expression::Transpose: return "transpose";
    case Expression::Permute: return "permute";
    case Expression::ReduceSum: return "rsum";
    case Expression::ReduceMax: return "rmax";
    case Expression::Broadcast: return "bcast";
    case Expression::Unsqueeze: return "unsqueeze";
    default: return "?";
  }
}
static std::string access_text(const TensorAccess& a) {
  std::ostringstream s;
  s << "(access v" << a.value;
  if (!a.view_shape.empty()) {
    s << " (view";
    for (auto d : a.view_shape) s << " " << d;
    s << ")";
  }
  for (const auto& i : a.indices) {
    switch (i.kind) {
      case AccessIndex::FullTile: s << " fulltile"; break;
      case AccessIndex::Elem: s << " (elem " << i.variable << ")"; break;
      default:
        s << (i.kind == AccessIndex::Tile ? " (tile " : " (clipped_tile ") << i.variable << " "
          << (i.width.symbolic ? i.width.symbol : std::to_string(i.width.constant)) << ")";
    }
  }
  s << ")";
  return s.str();
}
bool Expression::is_pure() const {
  if (kind == Store || kind == AllGather || kind == AllReduce) return false;
  for (auto& a : args)
    if (!a->is_pure()) return false;
  return true;
}
void Expression::reads(std::vector<int>& out) const {
  if (kind == Load || kind == AllGather || kind == AllReduce) {
    const int v = kind == Load ? access.value : source.value;
    if (std::find(out.begin(), out.end(), v) == out.end()) out.push_back(v);
  }
  for (auto& a : args) a->reads(out);
}
void Expression::accesses(std::vector<TensorAccess*>& out) {
  if (kind == Load || kind == Store || kind == AllGather || kind == AllReduce) out.push_back(&access);
  if (kind == AllGather || kind == AllReduce) out.push_back(&source);
  for (auto& a : args) a->accesses(out);
}
std::string Expression::text() const {
  switch (kind) {
    case ConstInt: return std::to_string(integer);
    case ConstF32: return "(float_bits " + std::to_string(f32_bits) + ")";
    case Load: return "(load " + access_text(access) + ")";
    case Store: return "(store " + access_text(access) + " " + args[0]->text() + ")";
    case AllGather:
      return "(all_gather " + access_text(source) + " " + access_text(access) + " " +
             std::to_string(axis) + ")";
    case AllReduce: return "(all_reduce " + access_text(source) + " " + access_text(access) + ")";
    case ReduceSum: case ReduceMax: case Broadcast: case Unsqueeze:
      return std::string("(") + op_token(kind) + " " + args[0]->text() + " " + std::to_string(axis) + ")";
    case Permute: {
      std::string s = "(permute " + args[0]->text();
      for (int a : axes) s += " " + std::to_string(a);
      return s + ")";
    }
    default: {
      std::string s = std::string("(") + op_token(kind);
      for (auto& a : args) s += " " + a->text();
      return s + ")";
    }
  }
}
static ExprPtr clone_expr(const ExprPtr& e) {
  auto c = std::make_shared<Expression>(*e);
  for (auto& a : c->args) a = clone_expr(a);
  return c;
}

void Statement::operations(std::vector<int>& out) const {
  if (!is_loop) {
    out.push_back(operation);
    return;
  }
  for (auto& s : body) s.operations(out);
}

// ------------------------------------------------------------------ expression decoding
namespace {

struct Decoder {
  const std::vector<Value>& values;
  const std::map<std::string, int64_t>* symbols = nullptr;

  int64_t integer(const Node& n) const {
    int64_t v;
    if (parse_int(n.atom(), v)) return v;
    if (symbols) {
      auto it = symbols->find(n.text);
      if (it != symbols->end()) return it->second;
    }
    throw SyntaxError(n.offset, "unresolved integer or symbol " + n.text);
  }
  int axis(const Node& n) const {
    int64_t v = integer(n);
    if (v < 0) throw SyntaxError(n.offset, "axis must be nonnegative");
    return int(v);
  }
  ExprPtr unary(Expression::Kind k, const Node& n) const {
    auto e = std::make_shared<Expression>();
    e->kind = k;
    e->args = {expression(n.args(1)[0])};
    return e;
  }
  ExprPtr binary(Expression::Kind k, const Node& n) const {
    auto e = std::make_shared<Expression>();
    e->kind = k;
    const auto& a = n.args(2);
    e->args = {expression(a[0]), expression(a[1])};
    return e;
  }
  ExprPtr with_axis(Expression::Kind k, const Node& n) const {
    auto e = std::make_shared<Expression>();
    e->kind = k;
    const auto& a = n.args(2);
    e->args = {expression(a[0])};
    e->axis = axis(a[1]);
    return e;
  }
  ExprPtr expression(const Node& n) const {
    auto e = std::make_shared<Expression>();
    if (n.is_atom) {
      int64_t v;
      if (parse_int(n.text, v) || (symbols && symbols->count(n.text) && ((v = symbols->at(n.text)), true))) {
        e->kind = Expression::ConstInt;
        e->integer = v;
        return e;
      }
      char* end = nullptr;
      float f = strtof(n.text.c_str(), &end);
      if (n.text.empty() || *end) throw SyntaxError(n.offset, "invalid scalar constant");
      e->kind = Expression::ConstF32;
      memcpy(&e->f32_bits, &f, 4);
      return e;
    }
    const std::string& op = n.op();
    if (op == "load") {
      const auto& a = n.args(2);
      e->kind = Expression::Load;
      e->access = access(a[0], a[1]);
      return e;
    }
    if (op == "store") {
      const auto& a = n.args(3);
      e->kind = Expression::Store;
      e->access = access(a[0], a[2]);
      e->args = {expression(a[1])};
      return e;
    }
    if (op == "+") return binary(Expression::Add, n);
    if (op == "-") return binary(Expression::Sub, n);
    if (op == "*") return binary(Expression::Mul, n);
    if (op == "/") return binary(Expression::Div, n);
    if (op == "@") return binary(Expression::Matmul, n);
    if (op == "max") return binary(Expression::Max, n);
    if (op == "sqr") return unary(Expression::Sqr, n);
    if (op == "sqrt") return unary(Expression::Sqrt, n);
    if (op == "sigmoid") return unary(Expression::Sigmoid, n);
    if (op == "relu") return unary(Expression::Relu, n);
    if (op == "exp") return unary(Expression::Exp, n);
    if (op == "transpose") return unary(Expression::Transpose, n);
    if (op == "permute") {
      // (permute value a0 a1 ...): result axis i is source axis a_i (the reference's ValueOp::Permute,
      // src/analysis/plan/expression.rs:164-181, as its batched-MLA fixtures spell it)
      if (n.children.size() < 3) throw SyntaxError(n.offset, "'permute' expects a value and at least two axes");
      e->kind = Expression::Permute;
      e->args = {expression(n.children[0])};
      std::vector<bool> seen(n.children.size() - 1, false);
      for (size_t i = 1; i < n.children.size(); ++i) {
        const int a = axis(n.children[i]);
        if (a < 0 || a >= int(seen.size()) || seen[a]) throw SyntaxError(n.children[i].offset, "permute axes must be a permutation");
        seen[a] = true;
        e->axes.push_back(a);
      }
      return e;
    }
    if (op == "rsum") return with_axis(Expression::ReduceSum, n);
    if (op == "rmax") return with_axis(Expression::ReduceMax, n);
    if (op == "bcast") return with_axis(Expression::Broadcast, n);
    if (op == "unsqueeze") return with_axis(Expression::Unsqueeze, n);
    if (op == "float_bits") {
      int64_t bits = integer(n.args(1)[0]);
      if (bits < 0 || bits > 0xFFFFFFFFll) throw SyntaxError(n.offset, "invalid FP32 bits");
      e->kind = Expression::ConstF32;
      e->f32_bits = uint32_t(bits);
      return e;
    }
    if (op == "all_gather") {
      const auto& a = n.args(5);
      e->kind = Expression::AllGather;
      e->source = access(a[0], a[1]);
      e->access = access(a[2], a[3]);
      e->axis = axis(a[4]);
      return e;
    }
    if (op == "all_reduce") {
      const auto& a = n.args(4);
      e->kind = Expression::AllReduce;
      e->source = access(a[0], a[1]);
      e->access = access(a[2], a[3]);
      return e;
    }
    throw SyntaxError(n.offset, "unsupported operation " + op);
  }
  TileWidth tile_width(const Node& n) const {
    TileWidth w;
    int64_t v;
    if (parse_int(n.atom(), v) || (symbols && symbols->count(n.text) && ((v = symbols->at(n.text)), true))) {
      if (v <= 0) throw SyntaxError(n.offset, "extent must be positive");
      w.constant = v;
    } else if (is_symbol_name(n.text)) {
      w.symbolic = true;
      w.symbol = n.text;
    } else {
      throw SyntaxError(n.offset, "unresolved integer or symbol " + n.text);
    }
    return w;
  }
  AccessIndex access_index(const Node& n) const {
    AccessIndex i;
    if (n.op() == "tile" || n.op() == "clipped_tile") {
      const auto& a = n.args(2);
      i.kind = n.op() == "tile" ? AccessIndex::Tile : AccessIndex::ClippedTile;
      i.variable = a[0].atom();
      i.width = tile_width(a[1]);
    } else if (n.op() == "elem") {
      i.kind = AccessIndex::Elem;
      i.variable = n.args(1)[0].atom();
    } else {
      throw SyntaxError(n.offset, "unsupported access index");
    }
    return i;
  }
  TensorAccess access(const Node& view, const Node& index) const {
    if (view.is_atom || view.op() != "view" || index.is_atom || index.op() != "keyed_index")
      throw SyntaxError(view.offset, "expected view and keyed_index");
    const auto& v = view.args(2);
    if (v[0].is_atom || (v[0].op() != "input" && v[0].op() != "output" && v[0].op() != "tensor") ||
        v[1].is_atom || v[1].op() != "layout")
      throw SyntaxError(v[0].offset, "invalid tensor view");
    const std::string& name = v[0].args(1)[0].atom();
    int id = -1;
    for (size_t i = 0; i < values.size(); ++i) {
      if (values[i].name == name) {
        if (id >= 0) throw SyntaxError(v[0].offset, "ambiguous tensor " + name);
        id = int(i);
      }
    }
    if (id < 0) throw SyntaxError(v[0].offset, "unknown tensor " + name);
    std::map<std::string, const Node*> slots;
    for (const auto& slot : index.children) {
      if (slot.is_atom || slot.op() != "slot") throw SyntaxError(slot.offset, "expected index slot");
      const auto& a = slot.args(2);
      if (!slots.emplace(a[0].atom(), &a[1]).second) throw SyntaxError(slot.offset, "duplicate index slot");
    }
    TensorAccess access;
    access.value = id;
    std::set<std::string> axes;
    std::vector<int64_t> shape;
    for (const auto& axis : v[1].children) {
      if (axis.is_atom || axis.op() != "axis") throw SyntaxError(axis.offset, "expected layout axis");
      const auto& a = axis.args(2);
      if (!axes.insert(a[0].atom()).second) throw SyntaxError(axis.offset, "duplicate layout axis");
      int64_t extent = integer(a[1]);
      if (extent <= 0) throw SyntaxError(a[1].offset, "extent must be positive");
      shape.push_back(extent);
      auto it = slots.find(a[0].text);
      if (it == slots.end() || (it->second->is_atom && it->second->text == "fulltile")) {
        access.indices.push_back(AccessIndex{});
      } else {
        access.indices.push_back(access_index(*it->second));
      }
      if (it != slots.end()) slots.erase(it);
    }
    if (!slots.empty()) throw SyntaxError(index.offset, "index slot absent from view");
    if (shape != values[id].shape) access.view_shape = shape;
    int64_t count = 1, base = 1;
    for (auto d : shape) count *= d;
    for (auto d : values[id].shape) base *= d;
    if (shape.empty() || count != base)
      throw SyntaxError(v[1].offset, "view element count differs from value");
    return access;
  }
};

bool uses_variable(const TensorAccess& a, const std::string& v) {
  for (auto& i : a.indices)
    if (i.kind != AccessIndex::FullTile && i.variable == v) return true;
  return false;
}

// store(dst, load(dst) + rhs) with dst not indexed by `variable` -> rhs, else nullptr.
const Expression* accumulation_rhs(const Expression& store, const std::string& variable) {
  if (store.kind != Expression::Store) return nullptr;
  const Expression& value = *store.args[0];
  if (value.kind != Expression::Add) return nullptr;
  const Expression& left = *value.args[0];
  if (left.kind != Expression::Load) return nullptr;
  if (!(left.access == store.access) || uses_variable(store.access, variable)) return nullptr;
  return value.args[1].get();
}

void rename_expression(Expression& e, const std::map<std::string, std::string>& names) {
  std::vector<TensorAccess*> accesses;
  e.accesses(accesses);
  for (auto* a : accesses)
    for (auto& i : a->indices) {
      auto it = names.find(i.variable);
      if (i.kind != AccessIndex::FullTile && it != names.end()) i.variable = it->second;
    }
}
void remap_expression(Expression& e, const std::vector<int>& ids) {
  std::vector<TensorAccess*> accesses;
  e.accesses(accesses);
  for (auto* a : accesses) a->value = ids[a->value];
}

void statement_json(const Statement& s, std::ostringstream& out) {
  std::vector<int> ops;
  s.operations(ops);
  out << "{\"operations\":[";
  for (size_t i = 0; i < ops.size(); ++i) out << (i ? "," : "") << ops[i];
  out << "]";
  if (s.is_loop) {
    out << ",\"loop\":{\"kind\":\""
        << (s.kind == LoopKind::Parallel ? "parallel" : s.kind == LoopKind::Sequential ? "sequential" : "split")
        << "\",\"domain\":{\"variable\":\"" << json_escape(s.domain.variable) << "\",\"start\":"
        << s.domain.start.json() << ",\"stop\":" << s.domain.stop.json() << ",\"step\":"
        << s.domain.step.json() << "},\"body\":[";
    for (size_t i = 0; i < s.body.size(); ++i) {
      if (i) out << ",";
      statement_json(s.body[i], out);
    }
    out << "]}";
  }
  out << "}";
}

void statement_text(const Statement& s, const std::vector<Operation>& ops, std::ostringstream& out) {
  if (!s.is_loop) {
    out << "(op " << s.operation << " " << ops[s.operation].expression->text() << ")";
    return;
  }
  out << "(" << (s.kind == LoopKind::Parallel ? "ploop" : "sloop") << " " << s.domain.variable << " "
      << s.domain.start.json() << " " << s.domain.stop.json() << " " << s.domain.step.json();
  for (auto& b : s.body) {
    out << " ";
    statement_text(b, ops, out);
  }
  out << ")";
}

}  // namespace

ExprPtr decode_expression(const Node& node, const std::vector<Value>& values,
                          const std::map<std::string, int64_t>* symbols) {
  return Decoder{values, symbols}.expression(node);
}

// ------------------------------------------------------------------ PhysicalPlan
std::set<std::string> PhysicalPlan::symbols() const {
  std::set<std::string> out;
  std::function<void(const std::vector<Statement>&, std::set<std::string>)> visit =
      [&](const std::vector<Statement>& nodes, std::set<std::string> scope) {
        for (auto& n : nodes) {
          if (!n.is_loop) continue;
          for (const IndexExpr* e : {&n.domain.start, &n.domain.stop, &n.domain.step}) {
            std::set<std::string> vars;
            e->collect_variables(vars);
            for (auto& v : vars)
              if (!scope.count(v)) out.insert(v);
          }
          auto nested = scope;
          nested.insert(n.domain.variable);
          visit(n.body, nested);
        }
      };
  visit(statements, {});
  for (auto& op : operations) {
    std::vector<TensorAccess*> accesses;
    op.expression->accesses(accesses);
    for (auto* a : accesses)
      for (auto& i : a->indices)
        if ((i.kind == AccessIndex::Tile || i.kind == AccessIndex::ClippedTile) && i.width.symbolic)
          out.insert(i.width.symbol);
  }
  return out;
}

static PhysicalPlan canonicalize(PhysicalPlan plan);

PhysicalPlan PhysicalPlan::bind_symbols(const std::map<std::string, int64_t>& bindings) const {
  const std::set<std::string> known = symbols();
  for (auto& kv : bindings) {
    if (kv.second <= 0) invalid("symbol " + kv.first + " must be bound to a positive integer");
  }
  for (auto& s : known)
    if (!bindings.count(s)) invalid("missing binding for symbol " + s);
  PhysicalPlan plan = *this;
  for (auto& op : plan.operations) op.expression = clone_expr(op.expression);
  std::function<void(std::vector<Statement>&, std::set<std::string>)> visit =
      [&](std::vector<Statement>& nodes, std::set<std::string> scope) {
        for (auto& n : nodes) {
          if (!n.is_loop) continue;
          // loop coordinates in scope are left alone even if a binding uses their name
          std::map<std::string, int64_t> visible;
          for (auto& kv : bindings)
            if (!scope.count(kv.first)) visible.insert(kv);
          n.domain.start = n.domain.start.bind(visible);
          n.domain.stop = n.domain.stop.bind(visible);
          n.domain.step = n.domain.step.bind(visible);
          auto nested = scope;
          nested.insert(n.domain.variable);
          visit(n.body, nested);
        }
      };
  visit(plan.statements, {});
  for (auto& op : plan.operations) {
    std::vector<TensorAccess*> accesses;
    op.expression->accesses(accesses);
    for (auto* a : accesses)
      for (auto& i : a->indices)
        if ((i.kind == AccessIndex::Tile || i.kind == AccessIndex::ClippedTile) && i.width.symbolic) {
          i.width.constant = bindings.at(i.width.symbol);
          i.width.symbolic = false;
          i.width.symbol.clear();
        }
  }
  return canonicalize(std::move(plan));
}

std::string PhysicalPlan::metadata_json() const {
  std::ostringstream out;
  auto binding = [&](const Binding& b) {
    out << "{\"name\":\"" << json_escape(b.tensor) << "\",\"value\":" << b.value << "}";
  };
  out << "{\"world_size\":" << world_size << ",\"inputs\":[";
  for (size_t i = 0; i < inputs.size(); ++i) {
    if (i) out << ",";
    binding(inputs[i]);
  }
  out << "],\"output\":";
  if (outputs.empty()) out << "null";
  else binding(outputs[0]);
  out << ",\"outputs\":[";
  for (size_t i = 0; i < outputs.size(); ++i) {
    if (i) out << ",";
    binding(outputs[i]);
  }
  out << "],\"mutable_inputs\":[],\"values\":[";
  for (size_t i = 0; i < values.size(); ++i) {
    if (i) out << ",";
    out << "{\"value\":" << i << ",\"dtype\":\"" << dtype_name(values[i].dtype) << "\",\"shape\":[";
    for (size_t d = 0; d < values[i].shape.size(); ++d) out << (d ? "," : "") << values[i].shape[d];
    out << "],\"storage\":\"" << storage_name(values[i].storage) << "\"}";
  }
  out << "],\"operations\":[";
  for (size_t i = 0; i < operations.size(); ++i) {
    if (i) out << ",";
    out << "{\"id\":" << i << ",\"inflows\":[";
    for (size_t k = 0; k < operations[i].inflows.size(); ++k) out << (k ? "," : "") << operations[i].inflows[k];
    out << "],\"outflows\":[";
    for (size_t k = 0; k < operations[i].outflows.size(); ++k) out << (k ? "," : "") << operations[i].outflows[k];
    out << "]}";
  }
  out << "],\"statements\":[";
  for (size_t i = 0; i < statements.size(); ++i) {
    if (i) out << ",";
    statement_json(statements[i], out);
  }
  out << "]}";
  return out.str();
}

std::string PhysicalPlan::structure_text() const {
  std::ostringstream out;
  out << target_name(target) << " world " << world_size << " inputs";
  for (auto& b : inputs) out << " " << b.tensor << "=" << b.value;
  out << " outputs";
  for (auto& b : outputs) out << " " << b.tensor << "=" << b.value;
  out << " values";
  for (auto& v : values) {
    out << " (" << dtype_name(v.dtype) << " " << storage_name(v.storage);
    for (auto d : v.shape) out << " " << d;
    out << ")";
  }
  out << " body";
  for (auto& s : statements) {
    out << " ";
    statement_text(s, operations, out);
  }
  return out.str();
}

uint64_t PhysicalPlan::hash() const {
  // FNV-1a over the canonical text; process-independent, unlike the reference's SipHash,
  // which it documents as process-local (src/analysis/plan/mod.rs:305-309).
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : structure_text()) {
    h ^= c;
    h *= 1099511628211ull;
  }
  return h;
}

static PhysicalPlan canonicalize(PhysicalPlan plan) {
  const std::set<std::string> symbols = plan.symbols();
  std::vector<int> order;
  for (auto& s : plan.statements) s.operations(order);
  std::vector<int> value_ids(plan.values.size(), -1), value_order;
  auto assign = [&](int id) {
    if (value_ids[id] < 0) {
      value_ids[id] = int(value_order.size());
      value_order.push_back(id);
    }
  };
  for (auto& b : plan.inputs) assign(b.value);
  for (int id : order) {
    for (int v : plan.operations[id].inflows) assign(v);
    for (int v : plan.operations[id].outflows) assign(v);
  }
  for (size_t i = 0; i < plan.values.size(); ++i) assign(int(i));
  std::vector<int> operation_ids(plan.operations.size(), 0);
  std::vector<Operation> operations;
  for (int id : order) {
    operation_ids[id] = int(operations.size());
    Operation op = plan.operations[id];
    op.expression = clone_expr(op.expression);
    for (auto& v : op.inflows) v = value_ids[v];
    for (auto& v : op.outflows) v = value_ids[v];
    remap_expression(*op.expression, value_ids);
    operations.push_back(std::move(op));
  }
  int next = 0;
  std::function<void(Statement&, const std::map<std::string, std::string>&)> visit =
      [&](Statement& s, const std::map<std::string, std::string>& names) {
        if (!s.is_loop) {
          s.operation = operation_ids[s.operation];
          rename_expression(*operations[s.operation].expression, names);
          return;
        }
        s.domain.start.rename(names);
        s.domain.stop.rename(names);
        s.domain.step.rename(names);
        auto nested = names;
        while (symbols.count("lv" + std::to_string(next))) ++next;
        const std::string variable = "lv" + std::to_string(next++);
        nested[s.domain.variable] = variable;
        s.domain.variable = variable;
        for (auto& b : s.body) visit(b, nested);
      };
  for (auto& s : plan.statements) visit(s, {});
  plan.operations = std::move(operations);
  std::vector<Value> values;
  for (int id : value_order) values.push_back(plan.values[id]);
  plan.values = std::move(values);
  for (auto& b : plan.inputs) b.value = value_ids[b.value];
  for (auto& b : plan.outputs) b.value = value_ids[b.value];
  return plan;
}

// ------------------------------------------------------------------ PlanBuilder
PlanBuilder::PlanBuilder(int world_size, Target target) : target_(target), world_size_(world_size) {
  if (world_size <= 0) invalid("world_size must be positive");
}
void PlanBuilder::require_open() const {
  if (finalized_) invalid("builder is finalized");
}
int PlanBuilder::add_value(DType dtype, std::vector<int64_t> shape, Storage storage, const std::string& name) {
  require_open();
  if (shape.empty()) invalid("positive shape required");
  for (auto d : shape)
    if (d <= 0) invalid("positive shape required");
  Value v{dtype, std::move(shape), storage, name.empty() ? "v" + std::to_string(values_.size()) : name};
  values_.push_back(std::move(v));
  return int(values_.size()) - 1;
}
void PlanBuilder::bind_input(const std::string& tensor, int value) {
  require_open();
  if (value < 0 || value >= int(values_.size())) invalid("unknown value");
  inputs_.push_back({tensor, value});
}
ExprPtr PlanBuilder::parse_expression(const std::string& text) const {
  try {
    return Decoder{values_}.expression(parse_sexpr(text));
  } catch (const SyntaxError& e) {
    invalid(e.what());
  }
}
int PlanBuilder::add_operation(std::vector<int> inflows, std::vector<int> outflows, const std::string& expression) {
  require_open();
  for (int v : inflows)
    if (v < 0 || v >= int(values_.size())) invalid("unknown value");
  for (int v : outflows)
    if (v < 0 || v >= int(values_.size())) invalid("unknown value");
  return add_operation_expr(std::move(inflows), std::move(outflows), parse_expression(expression));
}
int PlanBuilder::add_loop_expr(LoopKind kind, const std::string& variable, IndexExpr start, IndexExpr stop,
                               IndexExpr step, const std::vector<int>& body) {
  require_open();
  Statement s;
  s.is_loop = true;
  s.kind = kind;
  s.domain = {variable, std::move(start), std::move(stop), std::move(step)};
  for (int id : body) {
    if (id < 0 || id >= int(nodes_.size())) invalid("unknown statement");
    s.body.push_back(nodes_[id]);
  }
  nodes_.push_back(std::move(s));
  return int(nodes_.size()) - 1;
}
int PlanBuilder::add_operation_expr(std::vector<int> inflows, std::vector<int> outflows, ExprPtr expression) {
  require_open();
  for (int v : inflows)
    if (v < 0 || v >= int(values_.size())) invalid("unknown value");
  for (int v : outflows)
    if (v < 0 || v >= int(values_.size())) invalid("unknown value");
  Operation op{std::move(inflows), std::move(outflows), std::move(expression)};
  operations_.push_back(std::move(op));
  Statement s;
  s.operation = int(operations_.size()) - 1;
  nodes_.push_back(std::move(s));
  return int(nodes_.size()) - 1;
}
int PlanBuilder::add_loop(const std::string& kind, const std::string& variable, const std::string& start,
                          const std::string& stop, const std::string& step, const std::vector<int>& body) {
  require_open();
  Statement s;
  s.is_loop = true;
  if (kind == "parallel" || kind == "ploop") s.kind = LoopKind::Parallel;
  else if (kind == "sequential" || kind == "sloop") s.kind = LoopKind::Sequential;
  else invalid("expected parallel or sequential loop");
  s.domain.variable = variable;
  s.domain.start = parse_index(start);
  s.domain.stop = parse_index(stop);
  s.domain.step = parse_index(step);
  for (int id : body) {
    if (id < 0 || id >= int(nodes_.size())) invalid("unknown statement");
    s.body.push_back(nodes_[id]);
  }
  nodes_.push_back(std::move(s));
  return int(nodes_.size()) - 1;
}

PhysicalPlan PlanBuilder::build(const std::vector<int>& statement_ids, const std::string& output_tensor, int output) {
  require_open();
  if (output < 0 || output >= int(values_.size())) invalid("unknown value");
  PhysicalPlan plan;
  plan.target = target_;
  plan.world_size = world_size_;
  plan.values = values_;
  plan.operations = operations_;
  for (auto& op : plan.operations) op.expression = clone_expr(op.expression);
  for (int id : statement_ids) {
    if (id < 0 || id >= int(nodes_.size())) invalid("unknown statement");
    plan.statements.push_back(nodes_[id]);
  }
  plan.outputs.push_back({output_tensor, output});
  if (output_tensor.empty()) invalid("InvalidName: tensor names must not be empty");

  // membership: every operation belongs to exactly one statement
  std::vector<int> membership(plan.operations.size(), 0), listed;
  for (auto& s : plan.statements) s.operations(listed);
  for (int id : listed) ++membership[id];
  for (size_t i = 0; i < membership.size(); ++i) {
    if (membership[i] > 1)
      invalid("DuplicateStatementMembership: operation " + std::to_string(i) + " appears in multiple statements");
    if (membership[i] == 0)
      invalid("MissingStatementMembership: operation " + std::to_string(i) + " belongs to no statement");
  }
  // inputs
  std::set<std::string> names;
  std::set<int> input_values;
  for (auto& b : inputs_) {
    if (b.tensor.empty()) invalid("InvalidName: tensor names must not be empty");
    if (!names.insert(b.tensor).second) invalid("DuplicateInputTensor: " + b.tensor);
    input_values.insert(b.value);
  }
  for (size_t i = 0; i < plan.operations.size(); ++i) {
    auto& op = plan.operations[i];
    std::vector<TensorAccess*> accesses;
    op.expression->accesses(accesses);
    for (auto* a : accesses) {
      if (a->value < 0 || a->value >= int(plan.values.size()))
        invalid("InvalidValueId { value: " + std::to_string(a->value) + ", context: \"expression operand\" }");
      const size_t rank = a->view_shape.empty() ? plan.values[a->value].shape.size() : a->view_shape.size();
      if (a->indices.size() != rank) invalid("access rank differs from view or value");
    }
    for (int v : op.outflows)
      if (input_values.count(v)) invalid("BoundaryInputHasProducer { value: " + std::to_string(v) + " }");
  }
  plan.inputs = inputs_;
  std::stable_sort(plan.inputs.begin(), plan.inputs.end(),
                   [](const Binding& a, const Binding& b) { return a.tensor < b.tensor; });

  // normalise operands
  std::function<void(const std::vector<Statement>&, const std::string*)> normalize =
      [&](const std::vector<Statement>& nodes, const std::string* accum) {
        for (auto& s : nodes) {
          if (s.is_loop) {
            const bool reduction = s.kind == LoopKind::Sequential && s.body.size() == 1;
            normalize(s.body, reduction ? &s.domain.variable : nullptr);
            continue;
          }
          auto& op = plan.operations[s.operation];
          const Expression& e = *op.expression;
          const Expression* rhs = nullptr;
          bool accumulator = false;
          int destination = -1;
          if (e.kind == Expression::Store && e.args[0]->is_pure()) {
            destination = e.access.value;
            const Expression* acc = accum ? accumulation_rhs(e, *accum) : nullptr;
            accumulator = acc != nullptr;
            rhs = acc ? acc : e.args[0].get();
          } else if (e.kind == Expression::AllGather || e.kind == Expression::AllReduce) {
            destination = e.access.value;
            rhs = &e;
          } else {
            invalid("expected store with pure computation or all_gather");
          }
          if (op.outflows.size() != 1 || op.outflows[0] != destination)
            invalid("expression destination differs from declared outflow");
          std::vector<int> reads;
          rhs->reads(reads);
          std::set<int> declared;
          for (int v : op.inflows)
            if (!accumulator || std::find(op.outflows.begin(), op.outflows.end(), v) == op.outflows.end())
              declared.insert(v);
          if (declared != std::set<int>(reads.begin(), reads.end()))
            invalid("expression reads differ from declared inflows");
          op.inflows = reads;
        }
      };
  normalize(plan.statements, nullptr);

  // validate program
  for (size_t i = 0; i < plan.values.size(); ++i) {
    const bool boundary = input_values.count(int(i)) || plan.outputs[0].value == int(i);
    if (boundary && plan.values[i].storage != Storage::External)
      invalid("InvalidBoundaryStorage { value: " + std::to_string(i) + " }");
    if (!boundary && plan.values[i].storage == Storage::External)
      invalid("UnboundExternalValue { value: " + std::to_string(i) + " }");
    if (plan.values[i].storage == Storage::Register) {
      int owners = 0;
      for (auto& s : plan.statements) {
        std::vector<int> ops;
        s.operations(ops);
        bool touches = false;
        for (int id : ops) {
          auto& op = plan.operations[id];
          touches |= std::find(op.inflows.begin(), op.inflows.end(), int(i)) != op.inflows.end() ||
                     std::find(op.outflows.begin(), op.outflows.end(), int(i)) != op.outflows.end();
        }
        owners += touches;
      }
      if (owners > 1)
        invalid("CrossStatementStorage { value: " + std::to_string(i) + ", storage: Register }");
    }
  }
  std::set<int> available = input_values;
  std::function<void(const std::vector<Statement>&, std::set<std::string>&)> validate =
      [&](const std::vector<Statement>& nodes, std::set<std::string>& scope) {
        for (auto& s : nodes) {
          if (s.is_loop) {
            if (s.body.empty()) invalid("empty Loop body");
            if (!scope.insert(s.domain.variable).second) invalid("shadowed loop variable");
            validate(s.body, scope);
            scope.erase(s.domain.variable);
            continue;
          }
          auto& op = plan.operations[s.operation];
          std::vector<TensorAccess*> accesses;
          op.expression->accesses(accesses);
          for (auto* a : accesses)
            for (auto& i : a->indices) {
              if ((i.kind == AccessIndex::Tile || i.kind == AccessIndex::ClippedTile) && i.width.symbolic &&
                  scope.count(i.width.symbol))
                invalid("tile width " + i.width.symbol +
                        " must name a configuration symbol, not a loop coordinate");
              if (i.kind != AccessIndex::FullTile && !scope.count(i.variable))
                invalid("unbound index " + i.variable);
            }
          for (int v : op.inflows)
            if (!available.count(v)) invalid("MissingProducer { value: " + std::to_string(v) + " }");
          for (int v : op.outflows) available.insert(v);
        }
      };
  std::set<std::string> scope;
  validate(plan.statements, scope);
  if (!available.count(plan.outputs[0].value)) invalid("output has no producer");
  finalized_ = true;
  return canonicalize(std::move(plan));
}

}  // namespace trinity::host
