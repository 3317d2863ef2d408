// Text reader for loop/tensor IR: (seq a b), (ploop start stop step var body),
// (sloop start stop step var body), (store view rhs index), `dummy` subtrees dropped.
//
// Restates the part of the reference reader the native path needs
// (src/analysis/plan/ir.rs:85-128, :494-633) and its storage rule in brief
// (src/analysis/storage/mod.rs:127-141, :197-234): declared inputs and outputs are External; a
// written tensor touched by one top-level kernel only and always through the same index and
// view lives in a Register; every other tensor is Global.  A split loop
// (mloop start stop step var split count body) is normalised as the reference does
// (src/analysis/plan/ir.rs:527-599): a parallel loop over `split` in [0, count) around a
// sequential loop of `var` over the split's equal share of [start, stop).
//
// Three of the reference reader's rejections are restated with their message fragments
// (src/analysis/storage/mod.rs:303-312, :352-363; tests/streamed.rs:183-190, tests/ir.rs:52-63
// there): a parallel loop inside a sequential one ("parallel work inside"), a write to memory
// that an enclosing parallel loop does not index although the value depends on the loop ("not
// proven disjoint"), and a read of an intermediate tensor beyond what earlier kernels wrote
// ("not covered").  The interval reasoning is per axis over tile / elem / fulltile indices with
// numeric loop bounds; any other index form is taken as covering.
#include <algorithm>
#include <functional>

#include "plan.hpp"

namespace trinity::host {

namespace {

struct LoopScope {
  std::string variable;
  bool parallel = false, numeric = false;
  int64_t start = 0, stop = 0, step = 1;
};

// One load or store as the reader saw it: which elements it can touch, per axis, as a half-open
// interval (exact = the interval is touched without gaps).
struct AccessRecord {
  int kernel = 0;
  bool write = false;
  size_t offset = 0;
  bool known = true;                           // false: an index form the interval reasoning skips
  std::vector<std::pair<int64_t, int64_t>> range;
  bool exact = true;
  std::set<std::string> index_variables;       // loop variables the index mentions
  std::vector<std::string> unindexed_parallel; // enclosing parallel loops the index does not mention
  bool value_depends_on_unindexed = false;     // (writes) the stored value mentions one of those
};

struct TensorInfo {
  std::string role;            // input | output | tensor
  std::vector<int64_t> shape;  // first view seen = base shape
  std::set<int> kernels;       // top-level kernels touching it
  std::set<std::string> regions;  // distinct (view, index) spellings
  bool written = false;
  int value = -1;
  std::vector<AccessRecord> accesses;
};

void atoms_of(const Node& n, std::set<std::string>& out) {
  if (n.is_atom) {
    out.insert(n.text);
    return;
  }
  for (auto& c : n.children) atoms_of(c, out);
}

std::string spelling(const Node& n) {
  if (n.is_atom) return n.text;
  std::string s = "(" + n.text;
  for (auto& c : n.children) s += " " + spelling(c);
  return s + ")";
}

struct Reader {
  const std::map<std::string, int64_t>& symbols;
  const std::map<std::string, std::string>& dtypes;
  std::map<std::string, TensorInfo> tensors;
  std::vector<std::string> order;

  int64_t number(const Node& n) const {
    const std::string& a = n.atom();
    char* end = nullptr;
    long long v = strtoll(a.c_str(), &end, 10);
    if (!a.empty() && !*end) return v;
    auto it = symbols.find(a);
    if (it == symbols.end()) throw SyntaxError(n.offset, "unresolved symbol " + a);
    return it->second;
  }

  void flatten(const Node& n, std::vector<const Node*>& kernels) const {
    if (n.is_atom) {
      if (n.text == "dummy") return;
      throw SyntaxError(n.offset, "expected a statement");
    }
    if (n.op() == "seq") {
      const auto& a = n.args(2);
      flatten(a[0], kernels);
      flatten(a[1], kernels);
    } else if (n.op() != "dummy") {
      kernels.push_back(&n);
    }
  }

  std::vector<LoopScope> loops;   // enclosing loops of the node being collected, outermost first

  void collect(const Node& n, int kernel, bool is_store_destination) {
    if (n.is_atom) return;
    if (n.op() == "ploop" || n.op() == "sloop") {
      const auto& a = n.args(5);
      LoopScope scope;
      scope.variable = a[3].atom();
      scope.parallel = n.op() == "ploop";
      if (scope.parallel)
        for (auto& outer : loops)
          if (!outer.parallel)
            throw SyntaxError(n.offset, "parallel work inside a sequential loop (" + outer.variable + ") is not supported");
      try {
        scope.start = number(a[0]);
        scope.stop = number(a[1]);
        scope.step = number(a[2]);
        scope.numeric = scope.step > 0;
      } catch (const SyntaxError&) {
        scope.numeric = false;   // bounds that are expressions or unbound symbols: no interval reasoning
      }
      loops.push_back(scope);
      collect(a[4], kernel, false);
      loops.pop_back();
      return;
    }
    if (n.op() == "mloop") {
      // parallel over the split variable, sequential over the loop variable within a share
      const auto& a = n.args(7);
      LoopScope outer, inner;
      outer.variable = a[4].atom();
      outer.parallel = true;
      for (auto& enclosing : loops)
        if (!enclosing.parallel)
          throw SyntaxError(n.offset, "parallel work inside a sequential loop (" + enclosing.variable + ") is not supported");
      inner.variable = a[3].atom();
      try {
        outer.start = 0;
        outer.stop = number(a[5]);
        outer.step = 1;
        outer.numeric = outer.stop > 0;
        // over all splits the inner variable walks the whole range with the loop's own step
        inner.start = number(a[0]);
        inner.stop = number(a[1]);
        inner.step = number(a[2]);
        inner.numeric = inner.step > 0;
      } catch (const SyntaxError&) {
        outer.numeric = inner.numeric = false;
      }
      loops.push_back(outer);
      loops.push_back(inner);
      collect(a[6], kernel, false);
      loops.pop_back();
      loops.pop_back();
      return;
    }
    if (n.op() == "store") {
      const auto& a = n.args(3);
      AccessRecord* record = note_access(a[0], a[2], kernel, true);
      if (record && !record->unindexed_parallel.empty()) {
        std::set<std::string> mentioned;
        atoms_of(a[1], mentioned);
        for (auto& v : record->unindexed_parallel)
          if (mentioned.count(v)) record->value_depends_on_unindexed = true;
      }
      collect(a[1], kernel, false);
      return;
    }
    if (n.op() == "load") {
      const auto& a = n.args(2);
      note_access(a[0], a[1], kernel, false);
      return;
    }
    (void)is_store_destination;
    for (auto& c : n.children) collect(c, kernel, false);
  }

  // The interval of one axis that an index form can touch under the enclosing loops.
  void axis_range(const Node& form, int64_t extent, AccessRecord& r) {
    auto clip = [&](int64_t lo, int64_t hi) {
      r.range.emplace_back(lo < 0 ? 0 : lo, hi > extent ? extent : hi);
    };
    if (form.is_atom) {
      if (form.text == "fulltile") clip(0, extent);
      else { r.known = false; r.range.emplace_back(0, extent); }
      return;
    }
    const std::string& kind = form.op();
    if (kind != "tile" && kind != "clipped_tile" && kind != "elem") {
      r.known = false;
      r.range.emplace_back(0, extent);
      return;
    }
    const std::string& variable = form.children.at(0).atom();
    r.index_variables.insert(variable);
    int64_t width = 1;
    if (kind != "elem") {
      try {
        width = number(form.children.at(1));
      } catch (const SyntaxError&) {
        r.known = false;
      }
    }
    const LoopScope* loop = nullptr;
    for (auto& l : loops)
      if (l.variable == variable) loop = &l;
    if (!loop || !loop->numeric || !r.known || loop->stop <= loop->start) {
      r.known = false;
      r.range.emplace_back(0, extent);
      return;
    }
    const int64_t last = loop->start + (loop->stop - 1 - loop->start) / loop->step * loop->step;
    if (loop->step > width) r.exact = false;   // gaps between the tiles
    clip(loop->start, last + width);
  }

  AccessRecord* note_access(const Node& view, const Node& index, int kernel, bool write) {
    if (view.is_atom || view.op() != "view") throw SyntaxError(view.offset, "expected view");
    const auto& v = view.args(2);
    const std::string role = v[0].is_atom ? "" : v[0].op();
    if (role != "input" && role != "output" && role != "tensor") throw SyntaxError(view.offset, "unsupported view base");
    const std::string& name = v[0].args(1)[0].atom();
    if (v[1].is_atom || v[1].op() != "layout") throw SyntaxError(view.offset, "expected layout");
    std::vector<int64_t> shape;
    for (auto& axis : v[1].children) {
      const auto& a = axis.args(2);
      const int64_t size = number(a[1]);
      if (size <= 0) throw SyntaxError(axis.offset, "nonpositive tensor extent");
      shape.push_back(size);
    }
    if (shape.empty() || shape.size() > 3) throw SyntaxError(view.offset, "supported tensor ranks are 1, 2, 3");
    auto it = tensors.find(name);
    if (it == tensors.end()) {
      TensorInfo info;
      info.role = role;
      info.shape = shape;
      it = tensors.emplace(name, info).first;
      order.push_back(name);
    } else {
      int64_t a = 1, b = 1;
      for (auto d : shape) a *= d;
      for (auto d : it->second.shape) b *= d;
      if (it->second.role != role || a != b) throw SyntaxError(view.offset, "inconsistent view for " + name);
    }
    it->second.kernels.insert(kernel);
    it->second.regions.insert(spelling(v[1]) + spelling(index));
    it->second.written |= write;
    // interval record: slots are keyed by axis name
    AccessRecord record;
    record.kernel = kernel;
    record.write = write;
    record.offset = view.offset;
    if (index.is_atom || index.op() != "keyed_index" || index.children.size() != v[1].children.size()) {
      record.known = false;
    } else {
      for (size_t axis = 0; axis < v[1].children.size() && record.known; ++axis) {
        const std::string& axis_name = v[1].children[axis].children.at(0).atom();
        const Node* form = nullptr;
        for (auto& slot : index.children)
          if (!slot.is_atom && slot.op() == "slot" && slot.children.size() == 2 && slot.children[0].is_atom &&
              slot.children[0].text == axis_name)
            form = &slot.children[1];
        if (!form) { record.known = false; break; }
        axis_range(*form, shape[axis], record);
      }
    }
    for (auto& l : loops)
      if (l.parallel && !record.index_variables.count(l.variable)) record.unindexed_parallel.push_back(l.variable);
    it->second.accesses.push_back(record);
    return &it->second.accesses.back();
  }

  // The reader-level rejections that need the whole program (see the head of this file).
  void check_hazards(const std::string& name, const TensorInfo& t, bool in_register) const {
    if (in_register) return;
    for (auto& a : t.accesses) {
      if (a.write && a.known && a.value_depends_on_unindexed)
        throw SyntaxError(a.offset, "write to " + name + " is not proven disjoint across parallel loop " +
                                        a.unindexed_parallel.front());
    }
    if (t.role == "input") return;
    for (auto& read : t.accesses) {
      if (read.write || !read.known) continue;
      bool produced_here = false, covered = false, any_earlier = false;
      // Earlier exact writes as boxes; two boxes that agree on every axis but one and touch or
      // overlap on that axis are one box (halves of a tensor, rows of tiles written by several
      // kernels), merged until nothing changes.
      std::vector<std::vector<std::pair<int64_t, int64_t>>> boxes;
      for (auto& w : t.accesses) {
        if (!w.write) continue;
        if (w.kernel == read.kernel) produced_here = true;
        if (w.kernel >= read.kernel) continue;
        any_earlier = true;
        if (!w.known) { covered = true; break; }
        if (!w.exact || w.range.size() != read.range.size()) continue;
        boxes.emplace_back(w.range.begin(), w.range.end());
      }
      for (bool merged = true; merged && !covered;) {
        merged = false;
        for (size_t i = 0; i < boxes.size() && !merged; ++i)
          for (size_t j = i + 1; j < boxes.size() && !merged; ++j) {
            int differing = -1, count = 0;
            for (size_t axis = 0; axis < boxes[i].size(); ++axis)
              if (boxes[i][axis] != boxes[j][axis]) { differing = int(axis); ++count; }
            if (count == 0) { boxes.erase(boxes.begin() + j); merged = true; break; }
            if (count != 1) continue;
            auto& a = boxes[i][differing];
            const auto& b = boxes[j][differing];
            if (b.first > a.second || a.first > b.second) continue;   // a gap between them
            a.first = std::min(a.first, b.first);
            a.second = std::max(a.second, b.second);
            boxes.erase(boxes.begin() + j);
            merged = true;
          }
      }
      for (auto& box : boxes) {
        if (covered) break;
        bool inside = true;
        for (size_t axis = 0; axis < box.size(); ++axis)
          if (read.range[axis].first < box[axis].first || read.range[axis].second > box[axis].second) inside = false;
        if (inside) covered = true;
      }
      if (produced_here || covered) continue;   // accumulators and in-kernel values are the planner's business
      if (any_earlier)
        throw SyntaxError(read.offset, "read of " + name + " is not covered by the writes of earlier kernels");
    }
  }
};

}  // namespace

std::vector<PhysicalPlan> lower_ir(const std::string& text, const std::map<std::string, int64_t>& symbols,
                                   const std::map<std::string, std::string>& dtypes, Target target, int world_size) {
  Node root;
  try {
    root = parse_sexpr(text);
  } catch (const SyntaxError& e) {
    invalid(e.what());
  }
  try {
    Reader reader{symbols, dtypes, {}, {}, {}};
    std::vector<const Node*> kernels;
    reader.flatten(root, kernels);
    for (size_t k = 0; k < kernels.size(); ++k) reader.collect(*kernels[k], int(k), false);

    PlanBuilder builder(world_size, target);
    std::string output_name;
    int output_value = -1;
    for (const std::string& name : reader.order) {
      TensorInfo& t = reader.tensors[name];
      auto dt = dtypes.find(name);
      if (dt == dtypes.end()) invalid("missing dtype for " + name);
      Storage storage = Storage::Global;
      if (t.role == "input" || t.role == "output") storage = Storage::External;
      else if (t.written && t.kernels.size() == 1 && t.regions.size() == 1) storage = Storage::Register;
      reader.check_hazards(name, t, storage == Storage::Register);
      t.value = builder.add_value(parse_dtype(dt->second), t.shape, storage, name);
      if (t.role == "input") builder.bind_input(name, t.value);
      if (t.role == "output") {
        if (output_value >= 0) invalid("the native path takes exactly one output tensor");
        output_name = name;
        output_value = t.value;
      }
    }
    if (output_value < 0) invalid("the program declares no output tensor");

    std::function<IndexExpr(const Node&, const std::set<std::string>&)> index = [&](const Node& n, const std::set<std::string>& scope) {
      if (n.is_atom) {
        if (scope.count(n.text)) return IndexExpr::variable(n.text);
        char* end = nullptr;
        long long v = strtoll(n.text.c_str(), &end, 10);
        if (!n.text.empty() && !*end) return IndexExpr::constant(v);
        auto it = symbols.find(n.text);
        if (it != symbols.end()) return IndexExpr::constant(it->second);
        return IndexExpr::variable(n.text);  // stays symbolic until bind_symbols
      }
      const auto& a = n.args(2);
      IndexExpr e;
      if (n.op() == "+") e.kind = IndexExpr::Add;
      else if (n.op() == "-") e.kind = IndexExpr::Sub;
      else if (n.op() == "*") e.kind = IndexExpr::Mul;
      else if (n.op() == "/") e.kind = IndexExpr::Div;
      else throw SyntaxError(n.offset, "unsupported range expression");
      e.operands = {index(a[0], scope), index(a[1], scope)};
      return e;
    };

    std::function<std::vector<int>(const Node&, std::set<std::string>)> statements = [&](const Node& n, std::set<std::string> scope) {
      std::vector<int> out;
      if (n.is_atom) {
        if (n.text == "dummy") return out;
        throw SyntaxError(n.offset, "expected a statement");
      }
      if (n.op() == "seq") {
        const auto& a = n.args(2);
        for (int part = 0; part < 2; ++part)
          for (int id : statements(a[part], scope)) out.push_back(id);
        return out;
      }
      if (n.op() == "ploop" || n.op() == "sloop") {
        const auto& a = n.args(5);
        const std::string& variable = a[3].atom();
        IndexExpr start = index(a[0], scope), stop = index(a[1], scope), step = index(a[2], scope);
        auto nested = scope;
        if (!nested.insert(variable).second) throw SyntaxError(n.offset, "shadowed loop variable " + variable);
        std::vector<int> body = statements(a[4], nested);
        if (body.empty()) throw SyntaxError(n.offset, "empty loop body");
        out.push_back(builder.add_loop_expr(n.op() == "ploop" ? LoopKind::Parallel : LoopKind::Sequential, variable,
                                            start, stop, step, body));
        return out;
      }
      if (n.op() == "mloop") {
        const auto& a = n.args(7);
        const std::string& variable = a[3].atom();
        const std::string& split = a[4].atom();
        IndexExpr start = index(a[0], scope), stop = index(a[1], scope), step = index(a[2], scope);
        auto nested = scope;
        if (!nested.insert(variable).second) throw SyntaxError(n.offset, "shadowed loop variable " + variable);
        if (!nested.insert(split).second) throw SyntaxError(a[4].offset, "split variable shadows an active loop");
        const int64_t count = reader.number(a[5]);
        const IndexExpr first = start.bind({}), last = stop.bind({}), stride = step.bind({});
        if (!first.is_constant() || !last.is_constant())
          throw SyntaxError(n.offset, "mloop bounds must be numbers once the symbols are bound");
        const int64_t extent = last.value - first.value;
        if (count <= 0 || extent <= 0 || extent % count != 0 ||
            (stride.is_constant() && (stride.value <= 0 || (extent / count) % stride.value != 0)))
          throw SyntaxError(n.offset, "mloop split must exactly divide the iteration range");
        const int64_t chunk = extent / count;
        IndexExpr share;
        share.kind = IndexExpr::Mul;
        share.operands = {IndexExpr::variable(split), IndexExpr::constant(chunk)};
        IndexExpr inner_start;
        inner_start.kind = IndexExpr::Add;
        inner_start.operands = {IndexExpr::constant(first.value), share};
        IndexExpr inner_stop;
        inner_stop.kind = IndexExpr::Add;
        inner_stop.operands = {inner_start, IndexExpr::constant(chunk)};
        std::vector<int> body = statements(a[6], nested);
        if (body.empty()) throw SyntaxError(n.offset, "empty loop body");
        const int inner = builder.add_loop_expr(LoopKind::Sequential, variable, inner_start, inner_stop, step, body);
        out.push_back(builder.add_loop_expr(LoopKind::Parallel, split, IndexExpr::constant(0), IndexExpr::constant(count),
                                            IndexExpr::constant(1), {inner}));
        return out;
      }
      if (n.op() == "store") {
        ExprPtr e = decode_expression(n, builder.values(), &symbols);
        std::vector<int> reads;
        e->args[0]->reads(reads);
        out.push_back(builder.add_operation_expr(reads, {e->access.value}, e));
        return out;
      }
      throw SyntaxError(n.offset, "unsupported statement " + n.op());
    };
    std::vector<int> top;
    for (const Node* k : kernels)
      for (int id : statements(*k, {})) top.push_back(id);
    std::vector<PhysicalPlan> plans;
    plans.push_back(builder.build(top, output_name, output_value));
    return plans;
  } catch (const SyntaxError& e) {
    invalid(e.what());
  }
}

}  // namespace trinity::host
