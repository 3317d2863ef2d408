// Physical plan model: values, operations with expression trees, statements with explicit
// loops.  A C++ statement of the reference planner's data model and rules
// (src/analysis/plan/{mod,builder,normalize,bindings,expression,statement}.rs); the planner is
// pure data and never touches a GPU.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "sexpr.hpp"

namespace trinity::host {

// Error kinds map onto the Python exceptions the reference raises.
enum class ErrorKind { Value = 1, NotImplemented = 2, Runtime = 3, Type = 4 };
struct PlanError : std::runtime_error {
  ErrorKind kind;
  PlanError(ErrorKind k, const std::string& what) : std::runtime_error(what), kind(k) {}
};
[[noreturn]] inline void invalid(const std::string& what) { throw PlanError(ErrorKind::Value, what); }

enum class DType { Fp16, Bf16, Fp32 };
enum class Storage { External, Global, Register };
enum class Target { Hopper, Sm89, Sm120, Sm100 };
enum class LoopKind { Parallel, Sequential, Split };

const char* dtype_name(DType d);
const char* storage_name(Storage s);
const char* target_name(Target t);
DType parse_dtype(const std::string& s);
Storage parse_storage(const std::string& s);
Target parse_target(const std::string& s);
inline int dtype_bytes(DType d) { return d == DType::Fp32 ? 4 : 2; }

// Integer expression over loop variables and symbols.
struct IndexExpr {
  enum Kind { Constant, Variable, Add, Sub, Mul, Div } kind = Constant;
  int64_t value = 0;
  std::string name;
  std::vector<IndexExpr> operands;  // two for the binary kinds

  static IndexExpr constant(int64_t v) { IndexExpr e; e.kind = Constant; e.value = v; return e; }
  static IndexExpr variable(std::string n) { IndexExpr e; e.kind = Variable; e.name = std::move(n); return e; }
  bool is_constant() const { return kind == Constant; }
  bool operator==(const IndexExpr& o) const;
  void rename(const std::map<std::string, std::string>& names);
  void collect_variables(std::set<std::string>& out) const;
  IndexExpr bind(const std::map<std::string, int64_t>& symbols) const;  // folds constants
  std::string json() const;
};
IndexExpr parse_index(const std::string& text);

struct TileWidth {
  bool symbolic = false;
  int64_t constant = 0;
  std::string symbol;
  bool operator==(const TileWidth& o) const {
    return symbolic == o.symbolic && constant == o.constant && symbol == o.symbol;
  }
};

struct AccessIndex {
  enum Kind { FullTile, Tile, ClippedTile, Elem } kind = FullTile;
  std::string variable;
  TileWidth width;
  bool operator==(const AccessIndex& o) const {
    return kind == o.kind && variable == o.variable && width == o.width;
  }
  bool operator!=(const AccessIndex& o) const { return !(*this == o); }
};

struct TensorAccess {
  int value = -1;
  std::vector<AccessIndex> indices;
  std::vector<int64_t> view_shape;  // empty = the value's own shape
  bool operator==(const TensorAccess& o) const {
    return value == o.value && indices == o.indices && view_shape == o.view_shape;
  }
};

struct Expression;
using ExprPtr = std::shared_ptr<Expression>;
struct Expression {
  enum Kind {
    ConstInt, ConstF32, Load, Store, Add, Sub, Mul, Div, Matmul, Max, Sqr, Sqrt, Sigmoid, Relu,
    Exp, Transpose, Permute, ReduceSum, ReduceMax, Broadcast, Unsqueeze, AllGather, AllReduce
  } kind = ConstInt;
  int64_t integer = 0;
  uint32_t f32_bits = 0;
  TensorAccess access;        // Load; Store/AllGather/AllReduce destination
  TensorAccess source;        // AllGather/AllReduce source
  std::vector<ExprPtr> args;  // operands (Store: the stored value)
  int axis = 0;
  std::vector<int> axes;      // Permute: source axis of every result axis

  bool is_pure() const;                       // no Store / collective inside
  void reads(std::vector<int>& out) const;    // value ids loaded, first-use order, unique
  void accesses(std::vector<TensorAccess*>& out);
  std::string text() const;                   // canonical s-expression (used for equality/hash)
};

struct Value {
  DType dtype;
  std::vector<int64_t> shape;
  Storage storage;
  std::string name;  // may be empty until normalisation
};

struct Operation {
  std::vector<int> inflows, outflows;
  ExprPtr expression;
};

struct LoopDomain {
  std::string variable;
  IndexExpr start, stop, step;
};

struct Statement {
  bool is_loop = false;
  int operation = -1;
  LoopKind kind = LoopKind::Parallel;
  LoopDomain domain;
  std::vector<Statement> body;

  void operations(std::vector<int>& out) const;
};

struct Binding {
  std::string tensor;
  int value;
};

class PhysicalPlan {
 public:
  Target target = Target::Hopper;
  int world_size = 1;
  std::vector<Binding> inputs;   // sorted by tensor name
  std::vector<Binding> outputs;  // exactly one from the builder
  std::vector<Value> values;
  std::vector<Operation> operations;
  std::vector<Statement> statements;

  std::set<std::string> symbols() const;  // unbound tile widths and loop-bound symbols
  PhysicalPlan bind_symbols(const std::map<std::string, int64_t>& bindings) const;
  std::string metadata_json() const;
  std::string structure_text() const;  // canonical text of the whole body
  uint64_t hash() const;
  bool same_body(const PhysicalPlan& other) const { return structure_text() == other.structure_text(); }
};

class PlanBuilder {
 public:
  PlanBuilder(int world_size, Target target);
  int add_value(DType dtype, std::vector<int64_t> shape, Storage storage, const std::string& name);
  void bind_input(const std::string& tensor, int value);
  int add_operation(std::vector<int> inflows, std::vector<int> outflows, const std::string& expression);
  int add_loop(const std::string& kind, const std::string& variable, const std::string& start,
               const std::string& stop, const std::string& step, const std::vector<int>& body);
  PhysicalPlan build(const std::vector<int>& statements, const std::string& output_tensor, int output);

  ExprPtr parse_expression(const std::string& text) const;

  // Entry points for the text reader, which has already parsed its input.
  int add_operation_expr(std::vector<int> inflows, std::vector<int> outflows, ExprPtr expression);
  int add_loop_expr(LoopKind kind, const std::string& variable, IndexExpr start, IndexExpr stop, IndexExpr step,
                    const std::vector<int>& body);
  const std::vector<Value>& values() const { return values_; }

 private:
  void require_open() const;
  Target target_;
  int world_size_;
  bool finalized_ = false;
  std::vector<Binding> inputs_;
  std::vector<Value> values_;
  std::vector<Operation> operations_;
  std::vector<Statement> nodes_;  // statement nodes by id (operations and loops)
};

// Text reader: (seq ...), (ploop start stop step var body), (sloop ...), bare stores.
std::vector<PhysicalPlan> lower_ir(const std::string& text, const std::map<std::string, int64_t>& symbols,
                                   const std::map<std::string, std::string>& dtypes, Target target,
                                   int world_size);

// Decodes expression notation against `values`; `symbols` (may be null) resolves named integers.
ExprPtr decode_expression(const Node& node, const std::vector<Value>& values,
                          const std::map<std::string, int64_t>* symbols);

std::string json_escape(const std::string& s);

}  // namespace trinity::host
