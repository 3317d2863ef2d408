// S-expression reader for plan notation: atoms end at whitespace, '(' , ')' or ';';
// ';' starts a comment that runs to the end of the line; nesting is limited to 256 levels.
// Grammar and messages follow the reference reader (src/analysis/ir/syntax.rs:82-143).
#pragma once

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace trinity::host {

struct SyntaxError : std::runtime_error {
  size_t offset;
  SyntaxError(size_t at, const std::string& what)
      : std::runtime_error(what + " at byte " + std::to_string(at)), offset(at) {}
};

struct Node {
  size_t offset = 0;
  bool is_atom = false;
  std::string text;             // atom text, or the head of a list ("" if the list has none)
  std::vector<Node> children;   // list arguments (after the head)

  const std::string& op() const { return text; }
  const std::string& atom() const {
    if (!is_atom) throw SyntaxError(offset, "expected an atom");
    return text;
  }
  const std::vector<Node>& args(size_t count) const {
    if (is_atom || children.size() != count)
      throw SyntaxError(offset, "'" + text + "' expects " + std::to_string(count) + " arguments");
    return children;
  }
};

class SexprParser {
 public:
  explicit SexprParser(const std::string& text) : text_(text) {}

  Node parse_all() {
    skip();
    Node node = parse_node(0);
    skip();
    if (pos_ < text_.size()) throw SyntaxError(pos_, "unexpected trailing input");
    return node;
  }

 private:
  void skip() {
    while (pos_ < text_.size()) {
      const char c = text_[pos_];
      if (c == ';') {
        while (pos_ < text_.size() && text_[pos_] != '\n') ++pos_;
      } else if (c == ' ' || c == '\t' || c == '\n' || c == '\r') {
        ++pos_;
      } else {
        break;
      }
    }
  }
  static bool ends_atom(char c) {
    return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == '(' || c == ')' || c == ';';
  }
  Node parse_node(int depth) {
    if (depth > 256) throw SyntaxError(pos_, "expression nesting exceeds 256");
    if (pos_ >= text_.size()) throw SyntaxError(pos_, "unexpected end of input");
    Node node;
    node.offset = pos_;
    if (text_[pos_] == ')') throw SyntaxError(pos_, "unexpected ')'");
    if (text_[pos_] != '(') {
      const size_t start = pos_;
      while (pos_ < text_.size() && !ends_atom(text_[pos_])) ++pos_;
      node.is_atom = true;
      node.text = text_.substr(start, pos_ - start);
      return node;
    }
    ++pos_;
    skip();
    bool first = true;
    for (;;) {
      if (pos_ >= text_.size()) throw SyntaxError(node.offset, "unclosed expression");
      if (text_[pos_] == ')') {
        ++pos_;
        return node;
      }
      Node child = parse_node(depth + 1);
      if (first && child.is_atom) {
        node.text = child.text;
      } else {
        if (first) throw SyntaxError(child.offset, "expected an operator name");
        node.children.push_back(std::move(child));
      }
      first = false;
      skip();
    }
  }

  const std::string& text_;
  size_t pos_ = 0;
};

inline Node parse_sexpr(const std::string& text) { return SexprParser(text).parse_all(); }

}  // namespace trinity::host
