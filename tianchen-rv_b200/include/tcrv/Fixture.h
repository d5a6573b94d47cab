// In-memory form of the textual fixtures the drivers read: a module of `tcrv.exec.kernel`
// ops, each holding capabilities, variants and an optional dispatch, where a variant holds a
// typed `tcrv_rvv` body (runtime ABI values, setvl, one `with_vl` boundary with the compute
// ops).  The parser accepts the subset of MLIR's textual syntax those fixtures use; it is
// not an MLIR parser.  Envelope being mirrored:
// test/Target/RVV/explicit-selected-body-artifact-add.mlir:9-30 of the reference.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace tcrv {

// One attribute value.  `text` keeps the source spelling for printing.
struct Attr {
  enum Kind { String, Integer, SymbolRef, Array, Opaque } kind = Opaque;
  std::string text;             // source spelling (strings keep their quotes)
  std::string str;              // String: unquoted value; SymbolRef: name without '@'
  long long integer = 0;        // Integer
  std::vector<Attr> elements;   // Array
};

struct Op {
  std::vector<std::string> results;   // "%name"
  std::string name;                   // e.g. "tcrv_rvv.binary"
  std::string symbol;                 // "@sym" operand of symbol-defining ops, without '@'
  std::vector<std::string> operands;  // "%name"
  std::vector<std::pair<std::string, Attr>> attrs;  // source order
  std::vector<std::string> operandTypes;
  std::vector<std::string> resultTypes;
  std::vector<std::unique_ptr<Op>> body;  // single region, single block
  bool hasRegion = false;
  int line = 0;

  const Attr *attr(const std::string &key) const;
  std::string strAttr(const std::string &key) const;  // "" when absent or not a string
  bool intAttr(const std::string &key, long long &out) const;
  const Op *firstChild(const std::string &opName) const;
  std::vector<const Op *> children(const std::string &opName) const;
};

struct ParseResult {
  std::unique_ptr<Op> module;  // null on failure
  std::string error;           // "line N: message"
};

ParseResult parseFixture(const std::string &text);

// Prints an op tree back in the fixture syntax (used by the tcrv-opt look-alike to emit the
// module with the materialised plan ops).
std::string printOp(const Op &op, int indent = 0);

}  // namespace tcrv
