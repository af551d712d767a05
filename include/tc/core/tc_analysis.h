// What a sema-checked TC def MEANS for concrete input shapes: size symbols bound to numbers,
// the range of every index variable, the shape of every output.
//
// This replaces the part of the reference that goes through Halide (tc/core/tc2halide.cc):
//   * computeParamValueMap        (tc/core/halide_utils.cc:41-86): bind N, C1, ... to input dims,
//     "Mismatched sizes for dimension" / "Constant dimension expected size" on conflict;
//   * forwardBoundsInference      (tc/core/tc2halide.cc:270-498): each index variable gets the
//     largest range that keeps every tensor access in bounds, solved in rounds over the accesses
//     that depend on a single unsolved variable; `where i in a:b` fixes a range up front;
//   * output extents              (tc/core/tc2halide.cc:897-906): extent of dim d of an output is
//     the extent of the d-th left-hand-side index of the statement that first defines it.
// Index expressions are handled when they are affine in the index variables with integer
// coefficients (i, i + j, 2 * i + j, i + 3, ...); anything else contributes no constraint, and an
// index variable left unconstrained is an error that asks for a where clause, like the reference.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "tc/core/tensor.h"
#include "tc/lang/tree.h"
#include "tc/utils/compiler_options.h"

namespace tc {

// sum(coeff[v] * v) + constant over index variables; affine == false when the expression is not
// of that form.
struct AffineIndex {
  bool affine = true;
  std::map<std::string, int64_t> coeff;
  int64_t constant = 0;
  bool isSingleVar(std::string* name = nullptr) const;  // exactly 1 * v + 0
};

struct IndexRange {
  int64_t min = 0, max = -1;  // inclusive
  int64_t extent() const { return max - min + 1; }
};

struct TensorAccess {
  std::string tensor;
  std::vector<AffineIndex> indices;
  lang::TreeRef tree;  // the TK_ACCESS node
};

struct StatementAnalysis {
  lang::TreeRef tree;  // sema-checked TK_COMPREHENSION
  std::string lhs;
  std::vector<std::string> lhsIndices;
  int assignment = 0;  // '=', TK_PLUS_EQ, TK_PLUS_EQ_B, ...
  std::vector<std::string> reductionVars;
  std::map<std::string, IndexRange> ranges;  // every index variable of the statement
  std::vector<TensorAccess> reads;           // tensor reads of the right-hand side, left to right
};

struct TensorSymbol {
  std::string name;
  int scalarKind = 0;  // lang::TK_FLOAT, ...
  std::vector<int64_t> shape;
  bool isInput = false;
};

struct DefAnalysis {
  lang::TreeRef def;  // sema-checked TK_DEF
  std::string name;
  std::map<std::string, int64_t> sizes;  // N -> 32, ...
  std::vector<TensorSymbol> inputs, outputs;
  std::vector<StatementAnalysis> statements;
  const TensorSymbol* find(const std::string& tensor) const;
};

// Parses nothing: `parsedDef` comes from lang::Parser::parseFunction.  Runs Sema, binds sizes to
// `inputs`, infers ranges and output shapes.  Throws lang::ErrorReport.
DefAnalysis analyzeDef(const lang::TreeRef& parsedDef, const std::vector<const DLConstTensor*>& inputs,
                       const CompilerOptions& options = CompilerOptions());

DLDataType toDLDataType(int scalarKind);
int toScalarKind(const DLDataType& t);

}  // namespace tc
