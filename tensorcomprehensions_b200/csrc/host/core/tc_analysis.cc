// Size binding, range inference and output shapes for a TC def (see tc/core/tc_analysis.h).
#include "tc/core/tc_analysis.h"

#include <algorithm>
#include <climits>
#include <functional>
#include <set>
#include <sstream>

#include "tc/lang/error_report.h"
#include "tc/lang/sema.h"

namespace tc {

using lang::ErrorReport;
using lang::TreeRef;

bool AffineIndex::isSingleVar(std::string* name) const {
  if (!affine || constant != 0 || coeff.size() != 1 || coeff.begin()->second != 1) return false;
  if (name) *name = coeff.begin()->first;
  return true;
}

const TensorSymbol* DefAnalysis::find(const std::string& tensor) const {
  for (const auto& t : inputs)
    if (t.name == tensor) return &t;
  for (const auto& t : outputs)
    if (t.name == tensor) return &t;
  return nullptr;
}

DLDataType toDLDataType(int k) {
  using namespace lang;
  switch (k) {
    case TK_BOOL: return DLDataType{kDLUInt, 1, 1};
    case TK_UINT8: return DLDataType{kDLUInt, 8, 1};
    case TK_UINT16: return DLDataType{kDLUInt, 16, 1};
    case TK_UINT32: return DLDataType{kDLUInt, 32, 1};
    case TK_UINT64: return DLDataType{kDLUInt, 64, 1};
    case TK_INT8: return DLDataType{kDLInt, 8, 1};
    case TK_INT16: return DLDataType{kDLInt, 16, 1};
    case TK_INT32: return DLDataType{kDLInt, 32, 1};
    case TK_INT64: return DLDataType{kDLInt, 64, 1};
    case TK_FLOAT16: return DLDataType{kDLFloat, 16, 1};
    case TK_FLOAT: case TK_FLOAT32: return DLDataType{kDLFloat, 32, 1};
    case TK_DOUBLE: case TK_FLOAT64: return DLDataType{kDLFloat, 64, 1};
    default: throw std::runtime_error("not a scalar type kind: " + lang::kindToString(k));
  }
}

int toScalarKind(const DLDataType& t) {
  lang::TypeInfo::Code c = t.code == kDLFloat ? lang::TypeInfo::Float
                           : (t.code == kDLUInt || t.code == kDLBool) ? lang::TypeInfo::UInt
                                                                      : lang::TypeInfo::Int;
  return lang::TypeInfo(c, t.code == kDLBool ? 1 : t.bits).toScalarToken();
}

namespace {

// ----------------------------------------------------------------------------------------------
// expressions over sizes and index variables
// ----------------------------------------------------------------------------------------------
struct Scope {
  const std::map<std::string, int64_t>* sizes;
  const std::set<std::string>* indexVars;
};

AffineIndex nonAffine() {
  AffineIndex a;
  a.affine = false;
  return a;
}

AffineIndex toAffine(const TreeRef& e, const Scope& sc) {
  using namespace lang;
  AffineIndex r;
  switch (e->kind()) {
    case TK_CONST: {
      const double v = Const(e).value();
      if (v != (double)(int64_t)v) return nonAffine();
      r.constant = (int64_t)v;
      return r;
    }
    case TK_IDENT: {
      const std::string& n = Ident(e).name();
      auto it = sc.sizes->find(n);
      if (it != sc.sizes->end()) {
        r.constant = it->second;
        return r;
      }
      if (sc.indexVars->count(n)) {
        r.coeff[n] = 1;
        return r;
      }
      return nonAffine();
    }
    case '+': case '-': {
      if (e->trees().size() == 1) {  // unary minus
        AffineIndex a = toAffine(e->tree(0), sc);
        if (!a.affine) return a;
        for (auto& kv : a.coeff) kv.second = -kv.second;
        a.constant = -a.constant;
        return a;
      }
      AffineIndex a = toAffine(e->tree(0), sc), b = toAffine(e->tree(1), sc);
      if (!a.affine || !b.affine) return nonAffine();
      const int64_t sign = e->kind() == '+' ? 1 : -1;
      for (const auto& kv : b.coeff) {
        a.coeff[kv.first] += sign * kv.second;
        if (a.coeff[kv.first] == 0) a.coeff.erase(kv.first);
      }
      a.constant += sign * b.constant;
      return a;
    }
    case '*': {
      AffineIndex a = toAffine(e->tree(0), sc), b = toAffine(e->tree(1), sc);
      if (!a.affine || !b.affine) return nonAffine();
      if (!a.coeff.empty() && !b.coeff.empty()) return nonAffine();
      if (a.coeff.empty()) std::swap(a, b);  // b is the constant factor
      for (auto& kv : a.coeff) kv.second *= b.constant;
      a.constant *= b.constant;
      if (b.constant == 0) a.coeff.clear();
      return a;
    }
    default:
      return nonAffine();
  }
}

// A size expression without index variables (bounds of a where clause).
bool toConstant(const TreeRef& e, const Scope& sc, int64_t* out) {
  AffineIndex a = toAffine(e, sc);
  if (!a.affine || !a.coeff.empty()) return false;
  *out = a.constant;
  return true;
}

void collectReads(const TreeRef& e, const Scope& sc, std::vector<TensorAccess>* out) {
  if (e->isAtom()) return;
  if (e->kind() == lang::TK_ACCESS) {
    lang::Access a(e);
    TensorAccess t;
    t.tensor = a.name().name();
    t.tree = e;
    for (const auto& idx : a.arguments()) t.indices.push_back(toAffine(idx, sc));
    out->push_back(std::move(t));
    for (const auto& idx : a.arguments()) collectReads(idx, sc, out);  // indirect accesses
    return;
  }
  for (const auto& c : e->trees()) collectReads(c, sc, out);
}

void collectIndexVars(const TreeRef& e, const std::map<std::string, int64_t>& sizes,
                      const std::set<std::string>& tensors, std::set<std::string>* vars) {
  if (e->isAtom()) return;
  if (e->kind() == lang::TK_IDENT) {
    const std::string& n = lang::Ident(e).name();
    if (!sizes.count(n) && !tensors.count(n)) vars->insert(n);
    return;
  }
  if (e->kind() == lang::TK_ACCESS) {
    for (const auto& idx : lang::Access(e).arguments()) collectIndexVars(idx, sizes, tensors, vars);
    return;
  }
  for (const auto& c : e->trees()) collectIndexVars(c, sizes, tensors, vars);
}

int64_t floorDiv(int64_t a, int64_t b) {
  int64_t q = a / b, r = a % b;
  return (r != 0 && ((r < 0) != (b < 0))) ? q - 1 : q;
}
int64_t ceilDiv(int64_t a, int64_t b) { return -floorDiv(-a, b); }

// lo <= expr <= hi must hold for every value of the variables already solved.
struct Constraint {
  AffineIndex expr;
  int64_t lo, hi;
};

// ----------------------------------------------------------------------------------------------
// range inference for one statement
// ----------------------------------------------------------------------------------------------
void inferRanges(StatementAnalysis& st, const std::vector<Constraint>& initial,
                 const std::set<std::string>& allVars, const CompilerOptions& opts) {
  constexpr int64_t kNegInf = LLONG_MIN / 4, kPosInf = LLONG_MAX / 4;
  std::vector<Constraint> ineq = initial;
  std::set<std::string> unsolved;
  for (const auto& v : allVars)
    if (!st.ranges.count(v)) unsolved.insert(v);
  std::vector<std::string> unchecked;  // preconditions nobody checks at run time

  // Substitutes the solved variables: the constraint has to hold over their whole range, so the
  // lower bound meets the expression's minimum and the upper bound its maximum.
  auto eliminateSolved = [&](Constraint& c) {
    int64_t minShift = 0, maxShift = 0;
    for (auto it = c.expr.coeff.begin(); it != c.expr.coeff.end();) {
      auto r = st.ranges.find(it->first);
      if (r == st.ranges.end()) {
        ++it;
        continue;
      }
      const int64_t a = it->second * r->second.min, b = it->second * r->second.max;
      minShift += std::min(a, b);
      maxShift += std::max(a, b);
      it = c.expr.coeff.erase(it);
    }
    // lo <= rest + minShift  and  rest + maxShift <= hi
    c.lo -= minShift;
    c.hi -= maxShift;
  };
  auto describe = [](const Constraint& c) {
    std::stringstream ss;
    ss << c.lo << " <= ";
    bool first = true;
    for (const auto& kv : c.expr.coeff) {
      ss << (first ? "" : " + ") << kv.second << "*" << kv.first;
      first = false;
    }
    if (c.expr.constant || first) ss << (first ? "" : " + ") << c.expr.constant;
    ss << " <= " << c.hi;
    return ss.str();
  };

  for (auto& c : ineq) {
    const bool hadVars = !c.expr.coeff.empty();
    eliminateSolved(c);
    if (hadVars && c.expr.coeff.empty() && !(c.lo <= c.expr.constant && c.expr.constant <= c.hi))
      unchecked.push_back(describe(c));
  }

  while (!unsolved.empty()) {
    std::set<std::string> still;
    for (const std::string& v : unsolved) {
      int64_t lo = kNegInf, hi = kPosInf;
      std::vector<Constraint> rest;
      std::vector<std::string> used;
      for (const auto& c : ineq) {
        if (c.expr.coeff.size() == 1 && c.expr.coeff.begin()->first == v) {
          const int64_t k = c.expr.coeff.begin()->second, c0 = c.expr.constant;
          // c.lo <= k*v + c0 <= c.hi
          if (k > 0) {
            lo = std::max(lo, ceilDiv(c.lo - c0, k));
            hi = std::min(hi, floorDiv(c.hi - c0, k));
          } else {
            lo = std::max(lo, ceilDiv(c.hi - c0, k));
            hi = std::min(hi, floorDiv(c.lo - c0, k));
          }
          used.push_back(describe(c));
        } else {
          rest.push_back(c);
        }
      }
      if (lo != kNegInf && hi != kPosInf && lo > hi) {
        ErrorReport err(st.tree);
        err << "Inferred an empty range for variable " << v << ". Derived condition: ";
        for (size_t i = 0; i < used.size(); ++i) err << (i ? " && " : "") << used[i];
        throw err;
      }
      if (lo == kNegInf || hi == kPosInf) {
        still.insert(v);  // needs other variables solved first
      } else {
        st.ranges[v] = IndexRange{lo, hi};
        ineq.swap(rest);
      }
    }
    for (auto& c : ineq) {
      const bool hadVars = !c.expr.coeff.empty();
      eliminateSolved(c);
      if (hadVars && c.expr.coeff.empty() &&
          !(c.lo <= c.expr.constant && c.expr.constant <= c.hi))
        unchecked.push_back(describe(c));
    }
    if (still.size() == unsolved.size()) {
      ErrorReport err(st.tree);
      for (const auto& v : unsolved) err << "Unsolved variable: " << v << '\n';
      err << "Inferred constraint: ";
      for (size_t i = 0; i < ineq.size(); ++i) err << (i ? " && " : "") << describe(ineq[i]);
      err << '\n' << "Could not infer ranges for free variables. Use a where clause";
      throw err;
    }
    unsolved.swap(still);
  }

  // constraints without any variable (constant indices) that do not hold
  for (const auto& c : ineq)
    if (c.expr.coeff.empty() && !(c.lo <= c.expr.constant && c.expr.constant <= c.hi))
      unchecked.push_back(describe(c));
  if (!unchecked.empty()) {
    ErrorReport err(st.tree);
    err << "Required precondition will not be checked at runtime: ";
    for (size_t i = 0; i < unchecked.size(); ++i) err << (i ? " && " : "") << unchecked[i];
    if (opts.throwWarnings) throw err;
    lang::warn(err, opts);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------------
DefAnalysis analyzeDef(const TreeRef& parsedDef, const std::vector<const DLConstTensor*>& inputs,
                       const CompilerOptions& opts) {
  using namespace lang;
  DefAnalysis out;
  Sema sema(opts);
  out.def = sema.checkFunction(parsedDef);
  Def def(out.def);
  out.name = def.name().name();

  // ---- bind size symbols to the input shapes ------------------------------------------------
  if (def.params().size() != inputs.size())
    throw ErrorReport(out.def) << "expected " << def.params().size() << " inputs but got "
                               << inputs.size();
  for (size_t i = 0; i < inputs.size(); ++i) {
    Param p = def.params()[i];
    TensorType tt = p.tensorType();
    const DLConstTensor* t = inputs[i];
    if ((size_t)t->ndim != tt.dims().size())
      throw ErrorReport(p) << "expected a tensor with " << tt.dims().size()
                           << " dimensions but found " << t->ndim << " dimensions.";
    TensorSymbol sym;
    sym.name = p.ident().name();
    sym.scalarKind = tt.scalarType();
    sym.isInput = true;
    for (int d = 0; d < t->ndim; ++d) {
      TreeRef dim = tt.dims()[d];
      const int64_t size = t->shape[d];
      if (dim->kind() == TK_IDENT) {
        const std::string& n = Ident(dim).name();
        auto it = out.sizes.find(n);
        if (it == out.sizes.end()) {
          out.sizes[n] = size;
        } else if (it->second != size) {
          throw ErrorReport(dim) << "Mismatched sizes for dimension " << n << " previous value is "
                                 << it->second << " but found " << size << " here";
        }
      } else {
        const int64_t c = (int64_t)Const(dim).value();
        if (c != size)
          throw ErrorReport(dim) << "Constant dimension expected size " << c << " but found "
                                 << size;
      }
      sym.shape.push_back(size);
    }
    out.inputs.push_back(std::move(sym));
  }

  std::set<std::string> tensorNames;
  for (const auto& t : out.inputs) tensorNames.insert(t.name);
  for (const auto& r : def.returns()) tensorNames.insert(r.ident().name());

  // Shapes of the tensors defined so far (inputs + outputs of earlier statements).
  std::map<std::string, std::vector<IndexRange>> bounds;
  for (const auto& t : out.inputs) {
    std::vector<IndexRange> b;
    for (int64_t s : t.shape) b.push_back(IndexRange{0, s - 1});
    bounds[t.name] = b;
  }
  std::map<std::string, TensorSymbol> defined;  // outputs by name

  for (const auto& stmtView : def.statements()) {
    Comprehension c(stmtView);
    StatementAnalysis st;
    st.tree = c;
    st.lhs = c.ident().name();
    st.assignment = c.assignment()->kind();
    for (const auto& i : c.indices()) st.lhsIndices.push_back(i.name());
    for (const auto& r : c.reductionVariables()) st.reductionVars.push_back(r.name());

    std::set<std::string> vars(st.lhsIndices.begin(), st.lhsIndices.end());
    vars.insert(st.reductionVars.begin(), st.reductionVars.end());
    collectIndexVars(c.rhs(), out.sizes, tensorNames, &vars);
    // let-bound names are not index variables
    for (const auto& w : c.whereClauses())
      if (w->kind() == TK_LET) vars.erase(Let(w).name().name());
    Scope sc{&out.sizes, &vars};

    // explicit ranges: where v in lo:hi  (half-open)
    for (const auto& w : c.whereClauses()) {
      if (w->kind() != TK_RANGE_CONSTRAINT) continue;
      RangeConstraint rc(w);
      int64_t lo, hi;
      if (!toConstant(rc.start(), sc, &lo) || !toConstant(rc.end(), sc, &hi))
        throw ErrorReport(w) << "range bounds must be expressions of the tensor sizes";
      st.ranges[rc.ident().name()] = IndexRange{lo, hi - 1};
    }

    collectReads(c.rhs(), sc, &st.reads);
    for (const auto& w : c.whereClauses())
      if (w->kind() == TK_EXISTS) collectReads(Exists(w).exp(), sc, &st.reads);

    // every access stays inside its tensor
    std::vector<Constraint> constraints;
    auto constrain = [&](const std::string& tensor, const std::vector<AffineIndex>& idx) {
      auto b = bounds.find(tensor);
      if (b == bounds.end()) return;
      for (size_t d = 0; d < idx.size() && d < b->second.size(); ++d) {
        if (!idx[d].affine) continue;
        constraints.push_back(Constraint{idx[d], b->second[d].min, b->second[d].max});
      }
    };
    for (const auto& r : st.reads) constrain(r.tensor, r.indices);
    // a reduction or in-place update also reads the output at the left-hand-side indices
    if (st.assignment != '=' && bounds.count(st.lhs)) {
      std::vector<AffineIndex> lhsIdx;
      for (const auto& v : st.lhsIndices) {
        AffineIndex a;
        a.coeff[v] = 1;
        lhsIdx.push_back(a);
      }
      constrain(st.lhs, lhsIdx);
    }

    inferRanges(st, constraints, vars, opts);

    for (const auto& v : st.lhsIndices)
      if (!st.ranges.count(v))
        throw ErrorReport(c) << "Free variable " << v
                             << " was not solved in range inference. May not be used right-hand side";

    // the statement defines (or re-defines) the bounds of its output
    std::vector<IndexRange> ob;
    for (const auto& v : st.lhsIndices) ob.push_back(st.ranges.at(v));
    bounds[st.lhs] = ob;
    TensorSymbol& sym = defined[st.lhs];
    sym.name = st.lhs;
    sym.scalarKind = sema.typeOfExpr(c.rhs())->kind();
    sym.shape.clear();
    for (const auto& r : ob) sym.shape.push_back(r.extent());
    out.statements.push_back(std::move(st));
  }

  for (const auto& r : def.returns()) {
    auto it = defined.find(r.ident().name());
    if (it == defined.end())
      throw ErrorReport(r) << "output " << r.ident().name() << " is never written";
    out.outputs.push_back(it->second);
  }
  return out;
}

}  // namespace tc
