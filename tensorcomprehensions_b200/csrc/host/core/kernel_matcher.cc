// Statements of an analysed def -> launches of the tcb200 kernel families (see kernel_matcher.h).
#include "tc/core/kernel_matcher.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <set>

#include "tc/lang/error_report.h"

namespace tc {

using lang::ErrorReport;
using lang::TreeRef;

std::string MatchedLaunch::family() const {
  switch (problem.family) {
    case TCB200_FAMILY_CONTRACTION: return "contraction";
    case TCB200_FAMILY_TENSORDOT: return "tensordot";
    case TCB200_FAMILY_GROUP_CONV: return "group_conv";
    case TCB200_FAMILY_REDUCTION: return "reduction";
    case TCB200_FAMILY_COPY: return "copy";
    default: return "?";
  }
}

namespace {

[[noreturn]] void unmatched(const StatementAnalysis& st, const std::string& why) {
  throw ErrorReport(st.tree)
      << "no kernel family of the B200 backend matches this comprehension (" << why
      << "); supported: batched/transposed contractions O +=! A * B, tensordot with shared "
         "trailing indices, grouped convolution (each optionally followed by + bias and fmax(., 0)), sums of one tensor over "
         "adjacent indices";
}

struct Operand {
  std::string tensor;
  std::vector<std::string> vars;  // one index variable per dimension
  std::vector<int64_t> shape, strides;
  int value = -1;  // position in [inputs..., outputs...]
};

int valueIndex(const DefAnalysis& def, const std::string& tensor) {
  for (size_t i = 0; i < def.inputs.size(); ++i)
    if (def.inputs[i].name == tensor) return (int)i;
  for (size_t i = 0; i < def.outputs.size(); ++i)
    if (def.outputs[i].name == tensor) return (int)(def.inputs.size() + i);
  return -1;
}

bool isFloat32(const TensorSymbol* t) {
  return t && (t->scalarKind == lang::TK_FLOAT || t->scalarKind == lang::TK_FLOAT32);
}

// Every index of the access is a plain variable, no variable twice.
// With `ranges` (the lenient form): index variables whose range is the single value 0 count as the constant 0,
// so `h - r_kh` with a 1-wide r_kh is the plain index h (how the reference's convolution gradients are written,
// tensor_comprehensions/__init__.py:563-574, for the 1 x 1 filters its example uses); a dimension of extent 1
// that is indexed by such variables only is dropped from the operand (it does not change any stride).
bool plainOperand(const DefAnalysis& def, const TensorAccess& a, Operand* op,
                  const std::map<std::string, IndexRange>* ranges = nullptr) {
  const TensorSymbol* sym = def.find(a.tensor);
  if (!sym || sym->shape.size() != a.indices.size()) return false;
  op->tensor = a.tensor;
  op->value = valueIndex(def, a.tensor);
  const std::vector<int64_t> strides = makeStridesFromSizes(sym->shape);
  auto unit = [&](const std::string& v) {
    auto it = ranges->find(v);
    return it != ranges->end() && it->second.min == 0 && it->second.max == 0;
  };
  std::set<std::string> seen;
  for (size_t d = 0; d < a.indices.size(); ++d) {
    const AffineIndex& idx = a.indices[d];
    std::string v;
    if (!ranges) {
      if (!idx.isSingleVar(&v) || !seen.insert(v).second) return false;
    } else {
      if (!idx.affine || idx.constant != 0) return false;
      int live = 0;
      for (const auto& kv : idx.coeff) {
        if (unit(kv.first)) continue;
        if (kv.second != 1) return false;
        v = kv.first;
        ++live;
      }
      if (live > 1) return false;
      if (live == 0) {  // the constant 0: only a dimension of extent 1 can be dropped
        if (sym->shape[d] != 1) return false;
        continue;
      }
      if (!seen.insert(v).second) return false;
    }
    op->vars.push_back(v);
    op->shape.push_back(sym->shape[d]);
    op->strides.push_back(strides[d]);
  }
  return true;
}

int posOf(const std::vector<std::string>& vars, const std::string& v) {
  auto it = std::find(vars.begin(), vars.end(), v);
  return it == vars.end() ? -1 : (int)(it - vars.begin());
}

// Flattens `group` (given in the order it appears in `op`) to one strided dimension of `op`:
// consecutive positions, row-major.  Returns false if the variables are not adjacent.
bool flatten(const Operand& op, const std::vector<std::string>& group, int64_t* extent,
             int64_t* stride) {
  *extent = 1;
  *stride = 0;
  if (group.empty()) return true;
  std::vector<int> pos;
  for (const auto& v : group) {
    int p = posOf(op.vars, v);
    if (p < 0) return false;
    pos.push_back(p);
  }
  for (size_t i = 1; i < pos.size(); ++i)
    if (pos[i] != pos[i - 1] + 1) return false;
  for (int p : pos) *extent *= op.shape[p];
  *stride = op.strides[pos.back()];
  return true;
}

// The variables of `group` ordered as they appear in `op`.
std::vector<std::string> orderedIn(const Operand& op, const std::set<std::string>& group) {
  std::vector<std::string> r;
  for (const auto& v : op.vars)
    if (group.count(v)) r.push_back(v);
  return r;
}

bool sameOrder(const std::vector<std::string>& a, const std::vector<std::string>& b) { return a == b; }

// ----------------------------------------------------------------------------------------------
// reduction statement: tensordot / contraction
// ----------------------------------------------------------------------------------------------
bool matchProduct(const DefAnalysis& def, const StatementAnalysis& st, MatchedLaunch* out,
                  std::string* why) {
  const TreeRef rhs = lang::Comprehension(st.tree).rhs();
  if (rhs->kind() != '*' || rhs->trees().size() != 2 || rhs->tree(0)->kind() != lang::TK_ACCESS ||
      rhs->tree(1)->kind() != lang::TK_ACCESS || st.reads.size() != 2) {
    *why = "the right-hand side is not a product of two tensor accesses";
    return false;
  }
  Operand A, B, O;
  const TensorSymbol* osym = def.find(st.lhs);
  O.tensor = st.lhs;
  O.value = valueIndex(def, st.lhs);
  std::vector<std::string> reductionVars = st.reductionVars;
  if (plainOperand(def, st.reads[0], &A) && plainOperand(def, st.reads[1], &B)) {
    O.vars = st.lhsIndices;
    O.shape = osym->shape;
    O.strides = makeStridesFromSizes(O.shape);
  } else {
    // second reading: variables that only take the value 0 are that constant
    A = Operand();
    B = Operand();
    if (!plainOperand(def, st.reads[0], &A, &st.ranges) || !plainOperand(def, st.reads[1], &B, &st.ranges)) {
      *why = "an operand index is not a plain index variable";
      return false;
    }
    auto unit = [&](const std::string& v) { return st.ranges.at(v).min == 0 && st.ranges.at(v).max == 0; };
    const std::vector<int64_t> ostrides = makeStridesFromSizes(osym->shape);
    for (size_t d = 0; d < st.lhsIndices.size(); ++d) {
      if (unit(st.lhsIndices[d]) && osym->shape[d] == 1) continue;
      O.vars.push_back(st.lhsIndices[d]);
      O.shape.push_back(osym->shape[d]);
      O.strides.push_back(ostrides[d]);
    }
    reductionVars.clear();
    for (const auto& v : st.reductionVars)
      if (!unit(v)) reductionVars.push_back(v);
  }
  {
    std::set<std::string> seen(O.vars.begin(), O.vars.end());
    if (seen.size() != O.vars.size()) {
      *why = "an output index is repeated";
      return false;
    }
  }
  if (!isFloat32(def.find(A.tensor)) || !isFloat32(def.find(B.tensor)) || !isFloat32(osym)) {
    *why = "only float32 tensors are supported";
    return false;
  }
  // every index must start at 0 and span the tensors' full extents (no where-clause windows)
  for (const auto& kv : st.ranges)
    if (kv.second.min != 0) {
      *why = "index " + kv.first + " does not start at 0";
      return false;
    }
  auto fullExtent = [&](const Operand& op) {
    for (size_t d = 0; d < op.vars.size(); ++d)
      if (st.ranges.at(op.vars[d]).extent() != op.shape[d]) return false;
    return true;
  };
  if (!fullExtent(A) || !fullExtent(B)) {
    *why = "an index covers only part of an operand dimension";
    return false;
  }

  std::set<std::string> batch, mset, nset, kset;
  for (const auto& v : O.vars) {
    const bool a = posOf(A.vars, v) >= 0, b = posOf(B.vars, v) >= 0;
    if (a && b) batch.insert(v);
    else if (a) mset.insert(v);
    else if (b) nset.insert(v);
    else { *why = "output index " + v + " appears in no operand"; return false; }
  }
  for (const auto& v : reductionVars) {
    if (posOf(A.vars, v) >= 0 && posOf(B.vars, v) >= 0) kset.insert(v);
    else { *why = "reduction index " + v + " does not appear in both operands"; return false; }
  }
  if (kset.empty()) { *why = "no reduction index"; return false; }
  for (const auto& v : A.vars)
    if (!batch.count(v) && !mset.count(v) && !kset.count(v)) { *why = "unclassified index"; return false; }
  for (const auto& v : B.vars)
    if (!batch.count(v) && !nset.count(v) && !kset.count(v)) { *why = "unclassified index"; return false; }

  // A free index that leads the output and one operand while the other free indices of that operand sit behind
  // an index of the OTHER operand (d_I(n, c, hw) +=! d_O(n, r_m, hw) * W1(r_m, c): n, then c, then hw) is a batch
  // index over which the other operand is shared (batch stride 0).
  bool aLacksBatch = false, bLacksBatch = false;
  {
    auto contiguousIn = [&](const Operand& op, const std::set<std::string>& g) {
      int64_t e, sd;
      return flatten(op, orderedIn(op, g), &e, &sd);
    };
    if (batch.empty() && (!contiguousIn(O, mset) || !contiguousIn(O, nset))) {
      for (size_t i = 0; i < O.vars.size(); ++i) {
        const std::string v = O.vars[i];
        if (mset.count(v) && !bLacksBatch && !aLacksBatch && i < A.vars.size() && A.vars[i] == v) {
          mset.erase(v); batch.insert(v); bLacksBatch = true;
        } else if (mset.count(v) && bLacksBatch && i < A.vars.size() && A.vars[i] == v) {
          mset.erase(v); batch.insert(v);
        } else if (nset.count(v) && !aLacksBatch && !bLacksBatch && i < B.vars.size() && B.vars[i] == v) {
          nset.erase(v); batch.insert(v); aLacksBatch = true;
        } else if (nset.count(v) && aLacksBatch && i < B.vars.size() && B.vars[i] == v) {
          nset.erase(v); batch.insert(v);
        } else {
          break;
        }
        if (contiguousIn(O, mset) && contiguousIn(O, nset)) break;
      }
    }
  }

  // The group that is outer in O plays "M" and its operand plays "A" (multiplication commutes).
  if (!mset.empty() && !nset.empty()) {
    const int firstM = posOf(O.vars, *orderedIn(O, mset).begin());
    const int firstN = posOf(O.vars, *orderedIn(O, nset).begin());
    if (firstN < firstM) {
      std::swap(A, B);
      std::swap(mset, nset);
      std::swap(aLacksBatch, bLacksBatch);
    }
  }

  tcb200_problem_t& p = out->problem;
  memset(&p, 0, sizeof(p));
  p.accumulate = st.assignment == lang::TK_PLUS_EQ ? 1 : 0;
  out->output = O.value;

  // ---- tensordot: trailing batch indices innermost in all three tensors -----------------------
  std::vector<std::string> inner;
  for (int i = (int)O.vars.size() - 1; i >= 0 && batch.count(O.vars[i]); --i)
    inner.insert(inner.begin(), O.vars[i]);
  if (!inner.empty() && !aLacksBatch && !bLacksBatch) {
    auto tail = [&](const Operand& op) {
      if (op.vars.size() < inner.size()) return false;
      return std::equal(inner.begin(), inner.end(), op.vars.end() - inner.size());
    };
    std::set<std::string> innerSet(inner.begin(), inner.end()), outer;
    for (const auto& v : batch)
      if (!innerSet.count(v)) outer.insert(v);
    // layouts: O = [outer, M, N, inner]  A = [outer, M, K, inner]  B = [outer, K, N, inner]
    auto layout = [&](const Operand& op, const std::set<std::string>& g1,
                      const std::set<std::string>& g2) {
      std::vector<std::string> expect = orderedIn(O, outer);
      if (!sameOrder(orderedIn(op, outer), expect)) return false;
      std::vector<std::string> a = orderedIn(op, g1), b = orderedIn(op, g2);
      expect.insert(expect.end(), a.begin(), a.end());
      expect.insert(expect.end(), b.begin(), b.end());
      expect.insert(expect.end(), inner.begin(), inner.end());
      return op.vars == expect;
    };
    if (tail(A) && tail(B) && layout(O, mset, nset) && layout(A, mset, kset) && layout(B, kset, nset) &&
        sameOrder(orderedIn(A, mset), orderedIn(O, mset)) &&
        sameOrder(orderedIn(B, nset), orderedIn(O, nset)) &&
        sameOrder(orderedIn(A, kset), orderedIn(B, kset))) {
      auto prod = [&](const std::set<std::string>& g) {
        int64_t e = 1;
        for (const auto& v : g) e *= st.ranges.at(v).extent();
        return e;
      };
      if (!p.accumulate) {
        p.family = TCB200_FAMILY_TENSORDOT;
        p.td[0] = prod(outer);
        p.td[1] = prod(mset);
        p.td[2] = prod(kset);
        p.td[3] = prod(nset);
        p.td[4] = prod(innerSet);
        out->inputs = {A.value, B.value};
        return true;
      }
    }
    // not the tensordot layout: fall through and try to see it as a batched contraction
  }

  // ---- strided-batched contraction ----------------------------------------------------------------
  int64_t eB, eM, eN, eK, sBo, sBa, sBb, sMo, sMa, sNo, sNb, sKa, sKb;
  std::vector<std::string> bo = orderedIn(O, batch), mo = orderedIn(O, mset), no = orderedIn(O, nset),
                           ko = orderedIn(A, kset);
  if ((!aLacksBatch && !sameOrder(orderedIn(A, batch), bo)) || (!bLacksBatch && !sameOrder(orderedIn(B, batch), bo)) ||
      !sameOrder(orderedIn(A, mset), mo) || !sameOrder(orderedIn(B, nset), no) ||
      !sameOrder(orderedIn(B, kset), ko)) {
    *why = "index groups are ordered differently in the operands";
    return false;
  }
  int64_t e2;
  // Reduction indices that lead both operands but are separated from the rest of the reduction by a free index
  // (d_W1(m, c) +=! d_O(r_n, m, r_hw) * I(r_n, c, r_hw): r_n in front, r_hw behind m / c) act as a batch index
  // that is reduced as well: the launch runs one contraction per value of them and adds the results.
  std::vector<std::string> rb;
  if (bo.empty() && (!flatten(A, ko, &eK, &sKa) || !flatten(B, ko, &e2, &sKb))) {
    while (rb.size() < ko.size() && rb.size() < A.vars.size() && rb.size() < B.vars.size() &&
           A.vars[rb.size()] == ko[rb.size()] && B.vars[rb.size()] == ko[rb.size()])
      rb.push_back(ko[rb.size()]);
    if (rb.empty() || rb.size() == ko.size()) {
      *why = "the reduction indices are not contiguous in a tensor, so they do not flatten to one dimension";
      return false;
    }
    ko.erase(ko.begin(), ko.begin() + rb.size());
  }
  sBa = sBb = 0;
  if (!flatten(O, bo, &eB, &sBo) || (!aLacksBatch && !flatten(A, bo, &e2, &sBa)) ||
      (!bLacksBatch && !flatten(B, bo, &e2, &sBb)) || !flatten(O, mo, &eM, &sMo) || !flatten(A, mo, &e2, &sMa) || !flatten(O, no, &eN, &sNo) ||
      !flatten(B, no, &e2, &sNb) || !flatten(A, ko, &eK, &sKa) || !flatten(B, ko, &e2, &sKb)) {
    *why = "an index group is not contiguous in a tensor, so it does not flatten to one dimension";
    return false;
  }
  if (!rb.empty()) {
    int64_t eRa, eRb;
    if (!flatten(A, rb, &eRa, &sBa) || !flatten(B, rb, &eRb, &sBb) || eRa != eRb) {
      *why = "the leading reduction indices do not flatten to one dimension";
      return false;
    }
    eB = eRa;
    sBo = 0;
  }
  // batch indices must be the leading dimensions (uniform batch stride)
  for (size_t i = 0; i < bo.size(); ++i)
    if (O.vars[i] != bo[i] || (!aLacksBatch && A.vars[i] != bo[i]) || (!bLacksBatch && B.vars[i] != bo[i])) {
      *why = "batch indices are not the leading dimensions of all three tensors";
      return false;
    }
  // C: n innermost (or absent), m next
  if (!no.empty() && sNo != 1) { *why = "output columns are not contiguous"; return false; }
  if (no.empty() && !mo.empty() && sMo != 1) { *why = "output is not dense"; return false; }
  p.family = TCB200_FAMILY_CONTRACTION;
  p.batch = eB; p.M = eM; p.N = eN; p.K = eK;
  p.stride_a = bo.empty() && rb.empty() ? 0 : sBa;
  p.stride_b = bo.empty() && rb.empty() ? 0 : sBb;
  p.stride_c = bo.empty() ? 0 : sBo;
  p.batch_reduce = rb.empty() ? 0 : 1;
  p.ldc = no.empty() ? 1 : (mo.empty() ? eN : sMo);
  // A: k innermost -> k-major with row pitch = stride of m; else m innermost with pitch = stride of k
  if (sKa == 1) { p.a_k_major = 1; p.lda = mo.empty() ? eK : sMa; }
  else if (mo.empty() || sMa == 1) { p.a_k_major = 0; p.lda = sKa; }
  else { *why = "neither index group of the first operand is contiguous"; return false; }
  if (sKb == 1) { p.b_k_major = 1; p.ldb = no.empty() ? eK : sNb; }
  else if (no.empty() || sNb == 1) { p.b_k_major = 0; p.ldb = sKb; }
  else { *why = "neither index group of the second operand is contiguous"; return false; }
  out->inputs = {A.value, B.value};
  return true;
}

// ----------------------------------------------------------------------------------------------
// reduction statement: (grouped) convolution
// ----------------------------------------------------------------------------------------------
bool matchConv(const DefAnalysis& def, const StatementAnalysis& st, MatchedLaunch* out) {
  const TreeRef rhs = lang::Comprehension(st.tree).rhs();
  if (rhs->kind() != '*' || rhs->trees().size() != 2 || st.reads.size() != 2) return false;
  if (rhs->tree(0)->kind() != lang::TK_ACCESS || rhs->tree(1)->kind() != lang::TK_ACCESS) return false;
  for (int swap = 0; swap < 2; ++swap) {
    const TensorAccess& I = st.reads[swap], &W = st.reads[1 - swap];
    const TensorSymbol* isym = def.find(I.tensor), *wsym = def.find(W.tensor), *osym = def.find(st.lhs);
    if (!isym || !wsym || !isFloat32(isym) || !isFloat32(wsym) || !isFloat32(osym)) continue;
    const size_t r = st.lhsIndices.size();
    const bool grouped = r == 5;
    if (!(r == 5 || r == 4) || I.indices.size() != r || W.indices.size() != r) continue;
    const int g = grouped ? 1 : 0;  // extra leading index
    // O = (n, [g,] f, h, w)   I = (n, [g,] c, h+kh, w+kw)   W = ([g,] f, c, kh, kw)
    const std::string &n = st.lhsIndices[0], &f = st.lhsIndices[1 + g], &h = st.lhsIndices[2 + g],
                      &w = st.lhsIndices[3 + g];
    std::string v, c, kh, kw;
    auto single = [&](const AffineIndex& a, const std::string& want) {
      return a.isSingleVar(&v) && v == want;
    };
    // stride * x + other (tc/library/convolution.h:27-31 writes the strides as literal factors)
    auto sumOf = [&](const AffineIndex& a, const std::string& x, std::string* other, int64_t* stride) {
      if (!a.affine || a.constant != 0 || a.coeff.size() != 2) return false;
      auto it = a.coeff.find(x);
      if (it == a.coeff.end() || it->second < 1 || it->second > (1 << 16)) return false;
      *stride = it->second;
      for (const auto& kv : a.coeff)
        if (kv.first != x) {
          if (kv.second != 1) return false;
          *other = kv.first;
        }
      return true;
    };
    if (!single(I.indices[0], n)) continue;
    if (grouped && (!single(I.indices[1], st.lhsIndices[1]) || !single(W.indices[0], st.lhsIndices[1]))) continue;
    if (!I.indices[1 + g].isSingleVar(&c)) continue;
    int64_t sh = 1, sw = 1;
    if (!sumOf(I.indices[2 + g], h, &kh, &sh) || !sumOf(I.indices[3 + g], w, &kw, &sw)) continue;
    if (!single(W.indices[0 + g], f) || !single(W.indices[1 + g], c) || !single(W.indices[2 + g], kh) ||
        !single(W.indices[3 + g], kw))
      continue;
    std::set<std::string> red(st.reductionVars.begin(), st.reductionVars.end());
    if (red != std::set<std::string>{c, kh, kw}) continue;
    bool zeroBased = true;
    for (const auto& kv : st.ranges) zeroBased = zeroBased && kv.second.min == 0;
    if (!zeroBased) continue;
    tcb200_problem_t& p = out->problem;
    memset(&p, 0, sizeof(p));
    p.family = TCB200_FAMILY_GROUP_CONV;
    p.accumulate = st.assignment == lang::TK_PLUS_EQ ? 1 : 0;
    p.conv[0] = isym->shape[0];
    p.conv[1] = grouped ? isym->shape[1] : 1;
    p.conv[2] = isym->shape[1 + g];
    p.conv[3] = wsym->shape[0 + g];
    p.conv[4] = isym->shape[2 + g];
    p.conv[5] = isym->shape[3 + g];
    p.conv[6] = wsym->shape[2 + g];
    p.conv[7] = wsym->shape[3 + g];
    // output must be the full valid window
    p.conv_stride[0] = sh;
    p.conv_stride[1] = sw;
    if (p.conv[4] < p.conv[6] || p.conv[5] < p.conv[7]) continue;
    if (st.ranges.at(h).extent() != (p.conv[4] - p.conv[6]) / sh + 1 ||
        st.ranges.at(w).extent() != (p.conv[5] - p.conv[7]) / sw + 1 || st.ranges.at(c).extent() != p.conv[2])
      continue;
    out->inputs = {valueIndex(def, I.tensor), valueIndex(def, W.tensor)};
    out->output = valueIndex(def, st.lhs);
    return true;
  }
  return false;
}

// ----------------------------------------------------------------------------------------------
// reduction statement: sum of one tensor over a contiguous group of its indices
//   O(kept leading..., kept trailing...) +=! I(kept leading..., reduced..., kept trailing...)
// (C +=! A(r_m), C(m) +=! A(m, r_n): test/test_tc_mapper_harness-inl.h:60-146)
// ----------------------------------------------------------------------------------------------
bool matchReduction(const DefAnalysis& def, const StatementAnalysis& st, MatchedLaunch* out, std::string* why) {
  const TreeRef rhs = lang::Comprehension(st.tree).rhs();
  if (rhs->kind() != lang::TK_ACCESS || st.reads.size() != 1) return false;
  const TensorAccess& I = st.reads[0];
  const TensorSymbol* isym = def.find(I.tensor), *osym = def.find(st.lhs);
  if (!isym || !osym) return false;
  if (!isFloat32(isym) || !isFloat32(osym)) { *why = "only float32 tensors are supported"; return false; }
  // every input index a distinct variable spanning its whole dimension from 0
  std::vector<std::string> vars;
  for (size_t d = 0; d < I.indices.size(); ++d) {
    std::string v;
    if (!I.indices[d].isSingleVar(&v)) { *why = "an operand index is not a plain index variable"; return false; }
    if (std::find(vars.begin(), vars.end(), v) != vars.end()) { *why = "an operand index is repeated"; return false; }
    const IndexRange& r = st.ranges.at(v);
    if (r.min != 0 || r.extent() != isym->shape[d]) { *why = "index " + v + " does not span its dimension"; return false; }
    vars.push_back(v);
  }
  // the kept indices, in the input's order, must be exactly the output's indices; an output index that
  // is not an input index (C(i) +=! A(r_m) where i in 0:1) must have extent 1
  std::set<std::string> red(st.reductionVars.begin(), st.reductionVars.end());
  std::vector<std::string> kept, lhsKept;
  for (const auto& v : vars)
    if (!red.count(v)) kept.push_back(v);
  for (const auto& v : st.lhsIndices) {
    if (std::find(vars.begin(), vars.end(), v) != vars.end()) lhsKept.push_back(v);
    else if (st.ranges.at(v).min != 0 || st.ranges.at(v).extent() != 1) {
      *why = "output index " + v + " does not index the operand";
      return false;
    }
  }
  if (kept != lhsKept) { *why = "the output's indices are not the operand's kept indices in the same order"; return false; }
  for (const auto& v : red)
    if (std::find(vars.begin(), vars.end(), v) == vars.end()) { *why = "a reduction index does not index the operand"; return false; }
  if (red.empty()) return false;
  // reduced indices must be one contiguous run of the operand's dimensions
  int64_t A = 1, C = 1, B = 1;
  int phase = 0;  // 0: leading kept, 1: reduced, 2: trailing kept
  for (size_t d = 0; d < vars.size(); ++d) {
    const bool r = red.count(vars[d]) != 0;
    if (phase == 0 && r) phase = 1;
    else if (phase == 1 && !r) phase = 2;
    else if (phase == 2 && r) { *why = "the reduced indices are not adjacent dimensions of the operand"; return false; }
    (phase == 0 ? A : phase == 1 ? C : B) *= isym->shape[d];
  }
  tcb200_problem_t& p = out->problem;
  memset(&p, 0, sizeof(p));
  p.family = TCB200_FAMILY_REDUCTION;
  switch (st.assignment) {
    case lang::TK_MAX_EQ: case lang::TK_MAX_EQ_B: p.reduce_op = TCB200_REDUCE_MAX; break;
    case lang::TK_MIN_EQ: case lang::TK_MIN_EQ_B: p.reduce_op = TCB200_REDUCE_MIN; break;
    case lang::TK_TIMES_EQ: case lang::TK_TIMES_EQ_B: p.reduce_op = TCB200_REDUCE_PROD; break;
    default: p.reduce_op = TCB200_REDUCE_SUM; break;
  }
  // without '!' the output's old value takes part in the reduction
  p.accumulate = st.assignment == lang::TK_PLUS_EQ || st.assignment == lang::TK_MAX_EQ ||
                 st.assignment == lang::TK_MIN_EQ || st.assignment == lang::TK_TIMES_EQ;
  p.red[0] = A; p.red[1] = C; p.red[2] = B;
  out->inputs = {valueIndex(def, I.tensor)};
  out->output = valueIndex(def, st.lhs);
  return true;
}

// ----------------------------------------------------------------------------------------------
// elementwise follow-ups on the tensor just produced
// ----------------------------------------------------------------------------------------------
// O(idx) = O(idx) [+ Bias(sub)]: returns the access that is NOT the self access, or null.
bool isSelfAccess(const StatementAnalysis& st, const TensorAccess& a) {
  if (a.tensor != st.lhs || a.indices.size() != st.lhsIndices.size()) return false;
  for (size_t i = 0; i < a.indices.size(); ++i) {
    std::string v;
    if (!a.indices[i].isSingleVar(&v) || v != st.lhsIndices[i]) return false;
  }
  return true;
}

// Positions (in the left-hand side) of the variables a bias access is indexed by; empty = no match.
std::vector<int> biasPositions(const StatementAnalysis& st, const TensorAccess& b) {
  std::vector<int> pos;
  for (const auto& idx : b.indices) {
    std::string v;
    if (!idx.isSingleVar(&v)) return {};
    int p = posOf(st.lhsIndices, v);
    if (p < 0) return {};
    pos.push_back(p);
  }
  return pos;
}

bool matchBias(const DefAnalysis& def, const StatementAnalysis& st, MatchedLaunch* launch) {
  if (st.assignment != '=' || !st.reductionVars.empty() || st.reads.size() != 2) return false;
  const TreeRef rhs = lang::Comprehension(st.tree).rhs();
  if (rhs->kind() != '+' || rhs->trees().size() != 2) return false;
  if (rhs->tree(0)->kind() != lang::TK_ACCESS || rhs->tree(1)->kind() != lang::TK_ACCESS) return false;
  const int self = isSelfAccess(st, st.reads[0]) ? 0 : (isSelfAccess(st, st.reads[1]) ? 1 : -1);
  if (self < 0) return false;
  const TensorAccess& bias = st.reads[1 - self];
  const TensorSymbol* bsym = def.find(bias.tensor);
  if (!bsym || !bsym->isInput || !isFloat32(bsym)) return false;
  std::vector<int> pos = biasPositions(st, bias);
  if (pos.empty()) return false;
  tcb200_problem_t& p = launch->problem;
  if (p.epilogue != TCB200_EPI_NONE) return false;
  const int rank = (int)st.lhsIndices.size();
  if (p.family == TCB200_FAMILY_GROUP_CONV) {
    // B(g, f) on O(n, g, f, h, w); B(f) on O(n, f, h, w)
    const bool grouped = rank == 5;
    if (grouped ? (pos != std::vector<int>{1, 2}) : (pos != std::vector<int>{1})) return false;
  } else if (p.family == TCB200_FAMILY_CONTRACTION) {
    // bias over exactly the column group (trailing dims of O) or exactly the row group
    // (the dims between the batch dims and the column group); count dims from the launch's sizes
    int64_t cols = 1, rows = 1;
    int nColDims = 0;
    const TensorSymbol* osym = def.find(st.lhs);
    for (int d = rank - 1; d >= 0 && cols < p.N; --d) { cols *= osym->shape[d]; ++nColDims; }
    if (cols != p.N) return false;
    int nRowDims = 0;
    for (int d = rank - 1 - nColDims; d >= 0 && rows < p.M; --d) { rows *= osym->shape[d]; ++nRowDims; }
    std::vector<int> colPos, rowPos;
    for (int d = rank - nColDims; d < rank; ++d) colPos.push_back(d);
    for (int d = rank - nColDims - nRowDims; d < rank - nColDims; ++d) rowPos.push_back(d);
    if (pos == colPos && p.N > 1) p.bias_on_m = 0;
    else if (pos == rowPos && rows == p.M && p.batch == 1) p.bias_on_m = 1;
    else return false;
  } else {
    return false;
  }
  p.epilogue = TCB200_EPI_BIAS;
  launch->inputs.push_back(valueIndex(def, bias.tensor));
  return true;
}

bool matchRelu(const StatementAnalysis& st, MatchedLaunch* launch) {
  if (st.assignment != '=' || !st.reductionVars.empty() || st.reads.size() != 1) return false;
  const TreeRef rhs = lang::Comprehension(st.tree).rhs();
  if (rhs->kind() != lang::TK_BUILT_IN) return false;
  lang::BuiltIn b(rhs);
  if (b.name() != "fmax" || b.arguments().size() != 2) return false;
  int selfArg = -1;
  for (int i = 0; i < 2; ++i)
    if (b.arguments()[i]->kind() == lang::TK_ACCESS) selfArg = i;
  if (selfArg < 0 || !isSelfAccess(st, st.reads[0])) return false;
  const TreeRef zero = b.arguments()[1 - selfArg];
  if (zero->kind() != lang::TK_CONST || lang::Const(zero).value() != 0.0) return false;
  tcb200_problem_t& p = launch->problem;
  if (p.family == TCB200_FAMILY_TENSORDOT) return false;
  if (p.epilogue == TCB200_EPI_NONE && p.family == TCB200_FAMILY_CONTRACTION) p.epilogue = TCB200_EPI_RELU;
  else if (p.epilogue == TCB200_EPI_BIAS) p.epilogue = TCB200_EPI_BIAS_RELU;
  else return false;
  return true;
}

// O(i, j, ...) = I(i, j, ...): the same plain indices in the same order over the whole of both tensors.
bool matchCopy(const DefAnalysis& def, const StatementAnalysis& st, MatchedLaunch* out) {
  if (st.assignment != '=' || !st.reductionVars.empty() || st.reads.size() != 1) return false;
  const TreeRef rhs = lang::Comprehension(st.tree).rhs();
  if (rhs->kind() != lang::TK_ACCESS) return false;
  const TensorAccess& I = st.reads[0];
  const TensorSymbol* isym = def.find(I.tensor), *osym = def.find(st.lhs);
  if (!isym || !osym || I.tensor == st.lhs || !isFloat32(isym) || !isFloat32(osym)) return false;
  if (I.indices.size() != st.lhsIndices.size() || isym->shape != osym->shape) return false;
  int64_t elements = 1;
  for (size_t d = 0; d < I.indices.size(); ++d) {
    std::string v;
    if (!I.indices[d].isSingleVar(&v) || v != st.lhsIndices[d]) return false;
    const IndexRange& r = st.ranges.at(v);
    if (r.min != 0 || r.extent() != isym->shape[d]) return false;
    elements *= isym->shape[d];
  }
  if (elements <= 0) return false;
  tcb200_problem_t& p = out->problem;
  memset(&p, 0, sizeof(p));
  p.family = TCB200_FAMILY_COPY;
  p.red[0] = elements;
  out->inputs = {valueIndex(def, I.tensor)};
  out->output = valueIndex(def, st.lhs);
  return true;
}

}  // namespace

std::vector<MatchedLaunch> matchKernels(const DefAnalysis& def) {
  std::vector<MatchedLaunch> launches;
  for (size_t s = 0; s < def.statements.size(); ++s) {
    const StatementAnalysis& st = def.statements[s];
    const bool reduction = !st.reductionVars.empty();
    if (reduction) {
      const bool sum = st.assignment == lang::TK_PLUS_EQ_B || st.assignment == lang::TK_PLUS_EQ;
      MatchedLaunch l;
      std::string why;
      if (!sum) {  // max=, min=, *=: the reduction family takes them for one operand
        if (!matchReduction(def, st, &l, &why))
          unmatched(st, why.empty() ? "only sum reductions (+=, +=!) of a product map to a kernel family" : why);
      } else if (!matchConv(def, st, &l) && !matchReduction(def, st, &l, &why)) {
        if (!why.empty()) unmatched(st, why);  // one operand, but not a reduction this backend takes
        if (!matchProduct(def, st, &l, &why)) unmatched(st, why);
      }
      l.statements.push_back((int)s);
      launches.push_back(std::move(l));
      continue;
    }
    // elementwise statement: a whole-tensor copy is a launch of its own, anything else must extend the launch
    // that produced the same tensor just before
    {
      MatchedLaunch copy;
      if (matchCopy(def, st, &copy)) {
        copy.statements.push_back((int)s);
        launches.push_back(std::move(copy));
        continue;
      }
    }
    if (launches.empty() || def.outputs.empty() ||
        launches.back().output != valueIndex(def, st.lhs))
      unmatched(st, "an elementwise statement is only supported as the epilogue of the reduction "
                    "that produced the same tensor, or as a copy of a whole tensor");
    MatchedLaunch& l = launches.back();
    const StatementAnalysis& producer = def.statements[l.statements.front()];
    if (producer.lhsIndices.size() != st.lhsIndices.size())
      unmatched(st, "epilogue rank differs from its producer");
    for (const auto& v : st.lhsIndices)
      if (st.ranges.at(v).min != 0) unmatched(st, "epilogue covers only part of the tensor");
    if (!matchBias(def, st, &l) && !matchRelu(st, &l))
      unmatched(st, "not a '+ bias' or 'fmax(., 0)' epilogue");
    l.statements.push_back((int)s);
  }
  if (launches.empty() && !def.statements.empty())
    unmatched(def.statements.front(), "no reduction statement");
  return launches;
}

}  // namespace tc
