// Builders for the comprehension texts of the operator library (tc/library/*.h of the reference).
// The reference keeps every text as a literal with placeholders; here the texts are assembled from
// their parts, so the N-layer fully-connected chains and the strided convolutions share one
// generator each.  Every text below is matched by a kernel family of this backend.
#pragma once

#include <string>
#include <vector>

namespace tc {
namespace library_detail {

// func_fcrelu / func_2fcrelu / func_3fcrelu / func_4fcrelu (tc/library/fcrelu.h:22-28,
// 2fcrelu.h:21-30, 3fcrelu.h:22-34, 4fcrelu.h:21-35): layer l computes
//   Ol(b, x) +=! In(b, y) * Wl(x, y);  Ol(b, x) = Ol(b, x) + Bl(x);  Ol(b, x) = fmax(Ol(b, x), 0)
// with In = I for the first layer and O(l-1) after it; all Ol are outputs.
inline std::string fcreluChain(int layers, const std::string& name) {
  static const char* const kSize[] = {"M", "N", "O", "P", "Q"};
  static const char* const kIdx[] = {"m", "n", "o", "p", "q"};
  std::string params = "float(B," + std::string(kSize[0]) + ") I", outs, body;
  for (int l = 1; l <= layers; ++l) {
    const std::string L = std::to_string(l), in = l == 1 ? "I" : "O" + std::to_string(l - 1);
    const std::string x = kIdx[l], y = kIdx[l - 1], out = "O" + L + "(b, " + x + ")";
    params += ", float(" + std::string(kSize[l]) + "," + kSize[l - 1] + ") W" + L + ", float(" + kSize[l] + ") B" + L;
    outs += (l > 1 ? ", O" : "O") + L;
    body += "  " + out + " +=! " + in + "(b, " + y + ") * W" + L + "(" + x + ", " + y + ")\n";
    body += "  " + out + " = " + out + " + B" + L + "(" + x + ")\n";
    body += "  " + out + " = fmax(" + out + ", 0)\n";
  }
  return "def " + name + "(" + params + ") -> (" + outs + ") {\n" + body + "}\n";
}

// matmul in its four storage forms and its batched form (tc/library/matmul.h:24-45,
// batch_matmul.h:22-26): out(rows, cols) +=! lhs * rhs with an optional leading batch index.
inline std::string matmulText(const std::string& name, bool batched, bool transposeFirst, bool transposeSecond,
                              const char* lhs, const char* rhs, const char* out, const char* rowSize, const char* redSize,
                              const char* colSize, const char* row, const char* red, const char* col) {
  const std::string B = batched ? "B, " : "", b = batched ? "b, " : "";
  auto decl = [&](const char* t, const char* s0, const char* s1) {
    return "float(" + B + s0 + ", " + s1 + ") " + t;
  };
  auto use = [&](const char* t, const char* i0, const char* i1) {
    return std::string(t) + "(" + b + i0 + ", " + i1 + ")";
  };
  const std::string a = transposeFirst ? decl(lhs, redSize, rowSize) : decl(lhs, rowSize, redSize);
  const std::string c = transposeSecond ? decl(rhs, colSize, redSize) : decl(rhs, redSize, colSize);
  const std::string ai = transposeFirst ? use(lhs, red, row) : use(lhs, row, red);
  const std::string ci = transposeSecond ? use(rhs, col, red) : use(rhs, red, col);
  return "def " + name + "(" + a + ", " + c + ") -> (" + out + ") {\n  " + use(out, row, col) + " +=! " + ai + " * " + ci +
         "\n}\n";
}

// convolution / group_convolution with literal strides (tc/library/convolution.h:27-31,
// group_convolution.h:26-34): the image index is  stride * out + tap.
inline std::string conv2d(bool grouped, int strideH, int strideW) {
  const std::string g = grouped ? "g, " : "", G = grouped ? "G," : "";
  const std::string f = grouped ? "f" : "m", F = grouped ? "F" : "M";
  const std::string out = "O(n, " + g + f + ", h, w)";
  std::string s = "def " + std::string(grouped ? "group_convolution" : "convolution") + "(float(N," + G + "C,H,W) I, float(" +
                  G + F + ",C,KH,KW) W1, float(" + G + F + ") B) -> (O) {\n";
  s += "  " + out + " +=! I(n, " + g + "c, " + std::to_string(strideH) + " * h + kh, " + std::to_string(strideW) +
       " * w + kw) * W1(" + g + f + ", c, kh, kw)\n";
  s += "  " + out + " = " + out + " + B(" + g + f + ")\n}\n";
  return s;
}

}  // namespace library_detail
}  // namespace tc
