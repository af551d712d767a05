/*
 * CPU restatement of what the five Tensor Comprehensions on the hot path mean.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing the product ships may link, import or call
 * this file: it is the checker for the CUDA kernels (tests, the smoke check and
 * the cpu_baseline leg of the benchmark), never the thing measured or shipped.
 *
 * Each function is the loop nest that the reference's front-end lowers the TC
 * statement to: a separate zero-initialisation nest for a "+=!" reduction,
 * then an update nest whose loops run over the output indices in left-to-right
 * order with the reduction indices innermost in order of first use
 * (known answers: test/test_core.cc:93-127 for chained matmul,
 * test/test_core.cc:175-213 for group convolution; init identity
 * tc/core/tc2halide.cc:573-601; loop-order convention tc/core/tc2halide.cc:729-754;
 * valid-convolution extents (H-KH)+1 from test/test_inference.cc:190-212).
 * Tensors are dense row-major (docs/source/semantics.rst:17-19).
 *
 * Two accumulation flavours per nest: float (what the reference's generated
 * code does, one fused-or-not multiply-add at a time in textual order) and
 * double (used only to budget the rounding error of the float flavours).
 *
 * Parity status: the reference holds no numeric golden vector for this path
 * (its numeric tests are randomised comparisons against ATen), so none is stored
 * here either: tests/golden holds only front-end trees.  The structural known
 * answers above pin the loop order, and tests/test_oracle_cpu.py compares these
 * nests, live, with ATen-CPU (the library the reference's own harness compares
 * against: tc/benchmarks/batchmatmul.cc:67, tmm.cc:66, MLP_model.cc:537-541,
 * group_convolution.cc:83-101) on the seeded inputs of every benchmark.
 */
#include <stddef.h>
#include <stdint.h>

#define IDX2(i, j, d1) ((size_t)(i) * (d1) + (j))

/* O(n,c1,c3,h,w) +=! I0(n,c1,r_c2,h,w) * I1(n,r_c2,c3,h,w)   tc/examples/tensordot.cc:41-47 */
void oracle_tensordot_f32(const float* I0, const float* I1, float* O,
                          int64_t N, int64_t C1, int64_t C2, int64_t C3,
                          int64_t H, int64_t W, int accumulate_double) {
  const int64_t P = H * W;
  for (int64_t n = 0; n < N; ++n)
    for (int64_t c1 = 0; c1 < C1; ++c1)
      for (int64_t c3 = 0; c3 < C3; ++c3)
        for (int64_t p = 0; p < P; ++p)
          O[((n * C1 + c1) * C3 + c3) * P + p] = 0.0f;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t c1 = 0; c1 < C1; ++c1)
      for (int64_t c3 = 0; c3 < C3; ++c3)
        for (int64_t p = 0; p < P; ++p) {
          float* o = &O[((n * C1 + c1) * C3 + c3) * P + p];
          if (accumulate_double) {
            double acc = 0.0;
            for (int64_t c2 = 0; c2 < C2; ++c2)
              acc += (double)I0[((n * C1 + c1) * C2 + c2) * P + p] *
                     (double)I1[((n * C2 + c2) * C3 + c3) * P + p];
            *o = (float)acc;
          } else {
            float acc = *o;
            for (int64_t c2 = 0; c2 < C2; ++c2)
              acc = acc + I0[((n * C1 + c1) * C2 + c2) * P + p] *
                              I1[((n * C2 + c2) * C3 + c3) * P + p];
            *o = acc;
          }
        }
}

/* Z(b,n,k) +=! X(b,n,r_m) * Y(b,r_m,k)   tc/benchmarks/batchmatmul.cc:80-84 */
void oracle_batchmatmul_f32(const float* X, const float* Y, float* Z,
                            int64_t B, int64_t N, int64_t M, int64_t K,
                            int accumulate_double) {
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t n = 0; n < N; ++n)
      for (int64_t k = 0; k < K; ++k) {
        const float* x = X + (b * N + n) * M;
        const float* y = Y + b * M * K + k;
        if (accumulate_double) {
          double acc = 0.0;
          for (int64_t m = 0; m < M; ++m) acc += (double)x[m] * (double)y[m * K];
          Z[(b * N + n) * K + k] = (float)acc;
        } else {
          float acc = 0.0f;
          for (int64_t m = 0; m < M; ++m) acc = acc + x[m] * y[m * K];
          Z[(b * N + n) * K + k] = acc;
        }
      }
}

/* C(m,n) +=! A(m,r_k) * B(n,r_k)   tc/benchmarks/tmm.cc:79-83 */
void oracle_tmm_f32(const float* A, const float* B, float* C,
                    int64_t M, int64_t N, int64_t K, int accumulate_double) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      const float* a = A + m * K;
      const float* b = B + n * K;
      if (accumulate_double) {
        double acc = 0.0;
        for (int64_t k = 0; k < K; ++k) acc += (double)a[k] * (double)b[k];
        C[IDX2(m, n, N)] = (float)acc;
      } else {
        float acc = 0.0f;
        for (int64_t k = 0; k < K; ++k) acc = acc + a[k] * b[k];
        C[IDX2(m, n, N)] = acc;
      }
    }
}

/* O(n,g,f,h,w) +=! I(n,g,r_c,SH*h+r_kh,SW*w+r_kw) * W1(g,f,r_c,r_kh,r_kw)
 * O(n,g,f,h,w)  = O(n,g,f,h,w) + B(g,f)        tc/benchmarks/group_convolution.cc:124-132;
 * the strides are the literal factors of tc/library/convolution.h:27-31 and
 * tc/library/group_convolution.h:26-44.  The extent of h is the largest for which every access
 * stays in bounds: SH*h + (KH-1) <= H-1, i.e. (H-KH)/SH + 1 values (tc/core/tc2halide.cc:270-498).
 * Bias may be NULL (first statement only). */
void oracle_group_conv_strided_f32(const float* I, const float* W1, const float* Bias, float* O,
                                   int64_t N, int64_t G, int64_t C, int64_t F,
                                   int64_t H, int64_t W, int64_t KH, int64_t KW,
                                   int64_t SH, int64_t SW, int accumulate_double) {
  const int64_t OH = (H - KH) / SH + 1, OW = (W - KW) / SW + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t g = 0; g < G; ++g)
      for (int64_t f = 0; f < F; ++f)
        for (int64_t h = 0; h < OH; ++h)
          for (int64_t w = 0; w < OW; ++w) {
            double accd = 0.0;
            float accf = 0.0f;
            for (int64_t c = 0; c < C; ++c)
              for (int64_t kh = 0; kh < KH; ++kh)
                for (int64_t kw = 0; kw < KW; ++kw) {
                  float a = I[(((n * G + g) * C + c) * H + (SH * h + kh)) * W + (SW * w + kw)];
                  float b = W1[(((g * F + f) * C + c) * KH + kh) * KW + kw];
                  if (accumulate_double) accd += (double)a * (double)b;
                  else accf = accf + a * b;
                }
            float r = accumulate_double ? (float)accd : accf;
            if (Bias) r = r + Bias[g * F + f];
            O[(((n * G + g) * F + f) * OH + h) * OW + w] = r;
          }
}

/* O(a,b) +=! I(a,r_c,b): a sum over a contiguous group of the input's indices, the [A][C][B] view of
 * C +=! A(r_m) and C(m) +=! A(m,r_n) (test/test_tc_mapper_harness-inl.h:60-146).  The reduction loop is
 * innermost and runs in index order (tc/core/tc2halide.cc:729-754), starting from the identity 0
 * (tc/core/tc2halide.cc:573-601). */
/* The same nest for the other reduction assignments (tc/lang/tree.h TK_MAX_EQ_B, TK_MIN_EQ_B,
 * TK_TIMES_EQ_B): op 1 = max, 2 = min, 3 = product, starting from the operator's identity
 * (tc/core/tc2halide.cc:573-601). */
void oracle_reduce_op_f32(const float* I, float* O, int64_t A, int64_t C, int64_t B, int op) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t a = 0; a < A; ++a)
    for (int64_t b = 0; b < B; ++b) {
      double acc = op == 1 ? -3.402823466e38 : op == 2 ? 3.402823466e38 : op == 3 ? 1.0 : 0.0;
      for (int64_t c = 0; c < C; ++c) {
        double v = (double)I[(a * C + c) * B + b];
        if (op == 1) acc = v > acc ? v : acc;
        else if (op == 2) acc = v < acc ? v : acc;
        else if (op == 3) acc *= v;
        else acc += v;
      }
      O[a * B + b] = (float)acc;
    }
}

void oracle_reduce_f32(const float* I, float* O, int64_t A, int64_t C, int64_t B, int accumulate_double) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t a = 0; a < A; ++a)
    for (int64_t b = 0; b < B; ++b) {
      double accd = 0.0;
      float accf = 0.0f;
      for (int64_t c = 0; c < C; ++c) {
        float v = I[(a * C + c) * B + b];
        if (accumulate_double) accd += (double)v;
        else accf = accf + v;
      }
      O[a * B + b] = accumulate_double ? (float)accd : accf;
    }
}

/* Unit strides: the benchmark's own form. */
void oracle_group_conv_f32(const float* I, const float* W1, const float* Bias, float* O,
                           int64_t N, int64_t G, int64_t C, int64_t F,
                           int64_t H, int64_t W, int64_t KH, int64_t KW,
                           int accumulate_double) {
  oracle_group_conv_strided_f32(I, W1, Bias, O, N, G, C, F, H, W, KH, KW, 1, 1, accumulate_double);
}

/* O1(b,n) +=! I(b,m) * W1(n,m);  O1(b,n) = O1(b,n) + B1(n);  O1(b,n) = fmax(O1(b,n), 0)
 * tc/library/fcrelu.h:22-28.  relu==0 stops after the bias statement; Bias may be NULL. */
void oracle_fcrelu_f32(const float* I, const float* W1, const float* Bias, float* O,
                       int64_t B, int64_t N, int64_t M, int relu, int accumulate_double) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t n = 0; n < N; ++n) {
      const float* x = I + b * M;
      const float* w = W1 + n * M;
      float r;
      if (accumulate_double) {
        double acc = 0.0;
        for (int64_t m = 0; m < M; ++m) acc += (double)x[m] * (double)w[m];
        r = (float)acc;
      } else {
        float acc = 0.0f;
        for (int64_t m = 0; m < M; ++m) acc = acc + x[m] * w[m];
        r = acc;
      }
      if (Bias) r = r + Bias[n];
      if (relu) r = r > 0.0f ? r : 0.0f; /* fmaxf(r, 0) for non-NaN r */
      O[IDX2(b, n, N)] = r;
    }
}
