/*
 * CPU oracle: a plain-C restatement of the eigenmat operations that deepnet's
 * contrastive-divergence path calls.  TEST INFRASTRUCTURE ONLY: it is the checker
 * for the CUDA library and the timed CPU baseline, never a fallback for it.
 *
 * Every function cites the reference lines it follows (paths relative to the
 * reference project).  Matrices are float32, column-major, `size[0]` rows by
 * `size[1]` columns, exactly like `struct eigenmat` (eigenmat/eigenmat.h:11-16).
 *
 * Parity status: the reference's eigenmat.cc needs Eigen, which is neither vendored
 * in the reference nor installed, so it cannot be compiled; this port is pinned
 * against the numpy formulas of the reference's own tests (eigenmat/test.py,
 * cudamat/test_cudamat.py) and, for the random stream, against the published
 * Philox4x32-10 known-answer vectors.  Operations with no reference test
 * (sample_bernoulli, perturb_prob, choose_max*, the parameter update) are
 * "parity unpinned": restated from the source text only.
 *
 * Where eigenmat.cc is wrong or empty the cudamat kernel's meaning is used:
 *   add_row_mult / add_row_vec map the row vector with length h instead of w
 *   (eigenmat/eigenmat.cc:365,384) -> vec[column] as in cudamat_kernels.cu:546-567.
 *
 * Random numbers: eigenmat draws from ziggurat.cc's r4_uni, whose 32-bit SHR3 state
 * is held in an `unsigned long` and is degenerate on LP64.  The oracle therefore
 * takes the uniforms as an argument ("injected uniforms") or draws them from the
 * counter-based Philox4x32-10 stream that the CUDA library uses, so that both sides
 * see the same numbers.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ERROR_INCOMPATIBLE_DIMENSIONS -1
#define ERROR_TRANSPOSED -5
#define ERROR_TRANSPOSEDNESS -7
#define ERROR_UNSUPPORTED -9

typedef struct {
  float* data;
  int size[2];
  int is_trans;
  int owns_data;
} eigenmat;

static inline int same_shape(const eigenmat* a, const eigenmat* b) {
  return a->size[0] == b->size[0] && a->size[1] == b->size[1];
}
static inline long numel(const eigenmat* a) { return (long)a->size[0] * a->size[1]; }

/* ------------------------------------------------------------------ Philox4x32-10 */
/* Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3" (SC'11). */

static inline void philox_round(uint32_t c[4], const uint32_t k[2]) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
  const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
  const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
  const uint32_t n0 = hi1 ^ c[1] ^ k[0];
  const uint32_t n2 = hi0 ^ c[3] ^ k[1];
  c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}

void philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
  uint32_t k[2] = {key[0], key[1]};
  for (int r = 0; r < 10; r++) {
    if (r) { k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u; }
    philox_round(c, k);
  }
  memcpy(out, c, sizeof(c));
}

/* Word -> uniform in (0, 1]: the cudamat mapping (cudamat/cudamat_kernels.cu:120). */
static inline float word_to_uniform(uint32_t x) { return ((float)x + 1.0f) * 2.3283064365386963e-10f; }

/*
 * Stream layout shared with the CUDA library: the uniform of matrix element
 * (row r, column c) in sampling call number `call` under `seed` is word (c & 3) of
 * Philox(ctr = {r, c >> 2, call_lo, call_hi}, key = {seed_lo, seed_hi}).
 * `col0` offsets the column (a rank's first global column in data-parallel runs).
 */
static inline void philox_block(uint64_t seed, uint64_t call, uint32_t r, uint32_t cblk, uint32_t out[4]) {
  const uint32_t ctr[4] = {r, cblk, (uint32_t)call, (uint32_t)(call >> 32)};
  const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  philox4x32_10(ctr, key, out);
}

int philox_uniform(uint64_t seed, uint64_t call, int col0, eigenmat* target) {
  const int h = target->size[0], w = target->size[1];
  #pragma omp parallel for
  for (int c = 0; c < w; c++) {
    const uint32_t gc = (uint32_t)(c + col0);
    for (int r = 0; r < h; r++) {
      uint32_t o[4];
      philox_block(seed, call, (uint32_t)r, gc >> 2, o);
      target->data[(long)c * h + r] = word_to_uniform(o[gc & 3]);
    }
  }
  return 0;
}

/* Standard normals by Box-Muller on word pairs (0,1) and (2,3) of the block: columns
 * 4j, 4j+1 take cos/sin of the first pair, 4j+2, 4j+3 of the second.  cudamat's
 * generator is Box-Muller as well (cudamat/cudamat_kernels.cu:125-143). */
int philox_normal(uint64_t seed, uint64_t call, int col0, eigenmat* target) {
  const int h = target->size[0], w = target->size[1];
  #pragma omp parallel for
  for (int c = 0; c < w; c++) {
    const uint32_t gc = (uint32_t)(c + col0);
    for (int r = 0; r < h; r++) {
      uint32_t o[4];
      philox_block(seed, call, (uint32_t)r, gc >> 2, o);
      const int pair = (gc & 3) >> 1;
      const float u1 = word_to_uniform(o[2 * pair]), u2 = word_to_uniform(o[2 * pair + 1]);
      const float rad = sqrtf(-2.0f * logf(u1));
      const float ang = 6.283185307179586f * u2;
      target->data[(long)c * h + r] = (gc & 1) ? rad * sinf(ang) : rad * cosf(ang);
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ sampling ops */

/* eigenmat/eigenmat.cc:195-204: target = mat > u ? 1 : 0, u drawn in element order. */
int sample_bernoulli_u(const eigenmat* mat, const eigenmat* u, eigenmat* target) {
  if (!same_shape(mat, target) || !same_shape(mat, u)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat);
  #pragma omp parallel for
  for (long i = 0; i < len; i++) target->data[i] = mat->data[i] > u->data[i] ? 1 : 0;
  return 0;
}

/* eigenmat/eigenmat.cc:218-227: target = mat + mult * normal. */
int sample_gaussian_z(const eigenmat* mat, const eigenmat* z, eigenmat* target, float mult) {
  if (!same_shape(mat, target) || !same_shape(mat, z)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat);
  for (long i = 0; i < len; i++) target->data[i] = mat->data[i] + mult * z->data[i];
  return 0;
}

/* eigenmat/eigenmat.cc:238-247: target = -mat / log(u). */
int perturb_prob_u(const eigenmat* mat, const eigenmat* u, eigenmat* target) {
  if (!same_shape(mat, target) || !same_shape(mat, u)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat);
  for (long i = 0; i < len; i++) target->data[i] = -mat->data[i] / logf(u->data[i]);
  return 0;
}

/* eigenmat/eigenmat.cc:229-236: target = mat - log(-log(u)). */
int perturb_energy_u(const eigenmat* mat, const eigenmat* u, eigenmat* target) {
  if (!same_shape(mat, target) || !same_shape(mat, u)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat);
  for (long i = 0; i < len; i++) target->data[i] = mat->data[i] - logf(-logf(u->data[i]));
  return 0;
}

/* ------------------------------------------------------------------ broadcasts */

/* eigenmat/eigenmat.cc:260-278 (and add_col_mult :287-305): target = mat + mult*vec[row]. */
int add_col_mult(const eigenmat* mat, const eigenmat* vec, eigenmat* target, float mult) {
  const int h = mat->size[0], w = mat->size[1];
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (h != vec->size[0] || vec->size[1] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  for (int c = 0; c < w; c++)
    for (int r = 0; r < h; r++) target->data[(long)c * h + r] = mat->data[(long)c * h + r] + mult * vec->data[r];
  return 0;
}
int add_col_vec(const eigenmat* mat, const eigenmat* vec, eigenmat* target) {
  const int h = mat->size[0], w = mat->size[1];
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (h != vec->size[0] || vec->size[1] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  for (int c = 0; c < w; c++)
    for (int r = 0; r < h; r++) target->data[(long)c * h + r] = mat->data[(long)c * h + r] + vec->data[r];
  return 0;
}

/* eigenmat/eigenmat.cc:353-370 with the vector indexed by column (cudamat_kernels.cu:554-567). */
int add_row_mult(const eigenmat* mat, const eigenmat* vec, eigenmat* target, float mult) {
  const int h = mat->size[0], w = mat->size[1];
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (w != vec->size[1] || vec->size[0] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  for (int c = 0; c < w; c++)
    for (int r = 0; r < h; r++) target->data[(long)c * h + r] = mat->data[(long)c * h + r] + mult * vec->data[c];
  return 0;
}
int add_row_vec(const eigenmat* mat, const eigenmat* vec, eigenmat* target) {
  const int h = mat->size[0], w = mat->size[1];
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (w != vec->size[1] || vec->size[0] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  for (int c = 0; c < w; c++)
    for (int r = 0; r < h; r++) target->data[(long)c * h + r] = mat->data[(long)c * h + r] + vec->data[c];
  return 0;
}

/* eigenmat/eigenmat.cc:391-466: mult/div by column or row vector. */
#define BCAST_OP(NAME, BYROW, EXPR)                                                                       \
  int NAME(const eigenmat* mat, const eigenmat* vec, eigenmat* target) {                                  \
    const int h = mat->size[0], w = mat->size[1];                                                         \
    if (mat->is_trans) return ERROR_TRANSPOSED;                                                           \
    if (BYROW) {                                                                                          \
      if (w != vec->size[1] || vec->size[0] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS; \
    } else {                                                                                              \
      if (h != vec->size[0] || vec->size[1] != 1 || !same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS; \
    }                                                                                                     \
    for (int c = 0; c < w; c++)                                                                           \
      for (int r = 0; r < h; r++) {                                                                       \
        const float m = mat->data[(long)c * h + r];                                                       \
        const float v = vec->data[BYROW ? c : r];                                                         \
        target->data[(long)c * h + r] = EXPR;                                                             \
      }                                                                                                   \
    return 0;                                                                                             \
  }
BCAST_OP(mult_by_col_vec, 0, m * v)
BCAST_OP(mult_by_row_vec, 1, m * v)
BCAST_OP(div_by_col_vec, 0, m / v)
BCAST_OP(div_by_row_vec, 1, m / v)

/* ------------------------------------------------------------------ reductions */

/* eigenmat/eigenmat.cc:733-759: target (+)= mult * sum over axis (0: down each column). */
int add_sum_by_axis(const eigenmat* mat, eigenmat* target, int axis, float mult, float beta) {
  const int h = mat->size[0], w = mat->size[1];
  if (mat->is_trans) axis = 1 - axis;
  if (axis == 0) {
    if (numel(target) != w) return ERROR_INCOMPATIBLE_DIMENSIONS;
    for (int c = 0; c < w; c++) {
      float s = 0;
      for (int r = 0; r < h; r++) s += mat->data[(long)c * h + r];
      target->data[c] = (beta == 0 ? 0 : beta * target->data[c]) + mult * s;
    }
  } else if (axis == 1) {
    if (numel(target) != h) return ERROR_INCOMPATIBLE_DIMENSIONS;
    for (int r = 0; r < h; r++) {
      float s = 0;
      for (int c = 0; c < w; c++) s += mat->data[(long)c * h + r];
      target->data[r] = (beta == 0 ? 0 : beta * target->data[r]) + mult * s;
    }
  } else {
    return ERROR_UNSUPPORTED;
  }
  return 0;
}

/* eigenmat/eigenmat.cc:617-639. */
int max_by_axis(const eigenmat* mat, eigenmat* target, int axis) {
  const int h = mat->size[0], w = mat->size[1];
  if (axis == 0) {
    for (int c = 0; c < w; c++) {
      const float* d = &mat->data[(long)c * h];
      float mx = d[0];
      for (int r = 1; r < h; r++) if (mx < d[r]) mx = d[r];
      target->data[c] = mx;
    }
  } else if (axis == 1) {
    for (int r = 0; r < h; r++) {
      float mx = mat->data[r];
      for (int c = 1; c < w; c++) if (mx < mat->data[(long)c * h + r]) mx = mat->data[(long)c * h + r];
      target->data[r] = mx;
    }
  } else {
    return ERROR_UNSUPPORTED;
  }
  return 0;
}

/* eigenmat/eigenmat.cc:641-659: acc[argmax of each column] += 1; first maximum wins. */
int choose_max_and_accumulate(const eigenmat* mat, eigenmat* acc) {
  const int h = mat->size[0], w = mat->size[1];
  if (mat->is_trans) return ERROR_TRANSPOSED;
  if (!same_shape(mat, acc)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  for (int c = 0; c < w; c++) {
    const float* d = &mat->data[(long)c * h];
    int am = 0;
    for (int r = 1; r < h; r++) if (d[am] < d[r]) am = r;
    acc->data[(long)c * h + am] += 1;
  }
  return 0;
}

/* eigenmat/eigenmat.cc:661-685: one-hot of the arg-max along the axis. */
int choose_max_by_axis(const eigenmat* mat, eigenmat* target, int axis) {
  const int h = mat->size[0], w = mat->size[1];
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (axis == 0) {
    for (int c = 0; c < w; c++) {
      const float* d = &mat->data[(long)c * h];
      int am = 0;
      for (int r = 1; r < h; r++) if (d[am] < d[r]) am = r;
      for (int r = 0; r < h; r++) target->data[(long)c * h + r] = (r == am) ? 1 : 0;
    }
  } else if (axis == 1) {
    for (int r = 0; r < h; r++) {
      int am = 0;
      for (int c = 1; c < w; c++) if (mat->data[(long)am * h + r] < mat->data[(long)c * h + r]) am = c;
      for (int c = 0; c < w; c++) target->data[(long)c * h + r] = (c == am) ? 1 : 0;
    }
  } else {
    return ERROR_UNSUPPORTED;
  }
  return 0;
}

/* eigenmat/eigenmat.cc:686-708. */
int argmax_by_axis(const eigenmat* mat, eigenmat* target, int axis) {
  const int h = mat->size[0], w = mat->size[1];
  if (axis != 0) return ERROR_UNSUPPORTED;
  for (int c = 0; c < w; c++) {
    const float* d = &mat->data[(long)c * h];
    int am = 0;
    for (int r = 1; r < h; r++) if (d[am] < d[r]) am = r;
    target->data[c] = (float)am;
  }
  return 0;
}

/* eigenmat/eigenmat.cc:808-826: column softmax (max, exp, sum, divide). */
int apply_softmax(const eigenmat* mat, eigenmat* target) {
  const int h = mat->size[0], w = mat->size[1];
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  for (int c = 0; c < w; c++) {
    const float* d = &mat->data[(long)c * h];
    float* t = &target->data[(long)c * h];
    float mx = d[0];
    for (int r = 1; r < h; r++) if (mx < d[r]) mx = d[r];
    for (int r = 0; r < h; r++) t[r] = (float)exp(d[r] - mx);
    float s = 0;
    for (int r = 0; r < h; r++) s += t[r];
    for (int r = 0; r < h; r++) t[r] /= s;
  }
  return 0;
}

/* eigenmat/eigenmat.cc:1315-1319 and :865-866, :1088-1107. */
float euclid_norm(const eigenmat* mat) {
  const long len = numel(mat);
  double s = 0;
  for (long i = 0; i < len; i++) s += (double)mat->data[i] * mat->data[i];
  return (float)sqrt(s);
}
float sum_all(const eigenmat* mat) {
  const long len = numel(mat);
  double s = 0;
  for (long i = 0; i < len; i++) s += mat->data[i];
  return (float)s;
}
float vdot(const eigenmat* a, const eigenmat* b, int* err) {
  *err = 0;
  if (a->is_trans != b->is_trans) { *err = ERROR_TRANSPOSEDNESS; return 0; }
  if (!same_shape(a, b)) { *err = ERROR_INCOMPATIBLE_DIMENSIONS; return 0; }
  const long len = numel(a);
  double s = 0;
  for (long i = 0; i < len; i++) s += (double)a->data[i] * b->data[i];
  return (float)s;
}

/* ------------------------------------------------------------------ elementwise */

/* eigenmat/eigenmat.cc:869-878: 1 / (1 + exp(-x)); exp evaluated in double. */
int apply_sigmoid(const eigenmat* mat, eigenmat* target) {
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat);
  #pragma omp parallel for
  for (long i = 0; i < len; i++) target->data[i] = (float)(1 / (1 + exp(-mat->data[i])));
  return 0;
}
/* eigenmat/eigenmat.cc:927-938. */
int apply_exp(const eigenmat* mat, eigenmat* target) {
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat);
  for (long i = 0; i < len; i++) target->data[i] = expf(mat->data[i]);
  return 0;
}
/* eigenmat/eigenmat.cc:900-912: log(1 + exp(x)), stable form as cudamat_kernels.cu:427-438. */
int apply_log_1_plus_exp(const eigenmat* mat, eigenmat* target) {
  if (!same_shape(mat, target)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat);
  for (long i = 0; i < len; i++) {
    const float x = mat->data[i];
    target->data[i] = x > 0 ? x + log1pf(expf(-x)) : log1pf(expf(x));
  }
  return 0;
}

/* eigenmat/eigenmat.cc:1109-1122: mat1 += alpha * mat2. */
int add_mult(eigenmat* mat1, const eigenmat* mat2, float alpha) {
  if (mat1->is_trans != mat2->is_trans) return ERROR_TRANSPOSEDNESS;
  if (!same_shape(mat1, mat2)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat1);
  for (long i = 0; i < len; i++) mat1->data[i] += mat2->data[i] * alpha;
  return 0;
}
/* eigenmat/eigenmat.cc:280-285. */
int add_mult_sign(eigenmat* mat1, const eigenmat* mat2, float mult) {
  if (!same_shape(mat1, mat2)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(mat1);
  for (long i = 0; i < len; i++)
    mat1->data[i] += (mat2->data[i] == 0) ? 0 : ((mat2->data[i] > 0) ? mult : -mult);
  return 0;
}

/* ------------------------------------------------------------------ GEMM */

/* eigenmat/eigenmat.cc:1059-1086: target = beta*target + alpha*op(mat1)*op(mat2),
 * fp32 accumulation, k innermost so that every output is one running float sum. */
int dot(const eigenmat* mat1, const eigenmat* mat2, eigenmat* target, float beta, float alpha) {
  const int m = mat1->is_trans ? mat1->size[1] : mat1->size[0];
  const int k = mat1->is_trans ? mat1->size[0] : mat1->size[1];
  const int k2 = mat2->is_trans ? mat2->size[1] : mat2->size[0];
  const int n = mat2->is_trans ? mat2->size[0] : mat2->size[1];
  if (m != target->size[0] || n != target->size[1] || k != k2) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long lda = mat1->size[0], ldb = mat2->size[0];
  for (int j = 0; j < n; j++)
    for (int i = 0; i < m; i++) {
      float s = 0;
      for (int p = 0; p < k; p++) {
        const float a = mat1->is_trans ? mat1->data[(long)i * lda + p] : mat1->data[(long)p * lda + i];
        const float b = mat2->is_trans ? mat2->data[(long)p * ldb + j] : mat2->data[(long)j * ldb + p];
        s += a * b;
      }
      float* t = &target->data[(long)j * m + i];
      *t = (beta == 0 ? 0 : beta * *t) + alpha * s;
    }
  return 0;
}

/* ------------------------------------------------------------------ index ops */

/* eigenmat/eigenmat.cc:1321-1335 (selectCols): target[:, i] = source[:, indices[i]]. */
int selectCols(const eigenmat* source, eigenmat* target, const eigenmat* indices) {
  const int n = indices->size[0] * indices->size[1], h = source->size[0];
  if (target->size[0] != h || target->size[1] != n) return ERROR_INCOMPATIBLE_DIMENSIONS;
  for (int i = 0; i < n; i++) {
    int s = (int)indices->data[i];
    if (s < 0) s += source->size[1];   /* cudamat/cudamat_kernels.cu:728-731 */
    for (int j = 0; j < h; j++) target->data[(long)i * h + j] = source->data[(long)s * h + j];
  }
  return 0;
}

/* eigenmat/eigenmat.cc:1351-1367 (swapCols): column indices1[i] of source <-> column indices2[i] of target. */
int swapCols(eigenmat* source, eigenmat* target, const eigenmat* indices1, const eigenmat* indices2) {
  const int n = indices1->size[0] * indices1->size[1], h = source->size[0];
  for (int i = 0; i < n; i++) {
    const long so = (long)(int)indices1->data[i] * h, to = (long)(int)indices2->data[i] * h;
    for (int j = 0; j < h; j++) {
      const float temp = target->data[to + j];
      target->data[to + j] = source->data[so + j];
      source->data[so + j] = temp;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ parameter update */

/* deepnet/dbm.py:242,254 + deepnet/parameter.py:80-106 as one pass, in the order the
 * reference issues its calls:
 *   grad += suff * (-1/B);  delta *= momentum;  delta += l2 * w;  delta += l1*sign(w);
 *   delta += grad;  w += delta * (-eps);  grad = 0. */
int momentum_update(eigenmat* w, eigenmat* delta, eigenmat* grad, const eigenmat* suff, float inv_batch,
                    float momentum, float eps, float l2, float l1) {
  if (!same_shape(w, delta) || !same_shape(w, grad) || !same_shape(w, suff)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long len = numel(w);
  #pragma omp parallel for
  for (long i = 0; i < len; i++) {
    float g = grad->data[i] + suff->data[i] * (-inv_batch);
    float d = delta->data[i] * momentum;
    if (l2 != 0) d += w->data[i] * l2;
    if (l1 != 0) d += (w->data[i] == 0) ? 0 : ((w->data[i] > 0) ? l1 : -l1);
    d += g;
    w->data[i] += d * (-eps);
    delta->data[i] = d;
    grad->data[i] = 0;
  }
  return 0;
}
