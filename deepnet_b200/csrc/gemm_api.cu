// C entry points built on the fused matrix product: the reference `dot`
// (cudamat/cudamat.cu:1671-1696) and the fused calls that replace whole groups of
// reference operations on the contrastive-divergence path (deepnet/dbm.py:64-115,
// deepnet/edge.py:222-246, deepnet/parameter.py:80-106).
#include "gemm.cuh"

using namespace b200;

namespace {

int g_path = 0;       // 0 auto, 1 tensor cores only, 2 CUDA cores only
int g_dot_mode = 0;   // 0: fp32-grade (split TF32, 3 passes), 1: single TF32 pass
constexpr long kTcMinWork = 1L << 21;  // below this many multiply-adds `dot` stays on CUDA cores

inline int lead(const cudamat* m) { return m->is_trans ? m->size[1] : m->size[0]; }
inline int nonlead(const cudamat* m) { return m->is_trans ? m->size[0] : m->size[1]; }
inline GemmOperand operand(const cudamat* m, const float* ptr = nullptr) {
  GemmOperand o;
  o.ptr = ptr ? ptr : m->data_device;
  o.ld = m->size[0];
  o.trans = m->is_trans;
  o.bf16 = 0;
  return o;
}
// Plane 0 or 1 of the aux matrix stored at `aux` with lda floats per column.
inline GemmOperand aux_operand(const float* aux, int lda, int trans, int plane) {
  GemmOperand o;
  o.ptr = reinterpret_cast<const float*>(reinterpret_cast<const uint16_t*>(aux) + (long)plane * lda);
  o.ld = 2 * lda;
  o.trans = trans;
  o.bf16 = 1;
  return o;
}
// An aux handle must hold aux_rows(rows) x cols floats.
inline bool aux_shape_ok(const cudamat* aux, int rows, int cols) {
  return aux->size[0] == aux_rows(rows) && aux->size[1] == cols;
}

int run(const GemmProblem& g) {
  if (g_path == 2) return gemm_simt(g);
  if (gemm_tc_supported(g)) return gemm_tc(g);
  if (g_path == 1) return ERROR_UNSUPPORTED;
  return gemm_simt(g);
}

// hi may be null: the tensor core itself drops the low 13 mantissa bits of an fp32
// operand, so the matrix x can stand in for its own high part and only lo is stored.
__global__ void __launch_bounds__(256) k_split(const float* x, float* hi, float* lo, long n, bool vec) {
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {
    const long n4 = n >> 2;
    for (long i = tid; i < n4; i += nth) {
      const float4 v = reinterpret_cast<const float4*>(x)[i];
      float4 h, l;
      split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
      if (hi) reinterpret_cast<float4*>(hi)[i] = h;
      reinterpret_cast<float4*>(lo)[i] = l;
    }
    for (long i = (n4 << 2) + tid; i < n; i += nth) {
      float h, l;
      split_tf32(x[i], h, l);
      if (hi) hi[i] = h;
      lo[i] = l;
    }
  } else {
    for (long i = tid; i < n; i += nth) {
      float h, l;
      split_tf32(x[i], h, l);
      if (hi) hi[i] = h;
      lo[i] = l;
    }
  }
}

// aux matrix of x (rows x cols, contiguous columns): both bfloat16 planes in one pass.
__global__ void __launch_bounds__(256) k_split_aux(const float* x, uint16_t* aux, int rows, int lda, long n,
                                                   bool vec) {
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {   // rows % 4 == 0: four consecutive elements share a column
    for (long i = tid; i < (n >> 2); i += nth) {
      const float4 v = reinterpret_cast<const float4*>(x)[i];
      const long e = i << 2, c = e / rows, r = e - c * rows;
      ushort4 l, b;
      split_aux(v.x, l.x, b.x); split_aux(v.y, l.y, b.y); split_aux(v.z, l.z, b.z); split_aux(v.w, l.w, b.w);
      uint16_t* dst = aux + c * 2 * lda + r;
      *reinterpret_cast<ushort4*>(dst) = l;
      *reinterpret_cast<ushort4*>(dst + lda) = b;
    }
  } else {
    for (long i = tid; i < n; i += nth) {
      const long c = i / rows, r = i - c * rows;
      uint16_t l, b;
      split_aux(x[i], l, b);
      aux[c * 2 * lda + r] = l;
      aux[c * 2 * lda + lda + r] = b;
    }
  }
}

// aux holds aux_rows(rows) floats per column.
int launch_split_aux(const float* x, float* aux, int rows, long n) {
  if (n == 0) return 0;
  const bool vec = (rows % 4 == 0) && ((((uintptr_t)x) & 15) == 0) && ((((uintptr_t)aux) & 7) == 0);
  long blocks = ((vec ? n / 4 : n) + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  if (blocks < 1) blocks = 1;
  k_split_aux<<<(int)blocks, 256, 0, stream()>>>(x, reinterpret_cast<uint16_t*>(aux), rows, aux_rows(rows), n, vec);
  return check_launch();
}

int launch_split(const float* x, float* hi, float* lo, long n) {
  if (n == 0) return 0;
  const bool vec = (((uintptr_t)x | (uintptr_t)hi | (uintptr_t)lo) & 15) == 0;
  long blocks = ((vec ? (n + 3) / 4 : n) + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  k_split<<<(int)blocks, 256, 0, stream()>>>(x, hi, lo, n, vec);
  return check_launch();
}

// One pass of the parameter update, in the order the reference issues its calls
// (deepnet/dbm.py:242,254 then deepnet/parameter.py:89-106).  Products and sums are
// rounded separately (no fused multiply-add) so the result equals the call sequence's.
__device__ __forceinline__ void update_one(float& w, float& d, float g, float suff, float ninv_batch, float momentum,
                                           float neps, float l2, float l1) {
  g = __fadd_rn(g, __fmul_rn(suff, ninv_batch));
  d = __fmul_rn(d, momentum);
  if (l2 != 0.0f) d = __fadd_rn(d, __fmul_rn(w, l2));
  if (l1 != 0.0f) d = __fadd_rn(d, w == 0.0f ? 0.0f : (w > 0.0f ? l1 : -l1));
  d = __fadd_rn(d, g);
  w = __fadd_rn(w, __fmul_rn(d, neps));
}

template <bool kHasGrad, bool kSplit>
__global__ void __launch_bounds__(256) k_update(float* w, float* delta, float* grad, const float* suff,
                                                uint16_t* w_aux, int rows, int lda, long n, bool vec,
                                                float ninv_batch, float momentum, float neps, float l2, float l1) {
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {
    const long n4 = n >> 2;
    for (long i = tid; i < n4; i += nth) {
      float4 W = reinterpret_cast<float4*>(w)[i];
      float4 D = reinterpret_cast<float4*>(delta)[i];
      const float4 S = reinterpret_cast<const float4*>(suff)[i];
      float4 G = make_float4(0, 0, 0, 0);
      if (kHasGrad) G = reinterpret_cast<float4*>(grad)[i];
      update_one(W.x, D.x, G.x, S.x, ninv_batch, momentum, neps, l2, l1);
      update_one(W.y, D.y, G.y, S.y, ninv_batch, momentum, neps, l2, l1);
      update_one(W.z, D.z, G.z, S.z, ninv_batch, momentum, neps, l2, l1);
      update_one(W.w, D.w, G.w, S.w, ninv_batch, momentum, neps, l2, l1);
      reinterpret_cast<float4*>(w)[i] = W;
      reinterpret_cast<float4*>(delta)[i] = D;
      if (kHasGrad) reinterpret_cast<float4*>(grad)[i] = make_float4(0, 0, 0, 0);
      if (kSplit) {   // vec implies rows % 4 == 0: the four elements share a column
        const long e = i << 2, c = e / rows, r = e - c * rows;
        ushort4 L, B;
        split_aux(W.x, L.x, B.x); split_aux(W.y, L.y, B.y); split_aux(W.z, L.z, B.z); split_aux(W.w, L.w, B.w);
        uint16_t* dst = w_aux + c * 2 * lda + r;
        *reinterpret_cast<ushort4*>(dst) = L;
        *reinterpret_cast<ushort4*>(dst + lda) = B;
      }
    }
    for (long i = (n4 << 2) + tid; i < n; i += nth) {
      float W = w[i], D = delta[i];
      update_one(W, D, kHasGrad ? grad[i] : 0.0f, suff[i], ninv_batch, momentum, neps, l2, l1);
      w[i] = W; delta[i] = D;
      if (kHasGrad) grad[i] = 0.0f;
      if (kSplit) {
        const long c = i / rows, r = i - c * rows;
        uint16_t L, B;
        split_aux(W, L, B);
        w_aux[c * 2 * lda + r] = L;
        w_aux[c * 2 * lda + lda + r] = B;
      }
    }
  } else {
    for (long i = tid; i < n; i += nth) {
      float W = w[i], D = delta[i];
      update_one(W, D, kHasGrad ? grad[i] : 0.0f, suff[i], ninv_batch, momentum, neps, l2, l1);
      w[i] = W; delta[i] = D;
      if (kHasGrad) grad[i] = 0.0f;
      if (kSplit) {
        const long c = i / rows, r = i - c * rows;
        uint16_t L, B;
        split_aux(W, L, B);
        w_aux[c * 2 * lda + r] = L;
        w_aux[c * 2 * lda + lda + r] = B;
      }
    }
  }
}

}  // namespace

// One term of a fused product: op(a) is M x k, op(b) is k x N (handles carry is_trans).
// a_plane / b_plane: -1 = the handle is an fp32 matrix (read as TF32 on the tensor cores);
// 0 or 1 = the handle is an aux matrix and the term reads that bfloat16 plane of it, a_rows /
// b_rows then give the rows of the matrix the aux belongs to (its storage has them rounded up
// to a multiple of 8).  Both operands of a term are of the same kind.
struct b200_pass {
  cudamat* a;
  cudamat* b;
  int negate;
  int a_plane, b_plane;
  int a_rows, b_rows;
};
// out = act(alpha * sum_p (+/-) op(a_p).op(b_p) + beta * out + bias (x) col_scale)
struct b200_fused_gemm {
  int npass;
  b200_pass pass[kMaxPass];
  float alpha, beta;
  cudamat* bias;       // M x 1 or null
  cudamat* col_scale;  // 1 x N or null
  int activation;      // 0 identity, 1 logistic
  cudamat* out;        // M x N or null
  cudamat* out_aux;    // aux matrix of the result (M x N floats of storage), or null
  cudamat* sample;     // Bernoulli(result), or null
  cudamat* sample_aux; // aux matrix of the draw, or null
};

extern "C" {

// 0 auto (tensor cores when the operands are TMA-addressable), 1 tensor cores only
// (ERROR_UNSUPPORTED otherwise), 2 CUDA cores only.
int b200_set_gemm_path(int path) {
  g_path = path;
  return 0;
}
// Precision of `dot`: 0 = fp32-grade (operands split into TF32 hi/lo, three passes),
// 1 = one TF32 pass (about 1e-3 relative).
int b200_set_dot_precision(int mode) {
  g_dot_mode = mode;
  return 0;
}

// hi = x with the low 13 mantissa bits cleared (optional, may be null), lo = x - hi.
int split_tf32(cudamat* x, cudamat* hi, cudamat* lo) {
  if (!x->on_device || (hi && !hi->on_device) || !lo->on_device) return ERROR_NOT_ON_DEVICE;
  if ((hi && !same_shape(x, hi)) || !same_shape(x, lo)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  return launch_split(x->data_device, hi ? hi->data_device : nullptr, lo->data_device, numel(x));
}

// aux = the two bfloat16 planes of x (see split_aux); aux has the shape of x.
int split_bf16(cudamat* x, cudamat* aux) {
  if (!x->on_device || !aux->on_device) return ERROR_NOT_ON_DEVICE;
  if (x->is_trans || aux->is_trans) return ERROR_TRANSPOSED;
  if (!aux_shape_ok(aux, x->size[0], x->size[1])) return ERROR_INCOMPATIBLE_DIMENSIONS;
  return launch_split_aux(x->data_device, aux->data_device, x->size[0], numel(x));
}

int fused_gemm(rnd_struct* rnd_state, b200_fused_gemm* f) {
  if (f->npass <= 0 || f->npass > kMaxPass) return ERROR_UNSUPPORTED;
  GemmProblem g;
  g.npass = f->npass;
  g.tf32_operands = 1;
  // logical shape of an operand: an aux handle's storage rows are rounded up, the pass names the real ones
  auto rows_of = [](const cudamat* m, int plane, int rows) { return plane < 0 ? m->size[0] : rows; };
  auto lead_of = [&](const cudamat* m, int plane, int rows) { return m->is_trans ? m->size[1] : rows_of(m, plane, rows); };
  auto nonlead_of = [&](const cudamat* m, int plane, int rows) { return m->is_trans ? rows_of(m, plane, rows) : m->size[1]; };
  g.M = lead_of(f->pass[0].a, f->pass[0].a_plane, f->pass[0].a_rows);
  g.N = nonlead_of(f->pass[0].b, f->pass[0].b_plane, f->pass[0].b_rows);
  for (int q = 0; q < f->npass; q++) {
    const cudamat *a = f->pass[q].a, *b = f->pass[q].b;
    if (!a->on_device || !b->on_device) return ERROR_NOT_ON_DEVICE;
    const int pa = f->pass[q].a_plane, pb = f->pass[q].b_plane, ra = f->pass[q].a_rows, rb = f->pass[q].b_rows;
    if ((pa < 0) != (pb < 0) || pa > 1 || pb > 1) return ERROR_UNSUPPORTED;
    if (pa >= 0 && (a->size[0] != aux_rows(ra) || b->size[0] != aux_rows(rb))) return ERROR_INCOMPATIBLE_DIMENSIONS;
    const int k = nonlead_of(a, pa, ra);
    if (lead_of(a, pa, ra) != g.M || nonlead_of(b, pb, rb) != g.N || k != lead_of(b, pb, rb))
      return ERROR_INCOMPATIBLE_DIMENSIONS;
    g.pass[q].a = pa < 0 ? operand(a) : aux_operand(a->data_device, a->size[0], a->is_trans, pa);
    g.pass[q].b = pb < 0 ? operand(b) : aux_operand(b->data_device, b->size[0], b->is_trans, pb);
    g.pass[q].k = k;
    g.pass[q].negate = f->pass[q].negate;
  }
  GemmEpilogue& e = g.epi;
  e.alpha = f->alpha;
  e.beta = f->beta;
  e.bias = nullptr;
  e.col_scale = nullptr;
  e.activation = f->activation;
  e.out = e.out_aux = e.sample = e.sample_aux = nullptr;
  e.ldo = g.M;
  e.ld_aux = aux_rows(g.M);
  e.col0 = rng_col0();
  cudamat* outs[4] = {f->out, f->out_aux, f->sample, f->sample_aux};
  for (int i = 0; i < 4; i++) {
    if (!outs[i]) continue;
    if (!outs[i]->on_device) return ERROR_NOT_ON_DEVICE;
    if (outs[i]->is_trans) return ERROR_TRANSPOSED;
    const int want_rows = (i & 1) ? e.ld_aux : g.M;   // aux handles hold the rounded-up rows
    if (outs[i]->size[0] != want_rows || outs[i]->size[1] != g.N) return ERROR_INCOMPATIBLE_DIMENSIONS;
  }
  if (f->out) e.out = f->out->data_device;
  if (f->out_aux) e.out_aux = f->out_aux->data_device;
  if (f->sample) e.sample = f->sample->data_device;
  if (f->sample_aux) e.sample_aux = f->sample_aux->data_device;
  if (e.beta != 0.0f && !e.out) return ERROR_UNSUPPORTED;
  if (f->bias) {
    if (!f->bias->on_device) return ERROR_NOT_ON_DEVICE;
    if (numel(f->bias) != g.M) return ERROR_INCOMPATIBLE_DIMENSIONS;
    e.bias = f->bias->data_device;
  }
  if (f->col_scale) {
    if (!f->col_scale->on_device) return ERROR_NOT_ON_DEVICE;
    if (numel(f->col_scale) != g.N || !f->bias) return ERROR_INCOMPATIBLE_DIMENSIONS;
    e.col_scale = f->col_scale->data_device;
  }
  e.key = make_philox_key(0, 0);
  if (f->sample || f->sample_aux) {
    if (!rnd_state) return ERROR_GENERIC;
    e.key = make_philox_key(rnd_state->seed, rnd_state->calls);
    rnd_state->calls += 1;
  }
  return run(g);
}

// cudamat/cudamat.cu:1671-1696: target = beta * target + alpha * op(mat1) . op(mat2).
int dot(cudamat* mat1, cudamat* mat2, cudamat* target, float beta, float alpha) {
  if (!mat1->on_device || !mat2->on_device || !target->on_device) return ERROR_NOT_ON_DEVICE;
  if (lead(mat1) != lead(target) || nonlead(mat2) != nonlead(target) || nonlead(mat1) != lead(mat2))
    return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (target->is_trans) return ERROR_TRANSPOSED;
  const int m = lead(mat1), k = lead(mat2), n = nonlead(mat2);
  GemmProblem g;
  g.M = m;
  g.N = n;
  g.tf32_operands = 0;  // on CUDA cores `dot` multiplies full fp32 operands
  GemmEpilogue& e = g.epi;
  e.alpha = alpha;
  e.beta = beta;
  e.bias = e.col_scale = nullptr;
  e.activation = 0;
  e.out = target->data_device;
  e.out_aux = e.sample = e.sample_aux = nullptr;
  e.ldo = m;
  e.ld_aux = aux_rows(m);
  e.col0 = 0;
  e.key = make_philox_key(0, 0);
  g.npass = 1;
  g.pass[0].a = operand(mat1);
  g.pass[0].b = operand(mat2);
  g.pass[0].k = k;
  g.pass[0].negate = 0;
  if (m == 0 || n == 0) return 0;
  if (k == 0) {  // empty inner dimension: target = beta * target
    g.pass[0].k = 0;
    return gemm_simt(g);
  }
  const bool tc = g_path != 2 && gemm_tc_supported(g) && (g_path == 1 || (long)m * n * k >= kTcMinWork);
  if (!tc) {
    if (g_path == 1) return ERROR_UNSUPPORTED;
    return gemm_simt(g);
  }
  if (g_dot_mode == 1) return gemm_tc(g);
  // fp32-grade: x = hi + lo, the tensor core reads hi out of x itself (it ignores the low
  // 13 mantissa bits), lo goes to scratch; lo.hi + hi.lo + hi.hi, small terms first.  All three
  // terms are TF32 products: the cheaper bfloat16 correction terms of the aux matrices are
  // a few times less accurate (2^-18 against 2^-20 per term), which shows when a caller
  // subtracts two nearly equal products, as the positive and negative statistics are.
  const long na = numel(mat1), nb = numel(mat2);
  float* sa = (float*)workspace(2, (size_t)na * sizeof(float));
  float* sb = (float*)workspace(3, (size_t)nb * sizeof(float));
  if (!sa || !sb) return CUDA_ERROR;
  int err = launch_split(mat1->data_device, nullptr, sa, na);
  if (err) return err;
  err = launch_split(mat2->data_device, nullptr, sb, nb);
  if (err) return err;
  g.npass = 3;
  const float* ap[3] = {sa, mat1->data_device, mat1->data_device};
  const float* bp[3] = {mat2->data_device, sb, mat2->data_device};
  for (int q = 0; q < 3; q++) {
    g.pass[q].a = operand(mat1, ap[q]);
    g.pass[q].b = operand(mat2, bp[q]);
    g.pass[q].k = k;
    g.pass[q].negate = 0;
  }
  g.tf32_operands = 1;
  return gemm_tc(g);
}

// deepnet/dbm.py:242,254 + deepnet/parameter.py:80-106 in one pass over the parameter:
//   grad += suff * (-inv_batch); delta = momentum*delta + l2*w + l1*sign(w) + grad;
//   w -= eps * delta; grad = 0; and, when w_aux is given, the aux matrix of the new w.
// grad may be null (treated as zero and not written).  20 bytes of traffic per element
// without grad and aux; +8 with grad, +4 with w_aux.
int momentum_update(cudamat* w, cudamat* delta, cudamat* grad, cudamat* suff, cudamat* w_aux, float inv_batch,
                    float momentum, float eps, float l2, float l1) {
  if (!w->on_device || !delta->on_device || !suff->on_device) return ERROR_NOT_ON_DEVICE;
  if (!same_shape(w, delta) || !same_shape(w, suff)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (grad && (!grad->on_device || !same_shape(w, grad))) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (w_aux && (!w_aux->on_device || w->is_trans || !aux_shape_ok(w_aux, w->size[0], w->size[1])))
    return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long n = numel(w);
  if (n == 0) return 0;
  uintptr_t bits = (uintptr_t)w->data_device | (uintptr_t)delta->data_device | (uintptr_t)suff->data_device;
  if (grad) bits |= (uintptr_t)grad->data_device;
  if (w_aux) bits |= (uintptr_t)w_aux->data_device;
  const int rows = w->size[0];
  const bool vec = (bits & 15) == 0 && (!w_aux || rows % 4 == 0) && n % 4 == 0;
  long blocks = ((vec ? (n + 3) / 4 : n) + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  float* gp = grad ? grad->data_device : nullptr;
  uint16_t* ap = w_aux ? reinterpret_cast<uint16_t*>(w_aux->data_device) : nullptr;
#define LAUNCH_UPDATE(G, S)                                                                                       \
  k_update<G, S><<<(int)blocks, 256, 0, stream()>>>(w->data_device, delta->data_device, gp, suff->data_device, ap, \
                                                    rows, aux_rows(rows), n, vec, -inv_batch, momentum, -eps, l2, l1)
  if (grad && w_aux) LAUNCH_UPDATE(true, true);
  else if (grad) LAUNCH_UPDATE(true, false);
  else if (w_aux) LAUNCH_UPDATE(false, true);
  else LAUNCH_UPDATE(false, false);
#undef LAUNCH_UPDATE
  return check_launch();
}

}  // extern "C"
