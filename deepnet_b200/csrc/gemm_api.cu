// C entry points built on the fused matrix product: the reference `dot`
// (cudamat/cudamat.cu:1671-1696) and the fused calls that replace whole groups of
// reference operations on the contrastive-divergence path (deepnet/dbm.py:64-115,
// deepnet/edge.py:222-246, deepnet/parameter.py:80-106).
#include "gemm.cuh"

using namespace b200;

namespace {

int g_path = 0;       // 0 auto, 1 tensor cores only, 2 CUDA cores only
int g_dot_mode = 0;   // 0: fp32-grade (three TF32 terms), 1: single TF32 term
constexpr long kTcMinWork = 1L << 21;  // below this many multiply-adds `dot` stays on CUDA cores

inline int lead(const cudamat* m) { return m->is_trans ? m->size[1] : m->size[0]; }
inline int nonlead(const cudamat* m) { return m->is_trans ? m->size[0] : m->size[1]; }
inline GemmOperand operand(const cudamat* m, int part, const cudamat* aux = nullptr) {
  GemmOperand o;
  o.ptr = m->data_device;
  o.ld = m->size[0];
  o.trans = m->is_trans;
  o.part = part;
  o.aux = aux ? aux->data_device : nullptr;
  o.lda = aux ? aux->size[0] : 0;
  o.row0 = 0;
  return o;
}
// An aux handle holds aux_rows(rows) x cols floats.
inline bool aux_shape_ok(const cudamat* aux, const cudamat* m) {
  return aux->on_device && aux->size[0] == aux_rows(m->size[0]) && aux->size[1] == m->size[1];
}

int run(const GemmProblem& g) {
  if (product_is_scattered(g.epi.out)) return gemm_tc(g);   // (fails loudly when the tensor-core kernel cannot take it)
  if (g_path == 2) return gemm_simt(g);
  if (gemm_tc_supported(g)) {
    const int r = gemm_tc(g);
    // (a product with more operand pairs or tiles than one tensor-core launch carries)
    if (r != ERROR_UNSUPPORTED || g_path == 1) return r;
  } else if (g_path == 1) {
    return ERROR_UNSUPPORTED;
  }
  return gemm_simt(g);
}

// hi may be null: the tensor core itself drops the low 13 mantissa bits of an fp32
// operand, so the matrix x can stand in for its own high part and only lo is stored.
__global__ void __launch_bounds__(256) k_split(const float* x, float* hi, float* lo, long n, bool vec) {
  grid_dependents_launch();
  grid_dependency_wait();
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
  grid_dependents_launch();
  grid_dependency_wait();
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

// aux matrix of x in scaled half-precision form (split_f16): scale = 2^(*exp_dev + exp_const).
// `only_if` (optional): a device flag; the kernel returns at once when it is zero.
__global__ void __launch_bounds__(256) k_split_f16(const float* x, uint16_t* aux, int rows, int lda, long n, bool vec,
                                                   const float* exp_dev, int exp_const, const float* only_if) {
  grid_dependents_launch();
  grid_dependency_wait();
  if (only_if && *only_if == 0.0f) return;
  const float scale = exp2f((exp_dev ? *exp_dev : 0.0f) + (float)exp_const);
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  if (vec) {
    for (long i = tid; i < (n >> 2); i += nth) {
      const float4 v = reinterpret_cast<const float4*>(x)[i];
      const long e = i << 2, c = e / rows, r = e - c * rows;
      ushort4 l, h;
      split_f16(v.x, scale, l.x, h.x); split_f16(v.y, scale, l.y, h.y);
      split_f16(v.z, scale, l.z, h.z); split_f16(v.w, scale, l.w, h.w);
      uint16_t* dst = aux + c * 2 * lda + r;
      *reinterpret_cast<ushort4*>(dst) = l;
      *reinterpret_cast<ushort4*>(dst + lda) = h;
    }
  } else {
    for (long i = tid; i < n; i += nth) {
      const long c = i / rows, r = i - c * rows;
      uint16_t l, h;
      split_f16(x[i], scale, l, h);
      aux[c * 2 * lda + r] = l;
      aux[c * 2 * lda + lda + r] = h;
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
  if (launch_dependent(k_split_aux, dim3((unsigned)blocks), dim3(256), 0, stream(), x, reinterpret_cast<uint16_t*>(aux), rows,
                       aux_rows(rows), n, vec) != cudaSuccess)
    return set_error(cudaGetErrorString(cudaGetLastError()));
  return check_launch();
}

int launch_split(const float* x, float* hi, float* lo, long n) {
  if (n == 0) return 0;
  const bool vec = (((uintptr_t)x | (uintptr_t)hi | (uintptr_t)lo) & 15) == 0;
  long blocks = ((vec ? (n + 3) / 4 : n) + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  (void)launch_dependent(k_split, dim3((unsigned)blocks), dim3(256), 0, stream(), x, hi, lo, n, vec);
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

// kAux: 0 no aux, 1 bfloat16 parts, 2 scaled half-precision form.  For 2 the aux is written with
// the exponent the parameter has carried so far (`scale` = {exponent, copy, max |w| bits, redo flag})
// and the largest |w| of the new parameter is gathered into scale[2]; k_update_scale then checks
// that this exponent still fits the new parameter (it does unless the weights grew eightfold or
// shrank by more than half in one update) and only otherwise sets the flag that makes a second
// pass (k_split_f16) rewrite the aux with a new exponent.  One pass over the weights in the
// common case: 24 bytes per weight instead of 28.
template <bool kHasGrad, int kAux>
__global__ void __launch_bounds__(256) k_update(float* w, float* delta, float* grad, const float* suff,
                                                uint16_t* w_aux, float* scale, int rows, int lda, long n, bool vec,
                                                float ninv_batch, float momentum, float neps, float l2, float l1) {
  grid_dependents_launch();
  grid_dependency_wait();
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long)gridDim.x * blockDim.x;
  float wmax = 0.0f;
  const float f16_scale = kAux == 2 ? exp2f(scale[0]) : 1.0f;
  if (vec) {   // n % 4 == 0, and with an aux rows % 4 == 0: four consecutive elements share a column
    for (long i = tid; i < (n >> 2); i += nth) {
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
      if (kAux == 1) {
        const long e = i << 2, c = e / rows, r = e - c * rows;
        ushort4 L, B;
        split_aux(W.x, L.x, B.x); split_aux(W.y, L.y, B.y); split_aux(W.z, L.z, B.z); split_aux(W.w, L.w, B.w);
        uint16_t* dst = w_aux + c * 2 * lda + r;
        *reinterpret_cast<ushort4*>(dst) = L;
        *reinterpret_cast<ushort4*>(dst + lda) = B;
      }
      if (kAux == 2) {
        wmax = fmaxf(fmaxf(wmax, fmaxf(fabsf(W.x), fabsf(W.y))), fmaxf(fabsf(W.z), fabsf(W.w)));
        const long e = i << 2, c = e / rows, r = e - c * rows;
        ushort4 L, Hh;
        split_f16(W.x, f16_scale, L.x, Hh.x); split_f16(W.y, f16_scale, L.y, Hh.y);
        split_f16(W.z, f16_scale, L.z, Hh.z); split_f16(W.w, f16_scale, L.w, Hh.w);
        uint16_t* dst = w_aux + c * 2 * lda + r;
        *reinterpret_cast<ushort4*>(dst) = L;
        *reinterpret_cast<ushort4*>(dst + lda) = Hh;
      }
    }
  } else {
    for (long i = tid; i < n; i += nth) {
      float W = w[i], D = delta[i];
      update_one(W, D, kHasGrad ? grad[i] : 0.0f, suff[i], ninv_batch, momentum, neps, l2, l1);
      w[i] = W; delta[i] = D;
      if (kHasGrad) grad[i] = 0.0f;
      if (kAux == 1) {
        const long c = i / rows, r = i - c * rows;
        uint16_t L, B;
        split_aux(W, L, B);
        w_aux[c * 2 * lda + r] = L;
        w_aux[c * 2 * lda + lda + r] = B;
      }
      if (kAux == 2) {
        wmax = fmaxf(wmax, fabsf(W));
        const long c = i / rows, r = i - c * rows;
        uint16_t L, Hh;
        split_f16(W, f16_scale, L, Hh);
        w_aux[c * 2 * lda + r] = L;
        w_aux[c * 2 * lda + lda + r] = Hh;
      }
    }
  }
  if (kAux == 2) {   // non-negative floats order like their bit patterns
    const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(wmax));
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned*>(scale) + 2, m);
  }
}

// After an update in scaled half-precision form.  The exponent wanted for the new parameter puts
// the largest |w| * 2^e in (2^12, 2^13] (the fp16 limit is just under 2^16).  The aux was written
// with the exponent carried so far; it stands while the largest scaled magnitude stays within
// (2^11, 2^15].  Otherwise the wanted exponent is stored and scale[3] tells the second pass to
// rewrite the aux.  The maximum starts over.  A parameter that is all zero (or not finite) keeps
// its exponent.
__global__ void k_update_scale(float* scale) {
  grid_dependents_launch();
  grid_dependency_wait();
  const float m = __uint_as_float(reinterpret_cast<unsigned*>(scale)[2]);
  float redo = 0.0f;
  if (m > 0.0f && m < 3.0e38f) {
    const float want = fminf(fmaxf(floorf(log2f(8192.0f / m)), -100.0f), 100.0f);
    const float d = scale[0] - want;
    if (d < -1.0f || d > 2.0f) {
      scale[0] = want;
      redo = 1.0f;
    }
  }
  scale[1] = scale[0];
  scale[3] = redo;
  reinterpret_cast<unsigned*>(scale)[2] = 0u;
}

}  // namespace

namespace b200 {
int rewrite_f16_planes_if(const float* x, uint16_t* aux, int rows, long n, const float* exp_dev, const float* only_if) {
  if (n == 0) return 0;
  const bool svec = (rows % 4 == 0) && ((((uintptr_t)x) & 15) == 0);
  long sblocks = ((svec ? n / 4 : n) + 255) / 256;
  if (sblocks > (long)sm_count() * 8) sblocks = (long)sm_count() * 8;
  if (sblocks < 1) sblocks = 1;
  if (launch_dependent(k_split_f16, dim3((unsigned)sblocks), dim3(256), 0, stream(), x, aux, rows, aux_rows(rows), n, svec,
                       exp_dev, 0, only_if) != cudaSuccess)
    return set_error(cudaGetErrorString(cudaGetLastError()));
  return check_launch();
}
}  // namespace b200

// One term of a fused product: op(a) is M x k, op(b) is k x N (handles carry is_trans).
// a_part / b_part choose what of each fp32 matrix the term multiplies (kPartX, kPartLo32:
// a TF32 product; kPartLo16, kPartB16: a bfloat16 product); both of one width.  a_aux / b_aux:
// the aux matrix of a / b (or null): its bfloat16 parts are then read from there.
struct b200_pass {
  cudamat* a;
  cudamat* b;
  int negate;
  int a_part, b_part;
  cudamat* a_aux;
  cudamat* b_aux;
  // Row windows of the STORED matrices (0, 0 = all rows): a_rows > 0 restricts a (not transposed) to
  // rows [a_row0, a_row0 + a_rows), a panel of the output's rows; b_rows > 0 restricts b (transposed)
  // likewise, a panel of the output's columns.  Offsets are multiples of 8.
  int a_row0, a_rows, b_row0, b_rows;
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
  cudamat* out_aux;    // aux matrix of the result, or null
  cudamat* sample;     // Bernoulli(result), or null
  cudamat* sample_aux; // aux matrix of the draw, or null
  // scaled half-precision operands (parts kPartF16Lo / kPartF16Hi): the terms carry a factor
  // 2^(*scale_exp + scale_exp_const) (scale_exp: 1 x 1 device matrix or null), divided out of alpha;
  // aux_f16 != 0: out_aux / sample_aux are written in that form with exponent aux_exp
  cudamat* scale_exp;
  int scale_exp_const;
  int aux_f16;
  int aux_exp;
};

extern "C" {

// 0 auto (tensor cores when the operands are TMA-addressable), 1 tensor cores only
// (ERROR_UNSUPPORTED otherwise), 2 CUDA cores only.
int b200_set_gemm_path(int path) {
  g_path = path;
  return 0;
}
// Precision of `dot`: 0 = fp32-grade (three TF32 terms over x and x - tf32(x)),
// 1 = one TF32 term (about 1e-3 relative).
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

// aux = the bfloat16 planes of x (see split_aux in common.cuh); aux holds aux_rows(rows) x cols floats.
int split_bf16(cudamat* x, cudamat* aux) {
  if (!x->on_device || !aux->on_device) return ERROR_NOT_ON_DEVICE;
  if (x->is_trans || aux->is_trans) return ERROR_TRANSPOSED;
  if (!aux_shape_ok(aux, x)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  return launch_split_aux(x->data_device, aux->data_device, x->size[0], numel(x));
}

// aux = x in scaled half-precision form, scale 2^(*exp_dev + exp_const) (exp_dev: 1 x 1 device matrix or null).
int split_f16(cudamat* x, cudamat* aux, cudamat* exp_dev, int exp_const) {
  if (!x->on_device || !aux->on_device || (exp_dev && !exp_dev->on_device)) return ERROR_NOT_ON_DEVICE;
  if (x->is_trans || aux->is_trans) return ERROR_TRANSPOSED;
  if (!aux_shape_ok(aux, x)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const long n = numel(x);
  if (n == 0) return 0;
  const int rows = x->size[0];
  const bool vec = (rows % 4 == 0) && ((((uintptr_t)x->data_device) & 15) == 0);
  long blocks = ((vec ? n / 4 : n) + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  if (blocks < 1) blocks = 1;
  if (launch_dependent(k_split_f16, dim3((unsigned)blocks), dim3(256), 0, stream(), x->data_device,
                       reinterpret_cast<uint16_t*>(aux->data_device), rows, aux_rows(rows), n, vec,
                       exp_dev ? exp_dev->data_device : nullptr, exp_const, nullptr) != cudaSuccess)
    return set_error(cudaGetErrorString(cudaGetLastError()));
  return check_launch();
}

int fused_gemm(rnd_struct* rnd_state, b200_fused_gemm* f) {
  if (f->npass <= 0 || f->npass > kMaxPass) return ERROR_UNSUPPORTED;
  GemmProblem g;
  g.npass = f->npass;
  g.tf32_operands = 1;
  g.M = f->pass[0].a_rows > 0 ? f->pass[0].a_rows : lead(f->pass[0].a);
  g.N = f->pass[0].b_rows > 0 ? f->pass[0].b_rows : nonlead(f->pass[0].b);
  for (int q = 0; q < f->npass; q++) {
    const cudamat *a = f->pass[q].a, *b = f->pass[q].b;
    const b200_pass& ps = f->pass[q];
    if (!a->on_device || !b->on_device) return ERROR_NOT_ON_DEVICE;
    // a window selects rows of the stored matrix that run along M (a as stored) or N (b transposed)
    if (ps.a_rows > 0 && (a->is_trans || ps.a_row0 < 0 || (ps.a_row0 & 7) || ps.a_row0 + ps.a_rows > a->size[0])) return ERROR_UNSUPPORTED;
    if (ps.b_rows > 0 && (!b->is_trans || ps.b_row0 < 0 || (ps.b_row0 & 7) || ps.b_row0 + ps.b_rows > b->size[0])) return ERROR_UNSUPPORTED;
    const int m_q = ps.a_rows > 0 ? ps.a_rows : lead(a), n_q = ps.b_rows > 0 ? ps.b_rows : nonlead(b);
    if (m_q != g.M || n_q != g.N || nonlead(a) != lead(b)) return ERROR_INCOMPATIBLE_DIMENSIONS;
    const int pa = f->pass[q].a_part, pb = f->pass[q].b_part;
    if (pa < 0 || pa >= kNumParts || pb < 0 || pb >= kNumParts) return ERROR_UNSUPPORTED;
    // both operands of a term of one kind: fp32-wide, bfloat16, or scaled half precision (aux only)
    if (part_is_16bit(pa) != part_is_16bit(pb) || part_is_f16(pa) != part_is_f16(pb)) return ERROR_UNSUPPORTED;
    if (part_is_f16(pa) && (!f->pass[q].a_aux || !f->pass[q].b_aux)) return ERROR_UNSUPPORTED;
    const cudamat *xa = f->pass[q].a_aux, *xb = f->pass[q].b_aux;
    if ((xa && !aux_shape_ok(xa, a)) || (xb && !aux_shape_ok(xb, b))) return ERROR_INCOMPATIBLE_DIMENSIONS;
    g.pass[q].a = operand(a, pa, xa);
    g.pass[q].b = operand(b, pb, xb);
    if (ps.a_rows > 0) g.pass[q].a.row0 = ps.a_row0;
    if (ps.b_rows > 0) g.pass[q].b.row0 = ps.b_row0;
    g.pass[q].k = nonlead(a);
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
  e.aux_f16 = f->aux_f16;
  e.aux_exp = f->aux_exp;
  e.scale_exp = nullptr;
  e.scale_exp_const = f->scale_exp_const;
  if (f->scale_exp) {
    if (!f->scale_exp->on_device) return ERROR_NOT_ON_DEVICE;
    e.scale_exp = f->scale_exp->data_device;
  }
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
  e.aux_f16 = e.aux_exp = e.scale_exp_const = 0;
  e.scale_exp = nullptr;
  e.col0 = 0;
  e.key = make_philox_key(0, 0);
  g.npass = 1;
  g.pass[0].a = operand(mat1, kPartX);
  g.pass[0].b = operand(mat2, kPartX);
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
  // fp32-grade: x = tf32(x) + lo with lo = x - tf32(x); lo.x + x.lo + x.x, small terms first,
  // every term a TF32 product (the kernel derives lo from the staged tile of x).  The cheaper
  // bfloat16 correction terms are a few times less accurate (2^-18 against 2^-20 per term),
  // which shows when a caller subtracts two nearly equal products, as the positive and
  // negative statistics are.
  g.npass = 3;
  const int pa[3] = {kPartLo32, kPartX, kPartX}, pb[3] = {kPartX, kPartLo32, kPartX};
  for (int q = 0; q < 3; q++) {
    g.pass[q].a = operand(mat1, pa[q]);
    g.pass[q].b = operand(mat2, pb[q]);
    g.pass[q].k = k;
    g.pass[q].negate = 0;
  }
  g.tf32_operands = 1;
  return gemm_tc(g);
}

// deepnet/dbm.py:242,254 + deepnet/parameter.py:80-106 in one pass over the parameter:
//   grad += suff * (-inv_batch); delta = momentum*delta + l2*w + l1*sign(w) + grad;
//   w -= eps * delta; grad = 0; and, when w_aux is given, the aux matrix of the new w: its
//   bfloat16 parts, or with w_scale (1 x 4 device matrix {exponent, -, max |w| bits, -}) its
//   scaled half-precision form, written in the same pass with the exponent carried so far; a
//   second pass rewrites it only when the new w no longer fits that exponent.
// grad may be null (treated as zero and not written).  20 bytes of traffic per element
// without grad and aux; +8 with grad, +4 with either aux (+8 more in an update that changes the exponent).
// The update restricted to columns [col0, col0 + ncols) of the parameter (and of delta, grad, suff,
// w_aux): the statistics of a data-parallel update arrive panel by panel (each after its own
// all-reduce) and every panel is updated as it arrives.  In scaled half-precision form all panels
// use the exponent carried so far; the check of that exponent against the new parameter (and, if it
// no longer fits, the rewrite of the whole aux) runs with the panel that ends at the last column.
int momentum_update_columns(cudamat* w, cudamat* delta, cudamat* grad, cudamat* suff, cudamat* w_aux, cudamat* w_scale,
                            int col0, int ncols, float inv_batch, float momentum, float eps, float l2, float l1) {
  if (!w->on_device || !delta->on_device || !suff->on_device) return ERROR_NOT_ON_DEVICE;
  if (!same_shape(w, delta) || !same_shape(w, suff)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (grad && (!grad->on_device || !same_shape(w, grad))) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (w_aux && (w->is_trans || !aux_shape_ok(w_aux, w))) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (w_scale && (!w_aux || !w_scale->on_device || numel(w_scale) < 4)) return ERROR_INCOMPATIBLE_DIMENSIONS;
  if (w->is_trans && !(col0 == 0 && ncols == w->size[1])) return ERROR_TRANSPOSED;
  if (col0 < 0 || ncols < 0 || col0 + ncols > w->size[1]) return ERROR_INCOMPATIBLE_DIMENSIONS;
  const int rows = w->size[0];
  const long n = (long)rows * ncols, first = (long)rows * col0;
  const bool last_panel = col0 + ncols == w->size[1];
  float* sp = w_scale ? w_scale->data_device : nullptr;
  uint16_t* ap = w_aux ? reinterpret_cast<uint16_t*>(w_aux->data_device) : nullptr;
  const int mode = !w_aux ? 0 : (w_scale ? 2 : 1);
  const int lda = aux_rows(rows);
  if (n > 0) {
    float *wp = w->data_device + first, *dp = delta->data_device + first, *gp = grad ? grad->data_device + first : nullptr;
    const float* sfp = suff->data_device + first;
    uint16_t* app = ap ? ap + (long)col0 * 2 * lda : nullptr;
    uintptr_t bits = (uintptr_t)wp | (uintptr_t)dp | (uintptr_t)sfp;
    if (gp) bits |= (uintptr_t)gp;
    if (app) bits |= (uintptr_t)app;
    const bool vec = (bits & 15) == 0 && n % 4 == 0 && (!w_aux || rows % 4 == 0);
    long blocks = ((vec ? n / 4 : n) + 255) / 256;
    if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
    if (blocks < 1) blocks = 1;
#define LAUNCH_UPDATE(G, A)                                                                                          \
  (void)launch_dependent(k_update<G, A>, dim3((unsigned)blocks), dim3(256), 0, stream(), wp, dp, gp, sfp, app, sp, rows, lda, n, \
                         vec, -inv_batch, momentum, -eps, l2, l1)
    if (grad) {
      if (mode == 2) LAUNCH_UPDATE(true, 2);
      else if (mode == 1) LAUNCH_UPDATE(true, 1);
      else LAUNCH_UPDATE(true, 0);
    } else {
      if (mode == 2) LAUNCH_UPDATE(false, 2);
      else if (mode == 1) LAUNCH_UPDATE(false, 1);
      else LAUNCH_UPDATE(false, 0);
    }
#undef LAUNCH_UPDATE
    const int err = check_launch();
    if (err) return err;
  }
  if (mode != 2 || !last_panel) return 0;
  (void)launch_dependent(k_update_scale, dim3(1), dim3(1), 0, stream(), sp);
  int err = check_launch();
  if (err) return err;
  const long total = numel(w);
  if (total == 0) return 0;
  const bool svec = (rows % 4 == 0) && ((((uintptr_t)w->data_device) & 15) == 0);
  long sblocks = ((svec ? total / 4 : total) + 255) / 256;
  if (sblocks > (long)sm_count() * 8) sblocks = (long)sm_count() * 8;
  if (sblocks < 1) sblocks = 1;
  // (returns at once unless the exponent had to change)
  (void)launch_dependent(k_split_f16, dim3((unsigned)sblocks), dim3(256), 0, stream(), w->data_device, ap, rows, lda, total, svec,
                         sp, 0, sp + 3);
  return check_launch();
}

int momentum_update(cudamat* w, cudamat* delta, cudamat* grad, cudamat* suff, cudamat* w_aux, cudamat* w_scale,
                    float inv_batch, float momentum, float eps, float l2, float l1) {
  return momentum_update_columns(w, delta, grad, suff, w_aux, w_scale, 0, w->size[1], inv_batch, momentum, eps, l2, l1);
}

}  // extern "C"
