// Description of one fused matrix product shared by the tensor-core and the SIMT
// kernels:  out = act(alpha * sum_p (+/-) op(A_p) . op(B_p) + beta * out + bias (x) scale)
// with an optional Bernoulli draw of the result, and optionally the aux matrices (bfloat16
// parts) of result and draw for the products that read them next.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kMaxPass = 8;

// Which part of an fp32 matrix x a term multiplies.  The kernels derive the parts from x
// on the fly (the tensor-core kernel in shared memory, next to the tile TMA delivered), so
// only x itself lives in device memory:
//   kPartX     x, read as TF32 on the tensor cores (the hardware drops the low 13 mantissa bits)
//   kPartLo32  x - tf32(x), read as TF32 (keeps 10 of its up to 13 significant bits)
//   kPartLo16  bfloat16(x - tf32(x))
//   kPartB16   bfloat16(x)
// so that, small terms first,
//   a . b ~= lo32(a).x(b) + x(a).lo32(b) + x(a).x(b)      three TF32 products, 2^-20 per term
//   a . b ~= lo16(a).b16(b) + b16(a).lo16(b) + x(a).x(b)  one TF32 + two bfloat16 products
//                                                        (twice the TF32 rate), 2^-18 per term
// accumulate into one fp32 accumulator.  Both operands of a term are of the same width.
// The bfloat16 parts may instead be READ from an aux matrix of x kept in device memory (see
// split_aux): deriving them costs shared-memory bandwidth (the fp32 tile is read and two tiles
// are written, next to the tensor core's own operand reads), which bounds the big products.
//   kPartF16Lo, kPartF16Hi  the two planes of an aux matrix in scaled half-precision form (see
//                           split_f16): a . b * 2^(ea + eb) ~= hi.hi + hi.lo + lo.hi, read from memory only
enum { kPartX = 0, kPartLo32 = 1, kPartLo16 = 2, kPartB16 = 3, kPartF16Lo = 4, kPartF16Hi = 5, kNumParts = 6 };
inline bool part_is_16bit(int part) { return part >= kPartLo16; }
inline bool part_is_f16(int part) { return part >= kPartF16Lo; }
inline int part_plane(int part) { return (part == kPartB16 || part == kPartF16Hi) ? 1 : 0; }

// A column-major fp32 matrix in device memory: element (r, c) at ptr[c * ld + r].
// trans = 1 means the product uses its transpose.
struct GemmOperand {
  const float* ptr;
  int ld;
  int trans;
  int part;
  const float* aux;   // aux matrix of the same matrix (or null: bfloat16 parts are derived from ptr)
  int lda;            // floats per column of aux
  int row0;           // first stored row of the window the product reads (its length is M or N): a panel of the
                      // output rows (a, not transposed) or columns (b, transposed) without copying the operand
};

// One term of the sum: op(a) is M x k, op(b) is k x N.
struct GemmPass {
  GemmOperand a, b;
  int k;
  int negate;
};

struct GemmEpilogue {
  float alpha, beta;
  const float* bias;       // M entries or null: added per output row
  const float* col_scale;  // N entries or null: the bias of column n is bias[m] * col_scale[n]
  int activation;          // 0 identity, 1 logistic
  float* out;              // M x N result (may be null when only split/sample outputs are wanted)
  float* out_aux;          // aux matrix of the result, or null
  int aux_f16;             // 1: aux outputs in scaled half-precision form (exponent aux_exp), 0: bfloat16 parts
  int aux_exp;
  const float* scale_exp;  // device scalar or null: the products carry a factor 2^(*scale_exp + scale_exp_const)
  int scale_exp_const;     // (scaled half-precision operands), which the epilogue divides out of alpha
  float* sample;           // Bernoulli(result) draw, or null
  float* sample_aux;       // aux matrix of the draw (only plane 1 is written: a 0/1 value has no low part), or null
  int ldo;                 // leading dimension of every fp32 output
  int ld_aux;              // floats per column of the aux outputs (rows rounded up to 8)
  PhiloxKey key;           // random stream of this call (used when sample != null)
  int col0;                // global column of output column 0
};

struct GemmProblem {
  int M, N;
  int npass;
  // 1: part kPartX is read as TF32 (low 13 mantissa bits ignored), its meaning on the tensor
  // cores, which the CUDA-core kernel then reproduces; 0: kPartX is the full fp32 value.
  int tf32_operands;
  GemmPass pass[kMaxPass];
  GemmEpilogue epi;
};

// aux = x * 2^(*exp_dev) as two fp16 planes, written only when *only_if != 0 (a device flag): the
// second pass of an update whose exponent had to change.
int rewrite_f16_planes_if(const float* x, uint16_t* aux, int rows, long n, const float* exp_dev, const float* only_if);

// From now on a tensor-core product whose result is `match` stores columns [q * cols, (q + 1) * cols)
// of it to out[q] instead (same row layout), q < n; n = 0 ends it.  The data-parallel step registers
// the peers' receive buffers here, so that its statistics reach their owners while the product runs.
int set_product_scatter(const float* match, float* const* out, int n, int cols);
bool product_is_scattered(const float* out);
int gemm_simt(const GemmProblem& g);
// Returns ERROR_UNSUPPORTED when an operand is not addressable by TMA (leading
// dimension not a multiple of 4 floats or base not 16-byte aligned).
int gemm_tc(const GemmProblem& g);
bool gemm_tc_supported(const GemmProblem& g);

#ifdef __CUDACC__
// Applies the epilogue to one accumulator value and stores every requested output.
// `u` is the uniform of this element (only read when e.sample != null).
__device__ __forceinline__ void epilogue_store(const GemmEpilogue& e, float acc, int m, int n, float u) {
  const long idx = (long)n * e.ldo + m;
  float v = e.alpha * exp2f(-((e.scale_exp ? *e.scale_exp : 0.0f) + (float)e.scale_exp_const)) * acc;
  if (e.beta != 0.0f) v += e.beta * e.out[idx];
  if (e.bias) v += e.col_scale ? e.bias[m] * e.col_scale[n] : e.bias[m];
  if (e.activation == 1) v = sigmoid_accurate(v);
  if (e.out) e.out[idx] = v;
  const long aidx = (long)n * 2 * e.ld_aux + m;   // 16-bit word of plane 0
  if (e.out_aux) {
    uint16_t lo16, b16;
    if (e.aux_f16) split_f16(v, exp2f((float)e.aux_exp), lo16, b16);
    else split_aux(v, lo16, b16);
    reinterpret_cast<uint16_t*>(e.out_aux)[aidx] = lo16;
    reinterpret_cast<uint16_t*>(e.out_aux)[aidx + e.ld_aux] = b16;
  }
  const float s = u < v ? 1.0f : 0.0f;
  if (e.sample) e.sample[idx] = s;
  if (e.sample_aux) {
    const uint16_t one = e.aux_f16 ? __half_as_ushort(__float2half_rn(exp2f((float)e.aux_exp))) : (uint16_t)0x3f80;
    reinterpret_cast<uint16_t*>(e.sample_aux)[aidx + e.ld_aux] = s != 0.0f ? one : (uint16_t)0;
  }
}
#endif

}  // namespace b200
