// Description of one fused matrix product shared by the tensor-core and the SIMT
// kernels:  out = act(alpha * sum_p (+/-) op(A_p) . op(B_p) + beta * out + bias (x) scale)
// with optional TF32 hi/lo split outputs and a Bernoulli draw of the result.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kMaxPass = 8;

// A column-major matrix in device memory: element (r, c) at ptr[c * ld + r].
// trans = 1 means the product uses its transpose.
struct GemmOperand {
  const float* ptr;
  int ld;
  int trans;
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
  float* out_hi;           // TF32-exact high part of the result, or null
  float* out_lo;           // result - out_hi, or null
  float* sample;           // Bernoulli(result) draw, or null
  int ldo;                 // leading dimension of every output
  PhiloxKey key;           // random stream of this call (used when sample != null)
  int col0;                // global column of output column 0
};

struct GemmProblem {
  int M, N;
  int npass;
  // 1: operands are read as TF32 (low 13 mantissa bits ignored), the meaning of a pass on
  // the tensor cores, which the CUDA-core kernel then reproduces; 0: full fp32 operands.
  int tf32_operands;
  GemmPass pass[kMaxPass];
  GemmEpilogue epi;
};

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
  float v = e.alpha * acc;
  if (e.beta != 0.0f) v += e.beta * e.out[idx];
  if (e.bias) v += e.col_scale ? e.bias[m] * e.col_scale[n] : e.bias[m];
  if (e.activation == 1) v = sigmoid_accurate(v);
  if (e.out) e.out[idx] = v;
  if (e.out_hi || e.out_lo) {
    float hi, lo;
    split_tf32(v, hi, lo);
    if (e.out_hi) e.out_hi[idx] = hi;
    if (e.out_lo) e.out_lo[idx] = lo;
  }
  if (e.sample) e.sample[idx] = u < v ? 1.0f : 0.0f;
}
#endif

}  // namespace b200
