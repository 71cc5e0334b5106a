// fp32 CUDA-core product for operands the tensor-core path cannot address (leading
// dimensions that are not multiples of 4 floats, unaligned views) and for tiny
// problems.  64x64 output tile, 16-deep slices in shared memory, 4x4 outputs per
// thread, every edge bounds-checked.  Same pass list and epilogue as the tcgen05 kernel.
#include "gemm.cuh"

namespace b200 {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ float as_operand(float x, int tf32) {
  return tf32 ? __uint_as_float(__float_as_uint(x) & 0xffffe000u) : x;
}
// Element (r, c) of the stored matrix, as the part the term reads.
__device__ __forceinline__ float element(const GemmOperand& o, int r, int c, int tf32) {
  r += o.row0;
  if (o.part >= kPartLo16 && o.aux) {
    const long w = (long)c * 2 * o.lda + ((o.part == kPartB16 || o.part == kPartF16Hi) ? o.lda : 0) + r;
    const uint16_t bits = reinterpret_cast<const uint16_t*>(o.aux)[w];
    return o.part >= kPartF16Lo ? f16_to_float(bits) : bf16_to_float(bits);
  }
  if (o.part >= kPartF16Lo) return 0.0f;   // scaled half-precision parts exist in aux matrices only
  const float x = o.ptr[(long)c * o.ld + r];
  if (o.part == kPartX) return as_operand(x, tf32);
  if (o.part == kPartB16) return bf16_to_float(float_to_bf16(x));
  const float lo = x - as_operand(x, 1);
  return o.part == kPartLo32 ? as_operand(lo, 1) : bf16_to_float(float_to_bf16(lo));
}
__device__ __forceinline__ float load_a(const GemmOperand& a, int m, int k, int M, int K, int tf32) {
  if (m >= M || k >= K) return 0.0f;
  return a.trans ? element(a, k, m, tf32) : element(a, m, k, tf32);
}
__device__ __forceinline__ float load_b(const GemmOperand& b, int k, int n, int K, int N, int tf32) {
  if (n >= N || k >= K) return 0.0f;
  return b.trans ? element(b, n, k, tf32) : element(b, k, n, tf32);
}

__global__ void __launch_bounds__(256) k_gemm_simt(const __grid_constant__ GemmProblem g) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

  for (int p = 0; p < g.npass; p++) {
    const GemmPass& ps = g.pass[p];
    const float sgn = ps.negate ? -1.0f : 1.0f;
    for (int k0 = 0; k0 < ps.k; k0 += TK) {
      // stage the slices; the thread->element map follows the contiguous direction
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int m, k;
        if (ps.a.trans) { k = tid & 15; m = (tid >> 4) + 16 * i; }
        else { m = tid & 63; k = (tid >> 6) + 4 * i; }
        As[k][m] = sgn * load_a(ps.a, m0 + m, k0 + k, g.M, ps.k, g.tf32_operands);
        int n, kb;
        if (ps.b.trans) { n = tid & 63; kb = (tid >> 6) + 4 * i; }
        else { kb = tid & 15; n = (tid >> 4) + 16 * i; }
        Bs[kb][n] = load_b(ps.b, k0 + kb, n0 + n, ps.k, g.N, g.tf32_operands);
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < TK; k++) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; i++) a[i] = As[k][tx + 16 * i];
#pragma unroll
        for (int j = 0; j < 4; j++) b[j] = Bs[k][ty + 16 * j];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }

  const GemmEpilogue e = g.epi;  // private copy: no reloads of the parameter block after each store
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int n = n0 + ty + 16 * j;
    if (n >= g.N) continue;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int m = m0 + tx + 16 * i;
      if (m >= g.M) continue;
      float u = 0.0f;
      if (e.sample || e.sample_aux) {
        const int gc = n + e.col0;
        const uint4 w = philox4x32_10((uint32_t)m, (uint32_t)(gc >> 2), e.key);
        u = word_to_uniform(pick_word(w, gc & 3));
      }
      epilogue_store(e, acc[i][j], m, n, u);
    }
  }
}

}  // namespace

int gemm_simt(const GemmProblem& g) {
  if (g.M <= 0 || g.N <= 0) return 0;
  dim3 grid((g.M + TM - 1) / TM, (g.N + TN - 1) / TN);
  k_gemm_simt<<<grid, 256, 0, stream()>>>(g);
  return check_launch();
}

}  // namespace b200
