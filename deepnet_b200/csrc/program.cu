// A recorded list of operations run by one call from the host.
//
// The contrastive-divergence update is a fixed sequence of 10-60 library calls per minibatch
// (deepnet/dbm.py:268-274 drives them one by one from Python).  At the small configurations
// each call's host cost (argument marshalling in the caller's language, about 14 us from
// Python) exceeds the kernel it launches.  A caller therefore records the sequence once, as an
// array of b200_op, and replays it with b200_run_program: every launch of an update is then
// issued from C in one call.  The operations are the library's own entry points; the random
// stream advances exactly as if the calls had been made one by one.
#include "common.cuh"

struct b200_fused_gemm;

extern "C" {
int fused_gemm(rnd_struct* rnd_state, b200_fused_gemm* f);
int sum_by_axis(cudamat* mat, cudamat* target, int axis);
int add_sum_by_axis(cudamat* mat, cudamat* target, int axis, float mult);
int row_sum_diff(cudamat* a, cudamat* b, cudamat* target);
int add_sq_diff(cudamat* a, cudamat* b, cudamat* acc);
int momentum_update(cudamat* w, cudamat* delta, cudamat* grad, cudamat* suff, cudamat* w_aux, cudamat* w_scale,
                    float inv_batch, float momentum, float eps, float l2, float l1);
int momentum_update_columns(cudamat* w, cudamat* delta, cudamat* grad, cudamat* suff, cudamat* w_aux, cudamat* w_scale,
                            int col0, int ncols, float inv_batch, float momentum, float eps, float l2, float l1);
int dp_allreduce_begin(cudamat* mat, int slot);
int dp_allreduce_end(int slot);
int b200_set_sm_limit(int sms);
int dp_peer_update(cudamat* w, cudamat* delta, cudamat* w_aux, cudamat* w_scale, cudamat* pack, cudamat* b, cudamat* db,
                   float inv_batch, float mom_b, float eps_b, float mom_w, float eps_w, float l2, float l1);
int split_f16(cudamat* x, cudamat* aux, cudamat* exp_dev, int exp_const);
int split_bf16(cudamat* x, cudamat* aux);
int dp_allreduce(cudamat* mat);
int softmax_scaled(cudamat* mat, cudamat* scale, cudamat* target);
int sample_multinomial(rnd_struct* rnd_state, cudamat* probs, cudamat* nn, cudamat* target, int max_draws);
int div_by_row_vec(cudamat* mat, cudamat* vec, cudamat* target);
int add_scalar(cudamat* mat, float alpha, cudamat* target);
int assign_scalar(cudamat* mat, float alpha);
int copy_on_device(cudamat* mat1, cudamat* mat2);
int sample_bernoulli(rnd_struct* rnd_state, cudamat* mat, cudamat* target);
int softmax_sample(rnd_struct* rnd_state, cudamat* pre, cudamat* bias, cudamat* state, cudamat* sample);
}

enum {
  B200_OP_FUSED_GEMM = 0,      // gemm
  B200_OP_SUM_AXIS = 1,        // m0 mat, m1 target, i0 axis
  B200_OP_ADD_SUM_AXIS = 2,    // m0 mat, m1 target, i0 axis, f0 mult
  B200_OP_ROW_SUM_DIFF = 3,    // m0 a, m1 b, m2 target
  B200_OP_ADD_SQ_DIFF = 4,     // m0 a, m1 b, m2 acc
  B200_OP_MOMENTUM_UPDATE = 5, // m0 w, m1 delta, m2 grad?, m3 suff, m4 w_aux?, m5 w_scale?; f0 inv_batch, f1 momentum, f2 eps, f3 l2, f4 l1
  B200_OP_SPLIT_F16 = 6,       // m0 x, m1 aux, m2 exp_dev?, i0 exp_const
  B200_OP_SPLIT_BF16 = 7,      // m0 x, m1 aux
  B200_OP_ALLREDUCE = 8,       // m0
  B200_OP_SOFTMAX_SCALED = 9,  // m0 mat, m1 scale, m2 target
  B200_OP_SAMPLE_MULTINOMIAL = 10,  // m0 probs, m1 nn, m2 target, i0 max_draws
  B200_OP_DIV_BY_ROW = 11,     // m0 mat, m1 vec, m2 target
  B200_OP_ADD_SCALAR = 12,     // m0 mat, m1 target, f0 value
  B200_OP_ASSIGN_SCALAR = 13,  // m0 mat, f0 value
  B200_OP_COPY = 14,           // m0 source, m1 target
  B200_OP_SAMPLE_BERNOULLI = 15,   // m0 mat, m1 target
  B200_OP_SOFTMAX_SAMPLE = 16, // m0 pre, m1 bias?, m2 state, m3 sample?
  B200_OP_MOMENTUM_UPDATE_COLUMNS = 17,  // as 5, on columns [i0, i0 + i1)
  B200_OP_ALLREDUCE_BEGIN = 18,   // m0, i0 slot
  B200_OP_ALLREDUCE_END = 19,     // i0 slot
  B200_OP_SM_LIMIT = 20,          // i0 SMs the following kernels size their grids for (0 = all)
  B200_OP_DP_PEER_UPDATE = 21,    // m0 w, m1 delta, m2 w_aux?, m3 w_scale?, m4 pack, m5 b, m6 db; f0 inv_batch, f1 mom_b, f2 eps_b, f3 mom_w, f4 eps_w, f5 l2, f6 l1
  B200_OP_COUNT
};

struct b200_op {
  int kind;
  int i0, i1, i2;
  float f0, f1, f2, f3, f4, f5, f6, f7;
  cudamat* m[8];
  b200_fused_gemm* gemm;
};

// Runs ops[0..n) in order on the library stream.  Stops at the first failing operation and returns
// its error code; *failed_at (optional) receives its index.
extern "C" int b200_run_program(rnd_struct* rnd_state, b200_op* ops, int n, int* failed_at) {
  for (int i = 0; i < n; i++) {
    b200_op& o = ops[i];
    int err = ERROR_UNSUPPORTED;
    switch (o.kind) {
      case B200_OP_FUSED_GEMM: err = fused_gemm(rnd_state, o.gemm); break;
      case B200_OP_SUM_AXIS: err = sum_by_axis(o.m[0], o.m[1], o.i0); break;
      case B200_OP_ADD_SUM_AXIS: err = add_sum_by_axis(o.m[0], o.m[1], o.i0, o.f0); break;
      case B200_OP_ROW_SUM_DIFF: err = row_sum_diff(o.m[0], o.m[1], o.m[2]); break;
      case B200_OP_ADD_SQ_DIFF: err = add_sq_diff(o.m[0], o.m[1], o.m[2]); break;
      case B200_OP_MOMENTUM_UPDATE:
        err = momentum_update(o.m[0], o.m[1], o.m[2], o.m[3], o.m[4], o.m[5], o.f0, o.f1, o.f2, o.f3, o.f4);
        break;
      case B200_OP_SPLIT_F16: err = split_f16(o.m[0], o.m[1], o.m[2], o.i0); break;
      case B200_OP_SPLIT_BF16: err = split_bf16(o.m[0], o.m[1]); break;
      case B200_OP_ALLREDUCE: err = dp_allreduce(o.m[0]); break;
      case B200_OP_SOFTMAX_SCALED: err = softmax_scaled(o.m[0], o.m[1], o.m[2]); break;
      case B200_OP_SAMPLE_MULTINOMIAL: err = sample_multinomial(rnd_state, o.m[0], o.m[1], o.m[2], o.i0); break;
      case B200_OP_DIV_BY_ROW: err = div_by_row_vec(o.m[0], o.m[1], o.m[2]); break;
      case B200_OP_ADD_SCALAR: err = add_scalar(o.m[0], o.f0, o.m[1]); break;
      case B200_OP_ASSIGN_SCALAR: err = assign_scalar(o.m[0], o.f0); break;
      case B200_OP_COPY: err = copy_on_device(o.m[0], o.m[1]); break;
      case B200_OP_SAMPLE_BERNOULLI: err = sample_bernoulli(rnd_state, o.m[0], o.m[1]); break;
      case B200_OP_SOFTMAX_SAMPLE: err = softmax_sample(rnd_state, o.m[0], o.m[1], o.m[2], o.m[3]); break;
      case B200_OP_MOMENTUM_UPDATE_COLUMNS:
        err = momentum_update_columns(o.m[0], o.m[1], o.m[2], o.m[3], o.m[4], o.m[5], o.i0, o.i1, o.f0, o.f1, o.f2, o.f3, o.f4);
        break;
      case B200_OP_ALLREDUCE_BEGIN: err = dp_allreduce_begin(o.m[0], o.i0); break;
      case B200_OP_ALLREDUCE_END: err = dp_allreduce_end(o.i0); break;
      case B200_OP_SM_LIMIT: err = b200_set_sm_limit(o.i0); break;
      case B200_OP_DP_PEER_UPDATE:
        err = dp_peer_update(o.m[0], o.m[1], o.m[2], o.m[3], o.m[4], o.m[5], o.m[6], o.f0, o.f1, o.f2, o.f3, o.f4, o.f5, o.f6);
        break;
      default: break;
    }
    if (err) {
      if (failed_at) *failed_at = i;
      return err;
    }
  }
  return 0;
}
