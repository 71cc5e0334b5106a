/*
 * b200mat.h -- C ABI of libb200mat.so, an sm_100a replacement for the cudamat shared
 * library on the contrastive-divergence path of deepnet.
 *
 * Every entry point takes plain pointers and scalars (no C++ or framework types) and,
 * unless noted, returns 0 or one of the negative codes below.  Each declaration cites
 * the reference interface it replaces (paths relative to the reference project);
 * additions that have no counterpart there say so.  Matrices are float32,
 * column-major, size[0] rows by size[1] columns; operations are enqueued on one
 * library stream and the host blocks only where a value returns to it.
 */
#ifndef B200MAT_H_
#define B200MAT_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudamat/cudamat.cuh:1-9 */
#define ERROR_INCOMPATIBLE_DIMENSIONS -1
#define CUBLAS_ERROR -2
#define CUDA_ERROR -3
#define VIEW_ERROR -4
#define ERROR_TRANSPOSED -5
#define ERROR_GENERIC -6
#define ERROR_TRANSPOSEDNESS -7
#define ERROR_NOT_ON_DEVICE -8
#define ERROR_UNSUPPORTED -9
/* additions */
#define ERROR_NCCL -10
#define ERROR_DEVICE_TIMEOUT -11

/* cudamat/cudamat.cuh:21-29 (same layout) */
typedef struct cudamat {
  float* data_host;
  float* data_device;
  int on_device;
  int on_host;
  int size[2];
  int is_trans;
  int owns_data;
} cudamat;

/* cudamat/cudamat.cuh:31-34 held two device pointers; the same 16 bytes now hold the
 * Philox key and the count of sampling calls issued. */
typedef struct rnd_struct {
  unsigned long long seed;
  unsigned long long calls;
} rnd_struct;

/* ---- library, device, memory: cudamat/cudamat.cu:25-435 ---------------------------- */
const char* get_last_cuda_error(void);                          /* cudamat.cu:25 */
int cublas_init(void);                                          /* cudamat.cu:31 */
int cublas_shutdown(void);                                      /* cudamat.cu:39 */
int cuda_set_device(int deviceId);                              /* cudamat.cu:46 */
int init_random(rnd_struct* rnd_state, int seed, char* cudamatpath); /* cudamat.cu:55 */
int get_leading_dimension(cudamat* mat);                        /* cudamat.cu:87 */
int get_nonleading_dimension(cudamat* mat);                     /* cudamat.cu:91 */
void set_transpose(cudamat* mat, int is_trans);                 /* cudamat.cu:95 */
void cuda_sync_threads(void);                                   /* cudamat.cu:103 */
int allocate_device_memory(cudamat* mat);                       /* cudamat.cu:109 */
int copy_to_host(cudamat* mat);                                 /* cudamat.cu:153 */
int copy_to_device(cudamat* mat);                               /* cudamat.cu:167 */
int copy_on_device(cudamat* mat1, cudamat* mat2);               /* cudamat.cu:217 */
int free_device_memory(cudamat* mat);                           /* cudamat.cu:298 */
int set_shape(cudamat* mat, unsigned int m, unsigned int n);    /* cudamat.cu:312 */
int reshape(cudamat* mat, unsigned int m, unsigned int n);      /* cudamat.cu:321 */
int get_slice(cudamat* source, cudamat* target, unsigned int first_col, unsigned int last_col);        /* cudamat.cu:331 */
int get_vector_slice(cudamat* source, cudamat* target, unsigned int first_ind, unsigned int last_ind); /* cudamat.cu:355 */
void init_from_array(cudamat* mat, float* data, int m, int n);  /* cudamat.cu:397 */
void set_on_device(cudamat* mat);                               /* cudamat.cu:421 */
int init_empty(cudamat* mat, int m, int n);                     /* cudamat.cu:425 (zero-filled, as eigenmat/eigenmat.py:1339) */

/* ---- sampling: cudamat/cudamat.cu:437-590, eigenmat/eigenmat.cc:177-256 ------------- */
int fill_with_rand(rnd_struct* rnd_state, cudamat* mat);                           /* cudamat.cu:437 */
int fill_with_randn(rnd_struct* rnd_state, cudamat* mat);                          /* cudamat.cu:453 */
int sample_bernoulli(rnd_struct* rnd_state, cudamat* mat, cudamat* target);        /* cudamat.cu:469 */
int sample_bernoulli_tanh(rnd_struct* rnd_state, cudamat* mat, cudamat* target);   /* cudamat.cu:486 */
int sample_gaussian(rnd_struct* rnd_state, cudamat* mat, cudamat* target, float mult); /* cudamat.cu:520 */
int perturb_energy(rnd_struct* rnd_state, cudamat* mat, cudamat* target);          /* cudamat.cu:538 */
int perturb_prob(rnd_struct* rnd_state, cudamat* mat, cudamat* target);            /* cudamat.cu:556 */
int dropout(rnd_struct* rnd_state, cudamat* mat, float dropprob, float val);       /* cudamat.cu:574 */

/* ---- broadcasts: cudamat/cudamat.cu:592-876 ------------------------------------------ */
int add_col_vec(cudamat* mat, cudamat* vec, cudamat* target);                 /* cudamat.cu:592 */
int add_col_mult(cudamat* mat, cudamat* vec, cudamat* target, float mult);    /* cudamat.cu:617 */
int add_row_mult(cudamat* mat, cudamat* vec, cudamat* target, float mult);    /* cudamat.cu:735 */
int add_row_vec(cudamat* mat, cudamat* vec, cudamat* target);                 /* cudamat.cu:759 */
int mult_by_col_vec(cudamat* mat, cudamat* vec, cudamat* target);             /* cudamat.cu:783 */
int mult_by_row_vec(cudamat* mat, cudamat* vec, cudamat* target);             /* cudamat.cu:807 */
int div_by_col_vec(cudamat* mat, cudamat* vec, cudamat* target);              /* cudamat.cu:831 */
int div_by_row_vec(cudamat* mat, cudamat* vec, cudamat* target);              /* cudamat.cu:855 */

/* ---- comparisons and clamps: cudamat/cudamat.cu:878-1146 ----------------------------- */
int less_than_eq(cudamat* mat1, cudamat* mat2, cudamat* target);              /* cudamat.cu:878 */
int less_than(cudamat* mat1, cudamat* mat2, cudamat* target);                 /* cudamat.cu:901 */
int less_than_eq_scalar(cudamat* mat, float val, cudamat* target);            /* cudamat.cu:923 */
int less_than_scalar(cudamat* mat, float val, cudamat* target);               /* cudamat.cu:946 */
int greater_than_eq(cudamat* mat1, cudamat* mat2, cudamat* target);           /* cudamat.cu:968 */
int greater_than(cudamat* mat1, cudamat* mat2, cudamat* target);              /* cudamat.cu:991 */
int upper_bound(cudamat* mat1, cudamat* mat2, cudamat* target);               /* cudamat.cu:1014 */
int lower_bound(cudamat* mat1, cudamat* mat2, cudamat* target);               /* cudamat.cu:1038 */
int greater_than_eq_scalar(cudamat* mat, float val, cudamat* target);         /* cudamat.cu:1060 */
int greater_than_scalar(cudamat* mat, float val, cudamat* target);            /* cudamat.cu:1082 */
int upper_bound_scalar(cudamat* mat, float val, cudamat* target);             /* cudamat.cu:1103 */
int lower_bound_scalar(cudamat* mat, float val, cudamat* target);             /* cudamat.cu:1126 */

/* ---- reductions: cudamat/cudamat.cu:1148-1258, 1733, 2104, 2192; eigenmat.cc:733-759 -- */
int max_by_axis(cudamat* mat, cudamat* target, int axis);                     /* cudamat.cu:1148 */
int choose_max_and_accumulate(cudamat* mat, cudamat* acc);                    /* cudamat.cu:1178 */
int choose_max_by_axis(cudamat* mat, cudamat* target, int axis);              /* cudamat.cu:1203, meaning of eigenmat.cc:661 */
int argmax_by_axis(cudamat* mat, cudamat* target, int axis);                  /* cudamat.cu:1232 */
int sum_by_axis(cudamat* mat, cudamat* target, int axis);                     /* eigenmat/eigenmat.cc:746; cudamat/cudamat.py:1546 */
int add_sum_by_axis(cudamat* mat, cudamat* target, int axis, float mult);     /* eigenmat/eigenmat.cc:733; cudamat/cudamat.py:724 */
float vdot(cudamat* mat1, cudamat* mat2, int* err_code);                      /* cudamat.cu:1733 */
float euclid_norm(cudamat* mat, int* err_code);                               /* cudamat.cu:2104 */
float sum_all(cudamat* mat, int* err_code);                                   /* cudamat/cudamat.py:719-721 (vdot with ones) */
int softmax(cudamat* mat, cudamat* target);                                   /* cudamat.cu:2192 */
int softmax_overwrite(cudamat* mat);                                          /* cudamat.cu:2220 */
int apply_softmax(cudamat* mat, cudamat* target);                             /* eigenmat/eigenmat.cc:808 */

/* ---- elementwise: cudamat/cudamat.cu:1318-1670, 1763-2102 ---------------------------- */
int sign(cudamat* mat, cudamat* target);                                      /* cudamat.cu:1318 */
int apply_sigmoid(cudamat* mat, cudamat* target);                             /* cudamat.cu:1376 */
int apply_tanh(cudamat* mat, cudamat* target);                                /* cudamat.cu:1395 */
int apply_abs(cudamat* mat, cudamat* target);                                 /* cudamat.cu:1414 */
int apply_log_1_plus_exp(cudamat* mat, cudamat* target);                      /* cudamat.cu:1433 */
int apply_log(cudamat* mat, cudamat* target, float tiny);                     /* cudamat.cu:1452 */
int apply_exp(cudamat* mat, cudamat* target);                                 /* cudamat.cu:1471 */
int apply_sqrt(cudamat* mat, cudamat* target);                                /* cudamat.cu:1528 */
int apply_pow(cudamat* mat, float pow, cudamat* target);                      /* cudamat.cu:1547 */
int compute_cross_entropy_bernoulli(cudamat* mat, cudamat* p, cudamat* target, float tiny); /* cudamat.cu:1609 */
int correct_preds(cudamat* mat, cudamat* p, cudamat* target, float cutoff);   /* cudamat.cu:1630 */
int reciprocal(cudamat* mat, cudamat* target);                                /* cudamat.cu:1652 */
int add_mult(cudamat* mat1, cudamat* mat2, float alpha);                      /* cudamat.cu:1763 */
int add_mult_sign(cudamat* mat1, cudamat* mat2, float mult);                  /* cudamat.cu:1782 */
int add_elementwise(cudamat* mat1, cudamat* mat2, cudamat* target);           /* cudamat.cu:1803 */
int subtract_elementwise(cudamat* mat1, cudamat* mat2, cudamat* target);      /* cudamat.cu:1826 */
int divide_elementwise(cudamat* mat1, cudamat* mat2, cudamat* target);        /* cudamat.cu:1849 */
int mult_elementwise(cudamat* mat1, cudamat* mat2, cudamat* target);          /* cudamat.cu:1873 */
int apply_logistic_deriv(cudamat* mat1, cudamat* mat2, cudamat* target);      /* cudamat.cu:1940 */
int assign_scalar(cudamat* mat, float alpha);                                 /* cudamat.cu:2031 */
int mult_by_scalar(cudamat* mat, float alpha, cudamat* target);               /* cudamat.cu:2047 */
int divide_by_scalar(cudamat* mat, float alpha, cudamat* target);             /* cudamat.cu:2066 */
int add_scalar(cudamat* mat, float alpha, cudamat* target);                   /* cudamat.cu:2085 */

/* ---- index operations: cudamat/cudamat.cu:2120-2150 ----------------------------------- */
int selectRows(cudamat* source, cudamat* target, cudamat* indices);                         /* cudamat.cu:2120 (select_columns) */
int swapColumns(cudamat* source, cudamat* target, cudamat* indices1, cudamat* indices2);   /* cudamat.cu:2138 */
/* Device-resident data feed (no counterpart in the reference, whose GPUCache slices a device matrix
 * and swaps columns after drawing a permutation on the host, deepnet/datahandler.py:364-416):
 * out (h x count) = stored columns perm(start ..) of src (h x n fp32; or, packed != 0, one bit per
 * value, ceil(h / 32) x n words), perm a keyed bijection of [0, n) evaluated on the device,
 * normalised with mean / std (or both null), with the minibatch's aux matrix (aux_mode 0 none,
 * 1 bfloat16 parts, 2 scaled half precision with exponent aux_exp). */
int feed_gather(cudamat* src, int packed, int h, unsigned int key_lo, unsigned int key_hi, int shuffle, int start,
                cudamat* mean, cudamat* stdv, cudamat* out, cudamat* out_aux, int aux_mode, int aux_exp);
unsigned int feed_permutation_at(unsigned int pos, unsigned int n, unsigned int key_lo, unsigned int key_hi);
int copy_transpose(cudamat* source, cudamat* target);                                       /* cudamat.cu:271 */
int normlimit_by_axis(cudamat* mat, cudamat* target, int axis, float norm);                 /* cudamat.cu:1289 (axis 0 only, as there) */

/* ---- matrix product: cudamat/cudamat.cu:1671-1696 (cublasSgemm) ---------------------- */
/* target = beta * target + alpha * op(mat1) . op(mat2); tcgen05 split-TF32 when the
 * operands are TMA-addressable (leading dimension a multiple of 4, 16-byte aligned). */
int dot(cudamat* mat1, cudamat* mat2, cudamat* target, float beta, float alpha);

/* ================= additions: no counterpart in the reference ======================== */

/* What of an fp32 matrix x a term of a fused product multiplies.  The kernels derive the
 * parts from x on the fly, only x lives in device memory:
 *   B200_PART_X     x, read as TF32 on the tensor cores (the low 13 mantissa bits are dropped)
 *   B200_PART_LO32  x - tf32(x), read as TF32
 *   B200_PART_LO16  bfloat16(x - tf32(x))
 *   B200_PART_B16   bfloat16(x)
 * a . b ~= lo32(a).x(b) + x(a).lo32(b) + x(a).x(b)       three TF32 products, 2^-20 per term, or
 * a . b ~= lo16(a).b16(b) + b16(a).lo16(b) + x(a).x(b)   one TF32 + two bfloat16 products (twice
 *                                                        the TF32 rate), 2^-18 per term. */
enum { B200_PART_X = 0, B200_PART_LO32 = 1, B200_PART_LO16 = 2, B200_PART_B16 = 3,
       B200_PART_F16LO = 4, B200_PART_F16HI = 5 };

/* The bfloat16 parts of a rows x cols fp32 matrix x kept in device memory ("aux matrix"), for
 * the big products: deriving the parts in the kernel costs shared-memory bandwidth next to the
 * tensor core's own operand reads.  lda x cols floats of storage, lda = rows rounded up to a
 * multiple of 8; column c holds lda bfloat16 of plane 0, bf16(x - tf32(x)), then lda bfloat16
 * of plane 1, bf16(x) (the first `rows` of each in use).  An aux handle is an ordinary cudamat
 * of lda x cols. */
int split_bf16(cudamat* x, cudamat* aux);

/* The same storage in SCALED HALF-PRECISION form: with xs = x * 2^e (e = *exp_dev + exp_const;
 * exp_dev a 1 x 1 device matrix or NULL), plane 1 = hi = fp16(xs), plane 0 = lo = fp16(xs - hi).
 *   a . b * 2^(ea + eb) ~= hi(a).lo(b) + lo(a).hi(b) + hi(a).hi(b)      (B200_PART_F16HI / _F16LO)
 * is three half-precision products, no TF32 term and no fp32 operand read, below 2^-21 of
 * |a||b| per term; the caller names the exponent sum in b200_fused_gemm and the kernel divides
 * it out.  e must keep the largest |xs| inside the fp16 range (65504). */
int split_f16(cudamat* x, cudamat* aux, cudamat* exp_dev, int exp_const);

/* One term of a fused product: op(a) is M x k, op(b) is k x N (handles carry is_trans).
 * Both parts of a term are fp32-wide (X, LO32) or both bfloat16 (LO16, B16).  a_aux / b_aux:
 * NULL, or the aux matrix of a / b, from which the bfloat16 parts are then read. */
typedef struct b200_pass {
  cudamat* a;
  cudamat* b;
  int negate;
  int a_part, b_part;
  cudamat* a_aux;
  cudamat* b_aux;
  /* row windows of the stored matrices (0, 0 = all rows; offsets multiples of 8): a_rows > 0 restricts
   * a (not transposed) to rows [a_row0, a_row0 + a_rows), a panel of the output's rows; b_rows > 0
   * restricts b (transposed) likewise, a panel of the output's columns */
  int a_row0, a_rows, b_row0, b_rows;
} b200_pass;

/* out = act(alpha * sum_p (+/-) op(a_p).op(b_p) + beta * out + bias (x) col_scale).
 * Replaces dot / add_dot / mult / add_col_vec (or add_dot(b, NN)) / apply_sigmoid /
 * sample_bernoulli of deepnet/dbm.py:88-105 and logistic_layer.py:11-15, and the
 * dot + add_dot(mult=-1) pair of deepnet/edge.py:236,242, by one kernel. */
typedef struct b200_fused_gemm {
  int npass;             /* 1..8 */
  b200_pass pass[8];
  float alpha, beta;
  cudamat* bias;         /* M x 1 or NULL */
  cudamat* col_scale;    /* 1 x N or NULL: bias of column n is bias[m] * col_scale[n] */
  int activation;        /* 0 identity, 1 logistic */
  cudamat* out;          /* M x N or NULL */
  cudamat* out_aux;      /* aux matrix of the result, or NULL */
  cudamat* sample;       /* Bernoulli(result): consumes one sampling call, or NULL */
  cudamat* sample_aux;   /* aux matrix of the draw (plane 1 only: a 0/1 value has no low part), or NULL */
  cudamat* scale_exp;    /* scaled half-precision operands: the terms carry 2^(*scale_exp + scale_exp_const), */
  int scale_exp_const;   /*   divided out by the kernel (scale_exp: 1 x 1 device matrix or NULL) */
  int aux_f16;           /* != 0: out_aux / sample_aux in scaled half-precision form ... */
  int aux_exp;           /*   ... with this exponent */
} b200_fused_gemm;
int fused_gemm(rnd_struct* rnd_state, b200_fused_gemm* f);

/* lo = x - tf32(x); hi (may be NULL) = tf32(x): the split the kernels apply on the fly. */
int split_tf32(cudamat* x, cudamat* hi, cudamat* lo);

/* deepnet/dbm.py:242,254 + deepnet/parameter.py:80-106 as one pass over the parameter:
 * grad += -inv_batch * suff; delta = momentum*delta + l2*w + l1*sign(w) + grad;
 * w -= eps*delta; grad = 0; w_aux = aux matrix of the new w: its bfloat16 parts, or with w_scale
 * (1 x 4 device matrix {exponent, -, max |w| bits, -}, kept by this call: the exponent always
 * fits the new w) its scaled half-precision form.  grad, w_aux, w_scale may be NULL. */
int momentum_update(cudamat* w, cudamat* delta, cudamat* grad, cudamat* suff, cudamat* w_aux, cudamat* w_scale,
                    float inv_batch, float momentum, float eps, float l2, float l1);
/* The same on columns [col0, col0 + ncols) of the parameter: statistics that arrive panel by panel
 * (each after its own all-reduce) are applied as they arrive; the exponent check of the scaled
 * half-precision form runs with the panel that ends at the last column. */
int momentum_update_columns(cudamat* w, cudamat* delta, cudamat* grad, cudamat* suff, cudamat* w_aux, cudamat* w_scale,
                            int col0, int ncols, float inv_batch, float momentum, float eps, float l2, float l1);

/* Has no counterpart in the reference.  add_sum_by_axis for callers that must never reach
 * cudaMalloc (a host that gave the whole device to its own memory pool, or a loop that cannot
 * afford the device-wide synchronisation an allocation may bring): the partial sums live in a
 * fixed 128 KiB array inside the module (32768 floats, held on every GPU that loads the
 * library until exit) instead of the library's allocate-on-demand workspace.  A matrix whose
 * partial sums (splits x rows floats) do not fit is refused with ERROR_UNSUPPORTED.  The first
 * call on a device looks the array's address up: make it before any stream capture.  Calls
 * share the array, so calls that overlap on the GPU race; issue them in order on one stream. */
int add_sum_by_axis_noalloc(cudamat* mat, cudamat* target, int axis, float mult);

/* target = row sums of a minus row sums of b in one launch: a layer's bias statistics, positive minus
 * negative phase (deepnet/layer.py:202-213: sum(axis=1), then add_sums(axis=1, mult=-1)). */
int row_sum_diff(cudamat* a, cudamat* b, cudamat* target);

/* target[:, c] = counts over ndraws Gumbel-max draws from the softmax with energies energy[:, c]:
 * the loop of deepnet/ais.py:16-30 (perturb_energy_for_softmax_sampling + choose_max_and_accumulate
 * per draw) in one kernel on the same random stream (ndraws sampling calls). */
int sample_energy_softmax(rnd_struct* rnd_state, cudamat* energy, cudamat* target, int ndraws);

/* state[:, j] = softmax(pre[:, j] + bias); sample[:, j] = one categorical draw from it as a one-hot
 * column: deepnet/softmax_layer.py:11-16 (apply_softmax, perturb_prob_for_softmax_sampling,
 * choose_max(axis=0)) in one kernel on the same random stream.  bias and sample may be null
 * (no sampling call is consumed without sample). */
int softmax_sample(rnd_struct* rnd_state, cudamat* pre, cudamat* bias, cudamat* state, cudamat* sample);

/* target[:, j] = scale[j] * softmax(mat[:, j]): the six calls of
 * deepnet/replicated_softmax_layer.py:12-21 (max, add_row_mult, exp, sum, divide, mult_by_row). */
int softmax_scaled(cudamat* mat, cudamat* scale, cudamat* target);

/* target[:, i] = word counts of int(nn[i]) (at most max_draws) exponential-race draws from the
 * distribution proportional to probs[:, i]: the per-document loop of
 * deepnet/replicated_softmax_layer.py:43-60 as one kernel.  One sampling call per document. */
int sample_multinomial(rnd_struct* rnd_state, cudamat* probs, cudamat* nn, cudamat* target, int max_draws);

/* acc[0] += sum((a - b)^2), kept on the device (subtract + euclid_norm()**2 of
 * deepnet/logistic_layer.py:48-52 without the host round trip). */
int add_sq_diff(cudamat* a, cudamat* b, cudamat* acc);

/* Library control. */
int b200_device_count(void);
int b200_set_stream(void* cuda_stream);   /* NULL restores the library's own stream */
void* b200_get_stream(void);
void* b200_event_create(void);            /* CUDA events recorded on the library stream */
int b200_event_record(void* ev);
float b200_event_elapsed_ms(void* start, void* end);  /* blocks until `end`; < 0 on error */
void b200_event_destroy(void* ev);
int b200_read_status(void);               /* non-zero: a kernel's bounded wait gave up (blocks, clears) */
/* Iterations a device-side wait may spin before its kernel gives up (default 2^24, one to two
 * seconds; 0 restores the default).  No counterpart in the reference. */
int b200_set_wait_limit(unsigned int iterations);
/* Programmatic dependent launch of the step's kernels (each is scheduled while its predecessor on
 * the stream drains and touches global memory only after that one has completed): on by default;
 * 0 turns it off (so does B200_DEPENDENT_LAUNCH=0).  No counterpart in the reference. */
int b200_set_dependent_launch(int on);
/* SMs the library's kernels size their grids for (0 = all): leaves room for an all-reduce that runs
 * beside the persistent tensor-core kernel.  No counterpart in the reference. */
int b200_set_sm_limit(int sms);
int b200_sm_count(void);                  /* SMs in force (the device's, or the limit) */
/* Test hook, host side only: the next tensor-core product expects extra_bytes more per stage than
 * its copies deliver, so one of its bounded waits must run out (status word set, kernel returns).
 * No counterpart in the reference. */
int b200_test_inject_stage_bytes(int extra_bytes);
int b200_set_gemm_path(int path);         /* 0 auto, 1 tensor cores only, 2 CUDA cores only */
int b200_set_dot_precision(int mode);     /* 0 fp32-grade split TF32 (default), 1 one TF32 pass */
/* Split-K of the tensor-core product: 0 (default) = cut the inner dimension into work items when the
 * output tiles alone would leave most SMs idle, 1 = never, n > 1 = always n splits.  No counterpart
 * in the reference. */
int b200_set_split_k(int mode);
int set_rng_column_offset(int col0);      /* first global minibatch column of this process */
void* b200_host_alloc(size_t bytes);      /* pinned host memory */
void b200_host_free(void* p);
int copy_from_host_ptr(cudamat* mat, const float* src, size_t bytes);  /* async H2D into mat */
int b200_prefetch(cudamat* mat, const float* src, size_t bytes);       /* H2D on a second (copy) stream */
int b200_prefetch_wait(void);             /* library stream waits for the copies started so far */
int b200_prefetch_fence(void);            /* later copies wait for work already enqueued */
/* Device-to-host read-back on a stream of its own, ordered after the work enqueued so far (slot 0..7,
 * one pending read-back each); dst is pinned host memory; b200_readback_wait blocks until it has landed. */
int b200_readback_begin(cudamat* src, void* dst, size_t bytes, int slot);
int b200_readback_wait(int slot);

/* Data parallelism over NCCL: one process per GPU. */
int dp_unique_id(char* out128);
int dp_init(const char* id128, int nranks, int rank);
int dp_world_size(void);
int dp_rank(void);
int dp_allreduce(cudamat* mat);           /* in-place sum over ranks, on the library stream */
int dp_check(void);
int dp_destroy(void);
int dp_abort(void);
/* The all-reduce on a side stream, beside the kernels that follow on the library stream: begin waits
 * for what is enqueued so far and starts it (slot 0..7, one pending all-reduce each); end makes the
 * library stream wait for it. */
/* The exchange and the update of a data-parallel step over peer memory, without NCCL: rank r owns the
 * columns [r H/G, (r+1) H/G) of W.  The statistics product itself (the fused_gemm whose result is the
 * first rows(W) x cols(W) floats of `pack`) delivers every column panel to its owner: its epilogue
 * stores the tiles of panel q into rank q's receive buffer with plain stores over NVLink while the
 * product runs (when H/G is not a multiple of 256 the owners fetch the panels with plain loads
 * instead).  Once every rank's statistics are complete the owner adds the G partial statistics of its
 * columns, applies the momentum / decay update to its shard and stores the new shard and its 16-bit
 * planes into every rank's copy of W.
 * Bring-up: every rank exports {pack, W, W_aux, flags, receive buffer} (dp_peer_export,
 * dp_peer_export_flags, dp_peer_export_recv(elements of W, ...); dp_peer_handle_bytes() bytes each), the
 * ranks exchange them by any host channel and call dp_peer_setup with all of them in rank order; then
 * dp_peer_update once per update on every rank (pack = [W statistics | b_v | b_h] of this rank, b / db
 * the packed biases and their history).  Waits are bounded (b200_set_wait_limit; b200_read_status
 * tells).  H must be a multiple of G. */
int dp_peer_handle_bytes(void);
int dp_peer_export(cudamat* m, char* handle_out);
int dp_peer_export_flags(char* handle_out);
int dp_peer_export_recv(long floats, char* handle_out);
int dp_peer_setup(int nranks, int rank, const char* handles, cudamat* pack, cudamat* w, cudamat* w_aux);
int dp_peer_update(cudamat* w, cudamat* delta, cudamat* w_aux, cudamat* w_scale, cudamat* pack, cudamat* b, cudamat* db,
                   float inv_batch, float mom_b, float eps_b, float mom_w, float eps_w, float l2, float l1);
int dp_peer_close(void);
int dp_peer_mode(void);                  /* 0 not set up, 1 owners fetch the panels, 2 the statistics product delivers them */
int dp_allreduce_begin(cudamat* mat, int slot);
int dp_allreduce_end(int slot);
/* Waits (at most timeout_ms) for the work enqueued on the library stream, collectives included; on
 * time-out or an asynchronous NCCL error aborts the communicator and returns ERROR_NCCL. */
int dp_wait(int timeout_ms);

/* ---- a recorded training step: no counterpart in the reference ---------------------------- */
/* The update of deepnet/dbm.py:268-274 is 10-60 library calls per minibatch; at the small
 * configurations a call from the host language costs more than its kernel.  The caller records
 * the calls once as an array of b200_op and replays them with one call.  kind selects the entry
 * point (0 fused_gemm, 1 sum_by_axis, 2 add_sum_by_axis, 3 row_sum_diff, 4 add_sq_diff,
 * 5 momentum_update, 6 split_f16, 7 split_bf16, 8 dp_allreduce, 9 softmax_scaled, 10 sample_multinomial,
 * 11 div_by_row_vec, 12 add_scalar, 13 assign_scalar, 14 copy_on_device, 15 sample_bernoulli,
 * 16 softmax_sample, 17 momentum_update_columns, 18 dp_allreduce_begin, 19 dp_allreduce_end,
 * 20 b200_set_sm_limit, 21 dp_peer_update); m[], i0.., f0.. are its arguments in declaration order (matrices, then integers,
 * then floats; gemm for kind 0).  Stops at the first failure: returns its code, *failed_at its index. */
struct b200_fused_gemm;
typedef struct b200_op {
  int kind;
  int i0, i1, i2;
  float f0, f1, f2, f3, f4, f5, f6, f7;
  cudamat* m[8];
  struct b200_fused_gemm* gemm;
} b200_op;
int b200_run_program(rnd_struct* rnd_state, b200_op* ops, int n, int* failed_at);

#ifdef __cplusplus
}
#endif
#endif /* B200MAT_H_ */
