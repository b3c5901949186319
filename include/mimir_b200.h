/*
 * mimir_b200.h — C ABI of the B200 (sm_100a) forward-inference backend for Mímir.
 *
 * Everything here is plain C: pointers, sizes and ints.  No C++ or torch type crosses the
 * boundary.  Every function returns a MimirB200Status; on a non-zero status
 * mimir_b200_last_error() gives a thread-local message.  The library never throws and never
 * falls back to the CPU: an op it cannot run returns MIMIR_B200_E_UNSUPPORTED.
 *
 * Three groups of entry points:
 *   1. life cycle and device-memory budget  (mirror of MemoryGuard's verbs)
 *   2. per-op calls with HOST pointers      (mirror of ComputeEngine::linearForward,
 *      one call per `case LayerType::X` of Model::forwardPassView)
 *   3. whole-graph calls                    (mirror of Model::forwardPassView itself: the
 *      layer list is translated once, weights are uploaded once, activations stay in HBM)
 *
 * Layout conventions are the reference's: every activation is a flat row-major fp32 vector for
 * one sample (images CHW, sequences [seq, dim]); `batch` is a leading dimension added by this
 * backend and means "apply the reference op independently to each sample".
 */
#ifndef MIMIR_B200_H
#define MIMIR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MIMIR_B200_ABI_VERSION 3
#define MIMIR_B200_MAX_INPUTS 8
#define MIMIR_B200_MAX_DIMS 8
#define MIMIR_B200_MAX_SPLITS 16

typedef enum MimirB200Status {
  MIMIR_B200_OK = 0,
  MIMIR_B200_E_INVALID = 1,     /* bad argument / shape (reference: RUNTIME_CHECK -> throw, RuntimeAllocator.hpp:344-358) */
  MIMIR_B200_E_UNSUPPORTED = 2, /* layer type or shape this backend does not run; there is no CPU fallback */
  MIMIR_B200_E_OOM_BUDGET = 3,  /* device budget refused (reference: MemoryGuard::requestAllocation false, MemoryGuard.hpp:75-130) */
  MIMIR_B200_E_CUDA = 4,        /* a CUDA call failed; message carries cudaGetErrorString */
  MIMIR_B200_E_TIMEOUT = 5,     /* a bounded device-side wait gave up (kernel returned an error word) */
  MIMIR_B200_E_NOT_INIT = 6
} MimirB200Status;

/* GEMM operand precision.  All modes accumulate in fp32 in tensor memory.  Operands travel as 16-bit planes: IEEE half
 * by default (weights through a per-layer power-of-two scale), bfloat16 with MIMIR_B200_PLANES=bf16; the names date
 * from the bfloat16 planes and describe the number of MMAs per product.
 *   BF16X2 : both operands split into hi + lo planes, three MMAs (hi*hi + lo*hi + hi*lo) — the default for fp32
 *            graphs (within rel 1e-3 / abs 1e-4 of the CPU path).
 *   BF16W  : weights in one plane (exact when the checkpoint was pre-rounded to bf16), activations split hi + lo,
 *            two MMAs.
 *   BF16   : one plane per operand, one MMA (fastest; not within the fp32 tolerance: it is checked against the
 *            reference's arithmetic with the same operand rounding applied, not against the fp32 gate). */
typedef enum MimirB200Precision {
  MIMIR_B200_PREC_BF16X2 = 0,
  MIMIR_B200_PREC_BF16W = 1,
  MIMIR_B200_PREC_BF16 = 2
} MimirB200Precision;

/* Element-wise ops of mimir_b200_eltwise (reference: LayerOps.hpp:142-230, 556-623). */
typedef enum MimirB200Eltwise {
  MIMIR_B200_ELT_ADD = 0,      /* add_forward incl. scalar and `i % small_n` broadcast */
  MIMIR_B200_ELT_MULTIPLY = 1, /* multiply_forward (equal sizes only) */
  MIMIR_B200_ELT_GELU = 2,     /* tanh form, c = sqrt(2/3.14159265359f) */
  MIMIR_B200_ELT_SILU = 3,
  MIMIR_B200_ELT_RELU = 4,
  MIMIR_B200_ELT_TANH = 5,
  MIMIR_B200_ELT_SIGMOID = 6,
  MIMIR_B200_ELT_LEAKY_RELU = 7,   /* x > 0 ? x : alpha x (LayerOpsExt.hpp:29-39) */
  MIMIR_B200_ELT_SOFTPLUS = 8,     /* x > 20 ? x : log(1 + exp x) (LayerOpsExt.hpp:59-68) */
  MIMIR_B200_ELT_MISH = 9,         /* x tanh(softplus x) (LayerOpsExt.hpp:44-54) */
  MIMIR_B200_ELT_HARD_SIGMOID = 10,/* clamp((x + 3) / 6, 0, 1) (LayerOpsExt.hpp:73-82) */
  MIMIR_B200_ELT_HARD_SWISH = 11,  /* x hard_sigmoid(x) (LayerOpsExt.hpp:87-99) */
  MIMIR_B200_ELT_SUBTRACT = 12,    /* equal sizes (LayerOpsExt.hpp:105-122) */
  MIMIR_B200_ELT_DIVIDE = 13,      /* equal sizes, |divisor| < 1e-8 replaced by +-1e-8 (LayerOpsExt.hpp:127-148) */
  MIMIR_B200_ELT_ELU = 14          /* x >= 0 ? x : alpha (exp x - 1) (Model::elu_inplace, Model.hpp:505-509; static family only) */
} MimirB200Eltwise;

/* ---------------------------------------------------------------------------------------------
 * 1. Life cycle and budget
 * ------------------------------------------------------------------------------------------ */

/* Brings up the context of CUDA device `device` (one context per device, kept in a table) and makes that
 * device current on the calling thread: the per-op calls and model_create of this thread then run on it.
 * Sets the HBM budget that arena plans and weight uploads are checked against (0 = keep a limit set earlier
 * through guard_set_limit, else 90 % of the device's total memory).  Idempotent and thread-safe; a process may
 * initialise several devices (one host thread per device, or mimir_b200_replicas_*).  Model handles remember
 * their device and switch to it themselves.  Replaces the engine construction in Model::Model()
 * (Model.cpp:690-698, 753-878) and MemoryGuard::setLimit (MemoryGuard.hpp:47-60). */
int mimir_b200_init(int device, size_t hbm_budget_bytes);
/* Selection inside Mimir by environment, default off, with the conventions of the reference's accelerator switches
 * (env_flag_true / env_int, Model.cpp:704-722; MIMIR_VULKAN_LINEAR at Model.cpp:5110-5112):
 *   MIMIR_B200               any non-empty value other than "0" selects this backend
 *   MIMIR_B200_DEVICE        CUDA device index (default 0)
 *   MIMIR_B200_HBM_BUDGET_MB budget of the guard in MiB (unset or 0: 90 % of the device's memory)
 * env_selection only parses; init_from_env also calls mimir_b200_init when selected (*enabled = 1) and touches nothing
 * otherwise (*enabled = 0, status OK).  When selected and no usable GPU is there the status is the init error: there is
 * no silent CPU fallback inside the backend. */
int mimir_b200_env_selection(int* enabled, int* device, size_t* hbm_budget_bytes);
int mimir_b200_init_from_env(int* enabled);
/* The device the calling thread's per-op calls run on. */
int mimir_b200_current_device(int* device);
/* Releases every model handle on every device.  Replaces the engine teardown in Model::~Model()
 * (Model.cpp:726-741). */
int mimir_b200_shutdown(void);
const char* mimir_b200_last_error(void);
int mimir_b200_abi_version(void);

/* MemoryGuard verbs against the HBM budget (MemoryGuard.hpp:47-60 setLimit, 75-130
 * requestAllocation, 132-150 releaseAllocation, getCurrentUsage/getPeakUsage/getLimit). */
int mimir_b200_guard_set_limit(size_t bytes);
int mimir_b200_guard_request(size_t bytes, const char* tag); /* OK or E_OOM_BUDGET */
int mimir_b200_guard_release(size_t bytes);
int mimir_b200_guard_stats(size_t* limit, size_t* current, size_t* peak);
/* MemoryGuard::blockAllocations / freezeAllocations (MemoryGuard.hpp:37-72): while set, every request - the
 * explicit guard_request and the library's own arena, weight and workspace allocations - is refused with
 * E_OOM_BUDGET (blocked is checked before frozen, frozen before the limit, MemoryGuard.hpp:75-112); releases
 * stay possible.  guard_reset is MemoryGuard::reset (MemoryGuard.hpp:181-186): usage and peak back to zero.
 * guard_state reads both switches and the refused-attempt counters.  All guard verbs act on the calling
 * thread's current device and work before mimir_b200_init (host logic only). */
int mimir_b200_guard_block(int block);
int mimir_b200_guard_freeze(int freeze);
int mimir_b200_guard_reset(void);
int mimir_b200_guard_state(int* blocked, int* frozen, size_t* blocked_attempts, size_t* frozen_attempts);

/* RuntimeAllocator on the device (RuntimeAllocator.hpp:176-310): guarded device buffers with the reference's verbs,
 * for a host that keeps tensors of its own in HBM beside the planner's arena (the `mimir_b200_dev_*` calls and
 * `mimir_b200_model_forward_device` take such pointers).  Every verb acts on the calling thread's current device.
 *   tensor_alloc        allocate_tensor (RuntimeAllocator.hpp:191-225): fp32 tensor of `rank` extents, zero-filled like the
 *                       reference's std::vector<float>(numel, 0); refused with E_OOM_BUDGET when the local cap
 *                       (allocator_set_local_cap; the reference's max_ram_mb, 0 = none, which is the default here) or the
 *                       guard says no.  A non-positive extent or an element count that overflows is E_INVALID.
 *   buffer_alloc        allocate_buffer (RuntimeAllocator.hpp:228-260): raw bytes, zero-filled.
 *   buffer_free         what ~TensorHandle / ~BufferHandle do: frees and releases the bytes at the guard.  A pointer the
 *                       allocator does not own is E_INVALID.
 *   scratchpad_get      get_scratchpad (RuntimeAllocator.hpp:264-276): the pooled buffer of that tag when it holds at least
 *                       min_bytes, else a new buffer (a pooled one that is too small stays pooled, as in the reference).
 *   scratchpad_return   return_scratchpad (RuntimeAllocator.hpp:279-282): back to the pool under the tag it was allocated
 *                       with; the pool keeps one buffer per tag, a second one of the same tag is freed.
 *   allocator_stats     get_total_allocated / get_num_allocations (cumulative, reset by allocator_reset_stats) and the
 *                       guard's peak / current (get_peak_usage / get_current_usage).
 *   allocator_check_no_leaks   check_no_leaks (RuntimeAllocator.hpp:299-304): 1 when less than 10 MB are in use.
 * mimir_b200_shutdown frees what is still pooled or live. */
int mimir_b200_tensor_alloc(const int* shape, int rank, const char* name_or_null, float** device_ptr, size_t* bytes_or_null);
int mimir_b200_buffer_alloc(size_t bytes, const char* tag_or_null, void** device_ptr);
int mimir_b200_buffer_free(void* device_ptr);
int mimir_b200_scratchpad_get(size_t min_bytes, const char* tag_or_null, void** device_ptr, size_t* bytes_or_null);
int mimir_b200_scratchpad_return(void* device_ptr);
int mimir_b200_allocator_set_local_cap(size_t bytes);
int mimir_b200_allocator_stats(size_t* total_allocated, size_t* num_allocations, size_t* peak, size_t* current);
int mimir_b200_allocator_reset_stats(void);
int mimir_b200_allocator_check_no_leaks(int* ok);

/* ---------------------------------------------------------------------------------------------
 * 2. Per-op entry points, HOST pointers, synchronous (copy in, run, copy out).
 *    Drop-in for the Vulkan/OpenCL hook `bool ComputeEngine::linearForward(const float* input,
 *    const float* weights, const float* bias_or_null, float* output, int batch, int in_f,
 *    int out_f)` (VulkanCompute.hpp:209-210, OpenCLCompute.hpp:114-122), one per switch case.
 * ------------------------------------------------------------------------------------------ */

/* y[t,o] = sum_i W[o,i] x[t,i] (+ b[o]).  Replaces LayerOps::linear_forward (LayerOps.hpp:24-111)
 * and the accelerator call sites Model.cpp:5136-5144, 5184-5192.  `batch` = rows. */
int mimir_b200_linear_forward(const float* input, const float* weights, const float* bias_or_null,
                              float* output, int batch, int in_f, int out_f);
/* Same with the precision mode and a fused activation (MIMIR_B200_ELT_GELU/SILU/RELU or -1). */
int mimir_b200_linear_forward_ex(const float* input, const float* weights, const float* bias_or_null,
                                 float* output, int batch, int in_f, int out_f, int precision,
                                 int activation);
/* C[M,N] = A[M,K] B[K,N], row-major.  Replaces LayerOps::matmul_forward (LayerOps.hpp:692-724) /
 * HardwareOpt::matmul_fma_saturated (HardwareOpt.hpp:95-149). */
int mimir_b200_matmul(const float* A, const float* B, float* C, int M, int K, int N);
/* Self / multi-head attention on `batch` samples of [seq, embed].  Weight block = Wqkv[E][3E]
 * then Wout[E][E], no biases.  Replaces LayerOps::self_attention_forward (LayerOps.hpp:1004-1097)
 * as dispatched at Model.cpp:5904-5933. */
int mimir_b200_attention(const float* x, const float* wqkv_wout, float* y, int batch, int seq,
                         int embed, int heads, int causal);
/* NCHW x OIHW, square kernel, no bias, optional ReLU.  Replaces the inline Conv2d case
 * (Model.cpp:4897-5089). */
int mimir_b200_conv2d(const float* x, const float* w, float* y, int batch, int ic, int oc, int h,
                      int wd, int k, int stride, int pad, int relu);
/* `rows` independent groups of n; gamma/beta may be NULL.  Replaces LayerOps::layernorm_forward
 * (LayerOps.hpp:264-319). */
int mimir_b200_layernorm(const float* x, const float* gamma, const float* beta, float* y,
                         long long rows, int n, float eps);
/* One RMS over each sample's whole vector of n; gamma applied to flat indices < n_gamma.
 * Replaces LayerOpsExt::rms_norm_forward (LayerOpsExt.hpp:345-378). */
int mimir_b200_rmsnorm(const float* x, const float* gamma, long long n_gamma, float* y, int batch,
                       long long n, float eps);
/* CHW samples, G contiguous channel groups; act = -1 or MIMIR_B200_ELT_SILU (fused).
 * Replaces LayerOps::groupnorm_forward (LayerOps.hpp:488-550). */
int mimir_b200_groupnorm(const float* x, const float* gamma, const float* beta, float* y, int batch,
                         int channels, int h, int w, int groups, float eps, int act);
/* Softmax / log-softmax over each sample's whole vector (axis ignored, as in the reference).
 * Replaces LayerOps::softmax_forward (LayerOps.hpp:325-361). */
int mimir_b200_softmax(const float* x, float* y, int batch, long long n, int log_softmax);
/* Unary ops read `a` only; ADD/MULTIPLY read `b` of nb elements per sample
 * (nb == n, 1, or a divisor of n).  Replaces LayerOps.hpp:142-230, 556-623. */
int mimir_b200_eltwise(int op, const float* a, const float* b, float* y, int batch, long long n,
                       long long nb);
/* Same with the slope of LeakyReLU (ignored by the other ops). */
int mimir_b200_eltwise_alpha(int op, const float* a, const float* b, float* y, int batch, long long n,
                             long long nb, float alpha);
/* Row gather; ids given as floats are rounded like llround; id == padding_idx (when >= 0) or out
 * of range gives a zero row.  Replaces the Embedding case (Model.cpp:5301-5334; int ids:
 * Model.cpp:1152-1205).  Exactly one of ids_f32 / ids_i32 is non-NULL. */
int mimir_b200_embedding(const float* ids_f32, const int32_t* ids_i32, const float* table, float* y,
                         long long n_ids, int vocab, int dim, int padding_idx);
/* Nearest-neighbour upsample of CHW samples by integer factors.  Replaces
 * LayerOps::upsample_nearest_forward (LayerOps.hpp:802-827) as called at Model.cpp:6002-6017. */
int mimir_b200_upsample_nearest(const float* x, float* y, int batch, int channels, int in_h,
                                int in_w, int scale_h, int scale_w);
/* General permutation of a tensor of `ndim` dims (per sample).  Replaces
 * LayerOps::permute_forward (LayerOps.hpp:880-945). */
int mimir_b200_permute(const float* x, float* y, int batch, int ndim, const int* shape,
                       const int* dims);
/* mean over seq of [seq, dim] (Model.cpp:5571-5589) and mean over HxW per channel
 * (LayerOps.hpp:459-482). */
int mimir_b200_token_mean_pool(const float* x, float* y, int batch, int seq, int dim);
int mimir_b200_global_avgpool(const float* x, float* y, int batch, int channels, int h, int w);

/* ---- the remaining cases of the layer switch ("next" rows: cross attention and the long tail) ---- */

/* Cross attention on `batch` pairs of query [q_len, embed] and key/value [kv_len, embed] inputs.
 * Weight block = Wq[E][E], Wkv[E][2E] (K | V halves), Wout[E][E], input-major, no biases.  Replaces
 * LayerOps::cross_attention_forward (LayerOps.hpp:1116-1216) as dispatched at Model.cpp:5935-5996. */
int mimir_b200_cross_attention(const float* query, const float* key_value, const float* wq_wkv_wout,
                               float* y, int batch, int q_len, int kv_len, int embed, int heads,
                               int causal);
/* One filter per channel, weights [C][k][k] then bias[C] when `bias` is non-NULL.  Replaces
 * LayerOpsExt::depthwise_conv2d_forward (LayerOpsExt.hpp:442-497). */
int mimir_b200_depthwise_conv2d(const float* x, const float* w, const float* bias, float* y, int batch,
                                int channels, int h, int wd, int k, int stride, int pad);
/* x [ic][len], weights [oc][ic][k] (+ bias[oc]).  Replaces LayerOpsExt::conv1d_forward
 * (LayerOpsExt.hpp:388-437). */
int mimir_b200_conv1d(const float* x, const float* w, const float* bias, float* y, int batch, int ic,
                      int oc, int len, int k, int stride, int pad);
/* The ConvTranspose2d branch of the Conv2d case (Model.cpp:4946-4953, 5047-5079): output size
 * (h-1)*stride - 2*pad + k, taps gathered with the forward-convolution formula, no bias. */
int mimir_b200_conv_transpose2d(const float* x, const float* w, float* y, int batch, int ic, int oc,
                                int h, int wd, int k, int stride, int pad, int relu);
/* is_max != 0: MaxPool2d (Model.cpp:5508-5559); else AvgPool2d over the in-bounds taps
 * (LayerOps.hpp:404-453). */
int mimir_b200_pool2d(int is_max, const float* x, float* y, int batch, int channels, int h, int wd,
                      int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w);
/* mode 0 zero, 1 reflection, 2 replication (LayerOpsExt.hpp:582-690). */
int mimir_b200_pad2d(int mode, const float* x, float* y, int batch, int channels, int h, int wd,
                     int pad_h, int pad_w);
/* [C r^2, H, W] -> [C, H r, W r] (LayerOpsExt.hpp:749-795). */
int mimir_b200_pixel_shuffle(const float* x, float* y, int batch, int in_channels, int h, int wd, int r);
/* 2x bilinear upsample; half_pixel = 0: LayerOps::upsample_bilinear_forward (LayerOps.hpp:833-874),
 * 1: the variant dispatched for UpsampleBicubic (LayerOpsExt.hpp:695-744). */
int mimir_b200_upsample_bilinear(const float* x, float* y, int batch, int channels, int h, int wd,
                                 int out_h, int out_w, int half_pixel);
/* C[b] = A[b] (M x K) . B[b] (K x N) for nb matrices.  Replaces the BatchMatMul / MatMul cases
 * (Model.cpp:5847-5898). */
int mimir_b200_batch_matmul(const float* A, const float* B, float* C, long long nb, int M, int K, int N);
/* Inference BatchNorm of the reference: statistics over each sample's WHOLE vector, then
 * y[i] *= w[i] for i < n_w; no shift (Model.cpp:5387-5421). */
int mimir_b200_batchnorm_inference(const float* x, const float* w, long long n_w, float* y, int batch,
                                   long long n, float eps);
/* BatchNorm with running statistics, the inference branch of Model::computeBatchNorm / Normalization::batch_norm
 * (Model.cpp:4066-4148, Layers.hpp:932-970): x is [batch][channels][spatial];
 * y = (x - mean[c]) * (1 / sqrt(var[c] + eps)) * gamma[c] + beta[c]. */
int mimir_b200_batchnorm_running(const float* x, const float* gamma, const float* beta, const float* running_mean,
                                 const float* running_var, float* y, int batch, int channels, long long spatial,
                                 float eps);
/* BatchNorm with batch statistics, the training branch of Model::computeBatchNorm / Normalization::batch_norm
 * (Layers.hpp:932-970): per channel the mean and the biased variance over the batch and the spatial positions, then
 * y = (x - mean) * (1 / sqrt(var + eps)) * gamma[c] + beta[c].  The running statistics are neither read nor updated
 * (the reference does not update them either). */
int mimir_b200_batchnorm_batchstats(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels,
                                    long long spatial, float eps);
/* Conv::conv2d behind Model::computeConv2D (Layers.hpp:611-722, Model.cpp:3880-3888): CHW input, OIHW weights, optional
 * bias (NULL: none) added after the sum, stride, zero padding and dilation; out = (in + 2p - d (k - 1) - 1) / s + 1.
 * fp32 FMAs over (ic, kh, kw) ascending. */
int mimir_b200_conv2d_dilated(const float* x, const float* w, const float* bias, float* y, int batch, int in_c, int out_c,
                              int in_h, int in_w, int kernel, int stride, int padding, int dilation);
/* Conv::conv_transpose2d behind Model::computeConvTranspose2D (Layers.hpp:775-818, Model.cpp:4214-4221): the scatter form
 * y[oc][ih s + kh - p][iw s + kw - p] += x[ic][ih][iw] * w[oc][ic][kh][kw] on top of the bias; out = (in - 1) s - 2p + k.
 * Computed as a gather that visits the contributions of one output in the reference's order (ic, ih, iw ascending). */
int mimir_b200_conv_transpose2d_scatter(const float* x, const float* w, const float* bias, float* y, int batch, int in_c,
                                        int out_c, int in_h, int in_w, int kernel, int stride, int padding);
/* Attention core on separate, already projected Q / K / V, each [batch*seq][d_model] with the heads side by side
 * (Model::computeAttention, scalar branch, Model.cpp:4223-4289): softmax(Q_h K_h^T / sqrt(head_dim)) V_h per head,
 * no mask, no projections. */
int mimir_b200_attention_qkv(const float* q, const float* k, const float* v, float* y, int batch, int seq,
                             int d_model, int num_heads);

/* ---------------------------------------------------------------------------------------------
 * 3. Whole-graph entry points (activations stay on the device between layers)
 * ------------------------------------------------------------------------------------------ */

/* POD mirror of the `struct Layer` fields the forward ops read (Layers.hpp:86-309).  `type` is
 * the reference's normalised type string ("Linear", "Conv2d", "MultiHeadAttention", ...,
 * LayerTypes.hpp:13-120).  Strings are copied by model_create.  Zero / negative values keep the
 * reference's "unset" meaning (e.g. in_features == 0 => whole input). */
typedef struct MimirLayerDesc {
  const char* name;
  const char* type;
  const char* inputs[MIMIR_B200_MAX_INPUTS]; /* n_inputs == 0 => {"x"} (Model.cpp:4802) */
  int32_t n_inputs;
  const char* output;                        /* NULL or "" => "x" (Model.cpp:6655) */
  uint64_t params_count;
  int32_t in_features, out_features, in_channels, out_channels;
  int32_t input_height, input_width;
  int32_t kernel, stride, padding;           /* already resolved: get_kernel_h / get_stride_h / get_pad_h (Layers.hpp:250-257) */
  float eps;
  int32_t num_groups, affine, use_bias;
  int32_t vocab_size, embed_dim, padding_idx;
  int32_t num_heads, seq_len, causal;
  int32_t out_h, out_w, scale_h, scale_w;    /* UpsampleNearest reads out_h/out_w as the INPUT size (Model.cpp:6008-6009) */
  int32_t activation;                        /* != 0 => ReLU after Conv2d (Model.cpp:5081-5086) */
  int32_t n_dims;
  int32_t shape[MIMIR_B200_MAX_DIMS];        /* Permute */
  int32_t permute_dims[MIMIR_B200_MAX_DIMS];
  /* --- ABI version 2: fields read by the remaining switch cases ------------------------------ */
  int32_t head_dim;                          /* CrossAttention: embed_dim <= 0 => head_dim * num_heads (Model.cpp:5954-5957) */
  float leaky_relu_alpha;                    /* LeakyReLU: <= 0 => 0.01 (Model.cpp:5453) */
  int32_t kernel_w, stride_w, padding_w;     /* resolved get_kernel_w / get_stride_w / get_pad_w (AvgPool2d, LayerOps.hpp:408-413) */
  int32_t raw_kernel_h, raw_stride_h, raw_pad_h, raw_pad_w; /* the RAW Layer fields kernel_h / stride_h / pad_h / pad_w:
                                                DepthwiseConv2d, Conv1d and the pads read these, not the get_* helpers
                                                (LayerOpsExt.hpp:449-451, 395-398, 589-592) */
  int32_t n_splits;                          /* Split: number of entries of split_sizes (Model.cpp:5802-5815) */
  int32_t split_sizes[MIMIR_B200_MAX_SPLITS];
  int32_t num_chunks;                        /* Chunk (Model.cpp:5817-5832) */
  /* --- ABI version 3: PatchEmbed and Bilinear ------------------------------------------------- */
  int32_t seq_text, num_patches, patch_dim;  /* PatchEmbed: text tokens (without the time token), patches, flattened patch size
                                                (Layers.hpp:181-183, Model.cpp:5203-5243) */
  int32_t target_dim0;                       /* Bilinear: target_shape[0] (0 when the vector is empty), the output width used
                                                when embed_dim <= 0 (Model.cpp:5256) */
} MimirLayerDesc;

typedef struct MimirNamedInput {
  const char* name;   /* "x" / "__input__" is the main input (Model.cpp:4640-4642); others e.g. "mag", "mod" */
  const float* data;  /* host (model_forward) or device (model_forward_device) pointer */
  uint64_t per_sample;/* elements per sample */
  int32_t broadcast;  /* 1 => one copy shared by every sample of the batch (e.g. "mag"/"mod") */
} MimirNamedInput;

typedef struct MimirB200Stats {
  uint64_t arena_peak_bytes;   /* planned activation arena for the last plan */
  uint64_t weight_bytes;       /* device bytes held by uploaded weights */
  uint64_t kernels_launched;   /* kernels of this library launched since init */
  uint64_t flops_last_forward; /* algorithmic flops of the contraction layers in the last forward */
  uint64_t bytes_last_forward; /* algorithmic bytes (inputs + outputs + weights) of the HBM-bound layers */
  float    ms_last_forward;    /* device time of the last forward (CUDA events), 0 if not measured */
} MimirB200Stats;

typedef struct MimirB200Model* MimirB200ModelHandle;

/* Translates the layer list once.  Replaces the per-forward walk of `std::vector<Layer>`
 * (Model.cpp:4795-4891). */
int mimir_b200_model_create(const MimirLayerDesc* layers, int n_layers, MimirB200ModelHandle* out);
int mimir_b200_model_destroy(MimirB200ModelHandle m);
/* Sets the GEMM operand precision for this model (before upload_weights). */
int mimir_b200_model_set_precision(MimirB200ModelHandle m, int precision);
/* Cuts the batch of mimir_b200_model_forward (host pointers) into `micro_batches` pieces whose
 * host->device copy, layer loop and device->host copy overlap on three streams over two arena
 * buffers.  Takes effect at the next plan; the planned batch must be a multiple.  The reference has
 * no counterpart (it has no device boundary on its default path). */
int mimir_b200_model_set_pipeline(MimirB200ModelHandle m, int micro_batches);
/* Copies one layer's flat fp32 weight block (layout = the reference's, Layer::getWeights()).  The
 * host pointer is not kept (it may move: DynamicTensorAllocator.hpp:171-200).  Call again after
 * the weights change. */
int mimir_b200_model_upload_weights(MimirB200ModelHandle m, int layer_index, const float* host,
                                    uint64_t n);
/* Allocates (or re-allocates) the device block of one layer's `n` weights and returns its device
 * pointer for the caller to fill (weights that already live on the GPU, or a loader that streams them
 * in).  upload_weights is this plus one host-to-device copy. */
int mimir_b200_model_weights_device(MimirB200ModelHandle m, int layer_index, uint64_t n, float** dev);
int mimir_b200_model_num_layers(MimirB200ModelHandle m, int* n_layers);
/* Elements per sample of the graph's output tensor "x" in the current plan. */
int mimir_b200_model_output_len(MimirB200ModelHandle m, uint64_t* per_sample);
int mimir_b200_model_layer_info(MimirB200ModelHandle m, int layer_index, const char** name,
                                uint64_t* params_count);
/* Where the planner put a tensor inside one arena buffer: the graph input `input_name`, or the graph output when
 * `input_name` is NULL.  Byte offset and byte size for one (micro-)batch.  Input slots are handed on to later
 * tensors after their last consumer, so an output may share bytes with an input; the pipelined forward orders
 * its copies accordingly.  Diagnostic view of the plan (the reference's counterpart is
 * RuntimeAllocator::get_scratchpad's tag -> buffer map, RuntimeAllocator.hpp:240-280). */
int mimir_b200_model_tensor_slot(MimirB200ModelHandle m, const char* input_name, uint64_t* offset,
                                 uint64_t* bytes);
/* Streams the tensors "<layer name>/weights" (F32, or BF16 widened on the device) of a safetensors
 * checkpoint straight into the device weight blocks, through pinned staging buffers, without a host
 * copy of the model.  Replaces the layer-weights part of SafeTensorsReader::load
 * (Serialization/SafeTensorsReader.cpp:276-325): same tensor naming, same size check ("Size mismatch
 * for ..."), `strict` != 0 fails on a missing tensor ("Missing tensor in strict mode: ...") like
 * LoadOptions::strict_mode.  Other tensors in the file (tokenizer, encoder, optimizer) are ignored. */
int mimir_b200_model_load_safetensors(MimirB200ModelHandle m, const char* path, int strict,
                                      int* layers_loaded, unsigned long long* bytes_loaded);
/* Declares the per-sample size of a named graph input, then plans the activation arena for
 * `batch` samples: liveness over the layer list, offsets reused after the last consumer, peak
 * checked against the budget BEFORE anything is launched (E_OOM_BUDGET).  Mirrors
 * RuntimeAllocator::allocate_tensor / get_scratchpad (RuntimeAllocator.hpp:191-280). */
int mimir_b200_model_plan(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs,
                          int batch, uint64_t* arena_peak_bytes);
/* Host in, host out: H2D of the inputs, the layer loop, D2H of tensor "x".  Replaces
 * Model::forwardPassView (Model.cpp:4621-6824).  *out_len = per-sample output length. */
int mimir_b200_model_forward(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs,
                             int batch, float* out_host, uint64_t out_capacity, uint64_t* out_len);
/* Device in, device out, asynchronous on `stream` (a cudaStream_t, NULL = default stream). */
int mimir_b200_model_forward_device(MimirB200ModelHandle m, const MimirNamedInput* inputs,
                                    int n_inputs, int batch, float* out_dev, uint64_t out_capacity,
                                    uint64_t* out_len, void* stream);
/* Incremental decoding with a key / value cache.  The reference has none (its user guide says so,
 * docs/02-User-Guide/12-Transformer-GPT.md:34-37): generating token by token there re-runs the whole prefix
 * through Model::forwardPass.  For graphs whose layers all act per token (Embedding, Linear with seq_len,
 * LayerNorm with in_features, activations, element-wise layers, CAUSAL self-attention) row t of that full
 * forward depends on tokens 0..t only, so it can be produced from token t alone plus cached keys and values.
 *   decode_begin: on a planned model (pipeline 1); `inputs` declares the PER-TOKEN input sizes (data unused).
 *                 Builds a one-token plan that shares the model's weights and allocates caches of `max_seq`
 *                 positions per attention layer (2 * batch * max_seq * embed floats each; total in *cache_bytes).
 *                 E_UNSUPPORTED names the first layer that does not act per token (e.g. a whole-sample RMSNorm).
 *   prefill:      after decode_begin every mimir_b200_model_forward / _forward_device of the model itself (same
 *                 batch, seq_len <= max_seq) also stores its keys and values at positions 0 .. seq_len-1.
 *   decode_step:  one token per sample at position `pos` (0-based; the caches must hold positions 0 .. pos-1 of the
 *                 same sequences); returns what row `pos` of the full causal forward would be.
 *   decode_end:   frees the caches.  A new plan or upload_weights invalidates the decode state: call decode_begin again. */
int mimir_b200_model_decode_begin(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs,
                                  int batch, int max_seq, uint64_t* cache_bytes);
int mimir_b200_model_decode_step(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs,
                                 int batch, int pos, float* out_host, uint64_t out_capacity, uint64_t* out_len);
int mimir_b200_model_decode_end(MimirB200ModelHandle m);
/* ---- one process, several GPUs -------------------------------------------------------------------------
 * A full replica of the graph on each listed device; a batch is cut into contiguous slices (shard_range), one
 * host thread per device runs its slice through mimir_b200_model_forward, and every slice's result is copied
 * straight into its place in the caller's output buffer (pin it for full copy speed); then the threads are
 * joined.  No device talks to another.  The reference is a single process whose forward loops over samples on
 * the host (Model.cpp:4621-6824 called per sample; LuaScripting.cpp:625-683 holds the one context), so this is
 * the call such a process makes to use all GPUs of a box.  A rank that fails does not stop the others; the
 * status is the first failing rank's and the message names every failed rank ("replica 1 (device 1): ...").
 *   shard_range:        slice [begin, end) of `total` units for `rank` of `world`; the first total % world ranks
 *                       take one extra unit.  Pure host arithmetic.
 *   replicas_create:    mimir_b200_init(device, hbm_budget_bytes) + model_create + set_precision per device.
 *   upload_weights / set_pipeline / plan / forward: the model calls, fanned out; plan takes the TOTAL batch.
 *   inject_failure:     test hook - the next forward fails on that rank on the host, before anything is launched.
 *   selftest_join:      the fan-out / join with a stand-in job that touches no device (CPU-only check of the
 *                       failure reporting). */
typedef struct MimirB200Replicas* MimirB200ReplicasHandle;
int mimir_b200_shard_range(long long total, int world, int rank, long long* begin, long long* end);
int mimir_b200_replicas_create(const int* devices, int n_devices, size_t hbm_budget_bytes,
                               const MimirLayerDesc* layers, int n_layers, int precision,
                               MimirB200ReplicasHandle* out);
int mimir_b200_replicas_destroy(MimirB200ReplicasHandle h);
int mimir_b200_replicas_count(MimirB200ReplicasHandle h, int* n_devices);
int mimir_b200_replicas_upload_weights(MimirB200ReplicasHandle h, int layer_index, const float* host, uint64_t n);
int mimir_b200_replicas_set_pipeline(MimirB200ReplicasHandle h, int micro_batches);
int mimir_b200_replicas_plan(MimirB200ReplicasHandle h, const MimirNamedInput* inputs, int n_inputs,
                             int batch_total, uint64_t* arena_peak_bytes);
int mimir_b200_replicas_forward(MimirB200ReplicasHandle h, const MimirNamedInput* inputs, int n_inputs,
                                int batch_total, float* out_host, uint64_t out_capacity, uint64_t* out_len);
int mimir_b200_replicas_inject_failure(MimirB200ReplicasHandle h, int rank);
int mimir_b200_replicas_selftest_join(int n_ranks, int fail_rank);

/* Per-position argmax over rows of `n` (first maximum wins), for token ids.  No counterpart layer
 * in the reference (harness step of the decoder config). */
int mimir_b200_argmax_rows_device(const float* x_dev, int32_t* ids_dev, long long rows, int n,
                                  void* stream);
int mimir_b200_get_stats(MimirB200Stats* out);
/* Reads (and clears) the device word that bounded in-kernel waits set when they give up:
 * OK, or E_TIMEOUT.  model_forward and the host-pointer calls check it themselves. */
int mimir_b200_check_device(void* stream);
/* Runs the give-up path of the kernels' bounded waits on purpose: one thread block waits `limit_ns` (at most 100 ms)
 * on a barrier that nothing arrives on, then sets the device error word, drains and returns normally.  The next
 * mimir_b200_check_device returns E_TIMEOUT ("site 90"); calls after that work as usual.  Nothing faults or hangs.
 * No counterpart in the reference. */
int mimir_b200_selftest_wait_timeout(unsigned long long limit_ns, void* stream);
/* Live timing of the contraction (GEMM) kernel: while enabled, every launch is bracketed by CUDA
 * events on the launching stream; profile_read synchronises, returns the summed duration and the
 * number of launches, and clears the record.  No counterpart in the reference. */
int mimir_b200_profile_gemm(int enable);
int mimir_b200_profile_read(float* total_ms, int* launches);

/* ---------------------------------------------------------------------------------------------
 * Device-pointer forms of the per-op calls (inputs already resident in HBM, asynchronous on
 * `stream`).  The host-pointer forms above are these plus the copies.
 * ------------------------------------------------------------------------------------------ */
int mimir_b200_dev_layernorm(const float* x, const float* gamma, const float* beta, float* y,
                             long long rows, int n, float eps, void* stream);
int mimir_b200_dev_rmsnorm(const float* x, const float* gamma, long long n_gamma, float* y,
                           int batch, long long n, float eps, void* stream);
/* RMSNorm with device pointers that allocates nothing, for callers that cannot call cudaMalloc:
 * a step of a latency-critical serving loop (an allocation synchronises the device), a process
 * that has given all free device memory to its own pool, a plugin whose host forbids allocation.
 * This entry point has no counterpart in the reference.  Same arithmetic as
 * mimir_b200_dev_rmsnorm's chunked path (per-chunk sums of squares; for samples above 16 384
 * elements also the rounding errors of the reference's one sequential fp32 sum, so the result
 * agrees with the CPU path like the regular entry point's does; then normalise), but the partial
 * sums and error terms live in a fixed 192 KB array inside the library (held on every GPU that
 * loads it).
 * Limit: batch * ceil(n / 8192) <= 16384 and batch <= 65535, else E_INVALID.  It neither needs nor
 * calls mimir_b200_init.  The first call on each device looks up the array's device address, so
 * make that first call outside any stream capture.  All calls share the array: calls that may
 * overlap on the GPU (different streams, or threads) race on it; calls on one stream are safe, and
 * nothing needs clearing between calls. */
int mimir_b200_dev_rmsnorm_noalloc(const float* x, const float* gamma, long long n_gamma, float* y,
                                   int batch, long long n, float eps, void* stream);
int mimir_b200_dev_groupnorm(const float* x, const float* gamma, const float* beta, float* y,
                             int batch, int channels, int h, int w, int groups, float eps, int act,
                             void* stream);
int mimir_b200_dev_softmax(const float* x, float* y, int batch, long long n, int log_softmax,
                           void* stream);
int mimir_b200_dev_eltwise(int op, const float* a, const float* b, float* y, int batch, long long n,
                           long long nb, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MIMIR_B200_H */
