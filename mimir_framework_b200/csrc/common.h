// common.h — shared host-side plumbing of the backend: status codes, error text, the process-wide
// context (device, budget guard, launch counter) and the launch prototypes of every kernel file.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "mimir_b200.h"

namespace mb {

// ---- error text (thread-local, read through mimir_b200_last_error) -------------------------
std::string& last_error();
int fail(int status, const char* fmt, ...);

#define MB_CUDA(expr)                                                                         \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return ::mb::fail(MIMIR_B200_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                        __FILE__, __LINE__);                                                  \
  } while (0)

#define MB_TRY(expr)              \
  do {                            \
    int _s = (expr);              \
    if (_s != MIMIR_B200_OK) return _s; \
  } while (0)

// ---- budget guard: the device-side counterpart of MemoryGuard (MemoryGuard.hpp:16-206) -----
struct Guard {
  std::mutex mu;
  size_t limit = 0, current = 0, peak = 0;
  bool blocked = false, frozen = false;       // MemoryGuard::blockAllocations / freezeAllocations (MemoryGuard.hpp:37-72)
  size_t blocked_attempts = 0, frozen_attempts = 0;
  // 0 = granted, 1 = over the limit, 2 = blocked, 3 = frozen (the order of the checks in MemoryGuard::requestAllocation)
  int request_why(size_t bytes);
  bool request(size_t bytes) { return request_why(bytes) == 0; }
  void release(size_t bytes);
  void reset();                                // MemoryGuard::reset (MemoryGuard.hpp:181-186): usage and peak to zero
};

// Device buffers handed out by the RuntimeAllocator verbs (capi.cu): live ones by address, pooled scratchpads by tag.
struct OwnedBuffers {
  struct Buf { size_t bytes; std::string tag; };
  std::mutex mu;
  std::unordered_map<void*, Buf> live;
  std::map<std::string, std::pair<void*, size_t>> pool;
  size_t total_allocated = 0, num_allocations = 0, local_cap = 0;
};

struct Context {
  bool initialised = false;
  int device = 0;
  int sm_count = 148;
  Guard guard;
  OwnedBuffers owned;
  std::atomic<uint64_t> launches{0};
  // One device word that kernels with bounded waits set when a wait gives up.
  int* dev_error_word = nullptr;
  // Optional live timing of the contraction kernel: pairs of events recorded on the launching
  // stream around every GEMM launch while enabled (read back by mimir_b200_profile_read).
  bool prof_gemm = false;
  std::vector<cudaEvent_t> prof_events;
  MimirB200Stats stats{};
};
// One context per CUDA device, selected by the calling thread's current device (cudaGetDevice); slot 0 when no
// device is reachable, so that the host-only verbs (the budget guard) work on a machine without a GPU.
constexpr int MAX_DEVICES = 64;
Context& ctx();
Context& ctx_of(int device);

// Function attributes (opt-in shared memory sizes) belong to a device: set them once per device, not once per process.
struct PerDeviceOnce {
  std::mutex mu;
  uint64_t done = 0;
  template <class F>
  int run(F&& fn) {
    const int dev = ctx().device;
    std::lock_guard<std::mutex> lk(mu);
    if (done & (1ull << dev)) return MIMIR_B200_OK;
    const int s = fn();
    if (s == MIMIR_B200_OK) done |= (1ull << dev);
    return s;
  }
};

// Makes `device` current on the calling thread for the lifetime of the object (model handles carry their device).
struct DeviceScope {
  int prev = -1;
  explicit DeviceScope(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != device) cudaSetDevice(device); else prev = -1;
  }
  ~DeviceScope() { if (prev >= 0) cudaSetDevice(prev); }
};

// The device a model handle lives on (the calling thread's current device for a null handle); graph.cu.
int model_device(MimirB200ModelHandle m);

// Budgeted device allocation: every cudaMalloc of the backend goes through these.
int dev_alloc(void** p, size_t bytes, const char* tag);
void dev_free(void* p, size_t bytes);
// Frees every buffer of the RuntimeAllocator verbs on the current device (shutdown).
void release_owned_buffers();

inline void count_launch(int n = 1) { ctx().launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

// ---- kernel launchers (device pointers, asynchronous on `st`) -------------------------------
// Activation codes follow MimirB200Eltwise; -1 = none.

// gemm_sm100.cu --------------------------------------------------------------------------------
// Split planes: bf16 [planes][rows][kp] with kp = round_up(k, 64), zero padded.
inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline int64_t plane_elems(int64_t rows, int k) { return rows * static_cast<int64_t>(round_up(k, 64)); }
// The planes are 16-bit containers declared as __nv_bfloat16 throughout; what the 16 bits hold (bfloat16 or IEEE
// half) is a process-wide choice, see planes.cuh.  MIMIR_B200_PLANES=bf16 selects bfloat16 planes; half is the default.
int plane_format();
// Power of two that the weights of one layer are multiplied by before they become half planes (1 for bfloat16
// planes): brings the largest magnitude near 2^14 so that small weights keep their bits.  Synchronises `st`.
int weight_plane_scale(const float* w_dev, size_t n, cudaStream_t st, float* scale);
// fp32 [rows, k] -> planes (hi, and lo when planes == 2) of src * scale
int launch_split(const float* src, __nv_bfloat16* dst, int64_t rows, int k, int planes, cudaStream_t st, float scale = 1.0f);
// fp32 [k, n] (row-major, "input-major") -> planes of its transpose [n, kp], times scale
int launch_split_transposed(const float* src, __nv_bfloat16* dst, int k, int n, int planes, cudaStream_t st, float scale = 1.0f);

struct GemmArgs {
  const __nv_bfloat16* a = nullptr;  // [a_planes][m][kp]
  const __nv_bfloat16* w = nullptr;  // [w_planes][n][kp]
  int a_planes = 2, w_planes = 2;
  float w_scale = 1.0f;              // the weight planes hold w * w_scale (weight_plane_scale); divided out in the epilogue
  int m = 0, n = 0, k = 0;           // logical sizes; kp = round_up(k, 64)
  const float* bias = nullptr;       // [n] or null
  const float* residual = nullptr;   // fp32 [m, n] added after the activation, or null
  int activation = -1;
  float* out_f32 = nullptr;          // fp32 [m, ldo] or null
  int64_t ldo = 0;
  int out_nchw_hw = 0;               // > 0: out_f32/residual are [m / hw][n][hw] (conv output), ldo unused
  __nv_bfloat16* out_split = nullptr;  // planes [2][m][round_up(n,64)] for the next GEMM, or null
  // Shifted-GEMM convolution (conv_ks > 0): `a` is the zero-padded NHWC activation [samples*(h+2p)*(w+2p)][conv_c],
  // m counts padded-grid rows, k = conv_ks^2 * conv_c ordered (tap, channel), output is NCHW [samples][n][h][w].
  int conv_ks = 0, conv_c = 0, conv_pad = 0, conv_h = 0, conv_w = 0;
  // Grouped form (a_group_rows > 0, plain row-major GEMM only): the rows of `a` come in groups of a_group_rows, and group g
  // multiplies the w rows [g * w_group_rows, g * w_group_rows + n): a block-diagonal batch of small GEMMs in one launch
  // (attention scores Q_b K_b^T and P_b V_b per sample).  `w` then holds w_rows_total rows.
  int a_group_rows = 0, w_group_rows = 0;
  long long w_rows_total = 0;
  // Channel-major outputs (out_nchw_hw > 0 or conv_ks > 0): GroupNorm partials of the values stored, per 32-pixel block and
  // 32-channel chunk, for the GroupNorm that reads this output; gemm_gn_part_bytes() of scratch.  gn_cpg in {4, 8, 16, 32}.
  float* gn_part = nullptr;
  int gn_cpg = 0;
};
inline size_t gemm_gn_part_bytes(long long m, int n, int cpg) {
  return static_cast<size_t>((m + 31) / 32) * static_cast<size_t>((n + 31) / 32) * static_cast<size_t>(2 * (1 + 64 / cpg)) * sizeof(float);
}
// (mean, 1 / sqrt(var + eps)) per (sample, group) from those partials; `per` = rows of the GEMM's M index per sample
int launch_gn_stats_from_partials(const float* part, float* stats, int batch, int groups, int cpg, long long m, int n, int per, float eps,
                                  cudaStream_t st);
// y = act(a · wᵀ + bias) (+ residual); tcgen05 / TMEM / TMA.
int launch_gemm(const GemmArgs& g, cudaStream_t st);
// Runs the bounded-wait give-up path on purpose: one CTA waits `limit_ns` on a barrier nobody arrives on, sets the device
// error word (site 90) and returns after freeing its tensor memory.
int launch_wait_timeout_selftest(unsigned long long limit_ns, cudaStream_t st);
// fp32 weight-streaming kernel for very small m (<= 16 rows): y[m,n] = x[m,k] · w[n,k]ᵀ + bias.
int launch_skinny_linear(const float* x, const float* w, const float* bias, float* y, int m, int k, int n,
                         int activation, float* scratch, size_t scratch_bytes, cudaStream_t st, const float* residual = nullptr);
size_t skinny_scratch_bytes(int m, int k, int n);

// pointwise.cu ---------------------------------------------------------------------------------
int launch_eltwise(int op, const float* a, const float* b, float* y, int batch, int64_t n, int64_t nb,
                   cudaStream_t st, float alpha = 0.0f);
int launch_embedding(const float* ids_f32, const int32_t* ids_i32, const float* table, float* y, int64_t n_ids,
                     int vocab, int dim, int padding_idx, cudaStream_t st);
int launch_upsample_nearest(const float* x, float* y, int batch, int ch, int in_h, int in_w, int sh, int sw,
                            cudaStream_t st);
int launch_permute(const float* x, float* y, int batch, int nd, const int* shape, const int* dims, cudaStream_t st);
int launch_token_mean_pool(const float* x, float* y, int batch, int seq, int dim, cudaStream_t st);
int launch_global_avgpool(const float* x, float* y, int batch, int ch, int hw, cudaStream_t st);
int launch_argmax_rows(const float* x, int32_t* ids, int64_t rows, int n, cudaStream_t st);
// copies `n` floats per sample from src (per-sample stride n) into dst at offset `off` of a
// per-sample vector of `total` floats (Concat)
// (Concat); with `src_stride` > 0 the source is a slice of a larger per-sample vector (Split / Chunk)
int launch_copy_strided(const float* src, float* dst, int batch, int64_t n, int64_t total, int64_t off,
                        cudaStream_t st, int64_t src_stride = 0);
int launch_broadcast_rows(const float* src, float* dst, int batch, int64_t n, cudaStream_t st);

// norms.cu -------------------------------------------------------------------------------------
int launch_layernorm(const float* x, const float* gamma, const float* beta, float* y, int64_t rows, int64_t n,
                     float eps, cudaStream_t st);
// y_split (optional): the result as bf16 hi (+ lo) operand planes, `plane_stride` elements apart, written by the
// one-pass kernel; only where rmsnorm_onepass_ok() holds.  y may then be nullptr.
int launch_rmsnorm(const float* x, const float* gamma, int64_t n_gamma, float* y, int batch, int64_t n, float eps,
                   cudaStream_t st, __nv_bfloat16* y_split = nullptr, int planes = 0, int64_t plane_stride = 0);
bool rmsnorm_onepass_ok(int batch, int64_t n);
// The chunked norm / softmax paths keep partial results in a scratch buffer per (device, stream), allocated at first use.
// A stream that is about to be captured into a CUDA graph must have its buffer beforehand (no allocation while
// capturing) and keeps it, at a fixed address, until norm_scratch_release: call on the stream's device.
int norm_scratch_reserve(cudaStream_t st);
void norm_scratch_release(cudaStream_t st);
int launch_groupnorm(const float* x, const float* gamma, const float* beta, float* y, int batch, int ch, int hw,
                     int groups, float eps, int act, const float* residual, cudaStream_t st);
int launch_softmax(const float* x, float* y, int batch, int64_t n, int log_softmax, cudaStream_t st);
// stats[(sample * groups + g) * 2 + {0, 1}] = mean, 1 / sqrt(var + eps) of each GroupNorm slab
int launch_groupnorm_stats(const float* x, float* stats, int batch, int ch, int hw, int groups, float eps, cudaStream_t st);
int launch_groupnorm_apply(const float* x, const float* stats, const float* gamma, const float* beta, float* y, int batch, int ch, int hw,
                           int groups, float eps, int act, const float* residual, cudaStream_t st);

// attention.cu ---------------------------------------------------------------------------------
// Where the projected queries, keys and values of one attention call live: row-major fp32, sample b at
// q + b*q_len*ldq and k/v + b*kv_len*ldkv.
struct AttnView {
  const float* q = nullptr;
  const float* k = nullptr;
  const float* v = nullptr;
  long long ldq = 0, ldkv = 0;
  int q_len = 0, kv_len = 0;
  long long q_bstride = 0, kv_bstride = 0;  // elements between samples; 0 = q_len * ldq / kv_len * ldkv
  // decode steps replayed from a CUDA graph: the position lives in device memory (kv_len = *pos_dev + 1) and
  // kv_len above is the cache capacity the launch is sized for
  const int* pos_dev = nullptr;
};
// One query row per (sample, head) against kv_len cached keys / values (a decode step), keys cut into chunks
size_t attention_decode_scratch_bytes(int batch, int heads, int embed, int max_seq);
bool attention_decode_supported(const AttnView& a, int embed, int heads);
int launch_attention_decode(const AttnView& a, float* out, float* scratch, int batch, int embed, int heads, cudaStream_t st);
// K and V thirds of qkv [batch*seq][3E] -> cache[b][pos0 + s][E] of caches holding max_seq positions per sample
int launch_kv_cache_write(const float* qkv, float* kcache, float* vcache, int batch, int seq, int embed, int max_seq, int pos0,
                          cudaStream_t st, const int* pos_dev = nullptr);
// qkv fp32 [batch*seq, 3E] (Q | K | V thirds) -> attended fp32 [batch*seq, E]
int launch_attention_core(const float* qkv, float* out, int batch, int seq, int embed, int heads, int causal,
                          cudaStream_t st);
// general form (cross attention: queries and keys/values from different projections and lengths)
int launch_attention_core_view(const AttnView& a, float* out, int batch, int embed, int heads, int causal, cudaStream_t st);
// attention_tc.cu: the same core on tcgen05 (head_dim 64); `ws` holds the bf16 operand planes
// a single wide head as two block-diagonal GEMMs around a row softmax (attention_gemm.cu)
bool attention_gemm_supported(int batch, int seq, int embed, int heads);
size_t attention_gemm_ws_bytes(int batch, int seq, int embed);
int launch_attention_core_gemm(const float* qkv, int batch, int seq, int embed, int causal, void* ws, __nv_bfloat16* out_split,
                               cudaStream_t st);
bool attention_tc_supported(int seq, int embed, int heads);
size_t attention_tc_ws_bytes(int batch, int seq, int embed);
int launch_attention_core_tc(const float* qkv, float* out, int batch, int seq, int embed, int heads, int causal, void* ws,
                             cudaStream_t st, __nv_bfloat16* out_split = nullptr, int planes = 0,
                             const __nv_bfloat16* qkv_planes = nullptr);  // hi/lo planes [2][batch*seq][3E] instead of fp32 qkv

// conv2d.cu ------------------------------------------------------------------------------------
// im2col of NCHW fp32 into split planes [planes][batch*oh*ow][kp], k = ic*ks*ks ordered (ic, kh, kw)
int launch_im2col_split(const float* x, __nv_bfloat16* dst, int batch, int ic, int h, int w, int ks, int stride,
                        int pad, int oh, int ow, int planes, cudaStream_t st);
// NCHW fp32 -> zero-padded NHWC planes [planes][batch*(h+2p)*(w+2p)][c] (borders written as zero)
// A GroupNorm (+ SiLU) whose only consumer is the convolution can be applied on the way: `pre` carries its
// statistics and affine parameters.
struct PreNorm {
  const float* stats = nullptr;  // [batch][groups][2] from launch_groupnorm_stats; null = no normalisation
  const float* gamma = nullptr;
  const float* beta = nullptr;
  int groups = 1;
  int act = -1;                  // -1 or MIMIR_B200_ELT_SILU
};
// up != 0: x is [batch][c][h/2][w/2] and every source pixel covers a 2 x 2 block of the h x w image (nearest-neighbour upsample)
int launch_nchw_to_padded_nhwc_split(const float* x, __nv_bfloat16* dst, int batch, int c, int h, int w, int pad, int planes,
                                     cudaStream_t st, const PreNorm& pre = PreNorm(), int up = 0);
// OIHW fp32 -> planes [planes][oc][round_up(ks*ks*ic, 64)] with K ordered (kh, kw, ic)
int launch_conv_weight_planes(const float* w, __nv_bfloat16* dst, int oc, int ic, int ks, int planes, cudaStream_t st, float scale = 1.0f);

// direct fp32 convolution for layers with at most 8 output channels (stride 1, "same" padding): x NCHW, w OIHW, y NCHW
bool conv_small_oc_supported(int oc, int ks, int stride, int pad, int h, int wd, int batch, int act);
int launch_conv_small_oc(const float* x, const float* w, float* y, const float* residual, int batch, int ic, int oc, int h, int wd, int ks,
                         int pad, int act, cudaStream_t st);

// spatial.cu -----------------------------------------------------------------------------------
int launch_depthwise_conv2d(const float* x, const float* w, const float* bias, float* y, int batch, int ch, int h, int wd, int k,
                            int stride, int pad, int64_t w_count, cudaStream_t st);
int launch_conv1d(const float* x, const float* w, const float* bias, float* y, int batch, int ic, int oc, int len, int k, int stride,
                  int pad, int64_t w_count, cudaStream_t st);
int launch_conv_gather(const float* x, const float* w, float* y, int batch, int ic, int oc, int h, int wd, int oh, int ow, int k,
                       int stride, int pad, int relu, cudaStream_t st);
// EmbeddingBag / PatchEmbed / Bilinear / RNN-GRU-LSTM (sequence.cu); every tensor is [batch][per-sample elements]
int launch_embedding_bag(const float* ids, int64_t ids_ps, const float* offsets, int64_t off_ps, const float* table, float* y, int batch,
                         int vocab, int dim, int padding_idx, cudaStream_t st);
int launch_patch_embed(const float* x, const float* w, float* y, int batch, int d_model, int seq_text, int num_patches, int patch_dim,
                       cudaStream_t st);
int launch_bilinear(const float* x1, const float* x2, const float* w, const float* bias, float* y, int64_t rows, int in1, int in2,
                    int out_f, cudaStream_t st);
int launch_recurrent(int kind, const float* x, const float* w, float* y, int batch, int T, int I, int H, int use_bias, cudaStream_t st);
// the static compute family (Model::computeConv2D / computeConvTranspose2D / computeBatchNorm with batch statistics)
int launch_conv2d_dilated(const float* x, const float* w, const float* bias, float* y, int batch, int ic, int oc, int h, int wd, int k,
                          int stride, int pad, int dil, cudaStream_t st);
int launch_conv_transpose2d_scatter(const float* x, const float* w, const float* bias, float* y, int batch, int ic, int oc, int h, int wd,
                                    int k, int stride, int pad, cudaStream_t st);
int launch_batchnorm_batchstats(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels, long long spatial,
                                float eps, cudaStream_t st);
int launch_pool2d(int is_max, const float* x, float* y, int batch, int ch, int h, int wd, int kh, int kw, int sh, int sw, int ph, int pw,
                  cudaStream_t st);
int launch_pad2d(int mode, const float* x, float* y, int batch, int ch, int h, int wd, int ph, int pw, cudaStream_t st);
int launch_pixel_shuffle(const float* x, float* y, int batch, int ic, int h, int wd, int r, cudaStream_t st);
int launch_upsample_bilinear(const float* x, float* y, int batch, int ch, int h, int wd, int oh, int ow, int half_pixel,
                             cudaStream_t st);
int launch_batch_matmul(const float* a, const float* b, float* c, int64_t nb, int m, int k, int n, cudaStream_t st);
int launch_batchnorm_running(const float* x, const float* gamma, const float* beta, const float* mean, const float* var, float* y,
                             int batch, int channels, int64_t spatial, float eps, cudaStream_t st);
int launch_scale_prefix(float* y, const float* g, int batch, int64_t n, int64_t cnt, cudaStream_t st);
}  // namespace mb
