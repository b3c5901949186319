// capi.cu — the C ABI of include/mimir_b200.h: process context and HBM budget guard, the per-op
// entry points with host pointers (drop-in for ComputeEngine::linearForward,
// VulkanCompute.hpp:209-210), and their device-pointer forms.  The whole-graph entry points live
// in graph.cu.  No function here throws; none falls back to the CPU.
#include "ops.h"
#include "host_call.h"

#include <cstdlib>
#include <cstring>
#include <vector>

namespace mb {

// ---------------------------------------------------------------------------------------------
// context, errors, guard
// ---------------------------------------------------------------------------------------------
std::string& last_error() {
  thread_local std::string e;
  return e;
}

int fail(int status, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error() = buf;
  return status;
}

static Context g_ctx[MAX_DEVICES];

Context& ctx_of(int device) { return g_ctx[(device >= 0 && device < MAX_DEVICES) ? device : 0]; }

Context& ctx() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) {
    cudaGetLastError();  // no driver / no device: not an error of the caller's
    d = 0;
  }
  return ctx_of(d);
}

int Guard::request_why(size_t bytes) {
  std::lock_guard<std::mutex> lk(mu);
  if (blocked) { ++blocked_attempts; return 2; }
  if (frozen) { ++frozen_attempts; return 3; }
  if (limit != 0 && current + bytes > limit) return 1;
  current += bytes;
  if (current > peak) peak = current;
  return 0;
}
void Guard::reset() {
  std::lock_guard<std::mutex> lk(mu);
  current = 0;
  peak = 0;
}
void Guard::release(size_t bytes) {
  std::lock_guard<std::mutex> lk(mu);
  current = (bytes > current) ? 0 : current - bytes;
}

int dev_alloc(void** p, size_t bytes, const char* tag) {
  *p = nullptr;
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called");
  if (bytes == 0) return MIMIR_B200_OK;
  if (const int why = ctx().guard.request_why(bytes))
    return fail(MIMIR_B200_E_OOM_BUDGET, "HBM budget refused %zu bytes for %s (%s; limit %zu, in use %zu)", bytes, tag,
                why == 2 ? "allocations are blocked" : why == 3 ? "allocations are frozen" : "over the limit", ctx().guard.limit,
                ctx().guard.current);
  cudaError_t e = cudaMalloc(p, bytes);
  if (e != cudaSuccess) {
    ctx().guard.release(bytes);
    *p = nullptr;
    return fail(MIMIR_B200_E_CUDA, "cudaMalloc(%zu) for %s failed: %s", bytes, tag, cudaGetErrorString(e));
  }
  return MIMIR_B200_OK;
}

void dev_free(void* p, size_t bytes) {
  if (!p) return;
  cudaFree(p);
  ctx().guard.release(bytes);
}

void release_owned_buffers() {
  OwnedBuffers& ob = ctx().owned;
  std::lock_guard<std::mutex> lk(ob.mu);
  for (auto& kv : ob.live) dev_free(kv.first, kv.second.bytes);
  for (auto& kv : ob.pool) dev_free(kv.second.first, kv.second.second);
  ob.live.clear();
  ob.pool.clear();
}

// Reads (and clears) the word that kernels with bounded waits set when a wait gave up.
int check_device_error_word(cudaStream_t st) {
  int w = 0;
  MB_CUDA(cudaMemcpyAsync(&w, ctx().dev_error_word, sizeof(int), cudaMemcpyDeviceToHost, st));
  MB_CUDA(cudaStreamSynchronize(st));
  if (w != 0) {
    cudaMemsetAsync(ctx().dev_error_word, 0, sizeof(int), st);
    cudaStreamSynchronize(st);
    return fail(MIMIR_B200_E_TIMEOUT, "a device-side wait gave up (site %d)", w);
  }
  return MIMIR_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// op sequences on device pointers (shared by the per-op ABI and the graph executor)
// ---------------------------------------------------------------------------------------------
void precision_planes(int precision, int* a_planes, int* w_planes) {
  *a_planes = (precision == MIMIR_B200_PREC_BF16) ? 1 : 2;
  *w_planes = (precision == MIMIR_B200_PREC_BF16X2) ? 2 : 1;
}

size_t split_bytes(int64_t rows, int k, int planes) {
  return static_cast<size_t>(planes) * static_cast<size_t>(plane_elems(rows, k)) * sizeof(__nv_bfloat16);
}


// A handful of rows stream the fp32 weights once through every SM (exact fp32 arithmetic, so it serves every
// precision mode); a 128-row GEMM tile would keep one SM per 256 output columns busy with mostly empty rows.
bool linear_uses_skinny(int rows, int precision) {
  (void)precision;
  return rows <= 16;
}

size_t linear_ws_bytes(int rows, int in_f, int out_f, int precision, bool a_presplit) {
  if (linear_uses_skinny(rows, precision)) return align256(skinny_scratch_bytes(rows, in_f, out_f));
  if (a_presplit) return 0;
  int ap, wp;
  precision_planes(precision, &ap, &wp);
  return align256(split_bytes(rows, in_f, ap));
}

int linear_exec(const LinearExec& e, cudaStream_t st) {
  if (linear_uses_skinny(e.rows, e.precision)) {
    if (!e.x_f32 || !e.w_f32 || !e.y_f32) return fail(MIMIR_B200_E_INVALID, "linear: skinny path needs fp32 operands");
    return launch_skinny_linear(e.x_f32, e.w_f32, e.bias, e.y_f32, e.rows, e.in_f, e.out_f, e.activation, static_cast<float*>(e.ws),
                                e.ws_bytes, st, e.residual);
  }
  int ap, wp;
  precision_planes(e.precision, &ap, &wp);
  const __nv_bfloat16* a = e.x_split;
  if (!a) {
    if (!e.x_f32 || !e.ws) return fail(MIMIR_B200_E_INVALID, "linear: no activation operand");
    MB_TRY(launch_split(e.x_f32, static_cast<__nv_bfloat16*>(e.ws), e.rows, e.in_f, ap, st));
    a = static_cast<const __nv_bfloat16*>(e.ws);
  }
  GemmArgs g;
  g.a = a;
  g.w = e.w_split;
  g.a_planes = ap;
  g.w_planes = wp;
  g.w_scale = e.w_scale;
  g.m = e.rows;
  g.n = e.out_f;
  g.k = e.in_f;
  g.bias = e.bias;
  g.residual = e.residual;
  g.activation = e.activation;
  g.out_f32 = e.y_f32;
  g.ldo = e.out_f;
  g.out_nchw_hw = e.out_nchw_hw;
  g.out_split = e.y_split;
  return launch_gemm(g, st);
}

// Attention = QKV projection (GEMM) -> flash core -> output projection (GEMM).
// Workspace: split(x) | qkv fp32 | attended fp32 | split(attended)
size_t attention_ws_bytes(int batch, int seq, int embed, int heads, int precision) {
  int ap, wp;
  precision_planes(precision, &ap, &wp);
  const size_t rows = static_cast<size_t>(batch) * seq;
  size_t b = align256(split_bytes(static_cast<int64_t>(rows), embed, ap)) + align256(rows * 3 * embed * 4) + align256(rows * embed * 4);
  if (attention_tc_supported(seq, embed, heads)) b += align256(attention_tc_ws_bytes(batch, seq, embed));
  else if (attention_gemm_supported(batch, seq, embed, heads)) b += align256(attention_gemm_ws_bytes(batch, seq, embed));
  return b;
}

static bool no_qkv_planes() {
  static const bool off = [] { const char* v = getenv("MIMIR_B200_ATTN_QKV_PLANES"); return v && v[0] == '0'; }();
  return off;
}

int attention_exec(const AttentionExec& e, cudaStream_t st) {
  int ap, wp;
  precision_planes(e.precision, &ap, &wp);
  const int rows = e.batch * e.seq;
  uint8_t* ws = static_cast<uint8_t*>(e.ws);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ws);
  float* qkv = reinterpret_cast<float*>(ws + align256(split_bytes(rows, e.embed, ap)));
  float* att = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(qkv) + align256(static_cast<size_t>(rows) * 3 * e.embed * 4));
  uint8_t* tc_ws = reinterpret_cast<uint8_t*>(att) + align256(static_cast<size_t>(rows) * e.embed * 4);
  // a decode step of a few samples: both projections stream fp32 weights (transposed copies, W[out][in]) instead of
  // running 128-row GEMM tiles that are almost empty
  bool qkv_as_planes = false;
  const bool stream_w = e.decode_pos >= 0 && e.wqkv_t_f32 && e.wout_t_f32 && e.x && rows <= 16 && e.skinny_scratch;
  if (stream_w) {
    MB_TRY(launch_skinny_linear(e.x, e.wqkv_t_f32, nullptr, qkv, rows, e.embed, 3 * e.embed, -1, e.skinny_scratch, e.skinny_scratch_bytes, st));
  } else {
    if (!e.x_split) MB_TRY(launch_split(e.x, xs, rows, e.embed, ap, st));
    GemmArgs g;
    g.a = e.x_split ? e.x_split : xs; g.w = e.wqkv_split; g.a_planes = ap; g.w_planes = wp; g.w_scale = e.w_scale;
    g.m = rows; g.n = 3 * e.embed; g.k = e.embed; g.ldo = 3 * e.embed;
    // the tensor-core attention core takes Q and K straight from hi/lo planes written by this GEMM's epilogue (they
    // occupy the fp32 buffer's place: 2 planes x 2 bytes); a cache fill or decode step needs the fp32 rows
    qkv_as_planes = attention_tc_supported(e.seq, e.embed, e.heads) && !e.kcache && e.decode_pos < 0 && !no_qkv_planes();
    if (qkv_as_planes) g.out_split = reinterpret_cast<__nv_bfloat16*>(qkv);
    else g.out_f32 = qkv;
    MB_TRY(launch_gemm(g, st));
  }
  if (e.kcache)
    MB_TRY(launch_kv_cache_write(qkv, e.kcache, e.vcache, e.batch, e.seq, e.embed, e.max_seq, e.decode_pos < 0 ? 0 : e.decode_pos, st,
                                 e.decode_pos >= 0 ? e.pos_dev : nullptr));
  if (e.decode_pos >= 0) {
    // one new token per sample against the cached keys and values (all of them are in its past)
    if (!e.kcache || e.seq != 1) return fail(MIMIR_B200_E_INVALID, "attention: a decode step needs a cache and one token per sample");
    AttnView a;
    a.q = qkv; a.ldq = 3LL * e.embed; a.q_len = 1;
    a.k = e.kcache; a.v = e.vcache; a.ldkv = e.embed; a.kv_len = e.decode_pos + 1;
    a.kv_bstride = static_cast<long long>(e.max_seq) * e.embed;
    if (e.decode_scratch && attention_decode_supported(a, e.embed, e.heads)) {
      if (e.pos_dev) {  // sized for the whole cache; the kernels read the position themselves
        a.kv_len = e.max_seq;
        a.pos_dev = e.pos_dev;
      }
      MB_TRY(launch_attention_decode(a, att, e.decode_scratch, e.batch, e.embed, e.heads, st));
    } else if (e.pos_dev) {
      return fail(MIMIR_B200_E_UNSUPPORTED, "attention: this head layout cannot take its position from device memory");
    } else
      MB_TRY(launch_attention_core_view(a, att, e.batch, e.embed, e.heads, 0, st));
    if (stream_w) {
      return launch_skinny_linear(att, e.wout_t_f32, nullptr, e.y, rows, e.embed, e.embed, -1, e.skinny_scratch, e.skinny_scratch_bytes, st,
                                  e.residual);
    }
    MB_TRY(launch_split(att, xs, rows, e.embed, ap, st));
  } else
  // the attended rows go to the output projection as operand planes (the x planes are dead by now)
  if (attention_tc_supported(e.seq, e.embed, e.heads)) {
    MB_TRY(launch_attention_core_tc(qkv, nullptr, e.batch, e.seq, e.embed, e.heads, e.causal, tc_ws, st, xs, ap,
                                    qkv_as_planes ? reinterpret_cast<const __nv_bfloat16*>(qkv) : nullptr));
  } else if (attention_gemm_supported(e.batch, e.seq, e.embed, e.heads) && !e.kcache) {
    // one wide head: scores and P.V as block-diagonal GEMMs; the second one writes the output projection's planes
    MB_TRY(launch_attention_core_gemm(qkv, e.batch, e.seq, e.embed, e.causal, tc_ws, xs, st));
  } else {
    MB_TRY(launch_attention_core(qkv, att, e.batch, e.seq, e.embed, e.heads, e.causal, st));
    MB_TRY(launch_split(att, xs, rows, e.embed, ap, st));
  }
  GemmArgs o;
  o.a = xs; o.w = e.wout_split; o.a_planes = ap; o.w_planes = wp; o.w_scale = e.w_scale;
  o.m = rows; o.n = e.embed; o.k = e.embed; o.out_f32 = e.y; o.ldo = e.embed; o.residual = e.residual;
  return launch_gemm(o, st);
}

// Conv2d = im2col planes (per batch chunk) -> GEMM with an NCHW epilogue.
int conv_chunk_samples(int batch, int ohw, int k, int precision) {
  int ap, wp;
  precision_planes(precision, &ap, &wp);
  const size_t per_sample = split_bytes(ohw, k, ap);
  const size_t target = size_t(1) << 30;  // ~1 GB of im2col planes in flight
  long long c = static_cast<long long>(target / (per_sample ? per_sample : 1));
  if (c < 1) c = 1;
  if (c > batch) c = batch;
  return static_cast<int>(c);
}

bool conv_uses_shifted(int ic, int ks, int stride, int pad) {
  const char* off = getenv("MIMIR_B200_CONV_IM2COL");
  if (off && off[0] == '1') return false;
  return stride == 1 && (ks & 1) == 1 && pad == ks / 2 && ic % 32 == 0 && ks <= 7;
}

size_t conv_prenorm_bytes(int batch, int groups) { return align256(static_cast<size_t>(batch) * groups * 2 * sizeof(float)); }

size_t conv_gn_emit_bytes(int batch, int oc, int h, int w, int pad, int groups) {
  const long long rows = static_cast<long long>(batch) * (h + 2 * pad) * (w + 2 * pad);
  return align256(gemm_gn_part_bytes(rows, oc, oc / groups));
}

bool conv_can_emit_gn(int batch, int ic, int oc, int h, int w, int ks, int stride, int pad, int groups, int act) {
  static const bool on = [] { const char* e = getenv("MIMIR_B200_GN_EPILOGUE"); return e && e[0] == '1'; }();
  if (!on || groups <= 0 || oc % groups != 0) return false;
  const int cpg = oc / groups;
  if (!(cpg == 4 || cpg == 8 || cpg == 16 || cpg == 32)) return false;
  if (!conv_uses_shifted(ic, ks, stride, pad) || conv_small_oc_supported(oc, ks, stride, pad, h, w, batch, act)) return false;
  return static_cast<long long>(h + 2 * pad) * (w + 2 * pad) >= 64 && batch <= 65535;
}

size_t conv_ws_bytes(int batch, int ic, int h, int w, int ks, int stride, int pad, int precision) {
  int ap, wp;
  precision_planes(precision, &ap, &wp);
  if (conv_uses_shifted(ic, ks, stride, pad))
    return align256(static_cast<size_t>(ap) * batch * (h + 2 * pad) * (w + 2 * pad) * ic * sizeof(__nv_bfloat16));
  const int oh = (h + 2 * pad - ks) / stride + 1, ow = (w + 2 * pad - ks) / stride + 1;
  const int k = ic * ks * ks;
  return align256(split_bytes(static_cast<int64_t>(conv_chunk_samples(batch, oh * ow, k, precision)) * oh * ow, k, ap));
}

int conv_exec(const ConvExec& e, cudaStream_t st) {
  int ap, wp;
  precision_planes(e.precision, &ap, &wp);
  const int oh = (e.h + 2 * e.pad - e.ks) / e.stride + 1;
  const int ow = (e.w + 2 * e.pad - e.ks) / e.stride + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: empty output");
  const int ohw = oh * ow, k = e.ic * e.ks * e.ks;
  if (e.in_up && !conv_uses_shifted(e.ic, e.ks, e.stride, e.pad)) return fail(MIMIR_B200_E_INVALID, "Conv2d: an upsampled input needs the shifted-GEMM path");
  if (e.w_f32 != nullptr && e.pre_groups == 0 && !e.in_up && conv_small_oc_supported(e.oc, e.ks, e.stride, e.pad, e.h, e.w, e.batch, e.activation))
    return launch_conv_small_oc(e.x, e.w_f32, e.y, e.residual, e.batch, e.ic, e.oc, e.h, e.w, e.ks, e.pad, e.activation, st);
  if (conv_uses_shifted(e.ic, e.ks, e.stride, e.pad)) {
    // NCHW fp32 -> zero-padded NHWC planes, then one GEMM that walks the taps as shifted row offsets
    const long long rows = static_cast<long long>(e.batch) * (e.h + 2 * e.pad) * (e.w + 2 * e.pad);
    if (rows > 0x7fffffffLL) return fail(MIMIR_B200_E_UNSUPPORTED, "Conv2d: batch too large for one launch");
    PreNorm pre;
    const size_t planes_bytes = align256(static_cast<size_t>(ap) * rows * e.ic * sizeof(__nv_bfloat16));
    if (e.pre_groups > 0) {
      // statistics live behind the operand planes in the workspace (unless the producer's epilogue delivered them)
      float* stats = reinterpret_cast<float*>(static_cast<uint8_t*>(e.ws) + planes_bytes);
      // (of an upsampled input: over the source image, whose values are the same ones four times)
      if (e.pre_stats == nullptr)
        MB_TRY(launch_groupnorm_stats(e.x, stats, e.batch, e.ic, e.in_up ? (e.h >> 1) * (e.w >> 1) : e.h * e.w, e.pre_groups, e.pre_eps, st));
      pre.stats = e.pre_stats ? e.pre_stats : stats; pre.gamma = e.pre_gamma; pre.beta = e.pre_gamma ? e.pre_beta : nullptr; pre.groups = e.pre_groups; pre.act = e.pre_act;
    }
    MB_TRY(launch_nchw_to_padded_nhwc_split(e.x, static_cast<__nv_bfloat16*>(e.ws), e.batch, e.ic, e.h, e.w, e.pad, ap, st, pre, e.in_up));
    GemmArgs g;
    g.a = static_cast<const __nv_bfloat16*>(e.ws);
    g.w = e.w_split;
    g.a_planes = ap; g.w_planes = wp; g.w_scale = e.w_scale;
    g.m = static_cast<int>(rows); g.n = e.oc; g.k = k;
    g.activation = e.activation;
    g.out_f32 = e.y;
    g.residual = e.residual;
    g.ldo = e.oc;
    g.conv_ks = e.ks; g.conv_c = e.ic; g.conv_pad = e.pad; g.conv_h = e.h; g.conv_w = e.w;
    if (e.gn_stats_out != nullptr) {
      g.gn_part = reinterpret_cast<float*>(static_cast<uint8_t*>(e.ws) + planes_bytes + (e.pre_groups > 0 ? conv_prenorm_bytes(e.batch, e.pre_groups) : 0));
      g.gn_cpg = e.oc / e.gn_groups;
      MB_TRY(launch_gemm(g, st));
      return launch_gn_stats_from_partials(g.gn_part, e.gn_stats_out, e.batch, e.gn_groups, g.gn_cpg, rows, e.oc,
                                           (e.h + 2 * e.pad) * (e.w + 2 * e.pad), e.gn_eps, st);
    }
    return launch_gemm(g, st);
  }
  const int chunk = conv_chunk_samples(e.batch, ohw, k, e.precision);
  for (int b0 = 0; b0 < e.batch; b0 += chunk) {
    const int bc = (e.batch - b0 < chunk) ? (e.batch - b0) : chunk;
    MB_TRY(launch_im2col_split(e.x + static_cast<size_t>(b0) * e.ic * e.h * e.w, static_cast<__nv_bfloat16*>(e.ws), bc, e.ic,
                               e.h, e.w, e.ks, e.stride, e.pad, oh, ow, ap, st));
    GemmArgs g;
    g.a = static_cast<const __nv_bfloat16*>(e.ws);
    g.w = e.w_split;
    g.a_planes = ap; g.w_planes = wp; g.w_scale = e.w_scale;
    g.m = bc * ohw; g.n = e.oc; g.k = k;
    g.activation = e.activation;
    g.out_f32 = e.y + static_cast<size_t>(b0) * e.oc * ohw;
    g.residual = e.residual ? e.residual + static_cast<size_t>(b0) * e.oc * ohw : nullptr;
    g.out_nchw_hw = ohw;
    g.ldo = e.oc;
    MB_TRY(launch_gemm(g, st));
  }
  return MIMIR_B200_OK;
}

}  // namespace mb

// ---------------------------------------------------------------------------------------------
// extern "C": life cycle, guard, per-op entry points
// ---------------------------------------------------------------------------------------------
namespace {

using namespace mb;

std::mutex g_init_mu;

}  // namespace

extern "C" {

int mimir_b200_abi_version(void) { return MIMIR_B200_ABI_VERSION; }
const char* mimir_b200_last_error(void) { return mb::last_error().c_str(); }

int mimir_b200_init(int device, size_t hbm_budget_bytes) {
  std::lock_guard<std::mutex> lk(g_init_mu);
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count <= 0)
    return fail(MIMIR_B200_E_CUDA, "no CUDA device: %s (this backend has no CPU fallback)", cudaGetErrorString(e));
  if (device < 0 || device >= count || device >= MAX_DEVICES)
    return fail(MIMIR_B200_E_INVALID, "device %d out of range (0..%d)", device, (count < MAX_DEVICES ? count : MAX_DEVICES) - 1);
  // the device becomes current on the calling thread: per-op calls and model_create of this thread run on it
  MB_CUDA(cudaSetDevice(device));
  Context& c = ctx_of(device);
  if (c.initialised) {
    if (hbm_budget_bytes) c.guard.limit = hbm_budget_bytes;
    return MIMIR_B200_OK;
  }
  cudaDeviceProp prop;
  MB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(MIMIR_B200_E_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                prop.minor);
  c.device = device;
  c.sm_count = prop.multiProcessorCount;
  size_t free_b = 0, total_b = 0;
  MB_CUDA(cudaMemGetInfo(&free_b, &total_b));
  {
    std::lock_guard<std::mutex> gl(c.guard.mu);
    // a limit set through guard_set_limit before init (selection by environment) is kept
    if (hbm_budget_bytes) c.guard.limit = hbm_budget_bytes;
    else if (c.guard.limit == 0) c.guard.limit = static_cast<size_t>(total_b * 0.9);
  }
  c.initialised = true;
  void* w = nullptr;
  int s = dev_alloc(&w, 256, "error_word");
  if (s != MIMIR_B200_OK) {
    c.initialised = false;
    return s;
  }
  c.dev_error_word = static_cast<int*>(w);
  MB_CUDA(cudaMemset(c.dev_error_word, 0, 256));
  return MIMIR_B200_OK;
}

/* Selection by environment, with the reference's own conventions for its accelerator switches (Model.cpp:704-722, used at
 * Model.cpp:5110-5112): a flag is true for any non-empty value other than "0", an integer that does not parse keeps its
 * default.  Default off. */
int mimir_b200_env_selection(int* enabled, int* device, size_t* hbm_budget_bytes) {
  auto flag = [](const char* name) {
    const char* v = getenv(name);
    if (!v || v[0] == '\0') return false;
    return !(v[0] == '0' && v[1] == '\0');
  };
  auto integer = [](const char* name, long long dflt) {
    const char* v = getenv(name);
    if (!v || v[0] == '\0') return dflt;
    char* end = nullptr;
    const long long r = strtoll(v, &end, 10);
    return (end == v) ? dflt : r;
  };
  if (enabled) *enabled = flag("MIMIR_B200") ? 1 : 0;
  const long long dev = integer("MIMIR_B200_DEVICE", 0);
  if (device) *device = static_cast<int>(dev < 0 ? 0 : dev);
  const long long mb = integer("MIMIR_B200_HBM_BUDGET_MB", 0);
  if (hbm_budget_bytes) *hbm_budget_bytes = mb > 0 ? static_cast<size_t>(mb) << 20 : 0;
  return MIMIR_B200_OK;
}

int mimir_b200_init_from_env(int* enabled) {
  int on = 0, dev = 0;
  size_t budget = 0;
  mimir_b200_env_selection(&on, &dev, &budget);
  if (enabled) *enabled = 0;
  if (!on) return MIMIR_B200_OK;  // not selected: nothing is touched, the caller stays on its own path
  MB_TRY(mimir_b200_init(dev, budget));
  if (enabled) *enabled = 1;
  return MIMIR_B200_OK;
}

int mimir_b200_current_device(int* device) {
  if (!device) return fail(MIMIR_B200_E_INVALID, "current_device: null argument");
  MB_REQUIRE_INIT();
  *device = ctx().device;
  return MIMIR_B200_OK;
}

/* The guard verbs are host logic: they work before mimir_b200_init (on the calling thread's current device, device 0
 * on a machine without one), so a limit can be in place before the first allocation. */
int mimir_b200_guard_set_limit(size_t bytes) {
  std::lock_guard<std::mutex> lk(ctx().guard.mu);
  ctx().guard.limit = bytes;
  return MIMIR_B200_OK;
}
int mimir_b200_guard_request(size_t bytes, const char* tag) {
  if (const int why = ctx().guard.request_why(bytes))
    return fail(MIMIR_B200_E_OOM_BUDGET, "HBM budget refused %zu bytes for %s (%s)", bytes, tag ? tag : "?",
                why == 2 ? "allocations are blocked" : why == 3 ? "allocations are frozen" : "over the limit");
  return MIMIR_B200_OK;
}
int mimir_b200_guard_release(size_t bytes) {
  ctx().guard.release(bytes);
  return MIMIR_B200_OK;
}
int mimir_b200_guard_stats(size_t* limit, size_t* current, size_t* peak) {
  std::lock_guard<std::mutex> lk(ctx().guard.mu);
  if (limit) *limit = ctx().guard.limit;
  if (current) *current = ctx().guard.current;
  if (peak) *peak = ctx().guard.peak;
  return MIMIR_B200_OK;
}
int mimir_b200_guard_block(int block) {
  std::lock_guard<std::mutex> lk(ctx().guard.mu);
  ctx().guard.blocked = block != 0;
  return MIMIR_B200_OK;
}
int mimir_b200_guard_freeze(int freeze) {
  std::lock_guard<std::mutex> lk(ctx().guard.mu);
  ctx().guard.frozen = freeze != 0;
  return MIMIR_B200_OK;
}
int mimir_b200_guard_reset(void) {
  ctx().guard.reset();
  return MIMIR_B200_OK;
}
int mimir_b200_guard_state(int* blocked, int* frozen, size_t* blocked_attempts, size_t* frozen_attempts) {
  std::lock_guard<std::mutex> lk(ctx().guard.mu);
  if (blocked) *blocked = ctx().guard.blocked ? 1 : 0;
  if (frozen) *frozen = ctx().guard.frozen ? 1 : 0;
  if (blocked_attempts) *blocked_attempts = ctx().guard.blocked_attempts;
  if (frozen_attempts) *frozen_attempts = ctx().guard.frozen_attempts;
  return MIMIR_B200_OK;
}

/* RuntimeAllocator on the device (RuntimeAllocator.hpp:176-310). */
static int owned_alloc(size_t bytes, const char* tag, void** out) {
  if (!out) return fail(MIMIR_B200_E_INVALID, "allocator: null result pointer");
  *out = nullptr;
  MB_REQUIRE_INIT();
  if (bytes == 0) return fail(MIMIR_B200_E_INVALID, "allocator: zero bytes asked for %s", tag);
  OwnedBuffers& ob = ctx().owned;
  {
    // the optional local cap comes before the guard, as in allocate_tensor / allocate_buffer
    std::lock_guard<std::mutex> lk(ob.mu);
    size_t current = 0;
    mimir_b200_guard_stats(nullptr, &current, nullptr);
    if (ob.local_cap > 0 && current + bytes > ob.local_cap)
      return fail(MIMIR_B200_E_OOM_BUDGET, "allocator: %zu bytes for %s would exceed the local cap (%zu in use of %zu)", bytes, tag,
                  current, ob.local_cap);
  }
  void* p = nullptr;
  MB_TRY(dev_alloc(&p, bytes, tag));
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    dev_free(p, bytes);
    return fail(MIMIR_B200_E_CUDA, "allocator: clearing %zu bytes for %s failed", bytes, tag);
  }
  std::lock_guard<std::mutex> lk(ob.mu);
  ob.live[p] = OwnedBuffers::Buf{bytes, tag};
  ob.total_allocated += bytes;
  ob.num_allocations += 1;
  *out = p;
  return MIMIR_B200_OK;
}

int mimir_b200_tensor_alloc(const int* shape, int rank, const char* name, float** device_ptr, size_t* bytes_out) {
  if (!shape || rank <= 0 || !device_ptr) return fail(MIMIR_B200_E_INVALID, "tensor_alloc: bad arguments");
  size_t numel = 1;
  for (int i = 0; i < rank; ++i) {
    if (shape[i] <= 0) return fail(MIMIR_B200_E_INVALID, "tensor_alloc: extent %d of %s is %d", i, name ? name : "?", shape[i]);
    if (numel > (static_cast<size_t>(1) << 60) / static_cast<size_t>(shape[i]))
      return fail(MIMIR_B200_E_INVALID, "tensor_alloc: element count of %s overflows", name ? name : "?");
    numel *= static_cast<size_t>(shape[i]);
  }
  void* p = nullptr;
  MB_TRY(owned_alloc(numel * sizeof(float), name ? name : "", &p));
  *device_ptr = static_cast<float*>(p);
  if (bytes_out) *bytes_out = numel * sizeof(float);
  return MIMIR_B200_OK;
}
int mimir_b200_buffer_alloc(size_t bytes, const char* tag, void** device_ptr) { return owned_alloc(bytes, tag ? tag : "", device_ptr); }
int mimir_b200_buffer_free(void* device_ptr) {
  if (!device_ptr) return MIMIR_B200_OK;
  OwnedBuffers& ob = ctx().owned;
  std::lock_guard<std::mutex> lk(ob.mu);
  auto it = ob.live.find(device_ptr);
  if (it == ob.live.end()) return fail(MIMIR_B200_E_INVALID, "buffer_free: %p was not handed out by the allocator (or sits in the pool)", device_ptr);
  dev_free(device_ptr, it->second.bytes);
  ob.live.erase(it);
  return MIMIR_B200_OK;
}
int mimir_b200_scratchpad_get(size_t min_bytes, const char* tag, void** device_ptr, size_t* bytes_out) {
  if (!device_ptr) return fail(MIMIR_B200_E_INVALID, "scratchpad_get: null result pointer");
  const std::string t = tag ? tag : "scratchpad";
  OwnedBuffers& ob = ctx().owned;
  {
    std::lock_guard<std::mutex> lk(ob.mu);
    auto it = ob.pool.find(t);
    if (it != ob.pool.end() && it->second.second >= min_bytes) {
      *device_ptr = it->second.first;
      if (bytes_out) *bytes_out = it->second.second;
      ob.live[it->second.first] = OwnedBuffers::Buf{it->second.second, t};
      ob.pool.erase(it);
      return MIMIR_B200_OK;
    }
  }
  MB_TRY(owned_alloc(min_bytes, t.c_str(), device_ptr));
  if (bytes_out) *bytes_out = min_bytes;
  return MIMIR_B200_OK;
}
int mimir_b200_scratchpad_return(void* device_ptr) {
  if (!device_ptr) return MIMIR_B200_OK;
  OwnedBuffers& ob = ctx().owned;
  std::lock_guard<std::mutex> lk(ob.mu);
  auto it = ob.live.find(device_ptr);
  if (it == ob.live.end()) return fail(MIMIR_B200_E_INVALID, "scratchpad_return: %p was not handed out by the allocator", device_ptr);
  if (ob.pool.count(it->second.tag)) dev_free(device_ptr, it->second.bytes);  // one pooled buffer per tag
  else ob.pool[it->second.tag] = std::make_pair(device_ptr, it->second.bytes);
  ob.live.erase(it);
  return MIMIR_B200_OK;
}
int mimir_b200_allocator_set_local_cap(size_t bytes) {
  std::lock_guard<std::mutex> lk(ctx().owned.mu);
  ctx().owned.local_cap = bytes;
  return MIMIR_B200_OK;
}
int mimir_b200_allocator_stats(size_t* total_allocated, size_t* num_allocations, size_t* peak, size_t* current) {
  {
    std::lock_guard<std::mutex> lk(ctx().owned.mu);
    if (total_allocated) *total_allocated = ctx().owned.total_allocated;
    if (num_allocations) *num_allocations = ctx().owned.num_allocations;
  }
  return mimir_b200_guard_stats(nullptr, current, peak);
}
int mimir_b200_allocator_reset_stats(void) {
  std::lock_guard<std::mutex> lk(ctx().owned.mu);
  ctx().owned.total_allocated = 0;
  ctx().owned.num_allocations = 0;
  return MIMIR_B200_OK;
}
int mimir_b200_allocator_check_no_leaks(int* ok) {
  if (!ok) return fail(MIMIR_B200_E_INVALID, "check_no_leaks: null result pointer");
  size_t current = 0;
  mimir_b200_guard_stats(nullptr, &current, nullptr);
  *ok = (current / (1024 * 1024)) < 10 ? 1 : 0;
  return MIMIR_B200_OK;
}

int mimir_b200_linear_forward_ex(const float* input, const float* weights, const float* bias_or_null, float* output,
                                 int batch, int in_f, int out_f, int precision, int activation) {
  MB_REQUIRE_INIT();
  if (!input || !weights || !output || batch <= 0 || in_f <= 0) return fail(MIMIR_B200_E_INVALID, "Linear: bad arguments");
  if (out_f <= 0) return fail(MIMIR_B200_E_INVALID, "Linear: out_features not set");
  Temps t;
  LinearExec e;
  e.rows = batch; e.in_f = in_f; e.out_f = out_f; e.precision = precision; e.activation = activation;
  MB_TRY(t.upload(&e.x_f32, input, static_cast<size_t>(batch) * in_f, "linear.x"));
  MB_TRY(t.upload(&e.w_f32, weights, static_cast<size_t>(out_f) * in_f, "linear.w"));
  if (bias_or_null) MB_TRY(t.upload(&e.bias, bias_or_null, out_f, "linear.b"));
  MB_TRY(t.out(&e.y_f32, static_cast<size_t>(batch) * out_f, "linear.y"));
  e.ws_bytes = linear_ws_bytes(batch, in_f, out_f, precision, false);
  MB_TRY(t.alloc(&e.ws, e.ws_bytes, "linear.ws"));
  if (!linear_uses_skinny(batch, precision)) {
    int ap, wp;
    precision_planes(precision, &ap, &wp);
    void* wsplit;
    MB_TRY(t.alloc(&wsplit, split_bytes(out_f, in_f, wp), "linear.wsplit"));
    MB_TRY(weight_plane_scale(e.w_f32, static_cast<size_t>(out_f) * in_f, nullptr, &e.w_scale));
    MB_TRY(launch_split(e.w_f32, static_cast<__nv_bfloat16*>(wsplit), out_f, in_f, wp, nullptr, e.w_scale));
    e.w_split = static_cast<const __nv_bfloat16*>(wsplit);
  }
  MB_TRY(linear_exec(e, nullptr));
  return finish_download(output, e.y_f32, static_cast<size_t>(batch) * out_f);
}

int mimir_b200_linear_forward(const float* input, const float* weights, const float* bias_or_null, float* output, int batch,
                              int in_f, int out_f) {
  return mimir_b200_linear_forward_ex(input, weights, bias_or_null, output, batch, in_f, out_f, MIMIR_B200_PREC_BF16X2, -1);
}

int mimir_b200_matmul(const float* A, const float* B, float* C, int M, int K, int N) {
  MB_REQUIRE_INIT();
  if (!A || !B || !C || M <= 0 || K <= 0 || N <= 0) return fail(MIMIR_B200_E_INVALID, "MatMul: dimension mismatch");
  Temps t;
  const float *a, *b;
  float* c;
  MB_TRY(t.upload(&a, A, static_cast<size_t>(M) * K, "matmul.a"));
  MB_TRY(t.upload(&b, B, static_cast<size_t>(K) * N, "matmul.b"));
  MB_TRY(t.out(&c, static_cast<size_t>(M) * N, "matmul.c"));
  void *as, *bs;
  MB_TRY(t.alloc(&as, split_bytes(M, K, 2), "matmul.as"));
  MB_TRY(t.alloc(&bs, split_bytes(N, K, 2), "matmul.bs"));
  MB_TRY(launch_split(a, static_cast<__nv_bfloat16*>(as), M, K, 2, nullptr));
  GemmArgs g;
  MB_TRY(weight_plane_scale(b, static_cast<size_t>(K) * N, nullptr, &g.w_scale));
  MB_TRY(launch_split_transposed(b, static_cast<__nv_bfloat16*>(bs), K, N, 2, nullptr, g.w_scale));
  g.a = static_cast<const __nv_bfloat16*>(as);
  g.w = static_cast<const __nv_bfloat16*>(bs);
  g.m = M; g.n = N; g.k = K; g.out_f32 = c; g.ldo = N;
  MB_TRY(launch_gemm(g, nullptr));
  return finish_download(C, c, static_cast<size_t>(M) * N);
}

int mimir_b200_attention(const float* x, const float* wqkv_wout, float* y, int batch, int seq, int embed, int heads,
                         int causal) {
  MB_REQUIRE_INIT();
  if (!x || !wqkv_wout || !y || batch <= 0 || seq <= 0 || embed <= 0 || heads <= 0)
    return fail(MIMIR_B200_E_INVALID, "Attention: bad arguments");
  if (embed % heads != 0) return fail(MIMIR_B200_E_INVALID, "SelfAttention: embed_dim must be divisible by num_heads");
  Temps t;
  const size_t E = embed, rows = static_cast<size_t>(batch) * seq;
  AttentionExec e;
  e.batch = batch; e.seq = seq; e.embed = embed; e.heads = heads; e.causal = causal;
  const float* w;
  MB_TRY(t.upload(&e.x, x, rows * E, "attn.x"));
  MB_TRY(t.upload(&w, wqkv_wout, 4 * E * E, "attn.w"));
  MB_TRY(t.out(&e.y, rows * E, "attn.y"));
  void *wq, *wo;
  MB_TRY(t.alloc(&wq, split_bytes(3 * embed, embed, 2), "attn.wqkv"));
  MB_TRY(t.alloc(&wo, split_bytes(embed, embed, 2), "attn.wout"));
  MB_TRY(weight_plane_scale(w, 4 * E * E, nullptr, &e.w_scale));
  MB_TRY(launch_split_transposed(w, static_cast<__nv_bfloat16*>(wq), embed, 3 * embed, 2, nullptr, e.w_scale));
  MB_TRY(launch_split_transposed(w + 3 * E * E, static_cast<__nv_bfloat16*>(wo), embed, embed, 2, nullptr, e.w_scale));
  e.wqkv_split = static_cast<const __nv_bfloat16*>(wq);
  e.wout_split = static_cast<const __nv_bfloat16*>(wo);
  MB_TRY(t.alloc(&e.ws, attention_ws_bytes(batch, seq, embed, heads, e.precision), "attn.ws"));
  MB_TRY(attention_exec(e, nullptr));
  return finish_download(y, e.y, rows * E);
}

int mimir_b200_conv2d(const float* x, const float* w, float* y, int batch, int ic, int oc, int h, int wd, int k, int stride,
                      int pad, int relu) {
  MB_REQUIRE_INIT();
  if (!x || !w || !y || batch <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: bad arguments");
  if (ic <= 0 || oc <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: in_channels and out_channels must be set");
  if (k <= 0 || stride <= 0 || pad < 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: kernel_size must be set");
  const int oh = (h + 2 * pad - k) / stride + 1, ow = (wd + 2 * pad - k) / stride + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: empty output");
  Temps t;
  ConvExec e;
  e.batch = batch; e.ic = ic; e.oc = oc; e.h = h; e.w = wd; e.ks = k; e.stride = stride; e.pad = pad;
  e.activation = relu ? MIMIR_B200_ELT_RELU : -1;
  const float* wdv;
  MB_TRY(t.upload(&e.x, x, static_cast<size_t>(batch) * ic * h * wd, "conv.x"));
  MB_TRY(t.upload(&wdv, w, static_cast<size_t>(oc) * ic * k * k, "conv.w"));
  MB_TRY(t.out(&e.y, static_cast<size_t>(batch) * oc * oh * ow, "conv.y"));
  void* ws;
  MB_TRY(t.alloc(&ws, split_bytes(oc, ic * k * k, 2), "conv.wsplit"));
  e.w_f32 = wdv;
  MB_TRY(weight_plane_scale(wdv, static_cast<size_t>(oc) * ic * k * k, nullptr, &e.w_scale));
  if (conv_uses_shifted(ic, k, stride, pad)) MB_TRY(launch_conv_weight_planes(wdv, static_cast<__nv_bfloat16*>(ws), oc, ic, k, 2, nullptr, e.w_scale));
  else MB_TRY(launch_split(wdv, static_cast<__nv_bfloat16*>(ws), oc, ic * k * k, 2, nullptr, e.w_scale));
  e.w_split = static_cast<const __nv_bfloat16*>(ws);
  MB_TRY(t.alloc(&e.ws, conv_ws_bytes(batch, ic, h, wd, k, stride, pad, e.precision), "conv.ws"));
  MB_TRY(conv_exec(e, nullptr));
  return finish_download(y, e.y, static_cast<size_t>(batch) * oc * oh * ow);
}

int mimir_b200_layernorm(const float* x, const float* gamma, const float* beta, float* y, long long rows, int n, float eps) {
  MB_REQUIRE_INIT();
  if (!x || !y || rows <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "LayerNorm: invalid normalized_size");
  Temps t;
  const float *dx, *dg = nullptr, *db = nullptr;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(rows) * n, "ln.x"));
  if (gamma) MB_TRY(t.upload(&dg, gamma, n, "ln.g"));
  if (gamma && beta) MB_TRY(t.upload(&db, beta, n, "ln.b"));
  MB_TRY(t.out(&dy, static_cast<size_t>(rows) * n, "ln.y"));
  MB_TRY(launch_layernorm(dx, dg, db, dy, rows, n, eps, nullptr));
  return finish_download(y, dy, static_cast<size_t>(rows) * n);
}

int mimir_b200_rmsnorm(const float* x, const float* gamma, long long n_gamma, float* y, int batch, long long n, float eps) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "RMSNorm: empty input");
  Temps t;
  const float *dx, *dg = nullptr;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * n, "rms.x"));
  if (gamma && n_gamma > 0) MB_TRY(t.upload(&dg, gamma, static_cast<size_t>(n_gamma), "rms.g"));
  MB_TRY(t.out(&dy, static_cast<size_t>(batch) * n, "rms.y"));
  MB_TRY(launch_rmsnorm(dx, dg, dg ? n_gamma : 0, dy, batch, n, eps, nullptr));
  return finish_download(y, dy, static_cast<size_t>(batch) * n);
}

int mimir_b200_groupnorm(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels, int h,
                         int w, int groups, float eps, int act) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || channels <= 0 || h <= 0 || w <= 0) return fail(MIMIR_B200_E_INVALID, "GroupNorm: bad arguments");
  Temps t;
  const size_t n = static_cast<size_t>(batch) * channels * h * w;
  const float *dx, *dg = nullptr, *db = nullptr;
  float* dy;
  MB_TRY(t.upload(&dx, x, n, "gn.x"));
  if (gamma) MB_TRY(t.upload(&dg, gamma, channels, "gn.g"));
  if (gamma && beta) MB_TRY(t.upload(&db, beta, channels, "gn.b"));
  MB_TRY(t.out(&dy, n, "gn.y"));
  MB_TRY(launch_groupnorm(dx, dg, db, dy, batch, channels, h * w, groups, eps, act, nullptr, nullptr));
  return finish_download(y, dy, n);
}

int mimir_b200_softmax(const float* x, float* y, int batch, long long n, int log_softmax) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "Softmax: empty input");
  Temps t;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * n, "sm.x"));
  MB_TRY(t.out(&dy, static_cast<size_t>(batch) * n, "sm.y"));
  MB_TRY(launch_softmax(dx, dy, batch, n, log_softmax, nullptr));
  return finish_download(y, dy, static_cast<size_t>(batch) * n);
}

int mimir_b200_eltwise(int op, const float* a, const float* b, float* y, int batch, long long n, long long nb) {
  MB_REQUIRE_INIT();
  if (!a || !y || batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "eltwise: inputs must be non-empty");
  Temps t;
  const float *da, *db = nullptr;
  float* dy;
  MB_TRY(t.upload(&da, a, static_cast<size_t>(batch) * n, "elt.a"));
  if (b && nb > 0) MB_TRY(t.upload(&db, b, static_cast<size_t>(batch) * nb, "elt.b"));
  MB_TRY(t.out(&dy, static_cast<size_t>(batch) * n, "elt.y"));
  MB_TRY(launch_eltwise(op, da, db, dy, batch, n, nb, nullptr));
  return finish_download(y, dy, static_cast<size_t>(batch) * n);
}

int mimir_b200_embedding(const float* ids_f32, const int32_t* ids_i32, const float* table, float* y, long long n_ids,
                         int vocab, int dim, int padding_idx) {
  MB_REQUIRE_INIT();
  if (!table || !y || n_ids <= 0 || vocab <= 0 || dim <= 0) return fail(MIMIR_B200_E_INVALID, "Embedding: bad arguments");
  if ((ids_f32 == nullptr) == (ids_i32 == nullptr)) return fail(MIMIR_B200_E_INVALID, "Embedding: give exactly one id array");
  Temps t;
  const float *dt, *df = nullptr;
  const int32_t* di = nullptr;
  float* dy;
  MB_TRY(t.upload(&dt, table, static_cast<size_t>(vocab) * dim, "emb.table"));
  if (ids_f32) {
    MB_TRY(t.upload(&df, ids_f32, static_cast<size_t>(n_ids), "emb.ids"));
  } else {
    void* p;
    MB_TRY(t.alloc(&p, static_cast<size_t>(n_ids) * 4, "emb.ids"));
    MB_CUDA(cudaMemcpy(p, ids_i32, static_cast<size_t>(n_ids) * 4, cudaMemcpyHostToDevice));
    di = static_cast<const int32_t*>(p);
  }
  MB_TRY(t.out(&dy, static_cast<size_t>(n_ids) * dim, "emb.y"));
  MB_TRY(launch_embedding(df, di, dt, dy, n_ids, vocab, dim, padding_idx, nullptr));
  return finish_download(y, dy, static_cast<size_t>(n_ids) * dim);
}

int mimir_b200_upsample_nearest(const float* x, float* y, int batch, int channels, int in_h, int in_w, int scale_h,
                                int scale_w) {
  MB_REQUIRE_INIT();
  if (!x || !y) return fail(MIMIR_B200_E_INVALID, "UpsampleNearest: bad arguments");
  Temps t;
  const size_t n = static_cast<size_t>(batch) * channels * in_h * in_w;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, n, "up.x"));
  MB_TRY(t.out(&dy, n * scale_h * scale_w, "up.y"));
  MB_TRY(launch_upsample_nearest(dx, dy, batch, channels, in_h, in_w, scale_h, scale_w, nullptr));
  return finish_download(y, dy, n * scale_h * scale_w);
}

int mimir_b200_permute(const float* x, float* y, int batch, int ndim, const int* shape, const int* dims) {
  MB_REQUIRE_INIT();
  if (!x || !y || !shape || !dims || ndim <= 0 || ndim > MIMIR_B200_MAX_DIMS)
    return fail(MIMIR_B200_E_INVALID, "Permute: dims and shape cannot be empty");
  size_t per = 1;
  for (int i = 0; i < ndim; ++i) per *= static_cast<size_t>(shape[i] > 0 ? shape[i] : 0);
  if (per == 0) return fail(MIMIR_B200_E_INVALID, "Permute: bad shape");
  Temps t;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, per * batch, "perm.x"));
  MB_TRY(t.out(&dy, per * batch, "perm.y"));
  MB_TRY(launch_permute(dx, dy, batch, ndim, shape, dims, nullptr));
  return finish_download(y, dy, per * batch);
}

int mimir_b200_token_mean_pool(const float* x, float* y, int batch, int seq, int dim) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || seq <= 0 || dim <= 0)
    return fail(MIMIR_B200_E_INVALID, "TokenMeanPool: seq_len and embed_dim must be set");
  Temps t;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * seq * dim, "tmp.x"));
  MB_TRY(t.out(&dy, static_cast<size_t>(batch) * dim, "tmp.y"));
  MB_TRY(launch_token_mean_pool(dx, dy, batch, seq, dim, nullptr));
  return finish_download(y, dy, static_cast<size_t>(batch) * dim);
}

int mimir_b200_global_avgpool(const float* x, float* y, int batch, int channels, int h, int w) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || channels <= 0 || h <= 0 || w <= 0) return fail(MIMIR_B200_E_INVALID, "GlobalAvgPool: bad arguments");
  Temps t;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * channels * h * w, "gap.x"));
  MB_TRY(t.out(&dy, static_cast<size_t>(batch) * channels, "gap.y"));
  MB_TRY(launch_global_avgpool(dx, dy, batch, channels, h * w, nullptr));
  return finish_download(y, dy, static_cast<size_t>(batch) * channels);
}

// ---- device-pointer forms -------------------------------------------------------------------
int mimir_b200_dev_layernorm(const float* x, const float* gamma, const float* beta, float* y, long long rows, int n,
                             float eps, void* stream) {
  MB_REQUIRE_INIT();
  return launch_layernorm(x, gamma, beta, y, rows, n, eps, static_cast<cudaStream_t>(stream));
}
int mimir_b200_dev_rmsnorm(const float* x, const float* gamma, long long n_gamma, float* y, int batch, long long n, float eps,
                           void* stream) {
  MB_REQUIRE_INIT();
  return launch_rmsnorm(x, gamma, n_gamma, y, batch, n, eps, static_cast<cudaStream_t>(stream));
}
int mimir_b200_dev_groupnorm(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels, int h,
                             int w, int groups, float eps, int act, void* stream) {
  MB_REQUIRE_INIT();
  return launch_groupnorm(x, gamma, beta, y, batch, channels, h * w, groups, eps, act, nullptr, static_cast<cudaStream_t>(stream));
}
int mimir_b200_dev_softmax(const float* x, float* y, int batch, long long n, int log_softmax, void* stream) {
  MB_REQUIRE_INIT();
  return launch_softmax(x, y, batch, n, log_softmax, static_cast<cudaStream_t>(stream));
}
int mimir_b200_dev_eltwise(int op, const float* a, const float* b, float* y, int batch, long long n, long long nb,
                           void* stream) {
  MB_REQUIRE_INIT();
  return launch_eltwise(op, a, b, y, batch, n, nb, static_cast<cudaStream_t>(stream));
}
int mimir_b200_argmax_rows_device(const float* x_dev, int32_t* ids_dev, long long rows, int n, void* stream) {
  MB_REQUIRE_INIT();
  return launch_argmax_rows(x_dev, ids_dev, rows, n, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
