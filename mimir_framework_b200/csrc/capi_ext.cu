// capi_ext.cu — host-pointer entry points of the remaining switch cases (cross attention and the
// gather-style ops of spatial.cu), plus the cross-attention op sequence shared with the graph executor.
#include "host_call.h"

namespace mb {

// Workspace: split(query) | split(key_value) | Q fp32 | KV fp32 | attended fp32
size_t cross_attention_ws_bytes(int batch, int q_len, int kv_len, int embed, int precision) {
  int ap, wp;
  precision_planes(precision, &ap, &wp);
  const size_t qr = static_cast<size_t>(batch) * q_len, kr = static_cast<size_t>(batch) * kv_len;
  return align256(split_bytes(static_cast<int64_t>(qr), embed, ap)) + align256(split_bytes(static_cast<int64_t>(kr), embed, ap)) +
         align256(qr * embed * 4) + align256(kr * 2 * embed * 4) + align256(qr * embed * 4);
}

int cross_attention_exec(const CrossAttentionExec& e, cudaStream_t st) {
  int ap, wp;
  precision_planes(e.precision, &ap, &wp);
  const int qr = e.batch * e.q_len, kr = e.batch * e.kv_len, E = e.embed;
  uint8_t* p = static_cast<uint8_t*>(e.ws);
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(p);
  p += align256(split_bytes(qr, E, ap));
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(p);
  p += align256(split_bytes(kr, E, ap));
  float* q = reinterpret_cast<float*>(p);
  p += align256(static_cast<size_t>(qr) * E * 4);
  float* kv = reinterpret_cast<float*>(p);
  p += align256(static_cast<size_t>(kr) * 2 * E * 4);
  float* att = reinterpret_cast<float*>(p);
  MB_TRY(launch_split(e.q_in, qs, qr, E, ap, st));
  MB_TRY(launch_split(e.kv_in, ks, kr, E, ap, st));
  GemmArgs g;
  g.a = qs; g.w = e.wq_split; g.a_planes = ap; g.w_planes = wp; g.w_scale = e.w_scale;
  g.m = qr; g.n = E; g.k = E; g.out_f32 = q; g.ldo = E;
  MB_TRY(launch_gemm(g, st));
  GemmArgs h;
  h.a = ks; h.w = e.wkv_split; h.a_planes = ap; h.w_planes = wp; h.w_scale = e.w_scale;
  h.m = kr; h.n = 2 * E; h.k = E; h.out_f32 = kv; h.ldo = 2 * E;
  MB_TRY(launch_gemm(h, st));
  AttnView v;
  v.q = q; v.k = kv; v.v = kv + E;
  v.ldq = E; v.ldkv = 2LL * E;
  v.q_len = e.q_len; v.kv_len = e.kv_len;
  MB_TRY(launch_attention_core_view(v, att, e.batch, E, e.heads, e.causal, st));
  MB_TRY(launch_split(att, qs, qr, E, ap, st));  // the query planes are dead by now
  GemmArgs o;
  o.a = qs; o.w = e.wout_split; o.a_planes = ap; o.w_planes = wp; o.w_scale = e.w_scale;
  o.m = qr; o.n = E; o.k = E; o.out_f32 = e.y; o.ldo = E; o.residual = e.residual;
  return launch_gemm(o, st);
}

}  // namespace mb

extern "C" {

using namespace mb;

int mimir_b200_cross_attention(const float* query, const float* key_value, const float* w, float* y, int batch, int q_len,
                               int kv_len, int embed, int heads, int causal) {
  MB_REQUIRE_INIT();
  if (!query || !key_value || !w || !y || batch <= 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: bad arguments");
  if (q_len <= 0 || kv_len <= 0 || embed <= 0 || heads <= 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: invalid dimensions");
  if (embed % heads != 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: embed_dim must be divisible by num_heads");
  Temps t;
  const size_t E = embed, qr = static_cast<size_t>(batch) * q_len, kr = static_cast<size_t>(batch) * kv_len;
  CrossAttentionExec e;
  e.batch = batch; e.q_len = q_len; e.kv_len = kv_len; e.embed = embed; e.heads = heads; e.causal = causal;
  const float* dw;
  MB_TRY(t.upload(&e.q_in, query, qr * E, "xattn.q"));
  MB_TRY(t.upload(&e.kv_in, key_value, kr * E, "xattn.kv"));
  MB_TRY(t.upload(&dw, w, 4 * E * E, "xattn.w"));
  MB_TRY(t.out(&e.y, qr * E, "xattn.y"));
  void *wq, *wkv, *wo;
  MB_TRY(t.alloc(&wq, split_bytes(embed, embed, 2), "xattn.wq"));
  MB_TRY(t.alloc(&wkv, split_bytes(2 * embed, embed, 2), "xattn.wkv"));
  MB_TRY(t.alloc(&wo, split_bytes(embed, embed, 2), "xattn.wout"));
  MB_TRY(weight_plane_scale(dw, 4 * E * E, nullptr, &e.w_scale));
  MB_TRY(launch_split_transposed(dw, static_cast<__nv_bfloat16*>(wq), embed, embed, 2, nullptr, e.w_scale));
  MB_TRY(launch_split_transposed(dw + E * E, static_cast<__nv_bfloat16*>(wkv), embed, 2 * embed, 2, nullptr, e.w_scale));
  MB_TRY(launch_split_transposed(dw + 3 * E * E, static_cast<__nv_bfloat16*>(wo), embed, embed, 2, nullptr, e.w_scale));
  e.wq_split = static_cast<const __nv_bfloat16*>(wq);
  e.wkv_split = static_cast<const __nv_bfloat16*>(wkv);
  e.wout_split = static_cast<const __nv_bfloat16*>(wo);
  MB_TRY(t.alloc(&e.ws, cross_attention_ws_bytes(batch, q_len, kv_len, embed, e.precision), "xattn.ws"));
  MB_TRY(cross_attention_exec(e, nullptr));
  return finish_download(y, e.y, qr * E);
}

int mimir_b200_eltwise_alpha(int op, const float* a, const float* b, float* y, int batch, long long n, long long nb, float alpha) {
  MB_REQUIRE_INIT();
  if (!a || !y || batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "eltwise: inputs must be non-empty");
  Temps t;
  const float *da, *db = nullptr;
  float* dy;
  MB_TRY(t.upload(&da, a, static_cast<size_t>(batch) * n, "elt.a"));
  if (b && nb > 0) MB_TRY(t.upload(&db, b, static_cast<size_t>(batch) * nb, "elt.b"));
  MB_TRY(t.out(&dy, static_cast<size_t>(batch) * n, "elt.y"));
  MB_TRY(launch_eltwise(op, da, db, dy, batch, n, nb, nullptr, alpha));
  return finish_download(y, dy, static_cast<size_t>(batch) * n);
}

int mimir_b200_depthwise_conv2d(const float* x, const float* w, const float* bias, float* y, int batch, int channels, int h, int wd,
                                int k, int stride, int pad) {
  MB_REQUIRE_INIT();
  if (!x || !w || !y || batch <= 0 || channels <= 0 || h <= 0 || wd <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return fail(MIMIR_B200_E_INVALID, "DepthwiseConv2d: bad arguments");
  const int oh = (h + 2 * pad - k) / stride + 1, ow = (wd + 2 * pad - k) / stride + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "DepthwiseConv2d: empty output");
  Temps t;
  const float *dx, *dw, *db = nullptr;
  float* dy;
  const size_t nw = static_cast<size_t>(channels) * k * k;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * channels * h * wd, "dw.x"));
  MB_TRY(t.upload(&dw, w, nw, "dw.w"));
  if (bias) MB_TRY(t.upload(&db, bias, channels, "dw.b"));
  const size_t ny = static_cast<size_t>(batch) * channels * oh * ow;
  MB_TRY(t.out(&dy, ny, "dw.y"));
  MB_TRY(launch_depthwise_conv2d(dx, dw, db, dy, batch, channels, h, wd, k, stride, pad, static_cast<int64_t>(nw), nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_conv1d(const float* x, const float* w, const float* bias, float* y, int batch, int ic, int oc, int len, int k, int stride,
                      int pad) {
  MB_REQUIRE_INIT();
  if (!x || !w || !y || batch <= 0 || ic <= 0 || oc <= 0 || len <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return fail(MIMIR_B200_E_INVALID, "Conv1d: bad arguments");
  const int olen = (len + 2 * pad - k) / stride + 1;
  if (olen <= 0) return fail(MIMIR_B200_E_INVALID, "Conv1d: empty output");
  Temps t;
  const float *dx, *dw, *db = nullptr;
  float* dy;
  const size_t nw = static_cast<size_t>(oc) * ic * k;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * ic * len, "c1.x"));
  MB_TRY(t.upload(&dw, w, nw, "c1.w"));
  if (bias) MB_TRY(t.upload(&db, bias, oc, "c1.b"));
  const size_t ny = static_cast<size_t>(batch) * oc * olen;
  MB_TRY(t.out(&dy, ny, "c1.y"));
  MB_TRY(launch_conv1d(dx, dw, db, dy, batch, ic, oc, len, k, stride, pad, static_cast<int64_t>(nw), nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_conv_transpose2d(const float* x, const float* w, float* y, int batch, int ic, int oc, int h, int wd, int k, int stride,
                                int pad, int relu) {
  MB_REQUIRE_INIT();
  if (!x || !w || !y || batch <= 0 || ic <= 0 || oc <= 0 || h <= 0 || wd <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return fail(MIMIR_B200_E_INVALID, "ConvTranspose2d: bad arguments");
  const int oh = (h - 1) * stride - 2 * pad + k, ow = (wd - 1) * stride - 2 * pad + k;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "ConvTranspose2d: empty output");
  Temps t;
  const float *dx, *dw;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * ic * h * wd, "ct.x"));
  MB_TRY(t.upload(&dw, w, static_cast<size_t>(oc) * ic * k * k, "ct.w"));
  const size_t ny = static_cast<size_t>(batch) * oc * oh * ow;
  MB_TRY(t.out(&dy, ny, "ct.y"));
  MB_TRY(launch_conv_gather(dx, dw, dy, batch, ic, oc, h, wd, oh, ow, k, stride, pad, relu, nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_conv2d_dilated(const float* x, const float* w, const float* bias, float* y, int batch, int in_c, int out_c, int in_h,
                              int in_w, int kernel, int stride, int padding, int dilation) {
  MB_REQUIRE_INIT();
  if (!x || !w || !y || batch <= 0 || in_c <= 0 || out_c <= 0 || in_h <= 0 || in_w <= 0 || kernel <= 0 || stride <= 0 || padding < 0 ||
      dilation <= 0)
    return fail(MIMIR_B200_E_INVALID, "computeConv2D: bad arguments");
  const int oh = (in_h + 2 * padding - dilation * (kernel - 1) - 1) / stride + 1;
  const int ow = (in_w + 2 * padding - dilation * (kernel - 1) - 1) / stride + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "computeConv2D: empty output");
  Temps t;
  const float *dx, *dw, *db = nullptr;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * in_c * in_h * in_w, "sconv.x"));
  MB_TRY(t.upload(&dw, w, static_cast<size_t>(out_c) * in_c * kernel * kernel, "sconv.w"));
  if (bias) MB_TRY(t.upload(&db, bias, static_cast<size_t>(out_c), "sconv.b"));
  const size_t ny = static_cast<size_t>(batch) * out_c * oh * ow;
  MB_TRY(t.out(&dy, ny, "sconv.y"));
  MB_TRY(launch_conv2d_dilated(dx, dw, db, dy, batch, in_c, out_c, in_h, in_w, kernel, stride, padding, dilation, nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_conv_transpose2d_scatter(const float* x, const float* w, const float* bias, float* y, int batch, int in_c, int out_c,
                                        int in_h, int in_w, int kernel, int stride, int padding) {
  MB_REQUIRE_INIT();
  if (!x || !w || !y || batch <= 0 || in_c <= 0 || out_c <= 0 || in_h <= 0 || in_w <= 0 || kernel <= 0 || stride <= 0 || padding < 0)
    return fail(MIMIR_B200_E_INVALID, "computeConvTranspose2D: bad arguments");
  const int oh = (in_h - 1) * stride - 2 * padding + kernel, ow = (in_w - 1) * stride - 2 * padding + kernel;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "computeConvTranspose2D: empty output");
  Temps t;
  const float *dx, *dw, *db = nullptr;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * in_c * in_h * in_w, "sconvt.x"));
  MB_TRY(t.upload(&dw, w, static_cast<size_t>(out_c) * in_c * kernel * kernel, "sconvt.w"));
  if (bias) MB_TRY(t.upload(&db, bias, static_cast<size_t>(out_c), "sconvt.b"));
  const size_t ny = static_cast<size_t>(batch) * out_c * oh * ow;
  MB_TRY(t.out(&dy, ny, "sconvt.y"));
  MB_TRY(launch_conv_transpose2d_scatter(dx, dw, db, dy, batch, in_c, out_c, in_h, in_w, kernel, stride, padding, nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_batchnorm_batchstats(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels,
                                    long long spatial, float eps) {
  MB_REQUIRE_INIT();
  if (!x || !gamma || !beta || !y || batch <= 0 || channels <= 0 || spatial <= 0)
    return fail(MIMIR_B200_E_INVALID, "computeBatchNorm: bad arguments");
  Temps t;
  const float *dx, *dg, *db;
  float* dy;
  const size_t n = static_cast<size_t>(batch) * channels * spatial;
  MB_TRY(t.upload(&dx, x, n, "bnt.x"));
  MB_TRY(t.upload(&dg, gamma, static_cast<size_t>(channels), "bnt.g"));
  MB_TRY(t.upload(&db, beta, static_cast<size_t>(channels), "bnt.b"));
  MB_TRY(t.out(&dy, n, "bnt.y"));
  MB_TRY(launch_batchnorm_batchstats(dx, dg, db, dy, batch, channels, spatial, eps, nullptr));
  return finish_download(y, dy, n);
}

int mimir_b200_pool2d(int is_max, const float* x, float* y, int batch, int channels, int h, int wd, int kh, int kw, int stride_h,
                      int stride_w, int pad_h, int pad_w) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || channels <= 0 || h <= 0 || wd <= 0 || kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0)
    return fail(MIMIR_B200_E_INVALID, "Pool2d: bad arguments");
  const int oh = (h + 2 * pad_h - kh) / stride_h + 1, ow = (wd + 2 * pad_w - kw) / stride_w + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "MaxPool2d: output dimensions must be > 0");
  Temps t;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * channels * h * wd, "pool.x"));
  const size_t ny = static_cast<size_t>(batch) * channels * oh * ow;
  MB_TRY(t.out(&dy, ny, "pool.y"));
  MB_TRY(launch_pool2d(is_max, dx, dy, batch, channels, h, wd, kh, kw, stride_h, stride_w, pad_h, pad_w, nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_pad2d(int mode, const float* x, float* y, int batch, int channels, int h, int wd, int pad_h, int pad_w) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || channels <= 0 || h <= 0 || wd <= 0 || pad_h < 0 || pad_w < 0)
    return fail(MIMIR_B200_E_INVALID, "Pad2d: bad arguments");
  Temps t;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * channels * h * wd, "pad.x"));
  const size_t ny = static_cast<size_t>(batch) * channels * (h + 2 * pad_h) * (wd + 2 * pad_w);
  MB_TRY(t.out(&dy, ny, "pad.y"));
  MB_TRY(launch_pad2d(mode, dx, dy, batch, channels, h, wd, pad_h, pad_w, nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_pixel_shuffle(const float* x, float* y, int batch, int in_channels, int h, int wd, int r) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || in_channels <= 0 || h <= 0 || wd <= 0 || r <= 0)
    return fail(MIMIR_B200_E_INVALID, "PixelShuffle: bad arguments");
  Temps t;
  const float* dx;
  float* dy;
  const size_t n = static_cast<size_t>(batch) * in_channels * h * wd;
  MB_TRY(t.upload(&dx, x, n, "ps.x"));
  MB_TRY(t.out(&dy, n, "ps.y"));
  MB_TRY(launch_pixel_shuffle(dx, dy, batch, in_channels, h, wd, r, nullptr));
  return finish_download(y, dy, n);
}

int mimir_b200_upsample_bilinear(const float* x, float* y, int batch, int channels, int h, int wd, int out_h, int out_w,
                                 int half_pixel) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || channels <= 0 || h <= 0 || wd <= 0 || out_h <= 0 || out_w <= 0)
    return fail(MIMIR_B200_E_INVALID, "UpsampleBilinear: dimensions must be set");
  Temps t;
  const float* dx;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * channels * h * wd, "bil.x"));
  const size_t ny = static_cast<size_t>(batch) * channels * out_h * out_w;
  MB_TRY(t.out(&dy, ny, "bil.y"));
  MB_TRY(launch_upsample_bilinear(dx, dy, batch, channels, h, wd, out_h, out_w, half_pixel, nullptr));
  return finish_download(y, dy, ny);
}

int mimir_b200_batch_matmul(const float* A, const float* B, float* C, long long nb, int M, int K, int N) {
  MB_REQUIRE_INIT();
  if (!A || !B || !C || nb <= 0 || M <= 0 || K <= 0 || N <= 0) return fail(MIMIR_B200_E_INVALID, "BatchMatMul: bad arguments");
  Temps t;
  const float *da, *db;
  float* dc;
  MB_TRY(t.upload(&da, A, static_cast<size_t>(nb) * M * K, "bmm.a"));
  MB_TRY(t.upload(&db, B, static_cast<size_t>(nb) * K * N, "bmm.b"));
  MB_TRY(t.out(&dc, static_cast<size_t>(nb) * M * N, "bmm.c"));
  MB_TRY(launch_batch_matmul(da, db, dc, nb, M, K, N, nullptr));
  return finish_download(C, dc, static_cast<size_t>(nb) * M * N);
}

int mimir_b200_batchnorm_inference(const float* x, const float* w, long long n_w, float* y, int batch, long long n, float eps) {
  MB_REQUIRE_INIT();
  if (!x || !y || batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "BatchNorm: empty input");
  Temps t;
  const float *dx, *dw = nullptr;
  float* dy;
  MB_TRY(t.upload(&dx, x, static_cast<size_t>(batch) * n, "bn.x"));
  if (w && n_w > 0) MB_TRY(t.upload(&dw, w, static_cast<size_t>(n_w), "bn.w"));
  MB_TRY(t.out(&dy, static_cast<size_t>(batch) * n, "bn.y"));
  MB_TRY(launch_layernorm(dx, nullptr, nullptr, dy, batch, n, eps, nullptr));
  if (dw) MB_TRY(launch_scale_prefix(dy, dw, batch, n, n_w, nullptr));
  return finish_download(y, dy, static_cast<size_t>(batch) * n);
}

int mimir_b200_batchnorm_running(const float* x, const float* gamma, const float* beta, const float* running_mean,
                                 const float* running_var, float* y, int batch, int channels, long long spatial, float eps) {
  MB_REQUIRE_INIT();
  if (!x || !y || !gamma || !beta || !running_mean || !running_var) return fail(MIMIR_B200_E_INVALID, "BatchNorm: null argument");
  if (batch <= 0 || channels <= 0 || spatial <= 0) return fail(MIMIR_B200_E_INVALID, "BatchNorm: empty input");
  Temps t;
  const size_t n = static_cast<size_t>(batch) * channels * spatial;
  const float *dx, *dg, *db, *dm, *dv;
  float* dy;
  MB_TRY(t.upload(&dx, x, n, "bn.x"));
  MB_TRY(t.upload(&dg, gamma, channels, "bn.gamma"));
  MB_TRY(t.upload(&db, beta, channels, "bn.beta"));
  MB_TRY(t.upload(&dm, running_mean, channels, "bn.mean"));
  MB_TRY(t.upload(&dv, running_var, channels, "bn.var"));
  MB_TRY(t.out(&dy, n, "bn.y"));
  MB_TRY(launch_batchnorm_running(dx, dg, db, dm, dv, dy, batch, channels, spatial, eps, nullptr));
  return finish_download(y, dy, n);
}

int mimir_b200_attention_qkv(const float* q, const float* k, const float* v, float* y, int batch, int seq, int d_model,
                             int num_heads) {
  MB_REQUIRE_INIT();
  if (!q || !k || !v || !y) return fail(MIMIR_B200_E_INVALID, "attention: null argument");
  if (batch <= 0 || seq <= 0 || d_model <= 0 || num_heads <= 0 || d_model % num_heads != 0)
    return fail(MIMIR_B200_E_INVALID, "attention: d_model must be a positive multiple of num_heads");
  Temps t;
  const size_t n = static_cast<size_t>(batch) * seq * d_model;
  AttnView a;
  float* dy;
  MB_TRY(t.upload(&a.q, q, n, "attn.q"));
  MB_TRY(t.upload(&a.k, k, n, "attn.k"));
  MB_TRY(t.upload(&a.v, v, n, "attn.v"));
  MB_TRY(t.out(&dy, n, "attn.y"));
  a.ldq = d_model; a.ldkv = d_model; a.q_len = seq; a.kv_len = seq;
  MB_TRY(launch_attention_core_view(a, dy, batch, d_model, num_heads, 0, nullptr));
  return finish_download(y, dy, n);
}

}  // extern "C"
