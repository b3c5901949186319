// ops.h — device-pointer op sequences shared by the per-op C ABI (capi.cu) and the graph
// executor (graph.cu): each `*_ws_bytes` says how much workspace the sequence needs and each
// `*_exec` runs it asynchronously on a stream.
#pragma once

#include "common.h"

namespace mb {

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }
void precision_planes(int precision, int* a_planes, int* w_planes);
size_t split_bytes(int64_t rows, int k, int planes);
int check_device_error_word(cudaStream_t st);

struct LinearExec {
  int rows = 0, in_f = 0, out_f = 0;
  int precision = MIMIR_B200_PREC_BF16X2;
  const float* x_f32 = nullptr;             // fp32 [rows, in_f] (needed unless x_split is given)
  const __nv_bfloat16* x_split = nullptr;   // planes produced by an upstream GEMM epilogue
  const float* w_f32 = nullptr;             // fp32 [out_f, in_f] (skinny path)
  const __nv_bfloat16* w_split = nullptr;   // planes [w_planes][out_f][kp] (tensor-core path)
  float w_scale = 1.0f;                     // the planes hold W * w_scale (weight_plane_scale)
  const float* bias = nullptr;
  const float* residual = nullptr;          // same layout as y_f32
  int activation = -1;
  float* y_f32 = nullptr;
  __nv_bfloat16* y_split = nullptr;         // planes [2][rows][round_up(out_f, 64)]
  int out_nchw_hw = 0;
  void* ws = nullptr;
  size_t ws_bytes = 0;
};
bool linear_uses_skinny(int rows, int precision);
size_t linear_ws_bytes(int rows, int in_f, int out_f, int precision, bool a_presplit);
int linear_exec(const LinearExec& e, cudaStream_t st);

struct AttentionExec {
  int batch = 0, seq = 0, embed = 0, heads = 1, causal = 0;
  int precision = MIMIR_B200_PREC_BF16X2;
  const float* x = nullptr;                    // fp32 [batch*seq, embed]
  const __nv_bfloat16* x_split = nullptr;      // or: its operand planes, written by the producing layer
  const __nv_bfloat16* wqkv_split = nullptr;   // planes of Wqkv^T: [3E][round_up(E,64)]
  const __nv_bfloat16* wout_split = nullptr;   // planes of Wout^T: [E][round_up(E,64)]
  float w_scale = 1.0f;                        // both plane sets hold their weights times this (weight_plane_scale)
  const float* residual = nullptr;
  float* y = nullptr;
  void* ws = nullptr;
  // Key / value cache [batch][max_seq][embed] (optional).  decode_pos < 0: a normal forward that also stores its K and V
  // rows at positions 0 .. seq-1.  decode_pos >= 0: seq must be 1; the new token's K and V go to that position and
  // the query attends to positions 0 .. decode_pos.
  float* kcache = nullptr;
  float* vcache = nullptr;
  int max_seq = 0;
  int decode_pos = -1;
  const int* pos_dev = nullptr;     // decode steps replayed from a CUDA graph read the position here instead of decode_pos
  float* decode_scratch = nullptr;  // attention_decode_scratch_bytes(batch, heads, embed, max_seq), for decode steps
  // decode steps of <= 16 samples: fp32 copies of the projections as W[out][in] and the weight-streaming kernel's scratch
  const float* wqkv_t_f32 = nullptr;
  const float* wout_t_f32 = nullptr;
  float* skinny_scratch = nullptr;
  size_t skinny_scratch_bytes = 0;
};
size_t attention_ws_bytes(int batch, int seq, int embed, int heads, int precision);
int attention_exec(const AttentionExec& e, cudaStream_t st);

// CrossAttention (LayerOps.hpp:1116-1216): Q = query . Wq, K | V = key_value . Wkv, softmax core, . Wout
struct CrossAttentionExec {
  int batch = 0, q_len = 0, kv_len = 0, embed = 0, heads = 1, causal = 0;
  int precision = MIMIR_B200_PREC_BF16X2;
  const float* q_in = nullptr;                 // fp32 [batch*q_len, embed]
  const float* kv_in = nullptr;                // fp32 [batch*kv_len, embed]
  const __nv_bfloat16* wq_split = nullptr;     // planes of Wq^T:   [E][round_up(E,64)]
  const __nv_bfloat16* wkv_split = nullptr;    // planes of Wkv^T:  [2E][round_up(E,64)]
  const __nv_bfloat16* wout_split = nullptr;   // planes of Wout^T: [E][round_up(E,64)]
  float w_scale = 1.0f;                        // all three plane sets hold their weights times this
  const float* residual = nullptr;
  float* y = nullptr;
  void* ws = nullptr;
};
size_t cross_attention_ws_bytes(int batch, int q_len, int kv_len, int embed, int precision);
int cross_attention_exec(const CrossAttentionExec& e, cudaStream_t st);

struct ConvExec {
  int batch = 0, ic = 0, oc = 0, h = 0, w = 0, ks = 3, stride = 1, pad = 0;
  int precision = MIMIR_B200_PREC_BF16X2;
  int activation = -1;                         // MIMIR_B200_ELT_RELU when the layer asks for it
  const float* x = nullptr;                    // NCHW
  const __nv_bfloat16* w_split = nullptr;      // planes [oc][round_up(ic*ks*ks, 64)]
  const float* w_f32 = nullptr;                // OIHW fp32 (the direct kernel for a handful of output channels)
  float w_scale = 1.0f;                        // the planes hold W * w_scale
  const float* residual = nullptr;             // NCHW, same shape as y
  float* y = nullptr;
  void* ws = nullptr;
  // GroupNorm (+ SiLU) of the producing layer, applied while the operand planes are laid out (shifted path only):
  // x is then the GroupNorm's INPUT
  int pre_groups = 0;                          // > 0 switches it on
  const float* pre_gamma = nullptr;
  const float* pre_beta = nullptr;
  float pre_eps = 1e-5f;
  int pre_act = -1;
  // x is [ic][h/2][w/2]: the 2 x 2 nearest-neighbour upsample of the producing layer is applied while the operand planes
  // are laid out (shifted path only); h and w stay the convolution's own input size
  int in_up = 0;
  // The statistics of the folded GroupNorm already exist (the producer's epilogue emitted them): [batch][pre_groups][2]
  const float* pre_stats = nullptr;
  // This convolution's output feeds a GroupNorm of gn_groups groups: its GEMM epilogue leaves partials behind and
  // (mean, 1 / std) per (sample, group) go to gn_stats_out (shifted-GEMM path only; the workspace holds the partials)
  float* gn_stats_out = nullptr;
  int gn_groups = 0;
  float gn_eps = 1e-5f;
};
size_t conv_prenorm_bytes(int batch, int groups);
// scratch of the GroupNorm partials a shifted-GEMM convolution emits (behind the planes and the pre-norm statistics)
size_t conv_gn_emit_bytes(int batch, int oc, int h, int w, int pad, int groups);
// can this convolution's epilogue emit the statistics of a GroupNorm with `groups` groups over its output?
bool conv_can_emit_gn(int batch, int ic, int oc, int h, int w, int ks, int stride, int pad, int groups, int act);
// stride-1 "same" convolutions with a channel count that is a multiple of 32 run as shifted GEMMs over the
// padded NHWC activation; everything else goes through im2col planes.  The two paths want different
// weight-plane orders ((kh, kw, ic) vs (ic, kh, kw)).
bool conv_uses_shifted(int ic, int ks, int stride, int pad);
size_t conv_ws_bytes(int batch, int ic, int h, int w, int ks, int stride, int pad, int precision);
int conv_exec(const ConvExec& e, cudaStream_t st);

}  // namespace mb
