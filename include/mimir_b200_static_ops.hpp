// mimir_b200_static_ops.hpp — the legacy static dispatch family of Mímir's Model class
// (Model.hpp:388-429, Model.cpp:3880-4289) as thin wrappers over the per-op C ABI.
//
// Same names, argument order and container types as the reference's static members, so a call site such as
//     Model::computeLinear(input, output, params, /*use_hardware=*/true);
// becomes
//     mimir_b200::static_ops::computeLinear(input, output, params);
// `use_hardware` has no meaning here (there is no software path behind these calls) and is accepted and
// ignored.  Errors surface as std::runtime_error carrying mimir_b200_last_error(), which is how the
// reference reports shape errors (RuntimeAllocator.hpp:344-358).  mimir_b200_init must have been called.
//
// Covered: computeConv2D (bias, dilation), computeLinear, computeMaxPool2D, computeAvgPool2D, computeActivation
// (relu, leaky_relu, tanh, sigmoid, gelu, softmax, elu), computeBatchNorm (running or batch statistics),
// computeLayerNorm, computeConvTranspose2D (the scatter form), computeAttention.  An activation name the reference
// does not know leaves the data untouched there (Model.cpp:4026-4064) and here.
#pragma once

#include <algorithm>
#include <stdexcept>
#include <string>
#include <vector>

#include "mimir_b200.h"

namespace mimir_b200 {
namespace static_ops {

// Mirror of Model::LayerParams (Model.hpp:373-385): only the fields these wrappers read.
struct LayerParams {
  std::vector<float> weights;
  std::vector<float> bias;
  int in_features = 0;
  int out_features = 0;
  int kernel_size = 3;
  int stride = 1;
  int padding = 0;
  int dilation = 1;
  int groups = 1;
  bool use_hardware = true;
};

inline void check(int status) {
  if (status != MIMIR_B200_OK) throw std::runtime_error(mimir_b200_last_error());
}

// Model::computeLinear (Model.cpp:3890-3916): one input vector, W[out][in], optional bias.
inline void computeLinear(const std::vector<float>& input, std::vector<float>& output, const LayerParams& params,
                          bool /*use_hardware*/ = true) {
  if (static_cast<int>(input.size()) < params.in_features ||
      params.weights.size() < static_cast<size_t>(params.in_features) * params.out_features)
    throw std::runtime_error("computeLinear: input or weights smaller than in_features x out_features");
  output.assign(static_cast<size_t>(params.out_features), 0.0f);
  check(mimir_b200_linear_forward(input.data(), params.weights.data(), params.bias.empty() ? nullptr : params.bias.data(),
                                  output.data(), 1, params.in_features, params.out_features));
}

// Model::computeMaxPool2D / computeAvgPool2D (Model.cpp:3918-4024): CHW, no padding, stride < 0 means
// stride = kernel_size; the average divides by kernel_size^2 (every tap is inside without padding).
inline void computePool2D(bool is_max, const std::vector<float>& input, std::vector<float>& output, int in_h, int in_w,
                          int channels, int kernel_size, int stride) {
  if (stride < 0) stride = kernel_size;
  if (kernel_size <= 0 || stride <= 0 || channels <= 0 || in_h < kernel_size || in_w < kernel_size)
    throw std::runtime_error("computePool2D: invalid dimensions");
  if (input.size() < static_cast<size_t>(channels) * in_h * in_w) throw std::runtime_error("computePool2D: input too small");
  const int out_h = (in_h - kernel_size) / stride + 1, out_w = (in_w - kernel_size) / stride + 1;
  output.assign(static_cast<size_t>(out_h) * out_w * channels, 0.0f);
  check(mimir_b200_pool2d(is_max ? 1 : 0, input.data(), output.data(), 1, channels, in_h, in_w, kernel_size, kernel_size, stride,
                          stride, 0, 0));
}
inline void computeMaxPool2D(const std::vector<float>& input, std::vector<float>& output, int in_h, int in_w, int channels,
                             int kernel_size, int stride, bool /*use_hardware*/ = true) {
  computePool2D(true, input, output, in_h, in_w, channels, kernel_size, stride);
}
inline void computeAvgPool2D(const std::vector<float>& input, std::vector<float>& output, int in_h, int in_w, int channels,
                             int kernel_size, int stride, bool /*use_hardware*/ = true) {
  computePool2D(false, input, output, in_h, in_w, channels, kernel_size, stride);
}

// Model::computeActivation (Model.cpp:4026-4064), in place.  "gelu" is the tanh form of the layer op
// (LayerOps.hpp:556-568), not the clamped AVX2 approximation the reference's hardware branch uses
// (SIMD_Ops.hpp:115-121).  "softmax" is over the whole vector.
inline void computeActivation(std::vector<float>& data, const std::string& activation_type, float param = 0.0f,
                              bool /*use_hardware*/ = true) {
  if (data.empty()) return;
  const long long n = static_cast<long long>(data.size());
  if (activation_type == "softmax") {
    std::vector<float> out(data.size());
    check(mimir_b200_softmax(data.data(), out.data(), 1, n, 0));
    data.swap(out);
    return;
  }
  int op = -1;
  if (activation_type == "relu") op = MIMIR_B200_ELT_RELU;
  else if (activation_type == "leaky_relu") op = MIMIR_B200_ELT_LEAKY_RELU;
  else if (activation_type == "tanh") op = MIMIR_B200_ELT_TANH;
  else if (activation_type == "sigmoid") op = MIMIR_B200_ELT_SIGMOID;
  else if (activation_type == "gelu") op = MIMIR_B200_ELT_GELU;
  else if (activation_type == "elu") op = MIMIR_B200_ELT_ELU;  // Model::elu_inplace, Model.hpp:505-509
  else return;  // an unknown name is a no-op in the reference (Model.cpp:4026-4064)
  std::vector<float> out(data.size());
  check(mimir_b200_eltwise_alpha(op, data.data(), nullptr, out.data(), 1, n, 0, param));
  data.swap(out);
}

// Model::computeLayerNorm (Model.cpp:4150-4212), in place: groups of normalized_size, biased variance,
// gamma / beta indexed inside the group (either may be empty).
inline void computeLayerNorm(std::vector<float>& data, const std::vector<float>& gamma, const std::vector<float>& beta,
                             int normalized_size, float eps = 1e-5f, bool /*use_hardware*/ = true) {
  if (normalized_size <= 0 || data.size() % static_cast<size_t>(normalized_size) != 0)
    throw std::runtime_error("computeLayerNorm: data size is not a multiple of normalized_size");
  if ((!gamma.empty() && gamma.size() < static_cast<size_t>(normalized_size)) ||
      (!beta.empty() && beta.size() < static_cast<size_t>(normalized_size)))
    throw std::runtime_error("computeLayerNorm: gamma / beta shorter than normalized_size");
  std::vector<float> out(data.size());
  check(mimir_b200_layernorm(data.data(), gamma.empty() ? nullptr : gamma.data(), beta.empty() ? nullptr : beta.data(), out.data(),
                             static_cast<long long>(data.size() / static_cast<size_t>(normalized_size)), normalized_size, eps));
  data.swap(out);
}

// Model::computeConv2D -> Conv::conv2d (Model.cpp:3880-3888, Layers.hpp:611-722): CHW input, OIHW weights, optional bias,
// stride, zero padding, dilation.  Follows the scalar branch (Layers.hpp:690-721).  An AVX2 build of the reference adds
// every tap of the kernel-row remainder (all taps for kernels narrower than eight) to all eight lanes of its accumulator
// before the horizontal sum (Layers.hpp:658-666, 670-678), so there each such tap counts eight times.
inline void computeConv2D(const std::vector<float>& input, std::vector<float>& output, const LayerParams& params, int in_h, int in_w,
                          int in_c, int out_c, bool /*use_hardware*/ = true) {
  const int k = params.kernel_size, s = params.stride, p = params.padding, d = params.dilation;
  if (in_h <= 0 || in_w <= 0 || in_c <= 0 || out_c <= 0 || k <= 0 || s <= 0 || d <= 0 ||
      input.size() < static_cast<size_t>(in_c) * in_h * in_w || params.weights.size() < static_cast<size_t>(out_c) * in_c * k * k ||
      (!params.bias.empty() && params.bias.size() < static_cast<size_t>(out_c)))
    throw std::runtime_error("computeConv2D: input, weights or bias smaller than the stated dimensions");
  const int oh = (in_h + 2 * p - d * (k - 1) - 1) / s + 1, ow = (in_w + 2 * p - d * (k - 1) - 1) / s + 1;
  if (oh <= 0 || ow <= 0) throw std::runtime_error("computeConv2D: empty output");
  output.assign(static_cast<size_t>(out_c) * oh * ow, 0.0f);
  check(mimir_b200_conv2d_dilated(input.data(), params.weights.data(), params.bias.empty() ? nullptr : params.bias.data(), output.data(),
                                  1, in_c, out_c, in_h, in_w, k, s, p, d));
}

// Model::computeConvTranspose2D -> Conv::conv_transpose2d (Model.cpp:4214-4221, Layers.hpp:775-818): weights [out_c][in_c][k][k].
inline void computeConvTranspose2D(const std::vector<float>& input, std::vector<float>& output, const LayerParams& params, int in_h,
                                   int in_w, int in_c, int out_c, bool /*use_hardware*/ = true) {
  const int k = params.kernel_size, s = params.stride, p = params.padding;
  if (in_h <= 0 || in_w <= 0 || in_c <= 0 || out_c <= 0 || k <= 0 || s <= 0 ||
      input.size() < static_cast<size_t>(in_c) * in_h * in_w || params.weights.size() < static_cast<size_t>(out_c) * in_c * k * k ||
      (!params.bias.empty() && params.bias.size() < static_cast<size_t>(out_c)))
    throw std::runtime_error("computeConvTranspose2D: input, weights or bias smaller than the stated dimensions");
  const int oh = (in_h - 1) * s - 2 * p + k, ow = (in_w - 1) * s - 2 * p + k;
  if (oh <= 0 || ow <= 0) throw std::runtime_error("computeConvTranspose2D: empty output");
  output.assign(static_cast<size_t>(out_c) * oh * ow, 0.0f);
  check(mimir_b200_conv_transpose2d_scatter(input.data(), params.weights.data(), params.bias.empty() ? nullptr : params.bias.data(),
                                            output.data(), 1, in_c, out_c, in_h, in_w, k, s, p));
}

// Model::computeBatchNorm (Model.cpp:4066-4148), in place, data [batch][channels][spatial].  training = true takes the
// mean and the biased variance of each channel from the batch itself (Layers.hpp:940-959); the running statistics are
// not updated, as in the reference.
inline void computeBatchNorm(std::vector<float>& data, const std::vector<float>& gamma, const std::vector<float>& beta,
                             const std::vector<float>& running_mean, const std::vector<float>& running_var, int batch_size,
                             int channels, int spatial_size, float eps = 1e-5f, bool training = false, bool /*use_hardware*/ = true) {
  const size_t n = static_cast<size_t>(batch_size) * channels * spatial_size;
  const size_t c = static_cast<size_t>(channels);
  if (batch_size <= 0 || channels <= 0 || spatial_size <= 0 || data.size() < n || gamma.size() < c || beta.size() < c ||
      running_mean.size() < c || running_var.size() < c)
    throw std::runtime_error("computeBatchNorm: data or parameters smaller than batch x channels x spatial");
  std::vector<float> out(data.size());
  if (training)
    check(mimir_b200_batchnorm_batchstats(data.data(), gamma.data(), beta.data(), out.data(), batch_size, channels, spatial_size, eps));
  else
    check(mimir_b200_batchnorm_running(data.data(), gamma.data(), beta.data(), running_mean.data(), running_var.data(), out.data(),
                                       batch_size, channels, spatial_size, eps));
  std::copy(out.begin(), out.begin() + static_cast<std::ptrdiff_t>(n), data.begin());
}

// Model::computeAttention (Model.cpp:4223-4289): separate, already projected Q / K / V of one sequence, [seq_len][d_model]
// with the heads side by side; no mask.  Follows the reference's scalar branch; its AVX2 branch reads every head as a
// dense [seq_len][head_dim] block, which only coincides with this layout for num_heads = 1.
inline void computeAttention(const std::vector<float>& query, const std::vector<float>& key, const std::vector<float>& value,
                             std::vector<float>& output, int seq_len, int d_model, int num_heads, bool /*use_hardware*/ = true) {
  const size_t n = static_cast<size_t>(seq_len) * d_model;
  if (seq_len <= 0 || d_model <= 0 || num_heads <= 0 || d_model % num_heads != 0 || query.size() < n || key.size() < n ||
      value.size() < n)
    throw std::runtime_error("computeAttention: Q / K / V smaller than seq_len x d_model, or d_model not a multiple of num_heads");
  output.assign(n, 0.0f);
  check(mimir_b200_attention_qkv(query.data(), key.data(), value.data(), output.data(), 1, seq_len, d_model, num_heads));
}

}  // namespace static_ops
}  // namespace mimir_b200
