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
// Covered: computeLinear, computeMaxPool2D, computeAvgPool2D, computeActivation (relu, leaky_relu, tanh,
// sigmoid, gelu, softmax), computeLayerNorm, computeBatchNorm (inference), computeAttention.  Not covered,
// because their arithmetic differs from the layer ops this backend implements: computeConv2D /
// computeConvTranspose2D (Conv::conv2d adds a bias and takes a dilation; Conv::conv_transpose2d is the
// scatter form, Layers.hpp:611-830), computeBatchNorm with training = true, activation "elu".  Calling
// those here throws.
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
  else throw std::runtime_error("computeActivation: '" + activation_type + "' is not available on the B200 backend");
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

[[noreturn]] inline void not_available(const char* what) {
  throw std::runtime_error(std::string(what) + " has no B200 counterpart: its arithmetic differs from the layer ops "
                                               "(see the header of mimir_b200_static_ops.hpp)");
}
inline void computeConv2D(const std::vector<float>&, std::vector<float>&, const LayerParams&, int, int, int, int, bool = true) {
  not_available("computeConv2D");
}
inline void computeConvTranspose2D(const std::vector<float>&, std::vector<float>&, const LayerParams&, int, int, int, int,
                                   bool = true) {
  not_available("computeConvTranspose2D");
}

// Model::computeBatchNorm (Model.cpp:4066-4148), in place, data [batch][channels][spatial].  Inference only: with
// training = true the reference recomputes the statistics from the batch, which is outside the forward path.
inline void computeBatchNorm(std::vector<float>& data, const std::vector<float>& gamma, const std::vector<float>& beta,
                             const std::vector<float>& running_mean, const std::vector<float>& running_var, int batch_size,
                             int channels, int spatial_size, float eps = 1e-5f, bool training = false, bool /*use_hardware*/ = true) {
  if (training) not_available("computeBatchNorm(training = true)");
  const size_t n = static_cast<size_t>(batch_size) * channels * spatial_size;
  const size_t c = static_cast<size_t>(channels);
  if (batch_size <= 0 || channels <= 0 || spatial_size <= 0 || data.size() < n || gamma.size() < c || beta.size() < c ||
      running_mean.size() < c || running_var.size() < c)
    throw std::runtime_error("computeBatchNorm: data or parameters smaller than batch x channels x spatial");
  std::vector<float> out(data.size());
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
