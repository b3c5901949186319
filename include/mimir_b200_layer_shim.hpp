// mimir_b200_layer_shim.hpp — the only piece that is compiled against Mímir's own headers.
//
// Translates Mímir's `struct Layer` (Layers.hpp:86-309) into the POD MimirLayerDesc that the
// C ABI takes, resolving the helper accessors the forward ops use (get_kernel_h / get_stride_h /
// get_pad_h, Layers.hpp:250-257) so that the backend never needs Mímir's headers.
//
// Usage inside Mímir (or any program that links Mímir):
//     mimir_b200::GraphDescs g(model.getLayers());
//     mimir_b200_model_create(g.data(), g.size(), &handle);
//     for (i...) mimir_b200_model_upload_weights(handle, i, layers[i].getWeights(), layers[i].getWeightsSize());
#pragma once

#include <string>
#include <vector>
#include <cstring>

#include "Layers.hpp"     // Mímir
#include "mimir_b200.h"

#include <stdexcept>

namespace mimir_b200 {

// Reads MIMIR_B200 / MIMIR_B200_DEVICE / MIMIR_B200_HBM_BUDGET_MB and brings the backend up when it is selected (default
// off, like the reference's own accelerator switches, Model.cpp:5110-5112).  Returns whether it is selected; throws
// std::runtime_error - the reference's error convention (RuntimeAllocator.hpp:344-358) - when it is selected but cannot
// start: the backend has no CPU fallback of its own, the caller decides what happens then.
inline bool init_from_env() {
  int enabled = 0;
  if (mimir_b200_init_from_env(&enabled) != MIMIR_B200_OK) throw std::runtime_error(std::string("mimir_b200: ") + mimir_b200_last_error());
  return enabled != 0;
}

inline MimirLayerDesc describe(const Layer& L) {
  MimirLayerDesc d;
  std::memset(&d, 0, sizeof(d));
  d.name = L.name.c_str();
  d.type = L.type.c_str();  // normalised by Layer's constructor (Layers.hpp:229-235)
  d.n_inputs = 0;
  for (const auto& in : L.inputs) {
    if (d.n_inputs >= MIMIR_B200_MAX_INPUTS) break;
    d.inputs[d.n_inputs++] = in.c_str();
  }
  d.output = L.output.c_str();
  d.params_count = L.params_count;
  d.in_features = L.in_features;
  d.out_features = L.out_features;
  d.in_channels = L.in_channels;
  d.out_channels = L.out_channels;
  d.input_height = L.input_height;
  d.input_width = L.input_width;
  d.kernel = L.get_kernel_h();
  d.stride = L.get_stride_h();
  d.padding = L.get_pad_h();
  d.eps = L.eps;
  d.num_groups = L.num_groups;
  d.affine = L.affine ? 1 : 0;
  d.use_bias = L.use_bias ? 1 : 0;
  d.vocab_size = L.vocab_size;
  d.embed_dim = L.embed_dim;
  d.padding_idx = L.padding_idx;
  d.num_heads = L.num_heads;
  d.seq_len = L.seq_len;
  d.causal = L.causal ? 1 : 0;
  d.out_h = L.out_h;
  d.out_w = L.out_w;
  // UpsampleNearest truncates the float factors to int and treats <= 0 as 2 (Model.cpp:6011-6012)
  d.scale_h = static_cast<int>(L.scale_h);
  d.scale_w = static_cast<int>(L.scale_w);
  d.activation = (L.activation != ActivationType::NONE) ? 1 : 0;
  d.n_dims = 0;
  const size_t nd = L.permute_dims.size();
  if (nd <= MIMIR_B200_MAX_DIMS && L.shape.size() == nd) {
    d.n_dims = static_cast<int32_t>(nd);
    for (size_t i = 0; i < nd; ++i) {
      d.shape[i] = L.shape[i];
      d.permute_dims[i] = L.permute_dims[i];
    }
  }
  d.head_dim = L.head_dim;
  d.leaky_relu_alpha = L.leaky_relu_alpha;
  d.kernel_w = L.get_kernel_w();
  d.stride_w = L.get_stride_w();
  d.padding_w = L.get_pad_w();
  d.raw_kernel_h = L.kernel_h;
  d.raw_stride_h = L.stride_h;
  d.raw_pad_h = L.pad_h;
  d.raw_pad_w = L.pad_w;
  d.n_splits = 0;
  if (L.split_sizes.size() <= MIMIR_B200_MAX_SPLITS) {
    d.n_splits = static_cast<int32_t>(L.split_sizes.size());
    for (size_t i = 0; i < L.split_sizes.size(); ++i) d.split_sizes[i] = L.split_sizes[i];
  } else {
    d.n_splits = -1;  // more pieces than the descriptor carries: model_create refuses the layer
  }
  d.num_chunks = L.num_chunks;
  d.seq_text = L.seq_text;
  d.num_patches = L.num_patches;
  d.patch_dim = L.patch_dim;
  d.target_dim0 = L.target_shape.empty() ? 0 : L.target_shape[0];
  return d;
}

// Holds the descriptors for a whole layer list.  The strings stay owned by the Layers, so the
// Layer vector must outlive this object (model_create copies them).
class GraphDescs {
 public:
  explicit GraphDescs(const std::vector<Layer>& layers) {
    descs_.reserve(layers.size());
    for (const auto& L : layers) descs_.push_back(describe(L));
  }
  const MimirLayerDesc* data() const { return descs_.data(); }
  int size() const { return static_cast<int>(descs_.size()); }

 private:
  std::vector<MimirLayerDesc> descs_;
};

// The inverse, used by tools that build a Mímir graph from descriptors (e.g. to run the CPU path
// on exactly the graph the backend was given).
inline void apply(const MimirLayerDesc& d, Layer& L) {
  L.inputs.clear();
  for (int i = 0; i < d.n_inputs; ++i) L.inputs.emplace_back(d.inputs[i] ? d.inputs[i] : "x");
  L.output = (d.output && d.output[0]) ? d.output : "x";
  L.params_count = static_cast<size_t>(d.params_count);
  L.in_features = d.in_features;
  L.out_features = d.out_features;
  L.in_channels = d.in_channels;
  L.out_channels = d.out_channels;
  L.input_height = d.input_height;
  L.input_width = d.input_width;
  L.kernel_size = d.kernel;
  L.stride = d.stride > 0 ? d.stride : 1;
  L.padding = d.padding;
  L.eps = d.eps;
  L.num_groups = d.num_groups > 0 ? d.num_groups : 1;
  L.affine = d.affine != 0;
  L.use_bias = d.use_bias != 0;
  L.vocab_size = d.vocab_size;
  L.embed_dim = d.embed_dim;
  L.padding_idx = d.padding_idx;
  L.num_heads = d.num_heads;
  L.seq_len = d.seq_len;
  L.causal = d.causal != 0;
  L.out_h = d.out_h;
  L.out_w = d.out_w;
  L.scale_h = static_cast<float>(d.scale_h);
  L.scale_w = static_cast<float>(d.scale_w);
  L.activation = d.activation ? ActivationType::RELU : ActivationType::NONE;
  L.shape.assign(d.shape, d.shape + d.n_dims);
  L.permute_dims.assign(d.permute_dims, d.permute_dims + d.n_dims);
  L.head_dim = d.head_dim;
  L.leaky_relu_alpha = d.leaky_relu_alpha;
  L.kernel_h = d.raw_kernel_h;
  L.stride_h = d.raw_stride_h > 0 ? d.raw_stride_h : 1;
  L.pad_h = d.raw_pad_h;
  L.pad_w = d.raw_pad_w;
  L.kernel_w = (d.kernel_w > 0 && d.kernel_w != d.kernel) ? d.kernel_w : d.raw_kernel_h;
  if (d.stride_w > 0 && d.stride_w != d.stride) L.stride_w = d.stride_w;
  if (d.n_splits > 0) L.split_sizes.assign(d.split_sizes, d.split_sizes + d.n_splits);
  L.num_chunks = d.num_chunks;
  L.seq_text = d.seq_text;
  L.num_patches = d.num_patches;
  L.patch_dim = d.patch_dim;
  if (d.target_dim0 > 0) L.target_shape.assign(1, d.target_dim0);
}

}  // namespace mimir_b200
