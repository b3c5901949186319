// ref_shim.cpp — TEST INFRASTRUCTURE.  A C ABI over the reference's OWN CPU implementation.
//
// This file is ours; everything it calls (Model, Layer, ModelArchitectures, LayerOps via
// Model::forwardPassNamed) is compiled from the reference's sources where they lie (see Makefile).
// It exists so that tests and the benchmark's CPU arm can run Mímir's fp32 CPU path on exactly
// the graph, weights and inputs the CUDA backend is given.  Nothing in the product links it.
//
// Graphs are built the way the reference's tests build them (Tests/test_layers_all_types.cpp:40-62):
// Model::push(name, type, params) -> set Layer fields -> allocateParams() -> write the weight block
// through Layer::getWeights() -> forwardPassNamed(float_inputs, {}, /*training=*/false).

#include <omp.h>

#include <chrono>
#include <cstring>
#include <iostream>
#include <memory>
#include <sstream>
#include <streambuf>
#include <string>
#include <unordered_map>
#include <vector>

#include "Model.hpp"
#include "LayerOpsExt.hpp"
#include "MemoryGuard.hpp"
#include "Models/Registry/ModelArchitectures.hpp"
#include "Serialization/SafeTensorsWriter.hpp"
#include "mimir_b200_layer_shim.hpp"

namespace {

thread_local std::string g_err;

// The reference logs to std::cout / std::cerr from allocateParams and the first forward.
struct Quiet {
  std::streambuf *o, *e;
  std::ostringstream sink;
  Quiet() : o(std::cout.rdbuf(sink.rdbuf())), e(std::cerr.rdbuf(sink.rdbuf())) {}
  ~Quiet() {
    std::cout.rdbuf(o);
    std::cerr.rdbuf(e);
  }
};

struct RefModel {
  std::shared_ptr<Model> model;
  std::vector<MimirLayerDesc> descs;  // strings point into model->getLayers()
};

template <class F>
int guarded(F&& f) {
  try {
    Quiet q;
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown exception";
    return 1;
  }
}

void refresh_descs(RefModel* rm) {
  rm->descs.clear();
  for (const auto& L : rm->model->getLayers()) rm->descs.push_back(mimir_b200::describe(L));
}

}  // namespace

extern "C" {

const char* mimir_ref_last_error(void) { return g_err.c_str(); }

int mimir_ref_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}

int mimir_ref_set_guard_limit(unsigned long long bytes) {
  MemoryGuard::instance().setLimit(static_cast<size_t>(bytes));
  return 0;
}

// Builds a Model from descriptors with Model::push + field writes + allocateParams.
int mimir_ref_model_create(const MimirLayerDesc* layers, int n, void** out) {
  return guarded([&] {
    auto rm = std::make_unique<RefModel>();
    rm->model = std::make_shared<Model>();
    for (int i = 0; i < n; ++i) {
      const MimirLayerDesc& d = layers[i];
      rm->model->push(d.name ? d.name : ("l" + std::to_string(i)), d.type, static_cast<size_t>(d.params_count));
      Layer& L = rm->model->getMutableLayers().back();
      mimir_b200::apply(d, L);
    }
    rm->model->allocateParams();
    // zero the blocks so that un-set weights are deterministic
    for (auto& L : rm->model->getMutableLayers()) {
      if (L.params_count && L.getWeights()) std::memset(L.getWeights(), 0, L.params_count * sizeof(float));
    }
    refresh_descs(rm.get());
    *out = rm.release();
  });
}

// Builds a Model through the reference's registry (ModelArchitectures::create) from a JSON config.
int mimir_ref_model_create_registry(const char* arch, const char* cfg_json, void** out) {
  return guarded([&] {
    auto rm = std::make_unique<RefModel>();
    json cfg = (cfg_json && cfg_json[0]) ? json::parse(cfg_json) : json::object();
    rm->model = ModelArchitectures::create(arch, cfg);
    rm->model->allocateParams();
    for (auto& L : rm->model->getMutableLayers()) {
      if (L.params_count && L.getWeights()) std::memset(L.getWeights(), 0, L.params_count * sizeof(float));
    }
    refresh_descs(rm.get());
    *out = rm.release();
  });
}

int mimir_ref_model_destroy(void* h) {
  return guarded([&] { delete static_cast<RefModel*>(h); });
}

int mimir_ref_model_num_layers(void* h) { return static_cast<int>(static_cast<RefModel*>(h)->descs.size()); }

// Exports layer i as the POD descriptor (strings stay owned by the model).
int mimir_ref_model_layer_desc(void* h, int i, MimirLayerDesc* out) {
  auto* rm = static_cast<RefModel*>(h);
  if (i < 0 || i >= static_cast<int>(rm->descs.size())) {
    g_err = "layer index out of range";
    return 1;
  }
  *out = rm->descs[static_cast<size_t>(i)];
  return 0;
}

int mimir_ref_model_set_weights(void* h, int i, const float* w, unsigned long long n) {
  return guarded([&] {
    auto* rm = static_cast<RefModel*>(h);
    Layer& L = rm->model->getMutableLayers().at(static_cast<size_t>(i));
    if (n != L.params_count) throw std::runtime_error("set_weights: size != params_count");
    if (n) std::memcpy(L.getWeights(), w, n * sizeof(float));
  });
}

int mimir_ref_model_get_weights(void* h, int i, float* w, unsigned long long n) {
  return guarded([&] {
    auto* rm = static_cast<RefModel*>(h);
    Layer& L = rm->model->getMutableLayers().at(static_cast<size_t>(i));
    if (n != L.params_count) throw std::runtime_error("get_weights: size != params_count");
    if (n) std::memcpy(w, L.getWeights(), n * sizeof(float));
  });
}

// The Encoder's "mag"/"mod" vectors the registry transformer adds to the token embeddings
// (Encoder.cpp:97-116, TransformerModel.cpp:63-84).  Returns their length through *n.
int mimir_ref_model_get_mag_mod(void* h, float* mag, float* mod, int cap, int* n) {
  return guarded([&] {
    auto* rm = static_cast<RefModel*>(h);
    const auto& e = rm->model->getEncoder();
    const auto& a = e.getMagEmbedding();
    const auto& b = e.getModEmbedding();
    *n = static_cast<int>(a.size());
    if (a.size() != b.size()) throw std::runtime_error("mag/mod size mismatch");
    if (static_cast<int>(a.size()) > cap) throw std::runtime_error("mag/mod capacity too small");
    std::memcpy(mag, a.data(), a.size() * sizeof(float));
    std::memcpy(mod, b.data(), b.size() * sizeof(float));
  });
}

// Writes the model with the reference's own SafeTensorsWriter (tensors "<layer>/weights" plus its
// tokenizer / encoder blobs), so that the device loader can be tested against a real checkpoint.
int mimir_ref_model_save_safetensors(void* h, const char* path) {
  return guarded([&] {
    auto* rm = static_cast<RefModel*>(h);
    Mimir::Serialization::SaveOptions opt;
    opt.include_git_info = false;
    Mimir::Serialization::SafeTensorsWriter w;
    std::string err;
    if (!w.save(*rm->model, path, opt, &err)) throw std::runtime_error("SafeTensorsWriter::save failed: " + err);
  });
}

// The legacy static API, software branch (use_hardware = false): Model::computeAttention on separate Q / K / V and
// Model::computeBatchNorm with running statistics (Model.hpp:409-429).
int mimir_ref_compute_attention(const float* q, const float* k, const float* v, float* out, int seq, int d_model, int heads) {
  return guarded([&] {
    const size_t n = static_cast<size_t>(seq) * d_model;
    std::vector<float> Q(q, q + n), K(k, k + n), V(v, v + n), O;
    Model::computeAttention(Q, K, V, O, seq, d_model, heads, false);
    std::memcpy(out, O.data(), n * sizeof(float));
  });
}
int mimir_ref_compute_batchnorm(float* data, const float* gamma, const float* beta, const float* mean, const float* var,
                                int batch, int channels, int spatial, float eps) {
  return guarded([&] {
    const size_t n = static_cast<size_t>(batch) * channels * spatial;
    std::vector<float> d(data, data + n), g(gamma, gamma + channels), b(beta, beta + channels), m(mean, mean + channels),
        vv(var, var + channels);
    Model::computeBatchNorm(d, g, b, m, vv, batch, channels, spatial, eps, false, false);
    std::memcpy(data, d.data(), n * sizeof(float));
  });
}

// Model::computeConv2D / computeConvTranspose2D (Model.cpp:3880-3888, 4214-4221), Model::computeBatchNorm with training = true
// (software branch) and Model::computeActivation("elu").  out_len returns the element count the reference produced.
int mimir_ref_compute_conv2d(int transposed, const float* x, const float* w, const float* bias, float* out, unsigned long long cap,
                             unsigned long long* out_len, int in_h, int in_w, int in_c, int out_c, int k, int stride, int pad, int dil) {
  return guarded([&] {
    Model::LayerParams p;
    p.weights.assign(w, w + static_cast<size_t>(out_c) * in_c * k * k);
    if (bias) p.bias.assign(bias, bias + out_c);
    p.kernel_size = k;
    p.stride = stride;
    p.padding = pad;
    p.dilation = dil;
    const std::vector<float> in(x, x + static_cast<size_t>(in_c) * in_h * in_w);
    std::vector<float> y;
    if (transposed) Model::computeConvTranspose2D(in, y, p, in_h, in_w, in_c, out_c, false);
    else Model::computeConv2D(in, y, p, in_h, in_w, in_c, out_c, false);
    if (out_len) *out_len = y.size();
    if (y.size() > cap) throw std::runtime_error("compute_conv2d: output capacity too small");
    std::memcpy(out, y.data(), y.size() * sizeof(float));
  });
}
int mimir_ref_compute_batchnorm_training(float* data, const float* gamma, const float* beta, int batch, int channels, int spatial,
                                         float eps) {
  return guarded([&] {
    const size_t n = static_cast<size_t>(batch) * channels * spatial;
    std::vector<float> d(data, data + n), g(gamma, gamma + channels), b(beta, beta + channels), m(channels, 0.0f), vv(channels, 1.0f);
    Model::computeBatchNorm(d, g, b, m, vv, batch, channels, spatial, eps, true, false);
    std::memcpy(data, d.data(), n * sizeof(float));
  });
}
int mimir_ref_compute_activation(const char* name, float* data, unsigned long long n, float param) {
  return guarded([&] {
    std::vector<float> d(data, data + n);
    Model::computeActivation(d, name, param, false);
    std::memcpy(data, d.data(), n * sizeof(float));
  });
}

// LayerOpsExt::maxpool1d_forward (LayerOpsExt.hpp:504-538).  The layer switch of Model::forwardPassView has no case that
// calls it (a MaxPool1d layer throws there), so it is reached directly.
int mimir_ref_maxpool1d(const float* x, unsigned long long n, int in_channels, int kernel_h, int stride_h, int pad_h, float* out,
                        unsigned long long cap, unsigned long long* out_len) {
  return guarded([&] {
    Layer L;
    L.in_channels = in_channels;
    L.kernel_h = kernel_h;
    L.stride_h = stride_h;
    L.pad_h = pad_h;
    const std::vector<float> in(x, x + n);
    const std::vector<float> y = LayerOpsExt::maxpool1d_forward(in, L);
    if (out_len) *out_len = y.size();
    if (y.size() > cap) throw std::runtime_error("maxpool1d: output capacity too small");
    std::memcpy(out, y.data(), y.size() * sizeof(float));
  });
}

// One sample through Model::forwardPassNamed(training=false).  Returns seconds in *seconds.
int mimir_ref_model_forward(void* h, const MimirNamedInput* inputs, int n_inputs, float* out,
                            unsigned long long cap, unsigned long long* out_len, double* seconds) {
  return guarded([&] {
    auto* rm = static_cast<RefModel*>(h);
    std::unordered_map<std::string, std::vector<float>> fin;
    std::unordered_map<std::string, std::vector<int>> iin;
    for (int i = 0; i < n_inputs; ++i) {
      std::string name = inputs[i].name ? inputs[i].name : "x";
      if (name == "__input__") name = "x";
      fin[name] = std::vector<float>(inputs[i].data, inputs[i].data + inputs[i].per_sample);
    }
    const auto t0 = std::chrono::steady_clock::now();
    const std::vector<float>& y = rm->model->forwardPassNamedView(fin, iin, false);
    const auto t1 = std::chrono::steady_clock::now();
    if (seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
    if (out_len) *out_len = y.size();
    if (out) {
      if (y.size() > cap) throw std::runtime_error("forward: output capacity too small");
      std::memcpy(out, y.data(), y.size() * sizeof(float));
    }
  });
}

}  // extern "C"
