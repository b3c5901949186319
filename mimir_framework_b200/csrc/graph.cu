// graph.cu — whole-graph execution: the device-side counterpart of Model::forwardPassView
// (Model.cpp:4621-6824) and of the activation-memory subsystems (RuntimeAllocator.hpp:181-316,
// MemoryGuard.hpp:16-206).
//
//   model_create   copies the layer descriptors (the translated `std::vector<Layer>`).
//   upload_weights copies one layer's flat fp32 block to the device (the host pointer is never
//                  kept: it may move, DynamicTensorAllocator.hpp:171-200).
//   plan           resolves the name routing into tensor versions (a name may be redefined, e.g.
//                  "x"), infers every per-sample size, fuses what the graph allows (activation into
//                  the producing GEMM / GroupNorm, hi/lo planes straight from one GEMM to the next),
//                  computes liveness and assigns arena offsets that are reused after the last
//                  consumer, and checks the arena peak against the HBM budget before any launch.
//   forward        stages the inputs, runs the layers in index order on one stream, returns "x".
#include "ops.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

namespace mb {
namespace {

enum class LT {
  Linear, Attention, Conv2d, LayerNorm, RMSNorm, GroupNorm, Softmax, LogSoftmax, Act, Add, Multiply, Embedding,
  UpsampleNearest, Permute, Concat, Alias, TokenMeanPool, GlobalAvgPool,
  // the remaining switch cases
  CrossAttention, Split, DepthwiseConv2d, Conv1d, ConvTranspose2d, Pool2d, Pad2d, PixelShuffle, UpsampleBilinear, MatMul,
  BatchMatMul, BatchNorm, InstanceNorm, Binary2, Transpose, EmbeddingBag, PatchEmbed, Bilinear, Recurrent,
  Unsupported
};

struct TypeInfo { LT lt; int act; };

TypeInfo classify(const std::string& t) {
  if (t == "Linear") return {LT::Linear, -1};
  if (t == "SelfAttention" || t == "MultiHeadAttention") return {LT::Attention, -1};
  if (t == "Conv2d") return {LT::Conv2d, -1};
  if (t == "LayerNorm") return {LT::LayerNorm, -1};
  if (t == "RMSNorm") return {LT::RMSNorm, -1};
  if (t == "GroupNorm") return {LT::GroupNorm, -1};
  if (t == "Softmax") return {LT::Softmax, -1};
  if (t == "LogSoftmax") return {LT::LogSoftmax, -1};
  if (t == "GELU") return {LT::Act, MIMIR_B200_ELT_GELU};
  if (t == "SiLU") return {LT::Act, MIMIR_B200_ELT_SILU};
  if (t == "ReLU") return {LT::Act, MIMIR_B200_ELT_RELU};
  if (t == "Tanh") return {LT::Act, MIMIR_B200_ELT_TANH};
  if (t == "Sigmoid") return {LT::Act, MIMIR_B200_ELT_SIGMOID};
  if (t == "Add") return {LT::Add, -1};
  if (t == "Multiply") return {LT::Multiply, -1};
  if (t == "Embedding") return {LT::Embedding, -1};
  if (t == "UpsampleNearest") return {LT::UpsampleNearest, -1};
  if (t == "Permute") return {LT::Permute, -1};
  if (t == "Concat") return {LT::Concat, -1};
  // pass-through layers at inference (LayerOps.hpp:117-136, 629-662)
  if (t == "Identity" || t == "Reshape" || t == "Flatten" || t == "View" || t == "Dropout" || t == "Dropout2d" ||
      t == "AlphaDropout")
    return {LT::Alias, -1};
  // Squeeze / Unsqueeze only edit a shape vector that nobody reads (LayerOpsExt.hpp:160-208); Reparameterize
  // at inference copies mu, its first input (Model.cpp:5767-5770)
  if (t == "Squeeze" || t == "Unsqueeze" || t == "Reparameterize") return {LT::Alias, -1};
  if (t == "LeakyReLU") return {LT::Act, MIMIR_B200_ELT_LEAKY_RELU};
  if (t == "Softplus") return {LT::Act, MIMIR_B200_ELT_SOFTPLUS};
  if (t == "Mish") return {LT::Act, MIMIR_B200_ELT_MISH};
  if (t == "HardSigmoid") return {LT::Act, MIMIR_B200_ELT_HARD_SIGMOID};
  if (t == "HardSwish") return {LT::Act, MIMIR_B200_ELT_HARD_SWISH};
  if (t == "Subtract") return {LT::Binary2, MIMIR_B200_ELT_SUBTRACT};
  if (t == "Divide") return {LT::Binary2, MIMIR_B200_ELT_DIVIDE};
  if (t == "CrossAttention") return {LT::CrossAttention, -1};
  if (t == "Split") return {LT::Split, 0};
  if (t == "Chunk") return {LT::Split, 1};
  if (t == "Stack") return {LT::Concat, -1};  // flat append of equal-sized inputs (LayerOpsExt.hpp:245-272)
  if (t == "DepthwiseConv2d") return {LT::DepthwiseConv2d, -1};
  if (t == "Conv1d") return {LT::Conv1d, -1};
  if (t == "ConvTranspose2d") return {LT::ConvTranspose2d, -1};
  if (t == "MaxPool2d") return {LT::Pool2d, 1};
  if (t == "AvgPool2d") return {LT::Pool2d, 0};
  if (t == "AvgPool1d") return {LT::Pool2d, 2};  // one row per channel (LayerOpsExt.hpp:540-575)
  // LayerOpsExt::maxpool1d_forward (LayerOpsExt.hpp:504-538); the reference's own switch has no case that calls it
  if (t == "MaxPool1d") return {LT::Pool2d, 3};
  if (t == "EmbeddingBag") return {LT::EmbeddingBag, -1};
  if (t == "PatchEmbed") return {LT::PatchEmbed, -1};
  if (t == "Bilinear") return {LT::Bilinear, -1};
  if (t == "RNN") return {LT::Recurrent, 0};
  if (t == "GRU") return {LT::Recurrent, 1};
  if (t == "LSTM") return {LT::Recurrent, 2};
  if (t == "ZeroPad2d") return {LT::Pad2d, 0};
  if (t == "ReflectionPad2d") return {LT::Pad2d, 1};
  if (t == "ReplicationPad2d") return {LT::Pad2d, 2};
  if (t == "PixelShuffle") return {LT::PixelShuffle, -1};
  if (t == "UpsampleBilinear") return {LT::UpsampleBilinear, 0};
  if (t == "UpsampleBicubic") return {LT::UpsampleBilinear, 1};  // bilinear with half-pixel centres (LayerOpsExt.hpp:695-744)
  if (t == "MatMul") return {LT::MatMul, -1};
  if (t == "BatchMatMul") return {LT::BatchMatMul, -1};
  if (t == "BatchNorm2d" || t == "BatchNorm1d") return {LT::BatchNorm, -1};
  if (t == "InstanceNorm2d") return {LT::InstanceNorm, -1};
  if (t == "Transpose") return {LT::Transpose, -1};
  if (t == "TokenMeanPool") return {LT::TokenMeanPool, -1};
  if (t == "GlobalAvgPool2d" || t == "AdaptiveAvgPool2d") return {LT::GlobalAvgPool, -1};
  return {LT::Unsupported, -1};
}

struct LayerRT {
  // descriptor (strings owned here)
  std::string name, type, output;
  std::vector<std::string> inputs;
  MimirLayerDesc d{};
  LT lt = LT::Unsupported;
  int act_of_type = -1;
  // weights
  float* w_f32 = nullptr;
  size_t w_count = 0;
  __nv_bfloat16* w_split = nullptr;   // Linear / Conv2d operand, or Wqkv^T for attention
  float w_scale = 1.0f;               // every plane set of the layer holds its weights times this power of two
  size_t w_split_bytes = 0;
  __nv_bfloat16* w_split2 = nullptr;  // Wout^T for attention
  size_t w_split2_bytes = 0;
  __nv_bfloat16* w_split3 = nullptr;  // Wout^T for cross attention (w_split = Wq^T, w_split2 = Wkv^T)
  size_t w_split3_bytes = 0;
  int w_split_k = -1;                 // K the planes were built for (Linear in_features may be implicit)
  // plan
  std::vector<int> in_v;              // tensor versions read
  int out_v = -1;
  std::vector<int> piece_v;           // Split / Chunk: the tensors "<output>_i"
  std::vector<int64_t> piece_n;
  bool skip = false;                  // activation folded into its producer
  int fused_act = -1;                 // activation folded into this layer
  bool emit_split = false;            // GEMM writes hi/lo planes for the consuming Linear
  bool emit_f32 = true;
  bool read_split = false;            // Linear reads the producer's planes
  int res_v = -1;                     // residual tensor folded in from a following Add
  int pre_norm = -1;                  // Conv2d: index of the GroupNorm layer applied while its operand planes are laid out
  bool in_up = false;                 // Conv2d: in_v[0] is the INPUT of a 2 x 2 nearest upsample that the layout pass applies
  int gn_emit_for = -1;               // Conv2d: index of the GroupNorm layer whose statistics this layer's GEMM epilogue emits
  int gn_stats_from = -1;             // GroupNorm: index of the Conv2d layer that emits its statistics
  size_t gn_stats_off = 0;            // Conv2d with gn_emit_for >= 0: offset of the statistics [batch][groups][2] in the arena
  // decode twin (see mimir_b200_model_decode_begin): weights borrowed from the main model, key / value caches owned
  bool borrowed_f32 = false, borrowed_planes = false;
  float* kcache = nullptr;
  float* vcache = nullptr;
  size_t cache_bytes = 0;
  float* w_t_f32 = nullptr;           // attention of a twin with <= 16 samples: Wqkv^T [3E][E] then Wout^T [E][E], fp32
  size_t w_t_bytes = 0;
  size_t ws_off = 0, ws_bytes = 0;
  // resolved shapes (per sample)
  int rows_ps = 1, in_f = 0, out_f = 0;       // Linear
  int seq = 0, embed = 0, heads = 1;          // Attention (cross attention: seq = query length)
  int kv_len = 0;                             // CrossAttention
  int kk = 0, kw = 0, st = 1, sw = 1, pd = 0, pw = 0;  // resolved kernel / stride / pad of the spatial ops
  int mm_b = 1, mm_m = 0, mm_k = 0, mm_n = 0; // MatMul / BatchMatMul
  int h = 0, w = 0, oh = 0, ow = 0;           // Conv2d / GroupNorm / Upsample
  int ch = 0;
  int64_t norm_n = 0;                         // LayerNorm group size
};

struct TensorV {
  std::string name;
  int64_t n = 0;          // per-sample elements
  int producer = -1;      // layer index, -1 = graph input
  std::vector<int> consumers;
  int alias_of = -1;
  bool broadcast_input = false;
  bool want_f32 = true, want_split = false;
  int64_t split_rows_ps = 0;
  int split_k = 0;
  size_t off_f32 = 0, off_split = 0;
  int first = 0, last = 0;
};

struct Block { size_t off, size; };

// First-fit free list over one linear arena; freed ranges are merged with their neighbours.
struct ArenaSim {
  std::vector<Block> free_list;
  size_t end = 0, peak = 0;
  size_t alloc(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    for (size_t i = 0; i < free_list.size(); ++i) {
      if (free_list[i].size >= bytes) {
        const size_t off = free_list[i].off;
        free_list[i].off += bytes;
        free_list[i].size -= bytes;
        if (free_list[i].size == 0) free_list.erase(free_list.begin() + i);
        return off;
      }
    }
    // extend; if the last free block touches the end, grow from it
    if (!free_list.empty() && free_list.back().off + free_list.back().size == end) {
      const size_t off = free_list.back().off;
      end = off + bytes;
      free_list.pop_back();
      peak = std::max(peak, end);
      return off;
    }
    const size_t off = end;
    end += bytes;
    peak = std::max(peak, end);
    return off;
  }
  void release(size_t off, size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    Block b{off, bytes};
    auto it = std::lower_bound(free_list.begin(), free_list.end(), b, [](const Block& a, const Block& c) { return a.off < c.off; });
    it = free_list.insert(it, b);
    if (it + 1 != free_list.end() && it->off + it->size == (it + 1)->off) {
      it->size += (it + 1)->size;
      free_list.erase(it + 1);
    }
    if (it != free_list.begin() && (it - 1)->off + (it - 1)->size == it->off) {
      (it - 1)->size += it->size;
      free_list.erase(it);
    }
  }
};

}  // namespace
}  // namespace mb

struct MimirB200Model {
  std::vector<mb::LayerRT> layers;
  std::vector<mb::TensorV> tensors;
  std::map<std::string, int> input_v;  // graph input name -> tensor version
  int precision = MIMIR_B200_PREC_BF16X2;
  int device = 0;  // the CUDA device the model lives on: the creating thread's current device
  int planned_batch = 0;
  int out_v = -1;
  uint8_t* arena = nullptr;
  size_t arena_bytes = 0;
  size_t weight_bytes = 0;
  uint64_t flops = 0, hbm_bytes = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  float last_ms = 0.f;
  // Host-pointer forwards can be pipelined: the batch is cut into `pipeline` micro-batches that
  // flow through copy-in / compute / copy-out streams over two arena buffers.
  int pipeline = 1;
  int planned_micro = 0;
  bool out_in_input_slot = false;  // the output tensor shares bytes with a graph input's slot in the current plan
  uint8_t* arena2 = nullptr;
  cudaStream_t s_h2d = nullptr, s_comp = nullptr, s_d2h = nullptr;
  std::vector<cudaEvent_t> ev_h2d, ev_comp, ev_d2h;
  // The layer loop of one (batch, arena, bound pointers) combination, captured into a CUDA graph the second
  // time it is seen and replayed afterwards: one launch instead of one per layer.
  struct CachedGraph {
    std::vector<const void*> key;
    cudaGraphExec_t exec = nullptr;
    uint64_t launches = 0;  // kernels inside, for the launch counter
    int seen = 0;
    bool unusable = false;  // capture failed once: keep launching layer by layer
  };
  std::vector<CachedGraph> graphs;
  cudaStream_t s_capture = nullptr;
  // Incremental decoding: a second plan of the same layers for ONE token per sample, sharing this model's weights,
  // whose attention layers keep their keys and values in caches of max_seq positions.
  MimirB200Model* decode = nullptr;
  bool is_twin = false;
  int decode_pos = 0, max_seq = 0;
  uint64_t plan_epoch = 0, twin_epoch = 0;
  float* decode_scratch = nullptr;  // partial softmax results of the decode attention, shared by the twin's layers
  size_t decode_scratch_bytes = 0;
  int* pos_dev = nullptr;           // set when every attention layer of the twin can read its position on the device:
                                    // the step is then a fixed launch sequence and is replayed as a CUDA graph
  float* skinny_scratch = nullptr;  // K-slice partial sums of the weight-streaming projections of a twin's attention
  size_t skinny_scratch_bytes = 0;
};

namespace mb {
namespace {

std::mutex g_models_mu;
std::set<MimirB200Model*> g_models;

void drop_graphs(MimirB200Model* m) {
  for (auto& g : m->graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  m->graphs.clear();
}

int root_of(const std::vector<TensorV>& ts, int v) {
  while (ts[v].alias_of >= 0) v = ts[v].alias_of;
  return v;
}

void free_layer_weights(LayerRT& L, MimirB200Model* m) {
  if (L.borrowed_f32) L.w_f32 = nullptr;
  if (L.borrowed_planes) L.w_split = L.w_split2 = L.w_split3 = nullptr;
  if (L.w_f32) { dev_free(L.w_f32, L.w_count * 4); m->weight_bytes -= L.w_count * 4; L.w_f32 = nullptr; }
  if (L.w_split) { dev_free(L.w_split, L.w_split_bytes); m->weight_bytes -= L.w_split_bytes; L.w_split = nullptr; }
  if (L.w_split2) { dev_free(L.w_split2, L.w_split2_bytes); m->weight_bytes -= L.w_split2_bytes; L.w_split2 = nullptr; }
  if (L.w_split3) { dev_free(L.w_split3, L.w_split3_bytes); m->weight_bytes -= L.w_split3_bytes; L.w_split3 = nullptr; }
  L.w_split_k = -1;
}

// Builds the tensor-core operand planes of a layer's weights once its K is known.
int prepare_weight_planes(MimirB200Model* m, LayerRT& L, cudaStream_t st) {
  int ap, wp;
  precision_planes(m->precision, &ap, &wp);
  if (L.lt == LT::Linear) {
    if (linear_uses_skinny(L.rows_ps * m->planned_micro, m->precision)) return MIMIR_B200_OK;
    if (L.w_split && L.w_split_k == L.in_f) return MIMIR_B200_OK;
    if (L.w_split) { dev_free(L.w_split, L.w_split_bytes); m->weight_bytes -= L.w_split_bytes; L.w_split = nullptr; }
    L.w_split_bytes = split_bytes(L.out_f, L.in_f, wp);
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_split), L.w_split_bytes, "linear.w_planes"));
    m->weight_bytes += L.w_split_bytes;
    MB_TRY(weight_plane_scale(L.w_f32, static_cast<size_t>(L.out_f) * L.in_f, st, &L.w_scale));
    MB_TRY(launch_split(L.w_f32, L.w_split, L.out_f, L.in_f, wp, st, L.w_scale));
    L.w_split_k = L.in_f;
  } else if (L.lt == LT::Conv2d) {
    const int k = L.d.in_channels * L.d.kernel * L.d.kernel;
    if (L.w_split && L.w_split_k == k) return MIMIR_B200_OK;
    L.w_split_bytes = split_bytes(L.d.out_channels, k, wp);
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_split), L.w_split_bytes, "conv.w_planes"));
    m->weight_bytes += L.w_split_bytes;
    MB_TRY(weight_plane_scale(L.w_f32, static_cast<size_t>(L.d.out_channels) * k, st, &L.w_scale));
    if (conv_uses_shifted(L.d.in_channels, L.d.kernel, L.d.stride, L.d.padding))
      MB_TRY(launch_conv_weight_planes(L.w_f32, L.w_split, L.d.out_channels, L.d.in_channels, L.d.kernel, wp, st, L.w_scale));
    else
      MB_TRY(launch_split(L.w_f32, L.w_split, L.d.out_channels, k, wp, st, L.w_scale));
    L.w_split_k = k;
  } else if (L.lt == LT::Attention) {
    const int E = L.embed;
    if (L.w_split && L.w_split_k == E) return MIMIR_B200_OK;
    if (L.w_split) { dev_free(L.w_split, L.w_split_bytes); m->weight_bytes -= L.w_split_bytes; L.w_split = nullptr; }
    if (L.w_split2) { dev_free(L.w_split2, L.w_split2_bytes); m->weight_bytes -= L.w_split2_bytes; L.w_split2 = nullptr; }
    L.w_split_bytes = split_bytes(3 * E, E, wp);
    L.w_split2_bytes = split_bytes(E, E, wp);
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_split), L.w_split_bytes, "attn.wqkv_planes"));
    m->weight_bytes += L.w_split_bytes;
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_split2), L.w_split2_bytes, "attn.wout_planes"));
    m->weight_bytes += L.w_split2_bytes;
    MB_TRY(weight_plane_scale(L.w_f32, static_cast<size_t>(4) * E * E, st, &L.w_scale));
    MB_TRY(launch_split_transposed(L.w_f32, L.w_split, E, 3 * E, wp, st, L.w_scale));
    MB_TRY(launch_split_transposed(L.w_f32 + static_cast<size_t>(3) * E * E, L.w_split2, E, E, wp, st, L.w_scale));
    L.w_split_k = E;
  } else if (L.lt == LT::CrossAttention) {
    // block = Wq[E][E] | Wkv[E][2E] | Wout[E][E], input-major (Model.cpp:5975-5982)
    const int E = L.embed;
    if (L.w_split && L.w_split_k == E) return MIMIR_B200_OK;
    if (L.w_split) { dev_free(L.w_split, L.w_split_bytes); m->weight_bytes -= L.w_split_bytes; L.w_split = nullptr; }
    if (L.w_split2) { dev_free(L.w_split2, L.w_split2_bytes); m->weight_bytes -= L.w_split2_bytes; L.w_split2 = nullptr; }
    if (L.w_split3) { dev_free(L.w_split3, L.w_split3_bytes); m->weight_bytes -= L.w_split3_bytes; L.w_split3 = nullptr; }
    L.w_split_bytes = split_bytes(E, E, wp);
    L.w_split2_bytes = split_bytes(2 * E, E, wp);
    L.w_split3_bytes = split_bytes(E, E, wp);
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_split), L.w_split_bytes, "xattn.wq_planes"));
    m->weight_bytes += L.w_split_bytes;
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_split2), L.w_split2_bytes, "xattn.wkv_planes"));
    m->weight_bytes += L.w_split2_bytes;
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_split3), L.w_split3_bytes, "xattn.wout_planes"));
    m->weight_bytes += L.w_split3_bytes;
    const size_t EE = static_cast<size_t>(E) * E;
    MB_TRY(weight_plane_scale(L.w_f32, 4 * EE, st, &L.w_scale));
    MB_TRY(launch_split_transposed(L.w_f32, L.w_split, E, E, wp, st, L.w_scale));
    MB_TRY(launch_split_transposed(L.w_f32 + EE, L.w_split2, E, 2 * E, wp, st, L.w_scale));
    MB_TRY(launch_split_transposed(L.w_f32 + 3 * EE, L.w_split3, E, E, wp, st, L.w_scale));
    L.w_split_k = E;
  }
  return MIMIR_B200_OK;
}

// Per-sample output size of layer L given its input sizes; fills the resolved shape fields.
// Error texts follow the reference's RUNTIME_CHECK / throw messages where it has one.
int infer_layer(LayerRT& L, const std::vector<int64_t>& in_n, int64_t* out_n) {
  const MimirLayerDesc& d = L.d;
  const int64_t n0 = in_n.empty() ? 0 : in_n[0];
  switch (L.lt) {
    case LT::Linear: {
      if (d.out_features <= 0) return fail(MIMIR_B200_E_INVALID, "Linear: out_features not set");
      const int64_t in_f = d.in_features > 0 ? d.in_features : n0;
      L.in_f = static_cast<int>(in_f);
      L.out_f = d.out_features;
      if (d.seq_len > 0 && n0 == static_cast<int64_t>(d.seq_len) * in_f) L.rows_ps = d.seq_len;
      else if (n0 == in_f) L.rows_ps = 1;
      else return fail(MIMIR_B200_E_INVALID, "Linear (%s): input size %lld does not match in_features %lld", L.name.c_str(),
                       static_cast<long long>(n0), static_cast<long long>(in_f));
      const size_t need = static_cast<size_t>(in_f) * L.out_f + (d.use_bias ? L.out_f : 0);
      if (L.w_count < need) return fail(MIMIR_B200_E_INVALID, "Linear (%s): weights not uploaded or too small", L.name.c_str());
      *out_n = static_cast<int64_t>(L.rows_ps) * L.out_f;
      return MIMIR_B200_OK;
    }
    case LT::Attention: {
      L.seq = d.seq_len > 0 ? d.seq_len : 1;
      L.embed = d.embed_dim > 0 ? d.embed_dim : static_cast<int>(n0);
      L.heads = d.num_heads > 0 ? d.num_heads : 1;
      if (L.embed % L.heads != 0) return fail(MIMIR_B200_E_INVALID, "SelfAttention: embed_dim must be divisible by num_heads");
      if (n0 != static_cast<int64_t>(L.seq) * L.embed) return fail(MIMIR_B200_E_INVALID, "SelfAttention: input size mismatch");
      if (L.w_count < static_cast<size_t>(4) * L.embed * L.embed)
        return fail(MIMIR_B200_E_INVALID, "Attention: weights not initialized. Call allocateParams() first.");
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    case LT::Conv2d: {
      if (d.in_channels <= 0 || d.out_channels <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: in_channels and out_channels must be set");
      if (d.kernel <= 0 || d.stride <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: kernel_size must be set");
      int h = d.input_height > 0 ? d.input_height : 64, w = d.input_width > 0 ? d.input_width : 64;
      // size re-inference of Model.cpp:4916-4944
      if (n0 % d.in_channels == 0) {
        const int64_t hw = n0 / d.in_channels;
        if (static_cast<int64_t>(h) * w != hw) {
          if (d.input_height > 0 && hw % d.input_height == 0) { h = d.input_height; w = static_cast<int>(hw / h); }
          else if (d.input_width > 0 && hw % d.input_width == 0) { w = d.input_width; h = static_cast<int>(hw / w); }
          else {
            const int64_t s = llround(sqrt(static_cast<double>(hw)));
            if (s > 0 && s * s == hw) { h = static_cast<int>(s); w = static_cast<int>(s); }
          }
        }
      }
      if (static_cast<int64_t>(d.in_channels) * h * w != n0) return fail(MIMIR_B200_E_INVALID, "Conv2d (%s): input size mismatch", L.name.c_str());
      L.h = h; L.w = w; L.ch = d.in_channels;
      L.oh = (h + 2 * d.padding - d.kernel) / d.stride + 1;
      L.ow = (w + 2 * d.padding - d.kernel) / d.stride + 1;
      if (L.oh <= 0 || L.ow <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d (%s): empty output", L.name.c_str());
      if (L.w_count < static_cast<size_t>(d.out_channels) * d.in_channels * d.kernel * d.kernel)
        return fail(MIMIR_B200_E_INVALID, "Conv2d: weights invalid");
      *out_n = static_cast<int64_t>(d.out_channels) * L.oh * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::LayerNorm: {
      L.norm_n = d.in_features > 0 ? d.in_features : n0;
      if (L.norm_n <= 0 || n0 % L.norm_n != 0) return fail(MIMIR_B200_E_INVALID, "LayerNorm: invalid normalized_size");
      if (d.affine && L.w_count < static_cast<size_t>(L.norm_n) * (d.use_bias ? 2 : 1))
        return fail(MIMIR_B200_E_INVALID, "LayerNorm (%s): weights not uploaded or too small", L.name.c_str());
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    case LT::RMSNorm:
    case LT::Softmax:
    case LT::LogSoftmax:
    case LT::Act:
    case LT::Alias:
      if (n0 <= 0) return fail(MIMIR_B200_E_INVALID, "%s: empty input", L.type.c_str());
      *out_n = n0;
      return MIMIR_B200_OK;
    case LT::GroupNorm: {
      L.ch = d.in_channels > 0 ? d.in_channels : 64;
      L.h = d.input_height > 0 ? d.input_height : 32;
      L.w = d.input_width > 0 ? d.input_width : 32;
      if (d.num_groups <= 0 || L.ch % d.num_groups != 0) return fail(MIMIR_B200_E_INVALID, "GroupNorm: channels must be divisible by num_groups");
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "GroupNorm (%s): input size mismatch", L.name.c_str());
      if (d.affine && L.w_count < static_cast<size_t>(L.ch) * (d.use_bias ? 2 : 1))
        return fail(MIMIR_B200_E_INVALID, "GroupNorm (%s): weights not uploaded or too small", L.name.c_str());
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    case LT::Add:
    case LT::Multiply: {
      if (in_n.size() < 2) return fail(MIMIR_B200_E_INVALID, "%s layer requires 2 inputs, got %zu", L.type.c_str(), in_n.size());
      const int64_t a = in_n[0], b = in_n[1];
      if (a <= 0 || b <= 0) return fail(MIMIR_B200_E_INVALID, "Add: inputs must be non-empty");
      if (L.lt == LT::Multiply && a != b) return fail(MIMIR_B200_E_INVALID, "Multiply: input sizes must match");
      const int64_t big = std::max(a, b), small = std::min(a, b);
      if (big != small && small != 1 && big % small != 0)
        return fail(MIMIR_B200_E_INVALID, "Add: input sizes must match or be broadcastable");
      *out_n = big;
      return MIMIR_B200_OK;
    }
    case LT::Embedding: {
      if (L.w_count < static_cast<size_t>(std::max(1, d.vocab_size)) * std::max(1, d.embed_dim))
        return fail(MIMIR_B200_E_INVALID, "Embedding: invalid weight size");
      *out_n = n0 * std::max(1, d.embed_dim);
      return MIMIR_B200_OK;
    }
    case LT::UpsampleNearest: {
      if (d.out_h <= 0 || d.out_w <= 0 || d.in_channels <= 0)
        return fail(MIMIR_B200_E_INVALID, "UpsampleNearest: dimensions (out_h, out_w, in_channels) must be set");
      L.h = d.out_h; L.w = d.out_w; L.ch = d.in_channels;  // out_h/out_w are the INPUT size (Model.cpp:6008-6009)
      const int sh = d.scale_h > 0 ? d.scale_h : 2, sw = d.scale_w > 0 ? d.scale_w : 2;
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "UpsampleNearest (%s): input size mismatch", L.name.c_str());
      L.oh = L.h * sh; L.ow = L.w * sw;
      *out_n = static_cast<int64_t>(L.ch) * L.oh * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::Permute: {
      if (d.n_dims <= 0) return fail(MIMIR_B200_E_INVALID, "Permute: permute_dims must be configured");
      int64_t tot = 1;
      for (int i = 0; i < d.n_dims; ++i) tot *= d.shape[i];
      if (tot != n0) return fail(MIMIR_B200_E_INVALID, "Permute (%s): shape does not match the input size", L.name.c_str());
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    case LT::Concat: {
      if (in_n.size() < 2) return fail(MIMIR_B200_E_INVALID, "Concat requires at least 2 inputs, got %zu", in_n.size());
      int64_t s = 0;
      for (int64_t v : in_n) s += v;
      *out_n = s;
      return MIMIR_B200_OK;
    }
    case LT::TokenMeanPool:
      if (d.seq_len <= 0 || d.embed_dim <= 0) return fail(MIMIR_B200_E_INVALID, "TokenMeanPool: seq_len and embed_dim must be set");
      if (n0 != static_cast<int64_t>(d.seq_len) * d.embed_dim) return fail(MIMIR_B200_E_INVALID, "TokenMeanPool: input size mismatch");
      *out_n = d.embed_dim;
      return MIMIR_B200_OK;
    case LT::GlobalAvgPool: {
      L.ch = d.in_channels > 0 ? d.in_channels : 64;
      L.h = d.input_height > 0 ? d.input_height : 32;
      L.w = d.input_width > 0 ? d.input_width : 32;
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "GlobalAvgPool2d (%s): input size mismatch", L.name.c_str());
      *out_n = L.ch;
      return MIMIR_B200_OK;
    }
    case LT::Binary2: {
      if (in_n.size() < 2) return fail(MIMIR_B200_E_INVALID, "%s layer requires 2 inputs, got %zu", L.type.c_str(), in_n.size());
      if (in_n[0] != in_n[1] || n0 <= 0)
        return fail(MIMIR_B200_E_INVALID, "%s: size mismatch: %lld vs %lld", L.type.c_str(), static_cast<long long>(in_n[0]),
                    static_cast<long long>(in_n[1]));
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    case LT::CrossAttention: {
      if (in_n.size() < 2) return fail(MIMIR_B200_E_INVALID, "CrossAttention requires 2 inputs (query, key_value), got %zu", in_n.size());
      L.heads = d.num_heads > 0 ? d.num_heads : 1;
      L.embed = d.embed_dim;
      if (L.embed <= 0 && d.head_dim > 0) L.embed = d.head_dim * L.heads;
      if (L.embed <= 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: embed_dim must be configured (set layer.embed_dim or head_dim*num_heads)");
      if (in_n[0] % L.embed != 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: query input size must be divisible by embed_dim");
      if (in_n[1] % L.embed != 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: key/value input size must be divisible by embed_dim");
      L.seq = static_cast<int>(in_n[0] / L.embed);
      L.kv_len = static_cast<int>(in_n[1] / L.embed);
      if (L.seq <= 0 || L.kv_len <= 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: invalid sequence lengths");
      if (L.embed % L.heads != 0) return fail(MIMIR_B200_E_INVALID, "CrossAttention: embed_dim must be divisible by num_heads");
      if (L.w_count < static_cast<size_t>(4) * L.embed * L.embed)
        return fail(MIMIR_B200_E_INVALID, "CrossAttention: weights not initialized. Call allocateParams() first.");
      *out_n = in_n[0];
      return MIMIR_B200_OK;
    }
    case LT::Split: {
      L.piece_n.clear();
      if (L.act_of_type == 0) {  // Split (Model.cpp:5802-5815, LayerOps.hpp:759-795)
        if (d.n_splits < 0) return fail(MIMIR_B200_E_UNSUPPORTED, "Split (%s): more than %d pieces", L.name.c_str(), MIMIR_B200_MAX_SPLITS);
        if (d.n_splits == 0) return fail(MIMIR_B200_E_INVALID, "Split: split_sizes must be configured");
        int64_t tot = 0;
        for (int i = 0; i < d.n_splits; ++i) {
          if (d.split_sizes[i] <= 0) return fail(MIMIR_B200_E_INVALID, "Split: all split_sizes must be positive");
          L.piece_n.push_back(d.split_sizes[i]);
          tot += d.split_sizes[i];
        }
        if (tot != n0)
          return fail(MIMIR_B200_E_INVALID, "Split: sum of split_sizes (%lld) != input size (%lld)", static_cast<long long>(tot),
                      static_cast<long long>(n0));
      } else {  // Chunk (Model.cpp:5817-5832, LayerOpsExt.hpp:215-240): the first `remainder` chunks get one more
        if (d.num_chunks <= 0) return fail(MIMIR_B200_E_INVALID, "Chunk: num_chunks must be set");
        const int64_t base = n0 / d.num_chunks, rem = n0 % d.num_chunks;
        if (base == 0) return fail(MIMIR_B200_E_UNSUPPORTED, "Chunk (%s): more chunks than elements", L.name.c_str());
        for (int i = 0; i < d.num_chunks; ++i) L.piece_n.push_back(base + (i < rem ? 1 : 0));
      }
      *out_n = L.piece_n[0];
      return MIMIR_B200_OK;
    }
    case LT::DepthwiseConv2d: {  // LayerOpsExt.hpp:446-455: raw kernel_h / stride_h / pad_h
      L.ch = d.in_channels > 0 ? d.in_channels : 3;
      L.h = d.input_height > 0 ? d.input_height : 32;
      L.w = d.input_width > 0 ? d.input_width : 32;
      L.kk = d.raw_kernel_h > 0 ? d.raw_kernel_h : 3;
      L.st = d.raw_stride_h > 0 ? d.raw_stride_h : 1;
      L.pd = d.raw_pad_h >= 0 ? d.raw_pad_h : 0;
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "DepthwiseConv2d (%s): input size mismatch", L.name.c_str());
      L.oh = (L.h + 2 * L.pd - L.kk) / L.st + 1;
      L.ow = (L.w + 2 * L.pd - L.kk) / L.st + 1;
      if (L.oh <= 0 || L.ow <= 0) return fail(MIMIR_B200_E_INVALID, "DepthwiseConv2d (%s): empty output", L.name.c_str());
      if (L.w_count < static_cast<size_t>(L.ch) * L.kk * L.kk + (d.use_bias ? L.ch : 0))
        return fail(MIMIR_B200_E_INVALID, "DepthwiseConv2d (%s): weights not uploaded or too small", L.name.c_str());
      *out_n = static_cast<int64_t>(L.ch) * L.oh * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::Conv1d: {  // LayerOpsExt.hpp:392-399
      L.ch = d.in_channels > 0 ? d.in_channels : 1;
      const int oc = d.out_channels > 0 ? d.out_channels : 1;
      L.kk = d.raw_kernel_h > 0 ? d.raw_kernel_h : 3;
      L.st = d.raw_stride_h > 0 ? d.raw_stride_h : 1;
      L.pd = d.raw_pad_h >= 0 ? d.raw_pad_h : 0;
      if (n0 % L.ch != 0) return fail(MIMIR_B200_E_INVALID, "Conv1d (%s): input size is not a multiple of in_channels", L.name.c_str());
      L.w = static_cast<int>(n0 / L.ch);
      L.ow = (L.w + 2 * L.pd - L.kk) / L.st + 1;
      if (L.ow <= 0) return fail(MIMIR_B200_E_INVALID, "Conv1d (%s): empty output", L.name.c_str());
      if (L.w_count < static_cast<size_t>(oc) * L.ch * L.kk + (d.use_bias ? oc : 0))
        return fail(MIMIR_B200_E_INVALID, "Conv1d (%s): weights not uploaded or too small", L.name.c_str());
      L.out_f = oc;
      *out_n = static_cast<int64_t>(oc) * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::ConvTranspose2d: {  // Model.cpp:4908-4953
      if (d.in_channels <= 0 || d.out_channels <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: in_channels and out_channels must be set");
      if (d.kernel <= 0 || d.stride <= 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: kernel_size must be set");
      L.h = d.input_height > 0 ? d.input_height : 64;
      L.w = d.input_width > 0 ? d.input_width : 64;
      L.ch = d.in_channels;
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "ConvTranspose2d (%s): input size mismatch", L.name.c_str());
      L.oh = (L.h - 1) * d.stride - 2 * d.padding + d.kernel;
      L.ow = (L.w - 1) * d.stride - 2 * d.padding + d.kernel;
      if (L.oh <= 0 || L.ow <= 0) return fail(MIMIR_B200_E_INVALID, "ConvTranspose2d (%s): empty output", L.name.c_str());
      if (L.w_count < static_cast<size_t>(d.out_channels) * d.in_channels * d.kernel * d.kernel)
        return fail(MIMIR_B200_E_INVALID, "Conv2d: weights invalid");
      *out_n = static_cast<int64_t>(d.out_channels) * L.oh * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::Pool2d: {
      if (L.act_of_type >= 2) {  // AvgPool1d / MaxPool1d: raw kernel_h (default 2), raw stride_h (default = kernel), raw pad_h
        L.ch = d.in_channels > 0 ? d.in_channels : 1;
        if (n0 % L.ch != 0) return fail(MIMIR_B200_E_INVALID, "%s (%s): input size is not a multiple of in_channels", L.type.c_str(), L.name.c_str());
        L.h = 1; L.w = static_cast<int>(n0 / L.ch);
        L.kk = 1; L.kw = d.raw_kernel_h > 0 ? d.raw_kernel_h : 2;
        L.st = 1; L.sw = d.raw_stride_h > 0 ? d.raw_stride_h : L.kw;
        L.pd = 0; L.pw = d.raw_pad_h >= 0 ? d.raw_pad_h : 0;
        L.oh = 1; L.ow = (L.w + 2 * L.pw - L.kw) / L.sw + 1;
        if (L.ow <= 0) return fail(MIMIR_B200_E_INVALID, "%s (%s): empty output", L.type.c_str(), L.name.c_str());
        *out_n = static_cast<int64_t>(L.ch) * L.ow;
        return MIMIR_B200_OK;
      }
      const bool is_max = L.act_of_type == 1;
      L.ch = d.in_channels > 0 ? d.in_channels : 64;
      L.h = d.input_height > 0 ? d.input_height : (is_max ? 64 : 32);  // Model.cpp:5511-5512 vs LayerOps.hpp:416-417
      L.w = d.input_width > 0 ? d.input_width : (is_max ? 64 : 32);
      L.kk = d.kernel; L.st = d.stride; L.pd = d.padding;
      L.kw = is_max ? d.kernel : (d.kernel_w > 0 ? d.kernel_w : d.kernel);
      L.sw = is_max ? d.stride : (d.stride_w > 0 ? d.stride_w : d.stride);
      L.pw = is_max ? d.padding : d.padding_w;
      if (L.kk <= 0 || L.kw <= 0) return fail(MIMIR_B200_E_INVALID, "MaxPool2d: kernel_size must be > 0");
      if (L.st <= 0 || L.sw <= 0) return fail(MIMIR_B200_E_INVALID, "MaxPool2d: stride must be > 0");
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "%s (%s): input size mismatch", L.type.c_str(), L.name.c_str());
      L.oh = (L.h + 2 * L.pd - L.kk) / L.st + 1;
      L.ow = (L.w + 2 * L.pw - L.kw) / L.sw + 1;
      if (L.oh <= 0 || L.ow <= 0) return fail(MIMIR_B200_E_INVALID, "MaxPool2d: output dimensions must be > 0");
      *out_n = static_cast<int64_t>(L.ch) * L.oh * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::Pad2d: {  // LayerOpsExt.hpp:586-595, 618-624
      L.ch = d.in_channels > 0 ? d.in_channels : 3;
      L.h = d.input_height > 0 ? d.input_height : 32;
      L.w = d.input_width > 0 ? d.input_width : 32;
      L.pd = d.raw_pad_h >= 0 ? d.raw_pad_h : 1;
      L.pw = (L.act_of_type == 0) ? (d.raw_pad_w >= 0 ? d.raw_pad_w : 1) : L.pd;  // reflection / replication pad both axes by pad_h
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "%s (%s): input size mismatch", L.type.c_str(), L.name.c_str());
      L.oh = L.h + 2 * L.pd; L.ow = L.w + 2 * L.pw;
      *out_n = static_cast<int64_t>(L.ch) * L.oh * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::PixelShuffle: {  // LayerOpsExt.hpp:753-768
      L.kk = d.scale_h > 0 ? d.scale_h : 2;
      L.ch = d.in_channels > 0 ? d.in_channels : 12;
      L.h = d.input_height > 0 ? d.input_height : 32;
      L.w = d.input_width > 0 ? d.input_width : 32;
      if (L.ch % (L.kk * L.kk) != 0)
        return fail(MIMIR_B200_E_INVALID, "PixelShuffle: in_channels (%d) must be divisible by upscale_factor^2 (%d)", L.ch, L.kk * L.kk);
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "PixelShuffle (%s): input size mismatch", L.name.c_str());
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    case LT::UpsampleBilinear: {  // Model.cpp:6020-6054: out_h / out_w are the INPUT size, the factor is always 2
      if (d.out_h <= 0 || d.out_w <= 0 || (L.act_of_type == 0 && d.in_channels <= 0))
        return fail(MIMIR_B200_E_INVALID, "%s: dimensions must be set", L.type.c_str());
      L.h = d.out_h; L.w = d.out_w;
      L.ch = d.in_channels > 0 ? d.in_channels : 3;
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0) return fail(MIMIR_B200_E_INVALID, "%s (%s): input size mismatch", L.type.c_str(), L.name.c_str());
      L.oh = 2 * L.h; L.ow = 2 * L.w;
      *out_n = static_cast<int64_t>(L.ch) * L.oh * L.ow;
      return MIMIR_B200_OK;
    }
    case LT::MatMul:
    case LT::BatchMatMul: {  // Model.cpp:5847-5898: M = in_features, K = out_features, N = embed_dim, batch = seq_len
      if (in_n.size() < 2) return fail(MIMIR_B200_E_INVALID, "%s requires 2 inputs", L.type.c_str());
      const bool bmm = L.lt == LT::BatchMatMul;
      if (d.in_features <= 0 || d.out_features <= 0 || d.embed_dim <= 0 || (bmm && d.seq_len <= 0))
        return fail(MIMIR_B200_E_INVALID, "%s: dimensions (in_features, out_features, embed_dim) must be configured", L.type.c_str());
      L.mm_b = bmm ? d.seq_len : 1; L.mm_m = d.in_features; L.mm_k = d.out_features; L.mm_n = d.embed_dim;
      if (in_n[0] != static_cast<int64_t>(L.mm_b) * L.mm_m * L.mm_k) return fail(MIMIR_B200_E_INVALID, "%s: A size mismatch", L.type.c_str());
      if (in_n[1] != static_cast<int64_t>(L.mm_b) * L.mm_k * L.mm_n) return fail(MIMIR_B200_E_INVALID, "%s: B size mismatch", L.type.c_str());
      *out_n = static_cast<int64_t>(L.mm_b) * L.mm_m * L.mm_n;
      return MIMIR_B200_OK;
    }
    case LT::BatchNorm:
      if (n0 <= 0) return fail(MIMIR_B200_E_INVALID, "%s: empty input", L.type.c_str());
      *out_n = n0;
      return MIMIR_B200_OK;
    case LT::InstanceNorm: {  // LayerOpsExt.hpp:282-294
      L.ch = d.in_channels > 0 ? d.in_channels : 3;
      L.h = d.input_height > 0 ? d.input_height : 32;
      L.w = d.input_width > 0 ? d.input_width : 32;
      if (static_cast<int64_t>(L.ch) * L.h * L.w != n0)
        return fail(MIMIR_B200_E_INVALID, "InstanceNorm2d: input size mismatch. Expected %lld, got %lld",
                    static_cast<long long>(L.ch) * L.h * L.w, static_cast<long long>(n0));
      if (d.affine && L.w_count > 0 && L.w_count < static_cast<size_t>(2) * L.ch)
        return fail(MIMIR_B200_E_INVALID, "InstanceNorm2d (%s): weights too small", L.name.c_str());
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    case LT::EmbeddingBag: {  // Model.cpp:5336-5381: ids, optional offsets (num_bags + 1 entries); sum pooling
      if (L.w_count < static_cast<size_t>(std::max(1, d.vocab_size)) * std::max(1, d.embed_dim))
        return fail(MIMIR_B200_E_INVALID, "EmbeddingBag: invalid weight size");
      int64_t bags = 1;
      if (in_n.size() >= 2 && in_n[1] > 0) {
        if (in_n[1] < 2) return fail(MIMIR_B200_E_INVALID, "EmbeddingBag: offsets must have at least 2 entries");
        bags = in_n[1] - 1;
      }
      *out_n = bags * std::max(1, d.embed_dim);
      return MIMIR_B200_OK;
    }
    case LT::PatchEmbed: {  // Model.cpp:5203-5243
      const int d_model = d.embed_dim > 0 ? d.embed_dim : d.out_features;
      L.mm_b = std::max(1, d.seq_text); L.mm_m = std::max(1, d.num_patches); L.mm_k = std::max(1, d.patch_dim); L.mm_n = d_model;
      if (d_model <= 0 || n0 != static_cast<int64_t>(L.mm_b + 1) * d_model + static_cast<int64_t>(L.mm_m) * L.mm_k)
        return fail(MIMIR_B200_E_INVALID, "PatchEmbed: input size mismatch");
      if (L.w_f32 == nullptr || L.w_count != static_cast<size_t>(L.mm_k) * d_model + d_model)
        return fail(MIMIR_B200_E_INVALID, "PatchEmbed: weights not initialized or invalid size");
      *out_n = static_cast<int64_t>(L.mm_b + 1 + L.mm_m) * d_model;
      return MIMIR_B200_OK;
    }
    case LT::Bilinear: {  // Model.cpp:5247-5295: in1 = in_features, in2 = out_features, output width = embed_dim or target_shape[0]
      if (in_n.size() < 2) return fail(MIMIR_B200_E_INVALID, "Bilinear requires 2 inputs");
      const int in1 = std::max(1, d.in_features), in2 = std::max(1, d.out_features);
      const int out_f = d.embed_dim > 0 ? d.embed_dim : d.target_dim0;
      if (out_f <= 0) return fail(MIMIR_B200_E_INVALID, "Bilinear: set embed_dim (output dim) or target_shape[0]");
      if (in_n[0] % in1 != 0) return fail(MIMIR_B200_E_INVALID, "Bilinear: input0 size not divisible by in_features");
      if (in_n[1] % in2 != 0) return fail(MIMIR_B200_E_INVALID, "Bilinear: input1 size not divisible by out_features");
      if (in_n[0] / in1 != in_n[1] / in2) return fail(MIMIR_B200_E_INVALID, "Bilinear: batch mismatch between inputs");
      const size_t need = static_cast<size_t>(out_f) * in1 * in2 + (d.use_bias ? out_f : 0);
      if (L.w_f32 == nullptr || L.w_count < need) return fail(MIMIR_B200_E_INVALID, "Bilinear: weights not initialized/invalid size");
      L.mm_b = static_cast<int>(in_n[0] / in1); L.mm_m = in1; L.mm_k = in2; L.mm_n = out_f;
      *out_n = static_cast<int64_t>(L.mm_b) * out_f;
      return MIMIR_B200_OK;
    }
    case LT::Recurrent: {  // Model.cpp:6084-6262: x is [seq_len][in_features], the output [seq_len][out_features]
      if (d.seq_len <= 0) return fail(MIMIR_B200_E_INVALID, "Recurrent: seq_len must be set");
      if (d.in_features <= 0 || d.out_features <= 0) return fail(MIMIR_B200_E_INVALID, "Recurrent: in_features/out_features must be set");
      if (L.w_f32 == nullptr) return fail(MIMIR_B200_E_INVALID, "Recurrent: weights not initialized");
      if (n0 != static_cast<int64_t>(d.seq_len) * d.in_features)
        return fail(MIMIR_B200_E_INVALID, "Recurrent: input size mismatch (expected seq_len*in_features)");
      const size_t g = L.act_of_type == 0 ? 1 : (L.act_of_type == 1 ? 3 : 4), H = d.out_features, I = d.in_features;
      if (L.w_count < g * H * I + g * H * H + (d.use_bias ? 2 * g * H : 0))
        return fail(MIMIR_B200_E_INVALID, "%s: invalid weight size", L.type.c_str());
      L.mm_m = d.seq_len; L.mm_k = d.in_features; L.mm_n = d.out_features;
      *out_n = static_cast<int64_t>(d.seq_len) * d.out_features;
      return MIMIR_B200_OK;
    }
    case LT::Transpose: {  // Model.cpp:5649-5659: rows = in_features, cols = out_features
      if (d.in_features <= 0 || d.out_features <= 0) return fail(MIMIR_B200_E_INVALID, "Transpose: in_features and out_features must be set");
      if (n0 != static_cast<int64_t>(d.in_features) * d.out_features) return fail(MIMIR_B200_E_INVALID, "Transpose: input size mismatch");
      *out_n = n0;
      return MIMIR_B200_OK;
    }
    default:
      return fail(MIMIR_B200_E_UNSUPPORTED, "layer type '%s' (%s) is not supported by the B200 backend", L.type.c_str(), L.name.c_str());
  }
}

}  // namespace
}  // namespace mb

namespace mb {
namespace {

size_t f32_bytes(const TensorV& t, int batch) { return static_cast<size_t>(batch) * static_cast<size_t>(t.n) * 4; }
size_t splitv_bytes(const TensorV& t, int batch) { return split_bytes(static_cast<int64_t>(batch) * t.split_rows_ps, t.split_k, 2); }

int plan_model(MimirB200Model* m, const MimirNamedInput* inputs, int n_inputs, int batch) {
  if (batch <= 0) return fail(MIMIR_B200_E_INVALID, "plan: batch must be positive");
  if (batch % m->pipeline != 0)
    return fail(MIMIR_B200_E_INVALID, "plan: batch %d is not a multiple of the %d pipeline micro-batches", batch, m->pipeline);
  const int full_batch = batch;
  batch = batch / m->pipeline;  // everything below is sized for one micro-batch
  const int nl = static_cast<int>(m->layers.size());
  drop_graphs(m);  // offsets, fusion decisions and operand planes may all change
  if (!m->is_twin) ++m->plan_epoch;  // a decode twin made before this plan is stale
  m->tensors.clear();
  m->input_v.clear();
  m->planned_batch = 0;
  std::map<std::string, int> cur;
  for (int i = 0; i < n_inputs; ++i) {
    std::string name = (inputs[i].name && inputs[i].name[0]) ? inputs[i].name : "x";
    if (name == "__input__") name = "x";
    if (inputs[i].per_sample == 0) return fail(MIMIR_B200_E_INVALID, "plan: input '%s' is empty", name.c_str());
    TensorV t;
    t.name = name;
    t.n = static_cast<int64_t>(inputs[i].per_sample);
    t.broadcast_input = inputs[i].broadcast != 0;
    m->tensors.push_back(t);
    const int v = static_cast<int>(m->tensors.size()) - 1;
    cur[name] = v;
    m->input_v[name] = v;
    if (name == "x") cur["__input__"] = v;  // Model.cpp:4640-4642
  }
  for (int li = 0; li < nl; ++li) {
    LayerRT& L = m->layers[li];
    L.in_v.clear();
    L.out_v = -1;
    L.skip = false; L.fused_act = -1; L.emit_split = false; L.emit_f32 = true; L.read_split = false; L.res_v = -1; L.pre_norm = -1; L.in_up = false;
    L.ws_off = 0; L.ws_bytes = 0;
    std::vector<std::string> names = L.inputs;
    if (names.empty()) names.push_back("x");
    std::vector<int64_t> in_n;
    for (const auto& nm : names) {
      auto it = cur.find(nm);
      if (it == cur.end()) return fail(MIMIR_B200_E_INVALID, "Missing input tensor: %s (layer %d, %s)", nm.c_str(), li, L.name.c_str());
      L.in_v.push_back(it->second);
      in_n.push_back(m->tensors[it->second].n);
    }
    int64_t out_n = 0;
    MB_TRY(infer_layer(L, in_n, &out_n));
    L.piece_v.clear();
    if (L.lt == LT::Split) {
      // the pieces are stored as "<output>_<i>" and the layer's own output is piece 0 (Model.cpp:5808-5813)
      const std::string base = L.output.empty() ? "x" : L.output;
      for (size_t pi = 0; pi < L.piece_n.size(); ++pi) {
        TensorV pt;
        pt.name = base + "_" + std::to_string(pi);
        pt.n = L.piece_n[pi];
        pt.producer = li;
        m->tensors.push_back(pt);
        L.piece_v.push_back(static_cast<int>(m->tensors.size()) - 1);
        cur[pt.name] = L.piece_v.back();
      }
    }
    TensorV t;
    t.name = L.output.empty() ? "x" : L.output;
    t.n = out_n;
    t.producer = li;
    if (L.lt == LT::Alias) t.alias_of = root_of(m->tensors, L.in_v[0]);
    if (L.lt == LT::Split) t.alias_of = L.piece_v[0];
    m->tensors.push_back(t);
    L.out_v = static_cast<int>(m->tensors.size()) - 1;
    for (int v : L.in_v) m->tensors[v].consumers.push_back(li);
    cur[t.name] = L.out_v;
  }
  auto itx = cur.find("x");
  if (itx == cur.end()) return fail(MIMIR_B200_E_INVALID, "graph defines no tensor 'x'");
  m->out_v = itx->second;
  const int out_root = root_of(m->tensors, m->out_v);

  // consumers through aliases count for the root
  auto total_consumers = [&](int v) {
    size_t c = m->tensors[v].consumers.size();
    for (size_t a = 0; a < m->tensors.size(); ++a)
      if (m->tensors[a].alias_of == v) c += m->tensors[a].consumers.size() + 1;  // +1: the alias layer itself holds it
    return c;
  };

  // ---- fusion 1: activation into the producing GEMM / GroupNorm ---------------------------------
  for (int li = 0; li < nl; ++li) {
    LayerRT& A = m->layers[li];
    if (A.lt != LT::Act || A.act_of_type > MIMIR_B200_ELT_SIGMOID) continue;  // the epilogues know GELU..Sigmoid
    const int pv = A.in_v[0];
    TensorV& pt = m->tensors[pv];
    if (pt.alias_of >= 0 || pt.producer < 0 || pv == out_root || total_consumers(pv) != 1) continue;
    LayerRT& P = m->layers[pt.producer];
    if (P.fused_act >= 0 || P.out_v != pv) continue;
    const bool ok = (P.lt == LT::Linear) || (P.lt == LT::Conv2d && P.d.activation == 0) ||
                    (P.lt == LT::GroupNorm && A.act_of_type == MIMIR_B200_ELT_SILU);
    if (!ok) continue;
    P.fused_act = A.act_of_type;
    P.out_v = A.out_v;
    m->tensors[A.out_v].producer = pt.producer;
    pt.consumers.clear();
    pt.want_f32 = false;
    pt.producer = -2;  // dead
    A.skip = true;
  }
  // ---- fusion 1b: a residual Add into the epilogue of the layer that produces one of its operands -------
  for (int li = 0; li < nl; ++li) {
    LayerRT& A = m->layers[li];
    if (A.lt != LT::Add || A.skip || A.in_v.size() != 2) continue;
    if (m->tensors[A.in_v[0]].n != m->tensors[A.in_v[1]].n) continue;  // broadcast adds stay separate
    for (int side = 0; side < 2; ++side) {
      const int uv = A.in_v[side], ov = A.in_v[1 - side];
      TensorV& ut = m->tensors[uv];
      if (ut.alias_of >= 0 || ut.producer < 0 || uv == out_root || uv == ov || total_consumers(uv) != 1) continue;
      LayerRT& P = m->layers[ut.producer];
      if (P.out_v != uv || P.res_v >= 0 || P.skip) continue;
      // (a Linear on the weight-streaming path adds the residual in its finishing kernel)
      const bool gemm_like = P.lt == LT::Linear || P.lt == LT::Attention || P.lt == LT::CrossAttention || P.lt == LT::Conv2d;
      if (!gemm_like && P.lt != LT::GroupNorm) continue;
      // the other operand must already exist when P runs
      const int orr = root_of(m->tensors, ov);
      const TensorV& ot = m->tensors[orr];
      if (ot.producer >= ut.producer || ot.producer == -2 || !ot.want_f32) continue;
      P.res_v = ov;
      P.out_v = A.out_v;
      m->tensors[A.out_v].producer = ut.producer;
      // ov is now read by P instead of A
      for (int& c : m->tensors[ov].consumers)
        if (c == li) c = ut.producer;
      ut.consumers.clear();
      ut.want_f32 = false;
      ut.producer = -2;  // dead
      A.skip = true;
      break;
    }
  }
  // ---- fusion 1c: GroupNorm (+ SiLU) whose only consumer is a shifted-GEMM convolution: the convolution's layout
  //      kernel normalises on the fly from per-slab statistics, the normalised tensor never exists in memory ----
  // (MIMIR_B200_FUSE_GN_CONV=0 turns it off.  It removes a full write + read of the normalised tensor: the GroupNorm
  // becomes a read-only statistics sweep.  Measured on the UNet configuration: 6.60 against 6.80 ms per step.)
  const char* fuse_gn_env = getenv("MIMIR_B200_FUSE_GN_CONV");
  const bool fuse_gn = !(fuse_gn_env && fuse_gn_env[0] == '0');
  for (int li = 0; li < nl && fuse_gn; ++li) {
    LayerRT& P = m->layers[li];
    if (P.lt != LT::GroupNorm || P.skip || P.res_v >= 0) continue;
    if (P.fused_act >= 0 && P.fused_act != MIMIR_B200_ELT_SILU) continue;
    const int pv = P.out_v;
    TensorV& pt = m->tensors[pv];
    if (pt.alias_of >= 0 || pv == out_root || total_consumers(pv) != 1 || pt.consumers.size() != 1) continue;
    LayerRT& C = m->layers[pt.consumers[0]];
    if (C.lt != LT::Conv2d || C.skip || C.pre_norm >= 0 || C.in_v[0] != pv) continue;
    if (!conv_uses_shifted(C.d.in_channels, C.d.kernel, C.d.stride, C.d.padding)) continue;
    if (C.d.in_channels != P.ch || C.h != P.h || C.w != P.w) continue;
    // a convolution that takes the direct fp32 kernel reads the normalised tensor itself: it has no layout pass to fold into
    if (conv_small_oc_supported(C.d.out_channels, C.d.kernel, C.d.stride, C.d.padding, C.h, C.w, batch,
                                C.d.activation ? MIMIR_B200_ELT_RELU : C.fused_act))
      continue;
    const int xin = P.in_v[0];
    C.pre_norm = li;
    C.in_v[0] = xin;
    for (int& c : m->tensors[xin].consumers)
      if (c == li) c = pt.consumers[0];
    pt.consumers.clear();
    pt.want_f32 = false;
    pt.producer = -2;  // dead
    P.skip = true;
  }
  // ---- fusion 1d: a 2 x 2 nearest upsample read by shifted-GEMM convolutions: their layout pass gathers from the
  //      half-size source (and a folded GroupNorm takes its statistics there: the same values, each four times), so the
  //      upsampled tensor is read by nobody but residual adds - and is not produced at all when there are none ----
  static const bool fuse_up = [] { const char* e = getenv("MIMIR_B200_FUSE_UPSAMPLE"); return !(e && e[0] == '0'); }();
  for (int li = 0; li < nl && fuse_up; ++li) {
    LayerRT& U = m->layers[li];
    if (U.lt != LT::UpsampleNearest || U.skip || U.oh != 2 * U.h || U.ow != 2 * U.w) continue;
    const int uv = U.out_v, sv = root_of(m->tensors, U.in_v[0]);
    TensorV& ut = m->tensors[uv];
    if (ut.alias_of >= 0 || uv == out_root || !m->tensors[sv].want_f32 || m->tensors[sv].producer == -2) continue;
    bool aliased = false;
    for (const TensorV& t : m->tensors) aliased = aliased || t.alias_of == uv;
    if (aliased) continue;
    std::vector<int> keep;
    for (int ci : ut.consumers) {
      LayerRT& C = m->layers[ci];
      const bool conv_in = C.lt == LT::Conv2d && !C.skip && !C.in_up && C.in_v[0] == uv && C.res_v != uv && C.d.in_channels == U.ch &&
                           C.h == U.oh && C.w == U.ow && conv_uses_shifted(C.d.in_channels, C.d.kernel, C.d.stride, C.d.padding) &&
                           (C.pre_norm >= 0 || !conv_small_oc_supported(C.d.out_channels, C.d.kernel, C.d.stride, C.d.padding, C.h, C.w, batch,
                                                                        C.d.activation ? MIMIR_B200_ELT_RELU : C.fused_act));
      if (!conv_in) {
        keep.push_back(ci);
        continue;
      }
      C.in_up = true;
      C.in_v[0] = sv;
      m->tensors[sv].consumers.push_back(ci);
    }
    if (keep.size() == ut.consumers.size()) continue;  // nothing changed
    ut.consumers = keep;
    if (keep.empty()) {
      for (int& c : m->tensors[U.in_v[0]].consumers)
        if (c == li) c = -1;
      auto& sc = m->tensors[U.in_v[0]].consumers;
      sc.erase(std::remove(sc.begin(), sc.end(), -1), sc.end());
      ut.want_f32 = false;
      ut.producer = -2;  // dead
      U.skip = true;
    }
  }
  // ---- fusion 2: hi/lo planes straight from one GEMM epilogue into the next Linear -------------
  for (int li = 0; li < nl; ++li) {
    LayerRT& C = m->layers[li];
    if (C.lt != LT::Linear || C.skip) continue;
    if (linear_uses_skinny(C.rows_ps * batch, m->precision)) continue;
    const int v = C.in_v[0];
    TensorV& t = m->tensors[v];
    if (t.alias_of >= 0 || t.producer < 0 || v == out_root || total_consumers(v) != 1) continue;
    LayerRT& P = m->layers[t.producer];
    if (P.lt != LT::Linear || P.out_v != v || P.out_f != C.in_f || P.rows_ps != C.rows_ps || P.res_v >= 0) continue;
    if (linear_uses_skinny(P.rows_ps * batch, m->precision)) continue;
    P.emit_split = true;
    P.emit_f32 = false;
    C.read_split = true;
    t.want_f32 = false;
    t.want_split = true;
    t.split_rows_ps = P.rows_ps;
    t.split_k = P.out_f;
  }

  // ---- fusion 2b: a whole-sample RMSNorm whose only consumer is a tensor-core Linear / attention block writes
  //      that consumer's operand planes itself (the one-pass kernel holds the values in registers anyway) ----
  for (int li = 0; li < nl; ++li) {
    LayerRT& P = m->layers[li];
    if (P.lt != LT::RMSNorm || P.skip) continue;
    const int v = P.out_v;
    TensorV& t = m->tensors[v];
    if (t.alias_of >= 0 || v == out_root || total_consumers(v) != 1 || t.consumers.size() != 1) continue;
    if (!rmsnorm_onepass_ok(batch, t.n)) continue;
    LayerRT& C = m->layers[t.consumers[0]];
    if (C.skip || C.in_v[0] != v) continue;
    int k = 0;
    int64_t rows_ps = 0;
    if (C.lt == LT::Linear && !linear_uses_skinny(C.rows_ps * batch, m->precision)) {
      k = C.in_f; rows_ps = C.rows_ps;
    } else if (C.lt == LT::Attention) {
      k = C.embed; rows_ps = C.seq;
    } else {
      continue;
    }
    if (k <= 0 || k % 64 != 0 || rows_ps * k != t.n) continue;
    P.emit_split = true;
    P.emit_f32 = false;
    C.read_split = true;
    t.want_f32 = false;
    t.want_split = true;
    t.split_rows_ps = rows_ps;
    t.split_k = k;
  }

  // ---- liveness ------------------------------------------------------------------------------------
  const int nt = static_cast<int>(m->tensors.size());
  for (int v = 0; v < nt; ++v) {
    TensorV& t = m->tensors[v];
    t.first = (t.producer >= 0) ? t.producer : -1;
    t.last = t.first;
  }
  for (int v = 0; v < nt; ++v) {
    const int r = root_of(m->tensors, v);
    TensorV& rt = m->tensors[r];
    for (int c : m->tensors[v].consumers)
      if (!m->layers[c].skip) rt.last = std::max(rt.last, c);
    if (m->tensors[v].alias_of >= 0) rt.last = std::max(rt.last, m->tensors[v].producer);
  }
  m->tensors[out_root].last = nl;

  // ---- offsets ---------------------------------------------------------------------------------------
  // ---- fusion 1e: GroupNorm statistics out of the producing convolution's GEMM epilogue (MIMIR_B200_GN_EPILOGUE=1) ----
  //      A GroupNorm (folded into a convolution's layout pass or running on its own) whose input is the output of a shifted-GEMM
  //      convolution does not sweep that tensor for its mean and variance: the convolution's epilogue leaves per-block partials
  //      behind, a small kernel merges them, and the GroupNorm (or the layout pass) reads (mean, 1 / std) from there.
  for (auto& L : m->layers) { L.gn_emit_for = -1; L.gn_stats_from = -1; }
  for (int li = 0; li < nl; ++li) {
    LayerRT& G = m->layers[li];
    if (G.lt != LT::GroupNorm) continue;
    int xin = -1;
    if (G.skip) {  // folded: the statistics are taken over the consuming convolution's (possibly pre-upsample) input
      for (int ci = 0; ci < nl; ++ci)
        if (m->layers[ci].lt == LT::Conv2d && !m->layers[ci].skip && m->layers[ci].pre_norm == li) xin = m->layers[ci].in_v[0];
    } else {
      xin = G.in_v[0];
    }
    if (xin < 0) continue;
    const int xr = root_of(m->tensors, xin);
    const TensorV& xt = m->tensors[xr];
    if (xt.producer < 0) continue;
    LayerRT& P = m->layers[xt.producer];
    if (P.lt != LT::Conv2d || P.skip || P.gn_emit_for >= 0 || root_of(m->tensors, P.out_v) != xr || P.d.out_channels != G.ch) continue;
    if (!conv_can_emit_gn(batch, P.d.in_channels, P.d.out_channels, P.h, P.w, P.d.kernel, P.d.stride, P.d.padding, G.d.num_groups,
                          P.d.activation ? MIMIR_B200_ELT_RELU : P.fused_act))
      continue;
    P.gn_emit_for = li;
    G.gn_stats_from = xt.producer;
  }
  ArenaSim sim;
  auto place = [&](int v) {
    TensorV& t = m->tensors[v];
    if (t.alias_of >= 0 || t.producer == -2) return;
    if (t.want_f32) t.off_f32 = sim.alloc(f32_bytes(t, batch));
    if (t.want_split) t.off_split = sim.alloc(splitv_bytes(t, batch));
  };
  auto drop = [&](int v) {
    TensorV& t = m->tensors[v];
    if (t.alias_of >= 0 || t.producer == -2) return;
    if (t.want_f32) sim.release(t.off_f32, f32_bytes(t, batch));
    if (t.want_split) sim.release(t.off_split, splitv_bytes(t, batch));
  };
  for (int v = 0; v < nt; ++v)
    if (m->tensors[v].first == -1 && m->tensors[v].producer == -1) place(v);
  for (int v = 0; v < nt; ++v)
    if (m->tensors[v].producer == -1 && m->tensors[v].last == -1 && root_of(m->tensors, v) != out_root) drop(v);
  uint64_t flops = 0, hbm = 0;
  for (int li = 0; li < nl; ++li) {
    LayerRT& L = m->layers[li];
    if (!L.skip && L.lt != LT::Alias) {
      place(L.out_v);
      for (int pv : L.piece_v) place(pv);
      const int64_t rows = static_cast<int64_t>(batch) * L.rows_ps;
      switch (L.lt) {
        case LT::Linear:
          L.ws_bytes = linear_ws_bytes(static_cast<int>(rows), L.in_f, L.out_f, m->precision, L.read_split);
          flops += 2ull * rows * L.in_f * L.out_f;
          break;
        case LT::Attention: {
          const int64_t r = static_cast<int64_t>(batch) * L.seq;
          L.ws_bytes = attention_ws_bytes(batch, L.seq, L.embed, L.heads, m->precision);
          const uint64_t core = 4ull * batch * L.seq * L.seq * L.embed;
          flops += 2ull * r * L.embed * 4 * L.embed + (L.d.causal ? core / 2 : core);
          break;
        }
        case LT::CrossAttention: {
          L.ws_bytes = cross_attention_ws_bytes(batch, L.seq, L.kv_len, L.embed, m->precision);
          const uint64_t E = static_cast<uint64_t>(L.embed);
          flops += 2ull * batch * L.seq * E * E * 2 + 2ull * batch * L.kv_len * E * 2 * E + 4ull * batch * L.seq * L.kv_len * E;
          break;
        }
        case LT::Conv2d: {
          const int k = L.d.in_channels * L.d.kernel * L.d.kernel;
          L.ws_bytes = conv_ws_bytes(batch, L.d.in_channels, L.h, L.w, L.d.kernel, L.d.stride, L.d.padding, m->precision);
          if (L.pre_norm >= 0) L.ws_bytes += conv_prenorm_bytes(batch, m->layers[L.pre_norm].d.num_groups);
          if (L.gn_emit_for >= 0)
            L.ws_bytes += conv_gn_emit_bytes(batch, L.d.out_channels, L.h, L.w, L.d.padding, m->layers[L.gn_emit_for].d.num_groups);
          flops += 2ull * batch * L.oh * L.ow * k * L.d.out_channels;
          break;
        }
        default:
          L.ws_bytes = 0;
          for (int v : L.in_v) hbm += f32_bytes(m->tensors[v], batch);
          hbm += f32_bytes(m->tensors[L.out_v], batch);
          break;
      }
      if (L.ws_bytes) {
        L.ws_off = sim.alloc(L.ws_bytes);
        sim.release(L.ws_off, L.ws_bytes);
      }
    }
    for (int v = 0; v < nt; ++v) {
      const TensorV& t = m->tensors[v];
      // In a pipelined plan the slots of the graph inputs are never handed on: the copy-in of micro-batch c + 2 may then
      // run while micro-batch c is still being copied out of the same arena buffer (nothing else lives in an input slot).
      if (m->pipeline > 1 && t.producer == -1) continue;
      if (t.alias_of < 0 && t.producer != -2 && t.last == li) drop(v);
    }
  }
  // Does the output share bytes with a graph input's slot (possible only in un-pipelined plans, or when the graph returns
  // one of its inputs)?  The pipelined forward then orders copy-in after the copy-out two micro-batches back.
  m->out_in_input_slot = false;
  {
    const TensorV& ot = m->tensors[out_root];
    const size_t o0 = ot.off_f32, o1 = o0 + static_cast<size_t>(ot.n) * batch * 4;
    for (int v = 0; v < nt; ++v) {
      const TensorV& t = m->tensors[v];
      if (t.producer != -1 || t.alias_of >= 0) continue;
      const size_t i0 = t.off_f32, i1 = i0 + static_cast<size_t>(t.n) * (t.broadcast_input ? 1 : batch) * 4;
      if (v == out_root || (i0 < o1 && o0 < i1)) m->out_in_input_slot = true;
    }
  }
  m->flops = flops;
  m->hbm_bytes = hbm;

  // ---- budget check before anything is launched, then (re)allocate the arena -------------------------
  size_t need = sim.peak + 256;
  for (auto& L : m->layers) {  // the emitted GroupNorm statistics live behind the simulated arena for the whole forward
    if (L.gn_emit_for < 0) continue;
    need = (need + 255) & ~static_cast<size_t>(255);
    L.gn_stats_off = need;
    need += static_cast<size_t>(batch) * m->layers[L.gn_emit_for].d.num_groups * 2 * sizeof(float);
  }
  need += 256;
  if (m->arena && m->arena_bytes < need) {
    dev_free(m->arena, m->arena_bytes);
    if (m->arena2) dev_free(m->arena2, m->arena_bytes);
    m->arena = m->arena2 = nullptr;
    m->arena_bytes = 0;
  }
  if (!m->arena) {
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&m->arena), need, "activation arena"));
    m->arena_bytes = need;
  }
  if (m->pipeline > 1 && !m->arena2) {
    int s2 = dev_alloc(reinterpret_cast<void**>(&m->arena2), m->arena_bytes, "activation arena (second pipeline buffer)");
    if (s2 != MIMIR_B200_OK) return s2;
  }
  if (m->pipeline == 1 && m->arena2) {
    dev_free(m->arena2, m->arena_bytes);
    m->arena2 = nullptr;
  }
  m->planned_batch = full_batch;
  m->planned_micro = batch;
  for (auto& L : m->layers) MB_TRY(prepare_weight_planes(m, L, nullptr));
  MB_CUDA(cudaStreamSynchronize(nullptr));
  ctx().stats.arena_peak_bytes = need * (m->pipeline > 1 ? 2 : 1);
  return MIMIR_B200_OK;
}

struct Bound {
  std::vector<const float*> in_ptr;  // per tensor version: user device pointer overriding the arena
  float* out_ptr = nullptr;
};

int run_layers(MimirB200Model* m, int batch, const Bound& bnd, cudaStream_t st, uint8_t* arena) {
  auto f32p = [&](int v) -> float* {
    const int r = root_of(m->tensors, v);
    if (r < static_cast<int>(bnd.in_ptr.size()) && bnd.in_ptr[r]) return const_cast<float*>(bnd.in_ptr[r]);
    if (r == root_of(m->tensors, m->out_v) && bnd.out_ptr) return bnd.out_ptr;
    return reinterpret_cast<float*>(arena + m->tensors[r].off_f32);
  };
  auto splitp = [&](int v) -> __nv_bfloat16* { return reinterpret_cast<__nv_bfloat16*>(arena + m->tensors[v].off_split); };
  const int nl = static_cast<int>(m->layers.size());
  for (int li = 0; li < nl; ++li) {
    LayerRT& L = m->layers[li];
    if (L.skip || L.lt == LT::Alias) continue;
    const MimirLayerDesc& d = L.d;
    void* ws = L.ws_bytes ? static_cast<void*>(arena + L.ws_off) : nullptr;
    int s = MIMIR_B200_OK;
    switch (L.lt) {
      case LT::Linear: {
        LinearExec e;
        e.rows = batch * L.rows_ps; e.in_f = L.in_f; e.out_f = L.out_f; e.precision = m->precision;
        if (L.read_split) e.x_split = splitp(L.in_v[0]); else e.x_f32 = f32p(L.in_v[0]);
        e.w_f32 = L.w_f32;
        e.w_split = L.w_split;
        e.w_scale = L.w_scale;
        e.bias = d.use_bias ? L.w_f32 + static_cast<size_t>(L.in_f) * L.out_f : nullptr;
        e.activation = L.fused_act;
        if (L.res_v >= 0) e.residual = f32p(L.res_v);
        if (L.emit_f32) e.y_f32 = f32p(L.out_v);
        if (L.emit_split) e.y_split = splitp(L.out_v);
        e.ws = ws; e.ws_bytes = L.ws_bytes;
        s = linear_exec(e, st);
        break;
      }
      case LT::Attention: {
        AttentionExec e;
        e.batch = batch; e.seq = L.seq; e.embed = L.embed; e.heads = L.heads; e.causal = d.causal;
        e.precision = m->precision;
        if (L.read_split) e.x_split = splitp(L.in_v[0]); else e.x = f32p(L.in_v[0]);
        e.wqkv_split = L.w_split; e.wout_split = L.w_split2; e.w_scale = L.w_scale; e.y = f32p(L.out_v); e.ws = ws;
        if (L.res_v >= 0) e.residual = f32p(L.res_v);
        if (m->is_twin) {
          e.kcache = L.kcache; e.vcache = L.vcache; e.max_seq = m->max_seq; e.decode_pos = m->decode_pos;
          e.decode_scratch = m->decode_scratch;
          e.pos_dev = m->pos_dev;
          if (L.w_t_f32) {
            e.wqkv_t_f32 = L.w_t_f32;
            e.wout_t_f32 = L.w_t_f32 + static_cast<size_t>(3) * L.embed * L.embed;
            e.skinny_scratch = m->skinny_scratch;
            e.skinny_scratch_bytes = m->skinny_scratch_bytes;
          }
        } else if (m->decode && m->decode->twin_epoch == m->plan_epoch && batch == m->decode->planned_batch && L.seq <= m->decode->max_seq) {
          // a full forward of the main model doubles as the prefill: its keys and values land in the caches
          const LayerRT& T = m->decode->layers[static_cast<size_t>(li)];
          e.kcache = T.kcache; e.vcache = T.vcache; e.max_seq = m->decode->max_seq;
        }
        s = attention_exec(e, st);
        break;
      }
      case LT::Conv2d: {
        ConvExec e;
        e.batch = batch; e.ic = d.in_channels; e.oc = d.out_channels; e.h = L.h; e.w = L.w; e.ks = d.kernel;
        e.stride = d.stride; e.pad = d.padding; e.precision = m->precision;
        e.activation = d.activation ? MIMIR_B200_ELT_RELU : L.fused_act;
        e.x = f32p(L.in_v[0]); e.w_split = L.w_split; e.w_f32 = L.w_f32; e.w_scale = L.w_scale; e.y = f32p(L.out_v); e.ws = ws;
        if (L.res_v >= 0) e.residual = f32p(L.res_v);
        if (L.pre_norm >= 0) {
          const LayerRT& G = m->layers[L.pre_norm];
          e.pre_groups = G.d.num_groups;
          e.pre_gamma = G.d.affine ? G.w_f32 : nullptr;
          e.pre_beta = (G.d.affine && G.d.use_bias) ? G.w_f32 + G.ch : nullptr;
          e.pre_eps = G.d.eps;
          e.pre_act = G.fused_act;
          if (G.gn_stats_from >= 0) e.pre_stats = reinterpret_cast<const float*>(arena + m->layers[G.gn_stats_from].gn_stats_off);
        }
        e.in_up = L.in_up ? 1 : 0;
        if (L.gn_emit_for >= 0) {
          e.gn_stats_out = reinterpret_cast<float*>(arena + L.gn_stats_off);
          e.gn_groups = m->layers[L.gn_emit_for].d.num_groups;
          e.gn_eps = m->layers[L.gn_emit_for].d.eps;
        }
        s = conv_exec(e, st);
        break;
      }
      case LT::LayerNorm: {
        const float* g = d.affine ? L.w_f32 : nullptr;
        const float* b = (d.affine && d.use_bias) ? L.w_f32 + L.norm_n : nullptr;
        const int64_t rows = static_cast<int64_t>(batch) * (m->tensors[L.in_v[0]].n / L.norm_n);
        s = launch_layernorm(f32p(L.in_v[0]), g, b, f32p(L.out_v), rows, L.norm_n, d.eps, st);
        break;
      }
      case LT::RMSNorm: {
        const bool aff = d.affine && L.w_f32 && L.w_count > 0;
        const int64_t n = m->tensors[L.in_v[0]].n;
        int ap, wp;
        precision_planes(m->precision, &ap, &wp);
        s = launch_rmsnorm(f32p(L.in_v[0]), aff ? L.w_f32 : nullptr, aff ? static_cast<int64_t>(L.w_count) : 0,
                           L.emit_f32 ? f32p(L.out_v) : nullptr, batch, n, d.eps, st, L.emit_split ? splitp(L.out_v) : nullptr, ap,
                           static_cast<int64_t>(batch) * n);
        break;
      }
      case LT::GroupNorm: {
        const float* g = d.affine ? L.w_f32 : nullptr;
        const float* b = (d.affine && d.use_bias) ? L.w_f32 + L.ch : nullptr;
        const float* stats = L.gn_stats_from >= 0 ? reinterpret_cast<const float*>(arena + m->layers[L.gn_stats_from].gn_stats_off) : nullptr;
        s = launch_groupnorm_apply(f32p(L.in_v[0]), stats, g, b, f32p(L.out_v), batch, L.ch, L.h * L.w, d.num_groups, d.eps, L.fused_act,
                                   L.res_v >= 0 ? f32p(L.res_v) : nullptr, st);
        break;
      }
      case LT::Softmax:
      case LT::LogSoftmax:
        s = launch_softmax(f32p(L.in_v[0]), f32p(L.out_v), batch, m->tensors[L.in_v[0]].n, L.lt == LT::LogSoftmax, st);
        break;
      case LT::Act:
        s = launch_eltwise(L.act_of_type, f32p(L.in_v[0]), nullptr, f32p(L.out_v), batch, m->tensors[L.in_v[0]].n, 0, st,
                           d.leaky_relu_alpha > 0.0f ? d.leaky_relu_alpha : 0.01f);
        break;
      case LT::Add:
      case LT::Multiply: {
        int a = L.in_v[0], b = L.in_v[1];
        if (m->tensors[b].n > m->tensors[a].n) std::swap(a, b);  // `big` first (LayerOps.hpp:171-176)
        s = launch_eltwise(L.lt == LT::Add ? MIMIR_B200_ELT_ADD : MIMIR_B200_ELT_MULTIPLY, f32p(a), f32p(b), f32p(L.out_v), batch,
                           m->tensors[a].n, m->tensors[b].n, st);
        break;
      }
      case LT::Embedding:
        s = launch_embedding(f32p(L.in_v[0]), nullptr, L.w_f32, f32p(L.out_v), static_cast<int64_t>(batch) * m->tensors[L.in_v[0]].n,
                             std::max(1, d.vocab_size), std::max(1, d.embed_dim), d.padding_idx, st);
        break;
      case LT::UpsampleNearest:
        s = launch_upsample_nearest(f32p(L.in_v[0]), f32p(L.out_v), batch, L.ch, L.h, L.w, L.oh / L.h, L.ow / L.w, st);
        break;
      case LT::Permute:
        s = launch_permute(f32p(L.in_v[0]), f32p(L.out_v), batch, d.n_dims, d.shape, d.permute_dims, st);
        break;
      case LT::Concat: {
        int64_t off = 0;
        const int64_t total = m->tensors[L.out_v].n;
        for (int v : L.in_v) {
          s = launch_copy_strided(f32p(v), f32p(L.out_v), batch, m->tensors[v].n, total, off, st);
          if (s != MIMIR_B200_OK) break;
          off += m->tensors[v].n;
        }
        break;
      }
      case LT::CrossAttention: {
        CrossAttentionExec e;
        e.batch = batch; e.q_len = L.seq; e.kv_len = L.kv_len; e.embed = L.embed; e.heads = L.heads; e.causal = d.causal;
        e.precision = m->precision;
        e.q_in = f32p(L.in_v[0]); e.kv_in = f32p(L.in_v[1]);
        e.wq_split = L.w_split; e.wkv_split = L.w_split2; e.wout_split = L.w_split3; e.w_scale = L.w_scale;
        e.y = f32p(L.out_v); e.ws = ws;
        if (L.res_v >= 0) e.residual = f32p(L.res_v);
        s = cross_attention_exec(e, st);
        break;
      }
      case LT::Binary2:
        s = launch_eltwise(L.act_of_type, f32p(L.in_v[0]), f32p(L.in_v[1]), f32p(L.out_v), batch, m->tensors[L.in_v[0]].n,
                           m->tensors[L.in_v[1]].n, st);
        break;
      case LT::Split: {
        const int64_t total = m->tensors[L.in_v[0]].n;
        int64_t off = 0;
        for (size_t pi = 0; pi < L.piece_v.size(); ++pi) {
          s = launch_copy_strided(f32p(L.in_v[0]) + off, f32p(L.piece_v[pi]), batch, L.piece_n[pi], L.piece_n[pi], 0, st, total);
          if (s != MIMIR_B200_OK) break;
          off += L.piece_n[pi];
        }
        break;
      }
      case LT::DepthwiseConv2d:
        s = launch_depthwise_conv2d(f32p(L.in_v[0]), L.w_f32, d.use_bias ? L.w_f32 + static_cast<size_t>(L.ch) * L.kk * L.kk : nullptr,
                                    f32p(L.out_v), batch, L.ch, L.h, L.w, L.kk, L.st, L.pd, static_cast<int64_t>(L.w_count), st);
        break;
      case LT::Conv1d:
        s = launch_conv1d(f32p(L.in_v[0]), L.w_f32, d.use_bias ? L.w_f32 + static_cast<size_t>(L.out_f) * L.ch * L.kk : nullptr,
                          f32p(L.out_v), batch, L.ch, L.out_f, L.w, L.kk, L.st, L.pd, static_cast<int64_t>(L.w_count), st);
        break;
      case LT::ConvTranspose2d:
        s = launch_conv_gather(f32p(L.in_v[0]), L.w_f32, f32p(L.out_v), batch, d.in_channels, d.out_channels, L.h, L.w, L.oh, L.ow,
                               d.kernel, d.stride, d.padding, d.activation != 0, st);
        break;
      case LT::Pool2d:
        s = launch_pool2d((L.act_of_type == 1 || L.act_of_type == 3) ? 1 : 0, f32p(L.in_v[0]), f32p(L.out_v), batch, L.ch, L.h, L.w, L.kk, L.kw, L.st, L.sw, L.pd, L.pw, st);
        break;
      case LT::Pad2d:
        s = launch_pad2d(L.act_of_type, f32p(L.in_v[0]), f32p(L.out_v), batch, L.ch, L.h, L.w, L.pd, L.pw, st);
        break;
      case LT::PixelShuffle:
        s = launch_pixel_shuffle(f32p(L.in_v[0]), f32p(L.out_v), batch, L.ch, L.h, L.w, L.kk, st);
        break;
      case LT::UpsampleBilinear:
        s = launch_upsample_bilinear(f32p(L.in_v[0]), f32p(L.out_v), batch, L.ch, L.h, L.w, L.oh, L.ow, L.act_of_type, st);
        break;
      case LT::MatMul:
      case LT::BatchMatMul:
        s = launch_batch_matmul(f32p(L.in_v[0]), f32p(L.in_v[1]), f32p(L.out_v), static_cast<int64_t>(batch) * L.mm_b, L.mm_m, L.mm_k,
                                L.mm_n, st);
        break;
      case LT::BatchNorm: {
        // statistics over the whole sample, then y[i] *= w[i] for i < weight count; no shift (Model.cpp:5396-5416)
        const int64_t n = m->tensors[L.in_v[0]].n;
        s = launch_layernorm(f32p(L.in_v[0]), nullptr, nullptr, f32p(L.out_v), batch, n, d.eps, st);
        if (s == MIMIR_B200_OK && d.affine && L.w_f32 && L.w_count > 0)
          s = launch_scale_prefix(f32p(L.out_v), L.w_f32, batch, n, static_cast<int64_t>(L.w_count), st);
        break;
      }
      case LT::InstanceNorm: {
        const bool aff = d.affine && L.w_f32 && L.w_count >= static_cast<size_t>(2) * L.ch;
        s = launch_groupnorm(f32p(L.in_v[0]), aff ? L.w_f32 : nullptr, aff ? L.w_f32 + L.ch : nullptr, f32p(L.out_v), batch, L.ch,
                             L.h * L.w, L.ch, d.eps, -1, nullptr, st);
        break;
      }
      case LT::EmbeddingBag: {
        const bool has_off = L.in_v.size() >= 2 && m->tensors[L.in_v[1]].n > 0;
        s = launch_embedding_bag(f32p(L.in_v[0]), m->tensors[L.in_v[0]].n, has_off ? f32p(L.in_v[1]) : nullptr,
                                 has_off ? m->tensors[L.in_v[1]].n : 0, L.w_f32, f32p(L.out_v), batch, std::max(1, d.vocab_size),
                                 std::max(1, d.embed_dim), d.padding_idx, st);
        break;
      }
      case LT::PatchEmbed:
        s = launch_patch_embed(f32p(L.in_v[0]), L.w_f32, f32p(L.out_v), batch, L.mm_n, L.mm_b, L.mm_m, L.mm_k, st);
        break;
      case LT::Bilinear: {
        const size_t nw = static_cast<size_t>(L.mm_n) * L.mm_m * L.mm_k;
        s = launch_bilinear(f32p(L.in_v[0]), f32p(L.in_v[1]), L.w_f32, d.use_bias ? L.w_f32 + nw : nullptr, f32p(L.out_v),
                            static_cast<int64_t>(batch) * L.mm_b, L.mm_m, L.mm_k, L.mm_n, st);
        break;
      }
      case LT::Recurrent:
        s = launch_recurrent(L.act_of_type, f32p(L.in_v[0]), L.w_f32, f32p(L.out_v), batch, L.mm_m, L.mm_k, L.mm_n, d.use_bias != 0, st);
        break;
      case LT::Transpose: {
        const int shape[2] = {d.in_features, d.out_features}, dims[2] = {1, 0};
        s = launch_permute(f32p(L.in_v[0]), f32p(L.out_v), batch, 2, shape, dims, st);
        break;
      }
      case LT::TokenMeanPool:
        s = launch_token_mean_pool(f32p(L.in_v[0]), f32p(L.out_v), batch, d.seq_len, d.embed_dim, st);
        break;
      case LT::GlobalAvgPool:
        s = launch_global_avgpool(f32p(L.in_v[0]), f32p(L.out_v), batch, L.ch, L.h * L.w, st);
        break;
      default:
        return fail(MIMIR_B200_E_UNSUPPORTED, "layer type '%s' is not supported by the B200 backend", L.type.c_str());
    }
    if (s != MIMIR_B200_OK) return s;
  }
  return MIMIR_B200_OK;
}

bool graphs_enabled() {
  static const bool on = [] {
    const char* e = getenv("MIMIR_B200_GRAPH");
    return !(e && e[0] == '0');
  }();
  return on;
}

// run_layers through the graph cache.  The first call with a given set of pointers runs layer by layer (it also
// performs every one-time host-side setup the launch helpers do); the second is captured on a private stream;
// from then on the instantiated graph is launched into the caller's stream.
int run_layers_cached(MimirB200Model* m, int batch, const Bound& bnd, cudaStream_t st, uint8_t* arena) {
  // (a twin whose position is a launch argument changes from call to call)
  if (!graphs_enabled() || ctx().prof_gemm || (m->is_twin && !m->pos_dev)) return run_layers(m, batch, bnd, st, arena);
  std::vector<const void*> key;
  key.reserve(bnd.in_ptr.size() + 3);
  key.push_back(reinterpret_cast<const void*>(static_cast<uintptr_t>(batch)));
  key.push_back(arena);
  key.push_back(bnd.out_ptr);
  for (const float* p : bnd.in_ptr) key.push_back(p);
  MimirB200Model::CachedGraph* g = nullptr;
  for (auto& c : m->graphs)
    if (c.key == key) { g = &c; break; }
  if (!g) {
    if (m->graphs.size() >= 64) drop_graphs(m);  // callers that move their buffers every call never hit the cache
    m->graphs.emplace_back();
    g = &m->graphs.back();
    g->key = key;
  }
  if (g->exec) {
    MB_CUDA(cudaGraphLaunch(g->exec, st));
    count_launch(static_cast<int>(g->launches));
    return MIMIR_B200_OK;
  }
  if (g->unusable || g->seen++ == 0) return run_layers(m, batch, bnd, st, arena);
  if (!m->s_capture) {
    MB_CUDA(cudaStreamCreateWithFlags(&m->s_capture, cudaStreamNonBlocking));
    MB_TRY(norm_scratch_reserve(m->s_capture));
  }
  const uint64_t before = ctx().launches.load();
  if (cudaStreamBeginCapture(m->s_capture, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError();
    g->unusable = true;
    return run_layers(m, batch, bnd, st, arena);
  }
  const int s = run_layers(m, batch, bnd, m->s_capture, arena);
  cudaGraph_t graph = nullptr;
  const cudaError_t ce = cudaStreamEndCapture(m->s_capture, &graph);
  const uint64_t inside = ctx().launches.load() - before;
  ctx().launches.fetch_sub(inside);  // nothing ran yet
  if (s != MIMIR_B200_OK || ce != cudaSuccess || !graph) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    g->unusable = true;
    if (s != MIMIR_B200_OK) return s;
    return run_layers(m, batch, bnd, st, arena);
  }
  cudaGraphExec_t exec = nullptr;
  const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (ie != cudaSuccess || !exec) {
    cudaGetLastError();
    g->unusable = true;
    return run_layers(m, batch, bnd, st, arena);
  }
  g->exec = exec;
  g->launches = inside;
  MB_CUDA(cudaGraphLaunch(g->exec, st));
  count_launch(static_cast<int>(g->launches));
  return MIMIR_B200_OK;
}

int check_inputs(MimirB200Model* m, const MimirNamedInput* inputs, int n_inputs, int batch, std::vector<int>* vs) {
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (m->planned_batch != batch) return fail(MIMIR_B200_E_INVALID, "forward: model is planned for batch %d, not %d", m->planned_batch, batch);
  if (static_cast<size_t>(n_inputs) != m->input_v.size()) return fail(MIMIR_B200_E_INVALID, "forward: expected %zu inputs, got %d", m->input_v.size(), n_inputs);
  for (int i = 0; i < n_inputs; ++i) {
    std::string name = (inputs[i].name && inputs[i].name[0]) ? inputs[i].name : "x";
    if (name == "__input__") name = "x";
    auto it = m->input_v.find(name);
    if (it == m->input_v.end()) return fail(MIMIR_B200_E_INVALID, "forward: input '%s' was not declared to plan", name.c_str());
    const TensorV& t = m->tensors[it->second];
    if (static_cast<uint64_t>(t.n) != inputs[i].per_sample || t.broadcast_input != (inputs[i].broadcast != 0))
      return fail(MIMIR_B200_E_INVALID, "forward: input '%s' does not match the planned size", name.c_str());
    if (!inputs[i].data) return fail(MIMIR_B200_E_INVALID, "forward: input '%s' has no data", name.c_str());
    vs->push_back(it->second);
  }
  return MIMIR_B200_OK;
}

}  // namespace
}  // namespace mb

namespace mb {
int model_device(MimirB200ModelHandle m) { return m ? m->device : ctx().device; }
}  // namespace mb

extern "C" {

using namespace mb;

int mimir_b200_model_create(const MimirLayerDesc* layers, int n_layers, MimirB200ModelHandle* out) {
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called");
  if (!layers || n_layers <= 0 || !out) return fail(MIMIR_B200_E_INVALID, "model_create: no layers defined");
  auto m = std::make_unique<MimirB200Model>();
  m->device = ctx().device;
  m->layers.resize(static_cast<size_t>(n_layers));
  for (int i = 0; i < n_layers; ++i) {
    const MimirLayerDesc& d = layers[i];
    LayerRT& L = m->layers[static_cast<size_t>(i)];
    L.name = d.name ? d.name : ("layer" + std::to_string(i));
    L.type = d.type ? d.type : "";
    L.output = (d.output && d.output[0]) ? d.output : "x";
    if (d.n_inputs < 0 || d.n_inputs > MIMIR_B200_MAX_INPUTS) return fail(MIMIR_B200_E_INVALID, "layer %d: bad n_inputs", i);
    for (int j = 0; j < d.n_inputs; ++j) L.inputs.emplace_back(d.inputs[j] ? d.inputs[j] : "x");
    L.d = d;
    L.d.name = L.d.type = L.d.output = nullptr;
    for (auto& p : L.d.inputs) p = nullptr;
    if (L.d.n_dims < 0 || L.d.n_dims > MIMIR_B200_MAX_DIMS) return fail(MIMIR_B200_E_INVALID, "layer %d: bad n_dims", i);
    const TypeInfo ti = classify(L.type);
    L.lt = ti.lt;
    L.act_of_type = ti.act;
    if (L.lt == LT::Unsupported)
      return fail(MIMIR_B200_E_UNSUPPORTED, "layer %d (%s): type '%s' is not supported by the B200 backend (no CPU fallback)", i,
                  L.name.c_str(), L.type.c_str());
  }
  MimirB200Model* raw = m.release();
  {
    std::lock_guard<std::mutex> lk(g_models_mu);
    g_models.insert(raw);
  }
  *out = raw;
  return MIMIR_B200_OK;
}

static void destroy_model(MimirB200Model* m) {
  if (m->decode) {
    destroy_model(m->decode);
    m->decode = nullptr;
  }
  for (auto& L : m->layers) {
    if (L.kcache) dev_free(L.kcache, L.cache_bytes);
    if (L.vcache) dev_free(L.vcache, L.cache_bytes);
    if (L.w_t_f32) dev_free(L.w_t_f32, L.w_t_bytes);
    L.kcache = L.vcache = L.w_t_f32 = nullptr;
  }
  if (m->decode_scratch) dev_free(m->decode_scratch, m->decode_scratch_bytes);
  if (m->skinny_scratch) dev_free(m->skinny_scratch, m->skinny_scratch_bytes);
  if (m->pos_dev) dev_free(m->pos_dev, 256);
  m->pos_dev = nullptr;
  m->decode_scratch = m->skinny_scratch = nullptr;
  drop_graphs(m);
  if (m->s_capture) {
    norm_scratch_release(m->s_capture);
    cudaStreamDestroy(m->s_capture);
  }
  for (auto& L : m->layers) free_layer_weights(L, m);
  if (m->arena) dev_free(m->arena, m->arena_bytes);
  if (m->arena2) dev_free(m->arena2, m->arena_bytes);
  for (auto e : m->ev_h2d) cudaEventDestroy(e);
  for (auto e : m->ev_comp) cudaEventDestroy(e);
  for (auto e : m->ev_d2h) cudaEventDestroy(e);
  if (m->s_h2d) cudaStreamDestroy(m->s_h2d);
  if (m->s_comp) cudaStreamDestroy(m->s_comp);
  if (m->s_d2h) cudaStreamDestroy(m->s_d2h);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  delete m;
}

int mimir_b200_model_destroy(MimirB200ModelHandle m) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return MIMIR_B200_OK;
  {
    std::lock_guard<std::mutex> lk(g_models_mu);
    if (!g_models.erase(m)) return fail(MIMIR_B200_E_INVALID, "model_destroy: unknown handle");
  }
  cudaDeviceSynchronize();
  destroy_model(m);
  return MIMIR_B200_OK;
}

int mimir_b200_model_set_precision(MimirB200ModelHandle m, int precision) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (precision < MIMIR_B200_PREC_BF16X2 || precision > MIMIR_B200_PREC_BF16) return fail(MIMIR_B200_E_INVALID, "unknown precision %d", precision);
  if (precision != m->precision) {
    // operand planes depend on the precision: drop them, plan() rebuilds
    for (auto& L : m->layers) {
      if (L.w_split) { dev_free(L.w_split, L.w_split_bytes); m->weight_bytes -= L.w_split_bytes; L.w_split = nullptr; }
      if (L.w_split2) { dev_free(L.w_split2, L.w_split2_bytes); m->weight_bytes -= L.w_split2_bytes; L.w_split2 = nullptr; }
      if (L.w_split3) { dev_free(L.w_split3, L.w_split3_bytes); m->weight_bytes -= L.w_split3_bytes; L.w_split3 = nullptr; }
      L.w_split_k = -1;
    }
    m->planned_batch = 0;
  }
  m->precision = precision;
  return MIMIR_B200_OK;
}

int mimir_b200_model_weights_device(MimirB200ModelHandle m, int layer_index, uint64_t n, float** dev) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (layer_index < 0 || layer_index >= static_cast<int>(m->layers.size())) return fail(MIMIR_B200_E_INVALID, "upload_weights: layer index out of range");
  LayerRT& L = m->layers[static_cast<size_t>(layer_index)];
  if (n != L.d.params_count) return fail(MIMIR_B200_E_INVALID, "upload_weights: %llu values given, layer '%s' has params_count %llu",
                                          static_cast<unsigned long long>(n), L.name.c_str(), static_cast<unsigned long long>(L.d.params_count));
  cudaDeviceSynchronize();
  free_layer_weights(L, m);
  L.w_count = 0;
  if (dev) *dev = nullptr;
  if (n == 0) return MIMIR_B200_OK;
  MB_TRY(dev_alloc(reinterpret_cast<void**>(&L.w_f32), n * 4, "layer weights"));
  L.w_count = n;
  m->weight_bytes += n * 4;
  m->planned_batch = 0;  // planes are rebuilt by the next plan
  if (dev) *dev = L.w_f32;
  return MIMIR_B200_OK;
}

int mimir_b200_model_upload_weights(MimirB200ModelHandle m, int layer_index, const float* host, uint64_t n) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (n != 0 && !host) return fail(MIMIR_B200_E_INVALID, "upload_weights: null host pointer");
  float* dev = nullptr;
  MB_TRY(mimir_b200_model_weights_device(m, layer_index, n, &dev));
  if (n) MB_CUDA(cudaMemcpy(dev, host, n * 4, cudaMemcpyHostToDevice));
  return MIMIR_B200_OK;
}

int mimir_b200_model_layer_info(MimirB200ModelHandle m, int layer_index, const char** name, uint64_t* params_count) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (layer_index < 0 || layer_index >= static_cast<int>(m->layers.size())) return fail(MIMIR_B200_E_INVALID, "layer index out of range");
  const LayerRT& L = m->layers[static_cast<size_t>(layer_index)];
  if (name) *name = L.name.c_str();
  if (params_count) *params_count = L.d.params_count;
  return MIMIR_B200_OK;
}

int mimir_b200_model_tensor_slot(MimirB200ModelHandle m, const char* input_name, uint64_t* offset, uint64_t* bytes) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m || !offset || !bytes) return fail(MIMIR_B200_E_INVALID, "tensor_slot: null argument");
  if (m->planned_batch <= 0) return fail(MIMIR_B200_E_INVALID, "tensor_slot: plan the model first");
  int v = m->out_v;
  if (input_name) {
    auto it = m->input_v.find(input_name);
    if (it == m->input_v.end()) return fail(MIMIR_B200_E_INVALID, "tensor_slot: '%s' is not a graph input", input_name);
    v = it->second;
  }
  const TensorV& t = m->tensors[root_of(m->tensors, v)];
  *offset = t.off_f32;
  *bytes = static_cast<uint64_t>(t.n) * (t.broadcast_input ? 1 : m->planned_micro) * 4;
  return MIMIR_B200_OK;
}

int mimir_b200_model_output_len(MimirB200ModelHandle m, uint64_t* per_sample) {
  if (!m || !per_sample) return fail(MIMIR_B200_E_INVALID, "output_len: null argument");
  if (m->planned_batch <= 0) return fail(MIMIR_B200_E_INVALID, "output_len: plan the model first");
  *per_sample = static_cast<uint64_t>(m->tensors[root_of(m->tensors, m->out_v)].n);
  return MIMIR_B200_OK;
}

int mimir_b200_model_num_layers(MimirB200ModelHandle m, int* n) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m || !n) return fail(MIMIR_B200_E_INVALID, "null model handle");
  *n = static_cast<int>(m->layers.size());
  return MIMIR_B200_OK;
}

int mimir_b200_model_plan(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs, int batch, uint64_t* arena_peak_bytes) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (!inputs || n_inputs <= 0) return fail(MIMIR_B200_E_INVALID, "plan: no inputs declared");
  MB_TRY(plan_model(m, inputs, n_inputs, batch));
  if (arena_peak_bytes) *arena_peak_bytes = m->arena_bytes * (m->arena2 ? 2 : 1);
  ctx().stats.weight_bytes = m->weight_bytes;
  return MIMIR_B200_OK;
}

int mimir_b200_model_forward_device(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs, int batch, float* out_dev,
                                    uint64_t out_capacity, uint64_t* out_len, void* stream) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  std::vector<int> vs;
  MB_TRY(check_inputs(m, inputs, n_inputs, batch, &vs));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int out_root = root_of(m->tensors, m->out_v);
  const TensorV& ot = m->tensors[out_root];
  if (out_len) *out_len = static_cast<uint64_t>(ot.n);
  if (!out_dev || out_capacity < static_cast<uint64_t>(ot.n) * batch) return fail(MIMIR_B200_E_INVALID, "forward: output capacity too small");
  const int micro = m->planned_micro;
  // micro-batches run back to back on the caller's stream over the first arena buffer
  for (int c = 0; c < m->pipeline; ++c) {
    Bound b;
    b.in_ptr.assign(m->tensors.size(), nullptr);
    for (int i = 0; i < n_inputs; ++i) {
      const TensorV& t = m->tensors[vs[i]];
      if (t.broadcast_input) {
        // staged again for every micro-batch: the planner may hand the slot to a later tensor once
        // the input's last consumer has run
        float* slot = reinterpret_cast<float*>(m->arena + t.off_f32);
        MB_TRY(launch_broadcast_rows(static_cast<const float*>(inputs[i].data), slot, micro, t.n, st));
      } else {
        b.in_ptr[vs[i]] = static_cast<const float*>(inputs[i].data) + static_cast<size_t>(c) * micro * t.n;
      }
    }
    float* out_c = out_dev + static_cast<size_t>(c) * micro * ot.n;
    if (ot.producer >= 0) b.out_ptr = out_c;
    MB_TRY(run_layers_cached(m, micro, b, st, m->arena));
    if (ot.producer < 0) {  // the graph returns one of its inputs
      const float* src = b.in_ptr[out_root] ? b.in_ptr[out_root] : reinterpret_cast<float*>(m->arena + ot.off_f32);
      MB_CUDA(cudaMemcpyAsync(out_c, src, static_cast<size_t>(ot.n) * micro * 4, cudaMemcpyDeviceToDevice, st));
    }
  }
  ctx().stats.flops_last_forward = m->flops * m->pipeline;
  ctx().stats.bytes_last_forward = m->hbm_bytes * m->pipeline;
  return MIMIR_B200_OK;
}

static int ensure_pipeline_objects(MimirB200Model* m) {
  if (!m->s_comp) {
    MB_CUDA(cudaStreamCreateWithFlags(&m->s_h2d, cudaStreamNonBlocking));
    MB_CUDA(cudaStreamCreateWithFlags(&m->s_comp, cudaStreamNonBlocking));
    MB_CUDA(cudaStreamCreateWithFlags(&m->s_d2h, cudaStreamNonBlocking));
  }
  while (static_cast<int>(m->ev_h2d.size()) < m->pipeline) {
    cudaEvent_t a, b, c;
    MB_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
    MB_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
    MB_CUDA(cudaEventCreateWithFlags(&c, cudaEventDisableTiming));
    m->ev_h2d.push_back(a);
    m->ev_comp.push_back(b);
    m->ev_d2h.push_back(c);
  }
  return MIMIR_B200_OK;
}

int mimir_b200_model_forward(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs, int batch, float* out_host,
                             uint64_t out_capacity, uint64_t* out_len) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  std::vector<int> vs;
  MB_TRY(check_inputs(m, inputs, n_inputs, batch, &vs));
  const TensorV& ot = m->tensors[root_of(m->tensors, m->out_v)];
  if (out_len) *out_len = static_cast<uint64_t>(ot.n);
  if (!out_host || out_capacity < static_cast<uint64_t>(ot.n) * batch) return fail(MIMIR_B200_E_INVALID, "forward: output capacity too small");
  if (!m->ev0) {
    MB_CUDA(cudaEventCreate(&m->ev0));
    MB_CUDA(cudaEventCreate(&m->ev1));
  }
  MB_TRY(ensure_pipeline_objects(m));
  const int micro = m->planned_micro, P = m->pipeline;
  uint8_t* bufs[2] = {m->arena, m->arena2 ? m->arena2 : m->arena};
  MB_CUDA(cudaEventRecord(m->ev0, m->s_comp));
  // copy-in, compute and copy-out of consecutive micro-batches overlap; buffer c & 1 is reused by
  // micro-batch c + 2 only after its compute (inputs) and its copy-out (output) have finished
  for (int c = 0; c < P; ++c) {
    uint8_t* arena = bufs[c & 1];
    if (c >= 2) {
      // buffer c & 1: its inputs may be overwritten once micro-batch c - 2 has been computed; where the output shares
      // bytes with an input slot (see plan) the copy-in must also wait for the copy-out of micro-batch c - 2
      MB_CUDA(cudaStreamWaitEvent(m->s_h2d, m->ev_comp[c - 2], 0));
      if (m->out_in_input_slot) MB_CUDA(cudaStreamWaitEvent(m->s_h2d, m->ev_d2h[c - 2], 0));
    }
    for (int i = 0; i < n_inputs; ++i) {
      const TensorV& t = m->tensors[vs[i]];
      float* slot = reinterpret_cast<float*>(arena + t.off_f32);
      if (t.broadcast_input) {
        // every micro-batch: the slot may have been reused after the input's last consumer
        MB_CUDA(cudaMemcpyAsync(slot, inputs[i].data, static_cast<size_t>(t.n) * 4, cudaMemcpyHostToDevice, m->s_h2d));
        if (micro > 1) MB_TRY(launch_broadcast_rows(slot, slot + t.n, micro - 1, t.n, m->s_h2d));
      } else {
        const float* src = static_cast<const float*>(inputs[i].data) + static_cast<size_t>(c) * micro * t.n;
        MB_CUDA(cudaMemcpyAsync(slot, src, static_cast<size_t>(t.n) * micro * 4, cudaMemcpyHostToDevice, m->s_h2d));
      }
    }
    MB_CUDA(cudaEventRecord(m->ev_h2d[c], m->s_h2d));
    MB_CUDA(cudaStreamWaitEvent(m->s_comp, m->ev_h2d[c], 0));
    if (c >= 2) MB_CUDA(cudaStreamWaitEvent(m->s_comp, m->ev_d2h[c - 2], 0));
    Bound b;
    MB_TRY(run_layers_cached(m, micro, b, m->s_comp, arena));
    MB_CUDA(cudaEventRecord(m->ev_comp[c], m->s_comp));
    MB_CUDA(cudaStreamWaitEvent(m->s_d2h, m->ev_comp[c], 0));
    MB_CUDA(cudaMemcpyAsync(out_host + static_cast<size_t>(c) * micro * ot.n, arena + ot.off_f32, static_cast<size_t>(ot.n) * micro * 4,
                            cudaMemcpyDeviceToHost, m->s_d2h));
    MB_CUDA(cudaEventRecord(m->ev_d2h[c], m->s_d2h));
  }
  MB_CUDA(cudaEventRecord(m->ev1, m->s_comp));
  MB_CUDA(cudaStreamSynchronize(m->s_d2h));
  MB_CUDA(cudaStreamSynchronize(m->s_comp));
  MB_TRY(check_device_error_word(m->s_comp));
  cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1);
  ctx().stats.ms_last_forward = m->last_ms;
  ctx().stats.flops_last_forward = m->flops * P;
  ctx().stats.bytes_last_forward = m->hbm_bytes * P;
  return MIMIR_B200_OK;
}

// ---- incremental decoding ---------------------------------------------------------------------------
// The reference has no key / value cache (its documentation names the absence); a caller that generates token by
// token re-runs the whole prefix.  For graphs whose layers all act per token - Embedding, Linear with seq_len, LayerNorm
// with in_features, activations, element-wise layers, causal self-attention - row t of the full causal forward depends
// only on tokens 0..t, so one token per step against cached keys and values gives the same row.
static int token_wise(const LayerRT& L) {
  switch (L.lt) {
    case LT::Alias: case LT::Act: case LT::Add: case LT::Multiply: case LT::Binary2: case LT::Embedding:
      return MIMIR_B200_OK;
    case LT::Linear:
      if (L.d.seq_len > 0) return MIMIR_B200_OK;
      return fail(MIMIR_B200_E_UNSUPPORTED, "decode: Linear '%s' runs over the flattened sequence (seq_len = 0), not per token", L.name.c_str());
    case LT::LayerNorm:
      if (L.d.in_features > 0) return MIMIR_B200_OK;
      return fail(MIMIR_B200_E_UNSUPPORTED, "decode: LayerNorm '%s' normalises the whole sample (in_features = 0), not one token", L.name.c_str());
    case LT::Attention:
      if (L.d.causal) return MIMIR_B200_OK;
      return fail(MIMIR_B200_E_UNSUPPORTED, "decode: attention '%s' is not causal: every row depends on later tokens", L.name.c_str());
    default:
      return fail(MIMIR_B200_E_UNSUPPORTED, "decode: layer '%s' of type '%s' does not act per token", L.name.c_str(), L.type.c_str());
  }
}

int mimir_b200_model_decode_end(MimirB200ModelHandle m) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (m->decode) {
    cudaDeviceSynchronize();
    destroy_model(m->decode);
    m->decode = nullptr;
    drop_graphs(m);  // captured forwards may write into the caches that just went away
  }
  return MIMIR_B200_OK;
}

int mimir_b200_model_decode_begin(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs, int batch, int max_seq,
                                  uint64_t* cache_bytes) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (m->is_twin) return fail(MIMIR_B200_E_INVALID, "decode_begin: not a model handle");
  if (m->planned_batch <= 0) return fail(MIMIR_B200_E_INVALID, "decode_begin: plan the model first (its operand planes are shared)");
  if (m->pipeline != 1) return fail(MIMIR_B200_E_UNSUPPORTED, "decode_begin: set_pipeline(1) first");
  if (!inputs || n_inputs <= 0 || batch <= 0 || max_seq <= 0) return fail(MIMIR_B200_E_INVALID, "decode_begin: bad arguments");
  MB_TRY(mimir_b200_model_decode_end(m));
  for (const auto& L : m->layers) MB_TRY(token_wise(L));
  auto t = std::make_unique<MimirB200Model>();
  t->is_twin = true;
  t->device = m->device;
  t->precision = m->precision;
  t->max_seq = max_seq;
  t->layers = m->layers;  // descriptors, classification and weight pointers
  uint64_t bytes = 0;
  int status = MIMIR_B200_OK;
  for (auto& L : t->layers) {
    L.borrowed_f32 = true;
    L.borrowed_planes = (L.w_split != nullptr);
    L.kcache = L.vcache = nullptr;
    if (L.d.seq_len > 0) L.d.seq_len = 1;  // one token per sample and step
  }
  status = plan_model(t.get(), inputs, n_inputs, batch);
  for (auto& L : t->layers) {
    if (status != MIMIR_B200_OK) break;
    if (L.lt != LT::Attention) continue;
    L.cache_bytes = static_cast<size_t>(batch) * max_seq * L.embed * sizeof(float);
    status = dev_alloc(reinterpret_cast<void**>(&L.kcache), L.cache_bytes, "key cache");
    if (status == MIMIR_B200_OK) status = dev_alloc(reinterpret_cast<void**>(&L.vcache), L.cache_bytes, "value cache");
    bytes += 2 * L.cache_bytes;
    t->decode_scratch_bytes = std::max(t->decode_scratch_bytes, attention_decode_scratch_bytes(batch, L.heads, L.embed, max_seq));
    if (status == MIMIR_B200_OK && batch <= 16 && L.w_f32 && L.w_count >= static_cast<size_t>(4) * L.embed * L.embed) {
      // Wqkv [E][3E] and Wout [E][E] are stored input-major; the weight-streaming kernel reads W[out][in]
      const int E = L.embed;
      L.w_t_bytes = static_cast<size_t>(4) * E * E * sizeof(float);
      status = dev_alloc(reinterpret_cast<void**>(&L.w_t_f32), L.w_t_bytes, "attention weights, output-major");
      const int s1[2] = {E, 3 * E}, s2[2] = {E, E}, dims[2] = {1, 0};
      if (status == MIMIR_B200_OK) status = launch_permute(L.w_f32, L.w_t_f32, 1, 2, s1, dims, nullptr);
      if (status == MIMIR_B200_OK)
        status = launch_permute(L.w_f32 + static_cast<size_t>(3) * E * E, L.w_t_f32 + static_cast<size_t>(3) * E * E, 1, 2, s2, dims, nullptr);
      t->skinny_scratch_bytes = std::max(t->skinny_scratch_bytes, skinny_scratch_bytes(batch, E, 3 * E));
    }
  }
  bool pos_on_device = (status == MIMIR_B200_OK);
  for (const auto& L : t->layers)
    if (L.lt == LT::Attention) {
      const int hd = L.heads > 0 ? L.embed / L.heads : 0;
      pos_on_device = pos_on_device && hd > 0 && hd % 4 == 0 && hd <= 512 && L.embed % 4 == 0;
    }
  if (pos_on_device) status = dev_alloc(reinterpret_cast<void**>(&t->pos_dev), 256, "decode position");
  if (status == MIMIR_B200_OK && t->skinny_scratch_bytes)
    status = dev_alloc(reinterpret_cast<void**>(&t->skinny_scratch), t->skinny_scratch_bytes, "decode projection scratch");
  if (status == MIMIR_B200_OK && t->decode_scratch_bytes)
    status = dev_alloc(reinterpret_cast<void**>(&t->decode_scratch), t->decode_scratch_bytes, "decode attention scratch");
  if (status != MIMIR_B200_OK) {
    destroy_model(t.release());
    return status;
  }
  t->twin_epoch = m->plan_epoch;
  m->decode = t.release();
  drop_graphs(m);  // forwards captured so far do not fill the caches
  if (cache_bytes) *cache_bytes = bytes;
  return MIMIR_B200_OK;
}

int mimir_b200_model_decode_step(MimirB200ModelHandle m, const MimirNamedInput* inputs, int n_inputs, int batch, int pos,
                                 float* out_host, uint64_t out_capacity, uint64_t* out_len) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (!m->decode) return fail(MIMIR_B200_E_INVALID, "decode_step: decode_begin has not been called");
  if (m->decode->twin_epoch != m->plan_epoch || m->planned_batch <= 0)
    return fail(MIMIR_B200_E_INVALID, "decode_step: the model was planned or its weights changed since decode_begin; call decode_begin again");
  if (pos < 0 || pos >= m->decode->max_seq) return fail(MIMIR_B200_E_INVALID, "decode_step: position %d outside the cache of %d", pos, m->decode->max_seq);
  MimirB200Model* t = m->decode;
  t->decode_pos = pos;
  if (t->pos_dev) {
    // the previous step has fully drained (forward synchronises), so the word can be rewritten before this one starts
    MB_TRY(ensure_pipeline_objects(t));
    MB_CUDA(cudaMemcpyAsync(t->pos_dev, &t->decode_pos, sizeof(int), cudaMemcpyHostToDevice, t->s_comp));
  }
  return mimir_b200_model_forward(t, inputs, n_inputs, batch, out_host, out_capacity, out_len);
}

// Cuts the batch of the host-pointer forward into `micro_batches` pieces that overlap their
// copy-in, compute and copy-out (takes effect at the next plan; batch must be a multiple).
int mimir_b200_model_set_pipeline(MimirB200ModelHandle m, int micro_batches) {
  DeviceScope dev_scope(m ? m->device : ctx().device);
  if (!m) return fail(MIMIR_B200_E_INVALID, "null model handle");
  if (micro_batches < 1 || micro_batches > 1024) return fail(MIMIR_B200_E_INVALID, "set_pipeline: micro_batches must be in 1..1024");
  if (micro_batches != m->pipeline) m->planned_batch = 0;
  m->pipeline = micro_batches;
  return MIMIR_B200_OK;
}

int mimir_b200_get_stats(MimirB200Stats* out) {
  if (!out) return fail(MIMIR_B200_E_INVALID, "get_stats: null output");
  *out = ctx().stats;
  out->kernels_launched = ctx().launches.load();
  return MIMIR_B200_OK;
}

// Reads the device error word that bounded waits set; OK when no wait gave up.
int mimir_b200_check_device(void* stream) {
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called");
  return check_device_error_word(static_cast<cudaStream_t>(stream));
}

// Live timing of the contraction kernel with CUDA events on the launching stream.
int mimir_b200_selftest_wait_timeout(unsigned long long limit_ns, void* stream) {
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called");
  return launch_wait_timeout_selftest(limit_ns, static_cast<cudaStream_t>(stream));
}

int mimir_b200_profile_gemm(int enable) {
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called");
  ctx().prof_gemm = enable != 0;
  return MIMIR_B200_OK;
}
// Synchronises the device, sums the recorded GEMM durations and clears the record.
int mimir_b200_profile_read(float* total_ms, int* launches) {
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called");
  MB_CUDA(cudaDeviceSynchronize());
  float tot = 0.f;
  auto& ev = ctx().prof_events;
  for (size_t i = 0; i + 1 < ev.size(); i += 2) {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
    tot += ms;
    cudaEventDestroy(ev[i]);
    cudaEventDestroy(ev[i + 1]);
  }
  if (total_ms) *total_ms = tot;
  if (launches) *launches = static_cast<int>(ev.size() / 2);
  ev.clear();
  return MIMIR_B200_OK;
}

int mimir_b200_shutdown(void) {
  std::set<MimirB200Model*> models;
  {
    std::lock_guard<std::mutex> lk(g_models_mu);
    models.swap(g_models);
  }
  int prev = 0;
  const bool have_prev = cudaGetDevice(&prev) == cudaSuccess;
  for (int d = 0; d < MAX_DEVICES; ++d) {
    if (!ctx_of(d).initialised) continue;
    cudaSetDevice(d);
    cudaDeviceSynchronize();
  }
  for (auto* m : models) {
    cudaSetDevice(m->device);
    destroy_model(m);
  }
  for (int d = 0; d < MAX_DEVICES; ++d) {
    if (!ctx_of(d).initialised) continue;
    cudaSetDevice(d);
    release_owned_buffers();
  }
  if (have_prev) cudaSetDevice(prev); else cudaGetLastError();
  return MIMIR_B200_OK;
}

}  // extern "C"
