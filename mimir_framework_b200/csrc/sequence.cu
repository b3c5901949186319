// sequence.cu — EmbeddingBag, PatchEmbed, Bilinear and the recurrent layers (RNN / GRU / LSTM) of the layer switch in
// Model::forwardPassView (Model.cpp:5203-5295, 5336-5381, 6084-6262).  fp32 throughout; every sample of the batch is an
// independent forward of the reference, so the batch is the outermost grid dimension everywhere.
#include "common.h"

namespace mb {
namespace {

// EmbeddingBag (Model.cpp:5336-5381): one CTA per (bag, sample); a thread owns output columns and walks the bag's ids in
// order, so every column is summed in the reference's order.  offsets == nullptr: one bag over every id.
__global__ void embedding_bag_kernel(const float* __restrict__ ids, long long ids_ps, const float* __restrict__ offsets,
                                     long long off_ps, const float* __restrict__ table, float* __restrict__ y, int bags, int vocab,
                                     int dim, int padding_idx) {
  const int bag = blockIdx.x;
  const long long smp = blockIdx.y;
  const float* id_row = ids + smp * ids_ps;
  long long s = 0, e = ids_ps;
  if (offsets != nullptr) {
    // the reference narrows the rounded offset to int before clamping (Model.cpp:5355, 5365-5366)
    s = static_cast<int>(llround(static_cast<double>(offsets[smp * off_ps + bag])));
    e = static_cast<int>(llround(static_cast<double>(offsets[smp * off_ps + bag + 1])));
  }
  s = s < 0 ? 0 : (s > ids_ps ? ids_ps : s);
  e = e < s ? s : (e > ids_ps ? ids_ps : e);
  float* out = y + (smp * bags + bag) * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float acc = 0.0f;
    for (long long t = s; t < e; ++t) {
      const long long id = llround(static_cast<double>(__ldg(id_row + t)));
      if ((padding_idx >= 0 && id == padding_idx) || id < 0 || id >= vocab) continue;
      acc += __ldg(table + id * dim + d);
    }
    out[d] = acc;
  }
}

// PatchEmbed (Model.cpp:5203-5243): the text block is copied, every patch is projected: one thread per output element,
// the sum starts at the bias and runs over k ascending with the 1/sqrt(patch_dim) scale applied to the input element
// first, as the reference does.  W is [patch_dim][d_model]: consecutive threads read consecutive columns.
__global__ void patch_embed_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, long long in_ps,
                                   long long out_ps, int text, int d_model, int num_patches, int patch_dim, float inv) {
  const long long smp = blockIdx.y;
  const float* xs = x + smp * in_ps;
  float* ys = y + smp * out_ps;
  const float* b = w + static_cast<long long>(patch_dim) * d_model;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < out_ps;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (i < text) {
      ys[i] = xs[i];
      continue;
    }
    const int p = static_cast<int>((i - text) / d_model), d = static_cast<int>((i - text) - static_cast<long long>(p) * d_model);
    const float* xp = xs + text + static_cast<long long>(p) * patch_dim;
    float sum = __ldg(b + d);
    for (int k = 0; k < patch_dim; ++k) sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(__ldg(xp + k), inv), __ldg(w + static_cast<long long>(k) * d_model + d)));
    ys[i] = sum;
  }
}

// Bilinear (Model.cpp:5247-5295): one warp per (row, output); lanes stride over j (W[o][i][:] is contiguous), partial
// sums are combined by shuffles.  Products are taken as (x1 * W) * x2 like the reference; the order of the additions
// differs from its single running sum.
__global__ void bilinear_kernel(const float* __restrict__ x1, const float* __restrict__ x2, const float* __restrict__ w,
                                const float* __restrict__ bias, float* __restrict__ y, long long rows, int in1, int in2, int out_f) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long item = warp; item < rows * out_f; item += nwarps) {
    const long long r = item / out_f;
    const int o = static_cast<int>(item - r * out_f);
    const float* a = x1 + r * in1;
    const float* b = x2 + r * in2;
    const float* wo = w + static_cast<long long>(o) * in1 * in2;
    float acc = 0.0f;
    for (int i = 0; i < in1; ++i) {
      const float ai = __ldg(a + i);
      const float* wr = wo + static_cast<long long>(i) * in2;
      for (int j = lane; j < in2; j += 32) acc = fmaf(ai * __ldg(wr + j), __ldg(b + j), acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) y[item] = acc + (bias != nullptr ? __ldg(bias + o) : 0.0f);
  }
}

__device__ __forceinline__ float sigmoid_ref(float v) { return 1.0f / (1.0f + expf(-v)); }

__device__ __forceinline__ float warp_dot(const float* __restrict__ wrow, const float* v, int n, int lane) {
  float acc = 0.0f;
  for (int i = lane; i < n; i += 32) acc = fmaf(__ldg(wrow + i), v[i], acc);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  return acc;
}

// Recurrent layers (Model.cpp:6084-6262): one CTA per sample walks the T steps; the hidden state (and the LSTM cell)
// lives in shared memory, a warp owns hidden units h = warp, warp + nwarps, ... and computes their gate dot products
// with its lanes striding over the weight rows.  KIND 0 = RNN, 1 = GRU (r, z, n), 2 = LSTM (i, f, g, o).
// Shared memory: x_t[I] | h_prev[H] | h_next[H] | (LSTM) c[H].
template <int KIND>
__global__ void __launch_bounds__(256) recurrent_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                                                        int T, int I, int H, int use_bias) {
  extern __shared__ float rs[];
  constexpr int G = KIND == 0 ? 1 : (KIND == 1 ? 3 : 4);
  float* xt = rs;
  float* hp = xt + I;
  float* hn = hp + H;
  float* cp = hn + H;
  const float* Wih = w;
  const float* Whh = Wih + static_cast<long long>(G) * H * I;
  const float* bih = use_bias ? Whh + static_cast<long long>(G) * H * H : nullptr;
  const float* bhh = use_bias ? bih + static_cast<long long>(G) * H : nullptr;
  const long long smp = blockIdx.x;
  const float* xs = x + smp * T * I;
  float* ys = y + smp * T * H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    hp[h] = 0.0f;
    if (KIND == 2) cp[h] = 0.0f;
  }
  for (int t = 0; t < T; ++t) {
    for (int i = threadIdx.x; i < I; i += blockDim.x) xt[i] = xs[static_cast<long long>(t) * I + i];
    __syncthreads();  // x_t and h_prev (previous step's h_next copy) are in place
    for (int h = warp; h < H; h += nwarps) {
      float s[G], hh[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        s[g] = warp_dot(Wih + static_cast<long long>(g * H + h) * I, xt, I, lane);
        hh[g] = warp_dot(Whh + static_cast<long long>(g * H + h) * H, hp, H, lane);
      }
      if (lane == 0) {
        float b[G];
#pragma unroll
        for (int g = 0; g < G; ++g) b[g] = (bih ? __ldg(bih + g * H + h) : 0.0f) + (bhh ? __ldg(bhh + g * H + h) : 0.0f);
        float out;
        if (KIND == 0) {
          out = tanhf(s[0] + hh[0] + b[0]);
        } else if (KIND == 1) {
          const float r = sigmoid_ref(s[0] + hh[0] + b[0]);
          const float z = sigmoid_ref(s[1] + hh[1] + b[1]);
          const float n = tanhf(s[2] + b[2] + r * hh[2]);  // the hidden sum of the n gate is scaled by r (Model.cpp:6181)
          out = (1.0f - z) * n + z * hp[h];
        } else {
          const float ig = sigmoid_ref(s[0] + hh[0] + b[0]);
          const float fg = sigmoid_ref(s[1] + hh[1] + b[1]);
          const float gg = tanhf(s[2] + hh[2] + b[2]);
          const float og = sigmoid_ref(s[3] + hh[3] + b[3]);
          const float c = fg * cp[h] + ig * gg;
          cp[h] = c;  // only this warp touches cell h
          out = og * tanhf(c);
        }
        hn[h] = out;
        ys[static_cast<long long>(t) * H + h] = out;
      }
    }
    __syncthreads();  // every unit of step t is done reading h_prev
    for (int h = threadIdx.x; h < H; h += blockDim.x) hp[h] = hn[h];
  }
}

}  // namespace

int launch_embedding_bag(const float* ids, int64_t ids_ps, const float* offsets, int64_t off_ps, const float* table, float* y, int batch,
                         int vocab, int dim, int padding_idx, cudaStream_t st) {
  if (batch <= 0 || ids_ps < 0 || vocab <= 0 || dim <= 0) return fail(MIMIR_B200_E_INVALID, "EmbeddingBag: invalid dimensions");
  if (offsets != nullptr && off_ps < 2) return fail(MIMIR_B200_E_INVALID, "EmbeddingBag: offsets must have at least 2 entries");
  const int64_t bags = offsets != nullptr ? off_ps - 1 : 1;
  if (bags > 0x7fffffff || batch > 65535) return fail(MIMIR_B200_E_INVALID, "EmbeddingBag: too many bags or samples for one launch");
  const int threads = dim >= 256 ? 256 : (dim >= 128 ? 128 : (dim >= 64 ? 64 : 32));
  embedding_bag_kernel<<<dim3(static_cast<unsigned>(bags), batch), threads, 0, st>>>(ids, ids_ps, offsets, off_ps, table, y,
                                                                                    static_cast<int>(bags), vocab, dim, padding_idx);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_patch_embed(const float* x, const float* w, float* y, int batch, int d_model, int seq_text, int num_patches, int patch_dim,
                       cudaStream_t st) {
  if (batch <= 0 || batch > 65535 || d_model <= 0 || seq_text <= 0 || num_patches <= 0 || patch_dim <= 0)
    return fail(MIMIR_B200_E_INVALID, "PatchEmbed: invalid dimensions");
  const long long text = static_cast<long long>(seq_text + 1) * d_model;
  const long long in_ps = text + static_cast<long long>(num_patches) * patch_dim;
  const long long out_ps = static_cast<long long>(seq_text + 1 + num_patches) * d_model;
  if (text > 0x7fffffff) return fail(MIMIR_B200_E_INVALID, "PatchEmbed: text block too large");
  const long long blocks = std::min<long long>((out_ps + 255) / 256, 4096);
  patch_embed_kernel<<<dim3(static_cast<unsigned>(blocks), batch), 256, 0, st>>>(x, w, y, in_ps, out_ps, static_cast<int>(text), d_model,
                                                                                 num_patches, patch_dim,
                                                                                 1.0f / sqrtf(static_cast<float>(patch_dim)));
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_bilinear(const float* x1, const float* x2, const float* w, const float* bias, float* y, int64_t rows, int in1, int in2,
                    int out_f, cudaStream_t st) {
  if (rows <= 0 || in1 <= 0 || in2 <= 0 || out_f <= 0) return fail(MIMIR_B200_E_INVALID, "Bilinear: invalid dimensions");
  const long long items = rows * out_f;
  const long long blocks = std::min<long long>((items * 32 + 255) / 256, static_cast<long long>(ctx().sm_count) * 16);
  bilinear_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(x1, x2, w, bias, y, rows, in1, in2, out_f);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_recurrent(int kind, const float* x, const float* w, float* y, int batch, int T, int I, int H, int use_bias, cudaStream_t st) {
  if (batch <= 0 || T <= 0 || I <= 0 || H <= 0 || kind < 0 || kind > 2) return fail(MIMIR_B200_E_INVALID, "Recurrent: invalid dimensions");
  const size_t smem = (static_cast<size_t>(I) + 3 * static_cast<size_t>(H)) * sizeof(float);
  if (smem > 200 * 1024) return fail(MIMIR_B200_E_UNSUPPORTED, "Recurrent: in_features + 3 * out_features = %zu floats do not fit in shared memory", smem / 4);
  auto launch = [&](auto kernel) -> int {
    if (smem > 48 * 1024) MB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<batch, 256, smem, st>>>(x, w, y, T, I, H, use_bias);
    MB_CUDA(cudaGetLastError());
    count_launch();
    return MIMIR_B200_OK;
  };
  if (kind == 0) return launch(recurrent_kernel<0>);
  if (kind == 1) return launch(recurrent_kernel<1>);
  return launch(recurrent_kernel<2>);
}

}  // namespace mb
