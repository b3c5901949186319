// pointwise.cu — HBM-bound element-wise and data-movement ops.  Vectorised 128-bit accesses where
// the pointers and sizes allow it, grid-stride loops sized to the SM count.
//   eltwise            : LayerOps::add_forward / multiply_forward (LayerOps.hpp:142-230) and the
//                        activations (LayerOps.hpp:556-623)
//   embedding          : Embedding case of the layer switch (Model.cpp:5301-5334, 1152-1205)
//   upsample_nearest   : LayerOps::upsample_nearest_forward (LayerOps.hpp:802-827)
//   permute            : LayerOps::permute_forward (LayerOps.hpp:880-945)
//   token_mean_pool    : Model.cpp:5571-5589;  global_avgpool : LayerOps.hpp:459-482
#include "common.h"

namespace mb {
namespace {

__device__ __forceinline__ float act_apply(int op, float v, float alpha = 0.0f) {
  switch (op) {
    // LayerOpsExt.hpp:29-99
    case MIMIR_B200_ELT_LEAKY_RELU: return v > 0.0f ? v : alpha * v;
    case MIMIR_B200_ELT_ELU: return v >= 0.0f ? v : alpha * (expf(v) - 1.0f);  // Model.hpp:505-509
    case MIMIR_B200_ELT_SOFTPLUS: return v > 20.0f ? v : logf(1.0f + expf(v));
    case MIMIR_B200_ELT_MISH: return v * tanhf(v > 20.0f ? v : logf(1.0f + expf(v)));
    case MIMIR_B200_ELT_HARD_SIGMOID: return fmaxf(0.0f, fminf(1.0f, (v + 3.0f) / 6.0f));
    case MIMIR_B200_ELT_HARD_SWISH: return v * fmaxf(0.0f, fminf(1.0f, (v + 3.0f) / 6.0f));
    case MIMIR_B200_ELT_GELU: {
      const float c = 0.7978845608f;  // sqrt(2.0f / 3.14159265359f) in fp32
      return v * (0.5f * (1.0f + tanhf(c * (v + 0.044715f * v * v * v))));
    }
    case MIMIR_B200_ELT_SILU: return v * (1.0f / (1.0f + expf(-v)));
    case MIMIR_B200_ELT_RELU: return fmaxf(0.0f, v);
    case MIMIR_B200_ELT_TANH: return tanhf(v);
    case MIMIR_B200_ELT_SIGMOID: return 1.0f / (1.0f + expf(-v));
    default: return v;
  }
}

template <int OP>
__global__ void unary_kernel(const float* __restrict__ a, float* __restrict__ y, long long total, float alpha) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (vec) {
    const long long n4 = total >> 2;
    for (long long i = tid; i < n4; i += stride) {
      float4 v = __ldg(reinterpret_cast<const float4*>(a) + i);
      v.x = act_apply(OP, v.x, alpha); v.y = act_apply(OP, v.y, alpha); v.z = act_apply(OP, v.z, alpha); v.w = act_apply(OP, v.w, alpha);
      reinterpret_cast<float4*>(y)[i] = v;
    }
    for (long long i = (n4 << 2) + tid; i < total; i += stride) y[i] = act_apply(OP, a[i], alpha);
  } else {
    for (long long i = tid; i < total; i += stride) y[i] = act_apply(OP, a[i], alpha);
  }
}

// BOP: 0 add, 1 multiply, 2 subtract (LayerOpsExt.hpp:105-122), 3 divide (LayerOpsExt.hpp:127-148: a divisor
// closer to zero than 1e-8 is replaced by +-1e-8, +1e-8 for +-0)
template <int BOP>
__device__ __forceinline__ float bin_apply(float u, float w) {
  if (BOP == 0) return u + w;
  if (BOP == 1) return u * w;
  if (BOP == 2) return u - w;
  if (fabsf(w) < 1e-8f) w = (w >= 0.0f) ? 1e-8f : -1e-8f;
  return u / w;
}

// y[s, i] = a[s, i] op b[s, i % nb]; nb == n is the plain case
template <int BOP>
__global__ void binary_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y,
                              long long batch, long long n, long long nb) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long total = batch * n;
  const bool vec = (nb == n) && (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                                   reinterpret_cast<uintptr_t>(y)) & 15) == 0);
  if (vec) {
    const long long n4 = total >> 2;
    for (long long i = tid; i < n4; i += stride) {
      const float4 u = __ldg(reinterpret_cast<const float4*>(a) + i);
      const float4 w = __ldg(reinterpret_cast<const float4*>(b) + i);
      float4 r;
      r.x = bin_apply<BOP>(u.x, w.x); r.y = bin_apply<BOP>(u.y, w.y); r.z = bin_apply<BOP>(u.z, w.z); r.w = bin_apply<BOP>(u.w, w.w);
      reinterpret_cast<float4*>(y)[i] = r;
    }
    for (long long i = (n4 << 2) + tid; i < total; i += stride) y[i] = bin_apply<BOP>(a[i], b[i]);
  } else {
    for (long long i = tid; i < total; i += stride) {
      const long long s = i / n, j = i - s * n;
      const float w = b[s * nb + (j % nb)];
      y[i] = bin_apply<BOP>(a[i], w);
    }
  }
}

__global__ void embedding_kernel(const float* __restrict__ ids_f, const int32_t* __restrict__ ids_i,
                                 const float* __restrict__ table, float* __restrict__ y, long long n_ids, int vocab,
                                 int dim, int padding_idx) {
  // one warp per id row
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const bool vec = ((dim & 3) == 0) && (((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(y)) & 15) == 0);
  for (long long t = warp; t < n_ids; t += nwarps) {
    long long id;
    if (ids_f != nullptr) id = llround(static_cast<double>(ids_f[t]));  // Model.cpp:5322
    else id = ids_i[t];
    const bool zero = (padding_idx >= 0 && id == padding_idx) || id < 0 || id >= vocab;
    float* out = y + t * dim;
    const float* row = table + (zero ? 0 : id) * static_cast<long long>(dim);
    if (vec) {
      for (int d = lane; d < (dim >> 2); d += 32)
        reinterpret_cast<float4*>(out)[d] = zero ? make_float4(0.f, 0.f, 0.f, 0.f) : __ldg(reinterpret_cast<const float4*>(row) + d);
    } else {
      for (int d = lane; d < dim; d += 32) out[d] = zero ? 0.0f : __ldg(row + d);
    }
  }
}

__global__ void upsample_nearest_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int in_h,
                                        int in_w, int sh, int sw) {
  const int oh = in_h * sh, ow = in_w * sw;
  const long long total = planes * oh * ow;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride) {
    const int q = static_cast<int>(i % ow);
    const long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    const long long pl = t / oh;
    y[i] = __ldg(x + (pl * in_h + r / sh) * in_w + q / sw);
  }
}

// 2 x 2 nearest upsample of rows with an even width: a thread reads two neighbouring input pixels (64 bits)
// and writes the same four values (128 bits) into two output rows; all index math in 32 bits per plane row.
__global__ void upsample_nearest_2x2_kernel(const float* __restrict__ x, float* __restrict__ y, long long plane_rows, int in_w) {
  const int half_w = in_w >> 1;
  const long long total = plane_rows * half_w;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride) {
    const long long row = i / half_w;            // (plane, input row)
    const int q = static_cast<int>(i - row * half_w);
    const float2 v = __ldcs(reinterpret_cast<const float2*>(x + row * in_w) + q);
    const float4 o = make_float4(v.x, v.x, v.y, v.y);
    float* out = y + row * 4 * in_w + 4 * q;     // output row 2*r of the same plane: (plane*in_h + r) * 2 * (2*in_w)
    __stcs(reinterpret_cast<float4*>(out), o);
    __stcs(reinterpret_cast<float4*>(out + 2 * in_w), o);
  }
}

struct PermuteDesc {
  int nd;
  long long out_shape[MIMIR_B200_MAX_DIMS];
  long long in_stride_of_out[MIMIR_B200_MAX_DIMS];  // input stride of the dim that output dim i walks
  long long total;
};

__global__ void permute_kernel(const float* __restrict__ x, float* __restrict__ y, PermuteDesc d, long long batch) {
  const long long all = batch * d.total;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < all; i += stride) {
    const long long s = i / d.total;
    long long t = i - s * d.total, in_idx = 0;
    for (int k = d.nd - 1; k >= 0; --k) {
      const long long c = t % d.out_shape[k];
      t /= d.out_shape[k];
      in_idx += c * d.in_stride_of_out[k];
    }
    y[i] = __ldg(x + s * d.total + in_idx);
  }
}

// y[s, d] = (sum_t x[s, t, d]) * (1/seq): sequential in t like the reference
__global__ void token_mean_pool_kernel(const float* __restrict__ x, float* __restrict__ y, int batch, int seq, int dim) {
  const long long total = static_cast<long long>(batch) * dim;
  const float inv = 1.0f / static_cast<float>(seq);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long s = i / dim, d = i - s * dim;
    const float* p = x + s * seq * dim + d;
    float acc = 0.0f;
    for (int t = 0; t < seq; ++t) acc += __ldg(p + static_cast<long long>(t) * dim);
    y[i] = acc * inv;
  }
}

// one warp per (sample, channel) plane
__global__ void global_avgpool_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int hw) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long pl = warp; pl < planes; pl += nwarps) {
    const float* p = x + pl * hw;
    float acc = 0.0f;
    for (int i = lane; i < hw; i += 32) acc += __ldg(p + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[pl] = acc / static_cast<float>(hw);
  }
}

// first maximum wins, like a sequential scan
__global__ void argmax_rows_kernel(const float* __restrict__ x, int32_t* __restrict__ ids, long long rows, int n) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    const float* p = x + r * n;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lane; i < n; i += 32) {
      const float v = __ldg(p + i);
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) ids[r] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

__global__ void copy_strided_kernel(const float* __restrict__ src, float* __restrict__ dst, long long batch, long long n,
                                    long long total, long long off, long long src_stride) {
  const long long all = batch * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < all;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long s = i / n, j = i - s * n;
    dst[s * total + off + j] = __ldg(src + s * src_stride + j);
  }
}

int grid_for(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(ctx().sm_count) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

int launch_eltwise(int op, const float* a, const float* b, float* y, int batch, int64_t n, int64_t nb, cudaStream_t st,
                   float alpha) {
  if (batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "eltwise: inputs must be non-empty");
  const long long total = static_cast<long long>(batch) * n;
  const int threads = 256;
  const int grid = grid_for((total + 3) / 4, threads);
  switch (op) {
    case MIMIR_B200_ELT_ADD:
    case MIMIR_B200_ELT_MULTIPLY:
      if (!b || nb <= 0) return fail(MIMIR_B200_E_INVALID, "eltwise: second input missing");
      if (op == MIMIR_B200_ELT_MULTIPLY && nb != n) return fail(MIMIR_B200_E_INVALID, "Multiply: input sizes must match");
      if (nb != n && nb != 1 && (n % nb) != 0)
        return fail(MIMIR_B200_E_INVALID, "Add: input sizes must match or be broadcastable");
      if (op == MIMIR_B200_ELT_ADD) binary_kernel<0><<<grid, threads, 0, st>>>(a, b, y, batch, n, nb);
      else binary_kernel<1><<<grid, threads, 0, st>>>(a, b, y, batch, n, nb);
      break;
    case MIMIR_B200_ELT_SUBTRACT:
    case MIMIR_B200_ELT_DIVIDE:
      if (!b || nb != n)
        return fail(MIMIR_B200_E_INVALID, "%s: size mismatch: %lld vs %lld", op == MIMIR_B200_ELT_SUBTRACT ? "Subtract" : "Divide",
                    static_cast<long long>(n), static_cast<long long>(nb));
      if (op == MIMIR_B200_ELT_SUBTRACT) binary_kernel<2><<<grid, threads, 0, st>>>(a, b, y, batch, n, nb);
      else binary_kernel<3><<<grid, threads, 0, st>>>(a, b, y, batch, n, nb);
      break;
    case MIMIR_B200_ELT_GELU: unary_kernel<MIMIR_B200_ELT_GELU><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_SILU: unary_kernel<MIMIR_B200_ELT_SILU><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_RELU: unary_kernel<MIMIR_B200_ELT_RELU><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_TANH: unary_kernel<MIMIR_B200_ELT_TANH><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_SIGMOID: unary_kernel<MIMIR_B200_ELT_SIGMOID><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_LEAKY_RELU: unary_kernel<MIMIR_B200_ELT_LEAKY_RELU><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_ELU: unary_kernel<MIMIR_B200_ELT_ELU><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_SOFTPLUS: unary_kernel<MIMIR_B200_ELT_SOFTPLUS><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_MISH: unary_kernel<MIMIR_B200_ELT_MISH><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_HARD_SIGMOID: unary_kernel<MIMIR_B200_ELT_HARD_SIGMOID><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    case MIMIR_B200_ELT_HARD_SWISH: unary_kernel<MIMIR_B200_ELT_HARD_SWISH><<<grid, threads, 0, st>>>(a, y, total, alpha); break;
    default: return fail(MIMIR_B200_E_INVALID, "eltwise: unknown op %d", op);
  }
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_embedding(const float* ids_f32, const int32_t* ids_i32, const float* table, float* y, int64_t n_ids, int vocab,
                     int dim, int padding_idx, cudaStream_t st) {
  if (n_ids <= 0) return MIMIR_B200_OK;
  if ((ids_f32 == nullptr) == (ids_i32 == nullptr)) return fail(MIMIR_B200_E_INVALID, "embedding: give exactly one id array");
  const int threads = 256;
  embedding_kernel<<<grid_for(n_ids * 32, threads), threads, 0, st>>>(ids_f32, ids_i32, table, y, n_ids, vocab, dim, padding_idx);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_upsample_nearest(const float* x, float* y, int batch, int ch, int in_h, int in_w, int sh, int sw, cudaStream_t st) {
  if (batch <= 0 || ch <= 0 || in_h <= 0 || in_w <= 0 || sh <= 0 || sw <= 0)
    return fail(MIMIR_B200_E_INVALID, "UpsampleNearest: dimensions (out_h, out_w, in_channels) must be set");
  const long long planes = static_cast<long long>(batch) * ch;
  const long long total = planes * in_h * sh * in_w * sw;
  if (sh == 2 && sw == 2 && (in_w & 1) == 0 && ((reinterpret_cast<uintptr_t>(x) & 7) | (reinterpret_cast<uintptr_t>(y) & 15)) == 0) {
    const long long items = planes * in_h * (in_w >> 1);
    upsample_nearest_2x2_kernel<<<grid_for(items, 256), 256, 0, st>>>(x, y, planes * in_h, in_w);
    MB_CUDA(cudaGetLastError());
    count_launch();
    return MIMIR_B200_OK;
  }
  upsample_nearest_kernel<<<grid_for(total, 256), 256, 0, st>>>(x, y, planes, in_h, in_w, sh, sw);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_permute(const float* x, float* y, int batch, int nd, const int* shape, const int* dims, cudaStream_t st) {
  if (nd <= 0 || nd > MIMIR_B200_MAX_DIMS) return fail(MIMIR_B200_E_INVALID, "Permute: dims and shape cannot be empty");
  PermuteDesc d;
  d.nd = nd;
  long long in_stride[MIMIR_B200_MAX_DIMS];
  in_stride[nd - 1] = 1;
  for (int i = nd - 2; i >= 0; --i) in_stride[i] = in_stride[i + 1] * shape[i + 1];
  d.total = 1;
  unsigned seen = 0;
  for (int i = 0; i < nd; ++i) {
    if (dims[i] < 0 || dims[i] >= nd || shape[i] <= 0) return fail(MIMIR_B200_E_INVALID, "Permute: bad dims/shape");
    seen |= 1u << dims[i];
    d.out_shape[i] = shape[dims[i]];
    d.in_stride_of_out[i] = in_stride[dims[i]];
    d.total *= shape[i];
  }
  if (seen != (1u << nd) - 1) return fail(MIMIR_B200_E_INVALID, "Permute: dims is not a permutation");
  permute_kernel<<<grid_for(d.total * batch, 256), 256, 0, st>>>(x, y, d, batch);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_token_mean_pool(const float* x, float* y, int batch, int seq, int dim, cudaStream_t st) {
  if (seq <= 0 || dim <= 0) return fail(MIMIR_B200_E_INVALID, "TokenMeanPool: seq_len and embed_dim must be set");
  token_mean_pool_kernel<<<grid_for(static_cast<long long>(batch) * dim, 128), 128, 0, st>>>(x, y, batch, seq, dim);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_global_avgpool(const float* x, float* y, int batch, int ch, int hw, cudaStream_t st) {
  const long long planes = static_cast<long long>(batch) * ch;
  global_avgpool_kernel<<<grid_for(planes * 32, 256), 256, 0, st>>>(x, y, planes, hw);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_argmax_rows(const float* x, int32_t* ids, int64_t rows, int n, cudaStream_t st) {
  if (rows <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "argmax: empty input");
  argmax_rows_kernel<<<grid_for(rows * 32, 256), 256, 0, st>>>(x, ids, rows, n);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_copy_strided(const float* src, float* dst, int batch, int64_t n, int64_t total, int64_t off, cudaStream_t st,
                        int64_t src_stride) {
  if (batch <= 0 || n <= 0) return MIMIR_B200_OK;
  copy_strided_kernel<<<grid_for(static_cast<long long>(batch) * n, 256), 256, 0, st>>>(src, dst, batch, n, total, off,
                                                                                        src_stride > 0 ? src_stride : n);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_broadcast_rows(const float* src, float* dst, int batch, int64_t n, cudaStream_t st) {
  if (batch <= 0 || n <= 0) return MIMIR_B200_OK;
  copy_strided_kernel<<<grid_for(static_cast<long long>(batch) * n, 256), 256, 0, st>>>(src, dst, batch, n, n, 0, 0);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

}  // namespace mb
