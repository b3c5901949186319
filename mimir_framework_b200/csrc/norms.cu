// norms.cu — HBM-bound row reductions: LayerNorm, GroupNorm(+SiLU, +residual), RMSNorm, Softmax.
//   LayerNorm : LayerOps::layernorm_forward  (LayerOps.hpp:264-319)  rows of n, biased variance
//   GroupNorm : LayerOps::groupnorm_forward  (LayerOps.hpp:488-550)  row = one (sample, group) slab
//   RMSNorm   : LayerOpsExt::rms_norm_forward (LayerOpsExt.hpp:345-378) row = the whole sample
//   Softmax   : LayerOps::softmax_forward    (LayerOps.hpp:325-361)  row = the whole sample
//
// Two shapes of kernel per op:
//   * "row" kernels: one CTA per row, the row staged once in shared memory (<= 64 KB), statistics
//     by warp-shuffle + shared-memory reduction, one HBM read and one HBM write per element;
//   * "chunk" kernels for long rows: pass 1 reduces 8192-element chunks to partial statistics in a
//     small global scratch, pass 2 combines the partials of its row and writes the result, so that
//     a handful of very long rows (RMSNorm over a whole sample) still fills every SM.
#include "common.h"

namespace mb {
namespace {

constexpr int ROW_CACHE_FLOATS = 16384;  // 64 KB
constexpr int CHUNK = 8192;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions; `red` is 33 floats of shared memory. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = (lane < nw) ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ float silu(float v) { return v * (1.0f / (1.0f + expf(-v))); }

// Copies `len` floats global -> shared (128-bit when aligned) and returns this thread's partial sum.
__device__ __forceinline__ float stage_and_sum(const float* __restrict__ g, float* s, long long len) {
  float acc = 0.0f;
  if (((reinterpret_cast<uintptr_t>(g) & 15) == 0) && ((len & 3) == 0)) {
    const float4* g4 = reinterpret_cast<const float4*>(g);
    float4* s4 = reinterpret_cast<float4*>(s);
    for (long long i = threadIdx.x; i < (len >> 2); i += blockDim.x) {
      const float4 v = __ldg(g4 + i);
      s4[i] = v;
      acc += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (long long i = threadIdx.x; i < len; i += blockDim.x) {
      const float v = __ldg(g + i);
      s[i] = v;
      acc += v;
    }
  }
  return acc;
}

// Affine description shared by LayerNorm (index = position in the row) and GroupNorm (index =
// channel of the element).
struct Affine {
  const float* gamma;  // may be null
  const float* beta;   // may be null
  int per_channel;     // 0: gamma[i]; 1: gamma[(row % groups) * cpg + i / hw]
  int groups, cpg, hw;
  int act;             // -1 or MIMIR_B200_ELT_SILU
  const float* residual;  // same layout as x, added after the activation; may be null
};

__device__ __forceinline__ float finish(float xn, long long i, long long row, long long base, const Affine& a) {
  float v = xn;
  if (a.gamma != nullptr) {
    const long long gi = a.per_channel ? (static_cast<long long>(row % a.groups) * a.cpg + i / a.hw) : i;
    v *= __ldg(a.gamma + gi);
    if (a.beta != nullptr) v += __ldg(a.beta + gi);
  }
  if (a.act == MIMIR_B200_ELT_SILU) v = silu(v);
  if (a.residual != nullptr) v += __ldg(a.residual + base + i);
  return v;
}

// ---- mean / variance family ------------------------------------------------------------------
__global__ void meanvar_row_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int len, float eps,
                                   Affine a) {
  extern __shared__ __align__(16) float srow[];
  __shared__ float red[33];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = row * len;
    __syncthreads();
    const float mean = block_sum(stage_and_sum(x + base, srow, len), red) / static_cast<float>(len);
    float acc = 0.0f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      const float d = srow[i] - mean;
      acc += d * d;
    }
    const float var = block_sum(acc, red) / static_cast<float>(len);
    const float inv = 1.0f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < len; i += blockDim.x)
      y[base + i] = finish((srow[i] - mean) * inv, i, row, base, a);
  }
}

// pass 1: per chunk (count, mean, M2)
__global__ void meanvar_chunk_stats_kernel(const float* __restrict__ x, float* __restrict__ part, long long len, int chunks,
                                           int chunk_len) {
  extern __shared__ __align__(16) float sch[];
  __shared__ float red[33];
  const long long row = blockIdx.y;
  const int c = blockIdx.x;
  const long long off = static_cast<long long>(c) * chunk_len;
  const long long n = min(static_cast<long long>(chunk_len), len - off);
  const float* g = x + row * len + off;
  const float mean = block_sum(stage_and_sum(g, sch, n), red) / static_cast<float>(n);
  float acc = 0.0f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const float d = sch[i] - mean;
    acc += d * d;
  }
  const float m2 = block_sum(acc, red);
  if (threadIdx.x == 0) {
    float* p = part + (row * chunks + c) * 3;
    p[0] = static_cast<float>(n);
    p[1] = mean;
    p[2] = m2;
  }
}

// pass 2: combine the row's partials (pairwise-update formula of Chan et al.), normalise the chunk
__global__ void meanvar_chunk_apply_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ part,
                                           long long len, int chunks, int chunk_len, float eps, Affine a) {
  const long long row = blockIdx.y;
  const int c = blockIdx.x;
  float n = 0.0f, mean = 0.0f, m2 = 0.0f;
  for (int j = 0; j < chunks; ++j) {
    const float* p = part + (row * chunks + j) * 3;
    const float nb = p[0], mb_ = p[1], m2b = p[2];
    const float nt = n + nb;
    const float delta = mb_ - mean;
    mean += delta * (nb / nt);
    m2 += m2b + delta * delta * (n * nb / nt);
    n = nt;
  }
  const float inv = 1.0f / sqrtf(m2 / n + eps);
  const long long off = static_cast<long long>(c) * chunk_len;
  const long long cn = min(static_cast<long long>(chunk_len), len - off);
  const long long base = row * len;
  const float* g = x + base + off;
  float* o = y + base + off;
  if (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(o)) & 15) == 0 && (cn & 3) == 0 &&
      (!a.per_channel || (a.hw & 3) == 0) && (a.residual == nullptr || (reinterpret_cast<uintptr_t>(a.residual + base + off) & 15) == 0)) {
    for (long long i = threadIdx.x; i < (cn >> 2); i += blockDim.x) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(g) + i);
      const long long e = off + (i << 2);
      float4 r;
      r.x = finish((v.x - mean) * inv, e, row, base, a);
      r.y = finish((v.y - mean) * inv, e + 1, row, base, a);
      r.z = finish((v.z - mean) * inv, e + 2, row, base, a);
      r.w = finish((v.w - mean) * inv, e + 3, row, base, a);
      reinterpret_cast<float4*>(o)[i] = r;
    }
  } else {
    for (long long i = threadIdx.x; i < cn; i += blockDim.x) o[i] = finish((__ldg(g + i) - mean) * inv, off + i, row, base, a);
  }
}

// ---- RMS family ------------------------------------------------------------------------------
__global__ void rms_row_kernel(const float* __restrict__ x, const float* __restrict__ gamma, long long n_gamma,
                               float* __restrict__ y, long long rows, int len, float eps) {
  extern __shared__ __align__(16) float srow[];
  __shared__ float red[33];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = row * len;
    __syncthreads();
    stage_and_sum(x + base, srow, len);
    __syncthreads();
    float acc = 0.0f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) acc += srow[i] * srow[i];
    const float rms = sqrtf(block_sum(acc, red) / static_cast<float>(len) + eps);
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      float v = srow[i] / rms;
      if (gamma != nullptr && i < n_gamma) v *= __ldg(gamma + i);
      y[base + i] = v;
    }
  }
}

__global__ void rms_chunk_stats_kernel(const float* __restrict__ x, float* __restrict__ part, long long len, int chunks,
                                       int chunk_len) {
  __shared__ float red[33];
  const long long row = blockIdx.y;
  const long long off = static_cast<long long>(blockIdx.x) * chunk_len;
  const long long n = min(static_cast<long long>(chunk_len), len - off);
  const float* g = x + row * len + off;
  float acc = 0.0f;
  if ((reinterpret_cast<uintptr_t>(g) & 15) == 0 && (n & 3) == 0) {
    for (long long i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(g) + i);
      acc += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
  } else {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) acc += g[i] * g[i];
  }
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) part[row * chunks + blockIdx.x] = s;
}

__global__ void rms_chunk_apply_kernel(const float* __restrict__ x, const float* __restrict__ gamma, long long n_gamma,
                                       float* __restrict__ y, const float* __restrict__ part, long long len, int chunks,
                                       int chunk_len, float eps) {
  const long long row = blockIdx.y;
  float s = 0.0f;
  for (int j = 0; j < chunks; ++j) s += part[row * chunks + j];
  const float rms = sqrtf(s / static_cast<float>(len) + eps);
  const long long off = static_cast<long long>(blockIdx.x) * chunk_len;
  const long long cn = min(static_cast<long long>(chunk_len), len - off);
  const float* g = x + row * len + off;
  float* o = y + row * len + off;
  if (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(o)) & 15) == 0 && (cn & 3) == 0 &&
      (gamma == nullptr || ((reinterpret_cast<uintptr_t>(gamma + off) & 15) == 0 && off + cn <= n_gamma))) {
    for (long long i = threadIdx.x; i < (cn >> 2); i += blockDim.x) {
      float4 v = __ldg(reinterpret_cast<const float4*>(g) + i);
      v.x /= rms; v.y /= rms; v.z /= rms; v.w /= rms;
      if (gamma != nullptr) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(gamma + off) + i);
        v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
      }
      reinterpret_cast<float4*>(o)[i] = v;
    }
  } else {
    for (long long i = threadIdx.x; i < cn; i += blockDim.x) {
      float v = __ldg(g + i) / rms;
      if (gamma != nullptr && off + i < n_gamma) v *= __ldg(gamma + off + i);
      o[i] = v;
    }
  }
}

// ---- softmax family --------------------------------------------------------------------------
__global__ void softmax_row_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int len, int log_softmax) {
  extern __shared__ __align__(16) float srow[];
  __shared__ float red[33];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = row * len;
    __syncthreads();
    stage_and_sum(x + base, srow, len);
    __syncthreads();
    float m = -INFINITY;
    for (int i = threadIdx.x; i < len; i += blockDim.x) m = fmaxf(m, srow[i]);
    m = block_max(m, red);
    float acc = 0.0f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      const float e = expf(srow[i] - m);
      acc += e;
      if (!log_softmax) srow[i] = e;
    }
    const float sum = block_sum(acc, red);
    if (log_softmax) {
      const float ld = logf(sum);
      for (int i = threadIdx.x; i < len; i += blockDim.x) y[base + i] = (srow[i] - m) - ld;
    } else {
      const float inv = 1.0f / sum;
      for (int i = threadIdx.x; i < len; i += blockDim.x) y[base + i] = srow[i] * inv;
    }
  }
}

// pass 1: per chunk (max, sum of exp(x - max))
__global__ void softmax_chunk_stats_kernel(const float* __restrict__ x, float* __restrict__ part, long long len, int chunks,
                                           int chunk_len) {
  extern __shared__ __align__(16) float sch[];
  __shared__ float red[33];
  const long long row = blockIdx.y;
  const long long off = static_cast<long long>(blockIdx.x) * chunk_len;
  const long long n = min(static_cast<long long>(chunk_len), len - off);
  stage_and_sum(x + row * len + off, sch, n);
  __syncthreads();
  float m = -INFINITY;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, sch[i]);
  m = block_max(m, red);
  float acc = 0.0f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) acc += expf(sch[i] - m);
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) {
    part[(row * chunks + blockIdx.x) * 2] = m;
    part[(row * chunks + blockIdx.x) * 2 + 1] = s;
  }
}

__global__ void softmax_chunk_apply_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ part,
                                           long long len, int chunks, int chunk_len, int log_softmax) {
  const long long row = blockIdx.y;
  float m = -INFINITY;
  for (int j = 0; j < chunks; ++j) m = fmaxf(m, part[(row * chunks + j) * 2]);
  float sum = 0.0f;
  for (int j = 0; j < chunks; ++j) sum += part[(row * chunks + j) * 2 + 1] * expf(part[(row * chunks + j) * 2] - m);
  const float inv = 1.0f / sum, ld = logf(sum);
  const long long off = static_cast<long long>(blockIdx.x) * chunk_len;
  const long long cn = min(static_cast<long long>(chunk_len), len - off);
  const float* g = x + row * len + off;
  float* o = y + row * len + off;
  for (long long i = threadIdx.x; i < cn; i += blockDim.x) {
    const float v = __ldg(g + i);
    o[i] = log_softmax ? ((v - m) - ld) : expf(v - m) * inv;
  }
}

// ---- scratch for the chunk kernels -------------------------------------------------------------
constexpr size_t NORM_SCRATCH_BYTES = 8u << 20;
float* g_norm_scratch = nullptr;

int norm_scratch(float** out) {
  if (!g_norm_scratch) MB_TRY(dev_alloc(reinterpret_cast<void**>(&g_norm_scratch), NORM_SCRATCH_BYTES, "norm_scratch"));
  *out = g_norm_scratch;
  return MIMIR_B200_OK;
}

int threads_for(long long len) { return len <= 1024 ? 128 : (len <= 4096 ? 256 : 512); }

int grid_rows(long long rows) {
  const long long cap = static_cast<long long>(ctx().sm_count) * 8;
  return static_cast<int>(rows < cap ? rows : cap);
}

int meanvar_dispatch(const float* x, float* y, long long rows, long long len, float eps, const Affine& a, cudaStream_t st) {
  if (rows <= 0 || len <= 0) return fail(MIMIR_B200_E_INVALID, "norm: empty input");
  if (len <= ROW_CACHE_FLOATS) {
    static bool attr = false;
    if (!attr) {
      MB_CUDA(cudaFuncSetAttribute(meanvar_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ROW_CACHE_FLOATS * 4));
      attr = true;
    }
    meanvar_row_kernel<<<grid_rows(rows), threads_for(len), static_cast<size_t>(len) * 4, st>>>(x, y, rows, static_cast<int>(len), eps, a);
    MB_CUDA(cudaGetLastError());
    count_launch();
    return MIMIR_B200_OK;
  }
  const int chunks = static_cast<int>((len + CHUNK - 1) / CHUNK);
  if (static_cast<size_t>(rows) * chunks * 3 * sizeof(float) > NORM_SCRATCH_BYTES || rows > 65535)
    return fail(MIMIR_B200_E_UNSUPPORTED, "norm: %lld rows of %lld exceed the partial-statistics scratch", rows, len);
  float* part;
  MB_TRY(norm_scratch(&part));
  dim3 grid(chunks, static_cast<unsigned>(rows));
  meanvar_chunk_stats_kernel<<<grid, 256, CHUNK * 4, st>>>(x, part, len, chunks, CHUNK);
  MB_CUDA(cudaGetLastError());
  meanvar_chunk_apply_kernel<<<grid, 256, 0, st>>>(x, y, part, len, chunks, CHUNK, eps, a);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}

}  // namespace

int launch_layernorm(const float* x, const float* gamma, const float* beta, float* y, int64_t rows, int64_t n, float eps,
                     cudaStream_t st) {
  Affine a{gamma, gamma ? beta : nullptr, 0, 1, 1, 1, -1, nullptr};
  return meanvar_dispatch(x, y, rows, n, eps, a, st);
}

int launch_groupnorm(const float* x, const float* gamma, const float* beta, float* y, int batch, int ch, int hw, int groups,
                     float eps, int act, const float* residual, cudaStream_t st) {
  if (groups <= 0 || ch % groups != 0) return fail(MIMIR_B200_E_INVALID, "GroupNorm: channels must be divisible by num_groups");
  const int cpg = ch / groups;
  Affine a{gamma, gamma ? beta : nullptr, 1, groups, cpg, hw, act, residual};
  return meanvar_dispatch(x, y, static_cast<long long>(batch) * groups, static_cast<long long>(cpg) * hw, eps, a, st);
}

int launch_rmsnorm(const float* x, const float* gamma, int64_t n_gamma, float* y, int batch, int64_t n, float eps,
                   cudaStream_t st) {
  if (batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "RMSNorm: empty input");
  if (n <= ROW_CACHE_FLOATS) {
    static bool attr = false;
    if (!attr) {
      MB_CUDA(cudaFuncSetAttribute(rms_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ROW_CACHE_FLOATS * 4));
      attr = true;
    }
    rms_row_kernel<<<grid_rows(batch), threads_for(n), static_cast<size_t>(n) * 4, st>>>(x, gamma, n_gamma, y, batch, static_cast<int>(n), eps);
    MB_CUDA(cudaGetLastError());
    count_launch();
    return MIMIR_B200_OK;
  }
  const int chunks = static_cast<int>((n + CHUNK - 1) / CHUNK);
  if (static_cast<size_t>(batch) * chunks * sizeof(float) > NORM_SCRATCH_BYTES || batch > 65535)
    return fail(MIMIR_B200_E_UNSUPPORTED, "RMSNorm: input exceeds the partial-statistics scratch");
  float* part;
  MB_TRY(norm_scratch(&part));
  dim3 grid(chunks, static_cast<unsigned>(batch));
  rms_chunk_stats_kernel<<<grid, 256, 0, st>>>(x, part, n, chunks, CHUNK);
  MB_CUDA(cudaGetLastError());
  rms_chunk_apply_kernel<<<grid, 256, 0, st>>>(x, gamma, n_gamma, y, part, n, chunks, CHUNK, eps);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}

int launch_softmax(const float* x, float* y, int batch, int64_t n, int log_softmax, cudaStream_t st) {
  if (batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "Softmax: empty input");
  if (n <= ROW_CACHE_FLOATS) {
    static bool attr = false;
    if (!attr) {
      MB_CUDA(cudaFuncSetAttribute(softmax_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ROW_CACHE_FLOATS * 4));
      attr = true;
    }
    softmax_row_kernel<<<grid_rows(batch), threads_for(n), static_cast<size_t>(n) * 4, st>>>(x, y, batch, static_cast<int>(n), log_softmax);
    MB_CUDA(cudaGetLastError());
    count_launch();
    return MIMIR_B200_OK;
  }
  const int chunks = static_cast<int>((n + CHUNK - 1) / CHUNK);
  if (static_cast<size_t>(batch) * chunks * 2 * sizeof(float) > NORM_SCRATCH_BYTES || batch > 65535)
    return fail(MIMIR_B200_E_UNSUPPORTED, "Softmax: input exceeds the partial-statistics scratch");
  float* part;
  MB_TRY(norm_scratch(&part));
  dim3 grid(chunks, static_cast<unsigned>(batch));
  softmax_chunk_stats_kernel<<<grid, 256, CHUNK * 4, st>>>(x, part, n, chunks, CHUNK);
  MB_CUDA(cudaGetLastError());
  softmax_chunk_apply_kernel<<<grid, 256, 0, st>>>(x, y, part, n, chunks, CHUNK, log_softmax);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}


// ---------------------------------------------------------------------------------------------
// RMSNorm for callers that must not allocate
// ---------------------------------------------------------------------------------------------
// The chunked RMSNorm above keeps its per-chunk partial sums in a buffer obtained from cudaMalloc.
// Some callers cannot afford that: code running between the launches of a latency-critical
// serving loop (cudaMalloc synchronises the device), code that has handed all free device memory
// to its own pool, and plugins whose host forbids them to allocate.  For them the same two kernels
// run with the partial sums in this fixed array instead.  Every GPU that loads the library carries
// these 64 KB until the process exits.
namespace {

constexpr int NOALLOC_MAX_PARTIALS = 16384;  // floats; batch * ceil(n / 8192) must not exceed it
static __device__ __align__(256) float g_rms_noalloc_scratch[NOALLOC_MAX_PARTIALS];

constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {};  // device address of the array, per device

// `g_rms_noalloc_scratch` in host code is only a handle for the runtime, not something a kernel may
// dereference; the address kernels can use comes from cudaGetSymbolAddress, asked once per device
// while that device is current.
int noalloc_scratch_for_current_device(float** out) {
  int dev = -1;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fail(MIMIR_B200_E_UNSUPPORTED, "rmsnorm_noalloc: device index %d not supported", dev);
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_rms_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(MIMIR_B200_E_CUDA, "rmsnorm_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    g_noalloc_addr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_addr[dev];
  return MIMIR_B200_OK;
}

}  // namespace
}  // namespace mb

extern "C" int mimir_b200_dev_rmsnorm_noalloc(const float* x, const float* gamma, long long n_gamma, float* y, int batch,
                                              long long n, float eps, void* stream) {
  using namespace mb;
  if (!x || !y || batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "rmsnorm_noalloc: empty input");
  const long long chunks = (n + CHUNK - 1) / CHUNK;
  if (batch > 65535 || chunks * batch > NOALLOC_MAX_PARTIALS)
    return fail(MIMIR_B200_E_INVALID,
                "rmsnorm_noalloc: batch %d x %lld elements needs %lld partial sums, the fixed scratch holds %d "
                "(batch * ceil(n / %d) <= %d, batch <= 65535)",
                batch, n, chunks * batch, NOALLOC_MAX_PARTIALS, CHUNK, NOALLOC_MAX_PARTIALS);
  float* part = nullptr;
  MB_TRY(noalloc_scratch_for_current_device(&part));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float* g = (gamma && n_gamma > 0) ? gamma : nullptr;
  dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(batch));
  // every partial that pass 2 reads is written by pass 1 of the same call: nothing has to be cleared
  rms_chunk_stats_kernel<<<grid, 256, 0, st>>>(x, part, n, static_cast<int>(chunks), CHUNK);
  MB_CUDA(cudaGetLastError());
  rms_chunk_apply_kernel<<<grid, 256, 0, st>>>(x, g, g ? n_gamma : 0, y, part, n, static_cast<int>(chunks), CHUNK, eps);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}
