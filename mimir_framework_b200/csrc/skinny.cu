// skinny.cu — Linear for a handful of rows (m <= 16): a weight-streaming kernel, HBM-bound.
// Replaces LayerOps::linear_forward's vector mode (LayerOps.hpp:81-110) applied to a small batch:
// y[r, o] = sum_k x[r, k] * W[o, k] (+ b[o]), exact fp32 FMA arithmetic (no operand rounding).
//
// The registry transformer runs its MLP over the flattened sequence (in = 32768, out = 1024 and
// back), so with batch 8 each layer reads a 134 MB weight matrix for 8 rows: tensor cores have
// nothing to do; the job is to read W exactly once at full HBM rate.
//
// Layout of the work: grid = (out tiles of 64) x (K slices of 1024).  A CTA stages its x slice
// [m][1024] in shared memory once.  Each warp owns 8 output rows of W; 4 lanes share one W row and
// read 64 contiguous bytes of it per step (128-bit loads), x comes from shared memory as broadcast
// reads.  Partial sums over K slices go to a small global scratch and are reduced in a fixed order
// by a second kernel (deterministic, no atomics).
#include "common.h"

namespace mb {
namespace {

constexpr int SK_TILE_N = 64;
constexpr int SK_SLICE = 1024;
constexpr int SK_THREADS = 256;

__device__ __forceinline__ float sk_act(float v, int act) {
  switch (act) {
    case MIMIR_B200_ELT_GELU: {
      const float c = 0.7978845608f;
      return v * (0.5f * (1.0f + tanhf(c * (v + 0.044715f * v * v * v))));
    }
    case MIMIR_B200_ELT_SILU: return v * (1.0f / (1.0f + expf(-v)));
    case MIMIR_B200_ELT_RELU: return fmaxf(0.0f, v);
    case MIMIR_B200_ELT_TANH: return tanhf(v);
    case MIMIR_B200_ELT_SIGMOID: return 1.0f / (1.0f + expf(-v));
    default: return v;
  }
}

template <int MT>
__global__ void __launch_bounds__(SK_THREADS)
skinny_partial_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ part, int m, int k,
                      int n, int kslices) {
  extern __shared__ __align__(16) float xs_raw[];
  float (*xs)[SK_SLICE] = reinterpret_cast<float (*)[SK_SLICE]>(xs_raw);
  const int o_tile = blockIdx.x * SK_TILE_N;
  const int ks = blockIdx.y;
  const int k0 = ks * SK_SLICE;
  const int klen = min(SK_SLICE, k - k0);
  for (int i = threadIdx.x; i < MT * SK_SLICE; i += SK_THREADS) {
    const int r = i / SK_SLICE, c = i - r * SK_SLICE;
    xs[r][c] = (r < m && c < klen) ? __ldg(x + static_cast<long long>(r) * k + k0 + c) : 0.0f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane & 3;                      // position of this lane inside its group of 4
  const int o = o_tile + warp * 8 + (lane >> 2);
  float acc[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r] = 0.0f;
  if (o < n) {
    const float* wrow = w + static_cast<long long>(o) * k + k0;
    const bool vec = ((reinterpret_cast<uintptr_t>(wrow) & 15) == 0) && ((klen & 15) == 0);
    if (vec) {
#pragma unroll 4
      for (int c = q * 4; c < klen; c += 16) {
        const float4 wv = __ldg(reinterpret_cast<const float4*>(wrow + c));
#pragma unroll
        for (int r = 0; r < MT; ++r) {
          const float4 xv = *reinterpret_cast<const float4*>(&xs[r][c]);
          acc[r] = fmaf(wv.x, xv.x, acc[r]);
          acc[r] = fmaf(wv.y, xv.y, acc[r]);
          acc[r] = fmaf(wv.z, xv.z, acc[r]);
          acc[r] = fmaf(wv.w, xv.w, acc[r]);
        }
      }
    } else {
      for (int c = q; c < klen; c += 4) {
        const float wv = __ldg(wrow + c);
#pragma unroll
        for (int r = 0; r < MT; ++r) acc[r] = fmaf(wv, xs[r][c], acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 1);
    acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 2);
  }
  if (q == 0 && o < n) {
#pragma unroll
    for (int r = 0; r < MT; ++r)
      if (r < m) part[(static_cast<long long>(ks) * m + r) * n + o] = acc[r];
  }
}

__global__ void skinny_finish_kernel(const float* __restrict__ part, const float* __restrict__ bias, float* __restrict__ y,
                                     int m, int n, int kslices, int act) {
  const long long total = static_cast<long long>(m) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(i % n);
    float s = 0.0f;
    for (int ks = 0; ks < kslices; ++ks) s += part[static_cast<long long>(ks) * total + i];
    if (bias != nullptr) s += __ldg(bias + o);
    y[i] = sk_act(s, act);
  }
}

}  // namespace

size_t skinny_scratch_bytes(int m, int k, int n) {
  const size_t kslices = static_cast<size_t>((k + SK_SLICE - 1) / SK_SLICE);
  return kslices * static_cast<size_t>(m) * static_cast<size_t>(n) * sizeof(float);
}

int launch_skinny_linear(const float* x, const float* w, const float* bias, float* y, int m, int k, int n, int activation,
                         float* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (m <= 0 || m > 16 || k <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "skinny linear: m must be in 1..16");
  if (scratch == nullptr || scratch_bytes < skinny_scratch_bytes(m, k, n))
    return fail(MIMIR_B200_E_INVALID, "skinny linear: scratch too small");
  const int kslices = (k + SK_SLICE - 1) / SK_SLICE;
  dim3 grid((n + SK_TILE_N - 1) / SK_TILE_N, kslices);
  if (m <= 4) skinny_partial_kernel<4><<<grid, SK_THREADS, 4 * SK_SLICE * 4, st>>>(x, w, scratch, m, k, n, kslices);
  else if (m <= 8) skinny_partial_kernel<8><<<grid, SK_THREADS, 8 * SK_SLICE * 4, st>>>(x, w, scratch, m, k, n, kslices);
  else {
    static bool attr = false;
    if (!attr) {
      MB_CUDA(cudaFuncSetAttribute(skinny_partial_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * SK_SLICE * 4));
      attr = true;
    }
    skinny_partial_kernel<16><<<grid, SK_THREADS, 16 * SK_SLICE * 4, st>>>(x, w, scratch, m, k, n, kslices);
  }
  MB_CUDA(cudaGetLastError());
  const long long total = static_cast<long long>(m) * n;
  int fb = static_cast<int>((total + 255) / 256);
  if (fb > ctx().sm_count * 8) fb = ctx().sm_count * 8;
  skinny_finish_kernel<<<fb, 256, 0, st>>>(scratch, bias, y, m, n, kslices, activation);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}

}  // namespace mb
