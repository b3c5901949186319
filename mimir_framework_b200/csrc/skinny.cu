// skinny.cu — Linear for a handful of rows (m <= 16): a weight-streaming kernel, HBM-bound.
// Replaces LayerOps::linear_forward's vector mode (LayerOps.hpp:81-110) applied to a small batch:
// y[r, o] = sum_k x[r, k] * W[o, k] (+ b[o]), exact fp32 FMA arithmetic (no operand rounding).
//
// The registry transformer runs its MLP over the flattened sequence (in = 32768, out = 1024 and
// back), so with batch 8 each layer reads a 134 MB weight matrix for 8 rows: tensor cores have
// nothing to do; the job is to read W exactly once at full HBM rate.
//
// Layout of the work: an item is (tile of 8 x WR output rows) x (K slice of 512); one persistent CTA per SM
// takes items round-robin, so every SM streams the same number of bytes whatever the shape.  A warp owns WR
// rows of W; per step its 32 lanes cover 128 consecutive k (16 bytes per lane and row, 512 contiguous bytes
// per row and warp).  W never passes through registers on its way in: every warp runs its own ring of
// SK_STAGES shared-memory stages filled with asynchronous 16-byte copies (cp.async, zero-filled past the
// end of a row or of W) that run three steps ahead, across item boundaries, so ~96 KB per SM are in
// flight all the time; the x slice of the next item rides in the same copy groups into a double buffer.
// Each x vector read from shared memory is reused for all WR rows.  Every lane keeps WR x m partial sums; a
// recursive-halving exchange (N/2 + N/4 + ... shuffles instead of 5 N) leaves each lane with the finished
// sums of N / 32 outputs.  Partial sums over K slices go to a small global scratch and are reduced in a
// fixed order by a second kernel (deterministic, no atomics), which also adds bias, activation and a folded residual.
// (Letting the CTA that delivers a tile's last slice do that sum was measured and dropped: the fence it needs after
// every item drains the asynchronous copies, 0.34 -> 0.52 ms on the registry transformer.)  Unaligned operands or K % 4 != 0 take a
// plain-load kernel with the same arithmetic.
#include <cstdlib>

#include "common.h"

namespace mb {
namespace {

constexpr int SK_THREADS = 256;
constexpr int SK_WARPS = SK_THREADS / 32;
constexpr int SK_STEP = 128;   // k covered by one warp step
constexpr int SK_SLICE = 512;  // k covered by one CTA

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

template <int MT, int WR>
__device__ __forceinline__ void sk_fma_step(float (&acc)[MT * WR], const float4 (&wv)[WR], const float* __restrict__ xs, int c) {
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    const float4 xv = *reinterpret_cast<const float4*>(xs + r * SK_SLICE + c);
#pragma unroll
    for (int j = 0; j < WR; ++j) {
      float a = acc[j * MT + r];
      a = fmaf(wv[j].x, xv.x, a);
      a = fmaf(wv[j].y, xv.y, a);
      a = fmaf(wv[j].z, xv.z, a);
      a = fmaf(wv[j].w, xv.w, a);
      acc[j * MT + r] = a;
    }
  }
}

// MT = rows of x held (m <= MT), WR = rows of W per warp.
template <int MT, int WR>
__global__ void __launch_bounds__(SK_THREADS, 2)
skinny_partial_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ part, int m, int k, int n) {
  constexpr int N = MT * WR;   // partial sums per lane
  constexpr int PER = N / 32;  // finished sums per lane after the exchange
  static_assert(N % 32 == 0 && PER >= 1, "WR x MT must be a multiple of the warp size");
  extern __shared__ __align__(16) float xs[];  // [MT][SK_SLICE]
  const int ks = blockIdx.y;
  const int k0 = ks * SK_SLICE;
  const int klen = min(SK_SLICE, k - k0);
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 && (k & 3) == 0;
  // stage x (zero past m and past the end of K so that the main loop needs no row masks)
  for (int i = threadIdx.x; i < MT * (SK_SLICE / 4); i += SK_THREADS) {
    const int r = i / (SK_SLICE / 4), c = (i - r * (SK_SLICE / 4)) << 2;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < m) {
      const float* src = x + static_cast<long long>(r) * k + k0 + c;
      if (vec && c + 3 < klen) v = __ldg(reinterpret_cast<const float4*>(src));
      else {
        if (c + 0 < klen) v.x = __ldg(src + 0);
        if (c + 1 < klen) v.y = __ldg(src + 1);
        if (c + 2 < klen) v.z = __ldg(src + 2);
        if (c + 3 < klen) v.w = __ldg(src + 3);
      }
    }
    *reinterpret_cast<float4*>(xs + r * SK_SLICE + c) = v;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int o0 = (blockIdx.x * SK_WARPS + warp) * WR;
  float acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.0f;
  const float* wbase = w + static_cast<long long>(o0) * k + k0 + lane * 4;
  if (vec && klen == SK_SLICE && o0 + WR <= n) {
    // full tile: no masks, all loads of the four steps are independent of the arithmetic
#pragma unroll
    for (int st = 0; st < SK_SLICE / SK_STEP; ++st) {
      float4 wv[WR];
#pragma unroll
      for (int j = 0; j < WR; ++j)
        wv[j] = __ldcs(reinterpret_cast<const float4*>(wbase + static_cast<long long>(j) * k + st * SK_STEP));  // read once
      sk_fma_step<MT, WR>(acc, wv, xs, st * SK_STEP + lane * 4);
    }
  } else {
    for (int c = lane * 4; c < klen; c += SK_STEP) {
      float4 wv[WR];
#pragma unroll
      for (int j = 0; j < WR; ++j) {
        wv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (o0 + j < n) {
          const float* src = wbase + static_cast<long long>(j) * k + (c - lane * 4);
          if (vec && c + 3 < klen) wv[j] = __ldcs(reinterpret_cast<const float4*>(src));
          else {
            if (c + 0 < klen) wv[j].x = __ldg(src + 0);
            if (c + 1 < klen) wv[j].y = __ldg(src + 1);
            if (c + 2 < klen) wv[j].z = __ldg(src + 2);
            if (c + 3 < klen) wv[j].w = __ldg(src + 3);
          }
        }
      }
      sk_fma_step<MT, WR>(acc, wv, xs, c);
    }
  }
  // recursive halving: after the round with partner distance `mask` a lane keeps the half of its
  // values selected by that lane bit; it ends with acc[0..PER) = sums of indices lane * PER + t
#pragma unroll
  for (int half = N / 2, mask = 16; mask >= 1; half >>= 1, mask >>= 1) {
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? acc[i] : acc[i + half];
      const float keep = upper ? acc[i + half] : acc[i];
      acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
  }
#pragma unroll
  for (int t = 0; t < PER; ++t) {
    const int idx = lane * PER + t, j = idx / MT, r = idx - j * MT;
    if (r < m && o0 + j < n) part[(static_cast<long long>(ks) * m + r) * n + o0 + j] = acc[t];
  }
}

constexpr int SK_STAGES = 4;
constexpr int SK_STEPS = SK_SLICE / SK_STEP;  // steps per item

__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  const int bytes = valid ? 16 : 0;  // src-size 0: the 16 destination bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Persistent form for 16-byte aligned operands with k % 4 == 0.  Shared memory: x double buffer
// [2][MT][SK_SLICE], then the rings [warp][SK_STAGES][WR][SK_STEP].
template <int MT, int WR>
__global__ void __launch_bounds__(SK_THREADS, 1)
skinny_stream_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ part, int m, int k, int n,
                     int kslices, int items) {
  constexpr int N = MT * WR;
  constexpr int PER = N / 32;
  static_assert(N % 32 == 0 && PER >= 1, "WR x MT must be a multiple of the warp size");
  extern __shared__ __align__(16) float sk_smem[];
  float* xs = sk_smem;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* ring = sk_smem + 2 * MT * SK_SLICE + warp * (SK_STAGES * WR * SK_STEP);
  const int my_items = (items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int total_steps = my_items * SK_STEPS;

  // copy group of global step g (= this CTA's item g / SK_STEPS, step g % SK_STEPS): this warp's WR rows, and with
  // the first step of an item every thread's share of that item's x slice
  auto issue = [&](int g) {
    if (g < total_steps) {
      const int j = g / SK_STEPS, st = g - j * SK_STEPS;
      const int item = blockIdx.x + j * gridDim.x;
      const int tile = item / kslices, ks = item - tile * kslices;
      const int c = ks * SK_SLICE + st * SK_STEP + lane * 4;
      const long long o0 = (static_cast<long long>(tile) * SK_WARPS + warp) * WR;
      float* dst = ring + (g % SK_STAGES) * (WR * SK_STEP) + lane * 4;
#pragma unroll
      for (int jj = 0; jj < WR; ++jj) {
        const bool ok = (o0 + jj < n) && (c < k);
        cp_async16_zfill(dst + jj * SK_STEP, ok ? (w + (o0 + jj) * k + c) : w, ok);
      }
      if (st == 0) {
        float* xd = xs + (j & 1) * (MT * SK_SLICE);
        for (int i = threadIdx.x; i < MT * (SK_SLICE / 4); i += SK_THREADS) {
          const int r = i / (SK_SLICE / 4), cc = (i - r * (SK_SLICE / 4)) << 2;
          const int kc = ks * SK_SLICE + cc;
          const bool ok = (r < m) && (kc < k);
          cp_async16_zfill(xd + r * SK_SLICE + cc, ok ? (x + static_cast<long long>(r) * k + kc) : x, ok);
        }
      }
    }
    cp_async_commit();  // one group per step, empty past the end, so that the wait count stays fixed
  };
#pragma unroll
  for (int i = 0; i < SK_STAGES - 1; ++i) issue(i);

  float acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.0f;
  for (int j = 0; j < my_items; ++j) {
    const int item = blockIdx.x + j * gridDim.x;
    const int tile = item / kslices, ks = item - tile * kslices;
    const float* xj = xs + (j & 1) * (MT * SK_SLICE);
#pragma unroll
    for (int st = 0; st < SK_STEPS; ++st) {
      const int g = j * SK_STEPS + st;
      if (st == 1) issue(g + SK_STAGES - 1);  // (after the item's barrier: it may overwrite the x buffer of item j - 1)
      else if (st != 0) issue(g + SK_STAGES - 1);
      if (st == 0) {
        // the group of step g carries this item's x slice: wait for it, then let every thread's share become visible
        cp_async_wait<SK_STAGES - 2>();
        __syncthreads();
        issue(g + SK_STAGES - 1);
      } else {
        cp_async_wait<SK_STAGES - 1>();
      }
      const float* src = ring + (g % SK_STAGES) * (WR * SK_STEP) + lane * 4;
      float4 wv[WR];
#pragma unroll
      for (int jj = 0; jj < WR; ++jj) wv[jj] = *reinterpret_cast<const float4*>(src + jj * SK_STEP);
      sk_fma_step<MT, WR>(acc, wv, xj, st * SK_STEP + lane * 4);
    }
#pragma unroll
    for (int half = N / 2, mask = 16; mask >= 1; half >>= 1, mask >>= 1) {
      const bool upper = (lane & mask) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float send = upper ? acc[i] : acc[i + half];
        const float keep = upper ? acc[i + half] : acc[i];
        acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
      }
    }
    const long long o0 = (static_cast<long long>(tile) * SK_WARPS + warp) * WR;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      const int idx = lane * PER + t, jj = idx / MT, r = idx - jj * MT;
      if (r < m && o0 + jj < n) part[(static_cast<long long>(ks) * m + r) * n + o0 + jj] = acc[t];
    }
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = 0.0f;
  }
  cp_async_wait<0>();
}

__global__ void skinny_finish_kernel(const float* __restrict__ part, const float* __restrict__ bias, const float* __restrict__ residual,
                                     float* __restrict__ y, int m, int n, int kslices, int act) {
  const long long total = static_cast<long long>(m) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(i % n);
    // slices are added in slice order; eight loads are issued before the first add so that a long K (64 slices for
    // in_features = 32768) does not pay the memory latency once per slice
    float s = 0.0f;
    int ks = 0;
    for (; ks + 8 <= kslices; ks += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcs(part + static_cast<long long>(ks + u) * total + i);
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
    for (; ks < kslices; ++ks) s += __ldcs(part + static_cast<long long>(ks) * total + i);
    if (bias != nullptr) s += __ldg(bias + o);
    s = sk_act(s, act);
    if (residual != nullptr) s += __ldg(residual + i);  // a residual Add folded into this layer
    y[i] = s;
  }
}

template <int MT, int WR>
int launch_partial(const float* x, const float* w, float* scratch, int m, int k, int n, cudaStream_t st) {
  const int tiles = (n + SK_WARPS * WR - 1) / (SK_WARPS * WR), kslices = (k + SK_SLICE - 1) / SK_SLICE;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 && (k & 3) == 0;
  const char* plain = getenv("MIMIR_B200_SKINNY_PLAIN");
  if (vec && !(plain && plain[0] == '1') && static_cast<long long>(tiles) * kslices < (1LL << 30)) {
    constexpr int SMEM = (2 * MT * SK_SLICE + SK_WARPS * SK_STAGES * WR * SK_STEP) * 4;
    static PerDeviceOnce attr_once;
    MB_TRY(attr_once.run([&]() -> int {
      MB_CUDA(cudaFuncSetAttribute(skinny_stream_kernel<MT, WR>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
      return MIMIR_B200_OK;
    }));
    const int items = tiles * kslices;
    const int grid = items < ctx().sm_count ? items : ctx().sm_count;
    skinny_stream_kernel<MT, WR><<<grid, SK_THREADS, SMEM, st>>>(x, w, scratch, m, k, n, kslices, items);
  } else {
    constexpr int SMEM = MT * SK_SLICE * 4;
    dim3 grid(tiles, kslices);
    skinny_partial_kernel<MT, WR><<<grid, SK_THREADS, SMEM, st>>>(x, w, scratch, m, k, n);
  }
  MB_CUDA(cudaGetLastError());
  return MIMIR_B200_OK;
}

}  // namespace

size_t skinny_scratch_bytes(int m, int k, int n) {
  const size_t kslices = static_cast<size_t>((k + SK_SLICE - 1) / SK_SLICE);
  return kslices * static_cast<size_t>(m) * static_cast<size_t>(n) * sizeof(float);
}

int launch_skinny_linear(const float* x, const float* w, const float* bias, float* y, int m, int k, int n, int activation,
                         float* scratch, size_t scratch_bytes, cudaStream_t st, const float* residual) {
  if (m <= 0 || m > 16 || k <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "skinny linear: m must be in 1..16");
  if (scratch == nullptr || scratch_bytes < skinny_scratch_bytes(m, k, n))
    return fail(MIMIR_B200_E_INVALID, "skinny linear: scratch too small");
  if ((k + SK_SLICE - 1) / SK_SLICE > 65535) return fail(MIMIR_B200_E_UNSUPPORTED, "skinny linear: in_features %d too large", k);
  if (m <= 4) MB_TRY((launch_partial<4, 8>(x, w, scratch, m, k, n, st)));
  else if (m <= 8) MB_TRY((launch_partial<8, 8>(x, w, scratch, m, k, n, st)));
  else MB_TRY((launch_partial<16, 4>(x, w, scratch, m, k, n, st)));
  const long long total = static_cast<long long>(m) * n;
  int fb = static_cast<int>((total + 255) / 256);
  if (fb > ctx().sm_count * 8) fb = ctx().sm_count * 8;
  skinny_finish_kernel<<<fb, 256, 0, st>>>(scratch, bias, residual, y, m, n, (k + SK_SLICE - 1) / SK_SLICE, activation);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}

}  // namespace mb
