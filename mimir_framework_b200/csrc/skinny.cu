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
// every item drains the asynchronous copies, 0.34 -> 0.52 ms on the registry transformer.  Reading the next step's W vectors
// out of the ring while the current step's FMAs run, with a fifth stage, was measured too: no change, 0.260 -> 0.262 ms.)  Unaligned operands or K % 4 != 0 take a
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

// Which CTA of a grid of `grid` owns item `i` when `items` items are dealt out as contiguous, balanced ranges (the first
// items % grid CTAs take one more), and the range of CTA `b`.  Used by the streaming kernel and by the finishing kernel alike.
struct ItemSplit {
  int base, rem;  // items / grid, items % grid
  __host__ __device__ ItemSplit(int items, int grid) : base(items / grid), rem(items % grid) {}
  __host__ __device__ int first(int b) const { return b * base + (b < rem ? b : rem); }
  __host__ __device__ int count(int b) const { return base + (b < rem ? 1 : 0); }
  __host__ __device__ int owner(int i) const {
    const int big = rem * (base + 1);
    return i < big ? i / (base + 1) : rem + (i - big) / base;
  }
};

// Persistent form for 16-byte aligned operands with k % 4 == 0.  Shared memory: x double buffer
// [2][MT][SK_SLICE], then the rings [warp][SK_STAGES][WR][SK_STEP].
// A CTA owns a CONTIGUOUS range of items (item = tile * kslices + ks): consecutive items are consecutive K slices of the same
// output tile, so their partial sums stay in the accumulators and the exchange between lanes and the write of the partials
// happen once per (CTA, tile) instead of once per item.  Partial p of a tile is the one of the p-th CTA that touched it, in K
// order: part[(p * m + r) * n + o].
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
  const ItemSplit split(items, static_cast<int>(gridDim.x));
  const int my_first = split.first(static_cast<int>(blockIdx.x)), my_items = split.count(static_cast<int>(blockIdx.x));
  const int total_steps = my_items * SK_STEPS;
  const long long kk = k;

  // Copy group of this CTA's step g (item g / SK_STEPS, step g % SK_STEPS): this warp's WR rows of W, and with the first step
  // of an item every thread's share of that item's x slice.  The groups are issued in order, so (tile, ks, step) of the next
  // group and the address of its first row advance incrementally.
  int ig = 0, i_st = 0, i_j = 0;
  int i_tile = my_first / kslices, i_ks = my_first - i_tile * kslices;
  auto issue = [&]() {
    if (ig < total_steps) {
      const int c = i_ks * SK_SLICE + i_st * SK_STEP + lane * 4;
      const int o0 = (i_tile * SK_WARPS + warp) * WR;
      const float* src = w + static_cast<long long>(o0) * kk + c;
      float* dst = ring + (ig % SK_STAGES) * (WR * SK_STEP) + lane * 4;
      const bool col_ok = c < k;
#pragma unroll
      for (int jj = 0; jj < WR; ++jj) {
        const bool ok = col_ok && (o0 + jj < n);
        cp_async16_zfill(dst + jj * SK_STEP, ok ? src : w, ok);
        src += kk;
      }
      if (i_st == 0) {
        float* xd = xs + (i_j & 1) * (MT * SK_SLICE);
        for (int i = threadIdx.x; i < MT * (SK_SLICE / 4); i += SK_THREADS) {
          const int r = i / (SK_SLICE / 4), cc = (i - r * (SK_SLICE / 4)) << 2;
          const int kc = i_ks * SK_SLICE + cc;
          const bool ok = (r < m) && (kc < k);
          cp_async16_zfill(xd + r * SK_SLICE + cc, ok ? (x + r * kk + kc) : x, ok);
        }
      }
      if (++i_st == SK_STEPS) {
        i_st = 0;
        ++i_j;
        if (++i_ks == kslices) { i_ks = 0; ++i_tile; }
      }
    }
    ++ig;
    cp_async_commit();  // one group per step, empty past the end, so that the wait count stays fixed
  };
#pragma unroll
  for (int i = 0; i < SK_STAGES - 1; ++i) issue();

  float acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.0f;
  int tile = my_first / kslices, ks = my_first - tile * kslices;
  for (int j = 0; j < my_items; ++j) {
    const float* xj = xs + (j & 1) * (MT * SK_SLICE);
#pragma unroll
    for (int st = 0; st < SK_STEPS; ++st) {
      const int g = j * SK_STEPS + st;
      if (st == 0) {
        // the group of step g carries this item's x slice: wait for it, then let every thread's share become visible
        // (the next group may overwrite the x buffer of item j - 1: issued after the barrier)
        cp_async_wait<SK_STAGES - 2>();
        __syncthreads();
        issue();
      } else {
        issue();
        cp_async_wait<SK_STAGES - 1>();
      }
      const float* src = ring + (g % SK_STAGES) * (WR * SK_STEP) + lane * 4;
      float4 wv[WR];
#pragma unroll
      for (int jj = 0; jj < WR; ++jj) wv[jj] = *reinterpret_cast<const float4*>(src + jj * SK_STEP);
      sk_fma_step<MT, WR>(acc, wv, xj, st * SK_STEP + lane * 4);
    }
    const bool tile_ends = (ks + 1 == kslices) || (j + 1 == my_items);
    if (tile_ends) {
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
      // this CTA's place among the CTAs that touch the tile (they hold consecutive K ranges of it)
      const int p = static_cast<int>(blockIdx.x) - split.owner(tile * kslices);
      const int o0 = (tile * SK_WARPS + warp) * WR;
#pragma unroll
      for (int t = 0; t < PER; ++t) {
        const int idx = lane * PER + t, jj = idx / MT, r = idx - jj * MT;
        if (r < m && o0 + jj < n) part[(static_cast<long long>(p) * m + r) * n + o0 + jj] = acc[t];
      }
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = 0.0f;
    }
    if (++ks == kslices) { ks = 0; ++tile; }
  }
  cp_async_wait<0>();
}

// y = sum of a tile's partials in K order (+ bias, activation, folded residual).  grid > 0: the partials come from the
// streaming kernel launched with that many CTAs (one partial per CTA that touched the tile); grid == 0: one partial per K slice.
__global__ void skinny_finish_kernel(const float* __restrict__ part, const float* __restrict__ bias, const float* __restrict__ residual,
                                     float* __restrict__ y, int m, int n, int kslices, int act, int grid, int items, int tile_cols) {
  const long long total = static_cast<long long>(m) * n;
  const ItemSplit split(grid > 0 ? items : 1, grid > 0 ? grid : 1);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(i % n);
    int np = kslices;
    if (grid > 0) {
      const int tile = o / tile_cols;
      np = split.owner((tile + 1) * kslices - 1) - split.owner(tile * kslices) + 1;
    }
    // the partials are added in K order; eight loads are issued before the first add so that a long chain does not pay
    // the memory latency once per partial
    float s = 0.0f;
    int ks = 0;
    for (; ks + 8 <= np; ks += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcs(part + static_cast<long long>(ks + u) * total + i);
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
    for (; ks < np; ++ks) s += __ldcs(part + static_cast<long long>(ks) * total + i);
    if (bias != nullptr) s += __ldg(bias + o);
    s = sk_act(s, act);
    if (residual != nullptr) s += __ldg(residual + i);  // a residual Add folded into this layer
    y[i] = s;
  }
}

template <int MT, int WR>
int launch_partial(const float* x, const float* w, float* scratch, int m, int k, int n, cudaStream_t st, int* stream_grid, int* stream_items,
                   int* tile_cols) {
  const int tiles = (n + SK_WARPS * WR - 1) / (SK_WARPS * WR), kslices = (k + SK_SLICE - 1) / SK_SLICE;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0 && (k & 3) == 0;
  const char* plain = getenv("MIMIR_B200_SKINNY_PLAIN");
  *stream_grid = 0;
  *stream_items = 0;
  *tile_cols = SK_WARPS * WR;
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
    *stream_grid = grid;
    *stream_items = items;
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
  int sgrid = 0, sitems = 0, tile_cols = 0;
  if (m <= 4) MB_TRY((launch_partial<4, 8>(x, w, scratch, m, k, n, st, &sgrid, &sitems, &tile_cols)));
  else if (m <= 8) MB_TRY((launch_partial<8, 8>(x, w, scratch, m, k, n, st, &sgrid, &sitems, &tile_cols)));
  else MB_TRY((launch_partial<16, 4>(x, w, scratch, m, k, n, st, &sgrid, &sitems, &tile_cols)));
  const long long total = static_cast<long long>(m) * n;
  int fb = static_cast<int>((total + 255) / 256);
  if (fb > ctx().sm_count * 8) fb = ctx().sm_count * 8;
  skinny_finish_kernel<<<fb, 256, 0, st>>>(scratch, bias, residual, y, m, n, (k + SK_SLICE - 1) / SK_SLICE, activation, sgrid, sitems,
                                           tile_cols);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}

}  // namespace mb
