// norms.cu — HBM-bound row reductions: LayerNorm, GroupNorm(+SiLU, +residual), RMSNorm, Softmax.
//   LayerNorm : LayerOps::layernorm_forward  (LayerOps.hpp:264-319)  rows of n, biased variance
//   GroupNorm : LayerOps::groupnorm_forward  (LayerOps.hpp:488-550)  row = one (sample, group) slab
//   RMSNorm   : LayerOpsExt::rms_norm_forward (LayerOpsExt.hpp:345-378) row = the whole sample
//   Softmax   : LayerOps::softmax_forward    (LayerOps.hpp:325-361)  row = the whole sample
//
// Three shapes of kernel:
//   * warp-per-row (LayerNorm rows <= 1024): the row lives in registers, shuffles only;
//   * CTA-per-row streaming sweeps (at least one row per SM): first sweep from HBM, later sweeps from
//     L2, one HBM read and one HBM write per element;
//   * "chunk" kernels when there are only a few (long) rows: pass 1 reduces 8192-element chunks to
//     partial statistics in a small global scratch, pass 2 combines the partials of its row and
//     writes the result; rows are processed in groups that fit in L2 so that pass 2 reads from L2.
#include <cooperative_groups.h>

#include <map>
#include <mutex>
#include <utility>

#include "common.h"
#include "planes.cuh"
#include "sm100_ptx.cuh"


namespace mb {
namespace {

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

// Copies `len` floats global -> shared and returns this thread's partial sum.  128-bit loads, four
// in flight per thread before the first shared-memory store, so that a CTA keeps ~32 KB in flight.
__device__ __forceinline__ float stage_and_sum(const float* __restrict__ g, float* s, long long len) {
  float acc = 0.0f;
  if (((reinterpret_cast<uintptr_t>(g) & 15) == 0) && ((len & 3) == 0)) {
    const float4* g4 = reinterpret_cast<const float4*>(g);
    float4* s4 = reinterpret_cast<float4*>(s);
    const long long n4 = len >> 2;
    const long long step = blockDim.x;
    long long i = threadIdx.x;
    for (; i + 3 * step < n4; i += 4 * step) {
      const float4 a = __ldg(g4 + i), b = __ldg(g4 + i + step), c = __ldg(g4 + i + 2 * step), d = __ldg(g4 + i + 3 * step);
      s4[i] = a; s4[i + step] = b; s4[i + 2 * step] = c; s4[i + 3 * step] = d;
      acc += ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w)) + ((c.x + c.y) + (c.z + c.w)) + ((d.x + d.y) + (d.z + d.w));
    }
    for (; i < n4; i += step) {
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
    const long long gi = a.per_channel ? static_cast<long long>(static_cast<int>(row % a.groups) * a.cpg + static_cast<int>(static_cast<unsigned>(i) / static_cast<unsigned>(a.hw))) : i;
    v *= __ldg(a.gamma + gi);
    if (a.beta != nullptr) v += __ldg(a.beta + gi);
  }
  if (a.act == MIMIR_B200_ELT_SILU) v = silu(v);
  if (a.residual != nullptr) v += __ldg(a.residual + base + i);
  return v;
}

// ---- chunk kernels (mean / variance) ----------------------------------------------------------
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

// ---- chunk kernels (RMS) ---------------------------------------------------------------------
__global__ void rms_chunk_stats_kernel(const float* __restrict__ x, float* __restrict__ part, long long len, int chunks,
                                       int chunk_len) {
  __shared__ float red[33];
  const long long row = blockIdx.y;
  const long long off = static_cast<long long>(blockIdx.x) * chunk_len;
  const long long n = min(static_cast<long long>(chunk_len), len - off);
  const float* g = x + row * len + off;
  float acc = 0.0f;
  if ((reinterpret_cast<uintptr_t>(g) & 15) == 0 && (n & 3) == 0) {
    const float4* g4 = reinterpret_cast<const float4*>(g);
    const int n4 = static_cast<int>(n >> 2), step = blockDim.x;
    int i = threadIdx.x;
    for (; i + 3 * step < n4; i += 4 * step) {  // four loads in flight
      const float4 a = __ldg(g4 + i), b = __ldg(g4 + i + step), c = __ldg(g4 + i + 2 * step), d = __ldg(g4 + i + 3 * step);
      acc += ((a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w)) + ((b.x * b.x + b.y * b.y) + (b.z * b.z + b.w * b.w)) +
             ((c.x * c.x + c.y * c.y) + (c.z * c.z + c.w * c.w)) + ((d.x * d.x + d.y * d.y) + (d.z * d.z + d.w * d.w));
    }
    for (; i < n4; i += step) {
      const float4 v = __ldg(g4 + i);
      acc += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
  } else {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) acc += g[i] * g[i];
  }
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) part[row * chunks + blockIdx.x] = s;
}

// The reference sums the squares in ONE sequential fp32 chain, s = fma(x, x, s) (LayerOpsExt.hpp:353-356).
// Over a whole sample (786 432 elements in the decoder configuration) that chain loses a systematic
// 3.7e-4 of the sum, because addends far below the running sum's ulp are rounded on the sum's grid.
// The rounding error of one step depends only on the addend and on the binade of the running sum,
// so it can be reproduced in parallel: every thread replays a short stretch of the chain seeded with
// the (exact) prefix sum at its first element and accumulates the rounding errors of its steps.
// sequential result = exact sum + sum of these rounding errors.
constexpr int SEQ_PER_THREAD = 32;  // CHUNK / 256 threads

__global__ void __launch_bounds__(256) rms_seq_err_kernel(const float* __restrict__ x, const float* __restrict__ part,
                                                          double* __restrict__ seq_err, long long len, int chunks, int chunk_len) {
  __shared__ float wsum[8];
  __shared__ double werr[8];
  const long long row = blockIdx.y;
  const int c = blockIdx.x;
  const long long off = static_cast<long long>(c) * chunk_len;
  const int n = static_cast<int>(min(static_cast<long long>(chunk_len), len - off));
  const float* g = x + row * len + off;
  // this thread's 32 consecutive elements (one 128-byte line), straight into registers
  float mine[SEQ_PER_THREAD];
  const int first = threadIdx.x * SEQ_PER_THREAD;
  if (first + SEQ_PER_THREAD <= n && ((reinterpret_cast<uintptr_t>(g + first) & 15) == 0)) {
#pragma unroll
    for (int j = 0; j < SEQ_PER_THREAD; j += 4) {
      const float4 v4 = __ldg(reinterpret_cast<const float4*>(g + first + j));
      mine[j] = v4.x; mine[j + 1] = v4.y; mine[j + 2] = v4.z; mine[j + 3] = v4.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < SEQ_PER_THREAD; ++j) mine[j] = (first + j < n) ? __ldg(g + first + j) : 0.0f;
  }
  // sum of the squares before this chunk; only its binade matters, fp32 chunk sums added in double are ample
  double prefix = 0.0;
  for (int j = 0; j < c; ++j) prefix += static_cast<double>(part[row * chunks + j]);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  float local = 0.0f;
#pragma unroll
  for (int j = 0; j < SEQ_PER_THREAD; ++j) local = fmaf(mine[j], mine[j], local);
  // exclusive prefix of the per-thread sums: warp scan, then the eight warp totals
  float scan = local;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, scan, d);
    if (lane >= d) scan += t;
  }
  if (lane == 31) wsum[w] = scan;
  __syncthreads();
  float wbase = 0.0f;
  for (int k = 0; k < w; ++k) wbase += wsum[k];
  float sf = static_cast<float>(prefix + static_cast<double>(wbase + (scan - local)));  // on the chain's grid
  // replay this thread's stretch of the chain; every step's rounding error is recovered exactly with
  // error-free transformations: T = sf + v*v exactly equals s1 + e2 + e1, and nf = round(T)
  float err = 0.0f;
#pragma unroll
  for (int j = 0; j < SEQ_PER_THREAD; ++j) {
    if (first + j < n) {
      const float v = mine[j];
      const float nf = fmaf(v, v, sf);          // what the reference computes
      // (__fmul_rn / __fadd_rn are never contracted into an FMA, which would defeat the transformations)
      const float pr = __fmul_rn(v, v);
      const float e1 = fmaf(v, v, -pr);         // product error
      const float s1 = __fadd_rn(sf, pr);
      const float bb = __fadd_rn(s1, -sf);
      const float e2 = __fadd_rn(__fadd_rn(sf, -__fadd_rn(s1, -bb)), __fadd_rn(pr, -bb));  // TwoSum error
      err += __fadd_rn(__fadd_rn(__fadd_rn(nf, -s1), -e2), -e1);
      sf = nf;
    }
  }
  double e = static_cast<double>(err);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) e += __shfl_xor_sync(0xffffffffu, e, d);
  if (lane == 0) werr[w] = e;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int k = 0; k < 8; ++k) t += werr[k];
    seq_err[row * chunks + c] = t;
  }
}

__global__ void rms_chunk_apply_kernel(const float* __restrict__ x, const float* __restrict__ gamma, long long n_gamma,
                                       float* __restrict__ y, const float* __restrict__ part, long long len, int chunks,
                                       int chunk_len, float eps, const double* __restrict__ seq_err = nullptr) {
  const long long row = blockIdx.y;
  float rms;
  if (seq_err != nullptr) {
    // sum of squares as the reference's sequential fp32 loop produces it: exact sum + its rounding errors
    double sd = 0.0;
    for (int j = 0; j < chunks; ++j) sd += static_cast<double>(part[row * chunks + j]) + seq_err[row * chunks + j];
    rms = sqrtf(static_cast<float>(sd) / static_cast<float>(len) + eps);
  } else {
    float s = 0.0f;
    for (int j = 0; j < chunks; ++j) s += part[row * chunks + j];
    rms = sqrtf(s / static_cast<float>(len) + eps);
  }
  const long long off = static_cast<long long>(blockIdx.x) * chunk_len;
  const long long cn = min(static_cast<long long>(chunk_len), len - off);
  const float* g = x + row * len + off;
  float* o = y + row * len + off;
  if (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(o)) & 15) == 0 && (cn & 3) == 0 &&
      (gamma == nullptr || ((reinterpret_cast<uintptr_t>(gamma + off) & 15) == 0 && off + cn <= n_gamma))) {
    const float4* g4 = reinterpret_cast<const float4*>(g);
    const float4* w4 = gamma ? reinterpret_cast<const float4*>(gamma + off) : nullptr;
    float4* o4 = reinterpret_cast<float4*>(o);
    const int n4 = static_cast<int>(cn >> 2), step = blockDim.x;
    auto one = [&](int i, float4 v, float4 w) {
      v.x /= rms; v.y /= rms; v.z /= rms; v.w /= rms;
      if (w4 != nullptr) { v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w; }
      __stcs(o4 + i, v);
    };
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    int i = threadIdx.x;
    for (; i + 3 * step < n4; i += 4 * step) {  // eight loads in flight
      const float4 a = __ldcs(g4 + i), b = __ldcs(g4 + i + step), c = __ldcs(g4 + i + 2 * step), d = __ldcs(g4 + i + 3 * step);
      const float4 wa = w4 ? __ldg(w4 + i) : z, wb = w4 ? __ldg(w4 + i + step) : z, wc = w4 ? __ldg(w4 + i + 2 * step) : z,
                   wd = w4 ? __ldg(w4 + i + 3 * step) : z;
      one(i, a, wa); one(i + step, b, wb); one(i + 2 * step, c, wc); one(i + 3 * step, d, wd);
    }
    for (; i < n4; i += step) one(i, __ldcs(g4 + i), w4 ? __ldg(w4 + i) : z);
  } else {
    for (long long i = threadIdx.x; i < cn; i += blockDim.x) {
      float v = __ldg(g + i) / rms;
      if (gamma != nullptr && off + i < n_gamma) v *= __ldg(gamma + off + i);
      o[i] = v;
    }
  }
}

// ---- RMSNorm over a long sample in ONE pass over HBM ---------------------------------------------
// One CTA per 8192-element chunk keeps its chunk in shared memory from the load to the store (six
// CTAs per SM: 192 KB of the sample in flight per SM).  Between the two it needs (1) the sum of
// squares of the chunks before it in the sample - for the binade of the reference's running sum,
// see rms_seq_err_kernel; inside the chunk the running sum is interpolated - and (2) the sample's
// total.  Both travel through 64-bit slots {tag, fp32 value} in global memory, published with an
// atomic exchange (a plain store takes measurably longer to become visible to the pollers).  CTAs
// take their chunk from a ticket counter, so a CTA only ever waits for chunks whose CTAs started
// before it or belong to its own sample; the launcher only uses this kernel when a whole sample's
// CTAs are resident at once.  Every wait is bounded: after ~2 s (or when another CTA gave up) the
// CTA reports through the device error word and leaves without writing.
constexpr int OP_VEC = CHUNK / (256 * 4);  // float4 per thread

struct RmsOnePass {
  const float* x;
  const float* gamma;
  long long n_gamma;
  float* y;                 // fp32 output, or nullptr
  __nv_bfloat16* y_split;   // bf16 hi (and lo) planes, or nullptr
  long long plane_stride;   // elements between the hi and the lo plane
  int planes;
  int f16;                  // the planes hold IEEE half instead of bfloat16
  unsigned* ticket;         // [0] ticket counter, [1] abort flag
  unsigned long long* sum_slots;
  unsigned long long* err_slots;
  long long len;
  int chunks;
  float eps;
  int* err_word;
};

__device__ __forceinline__ unsigned long long slot_pack(float v) {
  return (1ull << 32) | static_cast<unsigned long long>(__float_as_uint(v));
}
// Polls one slot until its tag is set.  Returns false when the wait gave up.
__device__ __forceinline__ bool slot_wait(const unsigned long long* slot, volatile unsigned* abort_flag, int* err_word, int site,
                                          float* out) {
  const volatile unsigned long long* p = slot;
  unsigned long long v = *p;
  if ((v >> 32) == 0) {
    uint64_t t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    unsigned spins = 0;
    while (((v = *p) >> 32) == 0) {
      __nanosleep(64);
      if ((++spins & 0xFF) == 0) {
        if (*abort_flag) return false;
        uint64_t t1;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) {
          *abort_flag = 1u;
          atomicExch(err_word, site);
          return false;
        }
      }
    }
  }
  *out = __uint_as_float(static_cast<unsigned>(v & 0xffffffffull));
  return true;
}
__device__ __forceinline__ double block_sum_f64(double v, double* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  double t = 0.0;
#pragma unroll
  for (int k = 0; k < 8; ++k) t += red[k];
  return t;
}

__global__ void __launch_bounds__(256, 6) rms_onepass_kernel(const RmsOnePass p) {
  extern __shared__ __align__(128) float sx[];  // the chunk, zero beyond its end
  __shared__ __align__(8) uint64_t bar;
  __shared__ unsigned s_id;
  __shared__ int s_abort;
  __shared__ float redf[33];
  __shared__ double red[8];
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_id = atomicAdd(p.ticket, 1u);
    s_abort = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const long long row = s_id / static_cast<unsigned>(p.chunks);
  const int c = static_cast<int>(s_id % static_cast<unsigned>(p.chunks));
  const long long off = static_cast<long long>(c) * CHUNK;
  const int n = static_cast<int>(min(static_cast<long long>(CHUNK), p.len - off));
  const float* g = p.x + row * p.len + off;
  volatile unsigned* abort_flag = p.ticket + 1;

  // ---- the chunk into shared memory: bulk copies when source and size allow, plain loads otherwise ----
  const bool bulk = (reinterpret_cast<uintptr_t>(g) & 15) == 0 && (n & 3) == 0;
  bool ok = true;
  if (bulk) {
    if (tid == 0) {
      mbar_expect_tx(&bar, static_cast<uint32_t>(n) * 4u);
      for (int b0 = 0; b0 < n; b0 += 2048) bulk_load_1d(sx + b0, g + b0, static_cast<uint32_t>(min(2048, n - b0)) * 4u, &bar);
    }
    for (int i = n + tid; i < CHUNK; i += 256) sx[i] = 0.0f;
    if (!mbar_wait(&bar, 0, &s_abort, p.err_word, 20)) ok = false;
  } else {
    for (int i = tid; i < CHUNK; i += 256) sx[i] = (i < n) ? __ldg(g + i) : 0.0f;
  }
  __syncthreads();
  const float4* s4 = reinterpret_cast<const float4*>(sx);
  // ---- the chunk's sum of squares ----
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < OP_VEC; ++i) {
    const float4 v = s4[i * 256 + tid];
    acc += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
  }
  const float run = block_sum(acc, redf);
  const long long slot0 = row * p.chunks;
  if (tid == 0) atomicExch(p.sum_slots + slot0 + c, slot_pack(run));

  // ---- sum of the chunks before this one (only its binade matters) ----
  double before = 0.0;
  for (int j = tid; j < c; j += 256) {
    float t = 0.0f;
    ok = ok && slot_wait(p.sum_slots + slot0 + j, abort_flag, p.err_word, 21, &t);
    before += static_cast<double>(t);
  }
  const double prefix = block_sum_f64(before, red);

  // ---- replay the reference's chain s = fma(x, x, s) over this thread's elements and collect the
  //      rounding error of every step with error-free transformations (see rms_seq_err_kernel) ----
  float err = 0.0f;
#pragma unroll
  for (int i = 0; i < OP_VEC; ++i) {
    // Where the chain stood before this float4: only the binade of that value enters the rounding of a step,
    // so inside the chunk (1 % of a long sample) the running sum is taken as growing evenly.
    float sf = static_cast<float>(prefix) + run * (static_cast<float>((i * 256 + tid) * 4) * (1.0f / CHUNK));
    const float4 v = s4[i * 256 + tid];
    const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // the zero tail adds nothing and rounds nothing
      // One step of the chain, nf = RN(sf + a*a), and its rounding error nf - (sf + a*a), from three exact pieces:
      // a*a = pr + e1 (product and its error), d = nf - sf (exact while nf <= 2 sf, i.e. once the running sum
      // exceeds a single square) and d - pr (exact when a*a is not far below the sum's ulp; otherwise its own
      // rounding is 2^-24 of a rounding error).
      const float a = e4[j];
      const float nf = fmaf(a, a, sf);
      const float pr = __fmul_rn(a, a);
      const float e1 = fmaf(a, a, -pr);
      err += __fadd_rn(__fadd_rn(__fadd_rn(nf, -sf), -pr), -e1);
      sf = nf;
    }
  }
  const double chunk_err = block_sum_f64(static_cast<double>(err), red);
  if (tid == 0) atomicExch(p.err_slots + slot0 + c, slot_pack(static_cast<float>(chunk_err)));

  // ---- the sample's total: every chunk's sum and chain error ----
  double mine = 0.0;
  for (int j = tid; j < p.chunks; j += 256) {
    float e = 0.0f, s = 0.0f;
    ok = ok && slot_wait(p.err_slots + slot0 + j, abort_flag, p.err_word, 22, &e);
    ok = ok && slot_wait(p.sum_slots + slot0 + j, abort_flag, p.err_word, 23, &s);
    mine += static_cast<double>(s) + static_cast<double>(e);
  }
  const double sd = block_sum_f64(mine, red);
  if (__syncthreads_or(!ok)) {  // a wait gave up: the error word is set, nothing is written
    if (tid == 0) *abort_flag = 1u;
    return;
  }
  const float rms = sqrtf(static_cast<float>(sd) / static_cast<float>(p.len) + p.eps);
  const float inv_rms = 1.0f / rms;

  // ---- apply and store ----
  const long long base = row * p.len + off;
  const bool vec_out = (n & 3) == 0 && (p.y == nullptr || (reinterpret_cast<uintptr_t>(p.y + base) & 15) == 0) &&
                       (p.y_split == nullptr || ((reinterpret_cast<uintptr_t>(p.y_split + base) & 7) == 0 && (p.plane_stride & 3) == 0));
  const bool vec_gamma = p.gamma != nullptr && (reinterpret_cast<uintptr_t>(p.gamma + off) & 15) == 0 && off + n <= p.n_gamma;
#pragma unroll 2
  for (int i = 0; i < OP_VEC; ++i) {
    const int e0 = (i * 256 + tid) * 4;
    if (e0 >= n) break;
    const float4 v = s4[i * 256 + tid];
    // x / rms as one multiply by the reciprocal plus one correction step (what the division routine itself does,
    // minus its special-case handling: the quotient of two normal numbers comes out correctly rounded)
    float o[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q0 = o[j] * inv_rms;
      o[j] = fmaf(fmaf(-q0, rms, o[j]), inv_rms, q0);
    }
    if (vec_gamma) {
      const float4 gm = __ldg(reinterpret_cast<const float4*>(p.gamma + off + e0));
      o[0] *= gm.x; o[1] *= gm.y; o[2] *= gm.z; o[3] *= gm.w;
    } else if (p.gamma != nullptr) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (off + e0 + j < p.n_gamma) o[j] *= __ldg(p.gamma + off + e0 + j);
    }
    if (vec_out) {
      if (p.y != nullptr) __stcs(reinterpret_cast<float4*>(p.y + base + e0), make_float4(o[0], o[1], o[2], o[3]));
      if (p.y_split != nullptr) {
        uint32_t h01, h23, l01, l23;
        split_pair(o[0], o[1], p.f16, h01, l01);
        split_pair(o[2], o[3], p.f16, h23, l23);
        *reinterpret_cast<uint2*>(p.y_split + base + e0) = make_uint2(h01, h23);
        if (p.planes == 2) *reinterpret_cast<uint2*>(p.y_split + p.plane_stride + base + e0) = make_uint2(l01, l23);
      }
    } else {
      for (int j = 0; j < 4 && e0 + j < n; ++j) {
        if (p.y != nullptr) p.y[base + e0 + j] = o[j];
        if (p.y_split != nullptr) {
          uint16_t h, l;
          split_one(o[j], p.f16, h, l);
          uint16_t* y16 = reinterpret_cast<uint16_t*>(p.y_split);
          y16[base + e0 + j] = h;
          if (p.planes == 2) y16[p.plane_stride + base + e0 + j] = l;
        }
      }
    }
  }
}

// ---- chunk kernels (softmax) -------------------------------------------------------------------
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
  for (long long i = threadIdx.x; i < n; i += blockDim.x) acc += __expf(sch[i] - m);
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
    o[i] = log_softmax ? ((v - m) - ld) : __expf(v - m) * inv;
  }
}

// ---- CTA-per-row streaming kernels -----------------------------------------------------------
// For many rows of any length: one CTA owns a row and sweeps it two or three times with unrolled
// 128-bit loads — the first sweep comes from HBM, the later ones hit L2 (a CTA re-reads what it
// read a few hundred KB ago) — so HBM sees one read and one write per element while loads stay in
// flight through every phase; the only barriers are the block reductions between sweeps.
// The per-element work is kept far below the ~40 lane-operations a B200 can spend per element of
// an 8-byte-per-element stream: fast exp2-based exponentials, channel indices advanced
// incrementally instead of divided, gamma / beta read as 128-bit vectors.
enum { FAM_MEANVAR = 0, FAM_RMS = 1, FAM_SOFTMAX = 2 };

struct RowParams {
  const float* x;
  float* y;
  long long rows;
  long long len;
  float eps;
  Affine aff;            // FAM_MEANVAR
  const float* gamma;    // FAM_RMS
  long long n_gamma;     // FAM_RMS
  int log_softmax;       // FAM_SOFTMAX
  float* stats_out;      // FAM_MEANVAR: when set, only (mean, 1/std) of every row is written, no output sweep
  const float* stats_in; // FAM_MEANVAR: when set, (mean, 1/std) of every row are read here, no statistics sweep
};

__device__ __forceinline__ float silu_fast(float v) { return v * __fdividef(1.0f, 1.0f + __expf(-v)); }

// Visits the 128-bit vectors of a row in this thread's grid-stride order with four loads in flight
// before the first use (the rows are streamed from HBM / L2: memory-level parallelism is what counts).
template <bool STREAMING, class F>
__device__ __forceinline__ void for_each_vec4(const float4* __restrict__ g4, int n4, F body) {
  const int step = blockDim.x;
  int i = threadIdx.x;
  for (; i + 3 * step < n4; i += 4 * step) {
    float4 a, b, c, d;
    if (STREAMING) {
      a = __ldcs(g4 + i); b = __ldcs(g4 + i + step); c = __ldcs(g4 + i + 2 * step); d = __ldcs(g4 + i + 3 * step);
    } else {
      a = __ldg(g4 + i); b = __ldg(g4 + i + step); c = __ldg(g4 + i + 2 * step); d = __ldg(g4 + i + 3 * step);
    }
    body(i, a);
    body(i + step, b);
    body(i + 2 * step, c);
    body(i + 3 * step, d);
  }
  for (; i < n4; i += step) body(i, STREAMING ? __ldcs(g4 + i) : __ldg(g4 + i));
}

template <class F>
__device__ __forceinline__ void sweep_read(const float* __restrict__ g, long long n, bool vec, F f) {
  if (vec) {
    for_each_vec4<false>(reinterpret_cast<const float4*>(g), static_cast<int>(n >> 2), [&](int, const float4& v) {
      f(v.x); f(v.y); f(v.z); f(v.w);
    });
  } else {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) f(__ldg(g + i));
  }
}

template <class F>
__device__ __forceinline__ void sweep_write(const float* __restrict__ g, float* __restrict__ o, long long n, bool vec, F f) {
  if (vec) {
    float4* o4 = reinterpret_cast<float4*>(o);
    for_each_vec4<true>(reinterpret_cast<const float4*>(g), static_cast<int>(n >> 2), [&](int i, const float4& v) {
      const long long e = static_cast<long long>(i) << 2;
      float4 r;
      r.x = f(v.x, e); r.y = f(v.y, e + 1); r.z = f(v.z, e + 2); r.w = f(v.w, e + 3);
      __stcs(o4 + i, r);
    });
  } else {
    for (long long i = threadIdx.x; i < n; i += blockDim.x) o[i] = f(__ldg(g + i), i);
  }
}

// normalise + affine + activation + residual for one row, vector paths for the two affine layouts
// (g, o point at element `off` of the row; n elements are written)
__device__ __forceinline__ void meanvar_write_row(const float* __restrict__ g, float* __restrict__ o, long long n, bool vec,
                                                  float mean, float inv, long long row, long long base, const Affine& a,
                                                  long long off = 0) {
  const float* gam = (a.gamma && !a.per_channel) ? a.gamma + off : a.gamma;
  const float* bet = (a.beta && !a.per_channel) ? a.beta + off : a.beta;
  const float* res = a.residual ? a.residual + base + off : nullptr;
  const bool silu_on = a.act == MIMIR_B200_ELT_SILU;
  if (vec && !a.per_channel && (gam == nullptr || ((reinterpret_cast<uintptr_t>(gam) & 15) == 0 &&
                                                   (bet == nullptr || (reinterpret_cast<uintptr_t>(bet) & 15) == 0)))) {
    float4* o4 = reinterpret_cast<float4*>(o);
    for_each_vec4<true>(reinterpret_cast<const float4*>(g), static_cast<int>(n >> 2), [&](int i, const float4& v) {
      float4 r = make_float4((v.x - mean) * inv, (v.y - mean) * inv, (v.z - mean) * inv, (v.w - mean) * inv);
      if (gam != nullptr) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(gam) + i);
        r.x *= w.x; r.y *= w.y; r.z *= w.z; r.w *= w.w;
        if (bet != nullptr) {
          const float4 b = __ldg(reinterpret_cast<const float4*>(bet) + i);
          r.x += b.x; r.y += b.y; r.z += b.z; r.w += b.w;
        }
      }
      if (silu_on) { r.x = silu_fast(r.x); r.y = silu_fast(r.y); r.z = silu_fast(r.z); r.w = silu_fast(r.w); }
      if (res != nullptr) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(res) + i);
        r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w;
      }
      __stcs(o4 + i, r);
    });
    return;
  }
  if (vec && a.per_channel && (a.hw & 3) == 0) {
    // the four elements of a vector share a channel; the channel advances incrementally
    float4* o4 = reinterpret_cast<float4*>(o);
    const unsigned hw = static_cast<unsigned>(a.hw), estep = blockDim.x * 4u;
    unsigned c = static_cast<unsigned>((off + threadIdx.x * 4u) / hw), rem = static_cast<unsigned>((off + threadIdx.x * 4u) % hw);
    const int c0 = static_cast<int>(row % a.groups) * a.cpg;
    for_each_vec4<true>(reinterpret_cast<const float4*>(g), static_cast<int>(n >> 2), [&](int i, const float4& v) {
      float sc = inv, sh = -mean * inv;
      if (gam != nullptr) {
        const float w = __ldg(gam + c0 + c);
        sc *= w;
        sh *= w;
        if (bet != nullptr) sh += __ldg(bet + c0 + c);
      }
      float4 r = make_float4(fmaf(v.x, sc, sh), fmaf(v.y, sc, sh), fmaf(v.z, sc, sh), fmaf(v.w, sc, sh));
      if (silu_on) { r.x = silu_fast(r.x); r.y = silu_fast(r.y); r.z = silu_fast(r.z); r.w = silu_fast(r.w); }
      if (res != nullptr) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(res) + i);
        r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w;
      }
      __stcs(o4 + i, r);
      rem += estep;
      while (rem >= hw) { rem -= hw; ++c; }
    });
    return;
  }
  for (long long i = threadIdx.x; i < n; i += blockDim.x) o[i] = finish((__ldg(g + i) - mean) * inv, off + i, row, base, a);
}

// pass 2 of the mean/variance chunk path: combine the row's partials (pairwise-update formula of
// Chan et al.), normalise the chunk
__global__ void meanvar_chunk_apply_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ part,
                                           long long len, int chunks, int chunk_len, float eps, Affine a, long long row0) {
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
  const long long base = (row + row0) * len;  // x, y were advanced by row0 rows; gamma / residual are absolute
  const float* g = x + row * len + off;
  float* o = y + row * len + off;
  Affine al = a;
  if (al.residual) al.residual = a.residual;  // indexed with the absolute base below
  const bool vec = (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(o)) & 15) == 0) && ((cn & 3) == 0) &&
                   (a.residual == nullptr || (reinterpret_cast<uintptr_t>(a.residual + base + off) & 15) == 0) &&
                   (a.per_channel || a.gamma == nullptr || (off & 3) == 0);
  meanvar_write_row(g, o, cn, vec, mean, inv, row + row0, base, al, off);
}

// ---- a few rows of up to ~100 000 elements: one thread-block cluster per row -----------------------
// Each CTA of the cluster keeps a slice of the row in shared memory; the partial sums meet through
// distributed shared memory (every CTA reads all partials in the same order, so all agree bit for bit):
// first the sum for the mean, then the centred second moment, as the reference's two loops do
// (LayerOps.hpp:287-300).  One launch, one read and one write of the row, no global scratch.
constexpr int CLUSTER_SLICE_MAX = 12288;  // floats of shared memory per CTA (48 KB)

__global__ void __launch_bounds__(256) meanvar_cluster_kernel(const float* __restrict__ x, float* __restrict__ y, long long len,
                                                              int slice, float eps, Affine a) {
  namespace cg = cooperative_groups;
  cg::cluster_group cl = cg::this_cluster();
  extern __shared__ __align__(16) float sx[];
  __shared__ float red[33];
  __shared__ float part[2];
  const unsigned ncl = cl.num_blocks(), rank = cl.block_rank();
  const long long row = blockIdx.x / ncl;
  const long long off = static_cast<long long>(rank) * slice;
  const int n = static_cast<int>(max(0ll, min(static_cast<long long>(slice), len - off)));
  const long long base = row * len;
  const float acc = stage_and_sum(x + base + off, sx, n);
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) part[0] = s;
  cl.sync();
  float total = 0.0f;
  for (unsigned k = 0; k < ncl; ++k) total += *cl.map_shared_rank(&part[0], k);
  const float mean = total / static_cast<float>(len);
  float q = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float d = sx[i] - mean;
    q = fmaf(d, d, q);
  }
  const float m2 = block_sum(q, red);
  if (threadIdx.x == 0) part[1] = m2;
  cl.sync();
  float var = 0.0f;
  for (unsigned k = 0; k < ncl; ++k) var += *cl.map_shared_rank(&part[1], k);
  const float inv = 1.0f / sqrtf(var / static_cast<float>(len) + eps);
  float* o = y + base + off;
  // 16-byte path: four neighbours share a channel when the plane size is a multiple of 4 (slices start on multiples of 4)
  const bool vec = (n & 3) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0 &&
                   (a.residual == nullptr || (reinterpret_cast<uintptr_t>(a.residual + base + off) & 15) == 0) &&
                   (a.per_channel ? (a.hw & 3) == 0
                                  : ((a.gamma == nullptr || (reinterpret_cast<uintptr_t>(a.gamma + off) & 15) == 0) &&
                                     (a.beta == nullptr || (reinterpret_cast<uintptr_t>(a.beta + off) & 15) == 0)));
  if (vec) {
    const float4* s4 = reinterpret_cast<const float4*>(sx);
    const float4* g4 = (a.gamma && !a.per_channel) ? reinterpret_cast<const float4*>(a.gamma + off) : nullptr;
    const float4* b4 = (a.beta && !a.per_channel) ? reinterpret_cast<const float4*>(a.beta + off) : nullptr;
    const float4* r4 = a.residual ? reinterpret_cast<const float4*>(a.residual + base + off) : nullptr;
    const int ch0 = a.per_channel ? static_cast<int>(row % a.groups) * a.cpg : 0;
    const unsigned off_u = static_cast<unsigned>(off);
    for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
      const float4 v = s4[i];
      float4 r = make_float4((v.x - mean) * inv, (v.y - mean) * inv, (v.z - mean) * inv, (v.w - mean) * inv);
      if (a.per_channel) {
        if (a.gamma != nullptr) {
          const int gi = ch0 + static_cast<int>((off_u + 4u * static_cast<unsigned>(i)) / static_cast<unsigned>(a.hw));
          const float w = __ldg(a.gamma + gi);
          r.x *= w; r.y *= w; r.z *= w; r.w *= w;
          if (a.beta != nullptr) {
            const float b = __ldg(a.beta + gi);
            r.x += b; r.y += b; r.z += b; r.w += b;
          }
        }
      } else if (g4 != nullptr) {
        const float4 w = __ldg(g4 + i);
        r.x *= w.x; r.y *= w.y; r.z *= w.z; r.w *= w.w;
        if (b4 != nullptr) {
          const float4 b = __ldg(b4 + i);
          r.x += b.x; r.y += b.y; r.z += b.z; r.w += b.w;
        }
      }
      if (a.act == MIMIR_B200_ELT_SILU) {
        r.x = silu(r.x); r.y = silu(r.y); r.z = silu(r.z); r.w = silu(r.w);
      }
      if (r4 != nullptr) {
        const float4 t = __ldg(r4 + i);
        r.x += t.x; r.y += t.y; r.z += t.z; r.w += t.w;
      }
      __stcs(reinterpret_cast<float4*>(o) + i, r);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = finish((sx[i] - mean) * inv, off + i, row, base, a);
  }
  cl.sync();  // nobody leaves while a neighbour may still read its partial sums
}

template <int FAM, int THREADS>
__global__ void __launch_bounds__(THREADS, (THREADS <= 512) ? 2 : 1) sweep_row_kernel(RowParams p) {
  __shared__ float red[33];
  const long long n = p.len;
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const long long base = row * n;
    const float* g = p.x + base;
    float* o = p.y + base;
    bool vec = (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(o)) & 15) == 0) && ((n & 3) == 0) &&
               (n < (1LL << 31));
    if (FAM == FAM_MEANVAR) {
      if (p.aff.residual != nullptr && (reinterpret_cast<uintptr_t>(p.aff.residual + base) & 15) != 0) vec = false;
      // One statistics sweep: sums of (x - K) and (x - K)^2 with K = the row's first element, which
      // is exact algebra for mean and variance and loses nothing as long as K is within a few standard
      // deviations of the mean.  When the shift turns out to be poor (the correction term eats more than
      // 3/4 of the second moment) the variance is recomputed centred on the mean, as the reference does.
      if (p.stats_in != nullptr) {  // the statistics came with the producer's epilogue: one sweep only
        meanvar_write_row(g, o, n, vec, __ldg(p.stats_in + 2 * row), __ldg(p.stats_in + 2 * row + 1), row, base, p.aff);
        continue;
      }
      const float shift = __ldg(g);
      float s = 0.0f, q = 0.0f;
      sweep_read(g, n, vec, [&](float v) { const float d = v - shift; s += d; q = fmaf(d, d, q); });
      const float s1 = block_sum(s, red), s2 = block_sum(q, red);
      const float fn = static_cast<float>(n);
      const float mean = shift + s1 / fn;
      float m2 = s2 - s1 * (s1 / fn);
      if (s1 * (s1 / fn) > 0.75f * s2) {  // block-uniform
        float qc = 0.0f;
        sweep_read(g, n, vec, [&](float v) { const float d = v - mean; qc = fmaf(d, d, qc); });
        m2 = block_sum(qc, red);
      }
      const float inv = 1.0f / sqrtf(fmaxf(m2, 0.0f) / fn + p.eps);
      if (p.stats_out != nullptr) {
        if (threadIdx.x == 0) {
          p.stats_out[2 * row] = mean;
          p.stats_out[2 * row + 1] = inv;
        }
        continue;
      }
      meanvar_write_row(g, o, n, vec, mean, inv, row, base, p.aff);
    } else if (FAM == FAM_RMS) {
      float q = 0.0f;
      sweep_read(g, n, vec, [&](float v) { q = fmaf(v, v, q); });
      const float rinv = 1.0f / sqrtf(block_sum(q, red) / static_cast<float>(n) + p.eps);
      const float* gam = p.gamma;
      const long long ng = p.n_gamma;
      if (vec && (gam == nullptr || (ng >= n && (reinterpret_cast<uintptr_t>(gam) & 15) == 0))) {
        float4* o4 = reinterpret_cast<float4*>(o);
        for_each_vec4<true>(reinterpret_cast<const float4*>(g), static_cast<int>(n >> 2), [&](int i, const float4& vin) {
          float4 v = vin;
          v.x *= rinv; v.y *= rinv; v.z *= rinv; v.w *= rinv;
          if (gam != nullptr) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(gam) + i);
            v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
          }
          __stcs(o4 + i, v);
        });
      } else {
        sweep_write(g, o, n, false, [&](float v, long long e) {
          float r = v * rinv;
          if (gam != nullptr && e < ng) r *= __ldg(gam + e);
          return r;
        });
      }
    } else {
      // online (max, sum of exp) per thread without a data-dependent branch
      // running (max, sum of exp) per thread, rescaled once per 128-bit vector: 5 exponentials per 4
      // elements keep the transcendental unit below the memory time
      float m = -3.0e38f, sum = 0.0f;
      if (vec) {
        for_each_vec4<false>(reinterpret_cast<const float4*>(g), static_cast<int>(n >> 2), [&](int, const float4& v) {
          const float mn = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
          sum = sum * __expf(m - mn) + ((__expf(v.x - mn) + __expf(v.y - mn)) + (__expf(v.z - mn) + __expf(v.w - mn)));
          m = mn;
        });
      } else {
        sweep_read(g, n, false, [&](float v) {
          const float mn = fmaxf(m, v);
          sum = sum * __expf(m - mn) + __expf(v - mn);
          m = mn;
        });
      }
      const float gm = block_max(m, red);
      const float tot = block_sum(sum * __expf(m - gm), red);
      if (p.log_softmax) {
        const float ld = logf(tot);
        sweep_write(g, o, n, vec, [&](float v, long long) { return (v - gm) - ld; });
      } else {
        const float inv = 1.0f / tot;
        sweep_write(g, o, n, vec, [&](float v, long long) { return __expf(v - gm) * inv; });
      }
    }
  }
}

template <int FAM>
int launch_sweep_rows(const RowParams& p, cudaStream_t st) {
  const long long sms = ctx().sm_count;
  // rows in flight are re-read from L2: keep their footprint well inside it
  const bool big = p.len * 4 * 2 * sms > (40ll << 20);
  if (big) {
    long long blocks = sms < p.rows ? sms : p.rows;
    sweep_row_kernel<FAM, 1024><<<static_cast<int>(blocks), 1024, 0, st>>>(p);
  } else {
    int threads = 512;
    while (threads > 128 && static_cast<long long>(threads) * 16 > p.len) threads >>= 1;  // >= 4 vectors per thread
    long long blocks = sms * (1024 / threads) * 2;
    if (blocks > p.rows) blocks = p.rows;
    sweep_row_kernel<FAM, 512><<<static_cast<int>(blocks), threads, 0, st>>>(p);
  }
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

// The sweeps pay off when every SM has rows of its own.  They are at their best when the rows in flight
// stay inside L2 (the second sweep then never touches HBM), but measured on 1 MB rows (GroupNorm over
// 4 x 256 x 256 slabs, 148 MB in flight) they still beat the chunk path's many short launches, so only
// very long rows go to the chunk path (L2-sized row groups).
// MIMIR_B200_NORM_PATH=sweep|chunk overrides the choice (measurement aid).
inline bool use_sweeps(long long rows, long long len) {
  const char* v = getenv("MIMIR_B200_NORM_PATH");
  if (v && v[0] == 's') return true;
  if (v && v[0] == 'c') return false;
  const long long sms = ctx().sm_count;
  const long long in_flight = (rows < sms ? rows : sms) * len * 4;
  return rows >= sms && in_flight <= (1024ll << 20);
}

// ---- warp-per-row LayerNorm for short rows (token-wise norms): no block barrier at all --------
constexpr int WARP_ROW_MAX = 1024;  // floats

template <int NV>  // 128-bit vectors per lane
__global__ void __launch_bounds__(256) meanvar_warp_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows,
                                                           int len, float eps, Affine a) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int n4 = len >> 2;  // len is a multiple of 4 on this path
  const bool gvec = a.gamma == nullptr || ((reinterpret_cast<uintptr_t>(a.gamma) & 15) == 0 &&
                                           (a.beta == nullptr || (reinterpret_cast<uintptr_t>(a.beta) & 15) == 0));
  for (long long row = warp; row < rows; row += nwarps) {
    const long long base = row * len;
    const float4* g4 = reinterpret_cast<const float4*>(x + base);
    float4 v[NV];
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      v[j] = (i < n4) ? __ldg(g4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = warp_sum(s) / static_cast<float>(len);
    float q = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (lane + 32 * j < n4) {
        const float dx = v[j].x - mean, dy = v[j].y - mean, dz = v[j].z - mean, dw = v[j].w - mean;
        q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
      }
    }
    const float inv = 1.0f / sqrtf(warp_sum(q) / static_cast<float>(len) + eps);
    float4* o4 = reinterpret_cast<float4*>(y + base);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = lane + 32 * j;
      if (i < n4) {
        float4 r;
        if (!a.per_channel && gvec && a.act < 0 && a.residual == nullptr) {
          r = make_float4((v[j].x - mean) * inv, (v[j].y - mean) * inv, (v[j].z - mean) * inv, (v[j].w - mean) * inv);
          if (a.gamma != nullptr) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(a.gamma) + i);
            r.x *= w.x; r.y *= w.y; r.z *= w.z; r.w *= w.w;
            if (a.beta != nullptr) {
              const float4 b = __ldg(reinterpret_cast<const float4*>(a.beta) + i);
              r.x += b.x; r.y += b.y; r.z += b.z; r.w += b.w;
            }
          }
        } else {
          const long long e = static_cast<long long>(i) << 2;
          r.x = finish((v[j].x - mean) * inv, e, row, base, a);
          r.y = finish((v[j].y - mean) * inv, e + 1, row, base, a);
          r.z = finish((v[j].z - mean) * inv, e + 2, row, base, a);
          r.w = finish((v[j].w - mean) * inv, e + 3, row, base, a);
        }
        o4[i] = r;
      }
    }
  }
}

template <int NV>
int launch_warp_rows(const float* x, float* y, long long rows, int len, float eps, const Affine& a, cudaStream_t st) {
  long long blocks = (rows + 7) / 8;
  const long long cap = static_cast<long long>(ctx().sm_count) * 8;
  if (blocks > cap) blocks = cap;
  meanvar_warp_kernel<NV><<<static_cast<int>(blocks), 256, 0, st>>>(x, y, rows, len, eps, a);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

// ---- scratch for the chunk kernels -------------------------------------------------------------
// Partial statistics, and the ticket / slot words of the one-pass RMSNorm, live in an 8 MB buffer PER (device,
// stream): two calls on different streams (two models, two host threads) never share partials or tickets, and
// calls on one stream are ordered by the stream.  g_norm_mu is held while a call enqueues its launches, so the
// memset + kernel pairs of two host threads that use the same stream cannot interleave either.
constexpr size_t NORM_SCRATCH_BYTES = 8u << 20;
constexpr size_t NORM_SCRATCH_MAX_STREAMS = 32;
std::mutex g_norm_mu;
struct NormScratch {
  float* p = nullptr;
  bool pinned = false;  // reserved for a capture stream: its address is baked into CUDA graphs, never recycled
};
std::map<std::pair<int, cudaStream_t>, NormScratch> g_norm_scratch;

// Call with g_norm_mu held.
int norm_scratch(cudaStream_t st, float** out, bool pin = false) {
  int dev = 0;
  MB_CUDA(cudaGetDevice(&dev));
  const auto key = std::make_pair(dev, st);
  auto it = g_norm_scratch.find(key);
  if (it == g_norm_scratch.end()) {
    size_t loose = 0;
    for (auto& kv : g_norm_scratch) loose += kv.second.pinned ? 0 : 1;
    if (loose >= NORM_SCRATCH_MAX_STREAMS) {
      // streams come and go: once the table is full, wait for everything in flight and drop the unpinned buffers
      for (auto jt = g_norm_scratch.begin(); jt != g_norm_scratch.end();) {
        if (jt->second.pinned) { ++jt; continue; }
        MB_CUDA(cudaSetDevice(jt->first.first));
        MB_CUDA(cudaDeviceSynchronize());
        dev_free(jt->second.p, NORM_SCRATCH_BYTES);
        jt = g_norm_scratch.erase(jt);
      }
      MB_CUDA(cudaSetDevice(dev));
    }
    NormScratch ns;
    MB_TRY(dev_alloc(reinterpret_cast<void**>(&ns.p), NORM_SCRATCH_BYTES, "norm_scratch"));
    it = g_norm_scratch.emplace(key, ns).first;
  }
  if (pin) it->second.pinned = true;
  *out = it->second.p;
  return MIMIR_B200_OK;
}

// Rows longer than a cluster can hold go through the two-pass chunk kernels in groups of rows whose
// footprint stays inside L2 (so the second pass reads x from L2, not from HBM).
constexpr long long L2_GROUP_BYTES = 104ll << 20;

int meanvar_dispatch(const float* x, float* y, long long rows, long long len, float eps, const Affine& a, cudaStream_t st) {
  if (rows <= 0 || len <= 0) return fail(MIMIR_B200_E_INVALID, "norm: empty input");
  const bool al16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 &&
                    (a.residual == nullptr || (reinterpret_cast<uintptr_t>(a.residual) & 15) == 0);
  if (len <= WARP_ROW_MAX && (len & 3) == 0 && al16 && rows >= 64) {
    const int nv = static_cast<int>((len / 4 + 31) / 32);
    const int l = static_cast<int>(len);
    if (nv <= 2) return launch_warp_rows<2>(x, y, rows, l, eps, a, st);
    if (nv <= 4) return launch_warp_rows<4>(x, y, rows, l, eps, a, st);
    if (nv <= 6) return launch_warp_rows<6>(x, y, rows, l, eps, a, st);
    return launch_warp_rows<8>(x, y, rows, l, eps, a, st);
  }
  if (use_sweeps(rows, len)) {
    RowParams p{};
    p.x = x; p.y = y; p.rows = rows; p.len = len; p.eps = eps; p.aff = a;
    return launch_sweep_rows<FAM_MEANVAR>(p, st);
  }
  static const bool no_cluster = [] { const char* e = getenv("MIMIR_B200_NORM_CLUSTER"); return e && e[0] == '0'; }();
  if (!no_cluster && len <= 8ll * CLUSTER_SLICE_MAX && rows * 8 < 0x7fffffffLL) {
    int ncl = 1;
    while (ncl < 8 && (len + ncl - 1) / ncl > 4096) ncl *= 2;  // ~16 KB per CTA, at most the portable cluster size
    const int slice = static_cast<int>(((len + ncl - 1) / ncl + 3) & ~3ll);
    static PerDeviceOnce attr_once;  // static + dynamic shared memory of the largest slice is just above the 48 KB default
    MB_TRY(attr_once.run([&]() -> int {
      MB_CUDA(cudaFuncSetAttribute(meanvar_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CLUSTER_SLICE_MAX * 4));
      return MIMIR_B200_OK;
    }));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(rows * ncl));
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = static_cast<size_t>(slice) * sizeof(float);
    cfg.stream = st;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(ncl);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    MB_CUDA(cudaLaunchKernelEx(&cfg, meanvar_cluster_kernel, x, y, len, slice, eps, a));
    count_launch();
    return MIMIR_B200_OK;
  }
  const int chunks = static_cast<int>((len + CHUNK - 1) / CHUNK);
  std::lock_guard<std::mutex> scratch_lock(g_norm_mu);
  float* part;
  MB_TRY(norm_scratch(st, &part));
  long long group = L2_GROUP_BYTES / (len * 4);
  if (group < 1) group = 1;
  const long long cap_rows = static_cast<long long>(NORM_SCRATCH_BYTES / (sizeof(float) * 3)) / chunks;
  if (cap_rows < 1) return fail(MIMIR_B200_E_UNSUPPORTED, "norm: a row of %lld elements exceeds the partial-statistics scratch", len);
  if (group > cap_rows) group = cap_rows;
  if (group > 65535) group = 65535;
  for (long long r0 = 0; r0 < rows; r0 += group) {
    const long long nr = (rows - r0 < group) ? rows - r0 : group;
    dim3 grid(chunks, static_cast<unsigned>(nr));
    Affine ag = a;
    // the kernels index gamma / residual by absolute row: shift the pointers, keep row numbering
    meanvar_chunk_stats_kernel<<<grid, 256, CHUNK * 4, st>>>(x + r0 * len, part, len, chunks, CHUNK);
    MB_CUDA(cudaGetLastError());
    meanvar_chunk_apply_kernel<<<grid, 256, 0, st>>>(x + r0 * len, y + r0 * len, part, len, chunks, CHUNK, eps, ag, r0);
    MB_CUDA(cudaGetLastError());
    count_launch(2);
  }
  return MIMIR_B200_OK;
}

}  // namespace

int norm_scratch_reserve(cudaStream_t st) {
  std::lock_guard<std::mutex> lk(g_norm_mu);
  float* p = nullptr;
  return norm_scratch(st, &p, true);
}

void norm_scratch_release(cudaStream_t st) {
  std::lock_guard<std::mutex> lk(g_norm_mu);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  auto it = g_norm_scratch.find(std::make_pair(dev, st));
  if (it == g_norm_scratch.end()) return;
  dev_free(it->second.p, NORM_SCRATCH_BYTES);
  g_norm_scratch.erase(it);
}

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

// GroupNorm whose statistics [batch][groups][2] already exist (they came out of the producing convolution's epilogue): the
// output sweep alone.  Shapes the row sweeps do not take fall back to the full GroupNorm.
int launch_groupnorm_apply(const float* x, const float* stats, const float* gamma, const float* beta, float* y, int batch, int ch, int hw,
                           int groups, float eps, int act, const float* residual, cudaStream_t st) {
  if (groups <= 0 || ch % groups != 0) return fail(MIMIR_B200_E_INVALID, "GroupNorm: channels must be divisible by num_groups");
  const long long rows = static_cast<long long>(batch) * groups, len = static_cast<long long>(ch / groups) * hw;
  if (stats == nullptr || !use_sweeps(rows, len)) return launch_groupnorm(x, gamma, beta, y, batch, ch, hw, groups, eps, act, residual, st);
  RowParams p{};
  p.x = x; p.y = y; p.rows = rows; p.len = len; p.eps = eps;
  p.aff = Affine{gamma, gamma ? beta : nullptr, 1, groups, ch / groups, hw, act, residual};
  p.stats_in = stats;
  return launch_sweep_rows<FAM_MEANVAR>(p, st);
}

// (mean, 1 / sqrt(var + eps)) of every (sample, group) slab, for consumers that normalise on the fly
int launch_groupnorm_stats(const float* x, float* stats, int batch, int ch, int hw, int groups, float eps, cudaStream_t st) {
  if (groups <= 0 || ch % groups != 0) return fail(MIMIR_B200_E_INVALID, "GroupNorm: channels must be divisible by num_groups");
  RowParams p{};
  p.x = x;
  p.y = const_cast<float*>(x);  // never written on this path
  p.rows = static_cast<long long>(batch) * groups;
  p.len = static_cast<long long>(ch / groups) * hw;
  p.eps = eps;
  p.aff = Affine{nullptr, nullptr, 1, groups, ch / groups, hw, -1, nullptr};
  p.stats_out = stats;
  return launch_sweep_rows<FAM_MEANVAR>(p, st);
}

// ---- GroupNorm statistics from the partials a convolution's GEMM epilogue left behind ----------------------------------------
// One CTA per (group, sample) merges the (pixels, sum, sum of squares) entries of the 32-pixel blocks that hold the sample's rows
// with the pairwise formula of Chan et al., in double and in a fixed order: a thread takes blocks t, t + 128, ... and thread 0
// folds the 128 thread results in thread order.  A block belongs to the sample with its set 0 when its first row does, and
// with its set 1 when it starts in the sample before.
namespace {
struct Moments { double n, mean, m2; };
__device__ __forceinline__ void moments_merge(Moments& a, double nb, double mb, double m2b) {
  if (nb <= 0.0) return;
  const double nt = a.n + nb, delta = mb - a.mean;
  a.mean += delta * (nb / nt);
  a.m2 += m2b + delta * delta * (a.n * nb / nt);
  a.n = nt;
}
__global__ void __launch_bounds__(128) gn_stats_from_partials_kernel(const float* __restrict__ part, float* __restrict__ stats, int groups,
                                                                     int cpg, long long m, int nchunks, int per, float eps) {
  __shared__ Moments sh[128];
  const int g = blockIdx.x, smp = blockIdx.y, es = 1 + 64 / cpg;  // es: floats of one set's entry
  const int cc = (g * cpg) >> 5, gi = ((g * cpg) & 31) / cpg;
  const long long r_first = static_cast<long long>(smp) * per, r_last = min(m, r_first + per) - 1;
  const long long b0 = r_first >> 5, b1 = r_last >> 5;
  Moments acc{0.0, 0.0, 0.0};
  for (long long b = b0 + threadIdx.x; b <= b1; b += 128) {
    const int set = ((b << 5) / per == smp) ? 0 : 1;
    const float* e = part + (b * nchunks + cc) * (2 * es) + set * es;
    const double cnt = static_cast<double>(__ldg(e)) * cpg, sum = __ldg(e + 1 + 2 * gi), sq = __ldg(e + 2 + 2 * gi);
    if (cnt > 0.0) moments_merge(acc, cnt, sum / cnt, fmax(sq - sum * sum / cnt, 0.0));
  }
  sh[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    Moments t = sh[0];
    for (int i = 1; i < 128; ++i) moments_merge(t, sh[i].n, sh[i].mean, sh[i].m2);
    float* o = stats + (static_cast<long long>(smp) * groups + g) * 2;
    o[0] = static_cast<float>(t.mean);
    o[1] = 1.0f / sqrtf(static_cast<float>(t.n > 0.0 ? t.m2 / t.n : 0.0) + eps);
  }
}
}  // namespace

int launch_gn_stats_from_partials(const float* part, float* stats, int batch, int groups, int cpg, long long m, int n, int per, float eps,
                                  cudaStream_t st) {
  if (!part || !stats || batch <= 0 || groups <= 0 || per < 64 || !(cpg == 4 || cpg == 8 || cpg == 16 || cpg == 32) || groups * cpg != n ||
      batch > 65535)
    return fail(MIMIR_B200_E_INVALID, "GroupNorm statistics from partials: bad arguments");
  gn_stats_from_partials_kernel<<<dim3(groups, batch), 128, 0, st>>>(part, stats, groups, cpg, m, (n + 31) / 32, per, eps);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

// The one-pass kernel needs every CTA of a sample resident at once and a slot pair per chunk.
bool rmsnorm_onepass_ok(int batch, int64_t n) {
  static const bool off = [] { const char* e = getenv("MIMIR_B200_RMS_ONEPASS"); return e && e[0] == '0'; }();
  if (off || n <= 16384) return false;
  static int per_sm_dev[MAX_DEVICES];  // occupancy of the one-pass kernel, asked once per device (0 = not asked yet)
  static std::mutex per_sm_mu;
  int per_sm;
  {
    std::lock_guard<std::mutex> lk(per_sm_mu);
    int& slot = per_sm_dev[ctx().device];
    if (slot == 0) {
      int v = 0;
      cudaFuncSetAttribute(rms_onepass_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, rms_onepass_kernel, 256, CHUNK * sizeof(float)) != cudaSuccess) v = 0;
      slot = v > 0 ? v : -1;
    }
    per_sm = slot > 0 ? slot : 0;
  }
  const int64_t chunks = (n + CHUNK - 1) / CHUNK;
  if (chunks > static_cast<int64_t>(per_sm) * ctx().sm_count) return false;
  return static_cast<uint64_t>(batch) * chunks * 16 + 256 <= NORM_SCRATCH_BYTES && static_cast<uint64_t>(batch) * chunks < 0x7fffffffull;
}

int launch_rmsnorm(const float* x, const float* gamma, int64_t n_gamma, float* y, int batch, int64_t n, float eps,
                   cudaStream_t st, __nv_bfloat16* y_split, int planes, int64_t plane_stride) {
  if (batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "RMSNorm: empty input");
  if (rmsnorm_onepass_ok(batch, n)) {
    std::lock_guard<std::mutex> scratch_lock(g_norm_mu);
    float* scratch;
    MB_TRY(norm_scratch(st, &scratch));
    const int chunks = static_cast<int>((n + CHUNK - 1) / CHUNK);
    const size_t slots = static_cast<size_t>(batch) * chunks;
    MB_CUDA(cudaMemsetAsync(scratch, 0, 256 + slots * 16, st));
    RmsOnePass p{};
    p.x = x; p.gamma = gamma; p.n_gamma = gamma ? n_gamma : 0; p.y = y; p.y_split = y_split; p.plane_stride = plane_stride;
    p.planes = planes;
    p.f16 = plane_format() == PLANES_F16 ? 1 : 0;
    p.ticket = reinterpret_cast<unsigned*>(scratch);
    p.sum_slots = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(scratch) + 256);
    p.err_slots = p.sum_slots + slots;
    p.len = n; p.chunks = chunks; p.eps = eps; p.err_word = ctx().dev_error_word;
    rms_onepass_kernel<<<static_cast<unsigned>(slots), 256, CHUNK * sizeof(float), st>>>(p);
    MB_CUDA(cudaGetLastError());
    count_launch();
    return MIMIR_B200_OK;
  }
  if (y == nullptr || y_split != nullptr)
    return fail(MIMIR_B200_E_UNSUPPORTED, "RMSNorm: operand planes were requested for a shape the one-pass kernel does not take");
  // Below this length the sequential chain's rounding loss is < 1e-6 of the sum and any summation order
  // agrees with the reference; above it the chain is reproduced (rms_seq_err_kernel).
  constexpr long long FAITHFUL_FROM = 16384;
  if (n <= FAITHFUL_FROM && use_sweeps(batch, n)) {
    RowParams p{};
    p.x = x; p.y = y; p.rows = batch; p.len = n; p.eps = eps; p.gamma = gamma; p.n_gamma = gamma ? n_gamma : 0;
    return launch_sweep_rows<FAM_RMS>(p, st);
  }
  const int chunks = static_cast<int>((n + CHUNK - 1) / CHUNK);
  std::lock_guard<std::mutex> scratch_lock(g_norm_mu);
  float* part;
  MB_TRY(norm_scratch(st, &part));
  // scratch: [floats: partial sums | doubles: rounding errors], a third and two thirds of the buffer
  constexpr size_t ERR_OFFSET = (NORM_SCRATCH_BYTES / 3) & ~size_t(255);  // doubles start 256-byte aligned
  const long long cap_rows = static_cast<long long>(ERR_OFFSET / sizeof(float)) / chunks;
  if (cap_rows < 1) return fail(MIMIR_B200_E_UNSUPPORTED, "RMSNorm: a row of %lld elements exceeds the partial-statistics scratch", static_cast<long long>(n));
  static_assert((NORM_SCRATCH_BYTES - ERR_OFFSET) / sizeof(double) >= ERR_OFFSET / sizeof(float), "error region too small");
  double* errs = reinterpret_cast<double*>(reinterpret_cast<uint8_t*>(part) + ERR_OFFSET);
  long long group = L2_GROUP_BYTES / (n * 4);
  if (group < 1) group = 1;
  if (group > cap_rows) group = cap_rows;
  if (group > 65535) group = 65535;
  const bool faithful = n > FAITHFUL_FROM;
  for (long long r0 = 0; r0 < batch; r0 += group) {
    const long long nr = (batch - r0 < group) ? batch - r0 : group;
    dim3 grid(chunks, static_cast<unsigned>(nr));
    rms_chunk_stats_kernel<<<grid, 256, 0, st>>>(x + r0 * n, part, n, chunks, CHUNK);
    MB_CUDA(cudaGetLastError());
    if (faithful) {
      rms_seq_err_kernel<<<grid, 256, 0, st>>>(x + r0 * n, part, errs, n, chunks, CHUNK);
      MB_CUDA(cudaGetLastError());
      count_launch();
    }
    rms_chunk_apply_kernel<<<grid, 256, 0, st>>>(x + r0 * n, gamma, gamma ? n_gamma : 0, y + r0 * n, part, n, chunks, CHUNK, eps,
                                                 faithful ? errs : nullptr);
    MB_CUDA(cudaGetLastError());
    count_launch(2);
  }
  return MIMIR_B200_OK;
}

int launch_softmax(const float* x, float* y, int batch, int64_t n, int log_softmax, cudaStream_t st) {
  if (batch <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "Softmax: empty input");
  if (use_sweeps(batch, n)) {
    RowParams p{};
    p.x = x; p.y = y; p.rows = batch; p.len = n; p.log_softmax = log_softmax;
    return launch_sweep_rows<FAM_SOFTMAX>(p, st);
  }
  const int chunks = static_cast<int>((n + CHUNK - 1) / CHUNK);
  std::lock_guard<std::mutex> scratch_lock(g_norm_mu);
  float* part;
  MB_TRY(norm_scratch(st, &part));
  long long group = L2_GROUP_BYTES / (n * 4);
  if (group < 1) group = 1;
  const long long cap_rows = static_cast<long long>(NORM_SCRATCH_BYTES / (2 * sizeof(float))) / chunks;
  if (cap_rows < 1) return fail(MIMIR_B200_E_UNSUPPORTED, "Softmax: a row of %lld elements exceeds the partial-statistics scratch", static_cast<long long>(n));
  if (group > cap_rows) group = cap_rows;
  if (group > 65535) group = 65535;
  for (long long r0 = 0; r0 < batch; r0 += group) {
    const long long nr = (batch - r0 < group) ? batch - r0 : group;
    dim3 grid(chunks, static_cast<unsigned>(nr));
    softmax_chunk_stats_kernel<<<grid, 256, CHUNK * 4, st>>>(x + r0 * n, part, n, chunks, CHUNK);
    MB_CUDA(cudaGetLastError());
    softmax_chunk_apply_kernel<<<grid, 256, 0, st>>>(x + r0 * n, y + r0 * n, part, n, chunks, CHUNK, log_softmax);
    MB_CUDA(cudaGetLastError());
    count_launch(2);
  }
  return MIMIR_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm for callers that must not allocate
// ---------------------------------------------------------------------------------------------
// The chunked RMSNorm above keeps its per-chunk partial sums in a buffer obtained from cudaMalloc.
// Some callers cannot afford that: code running between the launches of a latency-critical
// serving loop (cudaMalloc synchronises the device), code that has handed all free device memory
// to its own pool, and plugins whose host forbids them to allocate.  For them the same kernels
// run with the partial sums (and, for samples above 16 384 elements, the replayed rounding errors
// of the reference's sequential sum) in this fixed array instead.  Every GPU that loads the library
// carries these 192 KB until the process exits.
namespace {

constexpr int NOALLOC_MAX_PARTIALS = 16384;  // batch * ceil(n / 8192) must not exceed it
struct NoAllocScratch {
  float part[NOALLOC_MAX_PARTIALS];    // per-chunk sums of squares
  double err[NOALLOC_MAX_PARTIALS];    // per-chunk rounding errors of the sequential chain
};
static __device__ __align__(256) NoAllocScratch g_rms_noalloc_scratch;

constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mu;
NoAllocScratch* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {};  // device address of the array, per device

// `g_rms_noalloc_scratch` in host code is only a handle for the runtime, not something a kernel may
// dereference; the address kernels can use comes from cudaGetSymbolAddress, asked once per device
// while that device is current.
int noalloc_scratch_for_current_device(NoAllocScratch** out) {
  int dev = -1;
  MB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fail(MIMIR_B200_E_UNSUPPORTED, "rmsnorm_noalloc: device index %d not supported", dev);
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_rms_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(MIMIR_B200_E_CUDA, "rmsnorm_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    g_noalloc_addr[dev] = static_cast<NoAllocScratch*>(p);
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
  NoAllocScratch* sc = nullptr;
  MB_TRY(noalloc_scratch_for_current_device(&sc));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float* g = (gamma && n_gamma > 0) ? gamma : nullptr;
  dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(batch));
  // every partial and error term that a later pass reads is written by an earlier pass of the same call:
  // nothing has to be cleared
  rms_chunk_stats_kernel<<<grid, 256, 0, st>>>(x, sc->part, n, static_cast<int>(chunks), CHUNK);
  MB_CUDA(cudaGetLastError());
  // above this length the reference's one sequential fp32 sum differs measurably from an exact sum, and the
  // difference is reproduced like in mimir_b200_dev_rmsnorm (same threshold)
  const bool faithful = n > 16384;
  if (faithful) {
    rms_seq_err_kernel<<<grid, 256, 0, st>>>(x, sc->part, sc->err, n, static_cast<int>(chunks), CHUNK);
    MB_CUDA(cudaGetLastError());
    count_launch();
  }
  rms_chunk_apply_kernel<<<grid, 256, 0, st>>>(x, g, g ? n_gamma : 0, y, sc->part, n, static_cast<int>(chunks), CHUNK, eps,
                                               faithful ? sc->err : nullptr);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}
