// attention.cu — the attention core between the QKV projection and the output projection.
// Replaces steps 3-5 of LayerOps::self_attention_forward (LayerOps.hpp:1044-1090): per head h and
// query row i, s_j = (Q_i . K_j) / sqrt(hd); causal rows skip j > i (the reference scores them
// -1e9 and keeps them out of the max, so they contribute exp(-1e9 - max) = 0); p = exp(s - max);
// p *= 1 / (sum p + 1e-9); O_i = sum_j p_j V_j.
//
// Flash-style: a CTA owns 64 query rows of one (sample, head) and walks the keys in tiles of 64
// with an online softmax, so the seq x seq score matrix never exists in memory.  fp32 arithmetic
// on the CUDA cores; K and Q tiles are held d-major in shared memory so that the 4x4 register
// blocks read them as conflict-free 128-bit vectors.
#include "common.h"

namespace mb {
namespace {

constexpr int BQ = 64, BKV = 64, LDT = 68;  // LDT: padded leading dimension of the d-major tiles

template <int HD>
__global__ void __launch_bounds__(256)
flash_attn_fp32_kernel(const AttnView a, float* __restrict__ out, int embed, int heads, int causal, float scale) {
  constexpr int CPT = HD / 16;  // output columns per thread
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm;                 // [HD][LDT]   Qt[d][row]
  float* Kt = Qt + HD * LDT;      // [HD][LDT]   Kt[d][key]
  float* Vs = Kt + HD * LDT;      // [BKV][HD]
  float* Pt = Vs + BKV * HD;      // [BKV][LDT]  Pt[key][row]

  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * BQ;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int seq = a.q_len, kvn = a.kv_len;
  const long long ldq = a.ldq, ldk = a.ldkv;
  const long long qbs = a.q_bstride ? a.q_bstride : seq * ldq, kbs = a.kv_bstride ? a.kv_bstride : kvn * ldk;
  const float* qb = a.q + b * qbs + h * HD;
  const float* kb = a.k + b * kbs + h * HD;
  const float* vb = a.v + b * kbs + h * HD;

  // Q tile, transposed into Qt (rows past q_len are zero)
  for (int i = tid; i < BQ * (HD / 4); i += 256) {
    const int r = i / (HD / 4), c4 = (i - r * (HD / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + r < seq) v = __ldg(reinterpret_cast<const float4*>(qb + (q0 + r) * ldq + c4));
    Qt[(c4 + 0) * LDT + r] = v.x; Qt[(c4 + 1) * LDT + r] = v.y; Qt[(c4 + 2) * LDT + r] = v.z; Qt[(c4 + 3) * LDT + r] = v.w;
  }

  float m_run[4], l_run[4], o_acc[4][CPT];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -1e30f;  // the reference's initial max (LayerOps.hpp:1052)
    l_run[i] = 0.0f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) o_acc[i][c] = 0.0f;
  }

  const int kv_end = causal ? min(kvn, q0 + BQ) : kvn;
  for (int k0 = 0; k0 < kv_end; k0 += BKV) {
    __syncthreads();  // previous tile fully consumed (also orders the Qt writes before first use)
    for (int i = tid; i < BKV * (HD / 4); i += 256) {
      const int r = i / (HD / 4), c4 = (i - r * (HD / 4)) * 4;
      float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
      if (k0 + r < kvn) {
        kv = __ldg(reinterpret_cast<const float4*>(kb + (k0 + r) * ldk + c4));
        vv = __ldg(reinterpret_cast<const float4*>(vb + (k0 + r) * ldk + c4));
      }
      Kt[(c4 + 0) * LDT + r] = kv.x; Kt[(c4 + 1) * LDT + r] = kv.y; Kt[(c4 + 2) * LDT + r] = kv.z; Kt[(c4 + 3) * LDT + r] = kv.w;
      *reinterpret_cast<float4*>(Vs + r * HD + c4) = vv;
    }
    __syncthreads();

    // S = Q K^T for this thread's 4 rows x 4 keys
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll 8
    for (int d = 0; d < HD; ++d) {
      const float4 q4 = *reinterpret_cast<const float4*>(Qt + d * LDT + ty * 4);
      const float4 k4 = *reinterpret_cast<const float4*>(Kt + d * LDT + tx * 4);
      const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] += qa[i] * ka[j];
    }

    // online softmax over the 64 keys of this tile (16 threads share a row)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = q0 + ty * 4 + i;
      float mx = -1e30f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kj = k0 + tx * 4 + j;
        const bool valid = (kj < kvn) && (!causal || kj <= qi);
        s[i][j] = valid ? s[i][j] * scale : -INFINITY;
        if (valid) mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run[i], mx);
      const float corr = expf(m_run[i] - m_new);
      float rs = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = (s[i][j] == -INFINITY) ? 0.0f : expf(s[i][j] - m_new);
        s[i][j] = p;
        rs += p;
      }
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
      l_run[i] = l_run[i] * corr + rs;
      m_run[i] = m_new;
#pragma unroll
      for (int c = 0; c < CPT; ++c) o_acc[i][c] *= corr;
    }
    // P^T to shared memory: Pt[key][row]
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<float4*>(Pt + (tx * 4 + j) * LDT + ty * 4) = make_float4(s[0][j], s[1][j], s[2][j], s[3][j]);
    __syncthreads();

    // O += P V
#pragma unroll 4
    for (int j = 0; j < BKV; ++j) {
      const float4 p4 = *reinterpret_cast<const float4*>(Pt + j * LDT + ty * 4);
      const float pa[4] = {p4.x, p4.y, p4.z, p4.w};
      float va[CPT];
#pragma unroll
      for (int c = 0; c < CPT; c += 2) {
        const float2 v2 = *reinterpret_cast<const float2*>(Vs + j * HD + tx * CPT + c);
        va[c] = v2.x;
        va[c + 1] = v2.y;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < CPT; ++c) o_acc[i][c] += pa[i] * va[c];
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qi = q0 + ty * 4 + i;
    if (qi >= seq) continue;
    const float inv = 1.0f / (l_run[i] + 1e-9f);  // LayerOps.hpp:1076
    float* o = out + (static_cast<long long>(b) * seq + qi) * embed + h * HD + tx * CPT;
#pragma unroll
    for (int c = 0; c < CPT; ++c) o[c] = o_acc[i][c] * inv;
  }
}

// Any head dimension: one CTA per (sample, head, group of AR query rows); the score rows live in shared memory.
// Every K and V row is read once per group (a warp per key computes the AR dot products; a thread per output
// column accumulates the AR weighted sums), which cuts the L2 traffic of the one-row form by AR.
constexpr int AR = 8;

__global__ void attn_row_kernel(const AttnView a, float* __restrict__ out, int embed, int heads, int hd, int causal, float scale) {
  extern __shared__ __align__(16) float sm[];
  float* q = sm;               // [AR][hd]
  float* p = sm + AR * hd;     // [AR][kv_len]
  __shared__ float red[AR][33];
  const int i0 = blockIdx.x * AR, h = blockIdx.y, b = blockIdx.z;
  const int seq = a.q_len, kvn = a.kv_len;
  const int nr = min(AR, seq - i0);  // query rows of this group
  const long long ld = a.ldkv;
  const long long qbs = a.q_bstride ? a.q_bstride : seq * a.ldq, kbs = a.kv_bstride ? a.kv_bstride : kvn * ld;
  const float* kb = a.k + b * kbs + h * hd;
  const float* vb = a.v + b * kbs + h * hd;
  for (int t = threadIdx.x; t < AR * hd; t += blockDim.x) {
    const int r = t / hd, d = t - r * hd;
    q[t] = (r < nr) ? a.q[b * qbs + (i0 + r) * a.ldq + h * hd + d] : 0.0f;
  }
  __syncthreads();
  // keys this group can see: row i0 + r sees min(i0 + r + 1, kvn) of them under the causal mask
  const int n_keys = causal ? min(i0 + nr, kvn) : kvn;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float mx[AR];
#pragma unroll
  for (int r = 0; r < AR; ++r) mx[r] = -1e30f;
  constexpr int KU = 4;  // keys per warp and pass: their K rows are loaded together, so four loads are in flight per lane
  for (int j0 = w * KU; j0 < n_keys; j0 += nw * KU) {  // a warp per key: coalesced reads of the K rows
    float dot[KU][AR];
#pragma unroll
    for (int u = 0; u < KU; ++u)
#pragma unroll
      for (int r = 0; r < AR; ++r) dot[u][r] = 0.0f;
    for (int d = lane; d < hd; d += 32) {
      float kv[KU];
#pragma unroll
      for (int u = 0; u < KU; ++u) kv[u] = (j0 + u < n_keys) ? __ldg(kb + static_cast<long long>(j0 + u) * ld + d) : 0.0f;
#pragma unroll
      for (int r = 0; r < AR; ++r) {
        const float qv = q[r * hd + d];
#pragma unroll
        for (int u = 0; u < KU; ++u) dot[u][r] += qv * kv[u];
      }
    }
#pragma unroll
    for (int u = 0; u < KU; ++u) {
      const int j = j0 + u;
      if (j >= n_keys) break;
#pragma unroll
      for (int r = 0; r < AR; ++r) {
        float dv = dot[u][r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dv += __shfl_xor_sync(0xffffffffu, dv, o);
        const bool visible = !causal || j <= i0 + r;
        const float sc = dv * scale;
        if (lane == 0) p[r * kvn + j] = visible ? sc : -INFINITY;  // exp(-inf - max) = 0, like the reference's -1e9
        if (visible) mx[r] = fmaxf(mx[r], sc);
      }
    }
  }
  // block max per row
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < AR; ++r) red[r][w] = mx[r];
  }
  __syncthreads();
  if (w < AR) {
    float t = (lane < nw) ? red[w][lane] : -1e30f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (lane == 0) red[w][32] = t;
  }
  __syncthreads();
  float acc[AR];
#pragma unroll
  for (int r = 0; r < AR; ++r) {
    acc[r] = 0.0f;
    const float m = red[r][32];
    for (int j = threadIdx.x; j < n_keys; j += blockDim.x) {
      const float e = expf(p[r * kvn + j] - m);
      p[r * kvn + j] = e;
      acc[r] += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
  }
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < AR; ++r) red[r][w] = acc[r];
  }
  __syncthreads();
  if (w < AR) {
    float t = (lane < nw) ? red[w][lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[w][32] = t;
  }
  __syncthreads();
  // O = P V.  A thread owns one output column; when the head is narrower than the CTA the keys are dealt to
  // G = blockDim / hd groups of threads whose partial sums meet in shared memory (the Q rows there are dead by
  // now) in group order, so the result does not depend on timing.  Four V loads are in flight per thread.
  const int G = (hd < static_cast<int>(blockDim.x)) ? static_cast<int>(blockDim.x) / hd : 1;
  const int g = static_cast<int>(threadIdx.x) / hd;
  float* accs = q;  // [AR][hd]
  for (int d0 = 0; d0 < hd; d0 += blockDim.x) {
    const int d = (G > 1) ? static_cast<int>(threadIdx.x) - g * hd : d0 + static_cast<int>(threadIdx.x);
    const bool active = (G > 1) ? (g < G) : (d < hd);
    float o[AR];
#pragma unroll
    for (int r = 0; r < AR; ++r) o[r] = 0.0f;
    if (active) {
      const float* vr = vb + d;
      int j = g;
      for (; j + 3 * G < n_keys; j += 4 * G) {
        const float v0 = __ldg(vr + static_cast<long long>(j) * ld), v1 = __ldg(vr + static_cast<long long>(j + G) * ld),
                    v2 = __ldg(vr + static_cast<long long>(j + 2 * G) * ld), v3 = __ldg(vr + static_cast<long long>(j + 3 * G) * ld);
#pragma unroll
        for (int r = 0; r < AR; ++r) {
          const float* pr = p + r * kvn + j;
          o[r] += pr[0] * v0;
          o[r] += pr[G] * v1;
          o[r] += pr[2 * G] * v2;
          o[r] += pr[3 * G] * v3;
        }
      }
      for (; j < n_keys; j += G) {
        const float v = __ldg(vr + static_cast<long long>(j) * ld);
#pragma unroll
        for (int r = 0; r < AR; ++r) o[r] += p[r * kvn + j] * v;
      }
    }
    if (G > 1) {
      for (int gg = 0; gg < G; ++gg) {
        __syncthreads();
        if (active && g == gg) {
#pragma unroll
          for (int r = 0; r < AR; ++r) accs[r * hd + d] = (gg == 0) ? o[r] : accs[r * hd + d] + o[r];
        }
      }
      __syncthreads();
      if (active && g == 0) {
#pragma unroll
        for (int r = 0; r < AR; ++r) o[r] = accs[r * hd + d];
      }
    }
    if (active && (G == 1 || g == 0)) {
#pragma unroll
      for (int r = 0; r < AR; ++r)
        if (r < nr) out[(static_cast<long long>(b) * seq + i0 + r) * embed + h * hd + d] = o[r] * (1.0f / (red[r][32] + 1e-9f));
    }
  }
}

template <int HD>
int launch_flash(const AttnView& a, float* out, int batch, int embed, int heads, int causal, float scale, cudaStream_t st) {
  constexpr int SMEM = (2 * HD * LDT + BKV * HD + BKV * LDT) * 4;
  static PerDeviceOnce attr_once;
  MB_TRY(attr_once.run([&]() -> int {
    MB_CUDA(cudaFuncSetAttribute(flash_attn_fp32_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    return MIMIR_B200_OK;
  }));
  dim3 grid((a.q_len + BQ - 1) / BQ, heads, batch);
  flash_attn_fp32_kernel<HD><<<grid, 256, SMEM, st>>>(a, out, embed, heads, causal, scale);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

}  // namespace

int launch_attention_core_view(const AttnView& a, float* out, int batch, int embed, int heads, int causal, cudaStream_t st) {
  if (batch <= 0 || a.q_len <= 0 || a.kv_len <= 0 || embed <= 0 || heads <= 0 || embed % heads != 0)
    return fail(MIMIR_B200_E_INVALID, "Attention: embed_dim must be divisible by num_heads");
  const int hd = embed / heads;
  const float scale = 1.0f / sqrtf(static_cast<float>(hd));
  const bool aligned = (((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15) == 0) &&
                       (embed % 4 == 0) && (a.ldq % 4 == 0) && (a.ldkv % 4 == 0) && batch <= 65535 && heads <= 65535;
  // a query tile of 64 rows would be almost empty for a decode step: the row kernel reads K and V once, a warp per key
  const bool few_rows = a.q_len <= 2 && static_cast<size_t>(AR) * (hd + a.kv_len) * 4 <= 200 * 1024;
  if (!few_rows) {
    if (aligned && hd == 32) return launch_flash<32>(a, out, batch, embed, heads, causal, scale, st);
    if (aligned && hd == 64) return launch_flash<64>(a, out, batch, embed, heads, causal, scale, st);
    if (aligned && hd == 128) return launch_flash<128>(a, out, batch, embed, heads, causal, scale, st);
  }
  const size_t smem = static_cast<size_t>(AR) * (hd + a.kv_len) * 4;
  if (smem > 200 * 1024 || batch > 65535 || heads > 65535)
    return fail(MIMIR_B200_E_UNSUPPORTED, "attention: %d keys with head_dim %d exceed the row kernel's shared memory", a.kv_len, hd);
  static PerDeviceOnce attr_once;  // the largest size the launcher admits, once per device
  MB_TRY(attr_once.run([&]() -> int {
    MB_CUDA(cudaFuncSetAttribute(attn_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    return MIMIR_B200_OK;
  }));
  dim3 grid((a.q_len + AR - 1) / AR, heads, batch);
  attn_row_kernel<<<grid, 256, smem, st>>>(a, out, embed, heads, hd, causal, scale);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

namespace {
__global__ void kv_cache_write_kernel(const float* __restrict__ qkv, float* __restrict__ kcache, float* __restrict__ vcache, long long total,
                                      int seq, int embed, int max_seq, int pos0, const int* __restrict__ pos_dev) {
  if (pos_dev) pos0 = *pos_dev;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(i % embed);
    const long long row = i / embed;  // b * seq + s
    const long long b = row / seq, s = row - b * seq;
    const long long dst = (b * max_seq + pos0 + s) * embed + d;
    kcache[dst] = __ldg(qkv + row * 3 * embed + embed + d);
    vcache[dst] = __ldg(qkv + row * 3 * embed + 2 * embed + d);
  }
}
}  // namespace

// ---- one query row per (sample, head) against a long key / value cache: the decode step ---------------
// The keys are cut into chunks of 128; a CTA of 128 threads takes one chunk of one (sample, head): a thread per key
// computes the score with 128-bit loads along its own K row (every load independent: hd / 4 in flight per
// thread), the chunk's softmax terms go through shared memory, then the threads regroup as (quad of output
// columns, key group) to accumulate P V with coalesced 128-bit loads of the V rows.  Each chunk leaves
// (max, sum, unnormalised O) in a scratch; a second kernel merges the chunks in chunk order.
namespace {
constexpr int DEC_CHUNK = 128;

__global__ void __launch_bounds__(DEC_CHUNK) attn_decode_chunk_kernel(const AttnView a, float* __restrict__ scratch, int heads, int hd,
                                                                     float scale) {
  extern __shared__ __align__(16) float dsm[];
  float* q = dsm;                  // [hd]
  float* pj = dsm + hd;            // [DEC_CHUNK]
  float* part = pj + DEC_CHUNK;    // [groups][hd]
  __shared__ float red[33];
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z, t = threadIdx.x;
  const int kvn = a.pos_dev ? (*a.pos_dev + 1) : a.kv_len, k0 = chunk * DEC_CHUNK;
  if (k0 >= kvn) return;  // (the launch is sized for the whole cache when the position comes from device memory)
  const int nk = min(DEC_CHUNK, kvn - k0);
  const long long ld = a.ldkv;
  const long long qbs = a.q_bstride ? a.q_bstride : a.q_len * a.ldq, kbs = a.kv_bstride ? a.kv_bstride : static_cast<long long>(a.kv_len) * ld;
  const float* kb = a.k + b * kbs + h * hd + static_cast<long long>(k0) * ld;
  const float* vb = a.v + b * kbs + h * hd + static_cast<long long>(k0) * ld;
  for (int d = t; d < hd; d += DEC_CHUNK) q[d] = a.q[b * qbs + h * hd + d];
  __syncthreads();
  const int nq = hd >> 2;
  float sc = -1e30f;
  if (t < nk) {
    const float4* kr = reinterpret_cast<const float4*>(kb + static_cast<long long>(t) * ld);
    float dot = 0.0f;
    for (int c0 = 0; c0 < nq; c0 += 8) {  // eight loads ahead of their use; d ascending like the reference's dot product
      float4 kv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) kv[u] = (c0 + u < nq) ? __ldg(kr + c0 + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (c0 + u < nq) {
          const float4 qv = *reinterpret_cast<const float4*>(q + 4 * (c0 + u));
          dot += qv.x * kv[u].x; dot += qv.y * kv[u].y; dot += qv.z * kv[u].z; dot += qv.w * kv[u].w;
        }
      }
    }
    sc = dot * scale;
  }
  // chunk maximum and sum (128 threads = 4 warps)
  float mx = sc;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((t & 31) == 0) red[t >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const float pv = (t < nk) ? expf(sc - mx) : 0.0f;
  pj[t] = pv;
  float sum = pv;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncthreads();  // red[] read by everybody, pj[] written
  if ((t & 31) == 0) red[8 + (t >> 5)] = sum;
  __syncthreads();
  sum = (red[8] + red[9]) + (red[10] + red[11]);
  // P V: thread = (column quad c, key group g)
  const int groups = (nq <= DEC_CHUNK) ? DEC_CHUNK / nq : 1;
  for (int c0 = 0; c0 < nq; c0 += DEC_CHUNK) {
    const int g = (groups > 1) ? t / nq : 0;
    const int c = (groups > 1) ? t - g * nq : c0 + t;
    const bool active = (groups > 1) ? (g < groups) : (c < nq);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
      const float4* vr = reinterpret_cast<const float4*>(vb) + c;
      const long long ld4 = ld >> 2;
      int j = g;
      for (; j + 7 * groups < nk; j += 8 * groups) {
        float4 vv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) vv[u] = __ldg(vr + static_cast<long long>(j + u * groups) * ld4);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float w = pj[j + u * groups];
          acc.x += w * vv[u].x; acc.y += w * vv[u].y; acc.z += w * vv[u].z; acc.w += w * vv[u].w;
        }
      }
      for (; j < nk; j += groups) {
        const float4 v4 = __ldg(vr + static_cast<long long>(j) * ld4);
        const float w = pj[j];
        acc.x += w * v4.x; acc.y += w * v4.y; acc.z += w * v4.z; acc.w += w * v4.w;
      }
      if (groups > 1) *reinterpret_cast<float4*>(part + g * hd + 4 * c) = acc;
    }
    float* dst = scratch + (((static_cast<long long>(b) * heads + h) * gridDim.x + chunk) * (hd + 2));
    if (groups > 1) {
      __syncthreads();
      if (t < nq) {
        float4 o = *reinterpret_cast<const float4*>(part + 4 * t);
        for (int gg = 1; gg < groups; ++gg) {
          const float4 x = *reinterpret_cast<const float4*>(part + gg * hd + 4 * t);
          o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
        }
        dst[2 + 4 * t] = o.x; dst[3 + 4 * t] = o.y; dst[4 + 4 * t] = o.z; dst[5 + 4 * t] = o.w;
      }
    } else if (active) {
      dst[2 + 4 * c] = acc.x; dst[3 + 4 * c] = acc.y; dst[4 + 4 * c] = acc.z; dst[5 + 4 * c] = acc.w;
    }
    if (t == 0 && c0 == 0) { dst[0] = mx; dst[1] = sum; }
  }
}

__global__ void attn_decode_merge_kernel(const float* __restrict__ scratch, float* __restrict__ out, int chunks_launched, int heads, int hd,
                                         int embed, const int* __restrict__ pos_dev) {
  const int h = blockIdx.x, b = blockIdx.y;
  const float* src = scratch + (static_cast<long long>(b) * heads + h) * chunks_launched * (hd + 2);
  const int chunks = pos_dev ? (*pos_dev + DEC_CHUNK) / DEC_CHUNK : chunks_launched;
  float m = -1e30f;  // the reference's initial maximum (LayerOps.hpp:1052)
  for (int c = 0; c < chunks; ++c) m = fmaxf(m, src[static_cast<long long>(c) * (hd + 2)]);
  float l = 0.0f;
  for (int c = 0; c < chunks; ++c) l += src[static_cast<long long>(c) * (hd + 2) + 1] * expf(src[static_cast<long long>(c) * (hd + 2)] - m);
  const float inv = 1.0f / (l + 1e-9f);  // LayerOps.hpp:1076
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.0f;
    for (int c = 0; c < chunks; ++c) o += src[static_cast<long long>(c) * (hd + 2) + 2 + d] * expf(src[static_cast<long long>(c) * (hd + 2)] - m);
    out[static_cast<long long>(b) * embed + h * hd + d] = o * inv;
  }
}
}  // namespace

size_t attention_decode_scratch_bytes(int batch, int heads, int embed, int max_seq) {
  const size_t chunks = static_cast<size_t>((max_seq + DEC_CHUNK - 1) / DEC_CHUNK);
  return static_cast<size_t>(batch) * heads * chunks * (static_cast<size_t>(embed / (heads > 0 ? heads : 1)) + 2) * sizeof(float);
}

bool attention_decode_supported(const AttnView& a, int embed, int heads) {
  if (heads <= 0 || embed % heads != 0) return false;
  const int hd = embed / heads;
  return a.q_len == 1 && hd % 4 == 0 && hd <= 512 && a.ldkv % 4 == 0 && a.kv_bstride % 4 == 0 &&
         ((reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v)) & 15) == 0;
}

// out [batch][embed]; `scratch` holds attention_decode_scratch_bytes(batch, heads, embed, kv_len)
int launch_attention_decode(const AttnView& a, float* out, float* scratch, int batch, int embed, int heads, cudaStream_t st) {
  if (!attention_decode_supported(a, embed, heads) || !scratch) return fail(MIMIR_B200_E_INVALID, "attention decode: unsupported layout");
  const int hd = embed / heads;
  const int chunks = (a.kv_len + DEC_CHUNK - 1) / DEC_CHUNK;
  if (chunks > 65535 || heads > 65535 || batch > 65535) return fail(MIMIR_B200_E_UNSUPPORTED, "attention decode: too many chunks / heads / samples for one launch");
  const int nq = hd / 4;
  const int groups = (nq <= DEC_CHUNK) ? DEC_CHUNK / nq : 1;
  const size_t smem = (static_cast<size_t>(hd) + DEC_CHUNK + static_cast<size_t>(groups) * hd) * sizeof(float);
  dim3 grid(chunks, heads, batch);
  attn_decode_chunk_kernel<<<grid, DEC_CHUNK, smem, st>>>(a, scratch, heads, hd, 1.0f / sqrtf(static_cast<float>(hd)));
  MB_CUDA(cudaGetLastError());
  dim3 mgrid(heads, batch);
  attn_decode_merge_kernel<<<mgrid, 128, 0, st>>>(scratch, out, chunks, heads, hd, embed, a.pos_dev);
  MB_CUDA(cudaGetLastError());
  count_launch(2);
  return MIMIR_B200_OK;
}

int launch_kv_cache_write(const float* qkv, float* kcache, float* vcache, int batch, int seq, int embed, int max_seq, int pos0,
                          cudaStream_t st, const int* pos_dev) {
  if (pos0 < 0 || pos0 + seq > max_seq) return fail(MIMIR_B200_E_INVALID, "KV cache: positions %d..%d exceed the cache of %d", pos0, pos0 + seq - 1, max_seq);
  const long long total = static_cast<long long>(batch) * seq * embed;
  long long blocks = (total + 255) / 256;
  if (blocks > ctx().sm_count * 16LL) blocks = ctx().sm_count * 16LL;
  kv_cache_write_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(qkv, kcache, vcache, total, seq, embed, max_seq, pos0, pos_dev);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_attention_core(const float* qkv, float* out, int batch, int seq, int embed, int heads, int causal,
                          cudaStream_t st) {
  if (batch <= 0 || seq <= 0 || embed <= 0 || heads <= 0 || embed % heads != 0)
    return fail(MIMIR_B200_E_INVALID, "SelfAttention: embed_dim must be divisible by num_heads");
  AttnView a;
  a.q = qkv; a.k = qkv + embed; a.v = qkv + 2 * embed;
  a.ldq = a.ldkv = 3LL * embed;
  a.q_len = a.kv_len = seq;
  return launch_attention_core_view(a, out, batch, embed, heads, causal, st);
}

}  // namespace mb
