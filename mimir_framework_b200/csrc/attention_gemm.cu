// attention_gemm.cu — the attention core of a single wide head (head_dim a multiple of 64 other than 64, e.g. the 512-wide
// head of a UNet mid block) on the tensor cores, as two block-diagonal GEMMs around a row softmax.
// Replaces steps 3-5 of LayerOps::self_attention_forward (LayerOps.hpp:1044-1090) for num_heads = 1:
//   S_b = Q_b K_b^T        one grouped GEMM launch over all samples (gemm_sm100.cu, grouped form), fp32 scores [B*S][S]
//   P   = softmax(S * scale) per row: causal rows skip j > i (the reference scores them -1e9 and keeps them out of the
//         maximum), p = exp(s - max), p *= 1 / (sum p + 1e-9)                                    (this file)
//   O_b = P_b V_b          a second grouped launch against the per-sample transposed V; its epilogue writes the operand
//         planes of the output projection.
// Every operand travels as hi + lo 16-bit planes and every product is taken with three MMAs (both sides are data, nothing
// is exact in one plane), so the result sits inside the same tolerance as the fp32 row kernel it replaces.
#include "common.h"
#include "ops.h"
#include "planes.cuh"

namespace mb {
namespace {

// Q and K planes [rows][E] out of the fp32 QKV rows [rows][3E]; one thread per 16-byte chunk (8 values) of Q or K
__global__ void attn_qk_planes_kernel(const float* __restrict__ qkv, __nv_bfloat16* __restrict__ qp, __nv_bfloat16* __restrict__ kp,
                                      long long rows, int E, int f16) {
  const int chunks = E >> 3;
  const long long total = rows * chunks * 2;
  const long long plane_stride = rows * static_cast<long long>(E);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long rc = i >> 1;
    const int which = static_cast<int>(i & 1);  // 0 = Q, 1 = K (neighbouring threads share the row's cache lines)
    const long long r = rc / chunks;
    const int c = static_cast<int>(rc - r * chunks) << 3;
    const float* s = qkv + r * 3 * E + which * E + c;
    const float4 a = __ldg(reinterpret_cast<const float4*>(s)), b = __ldg(reinterpret_cast<const float4*>(s + 4));
    uint32_t h[4], l[4];
    split_pair(a.x, a.y, f16, h[0], l[0]);
    split_pair(a.z, a.w, f16, h[1], l[1]);
    split_pair(b.x, b.y, f16, h[2], l[2]);
    split_pair(b.z, b.w, f16, h[3], l[3]);
    __nv_bfloat16* d = (which ? kp : qp) + r * E + c;
    *reinterpret_cast<uint4*>(d) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(d + plane_stride) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// V^T planes [B*E][S]: row b*E + e holds V[b*S + s][e] over s.  32 x 32 tiles through shared memory.
__global__ void attn_vt_planes_kernel(const float* __restrict__ qkv, __nv_bfloat16* __restrict__ vt, int batch, int S, int E, int f16) {
  __shared__ float tile[32][33];
  const int s0 = blockIdx.x * 32, e0 = blockIdx.y * 32, b = blockIdx.z;
  for (int i = threadIdx.y; i < 32; i += blockDim.y)
    tile[i][threadIdx.x] = __ldg(qkv + (static_cast<long long>(b) * S + s0 + i) * 3 * E + 2 * E + e0 + threadIdx.x);
  __syncthreads();
  const long long plane_stride = static_cast<long long>(batch) * E * S;
  uint16_t* d16 = reinterpret_cast<uint16_t*>(vt);
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    uint16_t h, l;
    split_one(tile[threadIdx.x][i], f16, h, l);
    const long long o = (static_cast<long long>(b) * E + e0 + i) * S + s0 + threadIdx.x;
    d16[o] = h;
    d16[o + plane_stride] = l;
  }
}

// One warp per score row: the reference's softmax (LayerOps.hpp:1052-1080) and the hi / lo planes of the probabilities.
__global__ void attn_softmax_planes_kernel(const float* __restrict__ scores, __nv_bfloat16* __restrict__ p, long long rows, int S,
                                           int causal, float scale, int f16) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long plane_stride = rows * static_cast<long long>(S);
  for (long long r = warp; r < rows; r += nwarps) {
    const int qi = static_cast<int>(r % S);  // position of this query row inside its sample
    const int valid = causal ? qi + 1 : S;   // keys 0 .. valid-1 take part
    const float* srow = scores + r * S;
    float mx = -1e30f;  // the reference's initial maximum
    for (int j = 2 * lane; j < valid; j += 64) {
      const float2 v = __ldg(reinterpret_cast<const float2*>(srow + j));
      mx = fmaxf(mx, v.x * scale);
      if (j + 1 < valid) mx = fmaxf(mx, v.y * scale);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    for (int j = 2 * lane; j < valid; j += 64) {
      const float2 v = __ldg(reinterpret_cast<const float2*>(srow + j));
      sum += expf(v.x * scale - mx);
      if (j + 1 < valid) sum += expf(v.y * scale - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / (sum + 1e-9f);
    for (int j = 2 * lane; j < S; j += 64) {
      float p0 = 0.0f, p1 = 0.0f;
      if (j < valid) {
        const float2 v = __ldg(reinterpret_cast<const float2*>(srow + j));
        p0 = expf(v.x * scale - mx) * inv;
        if (j + 1 < valid) p1 = expf(v.y * scale - mx) * inv;
      }
      uint32_t h, l;
      split_pair(p0, p1, f16, h, l);
      *reinterpret_cast<uint32_t*>(p + r * S + j) = h;
      *reinterpret_cast<uint32_t*>(p + r * S + j + plane_stride) = l;
    }
  }
}

size_t planes2(long long rows, long long k) { return align256(static_cast<size_t>(2) * rows * k * sizeof(__nv_bfloat16)); }

}  // namespace

bool attention_gemm_supported(int batch, int seq, int embed, int heads) {
  static const bool off = [] { const char* e = getenv("MIMIR_B200_ATTN_GEMM"); return e && e[0] == '0'; }();
  // one head; whole 128-row tiles per sample (a tile never straddles two samples); K dimensions whole 64-blocks
  return !off && heads == 1 && embed % 64 == 0 && embed > 64 && seq % 128 == 0 && seq <= 4096 && batch >= 1 && batch <= 65535 &&
         static_cast<long long>(batch) * seq * seq * 4 <= (1ll << 31);
}

size_t attention_gemm_ws_bytes(int batch, int seq, int embed) {
  const long long rows = static_cast<long long>(batch) * seq;
  return 2 * planes2(rows, embed) + planes2(static_cast<long long>(batch) * embed, seq) + align256(static_cast<size_t>(rows) * seq * 4) +
         planes2(rows, seq);
}

// qkv: fp32 [batch*seq][3*embed]; out_split: planes [2][batch*seq][embed] (the output projection's operand); `out_planes`
// of them are read by the consumer, both are written.
int launch_attention_core_gemm(const float* qkv, int batch, int seq, int embed, int causal, void* ws, __nv_bfloat16* out_split,
                               cudaStream_t st) {
  if (!attention_gemm_supported(batch, seq, embed, 1)) return fail(MIMIR_B200_E_UNSUPPORTED, "attention: shape not taken by the GEMM form");
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) != 0) return fail(MIMIR_B200_E_INVALID, "attention: QKV rows not 16-byte aligned");
  const long long rows = static_cast<long long>(batch) * seq;
  const int f16 = plane_format() == PLANES_F16 ? 1 : 0;
  uint8_t* w8 = static_cast<uint8_t*>(ws);
  __nv_bfloat16* qp = reinterpret_cast<__nv_bfloat16*>(w8);
  __nv_bfloat16* kp = reinterpret_cast<__nv_bfloat16*>(w8 + planes2(rows, embed));
  __nv_bfloat16* vt = reinterpret_cast<__nv_bfloat16*>(w8 + 2 * planes2(rows, embed));
  float* scores = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(vt) + planes2(static_cast<long long>(batch) * embed, seq));
  __nv_bfloat16* pp = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(scores) + align256(static_cast<size_t>(rows) * seq * 4));
  {
    const long long total = rows * (embed >> 3) * 2;
    const long long blocks = std::min<long long>((total + 255) / 256, static_cast<long long>(ctx().sm_count) * 16);
    attn_qk_planes_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(qkv, qp, kp, rows, embed, f16);
    MB_CUDA(cudaGetLastError());
    attn_vt_planes_kernel<<<dim3(seq / 32, embed / 32, batch), dim3(32, 8), 0, st>>>(qkv, vt, batch, seq, embed, f16);
    MB_CUDA(cudaGetLastError());
    count_launch(2);
  }
  GemmArgs s;
  s.a = qp; s.w = kp; s.a_planes = 2; s.w_planes = 2;
  s.m = static_cast<int>(rows); s.n = seq; s.k = embed;
  s.out_f32 = scores; s.ldo = seq;
  s.a_group_rows = seq; s.w_group_rows = seq; s.w_rows_total = rows;
  MB_TRY(launch_gemm(s, st));
  {
    const long long blocks = std::min<long long>((rows * 32 + 255) / 256, static_cast<long long>(ctx().sm_count) * 16);
    attn_softmax_planes_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(scores, pp, rows, seq, causal,
                                                                             1.0f / sqrtf(static_cast<float>(embed)), f16);
    MB_CUDA(cudaGetLastError());
    count_launch();
  }
  GemmArgs o;
  o.a = pp; o.w = vt; o.a_planes = 2; o.w_planes = 2;
  o.m = static_cast<int>(rows); o.n = embed; o.k = seq;
  o.out_split = out_split;
  o.a_group_rows = seq; o.w_group_rows = embed; o.w_rows_total = static_cast<long long>(batch) * embed;
  return launch_gemm(o, st);
}

}  // namespace mb
