// conv2d.cu — Conv2d lowered to the tensor-core GEMM.  Replaces the inline Conv2d case of the
// layer switch (Model.cpp:4897-5089): CHW activations, OIHW weights, square kernel, zero padding,
// no bias.  The reference itself computes im2col rows ordered (ic, kh, kw) (Model.cpp:5005-5029)
// times the transposed weights (Model.cpp:5032); here the im2col rows are produced directly as the
// bf16 hi/lo planes the GEMM consumes (one pass over the input, no fp32 column matrix), the OIHW
// weight block already is the K-major [oc][ic*k*k] operand, and the GEMM epilogue writes NCHW.
#include "common.h"
#include "planes.cuh"

namespace mb {
namespace {

// One thread produces 8 consecutive K entries of one output pixel.
__global__ void im2col_split_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ dst, long long rows, int ic, int h,
                                    int w, int ks, int stride, int pad, int oh, int ow, int k, int kp, int planes, int f16) {
  const int chunks = kp >> 3;
  const long long total = rows * chunks;
  const long long plane_stride = rows * static_cast<long long>(kp);
  const int ohw = oh * ow, kk = ks * ks;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    // consecutive threads write consecutive 16-byte chunks of one im2col row (coalesced stores, the
    // larger stream); the input, 1/k^2 of the size, is re-read through L1/L2
    const long long r = i / chunks;
    const int c = static_cast<int>(i - r * chunks);
    const long long smp = r / ohw;
    const int pix = static_cast<int>(r - smp * ohw);
    const int oy = pix / ow, ox = pix - oy * ow;
    const float* xs = x + smp * ic * h * w;
    __align__(16) uint16_t hi[8];
    __align__(16) uint16_t lo[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int kidx = c * 8 + j;
      float v = 0.0f;
      if (kidx < k) {
        const int ci = kidx / kk, t = kidx - ci * kk;
        const int ky = t / ks, kx = t - ky * ks;
        const int iy = oy * stride + ky - pad, ix = ox * stride + kx - pad;
        if (iy >= 0 && iy < h && ix >= 0 && ix < w) v = __ldg(xs + (static_cast<long long>(ci) * h + iy) * w + ix);
      }
      split_one(v, f16, hi[j], lo[j]);
    }
    __nv_bfloat16* d = dst + r * kp + c * 8;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(hi);
    if (planes == 2) *reinterpret_cast<uint4*>(d + plane_stride) = *reinterpret_cast<const uint4*>(lo);
  }
}

}  // namespace

int launch_im2col_split(const float* x, __nv_bfloat16* dst, int batch, int ic, int h, int w, int ks, int stride, int pad,
                        int oh, int ow, int planes, cudaStream_t st) {
  if (batch <= 0 || ic <= 0 || oh <= 0 || ow <= 0 || ks <= 0 || stride <= 0)
    return fail(MIMIR_B200_E_INVALID, "Conv2d: in_channels and out_channels must be set");
  const int k = ic * ks * ks, kp = round_up(k, 64);
  const long long rows = static_cast<long long>(batch) * oh * ow;
  const long long total = rows * (kp >> 3);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(ctx().sm_count) * 32;
  if (blocks > cap) blocks = cap;
  im2col_split_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(x, dst, rows, ic, h, w, ks, stride, pad, oh, ow, k, kp, planes, plane_format() == PLANES_F16);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

}  // namespace mb

// ---------------------------------------------------------------------------------------------
// Stride-1 "same" convolutions without a materialised im2col: the GEMM kernel sums one shifted
// GEMM per filter tap over the zero-padded NHWC activation matrix (see GemmParams::conv_*).  The
// two kernels below produce its operands.
// ---------------------------------------------------------------------------------------------
namespace mb {
namespace {

// One CTA per (sample, padded row yp, 64-channel block): 64 x 64 tiles through shared memory turn the
// W-contiguous NCHW rows into C-contiguous NHWC pixels; border pixels are written as zeros.  Sixteen
// coalesced loads are in flight per thread; on the way out a lane owns a channel pair, so a warp writes
// 128 contiguous bytes per pixel and plane as packed bf16x2.
constexpr int TP_C = 64, TP_X = 64;

__global__ void __launch_bounds__(256) nchw_to_padded_nhwc_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ dst,
                                                                  int c, int h, int w, int pad, int planes, long long plane_stride,
                                                                  const PreNorm pre, int f16) {
  __shared__ float tile[TP_C][TP_X + 1];
  const int hp = h + 2 * pad, wp = w + 2 * pad;
  const int cb = blockIdx.x * TP_C;
  const int yp = blockIdx.y;
  const int n = blockIdx.z;
  const int y = yp - pad;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool row_in = y >= 0 && y < h;
  const float* src = x + ((static_cast<long long>(n) * c + cb) * h + (row_in ? y : 0)) * w;
  const long long ch_stride = static_cast<long long>(h) * w;
  // this thread's 16 elements of a tile belong to 16 fixed channels: their scale / shift once per CTA
  float sc[16], sh[16];
  if (pre.stats != nullptr) {
    const int cpg = c / pre.groups;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int ch = cb + ((threadIdx.x + 256 * i) >> 6);
      sc[i] = 0.0f; sh[i] = 0.0f;
      if (ch < c) {
        const float* st = pre.stats + (static_cast<long long>(n) * pre.groups + ch / cpg) * 2;
        const float mean = __ldg(st), inv = __ldg(st + 1);
        const float g = pre.gamma != nullptr ? __ldg(pre.gamma + ch) : 1.0f;
        const float b = (pre.gamma != nullptr && pre.beta != nullptr) ? __ldg(pre.beta + ch) : 0.0f;
        sc[i] = inv * g;
        sh[i] = b - mean * inv * g;
      }
    }
  }
  for (int x0 = 0; x0 < wp; x0 += TP_X) {
    // tile[cc][xx] = x[n, cb + cc, y, x0 + xx - pad]; a warp reads 32 consecutive pixels of one channel
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = threadIdx.x + 256 * i;
      const int cc = idx >> 6, xx = idx & 63;
      const int xs = x0 + xx - pad;
      v[i] = (row_in && xs >= 0 && xs < w && cb + cc < c) ? __ldg(src + cc * ch_stride + xs) : 0.0f;
    }
    if (pre.stats != nullptr) {
      // GroupNorm (+ SiLU) of the producer applied here; the zero padding ring stays zero
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int xs = x0 + ((threadIdx.x + 256 * i) & 63) - pad;
        if (row_in && xs >= 0 && xs < w) {  // (channels past c are never stored)
          float r = fmaf(v[i], sc[i], sh[i]);
          if (pre.act == MIMIR_B200_ELT_SILU) r = r * __fdividef(1.0f, 1.0f + __expf(-r));
          v[i] = r;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = threadIdx.x + 256 * i;
      tile[idx >> 6][idx & 63] = v[i];
    }
    __syncthreads();
    const int c0 = cb + 2 * lane;
    if (c0 < c) {  // c is even (a multiple of 32)
#pragma unroll
      for (int i = 0; i < TP_X / 8; ++i) {
        const int xx = warp + 8 * i;
        const int xp = x0 + xx;
        if (xp < wp) {
          const float a = tile[2 * lane][xx], b = tile[2 * lane + 1][xx];
          uint32_t hi, lo;
          split_pair(a, b, f16, hi, lo);
          const long long o = ((static_cast<long long>(n) * hp + yp) * wp + xp) * c + c0;
          *reinterpret_cast<uint32_t*>(dst + o) = hi;
          if (planes == 2) *reinterpret_cast<uint32_t*>(dst + o + plane_stride) = lo;
        }
      }
    }
    __syncthreads();
  }
}

// dst[pl][o][(kh*ks + kw)*ic + i] = split(w[o][i][kh][kw]); the padded tail of K is zero
__global__ void conv_weight_planes_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ dst, int oc, int ic, int ks,
                                          int kp, int planes, int f16, float scale) {
  const int k = ks * ks * ic;
  const long long total = static_cast<long long>(oc) * kp;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(i / kp), kk = static_cast<int>(i - static_cast<long long>(o) * kp);
    float v = 0.0f;
    if (kk < k) {
      const int t = kk / ic, ci = kk - t * ic;
      v = __ldg(w + (static_cast<long long>(o) * ic + ci) * ks * ks + t);
    }
    uint16_t hi, lo;
    split_one(v * scale, f16, hi, lo);
    uint16_t* d16 = reinterpret_cast<uint16_t*>(dst);
    d16[i] = hi;
    if (planes == 2) d16[i + total] = lo;
  }
}

}  // namespace

int launch_nchw_to_padded_nhwc_split(const float* x, __nv_bfloat16* dst, int batch, int c, int h, int w, int pad, int planes,
                                     cudaStream_t st, const PreNorm& pre) {
  if (batch <= 0 || c <= 0 || h <= 0 || w <= 0 || pad < 0) return fail(MIMIR_B200_E_INVALID, "Conv2d: bad activation shape");
  const int hp = h + 2 * pad, wp = w + 2 * pad;
  if (hp > 65535 || batch > 65535) return fail(MIMIR_B200_E_UNSUPPORTED, "Conv2d: image too tall for the layout kernel");
  dim3 grid((c + TP_C - 1) / TP_C, hp, batch);
  if (pre.stats != nullptr && (pre.groups <= 0 || c % pre.groups != 0)) return fail(MIMIR_B200_E_INVALID, "Conv2d: bad fused GroupNorm");
  nchw_to_padded_nhwc_kernel<<<grid, 256, 0, st>>>(x, dst, c, h, w, pad, planes, static_cast<long long>(batch) * hp * wp * c, pre, plane_format() == PLANES_F16);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_conv_weight_planes(const float* w, __nv_bfloat16* dst, int oc, int ic, int ks, int planes, cudaStream_t st, float scale) {
  const int kp = round_up(ks * ks * ic, 64);
  const long long total = static_cast<long long>(oc) * kp;
  long long blocks = (total + 255) / 256;
  if (blocks > ctx().sm_count * 16) blocks = ctx().sm_count * 16;
  conv_weight_planes_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(w, dst, oc, ic, ks, kp, planes, plane_format() == PLANES_F16, scale);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

}  // namespace mb
