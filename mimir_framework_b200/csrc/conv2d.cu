// conv2d.cu — Conv2d lowered to the tensor-core GEMM.  Replaces the inline Conv2d case of the
// layer switch (Model.cpp:4897-5089): CHW activations, OIHW weights, square kernel, zero padding,
// no bias.  The reference itself computes im2col rows ordered (ic, kh, kw) (Model.cpp:5005-5029)
// times the transposed weights (Model.cpp:5032); here the im2col rows are produced directly as the
// bf16 hi/lo planes the GEMM consumes (one pass over the input, no fp32 column matrix), the OIHW
// weight block already is the K-major [oc][ic*k*k] operand, and the GEMM epilogue writes NCHW.
#include "common.h"

namespace mb {
namespace {

// One thread produces 8 consecutive K entries of one output pixel.
__global__ void im2col_split_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ dst, long long rows, int ic, int h,
                                    int w, int ks, int stride, int pad, int oh, int ow, int k, int kp, int planes) {
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
    __align__(16) __nv_bfloat16 hi[8];
    __align__(16) __nv_bfloat16 lo[8];
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
      hi[j] = __float2bfloat16_rn(v);
      lo[j] = __float2bfloat16_rn(v - __bfloat162float(hi[j]));
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
  im2col_split_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(x, dst, rows, ic, h, w, ks, stride, pad, oh, ow, k, kp, planes);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

}  // namespace mb
