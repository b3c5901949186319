// spatial.cu — the remaining cases of the layer switch that are plain gathers over CHW samples or small
// fp32 contractions.  One thread per output element, grid-stride, accumulation in the reference's
// loop order with fused multiply-adds (what its compiler emits), so results agree to the last bits.
//   depthwise_conv2d  : LayerOpsExt::depthwise_conv2d_forward (LayerOpsExt.hpp:442-497), bias when use_bias
//   conv1d            : LayerOpsExt::conv1d_forward (LayerOpsExt.hpp:388-437)
//   conv_transpose2d  : the ConvTranspose2d branch of the Conv2d case (Model.cpp:4946-4953, 5047-5079):
//                       the forward-convolution gather formula evaluated over the transposed-convolution
//                       output size — reproduced as is
//   pool2d            : MaxPool2d (Model.cpp:5508-5559), AvgPool2d (LayerOps.hpp:404-453; divides by
//                       the number of in-bounds taps)
//   pad2d             : zero / reflection / replication (LayerOpsExt.hpp:582-690)
//   pixel_shuffle     : LayerOpsExt.hpp:749-795
//   upsample_bilinear : LayerOps.hpp:833-874 (corner-aligned source index oh*scale) and the half-pixel
//                       variant the reference calls bicubic (LayerOpsExt.hpp:695-744)
//   batch_matmul      : BatchMatMul / MatMul cases (Model.cpp:5847-5898), k-sequential fp32
//   scale_prefix      : the affine step of the inference BatchNorm case (Model.cpp:5411-5416)
#include "common.h"

namespace mb {
namespace {

int grid_of(long long items, int threads) {
  long long b = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(ctx().sm_count) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

#define MB_GRID_STRIDE(i, total)                                                                   \
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < (total);   \
       i += static_cast<long long>(gridDim.x) * blockDim.x)

__global__ void depthwise_conv2d_kernel(const float* __restrict__ x, const float* __restrict__ wt, const float* __restrict__ bias,
                                        float* __restrict__ y, long long planes, int ch, int h, int w, int oh, int ow, int k,
                                        int stride, int pad, int w_count) {
  const long long total = planes * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    const long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    const long long pl = t / oh;
    const int c = static_cast<int>(pl % ch);
    const float* xp = x + pl * h * w;
    float sum = 0.0f;
    for (int kh = 0; kh < k; ++kh) {
      const int ih = r * stride + kh - pad;
      if (ih < 0 || ih >= h) continue;
      for (int kw = 0; kw < k; ++kw) {
        const int iw = q * stride + kw - pad;
        const int wi = c * k * k + kh * k + kw;
        if (iw >= 0 && iw < w && wi < w_count) sum = fmaf(__ldg(xp + ih * w + iw), __ldg(wt + wi), sum);
      }
    }
    if (bias != nullptr) sum += __ldg(bias + c);
    y[i] = sum;
  }
}

__global__ void conv1d_kernel(const float* __restrict__ x, const float* __restrict__ wt, const float* __restrict__ bias,
                              float* __restrict__ y, long long batch, int ic, int oc, int len, int olen, int k, int stride, int pad,
                              int w_count) {
  const long long total = batch * oc * olen;
  MB_GRID_STRIDE(i, total) {
    const int ol = static_cast<int>(i % olen);
    const long long t = i / olen;
    const int o = static_cast<int>(t % oc);
    const long long s = t / oc;
    const float* xs = x + s * ic * len;
    float sum = 0.0f;
    for (int c = 0; c < ic; ++c)
      for (int kk = 0; kk < k; ++kk) {
        const int il = ol * stride + kk - pad;
        const int wi = (o * ic + c) * k + kk;
        if (il >= 0 && il < len && wi < w_count) sum = fmaf(__ldg(xs + c * len + il), __ldg(wt + wi), sum);
      }
    if (bias != nullptr) sum += __ldg(bias + o);
    y[i] = sum;
  }
}

// Conv2d gather formula over an arbitrary output size (used for ConvTranspose2d, whose output size is the
// transposed-convolution one while the taps are gathered like a forward convolution).
__global__ void conv_gather_kernel(const float* __restrict__ x, const float* __restrict__ wt, float* __restrict__ y, long long batch,
                                   int ic, int oc, int h, int w, int oh, int ow, int k, int stride, int pad, int relu) {
  const long long total = batch * oc * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    t /= oh;
    const int o = static_cast<int>(t % oc);
    const long long s = t / oc;
    const float* xs = x + s * ic * h * w;
    float sum = 0.0f;
    for (int c = 0; c < ic; ++c)
      for (int kh = 0; kh < k; ++kh) {
        const int ih = r * stride + kh - pad;
        if (ih < 0 || ih >= h) continue;
        for (int kw = 0; kw < k; ++kw) {
          const int iw = q * stride + kw - pad;
          if (iw >= 0 && iw < w)
            sum = fmaf(__ldg(xs + (c * h + ih) * w + iw), __ldg(wt + ((o * ic + c) * k + kh) * k + kw), sum);
        }
      }
    y[i] = relu ? fmaxf(0.0f, sum) : sum;
  }
}

template <bool MAX>
__global__ void pool2d_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int h, int w, int oh, int ow,
                              int kh_n, int kw_n, int sh, int sw, int ph, int pw) {
  const long long total = planes * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    const long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    const long long pl = t / oh;
    const float* xp = x + pl * h * w;
    float acc = MAX ? -INFINITY : 0.0f;
    int count = 0;
    for (int kh = 0; kh < kh_n; ++kh) {
      const int ih = r * sh + kh - ph;
      if (ih < 0 || ih >= h) continue;
      for (int kw = 0; kw < kw_n; ++kw) {
        const int iw = q * sw + kw - pw;
        if (iw < 0 || iw >= w) continue;
        const float v = __ldg(xp + ih * w + iw);
        if (MAX) acc = fmaxf(acc, v); else acc += v;
        ++count;
      }
    }
    y[i] = MAX ? acc : (count > 0 ? acc / static_cast<float>(count) : 0.0f);
  }
}

// Conv::conv2d (Layers.hpp:611-722): bias and dilation; one thread per output element, fp32 FMAs over (ic, kh, kw)
// ascending like the reference's scalar loop.
__global__ void conv2d_dilated_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                      float* __restrict__ y, int batch, int ic, int oc, int h, int wd, int oh, int ow, int k,
                                      int stride, int pad, int dil) {
  const long long total = static_cast<long long>(batch) * oc * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    t /= oh;
    const int o = static_cast<int>(t % oc);
    const long long n = t / oc;
    const float* xs = x + n * ic * h * wd;
    const float* wo = w + static_cast<long long>(o) * ic * k * k;
    float acc = 0.0f;
    for (int c = 0; c < ic; ++c)
      for (int kh = 0; kh < k; ++kh) {
        const int ih = r * stride - pad + kh * dil;
        if (ih < 0 || ih >= h) continue;
        for (int kw = 0; kw < k; ++kw) {
          const int iw = q * stride - pad + kw * dil;
          if (iw < 0 || iw >= wd) continue;
          acc = fmaf(__ldg(xs + (static_cast<long long>(c) * h + ih) * wd + iw), __ldg(wo + (c * k + kh) * k + kw), acc);
        }
      }
    y[i] = bias != nullptr ? acc + __ldg(bias + o) : acc;
  }
}

// Conv::conv_transpose2d (Layers.hpp:775-818) as a gather: output (oh, ow) receives x[ic][ih][iw] * w[oc][ic][kh][kw] for every
// (ih, kh) with ih * stride + kh - pad == oh (and likewise in x).  Walking ic, ih, iw ascending visits them in the order
// the reference's scatter loop adds them; the sum starts at the bias, as there.
__global__ void conv_transpose2d_scatter_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                float* __restrict__ y, int batch, int ic, int oc, int h, int wd, int oh, int ow, int k,
                                                int stride, int pad) {
  const long long total = static_cast<long long>(batch) * oc * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    t /= oh;
    const int o = static_cast<int>(t % oc);
    const long long n = t / oc;
    const float* xs = x + n * ic * h * wd;
    float acc = bias != nullptr ? __ldg(bias + o) : 0.0f;
    // ih * stride + kh - pad = r with 0 <= kh < k  =>  (r + pad - k + 1) / stride <= ih <= (r + pad) / stride
    const int ih_lo = max(0, (r + pad - k + stride) / stride), ih_hi = min(h - 1, (r + pad) / stride);
    const int iw_lo = max(0, (q + pad - k + stride) / stride), iw_hi = min(wd - 1, (q + pad) / stride);
    for (int c = 0; c < ic; ++c) {
      const float* wc = w + (static_cast<long long>(o) * ic + c) * k * k;
      for (int ih = ih_lo; ih <= ih_hi; ++ih) {
        const int kh = r + pad - ih * stride;
        if (kh < 0 || kh >= k) continue;
        for (int iw = iw_lo; iw <= iw_hi; ++iw) {
          const int kw = q + pad - iw * stride;
          if (kw < 0 || kw >= k) continue;
          acc = fmaf(__ldg(xs + (static_cast<long long>(c) * h + ih) * wd + iw), __ldg(wc + kh * k + kw), acc);
        }
      }
    }
    y[i] = acc;
  }
}

// Normalization::batch_norm with training = true (Layers.hpp:932-970): one CTA per channel; mean, then the biased
// variance around it, over the batch and the spatial positions; then the affine map.
__global__ void __launch_bounds__(256) batchnorm_batchstats_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                   const float* __restrict__ beta, float* __restrict__ y, int batch,
                                                                   int channels, long long spatial, float eps) {
  __shared__ float red[8];
  __shared__ float bc;
  const int c = blockIdx.x;
  const long long per = static_cast<long long>(batch) * spatial;
  auto at = [&](long long j) { return (j / spatial) * channels * spatial + static_cast<long long>(c) * spatial + (j % spatial); };
  auto block_sum = [&](float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();  // the previous broadcast value has been read by everyone
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.0f;
      for (int i = 0; i < 8; ++i) s += red[i];
      bc = s;
    }
    __syncthreads();
    return bc;
  };
  float s = 0.0f;
  for (long long j = threadIdx.x; j < per; j += 256) s += x[at(j)];
  const float mean = block_sum(s) / static_cast<float>(per);
  float v = 0.0f;
  for (long long j = threadIdx.x; j < per; j += 256) {
    const float d = x[at(j)] - mean;
    v = fmaf(d, d, v);
  }
  const float var = block_sum(v) / static_cast<float>(per);
  const float inv = 1.0f / sqrtf(var + eps);
  const float g = __ldg(gamma + c), b = __ldg(beta + c);
  for (long long j = threadIdx.x; j < per; j += 256) {
    const long long idx = at(j);
    y[idx] = (x[idx] - mean) * inv * g + b;
  }
}

// mode 0 = zero, 1 = reflection, 2 = replication
__global__ void pad2d_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int h, int w, int ph, int pw,
                             int mode) {
  const int oh = h + 2 * ph, ow = w + 2 * pw;
  const long long total = planes * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    const long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    const long long pl = t / oh;
    int ih = r - ph, iw = q - pw;
    float v = 0.0f;
    if (mode == 0) {
      if (ih >= 0 && ih < h && iw >= 0 && iw < w) v = __ldg(x + (pl * h + ih) * w + iw);
    } else {
      if (mode == 1) {
        if (ih < 0) ih = -ih;
        if (ih >= h) ih = 2 * h - ih - 2;
        if (iw < 0) iw = -iw;
        if (iw >= w) iw = 2 * w - iw - 2;
      }
      ih = max(0, min(ih, h - 1));
      iw = max(0, min(iw, w - 1));
      v = __ldg(x + (pl * h + ih) * w + iw);
    }
    y[i] = v;
  }
}

__global__ void pixel_shuffle_kernel(const float* __restrict__ x, float* __restrict__ y, long long batch, int ic, int h, int w, int r) {
  const int oc = ic / (r * r), oh = h * r, ow = w * r;
  const long long total = batch * oc * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    long long t = i / ow;
    const int p = static_cast<int>(t % oh);
    t /= oh;
    const int o = static_cast<int>(t % oc);
    const long long s = t / oc;
    const int ih = p / r, iw = q / r;
    const int c = o * r * r + (p - ih * r) * r + (q - iw * r);
    y[i] = __ldg(x + ((s * ic + c) * h + ih) * w + iw);
  }
}

// half_pixel = 0: source index oh * (in/out); 1: (oh + 0.5) * (in/out) - 0.5 clamped to [0, in-1]
__global__ void upsample_bilinear_kernel(const float* __restrict__ x, float* __restrict__ y, long long planes, int h, int w, int oh,
                                         int ow, int half_pixel) {
  const float sch = static_cast<float>(h) / static_cast<float>(oh), scw = static_cast<float>(w) / static_cast<float>(ow);
  const long long total = planes * oh * ow;
  MB_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i % ow);
    const long long t = i / ow;
    const int r = static_cast<int>(t % oh);
    const long long pl = t / oh;
    float fh, fw;
    if (half_pixel) {
      fh = fmaf(static_cast<float>(r) + 0.5f, sch, -0.5f);
      fw = fmaf(static_cast<float>(q) + 0.5f, scw, -0.5f);
      fh = fmaxf(0.0f, fminf(fh, static_cast<float>(h) - 1.0f));
      fw = fmaxf(0.0f, fminf(fw, static_cast<float>(w) - 1.0f));
    } else {
      fh = static_cast<float>(r) * sch;
      fw = static_cast<float>(q) * scw;
    }
    const int h0 = static_cast<int>(floorf(fh)), w0 = static_cast<int>(floorf(fw));
    const int h1 = min(h0 + 1, h - 1), w1 = min(w0 + 1, w - 1);
    const float dh = fh - static_cast<float>(h0), dw = fw - static_cast<float>(w0);
    const float* xp = x + pl * h * w;
    const float v00 = __ldg(xp + h0 * w + w0), v01 = __ldg(xp + h0 * w + w1), v10 = __ldg(xp + h1 * w + w0),
                v11 = __ldg(xp + h1 * w + w1);
    y[i] = v00 * (1.0f - dh) * (1.0f - dw) + v01 * (1.0f - dh) * dw + v10 * dh * (1.0f - dw) + v11 * dh * dw;
  }
}

// C[b] = A[b] (M x K) . B[b] (K x N), fp32, k-sequential per output like the reference.  32 x 32 output
// tile per CTA, K walked in slabs of 32 through shared memory.
__global__ void __launch_bounds__(256) batch_matmul_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                           float* __restrict__ C, int M, int K, int N) {
  __shared__ float As[32][33], Bs[32][33];
  const long long b = blockIdx.z;
  const float* a = A + b * M * K;
  const float* bm = B + b * K * N;
  float* c = C + b * M * N;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 8 rows of threads, 4 outputs each
  const int row0 = blockIdx.y * 32, col0 = blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = ty * 4 + j;
      As[r][tx] = (row0 + r < M && k0 + tx < K) ? __ldg(a + static_cast<long long>(row0 + r) * K + k0 + tx) : 0.0f;
      Bs[r][tx] = (k0 + r < K && col0 + tx < N) ? __ldg(bm + static_cast<long long>(k0 + r) * N + col0 + tx) : 0.0f;
    }
    __syncthreads();
    const int kn = min(32, K - k0);
    for (int kk = 0; kk < kn; ++kk) {
      const float bv = Bs[kk][tx];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = fmaf(As[ty * 4 + j][kk], bv, acc[j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = row0 + ty * 4 + j;
    if (r < M && col0 + tx < N) c[static_cast<long long>(r) * N + col0 + tx] = acc[j];
  }
}

// (x - mean[c]) * inv_std[c] * gamma[c] + beta[c], in the reference's order of operations (Layers.hpp:961-966)
__global__ void batchnorm_running_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                         const float* __restrict__ mean, const float* __restrict__ var, float* __restrict__ y,
                                         long long total, int channels, long long spatial, float eps) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>((i / spatial) % channels);
    const float inv_std = 1.0f / sqrtf(__ldg(var + c) + eps);
    y[i] = __fadd_rn(__fmul_rn(__fmul_rn(__ldg(x + i) - __ldg(mean + c), inv_std), __ldg(gamma + c)), __ldg(beta + c));
  }
}

__global__ void scale_prefix_kernel(float* __restrict__ y, const float* __restrict__ g, long long batch, long long n, long long cnt) {
  const long long total = batch * cnt;
  MB_GRID_STRIDE(i, total) {
    const long long s = i / cnt, j = i - s * cnt;
    y[s * n + j] *= __ldg(g + j);
  }
}

}  // namespace

#define MB_LAUNCHED()            \
  MB_CUDA(cudaGetLastError());   \
  count_launch();                \
  return MIMIR_B200_OK

int launch_depthwise_conv2d(const float* x, const float* w, const float* bias, float* y, int batch, int ch, int h, int wd, int k,
                            int stride, int pad, int64_t w_count, cudaStream_t st) {
  if (batch <= 0 || ch <= 0 || h <= 0 || wd <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return fail(MIMIR_B200_E_INVALID, "DepthwiseConv2d: invalid dimensions");
  const int oh = (h + 2 * pad - k) / stride + 1, ow = (wd + 2 * pad - k) / stride + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "DepthwiseConv2d: empty output");
  const long long planes = static_cast<long long>(batch) * ch;
  depthwise_conv2d_kernel<<<grid_of(planes * oh * ow, 256), 256, 0, st>>>(
      x, w, bias, y, planes, ch, h, wd, oh, ow, k, stride, pad, static_cast<int>(std::min<int64_t>(w_count, 0x7fffffff)));
  MB_LAUNCHED();
}

int launch_conv1d(const float* x, const float* w, const float* bias, float* y, int batch, int ic, int oc, int len, int k, int stride,
                  int pad, int64_t w_count, cudaStream_t st) {
  if (batch <= 0 || ic <= 0 || oc <= 0 || len <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return fail(MIMIR_B200_E_INVALID, "Conv1d: invalid dimensions");
  const int olen = (len + 2 * pad - k) / stride + 1;
  if (olen <= 0) return fail(MIMIR_B200_E_INVALID, "Conv1d: empty output");
  conv1d_kernel<<<grid_of(static_cast<long long>(batch) * oc * olen, 256), 256, 0, st>>>(
      x, w, bias, y, batch, ic, oc, len, olen, k, stride, pad, static_cast<int>(std::min<int64_t>(w_count, 0x7fffffff)));
  MB_LAUNCHED();
}

int launch_conv_gather(const float* x, const float* w, float* y, int batch, int ic, int oc, int h, int wd, int oh, int ow, int k,
                       int stride, int pad, int relu, cudaStream_t st) {
  if (batch <= 0 || ic <= 0 || oc <= 0 || h <= 0 || wd <= 0 || oh <= 0 || ow <= 0 || k <= 0 || stride <= 0)
    return fail(MIMIR_B200_E_INVALID, "ConvTranspose2d: invalid dimensions");
  conv_gather_kernel<<<grid_of(static_cast<long long>(batch) * oc * oh * ow, 256), 256, 0, st>>>(x, w, y, batch, ic, oc, h, wd, oh, ow,
                                                                                                 k, stride, pad, relu);
  MB_LAUNCHED();
}

int launch_conv2d_dilated(const float* x, const float* w, const float* bias, float* y, int batch, int ic, int oc, int h, int wd, int k,
                          int stride, int pad, int dil, cudaStream_t st) {
  if (batch <= 0 || ic <= 0 || oc <= 0 || h <= 0 || wd <= 0 || k <= 0 || stride <= 0 || pad < 0 || dil <= 0)
    return fail(MIMIR_B200_E_INVALID, "computeConv2D: invalid dimensions");
  const int oh = (h + 2 * pad - dil * (k - 1) - 1) / stride + 1, ow = (wd + 2 * pad - dil * (k - 1) - 1) / stride + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "computeConv2D: empty output");
  conv2d_dilated_kernel<<<grid_of(static_cast<long long>(batch) * oc * oh * ow, 256), 256, 0, st>>>(x, w, bias, y, batch, ic, oc, h, wd,
                                                                                                    oh, ow, k, stride, pad, dil);
  MB_LAUNCHED();
}

int launch_conv_transpose2d_scatter(const float* x, const float* w, const float* bias, float* y, int batch, int ic, int oc, int h, int wd,
                                    int k, int stride, int pad, cudaStream_t st) {
  if (batch <= 0 || ic <= 0 || oc <= 0 || h <= 0 || wd <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return fail(MIMIR_B200_E_INVALID, "computeConvTranspose2D: invalid dimensions");
  const int oh = (h - 1) * stride - 2 * pad + k, ow = (wd - 1) * stride - 2 * pad + k;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "computeConvTranspose2D: empty output");
  conv_transpose2d_scatter_kernel<<<grid_of(static_cast<long long>(batch) * oc * oh * ow, 256), 256, 0, st>>>(x, w, bias, y, batch, ic, oc,
                                                                                                              h, wd, oh, ow, k, stride, pad);
  MB_LAUNCHED();
}

int launch_batchnorm_batchstats(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels, long long spatial,
                                float eps, cudaStream_t st) {
  if (batch <= 0 || channels <= 0 || spatial <= 0) return fail(MIMIR_B200_E_INVALID, "computeBatchNorm: invalid dimensions");
  batchnorm_batchstats_kernel<<<channels, 256, 0, st>>>(x, gamma, beta, y, batch, channels, spatial, eps);
  MB_LAUNCHED();
}

int launch_pool2d(int is_max, const float* x, float* y, int batch, int ch, int h, int wd, int kh, int kw, int sh, int sw, int ph, int pw,
                  cudaStream_t st) {
  if (batch <= 0 || ch <= 0 || h <= 0 || wd <= 0) return fail(MIMIR_B200_E_INVALID, "Pool2d: invalid dimensions");
  if (kh <= 0 || kw <= 0) return fail(MIMIR_B200_E_INVALID, "MaxPool2d: kernel_size must be > 0");
  if (sh <= 0 || sw <= 0) return fail(MIMIR_B200_E_INVALID, "MaxPool2d: stride must be > 0");
  const int oh = (h + 2 * ph - kh) / sh + 1, ow = (wd + 2 * pw - kw) / sw + 1;
  if (oh <= 0 || ow <= 0) return fail(MIMIR_B200_E_INVALID, "MaxPool2d: output dimensions must be > 0");
  const long long planes = static_cast<long long>(batch) * ch;
  const int grid = grid_of(planes * oh * ow, 256);
  if (is_max) pool2d_kernel<true><<<grid, 256, 0, st>>>(x, y, planes, h, wd, oh, ow, kh, kw, sh, sw, ph, pw);
  else pool2d_kernel<false><<<grid, 256, 0, st>>>(x, y, planes, h, wd, oh, ow, kh, kw, sh, sw, ph, pw);
  MB_LAUNCHED();
}

int launch_pad2d(int mode, const float* x, float* y, int batch, int ch, int h, int wd, int ph, int pw, cudaStream_t st) {
  if (batch <= 0 || ch <= 0 || h <= 0 || wd <= 0 || ph < 0 || pw < 0 || mode < 0 || mode > 2)
    return fail(MIMIR_B200_E_INVALID, "Pad2d: invalid dimensions");
  const long long planes = static_cast<long long>(batch) * ch;
  pad2d_kernel<<<grid_of(planes * (h + 2 * ph) * (wd + 2 * pw), 256), 256, 0, st>>>(x, y, planes, h, wd, ph, pw, mode);
  MB_LAUNCHED();
}

int launch_pixel_shuffle(const float* x, float* y, int batch, int ic, int h, int wd, int r, cudaStream_t st) {
  if (batch <= 0 || ic <= 0 || h <= 0 || wd <= 0 || r <= 0) return fail(MIMIR_B200_E_INVALID, "PixelShuffle: invalid dimensions");
  if (ic % (r * r) != 0)
    return fail(MIMIR_B200_E_INVALID, "PixelShuffle: in_channels (%d) must be divisible by upscale_factor^2 (%d)", ic, r * r);
  pixel_shuffle_kernel<<<grid_of(static_cast<long long>(batch) * ic * h * wd, 256), 256, 0, st>>>(x, y, batch, ic, h, wd, r);
  MB_LAUNCHED();
}

int launch_upsample_bilinear(const float* x, float* y, int batch, int ch, int h, int wd, int oh, int ow, int half_pixel,
                             cudaStream_t st) {
  if (batch <= 0 || ch <= 0 || h <= 0 || wd <= 0 || oh <= 0 || ow <= 0)
    return fail(MIMIR_B200_E_INVALID, "UpsampleBilinear: dimensions must be set");
  const long long planes = static_cast<long long>(batch) * ch;
  upsample_bilinear_kernel<<<grid_of(planes * oh * ow, 256), 256, 0, st>>>(x, y, planes, h, wd, oh, ow, half_pixel);
  MB_LAUNCHED();
}

int launch_batch_matmul(const float* a, const float* b, float* c, int64_t nb, int m, int k, int n, cudaStream_t st) {
  if (nb <= 0 || m <= 0 || k <= 0 || n <= 0) return fail(MIMIR_B200_E_INVALID, "BatchMatMul: invalid dimensions");
  if (nb > 65535) return fail(MIMIR_B200_E_UNSUPPORTED, "BatchMatMul: more than 65535 matrices in one call");
  dim3 grid((n + 31) / 32, (m + 31) / 32, static_cast<unsigned>(nb));
  batch_matmul_kernel<<<grid, 256, 0, st>>>(a, b, c, m, k, n);
  MB_LAUNCHED();
}

int launch_batchnorm_running(const float* x, const float* gamma, const float* beta, const float* mean, const float* var, float* y,
                             int batch, int channels, int64_t spatial, float eps, cudaStream_t st) {
  const long long total = static_cast<long long>(batch) * channels * spatial;
  if (total <= 0) return MIMIR_B200_OK;
  batchnorm_running_kernel<<<grid_of(total, 256), 256, 0, st>>>(x, gamma, beta, mean, var, y, total, channels, spatial, eps);
  MB_CUDA(cudaGetLastError());
  count_launch();
  return MIMIR_B200_OK;
}

int launch_scale_prefix(float* y, const float* g, int batch, int64_t n, int64_t cnt, cudaStream_t st) {
  if (cnt <= 0) return MIMIR_B200_OK;
  if (cnt > n) cnt = n;
  scale_prefix_kernel<<<grid_of(static_cast<long long>(batch) * cnt, 256), 256, 0, st>>>(y, g, batch, n, cnt);
  MB_LAUNCHED();
}

}  // namespace mb
